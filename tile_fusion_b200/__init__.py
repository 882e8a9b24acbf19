"""B200-native fused sparse-dense chains (GeMM-SpMM, SpMM-SpMM, SDDMM-SpMM)."""
