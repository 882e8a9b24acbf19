"""TEST INFRASTRUCTURE ONLY: CPU oracle of the fused sparse-dense chains.

``oracle.bindings.Oracle`` wraps the plain-C restatement (tf_oracle.c);
``oracle.bindings.Ref`` wraps the unmodified reference compiled in place
(_ref/libtf_ref.so, built by ``make -C oracle ref`` where the reference tree is
present).  Only tests, the smoke check and the benchmark's CPU-baseline leg may
import this package; the product package must not.
"""
