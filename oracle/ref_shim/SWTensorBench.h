// Empty stand-in: GCN_Layer_MKL_Forward_Utils.h includes the bench base class
// header but its kernels do not use it.
