// The tensor-core GEMM and implicit-convolution kernels with eight epilogue warps (two per tensor-memory lane
// quarter): the build of gemmlowp_tcgen05.cu for tiles whose time goes into the epilogue, i.e. short K.
#define CUGL_EPI_WARPS 8
#include "gemmlowp_tcgen05.cu"
