// The one-CTA tensor-core GEMM kernels with 256-column tiles and sixteen epilogue warps (four per tensor-memory
// lane quarter): short K with wide outputs, where a tile's time is the latency chain of its epilogue.
#define CUGL_EPI_WARPS 16
#include "gemmlowp_tcgen05.cu"
