// Generic quantized GEMM on the CUDA cores.  It exists for operands the TMA engine cannot address
// (row strides that are not multiples of 16 bytes, unaligned bases) and as an independent second
// implementation the tensor-core kernel is checked against bit for bit.  64 x 64 output tile per
// block, 4 x 4 outputs per thread, K staged through shared memory 32 at a time.
#include "kernels.cuh"

namespace cugl
{
namespace
{
constexpr int TM = 64, TN = 64, TK = 32;

__global__ void __launch_bounds__(256) gemmlowp_simt_kernel(GemmOperands op, EpilogueParams ep)
{
    __shared__ int8_t  sa8[TM][TK + 4]; // raw bytes; widened on use according to the operand type
    __shared__ int8_t  sb8[TN][TK + 4];
    const int          tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int          m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    const uint8_t     *A  = static_cast<const uint8_t *>(op.a);
    const uint8_t     *Bt = static_cast<const uint8_t *>(op.bt);
    int32_t            acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0;

    for (int k0 = 0; k0 < op.K; k0 += TK)
    {
        // 64 x 32 bytes per operand, 256 threads: 8 bytes each
        for (int i = threadIdx.x; i < TM * TK; i += 256)
        {
            const int r = i / TK, c = i % TK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            sa8[r][c]   = (m < op.M && k < op.K) ? static_cast<int8_t>(A[m * op.lda + k]) : 0;
            sb8[r][c]   = (n < op.N && k < op.K) ? static_cast<int8_t>(Bt[n * op.ldbt + k]) : 0;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < TK; ++k)
        {
            int32_t av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                const int8_t ra = sa8[ty * 4 + i][k];
                const int8_t rb = sb8[tx * 4 + i][k];
                av[i] = op.a_signed ? static_cast<int32_t>(ra) : static_cast<int32_t>(static_cast<uint8_t>(ra));
                bv[i] = op.b_signed ? static_cast<int32_t>(rb) : static_cast<int32_t>(static_cast<uint8_t>(rb));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        const int m = m0 + ty * 4 + i;
        if (m >= op.M) continue;
        const int32_t row_term = ep.rowsum != nullptr ? ep.b_off * ep.rowsum[m] : 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const int n = n0 + tx * 4 + j;
            if (n >= op.N) continue;
            int32_t v = acc[i][j] + row_term + ep.k_term;
            if (ep.colsum != nullptr) v += ep.a_off * ep.colsum[n];
            if (ep.bias != nullptr) v += ep.bias[n];
            if (ep.stage == CUGL_STAGE_NONE)
            {
                uint32_t *o = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(op.dst) + m * op.ldd + n * 4);
                *o          = raw_result_word(v, ep.accumulate != 0 ? *o : 0u, ep);
            }
            else
            {
                const int32_t mu = ep.mults != nullptr ? ep.mults[n] : ep.mult;
                const int32_t sh = ep.shifts != nullptr ? ep.shifts[n] : ep.shift;
                const int32_t r  = ep.stage == CUGL_STAGE_QUANTIZE_DOWN
                                       ? finalize_int(v + ep.result_offset, mu, sh, ep.lo, ep.hi)
                                       : finalize(v, mu, max(-sh, 0), max(sh, 0), ep.result_offset, ep.lo, ep.hi);
                static_cast<uint8_t *>(op.dst)[m * op.ldd + n] = static_cast<uint8_t>(r);
            }
        }
    }
}
} // namespace

cugl_status launch_gemmlowp_simt(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    if (op.M <= 0 || op.N <= 0) return CUGL_SUCCESS;
    dim3 grid((op.M + TM - 1) / TM, (op.N + TN - 1) / TN);
    if (grid.y > 65535)
    {
        return fail(ctx, CUGL_UNSUPPORTED_CONFIG, "gemmlowp_simt: N too large for the generic kernel");
    }
    gemmlowp_simt_kernel<<<grid, 256, 0, ctx->stream>>>(op, ep);
    return check_cuda(ctx, cudaGetLastError(), "gemmlowp_simt_kernel");
}
} // namespace cugl
