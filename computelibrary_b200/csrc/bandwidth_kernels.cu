// HBM-bound kernels of the quantized GEMM path: row / column reductions, the B re-layout done in
// prepare(), the S32 offset contribution, the stand-alone output stage, NHWC im2col and the weights
// reshape.  All of them move each byte once with 128-bit accesses where the addresses allow it.
#include "kernels.cuh"

namespace cugl
{
namespace
{
constexpr int kThreads = 256;

__device__ __forceinline__ int32_t sum4(uint32_t w, bool is_signed, int32_t acc)
{
    return is_signed ? __dp4a(static_cast<int32_t>(w), 0x01010101, acc)
                     : static_cast<int32_t>(__dp4a(w, 0x01010101u, static_cast<uint32_t>(acc)));
}

__device__ __forceinline__ int32_t warp_sum(int32_t v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

// ---- rowsum_A[m] = scalar * sum_k A[m,k] -------------------------------------------------------
// One warp per row: unaligned head bytes, a body of 16-byte vectors, tail bytes; shuffle reduction.
// CpuGemmLowpMatrixAReductionKernel::run_internal (CpuGemmLowpMatrixReductionKernel.cpp:133-204).
__global__ void __launch_bounds__(kThreads) reduce_rows_kernel(const uint8_t *__restrict__ a, bool is_signed, int M,
                                                               int K, int64_t lda, int32_t scalar,
                                                               int32_t *__restrict__ out)
{
    const int lane          = threadIdx.x & 31;
    const int warps_per_blk = kThreads / 32;
    for (int m = blockIdx.x * warps_per_blk + (threadIdx.x >> 5); m < M; m += gridDim.x * warps_per_blk)
    {
        const uint8_t *row  = a + static_cast<int64_t>(m) * lda;
        const int      head = min(K, static_cast<int>((16 - (reinterpret_cast<uintptr_t>(row) & 15)) & 15));
        int32_t        acc  = 0;
        if (lane < head)
        {
            acc += load_q8(row, lane, is_signed);
        }
        const int    nvec = (K - head) >> 4;
        const uint4 *v    = reinterpret_cast<const uint4 *>(row + head);
        int i = lane;
        for (; i + 96 < nvec; i += 128) // four independent 16-byte loads in flight per lane
        {
            const uint4 q0 = __ldg(v + i), q1 = __ldg(v + i + 32), q2 = __ldg(v + i + 64), q3 = __ldg(v + i + 96);
            int32_t     a0 = sum4(q0.x, is_signed, 0), a1 = sum4(q1.x, is_signed, 0);
            int32_t     a2 = sum4(q2.x, is_signed, 0), a3 = sum4(q3.x, is_signed, 0);
            a0 = sum4(q0.y, is_signed, a0), a1 = sum4(q1.y, is_signed, a1);
            a2 = sum4(q2.y, is_signed, a2), a3 = sum4(q3.y, is_signed, a3);
            a0 = sum4(q0.z, is_signed, a0), a1 = sum4(q1.z, is_signed, a1);
            a2 = sum4(q2.z, is_signed, a2), a3 = sum4(q3.z, is_signed, a3);
            a0 = sum4(q0.w, is_signed, a0), a1 = sum4(q1.w, is_signed, a1);
            a2 = sum4(q2.w, is_signed, a2), a3 = sum4(q3.w, is_signed, a3);
            acc += (a0 + a1) + (a2 + a3);
        }
        for (; i < nvec; i += 32)
        {
            const uint4 q = __ldg(v + i);
            acc           = sum4(q.x, is_signed, acc);
            acc           = sum4(q.y, is_signed, acc);
            acc           = sum4(q.z, is_signed, acc);
            acc           = sum4(q.w, is_signed, acc);
        }
        const int tail0 = head + (nvec << 4);
        if (tail0 + lane < K)
        {
            acc += load_q8(row, tail0 + lane, is_signed);
        }
        acc = warp_sum(acc);
        if (lane == 0)
        {
            out[m] = acc * scalar;
        }
    }
}

// ---- colsum_B[n] += sum over a K-slab of B[k,n] --------------------------------------------------
// A thread owns 16 consecutive columns and reads them with one 128-bit load per row, so a warp reads 512
// contiguous bytes of a row.  The bytes are summed as packed 16-bit pairs (signed bytes are biased by 128 first,
// the bias leaves again at the end): two adds per four columns and row.  A slab is at most 256 rows, which a
// 16-bit lane holds without overflow (256 * 255 < 2^16).  grid.y splits K; integer atomics combine the slabs
// (exact, order-independent).  out must be zero on entry; the scalar is applied by scale_vector_kernel.
// Needs B and ldb 16-byte aligned; reduce_cols_generic_kernel covers the rest and the ragged last columns.
// CpuGemmLowpMatrixBReductionKernel::run_internal (CpuGemmLowpMatrixReductionKernel.cpp:273-446).
constexpr int kColSlabRows = 256;
__global__ void __launch_bounds__(kThreads) reduce_cols_kernel(const uint8_t *__restrict__ b, bool is_signed, int K,
                                                               int n_vec, int64_t ldb, int k_per_block,
                                                               int32_t *__restrict__ out)
{
    const int unit = blockIdx.x * kThreads + threadIdx.x; // 16 columns
    if (unit >= n_vec)
    {
        return;
    }
    const int      k0   = blockIdx.y * k_per_block;
    const int      k1   = min(K, k0 + k_per_block);
    const uint32_t flip = is_signed ? 0x80808080u : 0u;
    uint32_t       even[4] = {0, 0, 0, 0}, odd[4] = {0, 0, 0, 0}; // columns 4w, 4w+2 | 4w+1, 4w+3 as 16-bit pairs
    const uint8_t *p = b + static_cast<int64_t>(k0) * ldb + 16 * static_cast<int64_t>(unit);
#pragma unroll 4
    for (int k = k0; k < k1; ++k, p += ldb)
    {
        const uint4    q    = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint32_t w[4] = {q.x ^ flip, q.y ^ flip, q.z ^ flip, q.w ^ flip};
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            even[j] += w[j] & 0x00ff00ffu;
            odd[j] += (w[j] >> 8) & 0x00ff00ffu;
        }
    }
    const int32_t bias = is_signed ? 128 * (k1 - k0) : 0;
    int32_t      *o    = out + 16 * unit;
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        atomicAdd(o + 4 * j + 0, static_cast<int32_t>(even[j] & 0xffffu) - bias);
        atomicAdd(o + 4 * j + 1, static_cast<int32_t>(odd[j] & 0xffffu) - bias);
        atomicAdd(o + 4 * j + 2, static_cast<int32_t>(even[j] >> 16) - bias);
        atomicAdd(o + 4 * j + 3, static_cast<int32_t>(odd[j] >> 16) - bias);
    }
}

// any alignment: one thread per column of [n_first, N)
__global__ void __launch_bounds__(kThreads) reduce_cols_generic_kernel(const uint8_t *__restrict__ b, bool is_signed,
                                                                       int K, int n_first, int N, int64_t ldb,
                                                                       int k_per_block, int32_t *__restrict__ out)
{
    const int n = n_first + blockIdx.x * kThreads + threadIdx.x;
    if (n >= N)
    {
        return;
    }
    const int k0 = blockIdx.y * k_per_block;
    const int k1 = min(K, k0 + k_per_block);
    int32_t   s  = 0;
    for (int k = k0; k < k1; ++k)
    {
        s += load_q8(b + static_cast<int64_t>(k) * ldb, n, is_signed);
    }
    atomicAdd(out + n, s);
}

__global__ void scale_vector_kernel(int32_t *v, int n, int32_t scalar)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
    {
        v[i] *= scalar;
    }
}

// ---- prepare(): B [K,N] (N contiguous) -> Bt [N, ldbt] (K contiguous) + column sums -------------
// 64 x 64 byte tiles through shared memory: reads are coalesced along N, writes along K.  Each block
// also reduces its 64 rows per column and adds the partial sums with integer atomics, so B is read
// exactly once for both products of prepare().  colsum (when not null) must be zero on entry.
__global__ void __launch_bounds__(kThreads) transpose_colsum_kernel(const uint8_t *__restrict__ b, bool is_signed,
                                                                    int K, int N, int64_t ldb,
                                                                    uint8_t *__restrict__ bt, int64_t ldbt,
                                                                    int32_t *__restrict__ colsum)
{
    __shared__ uint8_t tile[64][64 + 4];
    const int          k0 = blockIdx.y * 64;
    const int          n0 = blockIdx.x * 64;
    const int          tx = threadIdx.x & 63; // fastest index
    const int          ty = threadIdx.x >> 6; // 0..3
#pragma unroll 4
    for (int r = ty; r < 64; r += 4)
    {
        const int k = k0 + r, n = n0 + tx;
        tile[r][tx] = (k < K && n < N) ? b[static_cast<int64_t>(k) * ldb + n] : 0;
    }
    __syncthreads();
#pragma unroll 4
    for (int r = ty; r < 64; r += 4)
    {
        const int n = n0 + r, k = k0 + tx;
        if (n < N && k < K)
        {
            bt[static_cast<int64_t>(n) * ldbt + k] = tile[tx][r];
        }
    }
    if (colsum != nullptr && threadIdx.x < 64)
    {
        const int n = n0 + threadIdx.x;
        if (n < N)
        {
            int32_t s = 0;
#pragma unroll 8
            for (int r = 0; r < 64; ++r)
            {
                const uint8_t v = tile[r][threadIdx.x];
                s += is_signed ? static_cast<int32_t>(static_cast<int8_t>(v)) : static_cast<int32_t>(v);
            }
            atomicAdd(colsum + n, s);
        }
    }
}

// The same with 32-bit global accesses (four bytes per thread and instruction instead of one): K, N, both pitches and
// both base addresses multiples of 4.  A 64 x 64 tile is loaded as 16 words per row, transposed byte by byte out of
// shared memory (four byte reads and three permutes per output word) and stored as 16 words per output row.
__global__ void __launch_bounds__(kThreads) transpose_colsum_words_kernel(const uint8_t *__restrict__ b, bool is_signed,
                                                                          int K, int N, int64_t ldb,
                                                                          uint8_t *__restrict__ bt, int64_t ldbt,
                                                                          int32_t *__restrict__ colsum)
{
    __shared__ uint32_t tile[64][16 + 1]; // [k][n / 4], one word of padding per row
    const int           k0 = blockIdx.y * 64;
    const int           n0 = blockIdx.x * 64;
    const int           w  = threadIdx.x & 15; // word of the row
    const int           r4 = threadIdx.x >> 4; // 0..15
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        const int r = r4 + 16 * i, k = k0 + r, n = n0 + 4 * w;
        tile[r][w]  = (k < K && n < N) ? __ldg(reinterpret_cast<const uint32_t *>(b + static_cast<int64_t>(k) * ldb + n)) : 0u;
    }
    __syncthreads();
    const uint8_t *bytes = reinterpret_cast<const uint8_t *>(&tile[0][0]);
    constexpr int  kPitch = (16 + 1) * 4; // bytes per tile row
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        const int n = r4 + 16 * i, k = k0 + 4 * w; // output row n0 + n, output word w: bytes tile[4w .. 4w+3][n]
        if (n0 + n < N && k < K)
        {
            const uint32_t v = static_cast<uint32_t>(bytes[(4 * w + 0) * kPitch + n]) |
                               (static_cast<uint32_t>(bytes[(4 * w + 1) * kPitch + n]) << 8) |
                               (static_cast<uint32_t>(bytes[(4 * w + 2) * kPitch + n]) << 16) |
                               (static_cast<uint32_t>(bytes[(4 * w + 3) * kPitch + n]) << 24);
            *reinterpret_cast<uint32_t *>(bt + static_cast<int64_t>(n0 + n) * ldbt + k) = v;
        }
    }
    if (colsum != nullptr && threadIdx.x < 64)
    {
        const int n = n0 + threadIdx.x;
        if (n < N)
        {
            int32_t s = 0;
#pragma unroll 8
            for (int r = 0; r < 64; ++r)
            {
                const uint8_t v = bytes[r * kPitch + threadIdx.x];
                s += is_signed ? static_cast<int32_t>(static_cast<int8_t>(v)) : static_cast<int32_t>(v);
            }
            atomicAdd(colsum + n, s);
        }
    }
}

// ---- weights reshape: [OFM][K] -> [K][OFM] -------------------------------------------------------
// CpuWeightsReshapeKernel::run_op (CpuWeightsReshapeKernel.cpp:121-183) for NHWC weights.
__global__ void __launch_bounds__(kThreads) transpose_bytes_kernel(const uint8_t *__restrict__ src, int rows,
                                                                   int cols, uint8_t *__restrict__ dst)
{
    __shared__ uint8_t tile[64][64 + 4];
    const int          r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int          tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    src += static_cast<int64_t>(blockIdx.z) * rows * cols; // blockIdx.z: which matrix of the batch
    dst += static_cast<int64_t>(blockIdx.z) * rows * cols;
    for (int r = ty; r < 64; r += 4)
    {
        tile[r][tx] = (r0 + r < rows && c0 + tx < cols) ? src[static_cast<int64_t>(r0 + r) * cols + c0 + tx] : 0;
    }
    __syncthreads();
    for (int c = ty; c < 64; c += 4)
    {
        if (c0 + c < cols && r0 + tx < rows)
        {
            dst[static_cast<int64_t>(c0 + c) * rows + r0 + tx] = tile[tx][c];
        }
    }
}

// ---- S32 offset contribution (output stage NONE) --------------------------------------------------
// CpuGemmLowpOffsetContributionKernel (CpuGemmLowpOffsetContributionKernel.cpp:116-229).
__global__ void __launch_bounds__(kThreads) offset_contribution_kernel(int32_t *__restrict__ mm, int M, int N,
                                                                       int64_t ld_elems,
                                                                       const int32_t *__restrict__ colsum,
                                                                       const int32_t *__restrict__ rowsum,
                                                                       int32_t a_off, int32_t b_off, int32_t k_term,
                                                                       bool vec_ok)
{
    // blockIdx.y strides over rows, x over groups of four columns: no division anywhere
    const int groups = (N + 3) >> 2;
    for (int m = blockIdx.y; m < M; m += gridDim.y)
    {
        int32_t      *row   = mm + m * ld_elems;
        const int32_t rterm = k_term + (rowsum != nullptr ? b_off * __ldg(rowsum + m) : 0);
        for (int g = blockIdx.x * kThreads + threadIdx.x; g < groups; g += gridDim.x * kThreads)
        {
            const int n0 = g * 4;
            if (vec_ok && n0 + 4 <= N)
            {
                int4 v = *reinterpret_cast<int4 *>(row + n0);
                if (colsum != nullptr)
                {
                    const int4 c = __ldg(reinterpret_cast<const int4 *>(colsum + n0));
                    v.x += a_off * c.x, v.y += a_off * c.y, v.z += a_off * c.z, v.w += a_off * c.w;
                }
                v.x += rterm, v.y += rterm, v.z += rterm, v.w += rterm;
                *reinterpret_cast<int4 *>(row + n0) = v;
            }
            else
            {
                for (int n = n0; n < min(n0 + 4, N); ++n)
                {
                    row[n] += rterm + (colsum != nullptr ? a_off * colsum[n] : 0);
                }
            }
        }
    }
}

// ---- stand-alone output stage ---------------------------------------------------------------------
// CpuGemmLowpQuantizeDownInt32To{Uint8,Int8}ScaleByFixedPointKernel::run_internal
// (…ToUint8ScaleByFixedPointKernel.cpp:78-186).  A thread owns four consecutive columns -- their bias, multipliers and
// shifts stay in registers -- and walks down the rows (blockIdx.y strides over them): one 128-bit load and one 32-bit
// (8-bit output) or 64-bit (16-bit output) store per row, a warp covering 512 contiguous input bytes; no division.
template <bool kOut16>
__global__ void __launch_bounds__(kThreads) output_stage_kernel(const int32_t *__restrict__ in, int64_t ld_in_elems,
                                                                const int32_t *__restrict__ bias,
                                                                uint8_t *__restrict__ out, int64_t ld_out, int M,
                                                                int N, const int32_t *__restrict__ mults,
                                                                const int32_t *__restrict__ shifts, int32_t mult,
                                                                int32_t shift, int32_t offset, int32_t lo, int32_t hi,
                                                                bool vec_ok, bool integer_stage)
{
    const int n0 = (blockIdx.x * kThreads + threadIdx.x) * 4;
    if (n0 >= N)
    {
        return;
    }
    const bool full = n0 + 4 <= N;
    int32_t    cb[4], cm[4], cl[4], cr[4]; // bias, multiplier, left and right shift of this thread's columns
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const int     n  = min(n0 + j, N - 1);
        const int32_t sh = shifts != nullptr ? shifts[n] : shift;
        cb[j]            = bias != nullptr ? bias[n] : 0;
        cm[j]            = mults != nullptr ? mults[n] : mult;
        cl[j]            = max(-sh, 0);
        cr[j]            = integer_stage ? sh : max(sh, 0);
    }
    for (int m = blockIdx.y; m < M; m += gridDim.y)
    {
        const int32_t *src = in + m * ld_in_elems + n0;
        uint8_t       *dst = out + m * ld_out + n0 * (kOut16 ? 2 : 1);
        int32_t        v[4];
        if (full && vec_ok)
        {
            const int4 q = __ldcs(reinterpret_cast<const int4 *>(src)); // read once: streaming
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = (n0 + j < N) ? src[j] : 0;
        }
        uint32_t packed = 0, packed_hi = 0; // 8-bit: four bytes in packed; 16-bit: two halfwords in each
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const int32_t x = static_cast<int32_t>(static_cast<uint32_t>(v[j]) + static_cast<uint32_t>(cb[j]));
            const int32_t r = integer_stage
                                  ? finalize_int(static_cast<int32_t>(static_cast<uint32_t>(x) + static_cast<uint32_t>(offset)),
                                                 cm[j], cr[j], lo, hi)
                                  : finalize(x, cm[j], cl[j], cr[j], offset, lo, hi);
            if (kOut16)
            {
                (j < 2 ? packed : packed_hi) |= (static_cast<uint32_t>(r) & 0xffffu) << (16 * (j & 1));
            }
            else
            {
                packed |= (static_cast<uint32_t>(r) & 0xffu) << (8 * j);
            }
        }
        if (kOut16)
        {
            if (full && vec_ok)
            {
                *reinterpret_cast<uint2 *>(dst) = make_uint2(packed, packed_hi);
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n0 + j < N)
                        reinterpret_cast<uint16_t *>(dst)[j] = static_cast<uint16_t>((j < 2 ? packed : packed_hi) >> (16 * (j & 1)));
            }
        }
        else if (full && vec_ok)
        {
            *reinterpret_cast<uint32_t *>(dst) = packed;
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n0 + j < N) dst[j] = static_cast<uint8_t>(packed >> (8 * j));
        }
    }
}

// ---- NHWC im2col ------------------------------------------------------------------------------------
// dst row m = (b, yo, xo) holds kh*kw taps of C bytes in (ky, kx, c) order; an out-of-image tap is
// filled with the input zero point (directconv2d/impl.h:333-334).  VEC = bytes moved per thread and step.
// A block takes `rows_per_iter` consecutive output rows per step and spreads their VEC-byte units over its
// threads (consecutive threads write consecutive units: whole 128-byte lines); every index split is a 32-bit
// multiply-high division by a launch constant.
struct Im2colDivs
{
    FastDiv units, c, kw, wo, ho;
};

template <int VEC>
__global__ void __launch_bounds__(kThreads) im2col_nhwc_kernel(const uint8_t *__restrict__ src,
                                                               uint8_t *__restrict__ dst, int C, int W, int H,
                                                               int M, int kw, int kh, int sx, int sy, int pad_l,
                                                               int pad_t, int dil_x, int dil_y, int Wo, int Ho,
                                                               uint32_t pad_word, int64_t row_stride,
                                                               int rows_per_iter, const Im2colDivs dv)
{
    const int K             = kh * kw * C;
    const int units_per_row = static_cast<int>(row_stride / VEC);
    const int per_iter      = rows_per_iter * units_per_row;
    for (int64_t m0 = static_cast<int64_t>(blockIdx.x) * rows_per_iter; m0 < M;
         m0 += static_cast<int64_t>(gridDim.x) * rows_per_iter)
    {
        for (int i = threadIdx.x; i < per_iter; i += kThreads)
        {
            const int r = fast_div(i, dv.units);
            const int m = static_cast<int>(m0) + r;
            if (m >= M)
            {
                break;
            }
            const int off = (i - r * units_per_row) * VEC; // byte offset inside the row
            uint8_t  *d   = dst + static_cast<int64_t>(m) * row_stride + off;
            if (off >= K)
            {
                // zero the K padding that makes the row a multiple of 16 bytes
                if (VEC == 16) *reinterpret_cast<uint4 *>(d) = make_uint4(0, 0, 0, 0);
                else *d = 0;
                continue;
            }
            const int tap = fast_div(off, dv.c), c = off - tap * C;
            const int ky = fast_div(tap, dv.kw), kx = tap - ky * kw;
            const int q  = fast_div(m, dv.wo), xo = m - q * Wo;
            const int b  = fast_div(q, dv.ho), yo = q - b * Ho;
            const int yi = yo * sy - pad_t + ky * dil_y;
            const int xi = xo * sx - pad_l + kx * dil_x;
            const bool     inside = yi >= 0 && yi < H && xi >= 0 && xi < W;
            const uint8_t *sp     = src + ((static_cast<int64_t>(b) * H + yi) * W + xi) * C + c;
            if (VEC == 16)
            {
                uint4 v = make_uint4(pad_word, pad_word, pad_word, pad_word);
                if (inside) v = __ldg(reinterpret_cast<const uint4 *>(sp));
                *reinterpret_cast<uint4 *>(d) = v;
            }
            else
            {
                *d = inside ? *sp : static_cast<uint8_t>(pad_word);
            }
        }
    }
}

// ---- 2x2 space-to-depth lowering of stride-2 convolutions with at most four input channels -------------
// A 7x7 / stride 2 convolution over 3 channels has a 147-byte patch row, useless to a 16-byte gather.  Folding
// every 2x2 pixel block into 16 channels ((dy, dx, c) with c padded to 4) turns it into a 4x4 / stride 1
// convolution over 16 channels whose folded weights are zero wherever the original kernel has no tap:
// the sums are the same integers.  fold_input_kernel: dst[b][Y][X][(dy*2+dx)*4 + c] = src[b][2Y+dy][2X+dx][c];
// pixels beyond an odd edge and the padding channels hold the zero point (their weights are zero).
// One thread per folded pixel (16 output bytes).  kFast: three channels, an even image width and a 2-byte aligned
// tensor -- the two pixels of a row of the block are six contiguous bytes on a 2-byte boundary and come in as three
// 16-bit loads -- and fewer than 2^31 folded pixels, so that the index arithmetic is 32-bit.
template <bool kFast>
__global__ void __launch_bounds__(kThreads) fold_input_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                              int B, int H, int W, int C, int H2, int W2, uint32_t zp)
{
    const int64_t total = static_cast<int64_t>(B) * H2 * W2;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kThreads)
    {
        int     X, Y;
        int64_t b;
        if (kFast)
        {
            uint32_t q = static_cast<uint32_t>(i);
            X          = static_cast<int>(q % static_cast<uint32_t>(W2));
            q /= static_cast<uint32_t>(W2);
            Y = static_cast<int>(q % static_cast<uint32_t>(H2));
            b = q / static_cast<uint32_t>(H2);
        }
        else
        {
            X = static_cast<int>(i % W2);
            Y = static_cast<int>((i / W2) % H2);
            b = i / (static_cast<int64_t>(W2) * H2);
        }
        uint32_t w[4];
        if (kFast)
        {
            // W is even: the block's two columns both lie inside the image
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
            {
                const int y = 2 * Y + dy;
                uint32_t  p0 = zp * 0x01010101u, p1 = p0;
                if (y < H)
                {
                    const uint16_t *p = reinterpret_cast<const uint16_t *>(src + ((b * H + y) * W + 2 * X) * 3);
                    const uint32_t  h0 = __ldg(p), h1 = __ldg(p + 1), h2 = __ldg(p + 2); // c0 c1 | c2 c0' | c1' c2'
                    p0 = h0 | ((h1 & 0xffu) << 16) | (zp << 24);
                    p1 = (h1 >> 8) | (h2 << 8) | (zp << 24);
                }
                w[2 * dy]     = p0;
                w[2 * dy + 1] = p1;
            }
        }
        else
        {
#pragma unroll
            for (int q = 0; q < 4; ++q)
            {
                const int y = 2 * Y + (q >> 1), x = 2 * X + (q & 1);
                uint32_t  v = zp * 0x01010101u;
                if (y < H && x < W)
                {
                    const uint8_t *p = src + ((b * H + y) * W + x) * C;
                    v                = 0;
                    for (int c = 0; c < 4; ++c)
                    {
                        v |= (c < C ? static_cast<uint32_t>(p[c]) : zp) << (8 * c);
                    }
                }
                w[q] = v;
            }
        }
        reinterpret_cast<uint4 *>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// fold_weights_kernel: bt[n][((ty*kw2 + tx)*4 + dy*2 + dx)*4 + c] = w[n][2ty+dy-oy][2tx+dx-ox][c], zero where the
// original kernel has no such tap or channel.  (oy, ox) = parity of the top / left padding.
__global__ void __launch_bounds__(kThreads) fold_weights_kernel(const uint8_t *__restrict__ w, uint8_t *__restrict__ bt,
                                                                int64_t ldbt, int OFM, int kh, int kw, int C, int kh2,
                                                                int kw2, int oy, int ox)
{
    const int K2    = kh2 * kw2 * 16;
    const int total = OFM * K2;
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < total; i += gridDim.x * kThreads)
    {
        const int n = i / K2, k = i % K2;
        const int c = k & 3, dx = (k >> 2) & 1, dy = (k >> 3) & 1, t = k >> 4;
        const int tx = t % kw2, ty = t / kw2;
        const int ky = 2 * ty + dy - oy, kx = 2 * tx + dx - ox;
        uint8_t   v  = 0;
        if (ky >= 0 && ky < kh && kx >= 0 && kx < kw && c < C)
        {
            v = w[((static_cast<int64_t>(n) * kh + ky) * kw + kx) * C + c];
        }
        bt[n * ldbt + k] = v;
    }
}

int grid_for(int64_t work_items, int sm_count, int per_thread = 1)
{
    const int64_t blocks = (work_items + static_cast<int64_t>(kThreads) * per_thread - 1) /
                           (static_cast<int64_t>(kThreads) * per_thread);
    const int64_t cap    = static_cast<int64_t>(sm_count) * 8; // whole multiples of the SM count
    return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}
} // namespace

cugl_status launch_reduce_rows(cugl_context *ctx, const void *d_a, bool is_signed, int M, int K, int64_t lda,
                               int32_t scalar, int32_t *d_out)
{
    if (M <= 0) return CUGL_SUCCESS;
    const int rows_per_block = kThreads / 32;
    const int blocks         = grid_for(static_cast<int64_t>(M) * 32, ctx->sm_count);
    (void)rows_per_block;
    reduce_rows_kernel<<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_a), is_signed, M, K, lda,
                                                             scalar, d_out);
    return check_cuda(ctx, cudaGetLastError(), "reduce_rows_kernel");
}

cugl_status launch_reduce_cols(cugl_context *ctx, const void *d_b, bool is_signed, int K, int N, int64_t ldb,
                               int32_t scalar, int32_t *d_out)
{
    if (N <= 0) return CUGL_SUCCESS;
    CUGL_CUDA_TRY(ctx, cudaMemsetAsync(d_out, 0, sizeof(int32_t) * N, ctx->stream));
    if (K > 0)
    {
        const bool aligned = ((reinterpret_cast<uintptr_t>(d_b) | static_cast<uint64_t>(ldb)) & 15) == 0;
        const int  n_vec   = aligned ? N / 16 : 0; // 16-column units read with 128-bit loads
        // enough K slabs to fill the machine a few times over, at least 32 rows each, at most kColSlabRows
        auto slab_rows = [&](int gx) {
            int slabs = (ctx->sm_count * 4 + gx - 1) / gx;
            slabs     = max(1, min(slabs, (K + 31) / 32));
            return min(kColSlabRows, (K + slabs - 1) / slabs);
        };
        if (n_vec > 0)
        {
            const int gx          = (n_vec + kThreads - 1) / kThreads;
            const int k_per_block = slab_rows(gx);
            reduce_cols_kernel<<<dim3(gx, (K + k_per_block - 1) / k_per_block), kThreads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(d_b), is_signed, K, n_vec, ldb, k_per_block, d_out);
            CUGL_TRY(check_cuda(ctx, cudaGetLastError(), "reduce_cols_kernel"));
        }
        if (16 * n_vec < N)
        {
            const int gx          = (N - 16 * n_vec + kThreads - 1) / kThreads;
            const int k_per_block = slab_rows(gx);
            reduce_cols_generic_kernel<<<dim3(gx, (K + k_per_block - 1) / k_per_block), kThreads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(d_b), is_signed, K, 16 * n_vec, N, ldb, k_per_block, d_out);
            CUGL_TRY(check_cuda(ctx, cudaGetLastError(), "reduce_cols_generic_kernel"));
        }
    }
    if (scalar != 1)
    {
        scale_vector_kernel<<<(N + 255) / 256, 256, 0, ctx->stream>>>(d_out, N, scalar);
        CUGL_TRY(check_cuda(ctx, cudaGetLastError(), "scale_vector_kernel"));
    }
    return CUGL_SUCCESS;
}

cugl_status launch_transpose_colsum(cugl_context *ctx, const void *d_b, bool is_signed, int K, int N, int64_t ldb,
                                    void *d_bt, int64_t ldbt, int32_t *d_colsum)
{
    if (d_colsum != nullptr)
    {
        CUGL_CUDA_TRY(ctx, cudaMemsetAsync(d_colsum, 0, sizeof(int32_t) * N, ctx->stream));
    }
    if (K <= 0 || N <= 0) return CUGL_SUCCESS;
    dim3 grid((N + 63) / 64, (K + 63) / 64);
    const uint64_t bits = reinterpret_cast<uintptr_t>(d_b) | reinterpret_cast<uintptr_t>(d_bt) | static_cast<uint64_t>(ldb) |
                          static_cast<uint64_t>(ldbt) | static_cast<uint64_t>(K) | static_cast<uint64_t>(N);
    if ((bits & 3) == 0)
    {
        transpose_colsum_words_kernel<<<grid, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_b), is_signed, K, N,
                                                                          ldb, static_cast<uint8_t *>(d_bt), ldbt, d_colsum);
    }
    else
    {
        transpose_colsum_kernel<<<grid, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_b), is_signed, K, N,
                                                                    ldb, static_cast<uint8_t *>(d_bt), ldbt, d_colsum);
    }
    return check_cuda(ctx, cudaGetLastError(), "transpose_colsum_kernel");
}

cugl_status launch_transpose_bytes(cugl_context *ctx, const void *d_src, int rows, int cols, void *d_dst, int batch)
{
    if (rows <= 0 || cols <= 0 || batch <= 0) return CUGL_SUCCESS;
    dim3 grid((cols + 63) / 64, (rows + 63) / 64, batch);
    transpose_bytes_kernel<<<grid, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_src), rows, cols,
                                                               static_cast<uint8_t *>(d_dst));
    return check_cuda(ctx, cudaGetLastError(), "transpose_bytes_kernel");
}

cugl_status launch_offset_contribution(cugl_context *ctx, int32_t *d_mm, int M, int N, int K, int64_t ld_bytes,
                                       const int32_t *d_colsum, const int32_t *d_rowsum, int32_t a_off,
                                       int32_t b_off)
{
    if (M <= 0 || N <= 0) return CUGL_SUCCESS;
    const int32_t k_term = (a_off != 0 && b_off != 0)
                               ? static_cast<int32_t>(static_cast<uint32_t>(a_off) * static_cast<uint32_t>(b_off) *
                                                      static_cast<uint32_t>(K))
                               : 0;
    const int  groups = (N + 3) / 4;
    const int  gx     = max(1, min((groups + kThreads - 1) / kThreads, 8));
    const int  gy     = max(1, min(M, ctx->sm_count * 16 / gx));
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(d_mm) | static_cast<uint64_t>(ld_bytes) |
                          reinterpret_cast<uintptr_t>(d_colsum)) & 15) == 0;
    offset_contribution_kernel<<<dim3(gx, gy), kThreads, 0, ctx->stream>>>(d_mm, M, N, ld_bytes / 4,
                                                                           a_off != 0 ? d_colsum : nullptr,
                                                                           b_off != 0 ? d_rowsum : nullptr, a_off, b_off,
                                                                           k_term, vec_ok);
    return check_cuda(ctx, cudaGetLastError(), "offset_contribution_kernel");
}

cugl_status launch_output_stage(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes, const int32_t *d_bias,
                                void *d_out, int64_t ld_out_bytes, int M, int N, const int32_t *d_mults,
                                const int32_t *d_shifts, int32_t mult, int32_t shift, int32_t offset, int32_t lo,
                                int32_t hi, bool integer_stage, bool out16)
{
    if (M <= 0 || N <= 0) return CUGL_SUCCESS;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(d_in) | static_cast<uint64_t>(ld_in_bytes)) & 15) == 0 &&
                        ((reinterpret_cast<uintptr_t>(d_out) | static_cast<uint64_t>(ld_out_bytes)) & (out16 ? 7 : 3)) == 0;
    const int  gx = ((N + 3) / 4 + kThreads - 1) / kThreads;
    const int  gy = max(1, min(M, (ctx->sm_count * 16 + gx - 1) / gx));
    const dim3 blocks(gx, gy);
    if (out16)
    {
        output_stage_kernel<true><<<blocks, kThreads, 0, ctx->stream>>>(
            d_in, ld_in_bytes / 4, d_bias, static_cast<uint8_t *>(d_out), ld_out_bytes, M, N, d_mults, d_shifts, mult,
            shift, offset, lo, hi, vec_ok, integer_stage);
    }
    else
    {
        output_stage_kernel<false><<<blocks, kThreads, 0, ctx->stream>>>(
            d_in, ld_in_bytes / 4, d_bias, static_cast<uint8_t *>(d_out), ld_out_bytes, M, N, d_mults, d_shifts, mult,
            shift, offset, lo, hi, vec_ok, integer_stage);
    }
    return check_cuda(ctx, cudaGetLastError(), "output_stage_kernel");
}

cugl_status launch_im2col_nhwc(cugl_context *ctx, const void *d_src, void *d_dst, int C, int W, int H, int B, int kw,
                               int kh, int sx, int sy, int pad_l, int pad_t, int dil_x, int dil_y, int Wo, int Ho,
                               int pad_value, int64_t row_stride)
{
    const int64_t M64 = static_cast<int64_t>(B) * Ho * Wo;
    if (M64 <= 0) return CUGL_SUCCESS;
    if (M64 >= (1ll << 31) || row_stride >= (1ll << 24))
    {
        return fail(ctx, CUGL_UNSUPPORTED_CONFIG, "im2col: more than 2^31 output rows or rows of 16 MB and more");
    }
    const int      M        = static_cast<int>(M64);
    const uint32_t pb       = static_cast<uint32_t>(pad_value) & 0xffu;
    const uint32_t pad_word = pb * 0x01010101u;
    const bool     vec16    = (C % 16 == 0) && (row_stride % 16 == 0) &&
                       ((reinterpret_cast<uintptr_t>(d_src) | reinterpret_cast<uintptr_t>(d_dst)) & 15) == 0;
    const int vec   = vec16 ? 16 : 1;
    const int units = static_cast<int>(row_stride / vec);
    // about four units per thread and step, whole rows
    const int rows_per_iter = max(1, min(M, (4 * kThreads + units - 1) / units));
    Im2colDivs dv;
    dv.units = make_fastdiv(units);
    dv.c     = make_fastdiv(C);
    dv.kw    = make_fastdiv(kw);
    dv.wo    = make_fastdiv(Wo);
    dv.ho    = make_fastdiv(Ho);
    const int blocks = grid_for((static_cast<int64_t>(M) + rows_per_iter - 1) / rows_per_iter * kThreads, ctx->sm_count);
    if (vec16)
    {
        im2col_nhwc_kernel<16><<<blocks, kThreads, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), C, W, H, M, kw, kh, sx, sy, pad_l,
            pad_t, dil_x, dil_y, Wo, Ho, pad_word, row_stride, rows_per_iter, dv);
    }
    else
    {
        im2col_nhwc_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), C, W, H, M, kw, kh, sx, sy, pad_l,
            pad_t, dil_x, dil_y, Wo, Ho, pad_word, row_stride, rows_per_iter, dv);
    }
    return check_cuda(ctx, cudaGetLastError(), "im2col_nhwc_kernel");
}
cugl_status launch_fold_input(cugl_context *ctx, const void *d_src, void *d_dst, int B, int H, int W, int C, int H2,
                              int W2, int zero_point)
{
    const int blocks = grid_for(static_cast<int64_t>(B) * H2 * W2, ctx->sm_count);
    const bool fast = C == 3 && (W & 1) == 0 && (reinterpret_cast<uintptr_t>(d_src) & 1) == 0 &&
                      static_cast<int64_t>(B) * H2 * W2 <= 0x7fffffff;
    if (fast)
    {
        fold_input_kernel<true><<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_src),
                                                                      static_cast<uint8_t *>(d_dst), B, H, W, C, H2, W2,
                                                                      static_cast<uint32_t>(zero_point) & 0xffu);
    }
    else
    {
        fold_input_kernel<false><<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_src),
                                                                       static_cast<uint8_t *>(d_dst), B, H, W, C, H2, W2,
                                                                       static_cast<uint32_t>(zero_point) & 0xffu);
    }
    return check_cuda(ctx, cudaGetLastError(), "fold_input_kernel");
}

cugl_status launch_fold_weights(cugl_context *ctx, const void *d_w, void *d_bt, int64_t ldbt, int OFM, int kh, int kw,
                                int C, int kh2, int kw2, int oy, int ox)
{
    const int blocks = grid_for(static_cast<int64_t>(OFM) * kh2 * kw2 * 16, ctx->sm_count);
    fold_weights_kernel<<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint8_t *>(d_w),
                                                              static_cast<uint8_t *>(d_bt), ldbt, OFM, kh, kw, C, kh2,
                                                              kw2, oy, ox);
    return check_cuda(ctx, cudaGetLastError(), "fold_weights_kernel");
}
} // namespace cugl
