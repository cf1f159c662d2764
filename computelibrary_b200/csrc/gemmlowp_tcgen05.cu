// Quantized GEMM on the 5th-generation tensor cores (sm_100a): the replacement for the arm_gemm
// requantising int8 kernels (src/core/NEON/kernels/arm_gemm/gemm_qint8.cpp, quantized.cpp:55-267) and
// for CpuGemmLowpOffsetContributionOutputStageKernel, fused into one persistent kernel.
//
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A [128 x 128 B] and Bt [BLOCK_N x 128 B]
//               into a STAGES-deep ring of 128-byte-swizzled shared-memory buffers
//   warp 1      MMA issuer: tcgen05.mma.cta_group::1.kind::i8, M=128, N=BLOCK_N, K=32 per instruction,
//               int32 accumulators in tensor memory, double buffered (2 x BLOCK_N columns)
//   warps 2..5  epilogue: tcgen05.ld the accumulator rows, add the offset / bias terms, requantise
//               with the reference's SQDMULH + rounding shift, clamp, and store 8-bit (or int32) rows
//
// The epilogue of tile i overlaps the main loop of tile i+1 through the two accumulator buffers.
// Every wait is bounded: when a limit runs out the kernel raises a flag in shared memory, every role
// leaves its loop, the producer waits (bounded) for its copies in flight, tensor memory is freed and
// a status word is written for the host.
#include "kernels.cuh"

#include <cuda.h>

namespace cugl
{
namespace
{
constexpr int      BLOCK_M     = 128;
constexpr int      BLOCK_K     = 128; // bytes == int8 elements: one 128-byte swizzle row
constexpr int      UMMA_K      = 32;  // K per tcgen05.mma.kind::i8
constexpr int      kThreads    = 192;
constexpr int      kEpiThreads = 128;
constexpr int      A_STAGE     = BLOCK_M * BLOCK_K;
constexpr long long kSpinLimit = 4000000000ll; // clock64 ticks, about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t"
                 ".reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t"
                 "}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code)
{
    if (mbar_try_wait(bar, parity))
    {
        return true;
    }
    const long long t0 = clock64();
    uint32_t        n  = 0;
    while (!mbar_try_wait(bar, parity))
    {
        if ((++n & 0xff) == 0)
        {
            if (*abort_flag != 0)
            {
                return false;
            }
            if (clock64() - t0 > kSpinLimit)
            {
                *abort_flag = code;
                return false;
            }
        }
    }
    return true;
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :
                 : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// ---- tcgen05 -------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; 128 x BLOCK_N x 32, u8/s8 operands, int32 accumulate.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate)
{
    asm volatile("{\n\t"
                 ".reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
                 "}"
                 :
                 : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// mbarrier arrives once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                   "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                   "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                   "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle TMA applied: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte
// offset is unused for swizzled K-major tiles (set to 1), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Named barrier over the four epilogue warps that also AND-reduces a predicate, so that the warps
// take the "carry on / give up" decision together.
__device__ __forceinline__ bool epi_barrier_and(bool pred)
{
    uint32_t r;
    asm volatile("{\n\t"
                 ".reg .pred p, q;\n\t"
                 "setp.ne.u32 q, %1, 0;\n\t"
                 "bar.red.and.pred p, 1, 128, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t"
                 "}"
                 : "=r"(r)
                 : "r"(static_cast<uint32_t>(pred))
                 : "memory");
    return r != 0;
}
__device__ __forceinline__ void epi_barrier()
{
    asm volatile("bar.sync 2, 128;" ::: "memory");
}

struct TileParams
{
    uint8_t *dst;
    int64_t  ldd;
    int      M, N, K;
    uint32_t idesc;
    int      vec_ok; // dst base and ldd are 16-byte aligned
    int32_t *status;
};

template <int BLOCK_N, int STAGES>
struct SmemPlan
{
    static constexpr int B_STAGE    = BLOCK_N * BLOCK_K;
    static constexpr int STAGE      = A_STAGE + B_STAGE;
    static constexpr int OFF_A      = 0;
    static constexpr int OFF_B      = STAGES * A_STAGE;
    static constexpr int OFF_COL    = STAGES * STAGE;             // int4 per column
    static constexpr int OFF_BAR    = OFF_COL + BLOCK_N * 16;     // full[S], empty[S], tfull[2], tempty[2]
    static constexpr int OFF_MISC   = OFF_BAR + (2 * STAGES + 4) * 8; // tmem base, abort flag
    static constexpr int TOTAL      = OFF_MISC + 16;
    static constexpr int DYN_BYTES  = TOTAL + 1024;               // slack to align the base to 1024
    static constexpr int TMEM_COLS  = 2 * BLOCK_N;
};

template <int BLOCK_N, int STAGES, bool kS32Out>
__global__ void __launch_bounds__(kThreads, 1)
    gemmlowp_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const TileParams tp, const EpilogueParams ep)
{
    using P = SmemPlan<BLOCK_N, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const uint32_t sA       = smem_u32(smem + P::OFF_A);
    const uint32_t sB       = smem_u32(smem + P::OFF_B);
    int4          *s_col    = reinterpret_cast<int4 *>(smem + P::OFF_COL);
    const uint32_t bar_base = smem_u32(smem + P::OFF_BAR);
    auto           full_bar   = [&](int s) { return bar_base + 8u * s; };
    auto           empty_bar  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto           tfull_bar  = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto           tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    uint32_t      *s_tmem     = reinterpret_cast<uint32_t *>(smem + P::OFF_MISC);
    volatile int  *s_abort    = reinterpret_cast<volatile int *>(smem + P::OFF_MISC + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int num_m_blocks = (tp.M + BLOCK_M - 1) / BLOCK_M;
    const int num_n_blocks = (tp.N + BLOCK_N - 1) / BLOCK_N;
    const int num_tiles    = num_m_blocks * num_n_blocks;
    const int num_kb       = (tp.K + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a)
        {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kEpiThreads);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1)
    {
        tmem_alloc(smem_u32(s_tmem), P::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp == 0)
    {
        // ---------------------------------------------------------------- TMA producer
        int      s = 0;
        uint32_t ph = 0, issued = 0, parities = 0;
        bool     ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x)
        {
            const int m0 = (tile % num_m_blocks) * BLOCK_M;
            const int n0 = (tile / num_m_blocks) * BLOCK_N;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1, s_abort, DEV_TIMEOUT_PRODUCER));
                if (!ok)
                {
                    break;
                }
                if (lane == 0)
                {
                    mbar_expect_tx(full_bar(s), P::STAGE);
                    tma_load_2d(sA + s * A_STAGE, &tmap_a, kb * BLOCK_K, m0, full_bar(s));
                    tma_load_2d(sB + s * P::B_STAGE, &tmap_b, kb * BLOCK_K, n0, full_bar(s));
                }
                issued |= 1u << s;
                parities = (parities & ~(1u << s)) | (ph << s);
                __syncwarp();
                if (++s == STAGES)
                {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        if (!ok || *s_abort != 0)
        {
            // wait, with a limit of its own, until the copies already issued have landed
            for (int i = 0; i < STAGES; ++i)
            {
                if ((issued >> i) & 1u)
                {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(full_bar(i), (parities >> i) & 1u))
                    {
                        if (clock64() - t0 > kSpinLimit / 4)
                        {
                            *s_abort = DEV_TIMEOUT_DRAIN;
                            break;
                        }
                    }
                }
            }
        }
    }
    else if (warp == 1)
    {
        // ---------------------------------------------------------------- MMA issuer
        int      s = 0, as = 0;
        uint32_t ph = 0, aph = 0;
        bool     ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x)
        {
            ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(as), aph ^ 1, s_abort, DEV_TIMEOUT_MMA));
            if (!ok)
            {
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * BLOCK_N;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_MMA));
                if (!ok)
                {
                    break;
                }
                tc_fence_after();
                if (lane == 0)
                {
                    const uint64_t a_desc = make_kmajor_sw128_desc(sA + s * A_STAGE);
                    const uint64_t b_desc = make_kmajor_sw128_desc(sB + s * P::B_STAGE);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                    {
                        // advancing K by 32 bytes inside the swizzle row: +2 in 16-byte units
                        umma_i8(d_tmem, a_desc + 2u * k, b_desc + 2u * k, tp.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s)); // frees the smem stage once these MMAs have read it
                }
                __syncwarp();
                if (++s == STAGES)
                {
                    s = 0;
                    ph ^= 1;
                }
            }
            if (ok && lane == 0)
            {
                umma_commit(tfull_bar(as)); // accumulator complete
            }
            __syncwarp();
            if (++as == 2)
            {
                as = 0;
                aph ^= 1;
            }
        }
    }
    else
    {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        const int quad = warp & 3;          // tensor-memory lane quarter this warp may read
        const int et   = threadIdx.x - 64;  // 0..127
        const int r_in = quad * 32 + lane;  // row inside the tile
        int       as = 0;
        uint32_t  aph = 0;
        bool      ok = true;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x)
        {
            if (!epi_barrier_and(ok))
            {
                break;
            }
            const int m0 = (tile % num_m_blocks) * BLOCK_M;
            const int n0 = (tile / num_m_blocks) * BLOCK_N;
            // per-column terms of this tile: {offset + bias term, multiplier, right | left << 8, 0}
            for (int c = et; c < BLOCK_N; c += kEpiThreads)
            {
                const int n = n0 + c;
                int4      q = make_int4(0, 0, 0, 0);
                if (n < tp.N)
                {
                    int32_t t = ep.k_term;
                    if (ep.colsum != nullptr) t += ep.a_off * __ldg(ep.colsum + n);
                    if (ep.bias != nullptr) t += __ldg(ep.bias + n);
                    const int32_t sh = ep.shifts != nullptr ? __ldg(ep.shifts + n) : ep.shift;
                    q.x              = t;
                    q.y              = ep.mults != nullptr ? __ldg(ep.mults + n) : ep.mult;
                    q.z              = max(sh, 0) | (max(-sh, 0) << 8);
                }
                s_col[c] = q;
            }
            epi_barrier();
            ok = mbar_wait(tfull_bar(as), aph, s_abort, DEV_TIMEOUT_EPILOGUE);
            if (ok)
            {
                tc_fence_after();
                const int     m        = m0 + r_in;
                const bool    row_ok   = m < tp.M;
                const int32_t row_term = (ep.rowsum != nullptr && row_ok) ? ep.b_off * __ldg(ep.rowsum + m) : 0;
                const uint32_t t_row   = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * BLOCK_N;
                uint8_t *drow = tp.dst + static_cast<int64_t>(m) * tp.ldd;
#pragma unroll 1
                for (int ch = 0; ch < BLOCK_N / 32; ++ch)
                {
                    uint32_t v[32];
                    tmem_ld_x32(t_row + ch * 32, v);
                    tmem_ld_wait();
                    const int  nc   = n0 + ch * 32;
                    const bool full = nc + 32 <= tp.N;
                    if (kS32Out)
                    {
                        int32_t *o = reinterpret_cast<int32_t *>(drow) + nc;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                        {
                            v[j] = static_cast<uint32_t>(static_cast<int32_t>(v[j]) + s_col[ch * 32 + j].x + row_term);
                        }
                        if (row_ok)
                        {
                            if (full && tp.vec_ok)
                            {
#pragma unroll
                                for (int j = 0; j < 32; j += 4)
                                {
                                    *reinterpret_cast<uint4 *>(o + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                }
                            }
                            else
                            {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                {
                                    if (nc + j < tp.N) o[j] = static_cast<int32_t>(v[j]);
                                }
                            }
                        }
                    }
                    else
                    {
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                        {
                            uint32_t packed = 0;
#pragma unroll
                            for (int b = 0; b < 4; ++b)
                            {
                                const int4    q   = s_col[ch * 32 + j + b];
                                const int32_t acc = static_cast<int32_t>(v[j + b]) + q.x + row_term;
                                const int32_t r   = finalize(acc, q.y, q.z >> 8, q.z & 0xff, ep.result_offset, ep.lo,
                                                             ep.hi);
                                packed |= (static_cast<uint32_t>(r) & 0xffu) << (8 * b);
                            }
                            w[j >> 2] = packed;
                        }
                        if (row_ok)
                        {
                            uint8_t *o = drow + nc;
                            if (full && tp.vec_ok)
                            {
                                *reinterpret_cast<uint4 *>(o)      = make_uint4(w[0], w[1], w[2], w[3]);
                                *reinterpret_cast<uint4 *>(o + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                            }
                            else
                            {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                {
                                    if (nc + j < tp.N) o[j] = static_cast<uint8_t>(w[j >> 2] >> (8 * (j & 3)));
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(tempty_bar(as)); // accumulator buffer may be overwritten
            }
            if (++as == 2)
            {
                as = 0;
                aph ^= 1;
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
    {
        tc_fence_after();
        tmem_dealloc(tmem_base, P::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s_abort != 0)
    {
        atomicCAS(tp.status, 0, *s_abort);
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void                           *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
        {
            (void)cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// rows x K bytes, K contiguous, row stride ld; box = box_rows x 128 bytes, 128-byte swizzle; elements
// outside [0,K) x [0,rows) read as zero, which is what makes ragged M / N / K tiles exact.
bool encode_operand_map(CUtensorMap *map, const void *base, int rows, int K, int64_t ld, int box_rows)
{
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr)
    {
        return false;
    }
    const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
    const cuuint32_t box[2]     = {static_cast<cuuint32_t>(BLOCK_K), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2]    = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BLOCK_N, int STAGES, bool kS32Out>
cugl_status launch_variant(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    using P = SmemPlan<BLOCK_N, STAGES>;
    static_assert(P::DYN_BYTES <= 227 * 1024, "shared memory plan exceeds the sm_100 limit");
    CUtensorMap map_a, map_b;
    if (!encode_operand_map(&map_a, op.a, op.M, op.K, op.lda, BLOCK_M) ||
        !encode_operand_map(&map_b, op.bt, op.N, op.K, op.ldbt, BLOCK_N))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for a GEMM operand");
    }
    auto kernel = gemmlowp_tcgen05_kernel<BLOCK_N, STAGES, kS32Out>;
    static bool attr_set = false; // per instantiation
    if (!attr_set)
    {
        CUGL_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::DYN_BYTES));
        attr_set = true;
    }
    TileParams tp;
    tp.dst    = static_cast<uint8_t *>(op.dst);
    tp.ldd    = op.ldd;
    tp.M      = op.M;
    tp.N      = op.N;
    tp.K      = op.K;
    tp.idesc  = (2u << 4) | ((op.a_signed ? 1u : 0u) << 7) | ((op.b_signed ? 1u : 0u) << 10) |
               (static_cast<uint32_t>(BLOCK_N >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
    tp.vec_ok = ((reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd)) & 15) == 0;
    tp.status = ctx->d_status;
    const int tiles = ((op.M + BLOCK_M - 1) / BLOCK_M) * ((op.N + BLOCK_N - 1) / BLOCK_N);
    const int grid  = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    kernel<<<grid, kThreads, P::DYN_BYTES, ctx->stream>>>(map_a, map_b, tp, ep);
    return check_cuda(ctx, cudaGetLastError(), "gemmlowp_tcgen05_kernel");
}
} // namespace

bool gemmlowp_tcgen05_supported(const GemmOperands &op)
{
    if (op.M <= 0 || op.N <= 0 || op.K <= 0)
    {
        return false;
    }
    const uint64_t bits = reinterpret_cast<uintptr_t>(op.a) | reinterpret_cast<uintptr_t>(op.bt) |
                          static_cast<uint64_t>(op.lda) | static_cast<uint64_t>(op.ldbt);
    return (bits & 15) == 0 && get_encode_fn() != nullptr;
}

cugl_status launch_gemmlowp_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    const bool s32 = ep.stage == CUGL_STAGE_NONE;
    if (op.N > 128)
    {
        return s32 ? launch_variant<256, 4, true>(ctx, op, ep) : launch_variant<256, 4, false>(ctx, op, ep);
    }
    if (op.N > 64)
    {
        return s32 ? launch_variant<128, 6, true>(ctx, op, ep) : launch_variant<128, 6, false>(ctx, op, ep);
    }
    return s32 ? launch_variant<64, 8, true>(ctx, op, ep) : launch_variant<64, 8, false>(ctx, op, ep);
}
} // namespace cugl
