// Quantized GEMM on the 5th-generation tensor cores (sm_100a): the replacement for the arm_gemm
// requantising int8 kernels (src/core/NEON/kernels/arm_gemm/gemm_qint8.cpp, quantized.cpp:55-267) and
// for CpuGemmLowpOffsetContributionOutputStageKernel, fused into one persistent kernel.
//
//   producer warp(s)  TMA: cp.async.bulk.tensor tiles of A [128 x 128 B] and Bt [BLOCK_N x 128 B] into a
//                     STAGES-deep ring of 128-byte-swizzled shared-memory buffers (KSUB K sub-blocks per stage)
//   MMA warp          one lane issues tcgen05.mma.cta_group::1.kind::i8, M=128, N=BLOCK_N, K=32 per
//                     instruction; int32 accumulators in tensor memory, double buffered (2 x BLOCK_N columns)
//   epilogue warps    one (or two) per tensor-memory lane quarter: tcgen05.ld the accumulator rows, add the
//                     offset / bias terms, requantise with the reference's SQDMULH + rounding shift, clamp,
//                     and store 8-bit (or int32) rows
// Warp counts are compile-time (CUGL_PROD_WARPS, CUGL_EPI_WARPS); one producer and four epilogue warps
// measured fastest: every extra resident warp competes for issue slots with the single-thread issue loops.
//
// The epilogue of tile i overlaps the main loop of tile i+1 through the two accumulator buffers.
//
// Two kernels share these roles.  gemmlowp_tcgen05_kernel runs one CTA per 128 x BLOCK_N tile.
// gemmlowp_tcgen05_2cta_kernel runs a cluster of two CTAs (one SM pair) per 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and only HALF of the B tile, the
// tensor cores of both SMs read both halves, so 64 instead of 96 bytes are fetched from L2 per clock
// of tensor work and the same shared memory holds six stages instead of four.  No load is multicast.
//
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
#ifndef CUGL_PROD_WARPS
#define CUGL_PROD_WARPS 1
#endif
#ifndef CUGL_EPI_WARPS
#define CUGL_EPI_WARPS 4
#endif
// This file is compiled once per epilogue-warp count (gemmlowp_tcgen05_epi8.cu includes it with
// CUGL_EPI_WARPS = 8): four epilogue warps leave the issue slots to the single-thread producer and MMA loops,
// which is what long-K GEMMs want; short-K tiles spend their time in the epilogue and want eight.  The
// entry points carry the count in their names and gemmlowp_dispatch.cu chooses between them.
#define CUGL_TC_CAT2(a, b) a##_epi##b
#define CUGL_TC_CAT(a, b) CUGL_TC_CAT2(a, b)
#define CUGL_TC_NAME(x) CUGL_TC_CAT(x, CUGL_EPI_WARPS)
constexpr int      kProdWarps  = CUGL_PROD_WARPS;          // producer warps (one issuing lane each)
constexpr int      kProdLanes  = kProdWarps;               // independent copy issuers per CTA
constexpr int      kMmaWarp    = kProdWarps;               // index of the MMA-issuing warp
constexpr int      kFirstEpi   = kProdWarps + 1;           // first epilogue warp
constexpr int      kEpiWarps   = CUGL_EPI_WARPS;           // a multiple of 4: one or two per tensor-memory lane quarter
constexpr int      kEpiThreads = kEpiWarps * 32;
constexpr int      kThreads    = 32 * (kProdWarps + 1) + kEpiThreads;
static_assert(kEpiWarps == 4 || kEpiWarps == 8 || kEpiWarps == 16, "epilogue warps: 4, 8 or 16");
// The sixteen-warp build holds only the one-CTA GEMM kernels with 256-column tiles (row-major and channel-major):
// the kernels for short K and wide outputs, whose epilogue wants the most latency hiding.
#define CUGL_TC_FULL_BUILD (CUGL_EPI_WARPS <= 8)
constexpr int      A_STAGE     = BLOCK_M * BLOCK_K;

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
// The barrier's state without waiting: try_wait may suspend the thread for a hardware-chosen time when the phase is not
// complete, which a look-ahead that has other work to issue must not do.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t"
                 ".reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t"
                 "}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code, long long limit)
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
            if (clock64() - t0 > limit)
            {
                *abort_flag = code;
                return false;
            }
        }
    }
    return true;
}

// Programmatic dependent launch.  launch_dependents: the next kernel of the stream may be scheduled (it starts on SMs
// this grid has left, or never used) and run its prologue; wait: returns once the preceding kernel has completed and
// its memory operations are visible -- every access to global memory of a kernel launched that way comes after it.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void griddep_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :
                 : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// Im2col-mode tile load (NHWC tensor map made by cuTensorMapEncodeIm2col): BLOCK_M window origins starting at
// (w, h, n) and walking w, then h, then n inside the map's bounding box, channels [c, c + 128) of the pixel at
// origin + (off_w, off_h); pixels outside the image and origins beyond the last image read as zero.
__device__ __forceinline__ void tma_load_im2col(uint32_t dst, const CUtensorMap *map, int c, int w, int h, int n,
                                                uint16_t off_w, uint16_t off_h, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 :
                 : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
                   "h"(off_h)
                 : "memory");
}

// the same load in a cta_group::2 pipeline: the bytes are credited to the barrier at bar_cluster_addr in the leader CTA
__device__ __forceinline__ void tma_load_im2col_pair(uint32_t dst, const CUtensorMap *map, int c, int w, int h, int n,
                                                     uint16_t off_w, uint16_t off_h, uint32_t bar_cluster_addr)
{
    asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 :
                 : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c), "r"(w), "r"(h), "r"(n),
                   "h"(off_w), "h"(off_h)
                 : "memory");
}

// Tile store: a shared-memory box (written by ordinary stores, then fence_proxy_async_smem and a warp barrier) to global
// memory through the TMA unit; rows and columns beyond the tensor's extent are clipped.  Bulk-group completion: commit,
// then wait until the group's shared-memory reads (tma_store_wait_read) or all of it (tma_store_wait_all) are done.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
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

// The same for rows of 64 bytes in the 64-byte swizzle (the patch tiles of a 64-channel convolution: one filter tap per
// tile): 8-row groups 512 bytes apart, layout type 4.
__device__ __forceinline__ uint64_t make_kmajor_sw64_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(512 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(4) << 61;
    return d;
}

// Optional tracing: event e of the i-th tile this CTA processes, as a %globaltimer value (ns).
// Layout: trace[(cta * kTraceTiles + i) * kTraceEvents + e].  Events: 0 producer issued the first copy,
// 1 MMA issuer owns an accumulator, 2 first operand stage has landed, 3 last MMA issued, 4 epilogue sees the
// finished accumulator, 5 epilogue has stored the tile; slot 6 = clocks the MMA issuer waited for operands;
// 7 (convolution kernel) the gather warps have issued the tile's last copies.
constexpr int kTraceTiles  = 8;
constexpr int kTraceEvents = 8;
__device__ __forceinline__ void trace_event(long long *trace, int i, int e)
{
    if (trace != nullptr && i < kTraceTiles)
    {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        trace[(static_cast<long long>(blockIdx.x) * kTraceTiles + i) * kTraceEvents + e] = static_cast<long long>(t);
    }
}

__device__ __forceinline__ void trace_value(long long *trace, int i, int e, long long v)
{
    if (trace != nullptr && i < kTraceTiles)
    {
        trace[(static_cast<long long>(blockIdx.x) * kTraceTiles + i) * kTraceEvents + e] = v;
    }
}

// Named barrier over the eight epilogue warps that also AND-reduces a predicate, so that the warps
// take the "carry on / give up" decision together.
__device__ __forceinline__ bool epi_barrier_and(bool pred)
{
    uint32_t r;
    asm volatile("{\n\t"
                 ".reg .pred p, q;\n\t"
                 "setp.ne.u32 q, %1, 0;\n\t"
                 "bar.red.and.pred p, 1, %2, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t"
                 "}"
                 : "=r"(r)
                 : "r"(static_cast<uint32_t>(pred)), "n"(kEpiThreads)
                 : "memory");
    return r != 0;
}
__device__ __forceinline__ void epi_barrier()
{
    asm volatile("bar.sync 2, %0;" ::"n"(kEpiThreads) : "memory");
}
// The same two barriers for one of two epilogue groups of four warps (named barriers 3..6).
__device__ __forceinline__ bool epi_group_barrier_and(bool pred, int group)
{
    uint32_t r;
    asm volatile("{\n\t"
                 ".reg .pred p, q;\n\t"
                 "setp.ne.u32 q, %1, 0;\n\t"
                 "bar.red.and.pred p, %2, 128, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t"
                 "}"
                 : "=r"(r)
                 : "r"(static_cast<uint32_t>(pred)), "r"(3 + group)
                 : "memory");
    return r != 0;
}
__device__ __forceinline__ void epi_group_barrier(int group)
{
    asm volatile("bar.sync %0, 128;" ::"r"(5 + group) : "memory");
}

constexpr int kMaxExtraDst = 7; // push all-gather: this GPU's tile is also stored into up to 7 peers

struct TileParams
{
    uint8_t *dst;
    uint8_t *extra_dst[kMaxExtraDst]; // further copies of the output (peer GPUs' buffers), same ldd
    int      n_extra;
    int64_t  ldd;
    int      M, N, K;
    uint32_t idesc;
    int      vec_ok;  // row-major: vector_flags() of dst base, ldd and residual; channel-major: rows 8-byte aligned
    int      mode;    // kStageGeneric / kStageFast / kStageWide: encoding of the column terms (requant_pack4)
    uint32_t idesc_half; // SM-pair kernel: instruction descriptor of a half-width (N = 128) tile
    int      split_tail; // SM-pair kernel: split the tiles of a short last wave in two (see the kernel)
    const uint8_t *residual; // optional [M][ldd] bytes added to the output with unsigned saturation, then clamped
    uint32_t res_floor4, res_cap4; // the clamp bounds replicated into four bytes
    int      pair_drain; // one-CTA kernel, two accumulator buffers: drain two tiles of one column block together
    long long *trace; // optional per-CTA event timestamps (cugl_context_set_trace_buffer), else nullptr
    int32_t *status;
    int      raw_f32, raw_accumulate; // stage NONE: float destination / dst += result (EpilogueParams::out_f32, accumulate)
    float    raw_scale;               // dequantization scale of a float destination
    // Implicit convolution (conv_c != 0): tmap_a is an im2col-mode map of the NHWC input with 128 channels per load, a
    // tile row is an output pixel and the K axis runs over (ky, kx, c).  Exact for an input zero point of 0 only (the
    // fill value of out-of-image taps), and for C a multiple of 128.
    int      conv_c, conv_kw, conv_wo, conv_ho, conv_sx, conv_sy, conv_pl, conv_pt, conv_dx, conv_dy;
    FastDiv  conv_div_wo, conv_div_ho;
    int      tma_store;               // one-CTA row-major kernels: staged groups leave as bulk tensor stores (tmap_out)
    long long spin_limit;             // clock64 ticks a wait on a barrier may last before the kernel gives up
    int      withhold_kb;             // >= 0: CTA 0 leaves out the copies of this k-block ordinal (test instrument
                                      // of the give-up path, cugl_context_withhold_copy_once); -1 otherwise
};


// ---- cluster / cta_group::2 primitives ------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t num_clusters_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a cta_group::2 pipeline: data lands in this CTA's shared memory, the byte count is
// credited to the barrier at `bar_cluster_addr`, which lives in the leader CTA.  Not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t bar_cluster_addr)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];"
                 :
                 : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// 256 x N x 32 across the SM pair: each CTA contributes 128 rows of A and N/2 rows of B.
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate)
{
    asm volatile("{\n\t"
                 ".reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
                 "}"
                 :
                 : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so
// far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :
                 : "r"(bar), "h"(mask)
                 : "memory");
}

// Requantise + clamp + pack four accumulators of one row (columns c .. c+3 of the tile).  Three encodings of
// the per-column term, chosen on the host from the multipliers and shifts (TileParams::mode):
//   kStageGeneric : {term, multiplier, right | left << 8, -} and the full reference expression;
//   kStageFast    : every shift is a right shift and no multiplier is INT32_MIN, so the saturating corner of
//                   SQDMULH cannot occur: {term, multiplier, 1 << (shift-1) (0 for shift 0), shift};
//   kStageWide    : every shift s is >= 2, every multiplier m is in [0, 2^31) and there is no row term.  Then
//                   ((floor((v+t)*m / 2^31) + 2^(s-1)) >> s equals hi32(v*m + (t*m + 2^(30+s))) >> (s-1): the
//                   bracket is a 64-bit constant of the column, so one wide multiply-add and one shift replace
//                   five instructions.  {constant lo, constant hi, multiplier, s-1}.  Equal to the reference
//                   wherever its own 32-bit sums v+t and x + 2^(s-1) do not overflow.
//   kStagePack    : kStageWide whose clamp bounds are the whole range of the 8-bit output type (no activation bound
//                   tighter than the type, the case of every ReLU at zero point 0 and of every plain requantisation).
//                   The output offset joins the 64-bit column constant -- adding offset * 2^(s-1) before the final
//                   shift by s-1 equals adding offset after it -- and the clamp becomes the saturation of the
//                   instruction that packs two results into bytes (cvt.pack.sat): per element one wide multiply-add
//                   and one shift, per four elements two packs.  Needs s <= 22 with a non-zero offset so that the
//                   constant stays inside 64 bits.
constexpr int kStageGeneric = 0, kStageFast = 1, kStageWide = 2, kStagePack = 3, kStagePackS = 4; // 3: uint8, 4: int8 output
constexpr int kIntegerStageFlag = 1 << 16; // generic encoding, bit of q.z: the integer-multiply stage QUANTIZE_DOWN

template <int kMode>
__device__ __forceinline__ int32_t requant_one(uint32_t v, const int4 q, int32_t row_term, int32_t offset, int32_t lo,
                                               int32_t hi)
{
    if (kMode == kStageWide || kMode == kStagePack || kMode == kStagePackS)
    {
        const long long c64 = static_cast<long long>((static_cast<unsigned long long>(static_cast<uint32_t>(q.y)) << 32) |
                                                     static_cast<uint32_t>(q.x));
        const long long p   = static_cast<long long>(static_cast<int32_t>(v)) * q.z + c64;
        const int32_t   t   = static_cast<int32_t>(p >> 32) >> q.w;
        if (kMode == kStagePack || kMode == kStagePackS)
        {
            return t; // offset already inside c64; the caller saturates while packing (pack4_sat)
        }
        return max(__viaddmin_s32(t, offset, hi), lo);
    }
    const int32_t acc = static_cast<int32_t>(v) + q.x + row_term;
    if (kMode == kStageGeneric)
    {
        if (q.z & kIntegerStageFlag) // QUANTIZE_DOWN: the offset is already part of the column term
        {
            return finalize_int(acc, q.y, q.z & 0xff, lo, hi);
        }
        return finalize(acc, q.y, (q.z >> 8) & 0xff, q.z & 0xff, offset, lo, hi);
    }
    const int32_t  mh = __mulhi(acc, q.y);
    const uint32_t ml = static_cast<uint32_t>(acc) * static_cast<uint32_t>(q.y);
    const uint32_t d  = __funnelshift_l(ml, static_cast<uint32_t>(mh), 1);         // floor(acc*mult / 2^31)
    const int32_t  t  = static_cast<int32_t>(d + static_cast<uint32_t>(q.z)) >> q.w; // round-half-up shift
    return min(max(t + offset, lo), hi);
}

// Four int32 results saturated to the 8-bit output type and packed, r0 in the lowest byte.  cvt.pack.sat puts
// sat(a) into bits 15..8, sat(b) into bits 7..0 and the low half of c into the upper half of the result.
template <bool out_signed>
__device__ __forceinline__ uint32_t pack4_sat(int32_t r0, int32_t r1, int32_t r2, int32_t r3)
{
    uint32_t hi2, w;
    if (out_signed)
    {
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi2) : "r"(r3), "r"(r2), "r"(0));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi2));
    }
    else
    {
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi2) : "r"(r3), "r"(r2), "r"(0));
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(r1), "r"(r0), "r"(hi2));
    }
    return w;
}

template <int kMode>
__device__ __forceinline__ uint32_t requant_pack4(const uint32_t *v, const int4 *col, int32_t row_term, int32_t offset,
                                                  int32_t lo, int32_t hi)
{
    int32_t r[4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
    {
        r[b] = requant_one<kMode>(v[b], col[b], row_term, offset, lo, hi);
    }
    if (kMode == kStagePack || kMode == kStagePackS)
    {
        return pack4_sat<kMode == kStagePackS>(r[0], r[1], r[2], r[3]);
    }
    const uint32_t p01 = __byte_perm(static_cast<uint32_t>(r[0]), static_cast<uint32_t>(r[1]), 0x0040);
    const uint32_t p23 = __byte_perm(static_cast<uint32_t>(r[2]), static_cast<uint32_t>(r[3]), 0x0040);
    return __byte_perm(p01, p23, 0x5410);
}

// Store 32 consecutive outputs of one row held in registers (v: int32 values or w: packed bytes).
template <bool kS32Out>
__device__ __forceinline__ void store_chunk(const uint32_t *v, uint8_t *drow, int nc, bool row_ok, const TileParams &tp)
{
    if (!row_ok)
    {
        return;
    }
    const bool full = nc + 32 <= tp.N;
    if (kS32Out)
    {
        // v holds the int32 results; float conversion and accumulation into dst happen here (raw_result_word)
        uint32_t  *o     = reinterpret_cast<uint32_t *>(drow) + nc;
        const bool plain = tp.raw_f32 == 0 && tp.raw_accumulate == 0; // uniform over the launch
        EpilogueParams rp{};
        rp.out_f32    = tp.raw_f32;
        rp.accumulate = tp.raw_accumulate;
        rp.dq_scale   = tp.raw_scale;
        if (full && tp.vec_ok)
        {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
            {
                uint4 w = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (!plain)
                {
                    uint4 old = make_uint4(0, 0, 0, 0);
                    if (tp.raw_accumulate != 0) old = *reinterpret_cast<const uint4 *>(o + j);
                    w.x = raw_result_word(static_cast<int32_t>(w.x), old.x, rp);
                    w.y = raw_result_word(static_cast<int32_t>(w.y), old.y, rp);
                    w.z = raw_result_word(static_cast<int32_t>(w.z), old.z, rp);
                    w.w = raw_result_word(static_cast<int32_t>(w.w), old.w, rp);
                }
                *reinterpret_cast<uint4 *>(o + j) = w;
            }
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 32; ++j)
            {
                if (nc + j < tp.N)
                {
                    o[j] = plain ? v[j] : raw_result_word(static_cast<int32_t>(v[j]), tp.raw_accumulate != 0 ? o[j] : 0u, rp);
                }
            }
        }
    }
    else
    {
        uint8_t *o = drow + nc;
        if (full && (tp.vec_ok & 2))
        {
            // one 256-bit store: the lane writes a whole 32-byte sector instead of two halves
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o), "r"(v[0]), "r"(v[1]),
                         "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                         : "memory");
        }
        else if (full && tp.vec_ok)
        {
            *reinterpret_cast<uint4 *>(o)      = make_uint4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<uint4 *>(o + 16) = make_uint4(v[4], v[5], v[6], v[7]);
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 32; ++j)
            {
                if (nc + j < tp.N) o[j] = static_cast<uint8_t>(v[j >> 2] >> (8 * (j & 3)));
            }
        }
    }
}

template <bool kS32Out, int kMode>
__device__ __forceinline__ void process_chunk(uint32_t (&v)[32], const int4 *col, int32_t row_term,
                                              const EpilogueParams &ep)
{
    if (kS32Out)
    {
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            v[j] = static_cast<uint32_t>(static_cast<int32_t>(v[j]) + col[j].x + row_term);
        }
    }
    else
    {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
        {
            v[j >> 2] = requant_pack4<kMode>(v + j, col + j, row_term, ep.result_offset, ep.lo, ep.hi);
        }
    }
}

// Output staging of the multi-destination (push all-gather) epilogue.  A thread owns one row, so its direct
// stores are 16-byte pieces 'ldd' apart: harmless in local memory, where L2 merges them, but over NVLink every
// piece is a packet of its own.  Here a warp first collects 32 rows x kOutRowBytes columns in shared memory
// (piece p of row r at p ^ (r & (pieces - 1)): conflict-free both ways) and then stores them with one lane per
// piece, kOutRowBytes contiguous bytes per row, to every destination.  128 bytes per row with four epilogue
// warps, 64 with eight (shared memory holds 32 KB of staging at most beside the operand ring).
constexpr int kOutRowBytes   = kEpiWarps == 4 ? 128 : (kEpiWarps == 8 ? 64 : 32);
constexpr int kOutPieces     = kOutRowBytes / 16;
constexpr int kOutChunks     = kOutRowBytes / 32; // 32-column chunks per staged group
constexpr int kCmPitchWords  = 36;                // channel-major transpose stage (store_chunk_cm_staged)
constexpr int kCmStageBytes  = 8 * kCmPitchWords * 4;
constexpr int kOutStageBytes = 32 * kOutRowBytes > kCmStageBytes ? 32 * kOutRowBytes : kCmStageBytes;

// Swizzle of the staged rows.  The library's own flush reads the stage back with any conflict-free pattern (row & mask);
// a stage the TMA unit stores must follow the tensor map's swizzle: the 16-byte piece index XORed with address bits
// 7.. of the row, i.e. with row, row >> 1 or row >> 2 for rows of 128, 64 or 32 bytes.
constexpr int kOutSwShift = kOutRowBytes == 128 ? 0 : (kOutRowBytes == 64 ? 1 : 2);
__device__ __forceinline__ int stage_sw(int r, bool tma)
{
    return (tma ? (r >> kOutSwShift) : r) & (kOutPieces - 1);
}
__device__ __forceinline__ void stage_chunk(uint8_t *stage, const uint32_t *w, int group_chunk, int lane, bool tma = false)
{
    uint8_t *row = stage + lane * kOutRowBytes;
    const int sw = stage_sw(lane, tma);
    *reinterpret_cast<uint4 *>(row + (((2 * group_chunk) ^ sw) << 4))     = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(row + (((2 * group_chunk + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}

__device__ __forceinline__ void flush_stage(const uint8_t *stage, const TileParams &tp, int m_base, int n_group,
                                            int ncols_group, int lane, bool tma = false)
{
    __syncwarp();
    const int p = lane & (kOutPieces - 1);
#pragma unroll 2
    for (int it = 0; it < kOutPieces; ++it)
    {
        const int r = it * (32 / kOutPieces) + lane / kOutPieces;
        const int m = m_base + r;
        const int n = n_group + p * 16;
        if (p * 16 < ncols_group && m < tp.M && n < tp.N)
        {
            const uint4   val = *reinterpret_cast<const uint4 *>(stage + r * kOutRowBytes + ((p ^ stage_sw(r, tma)) << 4));
            const int64_t off = static_cast<int64_t>(m) * tp.ldd + n;
            if (n + 16 <= tp.N && tp.vec_ok)
            {
                *reinterpret_cast<uint4 *>(tp.dst + off) = val;
                for (int x = 0; x < tp.n_extra; ++x)
                {
                    *reinterpret_cast<uint4 *>(tp.extra_dst[x] + off) = val;
                }
            }
            else
            {
                const uint32_t w[4] = {val.x, val.y, val.z, val.w};
                for (int j = 0; j < 16 && n + j < tp.N; ++j)
                {
                    const uint8_t b    = static_cast<uint8_t>(w[j >> 2] >> (8 * (j & 3)));
                    tp.dst[off + j]    = b;
                    for (int x = 0; x < tp.n_extra; ++x)
                    {
                        tp.extra_dst[x][off + j] = b;
                    }
                }
            }
        }
    }
    __syncwarp();
}

// The same staged group (32 rows x kOutRowBytes, all of it valid) handed to the TMA unit: one bulk tensor store per
// warp and group instead of one row-strided store per lane, which keeps the warp off the load/store pipe and does
// not make it wait for the stores to be accepted.  The caller waits for the previous group's reads (stage_reuse_wait)
// before it writes into the stage again.
__device__ __forceinline__ void flush_stage_tma(const uint8_t *stage, const CUtensorMap *omap, int m_base, int n_group,
                                                int lane)
{
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0)
    {
        tma_store_2d(omap, smem_u32(stage), n_group, m_base);
        tma_store_commit();
    }
}
__device__ __forceinline__ void stage_reuse_wait(int lane)
{
    if (lane == 0)
    {
        tma_store_wait_read();
    }
    __syncwarp();
}

// Fused residual addition on 32 packed output bytes of one row: out = min(max(min(out + res, 255), floor), cap),
// the form the host has proved equal to quantize(dequantize(out) + dequantize(res)) followed by the activation.
__device__ __forceinline__ void load_residual(uint32_t (&r)[8], const uint8_t *rrow, int nc, bool row_ok,
                                              const TileParams &tp)
{
    if (!row_ok)
    {
        return;
    }
    if (nc + 32 <= tp.N && (tp.vec_ok & 2))
    {
        asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "l"(rrow + nc));
    }
    else if (nc + 32 <= tp.N && tp.vec_ok)
    {
        const uint4 r0 = __ldg(reinterpret_cast<const uint4 *>(rrow + nc));
        const uint4 r1 = __ldg(reinterpret_cast<const uint4 *>(rrow + nc + 16));
        r[0] = r0.x, r[1] = r0.y, r[2] = r0.z, r[3] = r0.w, r[4] = r1.x, r[5] = r1.y, r[6] = r1.z, r[7] = r1.w;
    }
    else
    {
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            uint32_t v = 0;
            for (int b = 0; b < 4; ++b)
            {
                if (nc + 4 * j + b < tp.N) v |= static_cast<uint32_t>(rrow[nc + 4 * j + b]) << (8 * b);
            }
            r[j] = v;
        }
    }
}
__device__ __forceinline__ void add_residual(uint32_t *w, const uint32_t (&r)[8], const TileParams &tp)
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        w[j] = add_clamp_u8x4(w[j], r[j], tp.res_floor4, tp.res_cap4);
    }
}

// Asks L2 for the residual bytes this thread will add to row m, columns [n_first, n_first + ncols): issued before the
// wait for the accumulator, so the DRAM latency passes behind the MMA and the requantisation.
__device__ __forceinline__ void prefetch_residual(const TileParams &tp, int m, int n_first, int ncols)
{
    if (m < tp.M)
    {
        const uint8_t *p = tp.residual + static_cast<int64_t>(m) * tp.ldd + n_first;
        for (int c = 0; c < ncols && n_first + c < tp.N; c += 128)
        {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p + c));
        }
    }
}

// Hand-back of accumulator buffers to the MMA issuer.  A warp may give its share of a buffer back as soon as its last
// tcgen05.ld from it has completed -- the values are in registers then -- so the arithmetic and the stores of the last
// chunk overlap the MMAs of the tile that reuses the buffer.  bar_a / bar_b: shared::cta addresses of the buffers'
// "empty" barriers (0: none); cluster: bar_a is a shared::cluster address (the leader CTA's barrier, SM-pair kernel).
struct AccRelease
{
    uint32_t bar_a, bar_b;
    bool     cluster;
};
__device__ __forceinline__ void release_accumulators(const AccRelease &r, int lane)
{
    tc_fence_before();
    __syncwarp();
    if (lane == 0)
    {
        if (r.cluster)
        {
            mbar_arrive_cluster(r.bar_a);
        }
        else
        {
            if (r.bar_a != 0) mbar_arrive(r.bar_a);
            if (r.bar_b != 0) mbar_arrive(r.bar_b);
        }
    }
}

// Shared epilogue of both kernels: one warp drains NCOLS consecutive columns (a multiple of 32) of its
// 32 accumulator rows from tensor memory, applies the offset / bias terms and the output stage, and
// stores.  The tensor-memory load of chunk i+1 is issued before chunk i is processed.
template <int NCOLS, bool kS32Out, int kMode>
__device__ __forceinline__ void drain_accumulator(uint32_t t_addr, const int4 *s_col, const TileParams &tp,
                                                  const EpilogueParams &ep, int m, int n_first, int32_t row_term,
                                                  uint8_t *stage, int lane, const AccRelease &rel,
                                                  const CUtensorMap *omap = nullptr)
{
    const bool row_ok = m < tp.M;
    const int64_t row_off = static_cast<int64_t>(m) * tp.ldd;
    uint8_t      *drow    = tp.dst + row_off;
    // omap: the warp's 32 rows x kOutRowBytes leave as one bulk tensor store from its staging area (one destination)
    const bool    tma     = !kS32Out && omap != nullptr && tp.n_extra == 0; // warp-uniform
    const bool    staged  = !kS32Out && (tp.n_extra > 0 || tma);            // warp-uniform
    // chunk c of the warp's columns into the stage; the group goes out when it is complete
    auto stage_and_flush = [&](const uint32_t *v, int c) {
        const int gc = c & (kOutChunks - 1);
        if (tma && gc == 0)
        {
            stage_reuse_wait(lane); // the previous group's store has read the stage
        }
        stage_chunk(stage, v, gc, lane, tma);
        if (gc == kOutChunks - 1 || c + 1 >= NCOLS / 32)
        {
            const int first = c & ~(kOutChunks - 1); // first chunk of this staged group
            const int ncols = (c + 1 - first) * 32;
            // A bulk tensor store clips at the tensor's edge in whole 16-byte units (measured: a 64-byte box over the
            // ragged end of a 200-byte row wrote bytes 200..207 too), so a group that crosses N leaves through the
            // lanes unless N itself ends on such a unit.
            const int n_group = n_first + first * 32;
            if (tma && ncols == kOutRowBytes && (n_group + kOutRowBytes <= tp.N || (tp.N & 15) == 0))
            {
                flush_stage_tma(stage, omap, m - lane, n_first + first * 32, lane);
            }
            else
            {
                flush_stage(stage, tp, m - lane, n_first + first * 32, ncols, lane, tma);
            }
        }
    };
    uint32_t   va[32], vb[32];
    tmem_ld_x32(t_addr, va);
#pragma unroll 1
    for (int ch = 0; ch < NCOLS / 32; ch += 2)
    {
        tmem_ld_wait();
        if (ch + 1 < NCOLS / 32)
        {
            tmem_ld_x32(t_addr + (ch + 1) * 32, vb);
        }
        else
        {
            release_accumulators(rel, lane); // nothing more to read from tensor memory
        }
        const bool with_res = !kS32Out && tp.residual != nullptr; // warp-uniform
        process_chunk<kS32Out, kMode>(va, s_col + ch * 32, row_term, ep);
        if (with_res)
        {
            // loaded after the arithmetic: requesting the bytes before it (eight more live registers) measured
            // slower in the sixteen-warp build, whose threads have 96 registers (305 -> 365 us on 802816 x 256 x 64)
            uint32_t res[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            load_residual(res, tp.residual + row_off, n_first + ch * 32, row_ok, tp);
            add_residual(va, res, tp);
        }
        if (staged)
        {
            stage_and_flush(va, ch);
        }
        else
        {
            store_chunk<kS32Out>(va, drow, n_first + ch * 32, row_ok, tp);
            for (int x = 0; x < tp.n_extra; ++x)
            {
                store_chunk<kS32Out>(va, tp.extra_dst[x] + row_off, n_first + ch * 32, row_ok, tp);
            }
        }
        if (ch + 1 < NCOLS / 32)
        {
            tmem_ld_wait();
            if (ch + 2 < NCOLS / 32)
            {
                tmem_ld_x32(t_addr + (ch + 2) * 32, va);
            }
            else
            {
                release_accumulators(rel, lane);
            }
            process_chunk<kS32Out, kMode>(vb, s_col + (ch + 1) * 32, row_term, ep);
            if (with_res)
            {
                uint32_t res[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                load_residual(res, tp.residual + row_off, n_first + (ch + 1) * 32, row_ok, tp);
                add_residual(vb, res, tp);
            }
            if (staged)
            {
                stage_and_flush(vb, ch + 1);
            }
            else
            {
                store_chunk<kS32Out>(vb, drow, n_first + (ch + 1) * 32, row_ok, tp);
                for (int x = 0; x < tp.n_extra; ++x)
                {
                    store_chunk<kS32Out>(vb, tp.extra_dst[x] + row_off, n_first + (ch + 1) * 32, row_ok, tp);
                }
            }
        }
    }
}

// 32 packed output bytes of one row to global memory; cols: valid columns from o on (>= 32: a whole chunk).
__device__ __forceinline__ void store_row32(uint8_t *o, const uint32_t *v, int cols, int vec_ok)
{
    if (o == nullptr)
    {
        return;
    }
    if (cols >= 32 && (vec_ok & 2))
    {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(o), "r"(v[0]), "r"(v[1]),
                     "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                     : "memory");
    }
    else if (cols >= 32 && vec_ok)
    {
        *reinterpret_cast<uint4 *>(o)      = make_uint4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<uint4 *>(o + 16) = make_uint4(v[4], v[5], v[6], v[7]);
    }
    else
    {
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            if (j < cols) o[j] = static_cast<uint8_t>(v[j >> 2] >> (8 * (j & 3)));
        }
    }
}
__device__ __forceinline__ void load_row32(uint32_t (&r)[8], const uint8_t *p, int cols, int vec_ok)
{
    if (p == nullptr)
    {
        return;
    }
    if (cols >= 32 && (vec_ok & 2))
    {
        asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "l"(p));
    }
    else if (cols >= 32 && vec_ok)
    {
        const uint4 r0 = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint4 r1 = __ldg(reinterpret_cast<const uint4 *>(p + 16));
        r[0] = r0.x, r[1] = r0.y, r[2] = r0.z, r[3] = r0.w, r[4] = r1.x, r[5] = r1.y, r[6] = r1.z, r[7] = r1.w;
    }
    else
    {
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            uint32_t v = 0;
            for (int b = 0; b < 4; ++b)
            {
                if (4 * j + b < cols) v |= static_cast<uint32_t>(p[4 * j + b]) << (8 * b);
            }
            r[j] = v;
        }
    }
}

// Everything the paired drain needs, by value: the function is a call of its own (its register allocation is then
// independent of the rest of the kernel, which matters in the sixteen-warp build with 96 registers per thread).
struct PairDrain
{
    uint32_t       t_a, t_b;       // tensor-memory addresses of the two buffers (lane quarter and first column applied)
    const int4    *col;            // terms of the first column
    uint8_t       *dst_a, *dst_b;  // output rows at the first column; nullptr: the row lies outside the matrix
    const uint8_t *res_a, *res_b;  // residual rows at the first column; nullptr: no residual (or no row)
    int            cols;           // valid columns from the first column on
    int            vec_ok;
    uint32_t       res_floor4, res_cap4;
    int32_t        offset, lo, hi; // wide encoding only
    AccRelease     rel;
    int            lane;
    // Output through the TMA unit (sixteen-warp build, 64 columns per warp): stage = shared-memory address of this warp's
    // staging area, two tiles of 32 rows x 64 bytes in the 64-byte swizzle (0: per-lane global stores); the two boxes go
    // to (n_first, row_a) and (n_first, row_b) of the output map
    uint32_t           stage;
    const CUtensorMap *omap;
    int                n_first, row_a, row_b;
    // A fused residual arrives the same way: before the warp's first tensor-memory load one lane requests the two
    // residual boxes into the stage (bulk tensor loads completing on the warp's own barrier res_bar, phase res_parity);
    // every lane adds its pieces in place before the boxes go out again.  rmap == nullptr: no residual this way.
    const CUtensorMap *rmap;
    uint32_t           res_bar, res_parity;
    volatile int      *abort_flag;
    long long          spin_limit;
};
constexpr int kPairStageBytes = 2 * 32 * 64; // per warp

template <int G, int kMode>
__device__ __forceinline__ void requant_columns_pair(const uint32_t *a, const uint32_t *b, const int4 *col,
                                                     const PairDrain &d, uint32_t *wa, uint32_t *wb)
{
#pragma unroll
    for (int h = 0; h < G / 4; ++h)
    {
        int32_t ra[4], rb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const int4 q = col[4 * h + j];
            ra[j]        = requant_one<kMode>(a[4 * h + j], q, 0, d.offset, d.lo, d.hi);
            rb[j]        = requant_one<kMode>(b[4 * h + j], q, 0, d.offset, d.lo, d.hi);
        }
        if (kMode == kStagePack || kMode == kStagePackS)
        {
            wa[h] = pack4_sat<kMode == kStagePackS>(ra[0], ra[1], ra[2], ra[3]);
            wb[h] = pack4_sat<kMode == kStagePackS>(rb[0], rb[1], rb[2], rb[3]);
        }
        else
        {
            wa[h] = __byte_perm(__byte_perm(static_cast<uint32_t>(ra[0]), static_cast<uint32_t>(ra[1]), 0x0040),
                                __byte_perm(static_cast<uint32_t>(ra[2]), static_cast<uint32_t>(ra[3]), 0x0040), 0x5410);
            wb[h] = __byte_perm(__byte_perm(static_cast<uint32_t>(rb[0]), static_cast<uint32_t>(rb[1]), 0x0040),
                                __byte_perm(static_cast<uint32_t>(rb[2]), static_cast<uint32_t>(rb[3]), 0x0040), 0x5410);
        }
    }
}

__device__ __forceinline__ void finish_chunk_pair(const PairDrain &d, int ch, uint32_t *wa, uint32_t *wb,
                                                  const uint32_t (&res_a)[8], const uint32_t (&res_b)[8])
{
    if (d.res_a != nullptr || d.res_b != nullptr)
    {
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            wa[j] = add_clamp_u8x4(wa[j], res_a[j], d.res_floor4, d.res_cap4);
            wb[j] = add_clamp_u8x4(wb[j], res_b[j], d.res_floor4, d.res_cap4);
        }
    }
    if (d.stage != 0)
    {
        // 64-byte rows, 16-byte piece p of row r at piece p ^ ((r >> 1) & 3): the tensor map's 64-byte swizzle
        if (ch == 0 && d.rmap == nullptr)
        {
            stage_reuse_wait(d.lane); // the previous pair's stores have read the stage (with a residual: request_residual_boxes)
        }
        const uint32_t row = d.stage + d.lane * 64, sw = (d.lane >> 1) & 3;
        const uint32_t p0 = ((2u * ch) ^ sw) << 4, p1 = ((2u * ch + 1u) ^ sw) << 4;
        if (d.rmap != nullptr)
        {
            if (ch == 0)
            {
                (void)mbar_wait(d.res_bar, d.res_parity, d.abort_flag, DEV_TIMEOUT_EPILOGUE, d.spin_limit); // gives up: flag set
            }
            uint32_t ra[8], rb[8];
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(ra[0]), "=r"(ra[1]), "=r"(ra[2]), "=r"(ra[3]) : "r"(row + p0) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(ra[4]), "=r"(ra[5]), "=r"(ra[6]), "=r"(ra[7]) : "r"(row + p1) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(rb[0]), "=r"(rb[1]), "=r"(rb[2]), "=r"(rb[3]) : "r"(row + 2048 + p0) : "memory");
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(rb[4]), "=r"(rb[5]), "=r"(rb[6]), "=r"(rb[7]) : "r"(row + 2048 + p1) : "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j)
            {
                wa[j] = add_clamp_u8x4(wa[j], ra[j], d.res_floor4, d.res_cap4);
                wb[j] = add_clamp_u8x4(wb[j], rb[j], d.res_floor4, d.res_cap4);
            }
        }
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + p0), "r"(wa[0]), "r"(wa[1]), "r"(wa[2]), "r"(wa[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + p1), "r"(wa[4]), "r"(wa[5]), "r"(wa[6]), "r"(wa[7]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + 2048 + p0), "r"(wb[0]), "r"(wb[1]), "r"(wb[2]), "r"(wb[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row + 2048 + p1), "r"(wb[4]), "r"(wb[5]), "r"(wb[6]), "r"(wb[7]) : "memory");
        if (ch == 1) // 64 columns per warp: the boxes are complete
        {
            fence_proxy_async_smem();
            __syncwarp();
            if (d.lane == 0)
            {
                tma_store_2d(d.omap, d.stage, d.n_first, d.row_a);
                tma_store_2d(d.omap, d.stage + 2048, d.n_first, d.row_b);
                tma_store_commit();
            }
        }
        return;
    }
    store_row32(d.dst_a != nullptr ? d.dst_a + ch * 32 : nullptr, wa, d.cols - ch * 32, d.vec_ok);
    store_row32(d.dst_b != nullptr ? d.dst_b + ch * 32 : nullptr, wb, d.cols - ch * 32, d.vec_ok);
}

// Two accumulator buffers that hold tiles of the same column block drained together (wide / pack encodings).  Every
// lane of a warp needs the 16-byte term of every column, so the per-element term read from shared memory is what the
// load/store pipe spends most of a short-K epilogue on; here a term is read once for two elements.
template <int kMode>
__device__ __forceinline__ void drain_pair_chunk_x32(const PairDrain &d, int ch, bool last)
{
    uint32_t va[32], vb[32];
    tmem_ld_x32(d.t_a + ch * 32, va);
    tmem_ld_x32(d.t_b + ch * 32, vb);
    tmem_ld_wait();
    if (last)
    {
        release_accumulators(d.rel, d.lane);
    }
    uint32_t wa[8], wb[8];
    requant_columns_pair<32, kMode>(va, vb, d.col + ch * 32, d, wa, wb);
    uint32_t res_a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, res_b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    load_row32(res_a, d.res_a != nullptr ? d.res_a + ch * 32 : nullptr, d.cols - ch * 32, d.vec_ok);
    load_row32(res_b, d.res_b != nullptr ? d.res_b + ch * 32 : nullptr, d.cols - ch * 32, d.vec_ok);
    finish_chunk_pair(d, ch, wa, wb, res_a, res_b);
}
// the same chunk read as two halves of sixteen columns: half the accumulator registers live at a time
template <int kMode>
__device__ __forceinline__ void drain_pair_chunk_x16(const PairDrain &d, int ch, bool last)
{
    uint32_t wa[8], wb[8];
    uint32_t res_a[8] = {0, 0, 0, 0, 0, 0, 0, 0}, res_b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    load_row32(res_a, d.res_a != nullptr ? d.res_a + ch * 32 : nullptr, d.cols - ch * 32, d.vec_ok);
    load_row32(res_b, d.res_b != nullptr ? d.res_b + ch * 32 : nullptr, d.cols - ch * 32, d.vec_ok);
#pragma unroll
    for (int h = 0; h < 2; ++h)
    {
        uint32_t va[16], vb[16];
        tmem_ld_x16(d.t_a + ch * 32 + h * 16, va);
        tmem_ld_x16(d.t_b + ch * 32 + h * 16, vb);
        tmem_ld_wait();
        if (last && h == 1)
        {
            release_accumulators(d.rel, d.lane);
        }
        requant_columns_pair<16, kMode>(va, vb, d.col + ch * 32 + h * 16, d, wa + 4 * h, wb + 4 * h);
    }
    finish_chunk_pair(d, ch, wa, wb, res_a, res_b);
}
// Paired drain with a fused residual: the warp's two residual boxes (32 rows x 64 bytes of each tile) into its staging
// area, completion on the warp's own barrier.  Called before the wait for the accumulators, so that the boxes travel
// while the pair's MMAs are still being issued; the previous pair's bulk stores must have read the stage first.
__device__ __forceinline__ void request_residual_boxes(const CUtensorMap *rmap, uint32_t stage, uint32_t res_bar, int n_first,
                                                       int row_a, int row_b, int lane)
{
    stage_reuse_wait(lane);
    if (lane == 0)
    {
        mbar_expect_tx(res_bar, kPairStageBytes);
        tma_load_2d(stage, rmap, n_first, row_a, res_bar);
        tma_load_2d(stage + 2048, rmap, n_first, row_b, res_bar);
    }
}

template <int NCOLS, int kMode>
__device__ __forceinline__ void drain_pair_x16(const PairDrain d)
{
    // (with a fused residual the caller has requested the warp's two residual boxes into the stage before it waited
    // for the accumulators: request_residual_boxes)
#pragma unroll 1
    for (int ch = 0; ch < NCOLS / 32; ++ch)
    {
        drain_pair_chunk_x16<kMode>(d, ch, ch == NCOLS / 32 - 1);
    }
}
template <int NCOLS, int kMode>
__device__ __noinline__ void drain_pair_x32(const PairDrain d)
{
#pragma unroll 1
    for (int ch = 0; ch < NCOLS / 32; ++ch)
    {
        drain_pair_chunk_x32<kMode>(d, ch, ch == NCOLS / 32 - 1);
    }
}

template <int NCOLS, int kMode>
__device__ __forceinline__ void drain_accumulator_pair(uint32_t t_a, uint32_t t_b, const int4 *s_col,
                                                       const TileParams &tp, const EpilogueParams &ep, int ma, int mb,
                                                       int n_first, int lane, const AccRelease &rel, uint32_t stage = 0,
                                                       const CUtensorMap *omap = nullptr, const CUtensorMap *rmap = nullptr,
                                                       uint32_t res_bar = 0, uint32_t res_parity = 0,
                                                       volatile int *abort_flag = nullptr)
{
    PairDrain d;
    d.stage = NCOLS == 64 ? stage : 0u, d.omap = omap, d.n_first = n_first, d.row_a = ma - lane, d.row_b = mb - lane;
    d.rmap  = (d.stage != 0 && tp.residual != nullptr) ? rmap : nullptr;
    d.res_bar = res_bar, d.res_parity = res_parity, d.abort_flag = abort_flag, d.spin_limit = tp.spin_limit;
    d.t_a = t_a, d.t_b = t_b, d.col = s_col;
    d.dst_a      = ma < tp.M ? tp.dst + static_cast<int64_t>(ma) * tp.ldd + n_first : nullptr;
    d.dst_b      = mb < tp.M ? tp.dst + static_cast<int64_t>(mb) * tp.ldd + n_first : nullptr;
    d.res_a      = (tp.residual != nullptr && d.rmap == nullptr && ma < tp.M) ? tp.residual + static_cast<int64_t>(ma) * tp.ldd + n_first : nullptr;
    d.res_b      = (tp.residual != nullptr && d.rmap == nullptr && mb < tp.M) ? tp.residual + static_cast<int64_t>(mb) * tp.ldd + n_first : nullptr;
    d.cols       = tp.N - n_first;
    d.vec_ok     = tp.vec_ok;
    d.res_floor4 = tp.res_floor4, d.res_cap4 = tp.res_cap4;
    d.offset = ep.result_offset, d.lo = ep.lo, d.hi = ep.hi;
    d.rel = rel, d.lane = lane;
    // sixteen epilogue warps (96 registers per thread): sixteen columns at a time (802816 x 256 x 64: 143 against 154 us;
    // level on the other shapes); eight and four warps measured level or better with whole 32-column loads
    if (kEpiWarps == 16) drain_pair_x16<NCOLS, kMode>(d);
    else drain_pair_x32<NCOLS, kMode>(d);
}

template <int BLOCK_N, int kGroups>
__device__ __forceinline__ void epilogue_warp_tile_pair(uint32_t tmem_a, uint32_t tmem_b, const int4 *s_col,
                                                        const TileParams &tp, const EpilogueParams &ep, int warp,
                                                        int lane, int m0a, int m0b, int n0, const AccRelease &rel,
                                                        uint32_t stage = 0, const CUtensorMap *omap = nullptr,
                                                        const CUtensorMap *rmap = nullptr, uint32_t res_bar = 0,
                                                        uint32_t res_parity = 0, volatile int *abort_flag = nullptr)
{
    constexpr int  NCOLS = BLOCK_N * kGroups / (kEpiWarps / 4);
    const int      quad  = warp & 3;                                      // tensor-memory lane quarter this warp may read
    const int      half  = kGroups == 1 ? (warp - kFirstEpi) >> 2 : 0;    // which share of the columns
    const uint32_t lanes = static_cast<uint32_t>(quad * 32) << 16;
    if (tp.mode == kStagePack)
    {
        drain_accumulator_pair<NCOLS, kStagePack>(tmem_a + lanes + half * NCOLS, tmem_b + lanes + half * NCOLS,
                                                  s_col + half * NCOLS, tp, ep, m0a + quad * 32 + lane, m0b + quad * 32 + lane,
                                                  n0 + half * NCOLS, lane, rel, stage, omap, rmap, res_bar, res_parity, abort_flag);
    }
    else if (tp.mode == kStagePackS)
    {
        drain_accumulator_pair<NCOLS, kStagePackS>(tmem_a + lanes + half * NCOLS, tmem_b + lanes + half * NCOLS,
                                                   s_col + half * NCOLS, tp, ep, m0a + quad * 32 + lane, m0b + quad * 32 + lane,
                                                   n0 + half * NCOLS, lane, rel, stage, omap, rmap, res_bar, res_parity, abort_flag);
    }
    else
    {
        drain_accumulator_pair<NCOLS, kStageWide>(tmem_a + lanes + half * NCOLS, tmem_b + lanes + half * NCOLS,
                                                  s_col + half * NCOLS, tp, ep, m0a + quad * 32 + lane, m0b + quad * 32 + lane,
                                                  n0 + half * NCOLS, lane, rel, stage, omap, rmap, res_bar, res_parity, abort_flag);
    }
}

// the term of output channel n in the encoding of tp.mode (see requant_pack4)
__device__ __forceinline__ int4 column_term(int n, const TileParams &tp, const EpilogueParams &ep)
{
    int4    q = make_int4(0, 0, 0, 0);
    int32_t t = ep.k_term;
    if (ep.colsum != nullptr) t += ep.a_off * __ldg(ep.colsum + n);
    if (ep.bias != nullptr) t += __ldg(ep.bias + n);
    const int32_t sh = ep.shifts != nullptr ? __ldg(ep.shifts + n) : ep.shift;
    q.x              = t;
    q.y              = ep.mults != nullptr ? __ldg(ep.mults + n) : ep.mult;
    if (tp.mode == kStageGeneric)
    {
        q.z = max(sh, 0) | (max(-sh, 0) << 8);
        if (ep.stage == CUGL_STAGE_QUANTIZE_DOWN)
        {
            q.x = static_cast<int32_t>(static_cast<uint32_t>(t) + static_cast<uint32_t>(ep.result_offset));
            q.z = (sh & 0xff) | kIntegerStageFlag;
        }
    }
    else if (tp.mode == kStageFast)
    {
        q.z = static_cast<int32_t>((1u << sh) >> 1);
        q.w = sh;
    }
    else
    {
        long long c64 = static_cast<long long>(t) * q.y + (1ll << (30 + sh));
        if (tp.mode == kStagePack || tp.mode == kStagePackS)
        {
            c64 += static_cast<long long>(ep.result_offset) << (31 + sh); // offset * 2^(s-1), in units of 2^32
        }
        q.z                 = q.y;
        q.x                 = static_cast<int32_t>(static_cast<uint32_t>(c64));
        q.y                 = static_cast<int32_t>(c64 >> 32);
        q.w                 = sh - 1;
    }
    return q;
}

// per-column terms of a tile
template <int BLOCK_N>
__device__ __forceinline__ void fill_column_terms(int4 *s_col, int et, int n0, const TileParams &tp,
                                                  const EpilogueParams &ep, int n_threads = kEpiThreads)
{
    for (int c = et; c < BLOCK_N; c += n_threads)
    {
        const int n = n0 + c;
        s_col[c]    = n < tp.N ? column_term(n, tp, ep) : make_int4(0, 0, 0, 0);
    }
}

// Channel-major epilogue.  The kernel was launched with the operand roles exchanged (weights on the 128-row
// side, activations on the BLOCK_N side), so a tensor-memory LANE is an output channel and a tensor-memory
// COLUMN an output row.  A thread then needs the output-stage term of ONE channel, held in four registers for
// the whole tile, instead of a 16-byte shared-memory read per element -- that read (512 bytes per warp and
// element column) is what bounds the row-major epilogue on short-K shapes.  The 32 lanes of a warp hold 32
// consecutive channels of one output row: each store instruction writes one 32-byte segment of dst.
//   tp.M = number of channels (dst columns), tp.N = number of rows of dst, tp.ldd = dst row pitch in bytes.
// Channel-major chunk (lane = channel, 32 output rows in registers) written through a 4x4 byte transpose in
// shared memory: every lane packs four rows of its channel into a word and stores the eight words (pitch 36
// words: conflict-free both ways); lane (i, g) = (lane / 4, lane % 4) then reads the eight words of channels
// 8g .. 8g+7 for rows 4i .. 4i+3, transposes two 4x4 byte blocks with eight byte permutes and stores eight
// contiguous bytes per row: 4 store instructions per lane and chunk instead of 32 byte stores.  The residual
// is loaded and added in the same shape.  Needs 8-byte aligned rows (tp.vec_ok) and is called by whole warps.

template <int kMode>
__device__ __forceinline__ void store_chunk_cm_staged(const uint32_t (&v)[32], const int4 q, const TileParams &tp,
                                                      const EpilogueParams &ep, int ch_base, int p0, int lane,
                                                      uint32_t *stage)
{
    // this lane's share of the transposed block: rows p0 + 4i .. + 3, channels ch .. ch + 7
    const int  i = lane >> 2, g = lane & 3;
    const int  ch   = ch_base + 8 * g;
    const bool full = ch + 8 <= tp.M;
    // the residual bytes are requested first: their latency passes while the chunk is requantised
    uint2 res[4] = {make_uint2(0, 0), make_uint2(0, 0), make_uint2(0, 0), make_uint2(0, 0)};
    if (tp.residual != nullptr && full)
    {
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            const int p = p0 + 4 * i + k;
            if (p < tp.N)
            {
                res[k] = __ldg(reinterpret_cast<const uint2 *>(tp.residual + static_cast<int64_t>(p) * tp.ldd + ch));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        int32_t r[4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
        {
            r[b] = requant_one<kMode>(v[4 * j + b], q, 0, ep.result_offset, ep.lo, ep.hi);
        }
        if (kMode == kStagePack || kMode == kStagePackS)
        {
            stage[j * kCmPitchWords + lane] = pack4_sat<kMode == kStagePackS>(r[0], r[1], r[2], r[3]);
        }
        else
        {
            const uint32_t p01 = __byte_perm(static_cast<uint32_t>(r[0]), static_cast<uint32_t>(r[1]), 0x0040);
            const uint32_t p23 = __byte_perm(static_cast<uint32_t>(r[2]), static_cast<uint32_t>(r[3]), 0x0040);
            stage[j * kCmPitchWords + lane] = __byte_perm(p01, p23, 0x5410);
        }
    }
    __syncwarp();
    const uint4 lo = *reinterpret_cast<const uint4 *>(stage + i * kCmPitchWords + 8 * g);
    const uint4 hi = *reinterpret_cast<const uint4 *>(stage + i * kCmPitchWords + 8 * g + 4);
    __syncwarp(); // the stage may be overwritten by the next chunk
    uint32_t t[4][2];
    {
        const uint32_t x0 = __byte_perm(lo.x, lo.y, 0x5140), x1 = __byte_perm(lo.x, lo.y, 0x7362);
        const uint32_t y0 = __byte_perm(lo.z, lo.w, 0x5140), y1 = __byte_perm(lo.z, lo.w, 0x7362);
        t[0][0] = __byte_perm(x0, y0, 0x5410), t[1][0] = __byte_perm(x0, y0, 0x7632);
        t[2][0] = __byte_perm(x1, y1, 0x5410), t[3][0] = __byte_perm(x1, y1, 0x7632);
    }
    {
        const uint32_t x0 = __byte_perm(hi.x, hi.y, 0x5140), x1 = __byte_perm(hi.x, hi.y, 0x7362);
        const uint32_t y0 = __byte_perm(hi.z, hi.w, 0x5140), y1 = __byte_perm(hi.z, hi.w, 0x7362);
        t[0][1] = __byte_perm(x0, y0, 0x5410), t[1][1] = __byte_perm(x0, y0, 0x7632);
        t[2][1] = __byte_perm(x1, y1, 0x5410), t[3][1] = __byte_perm(x1, y1, 0x7632);
    }
    if (ch >= tp.M)
    {
        return;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
    {
        const int p = p0 + 4 * i + k;
        if (p < tp.N)
        {
            const int64_t off = static_cast<int64_t>(p) * tp.ldd + ch;
            uint32_t      w0 = t[k][0], w1 = t[k][1];
            if (full)
            {
                if (tp.residual != nullptr)
                {
                    w0 = add_clamp_u8x4(w0, res[k].x, tp.res_floor4, tp.res_cap4);
                    w1 = add_clamp_u8x4(w1, res[k].y, tp.res_floor4, tp.res_cap4);
                }
                *reinterpret_cast<uint2 *>(tp.dst + off) = make_uint2(w0, w1);
            }
            else
            {
                for (int b = 0; b < 8 && ch + b < tp.M; ++b)
                {
                    uint32_t y = ((b < 4 ? w0 : w1) >> (8 * (b & 3))) & 0xffu;
                    if (tp.residual != nullptr)
                    {
                        y = min(max(min(y + tp.residual[off + b], 255u), tp.res_floor4 & 0xffu), tp.res_cap4 & 0xffu);
                    }
                    tp.dst[off + b] = static_cast<uint8_t>(y);
                }
            }
        }
    }
}

template <bool kS32Out, int kMode>
__device__ __forceinline__ void store_chunk_cm(const uint32_t (&v)[32], const int4 q, const TileParams &tp,
                                               const EpilogueParams &ep, int ch, int p0)
{
    if (ch >= tp.M || p0 >= tp.N)
    {
        return;
    }
    const int64_t base = static_cast<int64_t>(p0) * tp.ldd;
    const int     np   = min(32, tp.N - p0);
    if (kS32Out)
    {
        uint8_t *o = tp.dst + base + 4 * static_cast<int64_t>(ch);
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            if (j < np)
            {
                uint32_t *w = reinterpret_cast<uint32_t *>(o + j * tp.ldd);
                *w          = raw_result_word(static_cast<int32_t>(v[j]) + q.x, ep.accumulate != 0 ? *w : 0u, ep);
            }
        }
    }
    else if (tp.residual != nullptr)
    {
        uint8_t       *o  = tp.dst + base + ch;
        const uint8_t *r  = tp.residual + base + ch;
        const int      fl = static_cast<int>(tp.res_floor4 & 0xffu), cp = static_cast<int>(tp.res_cap4 & 0xffu);
        uint32_t       rs[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            rs[j] = j < np ? static_cast<uint32_t>(__ldg(r + j * tp.ldd)) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            int y = requant_one<kMode>(v[j], q, 0, ep.result_offset, ep.lo, ep.hi);
            if (kMode == kStagePack || kMode == kStagePackS) y = min(max(y, ep.lo), ep.hi); // no packing instruction here to saturate
            if (j < np) o[j * tp.ldd] = static_cast<uint8_t>(min(max(min(y + static_cast<int>(rs[j]), 255), fl), cp));
        }
    }
    else
    {
        uint8_t *o = tp.dst + base + ch;
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            int y = requant_one<kMode>(v[j], q, 0, ep.result_offset, ep.lo, ep.hi);
            if (kMode == kStagePack || kMode == kStagePackS) y = min(max(y, ep.lo), ep.hi); // no packing instruction here to saturate
            if (j < np) o[j * tp.ldd] = static_cast<uint8_t>(y);
        }
    }
}

template <int NPIX, bool kS32Out, int kMode>
__device__ __forceinline__ void drain_channel_major(uint32_t t_addr, const int4 q, const TileParams &tp,
                                                    const EpilogueParams &ep, int ch, int p_first, int lane,
                                                    uint32_t *stage)
{
    static_assert((NPIX / 32) % 2 == 0 || NPIX == 32, "chunks are drained in pairs");
    uint32_t va[32], vb[32];
    tmem_ld_x32(t_addr, va);
    if (!kS32Out && tp.vec_ok) // warp-uniform: rows of dst (and of the residual) are 8-byte aligned
    {
#pragma unroll 1
        for (int c = 0; c < NPIX / 32; c += 2)
        {
            tmem_ld_wait();
            if (c + 1 < NPIX / 32)
            {
                tmem_ld_x32(t_addr + (c + 1) * 32, vb);
            }
            if (p_first + c * 32 < tp.N)
            {
                store_chunk_cm_staged<kMode>(va, q, tp, ep, ch - lane, p_first + c * 32, lane, stage);
            }
            if (c + 1 < NPIX / 32)
            {
                tmem_ld_wait();
                if (c + 2 < NPIX / 32)
                {
                    tmem_ld_x32(t_addr + (c + 2) * 32, va);
                }
                if (p_first + (c + 1) * 32 < tp.N)
                {
                    store_chunk_cm_staged<kMode>(vb, q, tp, ep, ch - lane, p_first + (c + 1) * 32, lane, stage);
                }
            }
        }
        return;
    }
#pragma unroll 1
    for (int c = 0; c < NPIX / 32; c += 2)
    {
        tmem_ld_wait();
        if (c + 1 < NPIX / 32)
        {
            tmem_ld_x32(t_addr + (c + 1) * 32, vb);
        }
        store_chunk_cm<kS32Out, kMode>(va, q, tp, ep, ch, p_first + c * 32);
        if (c + 1 < NPIX / 32)
        {
            tmem_ld_wait();
            if (c + 2 < NPIX / 32)
            {
                tmem_ld_x32(t_addr + (c + 2) * 32, va);
            }
            store_chunk_cm<kS32Out, kMode>(vb, q, tp, ep, ch, p_first + (c + 1) * 32);
        }
    }
}

template <int BLOCK_N, bool kS32Out>
__device__ __forceinline__ void epilogue_warp_tile_cm(uint32_t tmem_acc, const TileParams &tp, const EpilogueParams &ep,
                                                      int warp, int lane, int m0, int n0, uint8_t *out_stage)
{
    static_assert(kCmStageBytes <= kOutStageBytes, "the transpose stage lives in the warp's output staging area");
    uint32_t *stage = reinterpret_cast<uint32_t *>(out_stage + (warp - kFirstEpi) * kOutStageBytes);
    constexpr int NPIX = BLOCK_N / (kEpiWarps / 4);
    const int     quad = warp & 3;                // tensor-memory lane quarter this warp may read
    const int     half = (warp - kFirstEpi) >> 2; // which share of the output rows
    const int     ch   = m0 + quad * 32 + lane;
    int4          q    = make_int4(0, 0, 0, 0);
    if (ch < tp.M)
    {
        if (kS32Out)
        {
            q.x = ep.k_term + (ep.colsum != nullptr ? ep.a_off * __ldg(ep.colsum + ch) : 0); // offset terms only
        }
        else
        {
            q = column_term(ch, tp, ep);
        }
    }
    const uint32_t t_addr = tmem_acc + (static_cast<uint32_t>(quad * 32) << 16) + half * NPIX;
    const int      p0     = n0 + half * NPIX;
    if (tp.mode == kStagePack && !kS32Out)
    {
        drain_channel_major<NPIX, kS32Out, kStagePack>(t_addr, q, tp, ep, ch, p0, lane, stage);
    }
    else if (tp.mode == kStagePackS && !kS32Out)
    {
        drain_channel_major<NPIX, kS32Out, kStagePackS>(t_addr, q, tp, ep, ch, p0, lane, stage);
    }
    else if (tp.mode == kStageWide && !kS32Out)
    {
        drain_channel_major<NPIX, kS32Out, kStageWide>(t_addr, q, tp, ep, ch, p0, lane, stage);
    }
    else if (tp.mode == kStageGeneric)
    {
        drain_channel_major<NPIX, kS32Out, kStageGeneric>(t_addr, q, tp, ep, ch, p0, lane, stage);
    }
    else
    {
        drain_channel_major<NPIX, kS32Out, kStageFast>(t_addr, q, tp, ep, ch, p0, lane, stage);
    }
}

// The part of a tile one epilogue warp owns: lane quarter (warp & 3) and half of the columns.
// kGroups = 2: the eight epilogue warps form two groups of four that drain alternate tiles, each warp all columns
// of its 32 rows (narrow tiles, whose time is latency rather than work).
template <int BLOCK_N, bool kS32Out, int kGroups = 1>
__device__ __forceinline__ void epilogue_warp_tile(uint32_t tmem_acc, const int4 *s_col, const TileParams &tp,
                                                   const EpilogueParams &ep, int warp, int lane, int m0, int n0,
                                                   uint8_t *out_stage, const AccRelease &rel,
                                                   const CUtensorMap *omap = nullptr)
{
    constexpr int NCOLS    = BLOCK_N * kGroups / (kEpiWarps / 4);
    uint8_t      *stage    = out_stage + (warp - kFirstEpi) * kOutStageBytes;
    const int     quad     = warp & 3;               // tensor-memory lane quarter this warp may read
    const int     half     = kGroups == 1 ? (warp - kFirstEpi) >> 2 : 0; // which share of the columns
    const int     m        = m0 + quad * 32 + lane;
    const int32_t row_term = (ep.rowsum != nullptr && m < tp.M) ? ep.b_off * __ldg(ep.rowsum + m) : 0;
    const uint32_t t_addr  = tmem_acc + (static_cast<uint32_t>(quad * 32) << 16) + half * NCOLS;
    if (tp.mode == kStagePack && !kS32Out)
    {
        drain_accumulator<NCOLS, kS32Out, kStagePack>(t_addr, s_col + half * NCOLS, tp, ep, m, n0 + half * NCOLS, row_term,
                                                      stage, lane, rel, omap);
    }
    else if (tp.mode == kStagePackS && !kS32Out)
    {
        drain_accumulator<NCOLS, kS32Out, kStagePackS>(t_addr, s_col + half * NCOLS, tp, ep, m, n0 + half * NCOLS, row_term,
                                                       stage, lane, rel, omap);
    }
    else if (tp.mode == kStageWide && !kS32Out)
    {
        drain_accumulator<NCOLS, kS32Out, kStageWide>(t_addr, s_col + half * NCOLS, tp, ep, m, n0 + half * NCOLS, row_term,
                                                      stage, lane, rel, omap);
    }
    else if (tp.mode == kStageGeneric)
    {
        drain_accumulator<NCOLS, kS32Out, kStageGeneric>(t_addr, s_col + half * NCOLS, tp, ep, m, n0 + half * NCOLS,
                                                         row_term, stage, lane, rel, omap);
    }
    else
    {
        drain_accumulator<NCOLS, kS32Out, kStageFast>(t_addr, s_col + half * NCOLS, tp, ep, m, n0 + half * NCOLS, row_term,
                                                      stage, lane, rel, omap);
    }
}

// KSUB = 128-byte K sub-blocks per pipeline stage.  One barrier hand-over (wait, MMAs, commit) costs the
// issuing thread about 550 clocks whatever it covers, more than the 512 clocks four MMAs keep the tensor
// cores busy, so a stage carries two sub-blocks (eight MMAs) wherever shared memory leaves room for three
// such stages.
// RESB > 0 (implicit convolution with one column block): the whole B operand stays in RESB bytes of shared memory for
// the life of the CTA and the ring holds A stages only.
template <int BLOCK_N, int STAGES, int KSUB, int ACC = 2, bool kPairTma = false, int RESB = 0>
struct SmemPlan
{
    static constexpr int ACC_STAGES = ACC; // accumulator buffers in tensor memory (ACC * BLOCK_N <= 512 columns)
    static_assert(ACC * BLOCK_N <= 512 && (ACC == 2 || ACC == 4), "tensor memory holds 512 columns");
    static_assert(STAGES >= kProdLanes, "the producer lanes of one round must own distinct stages");
    static constexpr int B_SUB      = BLOCK_N * BLOCK_K;          // one K sub-block of the B tile
    static constexpr int A_STAGE_K  = KSUB * A_STAGE;
    static constexpr int B_STAGE    = KSUB * B_SUB;
    static_assert(RESB % 1024 == 0, "the resident operand keeps the 1024-byte alignment of what follows");
    static constexpr int STAGE      = A_STAGE_K + (RESB != 0 ? 0 : B_STAGE);
    static constexpr int OFF_A      = 0;
    static constexpr int OFF_B      = STAGES * A_STAGE_K;         // the B slots of the ring, or the resident B operand
    static constexpr int OFF_COL    = STAGES * STAGE + RESB;      // int4 per column
    static constexpr int EPI_GROUPS = (kEpiWarps == 8 && BLOCK_N <= 128) ? 2 : 1; // see epilogue_warp_tile
    static constexpr int OFF_BAR    = OFF_COL + EPI_GROUPS * BLOCK_N * 16; // full[S], empty[S], tfull[ACC], tempty[ACC]
    static constexpr int OFF_MISC   = OFF_BAR + (2 * STAGES + 2 * ACC) * 8; // tmem base, abort flag
    // per epilogue warp: 32 rows x kOutRowBytes of output staging, 1024-byte aligned (a swizzled source of TMA stores)
    static constexpr int OFF_RESBAR = OFF_MISC + 16;              // kPairTma: one barrier per epilogue warp (residual boxes)
    static constexpr int OFF_OUT    = ((OFF_RESBAR + 8 * kEpiWarps + 1023) / 1024) * 1024;
    // kPairTma: the paired drain stages two tiles of 32 rows x 64 bytes per warp for its bulk tensor stores
    static constexpr int TOTAL      = OFF_OUT + kEpiWarps * (kPairTma ? kPairStageBytes : kOutStageBytes);
    static constexpr int DYN_BYTES  = TOTAL + 1024;               // slack to align the base to 1024
    static constexpr int TMEM_COLS  = ACC * BLOCK_N;
};

// kCM (channel-major): the launcher has exchanged the operand roles -- "A" is the weight matrix, "B" the
// activation matrix, tp.M the number of output channels and tp.N the number of output rows -- so the
// accumulator holds the transposed output tile and epilogue_warp_tile_cm writes it (see there).  Tiles are then
// ordered n-fastest, i.e. all row blocks of one channel block in turn.
template <int BLOCK_N, int STAGES, int KSUB, bool kS32Out, bool kCM, int ACC, bool kPairTma = false>
__global__ void __launch_bounds__(kThreads, 1)
    gemmlowp_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_res,
                            const __grid_constant__ TileParams tp, const EpilogueParams ep)
{
    using P = SmemPlan<BLOCK_N, STAGES, KSUB, ACC, kPairTma>;
    extern __shared__ uint8_t smem_raw[];
    // the 1024-byte aligned start of the dynamic shared memory, derived by pointer arithmetic on the __shared__ array
    // itself: a pointer rebuilt from an integer loses its address space and every access through it becomes a
    // generic load / store (slower, and tracked like a global access) instead of LDS / STS
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t sA       = smem_u32(smem + P::OFF_A);
    const uint32_t sB       = smem_u32(smem + P::OFF_B);
    int4          *s_col    = reinterpret_cast<int4 *>(smem + P::OFF_COL);
    const uint32_t bar_base = smem_u32(smem + P::OFF_BAR);
    auto           full_bar   = [&](int s) { return bar_base + 8u * s; };
    auto           empty_bar  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto           tfull_bar  = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto           tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + ACC + a); };
    uint32_t      *s_tmem     = reinterpret_cast<uint32_t *>(smem + P::OFF_MISC);
    volatile int  *s_abort    = reinterpret_cast<volatile int *>(smem + P::OFF_MISC + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int num_m_blocks = (tp.M + BLOCK_M - 1) / BLOCK_M;
    const int num_n_blocks = (tp.N + BLOCK_N - 1) / BLOCK_N;
    const int num_tiles    = num_m_blocks * num_n_blocks;
    const int num_kb       = (tp.K + KSUB * BLOCK_K - 1) / (KSUB * BLOCK_K); // pipeline stages per tile

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC; ++a)
        {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kEpiWarps / (kCM ? 1 : P::EPI_GROUPS)); // the warps of the group that drains it
        }
        if (kPairTma)
        {
            for (int w = 0; w < kEpiWarps; ++w)
            {
                mbar_init(smem_u32(smem + P::OFF_RESBAR) + 8u * w, 1); // the warp's residual boxes have landed
            }
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp)
    {
        tmem_alloc(smem_u32(s_tmem), P::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    griddep_launch_dependents();
    griddep_wait(); // the prologue above touched no global memory

    if (warp < kProdWarps)
    {
        // ---------------------------------------------------------------- TMA producer
        // kProdWarps warps issue copies independently of each other (one lane each): warp j owns the k-blocks
        // g = j, j + kProdWarps, ... of this CTA's (tile, k-block) sequence.  One thread alone sustains only
        // about one stage per 600 clocks (wait + expect_tx + two tensor copies), less than the tensor cores
        // consume.
        if (lane == 0)
        {
            const int issuer   = warp; // this warp's share of the k-block sequence
            const int my_tiles = static_cast<int>(blockIdx.x) < num_tiles
                                     ? (num_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1
                                     : 0;
            const int total_kb = my_tiles * num_kb;
            uint32_t  issued = 0, parities = 0;
            bool      ok = true;
            int       ti = 0, kb = issuer; // (tile ordinal, k-block) of g, kept incrementally
            while (kb >= num_kb)
            {
                kb -= num_kb;
                ++ti;
            }
            int      st = issuer % STAGES;
            uint32_t ph = static_cast<uint32_t>(issuer / STAGES) & 1u;
            for (int g = issuer; g < total_kb; g += kProdLanes)
            {
                ok = mbar_wait(empty_bar(st), ph ^ 1, s_abort, DEV_TIMEOUT_PRODUCER, tp.spin_limit);
                if (!ok)
                {
                    break;
                }
                const int tile = static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x);
                const int m0   = (kCM ? tile / num_n_blocks : tile % num_m_blocks) * BLOCK_M;
                const int n0   = (kCM ? tile % num_n_blocks : tile / num_m_blocks) * BLOCK_N;
                if (kb == 0) trace_event(tp.trace, ti, 0);
                if (!kCM && tp.conv_c != 0)
                {
                    // window origin of the tile's first output pixel; sub-blocks beyond K are not loaded at all (the
                    // MMA loop leaves them out as well)
                    const int t  = fast_div(m0, tp.conv_div_wo);
                    const int q  = m0 - t * tp.conv_wo;
                    const int n  = fast_div(t, tp.conv_div_ho);
                    const int pp = t - n * tp.conv_ho;
                    const int w0 = q * tp.conv_sx - tp.conv_pl, h0 = pp * tp.conv_sy - tp.conv_pt;
                    const int left  = (tp.K - kb * KSUB * BLOCK_K + BLOCK_K - 1) / BLOCK_K;
                    const int valid = left < KSUB ? left : KSUB;
                    if (tp.conv_c == 64)
                    {
                        // 64 channels: a 128-byte K block is two filter taps, loaded as two tiles of 128 pixels x 64 bytes
                        // (64-byte swizzle) one behind the other; the last block of an odd tap count holds one
                        const int taps_left = (tp.K >> 6) - 2 * kb * KSUB;
                        const int taps      = taps_left < 2 * KSUB ? taps_left : 2 * KSUB;
                        mbar_expect_tx(full_bar(st), taps * (A_STAGE / 2) + valid * P::B_SUB);
#pragma unroll
                        for (int j = 0; j < 2 * KSUB; ++j)
                        {
                            if (j < taps)
                            {
                                const int tap = 2 * kb * KSUB + j;
                                const int ky = tap / tp.conv_kw, kx = tap - ky * tp.conv_kw;
                                tma_load_im2col(sA + st * P::A_STAGE_K + j * (A_STAGE / 2), &tmap_a, 0, w0, h0, n,
                                                static_cast<uint16_t>(kx * tp.conv_dx),
                                                static_cast<uint16_t>(ky * tp.conv_dy), full_bar(st));
                            }
                        }
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
                            if (sub < valid)
                            {
                                tma_load_2d(sB + st * P::B_STAGE + sub * P::B_SUB, &tmap_b, (kb * KSUB + sub) * BLOCK_K, n0,
                                            full_bar(st));
                            }
                        }
                    }
                    else
                    {
                        mbar_expect_tx(full_bar(st), valid * (A_STAGE + P::B_SUB));
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
                            if (sub < valid)
                            {
                                const int k0  = (kb * KSUB + sub) * BLOCK_K;
                                const int tap = k0 / tp.conv_c, c0 = k0 - tap * tp.conv_c;
                                const int ky = tap / tp.conv_kw, kx = tap - ky * tp.conv_kw;
                                tma_load_im2col(sA + st * P::A_STAGE_K + sub * A_STAGE, &tmap_a, c0, w0, h0, n,
                                                static_cast<uint16_t>(kx * tp.conv_dx),
                                                static_cast<uint16_t>(ky * tp.conv_dy), full_bar(st));
                                tma_load_2d(sB + st * P::B_STAGE + sub * P::B_SUB, &tmap_b, k0, n0, full_bar(st));
                            }
                        }
                    }
                    issued |= 1u << st;
                    parities = (parities & ~(1u << st)) | (ph << st);
                }
                else if (g != tp.withhold_kb || blockIdx.x != 0)
                {
                    mbar_expect_tx(full_bar(st), P::STAGE);
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub)
                    {
                        const int k0 = (kb * KSUB + sub) * BLOCK_K; // beyond K: the copy delivers zeros
                        tma_load_2d(sA + st * P::A_STAGE_K + sub * A_STAGE, &tmap_a, k0, m0, full_bar(st));
                        tma_load_2d(sB + st * P::B_STAGE + sub * P::B_SUB, &tmap_b, k0, n0, full_bar(st));
                    }
                    issued |= 1u << st;
                    parities = (parities & ~(1u << st)) | (ph << st);
                }
                // advance g by kProdLanes
                kb += kProdLanes;
                while (kb >= num_kb)
                {
                    kb -= num_kb;
                    ++ti;
                }
                st += kProdLanes;
                if (st >= STAGES)
                {
                    st -= STAGES;
                    ph ^= 1;
                }
            }
            if (!ok || *s_abort != 0)
            {
                // wait, with a limit of its own, until the copies this lane issued have landed
                for (int i = 0; i < STAGES; ++i)
                {
                    if ((issued >> i) & 1u)
                    {
                        const long long t0 = clock64();
                        while (!mbar_try_wait(full_bar(i), (parities >> i) & 1u))
                        {
                            if (clock64() - t0 > tp.spin_limit)
                            {
                                *s_abort = DEV_TIMEOUT_DRAIN;
                                break;
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    else if (warp == kMmaWarp)
    {
        // ---------------------------------------------------------------- MMA issuer
        // One lane runs the whole loop: tcgen05.mma / commit are single-thread instructions, and 32 lanes
        // polling the same barrier only slow the hand-over down.
        if (lane == 0)
        {
            int      s = 0, as = 0;
            uint32_t ph = 0, aph = 0;
            bool     ok = true, have = false; // have: the current stage's operands are known to have landed
            int      ti = 0;
            // 64-channel convolution through im2col-mode loads: the A stage holds 64-byte rows, a filter tap per 8 KB
            const bool     a_sw64  = !kCM && tp.conv_c == 64;
            const uint64_t a_desc0 = a_sw64 ? make_kmajor_sw64_desc(sA) : make_kmajor_sw128_desc(sA);
            const uint64_t b_desc0 = make_kmajor_sw128_desc(sB);
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++ti)
            {
                ok = mbar_wait(tempty_bar(as), aph ^ 1, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                if (!ok)
                {
                    break;
                }
                trace_event(tp.trace, ti, 1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BLOCK_N;
                long long      waited = 0;
                for (int kb = 0; kb < num_kb; ++kb)
                {
                    if (!have)
                    {
                        const long long w0 = tp.trace != nullptr ? clock64() : 0;
                        ok = mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                        if (tp.trace != nullptr) waited += clock64() - w0;
                        if (!ok)
                        {
                            break;
                        }
                    }
                    // Ask for the NEXT stage's barrier now: the answer travels while this stage's MMAs and
                    // commit are being issued, which takes the barrier round trip off the issue path.
                    int      sn  = s + 1;
                    uint32_t phn = ph;
                    if (sn == STAGES)
                    {
                        sn = 0;
                        phn ^= 1;
                    }
                    have = mbar_test_wait(full_bar(sn), phn);
                    tc_fence_after();
                    if (kb == 0) trace_event(tp.trace, ti, 2);
                    // stage offset in 16-byte units; advancing K by 32 bytes inside the swizzle row: +2
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * P::A_STAGE_K) >> 4);
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * P::B_STAGE) >> 4);
                    // A stage wholly inside K and 128-byte-swizzle operands (the common case): the MMAs back to back with
                    // nothing to test on the issuing thread's critical path.  Else the K steps beyond K are left out (zero
                    // fill, or with im2col-mode loads not loaded at all) and 64-byte-swizzle A tiles are addressed tap by tap.
                    if ((kb + 1) * KSUB * BLOCK_K <= tp.K && !a_sw64)
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
                                umma_i8(d_tmem, a_desc + static_cast<uint64_t>((sub * A_STAGE) >> 4) + 2u * k,
                                        b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, tp.idesc,
                                        (kb | sub | k) != 0 ? 1u : 0u);
                            }
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
                                if ((kb * KSUB + sub) * BLOCK_K + k * UMMA_K < tp.K)
                                {
                                    // 32 bytes on inside the swizzled row: + 2; 64-byte rows: the next tap's tile after two steps
                                    const uint32_t a_k = a_sw64 ? static_cast<uint32_t>((k >> 1) * ((A_STAGE / 2) >> 4) + 2 * (k & 1))
                                                                : 2u * k;
                                    umma_i8(d_tmem, a_desc + static_cast<uint64_t>((sub * A_STAGE) >> 4) + a_k,
                                            b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, tp.idesc,
                                            (kb | sub | k) != 0 ? 1u : 0u);
                                }
                            }
                        }
                    }
                    umma_commit(empty_bar(s)); // frees the smem stage once these MMAs have read it
                    s  = sn;
                    ph = phn;
                }
                if (ok)
                {
                    umma_commit(tfull_bar(as)); // accumulator complete
                    trace_event(tp.trace, ti, 3);
                    trace_value(tp.trace, ti, 6, waited); // clocks spent waiting for operands
                }
                if (++as == ACC)
                {
                    as = 0;
                    aph ^= 1;
                }
            }
        }
        __syncwarp();
    }
    else
    {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // One group of all epilogue warps, or (narrow tiles, eight warps) two groups of four draining alternate
        // tiles: accumulator buffer and phase follow from the tile ordinal, so the groups need not talk.
        constexpr int kGroups = kCM ? 1 : P::EPI_GROUPS;
        const int     group   = kGroups == 1 ? 0 : (warp - kFirstEpi) >> 2;
        const int     et      = threadIdx.x - 32 * kFirstEpi - group * 128; // thread index inside the group
        int4         *g_col   = s_col + group * BLOCK_N;
        bool          ok      = true;
        int           ti = 0;
        int           filled_n0 = -1;
        // Paired drain (see drain_accumulator_pair): the tile this group drains next (kStride ordinals on) is drained
        // together with the current one when it lies in the same column block and its accumulator buffer belongs
        // to the same phase.  The MMA warp is untouched: it fills the partner buffer while the first one waits
        // here, and meets both released afterwards.
        // Only the 256-column tiles with their two buffers: with four buffers and two epilogue groups, and in the
        // implicit convolution, pairing measured slower (the MMA warp can no longer run two tiles ahead).
        constexpr int  kStride  = 1;
        // Two buffers only: with 128-column tiles in four buffers, pairs (0, 1) and (2, 3) drained by sixteen warps while
        // the MMA warp fills the other pair, the same layers measured slower (802816 x 256 x 64: 164 against 133 us).
        constexpr bool kCanPair = !kCM && !kS32Out && kGroups == 1 && ACC == 2;
        int            skip     = -1; // ordinal of a tile already drained as the partner of an earlier one
        uint32_t       n_res_pairs = 0; // kPairTma: pairs whose residual this warp has fetched (phase of its barrier)
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++ti)
        {
            if ((kGroups > 1 && (ti & 1) != group) || ti == skip)
            {
                continue;
            }
            const int      as  = ti % ACC;
            const uint32_t aph = static_cast<uint32_t>(ti / ACC) & 1u;
            const int      m0  = (kCM ? tile / num_n_blocks : tile % num_m_blocks) * BLOCK_M;
            const int      n0  = (kCM ? tile % num_n_blocks : tile / num_m_blocks) * BLOCK_N;
            // The warps of a group meet only where the column terms change (tiles are ordered m-fastest, so the terms
            // usually carry over): between such points every warp waits for its accumulator, drains its share and hands
            // it back on its own, and a slow warp holds nobody up.  A warp whose wait ran out keeps walking the tile
            // list without working, so that the barrier counts stay whole until all leave together.
            if (!kCM && n0 != filled_n0)
            {
                if (!(kGroups == 1 ? epi_barrier_and(ok) : epi_group_barrier_and(ok, group)))
                {
                    break; // the old terms are no longer read by anyone; someone gave up
                }
                fill_column_terms<BLOCK_N>(g_col, et, n0, tp, ep, kEpiThreads / kGroups);
                filled_n0 = n0;
                if (kGroups == 1) epi_barrier();
                else epi_group_barrier(group);
            }
            if (!ok)
            {
                continue;
            }
            const int tile_b   = tile + kStride * static_cast<int>(gridDim.x);
            bool      pair_now = false;
            if (kCanPair && tp.pair_drain != 0 && (tp.mode == kStageWide || tp.mode == kStagePack || tp.mode == kStagePackS) && (as & 1) == 0)
            {
                pair_now = tile_b < num_tiles && tile_b / num_m_blocks == tile / num_m_blocks;
            }
            const int m0b = kCanPair ? (tile_b % num_m_blocks) * BLOCK_M : 0;
            // kPairTma: the warp's share of both tiles leaves as two bulk tensor stores from its staging area, and a fused
            // residual arrives there as two bulk tensor loads, requested here, ahead of the accumulators
            const uint32_t pair_stage =
                (kPairTma && kCanPair && pair_now && tp.tma_store != 0)
                    ? smem_u32(smem + P::OFF_OUT) + static_cast<uint32_t>(warp - kFirstEpi) * kPairStageBytes
                    : 0u;
            const bool     res_tma = pair_stage != 0 && tp.residual != nullptr;
            const uint32_t res_bar = smem_u32(smem + P::OFF_RESBAR) + 8u * static_cast<uint32_t>(warp - kFirstEpi);
            if (res_tma)
            {
                constexpr int NCOLS = BLOCK_N * kGroups / (kEpiWarps / 4);
                const int     first = n0 + (kGroups == 1 ? (warp - kFirstEpi) >> 2 : 0) * NCOLS;
                request_residual_boxes(&tmap_res, pair_stage, res_bar, first, m0 + (warp & 3) * 32, m0b + (warp & 3) * 32, lane);
                // (asking the pair after this one into L2 as well, a drain ahead, measured slower: 142 against 135 us)
            }
            else if (!kCM && !kS32Out && tp.residual != nullptr)
            {
                constexpr int NCOLS = BLOCK_N * kGroups / (kEpiWarps / 4);
                const int     row   = (warp & 3) * 32 + lane;
                const int     first = n0 + (kGroups == 1 ? (warp - kFirstEpi) >> 2 : 0) * NCOLS;
                prefetch_residual(tp, m0 + row, first, NCOLS);
                if (pair_now)
                {
                    prefetch_residual(tp, m0b + row, first, NCOLS);
                }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(as), aph, s_abort, DEV_TIMEOUT_EPILOGUE, tp.spin_limit));
            if (ok && pair_now)
            {
                ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(as + kStride), aph, s_abort, DEV_TIMEOUT_EPILOGUE, tp.spin_limit));
            }
            if (ok)
            {
                tc_fence_after();
                if (et == 0) trace_event(tp.trace, ti, 4);
                // one arrival per warp and buffer, made inside the drain as soon as the warp's last load has landed
                const AccRelease rel{tempty_bar(as), pair_now ? tempty_bar(as + kStride) : 0u, false};
                if (kCM)
                {
                    epilogue_warp_tile_cm<BLOCK_N, kS32Out>(tmem_base + as * BLOCK_N, tp, ep, warp, lane, m0, n0,
                                                            smem + P::OFF_OUT);
                    release_accumulators(rel, lane);
                }
                else if (kCanPair && pair_now)
                {
                    epilogue_warp_tile_pair<BLOCK_N, kGroups>(tmem_base + as * BLOCK_N, tmem_base + (as + kStride) * BLOCK_N,
                                                              g_col, tp, ep, warp, lane, m0, m0b, n0, rel, pair_stage, &tmap_out,
                                                              &tmap_res, res_bar, n_res_pairs & 1u, s_abort);
                }
                else
                {
                    epilogue_warp_tile<BLOCK_N, kS32Out, kGroups>(tmem_base + as * BLOCK_N, g_col, tp, ep, warp, lane,
                                                                  m0, n0, smem + P::OFF_OUT, rel,
                                                                  (tp.tma_store != 0 && !kPairTma) ? &tmap_out : nullptr);
                }
                __syncwarp();
                if (et == 0) trace_event(tp.trace, ti, 5);
                if (pair_now)
                {
                    skip = ti + kStride;
                }
            }
            if (res_tma)
            {
                if (*s_abort != 0) // a wait was given up: let this warp's residual boxes land before anything else
                {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(res_bar, n_res_pairs & 1u) && clock64() - t0 < tp.spin_limit)
                    {
                    }
                }
                ++n_res_pairs;
            }
        }
        if (tp.tma_store != 0 && lane == 0)
        {
            tma_store_wait_all(); // this warp's bulk stores: shared memory stays valid until they have read it
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp)
    {
        tc_fence_after();
        tmem_dealloc(tmem_base, P::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s_abort != 0)
    {
        atomicCAS(tp.status, 0, *s_abort);
    }
}


#if CUGL_TC_FULL_BUILD
// ---------------------------------------------------------------------------------------------------
// Two-CTA kernel: a cluster of two CTAs (an SM pair) per 256 x 256 output tile.
//   CTA rank r stages rows [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of Bt (its half of the
//   B tile), owns the accumulator rows [m0 + 128 r, +128) x 256 columns in its tensor memory and runs
//   the epilogue for them.  The MMA issuer of rank 0 drives the tensor cores of both SMs.
//   Barriers: full[] lives in rank 0 and collects the bytes of both CTAs' copies; empty[] and tfull[]
//   exist in both CTAs and are signalled together by a multicast tcgen05.commit; tempty[] lives in rank 0
//   and is arrived on by the sixteen epilogue warps of the pair.
// ---------------------------------------------------------------------------------------------------
template <int STAGES, int KSUB>
struct SmemPlan2
{
    static constexpr int BLOCK_N   = 256;
    static constexpr int B_SUB     = (BLOCK_N / 2) * BLOCK_K; // one K sub-block of this CTA's half of the B tile
    static constexpr int A_STAGE_K = KSUB * A_STAGE;
    static constexpr int B_STAGE   = KSUB * B_SUB;
    static constexpr int STAGE     = A_STAGE_K + B_STAGE;
    static constexpr int OFF_A     = 0;
    static constexpr int OFF_B     = STAGES * A_STAGE_K;
    static constexpr int OFF_COL   = STAGES * STAGE;
    static constexpr int OFF_BAR   = OFF_COL + BLOCK_N * 16;
    static constexpr int OFF_MISC  = OFF_BAR + (2 * STAGES + 4) * 8;
    static constexpr int OFF_OUT   = ((OFF_MISC + 16 + 1023) / 1024) * 1024; // staging: a swizzled source of TMA stores
    static constexpr int TOTAL     = OFF_OUT + kEpiWarps * kOutStageBytes;
    static constexpr int DYN_BYTES = TOTAL + 1024;
    static constexpr int TMEM_COLS = 2 * BLOCK_N;
};

template <int STAGES, int KSUB, bool kS32Out>
__global__ void __launch_bounds__(kThreads, 1)
    gemmlowp_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                 const __grid_constant__ CUtensorMap tmap_b,
                                 const __grid_constant__ CUtensorMap tmap_bh, const __grid_constant__ CUtensorMap tmap_out,
                                 const __grid_constant__ TileParams tp, const EpilogueParams ep)
{
    using P               = SmemPlan2<STAGES, KSUB>;
    constexpr int BLOCK_N = P::BLOCK_N;
    extern __shared__ uint8_t smem_raw[];
    // the 1024-byte aligned start of the dynamic shared memory, derived by pointer arithmetic on the __shared__ array
    // itself: a pointer rebuilt from an integer loses its address space and every access through it becomes a
    // generic load / store (slower, and tracked like a global access) instead of LDS / STS
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t sA         = smem_u32(smem + P::OFF_A);
    const uint32_t sB         = smem_u32(smem + P::OFF_B);
    int4          *s_col      = reinterpret_cast<int4 *>(smem + P::OFF_COL);
    const uint32_t bar_base   = smem_u32(smem + P::OFF_BAR);
    auto           full_bar   = [&](int s) { return bar_base + 8u * s; };
    auto           empty_bar  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto           tfull_bar  = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto           tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    uint32_t      *s_tmem     = reinterpret_cast<uint32_t *>(smem + P::OFF_MISC);
    volatile int  *s_abort    = reinterpret_cast<volatile int *>(smem + P::OFF_MISC + 4);

    const int      warp   = threadIdx.x >> 5;
    const int      lane   = threadIdx.x & 31;
    const uint32_t rank   = cluster_ctarank();
    const bool     leader = rank == 0;

    const int num_m_blocks = (tp.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
    const int num_n_blocks = (tp.N + BLOCK_N - 1) / BLOCK_N;
    const int num_tiles    = num_m_blocks * num_n_blocks;
    const int num_kb       = (tp.K + KSUB * BLOCK_K - 1) / (KSUB * BLOCK_K); // pipeline stages per tile
    const int first_tile   = static_cast<int>(cluster_id_x());
    const int tile_stride  = static_cast<int>(num_clusters_x());
    // Tail split.  With T tiles on G SM pairs the last wave holds T mod G tiles and costs as much as a full
    // one.  When twice that many fit into one wave, each of those tiles is processed as two 256 x 128 halves
    // (tmap_bh: 64-row boxes of B per CTA, an MMA of N = 128) by two pairs, and the wave takes half the time.
    // Work items v = 0 .. num_items-1: v < first_split is tile v; above, item first_split + 2j + h is half h of
    // tile first_split + j.
    const int tail        = num_tiles % tile_stride;
    const int n_split     = (tp.split_tail != 0 && tail > 0 && 2 * tail <= tile_stride) ? tail : 0;
    const int first_split = num_tiles - n_split;
    const int num_items   = num_tiles + n_split;
    auto      item_tile   = [&](int v) { return v < first_split ? v : first_split + ((v - first_split) >> 1); };
    auto      item_half   = [&](int v) { return v < first_split ? -1 : ((v - first_split) & 1); }; // -1: whole tile

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), 1);  // used in the leader only: its producer's arrive + both CTAs' bytes
            mbar_init(empty_bar(s), 1); // multicast commit of the leader's MMA issuer
        }
        for (int a = 0; a < 2; ++a)
        {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * kEpiWarps); // used in the leader only: the epilogue warps of both CTAs
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp)
    {
        tmem_alloc_pair(smem_u32(s_tmem), P::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync(); // the peer's barriers are initialised before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    griddep_launch_dependents();
    griddep_wait(); // the prologue above touched no global memory

    if (warp < kProdWarps)
    {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        // Same independent issue loops as the one-CTA kernel; the byte counts of both CTAs' copies are
        // credited to the leader's "full" barrier, whose expected total the leader's lane announces.
        if (lane == 0)
        {
            const int issuer   = warp;
            const int my_tiles = first_tile < num_items ? (num_items - 1 - first_tile) / tile_stride + 1 : 0;
            const int total_kb = my_tiles * num_kb;
            int       ti = 0, kb = issuer;
            while (kb >= num_kb)
            {
                kb -= num_kb;
                ++ti;
            }
            int      st = issuer % STAGES;
            uint32_t ph = static_cast<uint32_t>(issuer / STAGES) & 1u;
            for (int g = issuer; g < total_kb; g += kProdLanes)
            {
                if (!mbar_wait(empty_bar(st), ph ^ 1, s_abort, DEV_TIMEOUT_PRODUCER, tp.spin_limit))
                {
                    break;
                }
                const int item = first_tile + ti * tile_stride;
                const int tile = item_tile(item), half = item_half(item);
                const int m0   = (tile % num_m_blocks) * 2 * BLOCK_M + static_cast<int>(rank) * BLOCK_M;
                const int n0   = (tile / num_m_blocks) * BLOCK_N +
                               (half < 0 ? static_cast<int>(rank) * (BLOCK_N / 2)
                                         : half * (BLOCK_N / 2) + static_cast<int>(rank) * (BLOCK_N / 4));
                if (kb == 0) trace_event(tp.trace, ti, 0);
                const uint32_t leader_full = map_to_cta(full_bar(st), 0);
                const bool     withheld    = g == tp.withhold_kb && blockIdx.x == 0; // the leader of cluster 0
                if (tp.conv_c != 0)
                {
                    // implicit convolution: im2col-mode loads of this CTA's 128 output pixels; K sub-blocks beyond K are
                    // neither loaded nor multiplied
                    const int t  = fast_div(m0, tp.conv_div_wo);
                    const int q  = m0 - t * tp.conv_wo;
                    const int n  = fast_div(t, tp.conv_div_ho);
                    const int pp = t - n * tp.conv_ho;
                    const int w0 = q * tp.conv_sx - tp.conv_pl, h0 = pp * tp.conv_sy - tp.conv_pt;
                    const int left  = (tp.K - kb * KSUB * BLOCK_K + BLOCK_K - 1) / BLOCK_K;
                    const int valid = left < KSUB ? left : KSUB;
                    if (leader)
                    {
                        mbar_expect_tx(full_bar(st), 2 * valid * (A_STAGE + (half < 0 ? P::B_SUB : P::B_SUB / 2)));
                    }
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub)
                    {
                        if (sub < valid)
                        {
                            const int k0  = (kb * KSUB + sub) * BLOCK_K;
                            const int tap = k0 / tp.conv_c, c0 = k0 - tap * tp.conv_c;
                            const int ky = tap / tp.conv_kw, kx = tap - ky * tp.conv_kw;
                            tma_load_im2col_pair(sA + st * P::A_STAGE_K + sub * A_STAGE, &tmap_a, c0, w0, h0, n,
                                                 static_cast<uint16_t>(kx * tp.conv_dx),
                                                 static_cast<uint16_t>(ky * tp.conv_dy), leader_full);
                            tma_load_2d_pair(sB + st * P::B_STAGE + sub * P::B_SUB, half < 0 ? &tmap_b : &tmap_bh, k0, n0,
                                             leader_full);
                        }
                    }
                }
                else
                {
                    if (leader && !withheld)
                    {
                        // the bytes of both CTAs
                        mbar_expect_tx(full_bar(st), half < 0 ? 2 * P::STAGE : 2 * (P::A_STAGE_K + P::B_STAGE / 2));
                    }
#pragma unroll
                    for (int sub = 0; sub < KSUB && !withheld; ++sub)
                    {
                        const int k0 = (kb * KSUB + sub) * BLOCK_K;
                        tma_load_2d_pair(sA + st * P::A_STAGE_K + sub * A_STAGE, &tmap_a, k0, m0, leader_full);
                        tma_load_2d_pair(sB + st * P::B_STAGE + sub * P::B_SUB, half < 0 ? &tmap_b : &tmap_bh, k0, n0,
                                         leader_full);
                    }
                }
                kb += kProdLanes;
                while (kb >= num_kb)
                {
                    kb -= num_kb;
                    ++ti;
                }
                st += kProdLanes;
                if (st >= STAGES)
                {
                    st -= STAGES;
                    ph ^= 1;
                }
            }
        }
        __syncwarp();
    }
    else if (warp == kMmaWarp)
    {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (leader && lane == 0)
        {
            int      s = 0, as = 0;
            uint32_t ph = 0, aph = 0;
            bool     ok = true, have = false; // have: the current stage's operands are known to have landed
            int      ti = 0;
            const uint64_t a_desc0 = make_kmajor_sw128_desc(sA);
            const uint64_t b_desc0 = make_kmajor_sw128_desc(sB);
            for (int item = first_tile; item < num_items && ok; item += tile_stride, ++ti)
            {
                const uint32_t idesc = item_half(item) < 0 ? tp.idesc : tp.idesc_half;
                ok = mbar_wait(tempty_bar(as), aph ^ 1, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                if (!ok)
                {
                    break;
                }
                trace_event(tp.trace, ti, 1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BLOCK_N;
                long long      waited = 0;
                for (int kb = 0; kb < num_kb; ++kb)
                {
                    if (!have)
                    {
                        const long long w0 = tp.trace != nullptr ? clock64() : 0;
                        ok = mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                        if (tp.trace != nullptr) waited += clock64() - w0;
                        if (!ok)
                        {
                            break;
                        }
                    }
                    // Ask for the NEXT stage's barrier now: the answer travels while this stage's MMAs and
                    // commit are being issued, which takes the barrier round trip off the issue path.
                    int      sn  = s + 1;
                    uint32_t phn = ph;
                    if (sn == STAGES)
                    {
                        sn = 0;
                        phn ^= 1;
                    }
                    have = mbar_test_wait(full_bar(sn), phn);
                    tc_fence_after();
                    if (kb == 0) trace_event(tp.trace, ti, 2);
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * P::A_STAGE_K) >> 4);
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((s * P::B_STAGE) >> 4);
                    // a stage that lies wholly inside K (all but the last one): the MMAs back to back, nothing to test on the
                    // issuing thread's critical path; the last stage leaves out the K steps beyond K (zero fill, or with
                    // im2col-mode loads not loaded at all)
                    if ((kb + 1) * KSUB * BLOCK_K <= tp.K)
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
                                umma_i8_pair(d_tmem, a_desc + static_cast<uint64_t>((sub * A_STAGE) >> 4) + 2u * k,
                                             b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, idesc,
                                             (kb | sub | k) != 0 ? 1u : 0u);
                            }
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
                                if ((kb * KSUB + sub) * BLOCK_K + k * UMMA_K < tp.K)
                                {
                                    umma_i8_pair(d_tmem, a_desc + static_cast<uint64_t>((sub * A_STAGE) >> 4) + 2u * k,
                                                 b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, idesc,
                                                 (kb | sub | k) != 0 ? 1u : 0u);
                                }
                            }
                        }
                    }
                    umma_commit_pair(empty_bar(s)); // frees this stage in both CTAs
                    s  = sn;
                    ph = phn;
                }
                if (ok)
                {
                    umma_commit_pair(tfull_bar(as)); // accumulator complete, both CTAs
                    trace_event(tp.trace, ti, 3);
                    trace_value(tp.trace, ti, 6, waited); // clocks spent waiting for operands
                }
                if (++as == 2)
                {
                    as = 0;
                    aph ^= 1;
                }
            }
        }
        __syncwarp();
    }
    else
    {
        // ---------------------------------------------------------------- epilogue (warps 2..9, both CTAs)
        const int et = threadIdx.x - 32 * kFirstEpi; // 0 .. kEpiThreads-1
        int       as = 0;
        uint32_t  aph = 0;
        bool      ok = true;
        int       ti = 0;
        int       filled_n0 = -1;
        for (int item = first_tile; item < num_items; item += tile_stride, ++ti)
        {
            if (!epi_barrier_and(ok))
            {
                break;
            }
            const int tile = item_tile(item), half = item_half(item);
            const int m0   = (tile % num_m_blocks) * 2 * BLOCK_M + static_cast<int>(rank) * BLOCK_M;
            const int n0   = (tile / num_m_blocks) * BLOCK_N + (half > 0 ? BLOCK_N / 2 : 0);
            if (n0 != filled_n0) // tiles are ordered m-fastest: the column terms usually carry over
            {
                fill_column_terms<BLOCK_N>(s_col, et, n0, tp, ep);
                filled_n0 = n0;
                epi_barrier();
            }
            ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(as), aph, s_abort, DEV_TIMEOUT_EPILOGUE, tp.spin_limit));
            if (ok)
            {
                tc_fence_after();
                if (et == 0) trace_event(tp.trace, ti, 4);
                const AccRelease rel{map_to_cta(tempty_bar(as), 0), 0u, true}; // one arrival per warp, at the leader
                if (half < 0)
                {
                    epilogue_warp_tile<BLOCK_N, kS32Out>(tmem_base + as * BLOCK_N, s_col, tp, ep, warp, lane, m0, n0,
                                                         smem + P::OFF_OUT, rel, tp.tma_store != 0 ? &tmap_out : nullptr);
                }
                else
                {
                    epilogue_warp_tile<BLOCK_N / 2, kS32Out>(tmem_base + as * BLOCK_N, s_col, tp, ep, warp, lane, m0, n0,
                                                             smem + P::OFF_OUT, rel, tp.tma_store != 0 ? &tmap_out : nullptr);
                }
                __syncwarp();
                if (et == 0) trace_event(tp.trace, ti, 5);
            }
            if (++as == 2)
            {
                as = 0;
                aph ^= 1;
            }
        }
        if (tp.tma_store != 0 && lane == 0)
        {
            tma_store_wait_all(); // this warp's bulk stores: shared memory stays valid until they have read it
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync(); // neither CTA leaves (or frees tensor memory) while its peer may still touch it
    if (warp == kMmaWarp)
    {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, P::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s_abort != 0)
    {
        atomicCAS(tp.status, 0, *s_abort);
    }
}


// ---------------------------------------------------------------------------------------------------
// Implicit-GEMM convolution (NHWC, 8-bit): the same one-CTA pipeline, but the A tile (128 output pixels x
// 128 bytes of the (ky, kx, c) patch axis) is gathered straight from the input tensor by four extra warps
// instead of being read from a materialised im2col matrix, which is never written.  This is the role of
// CpuIm2ColKernel + the arm_gemm "indirect" mode (src/cpu/operators/internal/CpuGemmAssemblyDispatch.cpp:396-431).
// Eight gather threads share one tile row: each loads one 16-byte piece per K sub-block (a piece never straddles
// a filter tap because C is a multiple of 16) and stores it with the 128-byte swizzle the tensor cores
// expect (piece j of row r lands at piece j ^ (r & 7)).  The copies are cp.async (global -> shared without
// registers) and the stage's barrier is told to arrive when they land (cp.async.mbarrier.arrive), so a whole
// ring of stages is in flight per thread.  Out-of-image taps copy 16 bytes of the input zero point from a small
// pad buffer, exactly what im2col would have written (the reference's indirect mode points such taps at a
// zero-point row as well), so the offset terms of the epilogue need no correction.
// ---------------------------------------------------------------------------------------------------
struct ConvGeom
{
    const uint8_t *src; // [B][H][W][C]
    const uint8_t *pad; // 16 bytes of the input zero point per gather thread (kConvPadBytes in all)
    int            C, W, H, kw, kh, sx, sy, pad_l, pad_t, dil_x, dil_y, Wo, Ho;
    FastDiv        div_wo, div_ho;
};

// One entry per 16-byte piece of the patch axis: where the piece lies relative to the top-left tap of an
// output pixel.  Built once per CTA in shared memory so that the gather loop has no division in it.
struct TapEntry
{
    int32_t  offset; // bytes from the (ky = 0, kx = 0, c = 0) element, in the input tensor
    uint32_t dydx;   // (ky * dilation_y) << 16 | (kx * dilation_x)
};
constexpr int kConvMaxPieces = 1024; // K <= 16384 bytes

constexpr int kGatherWarps  = 8;
static_assert(kConvPadBytes >= 16 * 32 * kGatherWarps, "one pad piece per gather thread");
constexpr int kFirstGather  = kFirstEpi + kEpiWarps;
constexpr int kConvThreads  = kThreads + 32 * kGatherWarps;

// RESB > 0: a convolution with a single column block (N <= BLOCK_N) whose weights fit into RESB bytes.  Every tile of
// every CTA multiplies by the same B operand, so the producer thread loads it once and the ring carries patches only:
// a third less traffic from L2 into shared memory for 64 output channels, and a deeper ring in the space set free.
// MT = 2 (with a resident B operand, four accumulator buffers and two epilogue groups): a unit of work is 256 output
// pixels, two 128-row tiles that share every hand-over -- one stage barrier, one commit and one accumulator-ready signal
// for both, where a 64-column tile is bound by exactly those (the tensor pipe is busy a quarter of the time).  A stage
// holds the patches of both tiles for one K step; epilogue group g drains tile g of every unit.
template <int BLOCK_N, int STAGES, int KSUB, int ACC, int RESB = 0, int MT = 1>
__global__ void __launch_bounds__(kConvThreads, 1)
    gemmlowp_conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_out,
                                 const __grid_constant__ TileParams tp, const EpilogueParams ep, const ConvGeom cg)
{
    using P = SmemPlan<BLOCK_N, STAGES, MT * KSUB, ACC, false, RESB>; // the A ring: MT x KSUB sub-tiles per stage
    static_assert(MT == 1 || (MT == 2 && RESB != 0 && ACC == 4 && P::EPI_GROUPS == 2), "double tiles: resident B, four buffers, two groups");
    constexpr int UNIT_M = MT * BLOCK_M;
    extern __shared__ uint8_t smem_raw[];
    // the 1024-byte aligned start of the dynamic shared memory, derived by pointer arithmetic on the __shared__ array
    // itself: a pointer rebuilt from an integer loses its address space and every access through it becomes a
    // generic load / store (slower, and tracked like a global access) instead of LDS / STS
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    const uint32_t sA         = smem_u32(smem + P::OFF_A);
    const uint32_t sB         = smem_u32(smem + P::OFF_B);
    int4          *s_col      = reinterpret_cast<int4 *>(smem + P::OFF_COL);
    const uint32_t bar_base   = smem_u32(smem + P::OFF_BAR);
    auto           full_bar   = [&](int s) { return bar_base + 8u * s; };
    auto           empty_bar  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto           tfull_bar  = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto           tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + ACC + a); };
    uint32_t      *s_tmem     = reinterpret_cast<uint32_t *>(smem + P::OFF_MISC);
    volatile int  *s_abort    = reinterpret_cast<volatile int *>(smem + P::OFF_MISC + 4);
    TapEntry      *s_taps     = reinterpret_cast<TapEntry *>(smem + P::TOTAL);
    const uint32_t bres_bar   = smem_u32(smem + P::OFF_MISC + 8); // RESB: the resident B operand has landed

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int num_m_blocks = (tp.M + UNIT_M - 1) / UNIT_M; // units (MT tiles each) along M
    const int num_n_blocks = (tp.N + BLOCK_N - 1) / BLOCK_N;
    const int num_tiles    = num_m_blocks * num_n_blocks;
    const int num_kb       = (tp.K + KSUB * BLOCK_K - 1) / (KSUB * BLOCK_K);
    const int my_tiles     = static_cast<int>(blockIdx.x) < num_tiles
                                 ? (num_tiles - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1
                                 : 0;

    for (int p = threadIdx.x; p < (tp.K >> 4); p += kConvThreads)
    {
        const int kbyte = p << 4;
        const int tap = kbyte / cg.C, c = kbyte - tap * cg.C;
        const int ky = tap / cg.kw, kx = tap - ky * cg.kw;
        TapEntry  e;
        e.offset  = (ky * cg.dil_y * cg.W + kx * cg.dil_x) * cg.C + c;
        e.dydx    = (static_cast<uint32_t>(ky * cg.dil_y) << 16) | static_cast<uint32_t>(kx * cg.dil_x);
        s_taps[p] = e;
    }
    if (threadIdx.x == 0)
    {
        for (int s = 0; s < STAGES; ++s)
        {
            // B copy (expect_tx arrive; none with a resident B) + one deferred arrival per gather thread
            mbar_init(full_bar(s), (RESB != 0 ? 0 : 1) + 32 * kGatherWarps);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(bres_bar, 1);
        for (int a = 0; a < ACC; ++a)
        {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kEpiWarps / P::EPI_GROUPS); // the warps of the group that drains it
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp)
    {
        tmem_alloc(smem_u32(s_tmem), P::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    griddep_launch_dependents();
    griddep_wait(); // the prologue above touched no global memory

    if (warp < kProdWarps)
    {
        // ---------------------------------------------------------------- TMA producer: weights only
        if (RESB != 0)
        {
            if (warp == 0 && lane == 0)
            {
                // the whole operand once: K sub-blocks of BLOCK_N rows x 128 bytes (zero fill beyond K and N)
                const int n_sub = (tp.K + BLOCK_K - 1) / BLOCK_K;
                mbar_expect_tx(bres_bar, n_sub * P::B_SUB);
                for (int sub = 0; sub < n_sub; ++sub)
                {
                    tma_load_2d(sB + sub * P::B_SUB, &tmap_b, sub * BLOCK_K, 0, bres_bar);
                }
                (void)mbar_wait(bres_bar, 0, s_abort, DEV_TIMEOUT_PRODUCER, tp.spin_limit); // landed before the CTA may leave
            }
        }
        else if (warp == 0 && lane == 0)
        {
            int      st = 0;
            uint32_t ph = 0;
            for (int ti = 0; ti < my_tiles; ++ti)
            {
                const int tile = static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x);
                const int n0   = (tile / num_m_blocks) * BLOCK_N;
                bool      ok   = true;
                for (int kb = 0; kb < num_kb && ok; ++kb)
                {
                    ok = mbar_wait(empty_bar(st), ph ^ 1, s_abort, DEV_TIMEOUT_PRODUCER, tp.spin_limit);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(st), P::B_STAGE);
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub)
                    {
                        tma_load_2d(sB + st * P::B_STAGE + sub * P::B_SUB, &tmap_b, (kb * KSUB + sub) * BLOCK_K, n0,
                                    full_bar(st));
                    }
                    if (++st == STAGES)
                    {
                        st = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
            }
        }
        __syncwarp();
    }
    else if (warp == kMmaWarp)
    {
        // ---------------------------------------------------------------- MMA issuer (as the GEMM kernel)
        if (lane == 0)
        {
            int      s = 0, as = 0;
            uint32_t ph = 0, aph = 0;
            bool     ok = true, have = false;
            const uint64_t a_desc0 = make_kmajor_sw128_desc(sA);
            const uint64_t b_desc0 = make_kmajor_sw128_desc(sB);
            if (RESB != 0)
            {
                ok = mbar_wait(bres_bar, 0, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
            }
            for (int ti = 0; ti < my_tiles && ok; ++ti)
            {
                ok = mbar_wait(tempty_bar(as), aph ^ 1, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                if (MT == 2 && ok)
                {
                    ok = mbar_wait(tempty_bar(as + 1), aph ^ 1, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                }
                if (!ok) break;
                tc_fence_after();
                trace_event(tp.trace, ti, 1);
                const uint32_t d_tmem = tmem_base + as * BLOCK_N; // (MT == 2: tile 1 of the unit in the next buffer)
                for (int kb = 0; kb < num_kb; ++kb)
                {
                    if (!have)
                    {
                        ok = mbar_wait(full_bar(s), ph, s_abort, DEV_TIMEOUT_MMA, tp.spin_limit);
                        if (!ok) break;
                    }
                    if (kb == 0) trace_event(tp.trace, ti, 2);
                    int      sn  = s + 1;
                    uint32_t phn = ph;
                    if (sn == STAGES)
                    {
                        sn = 0;
                        phn ^= 1;
                    }
                    have = mbar_test_wait(full_bar(sn), phn);
                    tc_fence_after();
                    // the A rows were written by cp.async (generic proxy); the MMA reads through the async proxy
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * P::A_STAGE_K) >> 4);
                    // the ring slot, or this stage's K sub-blocks of the resident operand
                    const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(((RESB != 0 ? kb : s) * KSUB * P::B_SUB) >> 4);
                    // a stage that lies wholly inside K: the MMAs back to back, nothing to test on the issuing thread's
                    // path (it shares its scheduler with epilogue and gather warps, so every instruction it saves counts)
                    if ((kb + 1) * KSUB * BLOCK_K <= tp.K)
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) // the two tiles alternate: independent accumulators
                                {
                                    umma_i8(d_tmem + mt * BLOCK_N,
                                            a_desc + static_cast<uint64_t>(((mt * KSUB + sub) * A_STAGE) >> 4) + 2u * k,
                                            b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, tp.idesc,
                                            (kb | sub | k) != 0 ? 1u : 0u);
                                }
                            }
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int sub = 0; sub < KSUB; ++sub)
                        {
#pragma unroll
                            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                            {
                                // a K step that lies wholly beyond K multiplies zero fill: left out (short K)
                                if ((kb * KSUB + sub) * BLOCK_K + k * UMMA_K < tp.K)
                                {
#pragma unroll
                                    for (int mt = 0; mt < MT; ++mt)
                                    {
                                        umma_i8(d_tmem + mt * BLOCK_N,
                                                a_desc + static_cast<uint64_t>(((mt * KSUB + sub) * A_STAGE) >> 4) + 2u * k,
                                                b_desc + static_cast<uint64_t>((sub * P::B_SUB) >> 4) + 2u * k, tp.idesc,
                                                (kb | sub | k) != 0 ? 1u : 0u);
                                    }
                                }
                            }
                        }
                    }
                    umma_commit(empty_bar(s));
                    s  = sn;
                    ph = phn;
                }
                if (ok)
                {
                    trace_event(tp.trace, ti, 3);
                    umma_commit(tfull_bar(as));
                }
                as += MT; // one accumulator-ready signal per unit: on the barrier of its first buffer
                if (as == ACC)
                {
                    as = 0;
                    aph ^= 1;
                }
            }
        }
        __syncwarp();
    }
    else if (warp < kFirstGather)
    {
        // ---------------------------------------------------------------- epilogue (groups as in the GEMM kernel)
        constexpr int kGroups = P::EPI_GROUPS;
        const int     group   = kGroups == 1 ? 0 : (warp - kFirstEpi) >> 2;
        const int     et      = threadIdx.x - 32 * kFirstEpi - group * 128;
        int4         *g_col   = s_col + group * BLOCK_N;
        bool          ok      = true;
        int           filled_n0 = -1;
        for (int ti = 0; ti < my_tiles; ++ti)
        {
            if (MT == 1 && kGroups > 1 && (ti & 1) != group)
            {
                continue; // (MT == 2: every group works on every unit, group g on its tile g)
            }
            if (!(kGroups == 1 ? epi_barrier_and(ok) : epi_group_barrier_and(ok, group)))
            {
                break;
            }
            // buffer of this group's tile, and the buffer whose barrier announces the unit's accumulators
            const int      as_first = MT == 1 ? ti % ACC : MT * (ti % (ACC / MT));
            const int      as       = MT == 1 ? as_first : as_first + group;
            const uint32_t aph  = static_cast<uint32_t>(ti / (ACC / MT)) & 1u;
            const int      tile = static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x);
            const int      m0   = (tile % num_m_blocks) * UNIT_M + (MT == 1 ? 0 : group * BLOCK_M);
            const int      n0   = (tile / num_m_blocks) * BLOCK_N;
            if (n0 != filled_n0) // tiles are ordered m-fastest: the column terms usually carry over
            {
                fill_column_terms<BLOCK_N>(g_col, et, n0, tp, ep, kEpiThreads / kGroups);
                filled_n0 = n0;
                if (kGroups == 1) epi_barrier();
                else epi_group_barrier(group);
            }
            ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(as_first), aph, s_abort, DEV_TIMEOUT_EPILOGUE, tp.spin_limit));
            if (ok)
            {
                tc_fence_after();
                if (et == 0) trace_event(tp.trace, ti, 4);
                const AccRelease rel{tempty_bar(as), 0u, false};
                epilogue_warp_tile<BLOCK_N, false, kGroups>(tmem_base + as * BLOCK_N, g_col, tp, ep, warp, lane, m0, n0,
                                                            smem + P::OFF_OUT, rel, tp.tma_store != 0 ? &tmap_out : nullptr);
                if (et == 0) trace_event(tp.trace, ti, 5);
                __syncwarp();
            }
        }
        if (tp.tma_store != 0 && lane == 0)
        {
            tma_store_wait_all(); // this warp's bulk stores: shared memory stays valid until they have read it
        }
    }
    else
    {
        // ---------------------------------------------------------------- A gather
        // Thread layout: 8 consecutive threads copy the eight 16-byte pieces of one 128-byte tile row (coalesced
        // 64..128-byte runs of the input), 32 rows per pass, kRowsPerThread passes per K sub-block.
        constexpr int kRowsPerThread = BLOCK_M / (kGatherWarps * 4); // 128 rows / (threads / 8)
        const int     gt             = threadIdx.x - 32 * kFirstGather;
        const int     piece          = gt & 7;
        const int     row0           = gt >> 3;
        const uint8_t *pad_src       = cg.pad + 16 * gt; // every thread its own copy: no single hot line
        const int      last_piece    = (tp.K >> 4) - 1;
        int           st = 0;
        uint32_t      ph = 0;
        bool          ok = true;
        for (int ti = 0; ti < my_tiles && ok; ++ti)
        {
            const int tile = static_cast<int>(blockIdx.x) + ti * static_cast<int>(gridDim.x);
            const int m0   = (tile % num_m_blocks) * UNIT_M;
            int            yi0[MT * kRowsPerThread], xi0[MT * kRowsPerThread];
            const uint8_t *base[MT * kRowsPerThread];
#pragma unroll
            for (int i = 0; i < MT * kRowsPerThread; ++i)
            {
                // rows beyond M repeat the last pixel (never stored); i / kRowsPerThread is the tile of the unit
                const int m  = min(m0 + (i / kRowsPerThread) * BLOCK_M + row0 + 32 * (i % kRowsPerThread), tp.M - 1);
                const int q  = fast_div(m, cg.div_wo), xo = m - q * cg.Wo;
                const int bi = fast_div(q, cg.div_ho), yo = q - bi * cg.Ho;
                yi0[i]       = yo * cg.sy - cg.pad_t;
                xi0[i]       = xo * cg.sx - cg.pad_l;
                // address of tap (0, 0), channel 0 of this pixel; outside the tensor for border pixels, where it is
                // only ever used after the bounds test below
                base[i] = cg.src + (static_cast<long long>(bi) * cg.H * cg.W + static_cast<long long>(yi0[i]) * cg.W + xi0[i]) * cg.C;
            }
            for (int kb = 0; kb < num_kb; ++kb)
            {
                if (lane == 0)
                {
                    ok = mbar_wait(empty_bar(st), ph ^ 1, s_abort, DEV_TIMEOUT_PRODUCER, tp.spin_limit);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (kb == 0 && gt == 0) trace_event(tp.trace, ti, 0);
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                {
                    // beyond K the weights are zero (TMA fill), so whatever bytes the stage still holds there
                    // multiply to nothing: no copy
                    if ((kb * KSUB + sub) * 8 + piece > last_piece)
                    {
                        continue;
                    }
                    const TapEntry e  = s_taps[(kb * KSUB + sub) * 8 + piece];
                    const int      dy = static_cast<int>(e.dydx >> 16), dx = static_cast<int>(e.dydx & 0xffffu);
#pragma unroll
                    for (int i = 0; i < MT * kRowsPerThread; ++i)
                    {
                        const bool     in  = static_cast<unsigned>(yi0[i] + dy) < static_cast<unsigned>(cg.H) &&
                                        static_cast<unsigned>(xi0[i] + dx) < static_cast<unsigned>(cg.W);
                        const uint8_t *src = in ? base[i] + e.offset : pad_src;
                        const int      r   = row0 + 32 * (i % kRowsPerThread);
                        const uint32_t dst = sA + st * P::A_STAGE_K + ((i / kRowsPerThread) * KSUB + sub) * A_STAGE + r * 128 +
                                             ((piece ^ (r & 7)) << 4);
                        // .cg: through L2 only -- measured 5 to 20 % faster than .ca on every layer shape (an L1 miss
                        // of .ca lands in shared memory sector by sector)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                    }
                }
                // this thread's arrival on the stage's barrier happens when its copies above have landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(st)) : "memory");
                if (kb == num_kb - 1 && gt == 0) trace_event(tp.trace, ti, 7);
                if (++st == STAGES)
                {
                    st = 0;
                    ph ^= 1;
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory"); // nothing of this thread's is in flight when the CTA leaves
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp)
    {
        tc_fence_after();
        tmem_dealloc(tmem_base, P::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *s_abort != 0)
    {
        atomicCAS(tp.status, 0, *s_abort);
    }
}

#endif // CUGL_TC_FULL_BUILD

// encoding of the output stage for this launch (see requant_pack4)
// two accumulator buffers of one column block drained together (drain_accumulator_pair): short K, one destination,
// the wide / pack encodings of the output stage
inline bool wants_pair_drain(const GemmOperands &op)
{
    return op.pair_drain >= 0 && op.K <= 512 && op.n_extra_dst == 0 && op.wide_stage && !op.generic_stage;
}

int stage_mode(const GemmOperands &op, const EpilogueParams &ep)
{
    if (op.generic_stage)
    {
        return kStageGeneric;
    }
    if (!op.wide_stage)
    {
        return kStageFast;
    }
    const int32_t tlo = ep.out_signed != 0 ? -128 : 0, thi = ep.out_signed != 0 ? 127 : 255;
    const bool    whole_range = ep.lo == tlo && ep.hi == thi;
    if (op.pack_stage >= 0 && whole_range && (ep.result_offset == 0 || op.max_shift <= 22))
    {
        return ep.out_signed != 0 ? kStagePackS : kStagePack;
    }
    return kStageWide;
}

void fill_conv_params(TileParams &tp, const GemmOperands &op)
{
    tp.conv_c = 0;
    if (op.conv != nullptr)
    {
        const ConvOperands &cv = *op.conv;
        tp.conv_c = cv.C, tp.conv_kw = cv.kw, tp.conv_wo = cv.Wo, tp.conv_ho = cv.Ho, tp.conv_sx = cv.sx, tp.conv_sy = cv.sy;
        tp.conv_pl = cv.pad_l, tp.conv_pt = cv.pad_t, tp.conv_dx = cv.dil_x, tp.conv_dy = cv.dil_y;
        tp.conv_div_wo = make_fastdiv(cv.Wo), tp.conv_div_ho = make_fastdiv(cv.Ho);
    }
}

void fill_extra_dst(TileParams &tp, const GemmOperands &op)
{
    tp.residual   = static_cast<const uint8_t *>(op.residual);
    tp.res_floor4 = static_cast<uint32_t>(op.res_floor & 0xff) * 0x01010101u;
    tp.res_cap4   = static_cast<uint32_t>(op.res_cap & 0xff) * 0x01010101u;
    tp.n_extra    = op.n_extra_dst;
    // paired drain: where the tile's time is its epilogue (K = 64: 227 -> 173 us, 128: 120 -> 96, 256: 67 -> 61,
    // 512: 43 -> 43); with a longer main loop the MMA of the next tile should overlap the drain instead
    tp.pair_drain = wants_pair_drain(op) ? 1 : 0;
    for (int i = 0; i < kMaxExtraDst; ++i)
    {
        tp.extra_dst[i] = i < op.n_extra_dst ? static_cast<uint8_t *>(op.extra_dst[i]) : nullptr;
    }
}

// TileParams::vec_ok of a row-major output: 0 = byte stores; bit 0 = every row piece is 16-byte aligned; bit 1 = 32-byte
// aligned as well (one 256-bit access per 32 output bytes, i.e. a whole DRAM sector per lane)
int vector_flags(uint64_t address_bits)
{
    return (address_bits & 15) != 0 ? 0 : ((address_bits & 31) != 0 ? 1 : 3);
}

uint64_t extra_dst_bits(const GemmOperands &op)
{
    uint64_t bits = reinterpret_cast<uintptr_t>(op.residual);
    for (int i = 0; i < op.n_extra_dst; ++i)
    {
        bits |= reinterpret_cast<uintptr_t>(op.extra_dst[i]);
    }
    return bits;
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

// Output through bulk tensor stores from the warps' staging areas (drain_accumulator): the eight- and four-warp builds,
// one 8-bit destination, 16-byte aligned base and pitch.  Box = 32 rows x kOutRowBytes in the swizzle the staging
// uses.  *use says whether the launch may use the map; false is returned only when the encoding itself failed.
bool encode_out_map(const GemmOperands &op, CUtensorMap *map, bool *use, int row_bytes = kOutRowBytes,
                    bool any_build = false)
{
    *use = (kEpiWarps <= 8 || any_build) && op.tma_store >= 0 && op.n_extra_dst == 0 &&
           ((reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd)) & 15) == 0;
    if (!*use)
    {
        return true;
    }
    EncodeTiledFn    fn         = get_encode_fn();
    const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(op.N), static_cast<cuuint64_t>(op.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(op.ldd)};
    const cuuint32_t box[2]     = {static_cast<cuuint32_t>(row_bytes), 32};
    const cuuint32_t estr[2]    = {1, 1};
    return fn != nullptr &&
           fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, op.dst, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                               : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B),
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

using EncodeIm2colFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeIm2colFn get_encode_im2col_fn()
{
    static EncodeIm2colFn fn = []() -> EncodeIm2colFn {
        void                           *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
        {
            (void)cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeIm2colFn>(p);
    }();
    return fn;
}

// Im2col-mode map of an NHWC byte tensor: a load delivers BLOCK_M window origins x 128 channels (128-byte swizzle, the
// K-major tile the tensor cores read).  The bounding box of the origins runs from -pad to the origin of the last output
// pixel in each dimension, the traversal stride is the convolution stride; taps outside the image read as zero.
bool encode_im2col_map(CUtensorMap *map, const ConvOperands &cv)
{
    EncodeIm2colFn fn = get_encode_im2col_fn();
    if (fn == nullptr)
    {
        return false;
    }
    const cuuint64_t dims[4]    = {static_cast<cuuint64_t>(cv.C), static_cast<cuuint64_t>(cv.W), static_cast<cuuint64_t>(cv.H),
                                   static_cast<cuuint64_t>(cv.B)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(cv.C), static_cast<cuuint64_t>(cv.C) * cv.W,
                                   static_cast<cuuint64_t>(cv.C) * cv.W * cv.H};
    const int        lower[2]   = {-cv.pad_l, -cv.pad_t};
    const int        upper[2]   = {(cv.Wo - 1) * cv.sx - cv.pad_l - (cv.W - 1), (cv.Ho - 1) * cv.sy - cv.pad_t - (cv.H - 1)};
    const cuuint32_t estr[4]    = {1, static_cast<cuuint32_t>(cv.sx), static_cast<cuuint32_t>(cv.sy), 1};
    const bool       narrow     = cv.C == 64; // one tap = 64 bytes: 64-byte rows in the 64-byte swizzle
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(cv.src), dims, strides, lower, upper,
              static_cast<cuuint32_t>(narrow ? 64 : BLOCK_K), static_cast<cuuint32_t>(BLOCK_M), estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, narrow ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// what the im2col-mode route needs besides the GEMM conditions
bool conv_tma_supported(const GemmOperands &op)
{
    const ConvOperands &cv = *op.conv;
    const int           up_w = (cv.Wo - 1) * cv.sx - cv.pad_l - (cv.W - 1), up_h = (cv.Ho - 1) * cv.sy - cv.pad_t - (cv.H - 1);
    auto                corner_ok = [](int v) { return v >= -128 && v <= 127; };
    return ((cv.C % BLOCK_K) == 0 || cv.C == 64) && (reinterpret_cast<uintptr_t>(cv.src) & 15) == 0 && cv.sx >= 1 && cv.sx <= 8 &&
           cv.sy >= 1 && cv.sy <= 8 && corner_ok(-cv.pad_l) && corner_ok(-cv.pad_t) && corner_ok(up_w) && corner_ok(up_h) &&
           (cv.kw - 1) * cv.dil_x < 256 && (cv.kh - 1) * cv.dil_y < 256 && get_encode_im2col_fn() != nullptr;
}

// Programmatic stream serialization pays where launches are issued one by one (QASYMM8 ResNet-50, batch 256, layer
// by layer: 2.74 -> 2.67 ms); inside a captured graph, whose launches are packed already, the programmatic edges
// measured 1 % slower (2.594 -> 2.618 ms), so a capturing stream gets plain launches.
inline bool use_dependent_launch(const cugl_context *ctx)
{
    if (ctx->dependent_launch == 0)
    {
        return false;
    }
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &st) != cudaSuccess)
    {
        (void)cudaGetLastError();
        return false;
    }
    return st == cudaStreamCaptureStatusNone;
}

// Launch with programmatic stream serialization (see griddep_wait): the kernel may start its prologue while the
// previous kernel of the stream is finishing.  ctx->dependent_launch == 0 or a capturing stream: a plain launch.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(cugl_context *ctx, void (*kernel)(KArgs...), int grid, int threads, int smem_bytes, Args &&...args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim         = dim3(static_cast<unsigned>(threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cfg.stream           = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs    = attr;
    cfg.numAttrs = use_dependent_launch(ctx) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <int BLOCK_N, int STAGES, int KSUB, bool kS32Out, bool kPairTma = false>
cugl_status launch_variant(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    constexpr int ACC = BLOCK_N <= 128 ? 4 : 2; // narrow tiles: four accumulator buffers in the 512 columns
    using P = SmemPlan<BLOCK_N, STAGES, KSUB, ACC, kPairTma>;
    static_assert(P::DYN_BYTES <= 227 * 1024, "shared memory plan exceeds the sm_100 limit");
    CUtensorMap map_a, map_b;
    if (!(op.conv != nullptr ? encode_im2col_map(&map_a, *op.conv)
                             : encode_operand_map(&map_a, op.a, op.M, op.K, op.lda, BLOCK_M)) ||
        !encode_operand_map(&map_b, op.bt, op.N, op.K, op.ldbt, BLOCK_N))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncode failed for a GEMM operand");
    }
    CUtensorMap map_out   = map_a; // placeholder when unused
    bool        tma_store = false;
    if (!kS32Out && !(kPairTma ? encode_out_map(op, &map_out, &tma_store, 64, true) : encode_out_map(op, &map_out, &tma_store)))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for the output tiles");
    }
    CUtensorMap map_res = map_out; // the same geometry over the residual matrix (paired drain through the TMA unit)
    if (kPairTma && tma_store && op.residual != nullptr)
    {
        GemmOperands r = op;
        r.dst          = const_cast<void *>(op.residual);
        bool use       = false;
        if ((reinterpret_cast<uintptr_t>(op.residual) & 15) != 0 || !encode_out_map(r, &map_res, &use, 64, true) || !use)
        {
            return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for the residual tiles");
        }
    }
    auto kernel = gemmlowp_tcgen05_kernel<BLOCK_N, STAGES, KSUB, kS32Out, false, ACC, kPairTma>;
    static bool attr_set[64] = {}; // per instantiation and device
    if (!attr_set[ctx->device & 63])
    {
        CUGL_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::DYN_BYTES));
        attr_set[ctx->device & 63] = true;
    }
    TileParams tp;
    tp.dst    = static_cast<uint8_t *>(op.dst);
    tp.ldd    = op.ldd;
    fill_extra_dst(tp, op);
    tp.M      = op.M;
    tp.N      = op.N;
    tp.K      = op.K;
    tp.idesc  = (2u << 4) | ((op.a_signed ? 1u : 0u) << 7) | ((op.b_signed ? 1u : 0u) << 10) |
               (static_cast<uint32_t>(BLOCK_N >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
    tp.vec_ok = vector_flags(reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd) | extra_dst_bits(op));
    tp.status  = ctx->d_status;
    tp.tma_store = 0;
    fill_conv_params(tp, op);
    tp.spin_limit  = ctx->spin_limit;
    tp.withhold_kb = ctx->withhold_kb;
    ctx->withhold_kb = -1;
    tp.mode    = stage_mode(op, ep);
    tp.trace   = ctx->d_trace;
    tp.raw_f32 = ep.out_f32, tp.raw_accumulate = ep.accumulate, tp.raw_scale = ep.dq_scale;
    tp.idesc_half = 0;
    tp.split_tail = 0;
    const int tiles = ((op.M + BLOCK_M - 1) / BLOCK_M) * ((op.N + BLOCK_N - 1) / BLOCK_N);
    const int grid  = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    tp.tma_store = tma_store ? 1 : 0;
    CUGL_CUDA_TRY(ctx, launch_dependent(ctx, kernel, grid, kThreads, P::DYN_BYTES, map_a, map_b, map_out, map_res, tp, ep));
    return check_cuda(ctx, cudaGetLastError(), "gemmlowp_tcgen05_kernel");
}

// Channel-major launch: weights on the 128-row side of the tile, BLOCK_N rows of the activation matrix on the other.
template <int BLOCK_N, int STAGES, int KSUB, bool kS32Out>
cugl_status launch_variant_cm(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    using P = SmemPlan<BLOCK_N, STAGES, KSUB>;
    static_assert(P::DYN_BYTES <= 227 * 1024, "shared memory plan exceeds the sm_100 limit");
    CUtensorMap map_w, map_x;
    if (!encode_operand_map(&map_w, op.bt, op.N, op.K, op.ldbt, BLOCK_M) ||
        !encode_operand_map(&map_x, op.a, op.M, op.K, op.lda, BLOCK_N))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for a GEMM operand");
    }
    auto kernel = gemmlowp_tcgen05_kernel<BLOCK_N, STAGES, KSUB, kS32Out, true, 2>;
    static bool attr_set[64] = {}; // per instantiation and device
    if (!attr_set[ctx->device & 63])
    {
        CUGL_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::DYN_BYTES));
        attr_set[ctx->device & 63] = true;
    }
    TileParams tp;
    tp.dst    = static_cast<uint8_t *>(op.dst);
    tp.ldd    = op.ldd;
    fill_extra_dst(tp, op);
    tp.M      = op.N; // tensor-memory lanes: output channels
    tp.N      = op.M; // tensor-memory columns: output rows
    tp.K      = op.K;
    tp.idesc  = (2u << 4) | ((op.b_signed ? 1u : 0u) << 7) | ((op.a_signed ? 1u : 0u) << 10) |
               (static_cast<uint32_t>(BLOCK_N >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
    tp.vec_ok  = ((reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd) | extra_dst_bits(op)) & 7) == 0;
    tp.status  = ctx->d_status;
    tp.tma_store = 0;
    tp.conv_c  = 0;
    tp.spin_limit  = ctx->spin_limit;
    tp.withhold_kb = ctx->withhold_kb;
    ctx->withhold_kb = -1;
    tp.mode    = stage_mode(op, ep);
    tp.trace   = ctx->d_trace;
    tp.raw_f32 = ep.out_f32, tp.raw_accumulate = ep.accumulate, tp.raw_scale = ep.dq_scale;
    tp.idesc_half = 0;
    tp.split_tail = 0;
    const int tiles = ((op.N + BLOCK_M - 1) / BLOCK_M) * ((op.M + BLOCK_N - 1) / BLOCK_N);
    const int grid  = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    CUGL_CUDA_TRY(ctx, launch_dependent(ctx, kernel, grid, kThreads, P::DYN_BYTES, map_w, map_x, map_w, map_w, tp, ep)); // (no bulk stores on this path)
    return check_cuda(ctx, cudaGetLastError(), "gemmlowp_tcgen05_kernel (channel-major)");
}

#if CUGL_TC_FULL_BUILD
template <int STAGES, int KSUB, bool kS32Out>
cugl_status launch_variant_2cta(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep)
{
    using P = SmemPlan2<STAGES, KSUB>;
    static_assert(P::DYN_BYTES <= 227 * 1024, "shared memory plan exceeds the sm_100 limit");
    CUtensorMap map_a, map_b, map_bh;
    if (!(op.conv != nullptr ? encode_im2col_map(&map_a, *op.conv)
                             : encode_operand_map(&map_a, op.a, op.M, op.K, op.lda, BLOCK_M)) ||
        !encode_operand_map(&map_b, op.bt, op.N, op.K, op.ldbt, P::BLOCK_N / 2) ||
        !encode_operand_map(&map_bh, op.bt, op.N, op.K, op.ldbt, P::BLOCK_N / 4))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for a GEMM operand");
    }
    CUtensorMap map_out   = map_a; // placeholder when unused
    bool        tma_store = false;
    if (!kS32Out && !encode_out_map(op, &map_out, &tma_store))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for the output tiles");
    }
    auto kernel = gemmlowp_tcgen05_2cta_kernel<STAGES, KSUB, kS32Out>;
    static bool attr_set[64] = {}; // per instantiation and device
    if (!attr_set[ctx->device & 63])
    {
        CUGL_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::DYN_BYTES));
        attr_set[ctx->device & 63] = true;
    }
    TileParams tp;
    tp.dst    = static_cast<uint8_t *>(op.dst);
    tp.ldd    = op.ldd;
    fill_extra_dst(tp, op);
    tp.M      = op.M;
    tp.N      = op.N;
    tp.K      = op.K;
    tp.idesc  = (2u << 4) | ((op.a_signed ? 1u : 0u) << 7) | ((op.b_signed ? 1u : 0u) << 10) |
               (static_cast<uint32_t>(P::BLOCK_N >> 3) << 17) | (static_cast<uint32_t>((2 * BLOCK_M) >> 4) << 24);
    tp.idesc_half = (tp.idesc & ~(0x3fu << 17)) | (static_cast<uint32_t>((P::BLOCK_N / 2) >> 3) << 17);
    tp.split_tail = op.split_tail >= 0 ? 1 : 0;
    tp.vec_ok = vector_flags(reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd) | extra_dst_bits(op));
    tp.status  = ctx->d_status;
    tp.tma_store = 0;
    fill_conv_params(tp, op);
    tp.spin_limit  = ctx->spin_limit;
    tp.withhold_kb = ctx->withhold_kb;
    ctx->withhold_kb = -1;
    tp.mode    = stage_mode(op, ep);
    tp.trace   = ctx->d_trace;
    tp.raw_f32 = ep.out_f32, tp.raw_accumulate = ep.accumulate, tp.raw_scale = ep.dq_scale;
    const int tiles    = ((op.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((op.N + P::BLOCK_N - 1) / P::BLOCK_N);
    const int pairs    = ctx->sm_count / 2;
    const int clusters = tiles < pairs ? tiles : pairs;

    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(2 * clusters, 1, 1);
    cfg.blockDim         = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = P::DYN_BYTES;
    cfg.stream           = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id               = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = use_dependent_launch(ctx) ? 2 : 1;
    tp.tma_store = tma_store ? 1 : 0;
    CUGL_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_bh, map_out, tp, ep));
    return CUGL_SUCCESS;
}

template <int BLOCK_N, int STAGES, int KSUB, int ACC, int RESB = 0, int MT = 1>
cugl_status launch_conv_variant(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                const ConvOperands &cv)
{
    using P = SmemPlan<BLOCK_N, STAGES, MT * KSUB, ACC, false, RESB>;
    // the tap table: one entry per 16 bytes of K; with a resident B operand K is at most RESB / BLOCK_N bytes
    constexpr int kTapEntries = RESB != 0 ? RESB / BLOCK_N / 16 : kConvMaxPieces;
    constexpr int kDynBytes   = P::DYN_BYTES + kTapEntries * static_cast<int>(sizeof(TapEntry));
    static_assert(kDynBytes <= 227 * 1024, "shared memory plan exceeds the sm_100 limit");
    static_assert(P::TOTAL % 8 == 0, "the tap table follows the plan");
    CUtensorMap map_b;
    if (!encode_operand_map(&map_b, op.bt, op.N, op.K, op.ldbt, BLOCK_N))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for the weights operand");
    }
    CUtensorMap map_out   = map_b; // placeholder when unused
    bool        tma_store = false;
    if (!encode_out_map(op, &map_out, &tma_store))
    {
        return fail(ctx, CUGL_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed for the output tiles");
    }
    auto        kernel = gemmlowp_conv_tcgen05_kernel<BLOCK_N, STAGES, KSUB, ACC, RESB, MT>;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device & 63])
    {
        CUGL_CUDA_TRY(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynBytes));
        attr_set[ctx->device & 63] = true;
    }
    TileParams tp;
    tp.dst    = static_cast<uint8_t *>(op.dst);
    tp.ldd    = op.ldd;
    fill_extra_dst(tp, op);
    tp.M      = op.M;
    tp.N      = op.N;
    tp.K      = op.K;
    tp.idesc  = (2u << 4) | ((op.a_signed ? 1u : 0u) << 7) | ((op.b_signed ? 1u : 0u) << 10) |
               (static_cast<uint32_t>(BLOCK_N >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
    tp.vec_ok = vector_flags(reinterpret_cast<uintptr_t>(op.dst) | static_cast<uint64_t>(op.ldd) | extra_dst_bits(op));
    tp.status  = ctx->d_status;
    tp.tma_store = 0;
    tp.conv_c  = 0;
    tp.spin_limit  = ctx->spin_limit;
    tp.withhold_kb = ctx->withhold_kb;
    ctx->withhold_kb = -1;
    tp.mode    = stage_mode(op, ep);
    tp.trace   = ctx->d_trace;
    tp.raw_f32 = ep.out_f32, tp.raw_accumulate = ep.accumulate, tp.raw_scale = ep.dq_scale;
    tp.idesc_half = 0;
    tp.split_tail = 0;
    ConvGeom cg;
    cg.src   = static_cast<const uint8_t *>(cv.src);
    cg.pad   = static_cast<const uint8_t *>(cv.pad);
    cg.C     = cv.C;
    cg.W     = cv.W;
    cg.H     = cv.H;
    cg.kw    = cv.kw;
    cg.kh    = cv.kh;
    cg.sx    = cv.sx;
    cg.sy    = cv.sy;
    cg.pad_l = cv.pad_l;
    cg.pad_t = cv.pad_t;
    cg.dil_x = cv.dil_x;
    cg.dil_y = cv.dil_y;
    cg.Wo    = cv.Wo;
    cg.Ho    = cv.Ho;
    cg.div_wo = make_fastdiv(cv.Wo);
    cg.div_ho = make_fastdiv(cv.Ho);
    const int tiles = ((op.M + MT * BLOCK_M - 1) / (MT * BLOCK_M)) * ((op.N + BLOCK_N - 1) / BLOCK_N); // units of MT tiles
    const int grid  = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    tp.tma_store = tma_store ? 1 : 0;
    CUGL_CUDA_TRY(ctx, launch_dependent(ctx, kernel, grid, kConvThreads, kDynBytes, map_b, map_out, tp, ep, cg));
    return check_cuda(ctx, cudaGetLastError(), "gemmlowp_conv_tcgen05_kernel");
}
#endif // CUGL_TC_FULL_BUILD
} // namespace

bool CUGL_TC_NAME(gemmlowp_tcgen05_supported)(const GemmOperands &op)
{
    if (op.M <= 0 || op.N <= 0 || op.K <= 0)
    {
        return false;
    }
    const uint64_t bits = reinterpret_cast<uintptr_t>(op.a) | reinterpret_cast<uintptr_t>(op.bt) |
                          static_cast<uint64_t>(op.lda) | static_cast<uint64_t>(op.ldbt);
    return (bits & 15) == 0 && get_encode_fn() != nullptr;
}

// implicit convolution through im2col-mode loads (op.conv set): the weights as for the GEMM, the input tensor as above
bool CUGL_TC_NAME(gemmlowp_conv_tma_supported)(const GemmOperands &op)
{
    if (op.conv == nullptr || op.M <= 0 || op.N <= 0 || op.K <= 0 || (op.K % (op.conv->C == 64 ? 64 : BLOCK_K)) != 0)
    {
        return false;
    }
    const uint64_t bits = reinterpret_cast<uintptr_t>(op.bt) | static_cast<uint64_t>(op.ldbt);
    return (bits & 15) == 0 && get_encode_fn() != nullptr && conv_tma_supported(op);
}

// The SM-pair kernel pays off once a tile spans both halves: more than 128 rows and more than 128 columns.
bool CUGL_TC_NAME(gemmlowp_tcgen05_uses_pair)(const GemmOperands &op)
{
    return op.N > 128 && op.M > 128;
}

cugl_status CUGL_TC_NAME(launch_gemmlowp_tcgen05)(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                    bool allow_pair)
{
    const bool s32 = ep.stage == CUGL_STAGE_NONE;
    // channel-major accumulators: no row-sum term (it would be a per-column quantity there) and one destination
    if (op.channel_major > 0 && ep.rowsum == nullptr && op.n_extra_dst == 0 && op.conv == nullptr)
    {
        return s32 ? launch_variant_cm<256, 4, 1, true>(ctx, op, ep) : launch_variant_cm<256, 4, 1, false>(ctx, op, ep);
    }
#if CUGL_TC_FULL_BUILD
    if (allow_pair && CUGL_TC_NAME(gemmlowp_tcgen05_uses_pair)(op) && !(op.conv != nullptr && op.conv->C == 64)) // (64-byte-swizzle tiles: one-CTA kernels)
    {
        return s32 ? launch_variant_2cta<3, 2, true>(ctx, op, ep) : launch_variant_2cta<3, 2, false>(ctx, op, ep);
    }
#else
    (void)allow_pair;
#endif
    const int block_n = op.block_n > 0 ? op.block_n : (op.N > 128 ? 256 : (op.N > 64 ? 128 : 64));
#if !CUGL_TC_FULL_BUILD
    // sixteen epilogue warps with a paired drain: a ring of three stages leaves room for the staging areas of its
    // bulk tensor stores
    if (!s32 && wants_pair_drain(op) && op.tma_store >= 0 && op.n_extra_dst == 0 && (op.N & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(op.dst) | reinterpret_cast<uintptr_t>(op.residual) | static_cast<uint64_t>(op.ldd)) & 15) == 0)
    {
        return launch_variant<256, 3, 1, false, true>(ctx, op, ep);
    }
#endif
    if (block_n > 128 || !CUGL_TC_FULL_BUILD)
    {
        return s32 ? launch_variant<256, 4, 1, true>(ctx, op, ep) : launch_variant<256, 4, 1, false>(ctx, op, ep);
    }
#if CUGL_TC_FULL_BUILD
    // K of at most one 128-byte block: a tile is a single stage, so one-block stages and a ring twice as deep keep
    // twice as many tiles' operands in flight (the loads of such layers are bound by latency, not by bandwidth)
    const bool one_block = op.K <= BLOCK_K && !s32;
    if (block_n > 64)
    {
        if (one_block) return launch_variant<128, 6, 1, false>(ctx, op, ep);
        return s32 ? launch_variant<128, 3, 2, true>(ctx, op, ep) : launch_variant<128, 3, 2, false>(ctx, op, ep);
    }
    if (one_block) return launch_variant<64, 8, 1, false>(ctx, op, ep);
    return s32 ? launch_variant<64, 4, 2, true>(ctx, op, ep) : launch_variant<64, 4, 2, false>(ctx, op, ep);
#endif
}
} // namespace cugl

#if CUGL_TC_FULL_BUILD
namespace cugl
{
bool CUGL_TC_NAME(gemmlowp_conv_tcgen05_supported)(const GemmOperands &op, const ConvOperands &cv)
{
    const uint64_t bits = reinterpret_cast<uintptr_t>(cv.src) | reinterpret_cast<uintptr_t>(cv.pad) |
                          reinterpret_cast<uintptr_t>(op.bt) | static_cast<uint64_t>(op.ldbt);
    // the tap table holds K / 16 entries with 32-bit offsets inside one image and 16-bit tap displacements
    const long long image_bytes = static_cast<long long>(cv.H) * cv.W * cv.C;
    return op.M > 0 && op.N > 0 && op.K >= 16 && op.K <= 16 * kConvMaxPieces && (bits & 15) == 0 && (cv.C % 16) == 0 &&
           cv.pad != nullptr && image_bytes < (1ll << 31) && cv.kh * cv.dil_y < 65536 && cv.kw * cv.dil_x < 65536 &&
           get_encode_fn() != nullptr;
}

cugl_status CUGL_TC_NAME(launch_gemmlowp_conv_tcgen05)(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                         const ConvOperands &cv)
{
    if (ep.stage == CUGL_STAGE_NONE)
    {
        return fail(ctx, CUGL_UNSUPPORTED_CONFIG, "implicit convolution needs a quantize-down output stage");
    }
    const int block_n = op.block_n > 0 ? op.block_n : (op.N > 128 ? 256 : (op.N > 64 ? 128 : 64));
    if (block_n > 128)
    {
        return launch_conv_variant<256, 4, 1, 2>(ctx, op, ep, cv);
    }
    if (block_n > 64)
    {
        return launch_conv_variant<128, 3, 2, 4>(ctx, op, ep, cv);
    }
    // narrow tiles: four accumulator buffers keep more tiles in flight (56x56x64 -> 64, batch 256: 131 -> 115 us;
    // eight one-block stages instead of four two-block stages measured slower: 129 us)
    constexpr int kResidentB = 40 * 1024; // K <= 640: the weights of a 3x3 x 64 or a folded 7x7 x 3 filter bank
    if (op.resident_b >= 0 && op.N <= 64 && ((op.K + BLOCK_K - 1) / BLOCK_K) * 64 * BLOCK_K <= kResidentB)
    {
        if constexpr (kEpiWarps == 8) // (two epilogue groups: one per tile of a unit)
        {
            // enough output for a 256-row unit on every SM, and more than two K blocks per tile (802816 x 64 x 576:
            // 93.6 -> 87.4 us; with K = 256, two hand-overs per tile either way, the folded stem measured slower: 231 -> 246)
            if (op.double_tile >= 0 && op.M > 2 * BLOCK_M * ctx->sm_count && op.K > 2 * BLOCK_K)
            {
                return launch_conv_variant<64, 5, 1, 4, kResidentB, 2>(ctx, op, ep, cv);
            }
        }
        return launch_conv_variant<64, 5, 2, 4, kResidentB>(ctx, op, ep, cv);
    }
    return launch_conv_variant<64, 4, 2, 4>(ctx, op, ep, cv);
}
} // namespace cugl
#endif // CUGL_TC_FULL_BUILD
