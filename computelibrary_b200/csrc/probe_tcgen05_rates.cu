// Measures, on one SM with nothing else running, what the thread that issues tensor-core work pays per instruction:
//   * tcgen05.mma kind::i8, M = 128 (cta_group::1), for N = 16 .. 256: clocks from one issue to the next in a long
//     chain (the issue is back-pressured by the tensor pipe, so this is the pipe's rate for that shape);
//   * tcgen05.commit after groups of 0 .. 16 MMAs;
//   * mbarrier try_wait / test_wait / arrive and the fences of the issue loop.
// The figures bound what a tile shape can reach: the roofline of a 64-column tile is not the one of a 256-column tile.
// Prints one JSON object.  Every wait is bounded; operands are whatever bytes the kernel writes into shared memory.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

namespace
{
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// K-major operand tile in the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ uint32_t idesc_i8(int n)
{
    return (2u << 4) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// waits for the phase with a clock limit; false when it ran out
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity)
{
    const long long t0 = clock64();
    uint32_t        n  = 0;
    while (!try_wait(bar, parity))
    {
        if ((++n & 255u) == 0 && clock64() - t0 > 2000000000ll)
        {
            return false;
        }
    }
    return true;
}

constexpr int kChainVariants = 6;  // N = 16, 32, 64, 128, 256 and N = 64 over four accumulators in rotation
constexpr int kGroupVariants = 10; // (MMAs per commit, N)
constexpr int kOps           = 7;
constexpr int kResults       = kChainVariants + kGroupVariants + kOps + 1; // + error flag
constexpr int kSmemBytes     = 4 * (16 + 32) * 1024 + 1024;                // four stages of A (16 KB) and B (32 KB)

__global__ void __launch_bounds__(128, 1) probe_kernel(double *out)
{
    extern __shared__ uint8_t raw[];
    uint8_t *smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    __shared__ uint32_t             s_tmem;
    __shared__ __align__(8) uint64_t s_bar[kChainVariants + kGroupVariants + 1];
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 4 * (16 + 32) * 1024 / 4; i += blockDim.x)
    {
        reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u * (i & 3);
    }
    constexpr int kGroups = 64; // commits per group variant
    if (threadIdx.x == 0)
    {
        for (int v = 0; v < kChainVariants; ++v)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_bar[v])) : "memory");
        }
        for (int v = 0; v < kGroupVariants; ++v)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_bar[kChainVariants + v])), "r"(kGroups) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_bar[kChainVariants + kGroupVariants])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    if (threadIdx.x == 0)
    {
        bool           ok = true;
        const uint64_t a0 = kmajor_sw128_desc(smem_u32(smem)), b0 = kmajor_sw128_desc(smem_u32(smem) + 4 * 16 * 1024);
        // ---- chains of 256 MMAs, eight per stage of operands, as the kernels' issue loops walk them
        const int chain_n[kChainVariants]    = {16, 32, 64, 128, 256, 64};
        const int chain_accs[kChainVariants] = {1, 1, 1, 1, 1, 4};
        for (int v = 0; v < kChainVariants && ok; ++v)
        {
            const int      n = chain_n[v];
            const uint32_t idesc = idesc_i8(n), amask = static_cast<uint32_t>(chain_accs[v] - 1), bar = smem_u32(&s_bar[v]);
            constexpr int  kMmas = 256;
            const long long t0 = clock64();
            for (int i = 0; i < kMmas; i += 8)
            {
                const int      st = (i >> 3) & 3;
                const uint64_t a = a0 + static_cast<uint64_t>((st * 16 * 1024) >> 4), b = b0 + static_cast<uint64_t>((st * 32 * 1024) >> 4);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    umma(tmem + (static_cast<uint32_t>(i + j) & amask) * n, a + 2u * (j & 3), b + 2u * (j & 3), idesc,
                         i + j >= chain_accs[v] ? 1u : 0u);
                }
            }
            commit(bar);
            ok = bounded_wait(bar, 0);
            out[v] = static_cast<double>(clock64() - t0) / kMmas;
        }
        // ---- groups of k MMAs, each followed by a commit
        const int group_k[kGroupVariants] = {0, 1, 2, 4, 8, 16, 2, 8, 2, 8};
        const int group_n[kGroupVariants] = {64, 64, 64, 64, 64, 64, 128, 128, 256, 256};
        for (int v = 0; v < kGroupVariants && ok; ++v)
        {
            const int      k = group_k[v], n = group_n[v];
            const uint32_t idesc = idesc_i8(n), bar = smem_u32(&s_bar[kChainVariants + v]);
            const long long t0 = clock64();
            for (int g = 0; g < kGroups; ++g)
            {
                for (int j = 0; j < k; ++j)
                {
                    umma(tmem + (g & 1) * n, a0 + 2u * (j & 3), b0 + 2u * (j & 3), idesc, j ? 1u : 0u);
                }
                commit(bar);
            }
            ok = bounded_wait(bar, 0);
            out[kChainVariants + v] = static_cast<double>(clock64() - t0) / kGroups;
        }
        // ---- the small instructions of an issue loop
        const uint32_t bar = smem_u32(&s_bar[kChainVariants + kGroupVariants]);
        asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory"); // phase 0 complete
        constexpr int R = 256;
        uint32_t      acc = 0;
        double       *ops = out + kChainVariants + kGroupVariants;
        long long     t0  = clock64();
        for (int i = 0; i < R; ++i) acc += try_wait(bar, 0) ? 1u : 0u;
        ops[0] = static_cast<double>(clock64() - t0) / R; // try_wait, phase complete
        t0     = clock64();
        for (int i = 0; i < R; ++i) acc += try_wait(bar, 1) ? 1u : 0u;
        ops[1] = static_cast<double>(clock64() - t0) / R; // try_wait, phase not complete
        t0     = clock64();
        for (int i = 0; i < R; ++i) acc += test_wait(bar, 0) ? 1u : 0u;
        ops[2] = static_cast<double>(clock64() - t0) / R;
        t0     = clock64();
        for (int i = 0; i < R; ++i) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        ops[3] = static_cast<double>(clock64() - t0) / R;
        t0     = clock64();
        for (int i = 0; i < R; ++i) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        ops[4] = static_cast<double>(clock64() - t0) / R;
        t0     = clock64();
        for (int i = 0; i < R; ++i) asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
        ops[5] = static_cast<double>(clock64() - t0) / R;
        t0     = clock64();
        for (int i = 0; i < R; ++i) acc += static_cast<uint32_t>(clock64());
        ops[6] = static_cast<double>(clock64() - t0) / R; // the clock read itself (included in every figure once per loop)
        out[kResults - 1] = ok ? 0.0 : 1.0 + (acc == 0xffffffffu ? 1.0 : 0.0);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
    {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}
} // namespace

int main()
{
    double *d_out = nullptr;
    if (cudaMalloc(&d_out, kResults * sizeof(double)) != cudaSuccess ||
        cudaMemset(d_out, 0, kResults * sizeof(double)) != cudaSuccess ||
        cudaFuncSetAttribute(probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    {
        std::fprintf(stderr, "setup failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    double h[kResults];
    for (int rep = 0; rep < 3; ++rep) // the last of three runs is reported
    {
        probe_kernel<<<1, 128, kSmemBytes>>>(d_out);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess)
        {
            std::fprintf(stderr, "kernel failed: %s\n", cudaGetErrorString(e));
            return 1;
        }
    }
    cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
    if (h[kResults - 1] != 0.0)
    {
        std::fprintf(stderr, "a wait ran out\n");
        return 1;
    }
    const int   chain_n[kChainVariants] = {16, 32, 64, 128, 256, 64};
    const char *chain_tag[kChainVariants] = {"", "", "", "", "", "_4acc"};
    const int   group_k[kGroupVariants] = {0, 1, 2, 4, 8, 16, 2, 8, 2, 8};
    const int   group_n[kGroupVariants] = {64, 64, 64, 64, 64, 64, 128, 128, 256, 256};
    const char *ops[kOps] = {"try_wait_complete", "try_wait_incomplete", "test_wait", "tcgen05_fence_after", "fence_proxy_async",
                             "mbarrier_arrive", "clock_read"};
    std::printf("{\"unit\": \"SM clocks\", \"mma_m128_i8_clocks_per_instruction\": {");
    for (int v = 0; v < kChainVariants; ++v)
    {
        std::printf("%s\"n%d%s\": %.1f", v ? ", " : "", chain_n[v], chain_tag[v], h[v]);
    }
    std::printf("}, \"ideal_clocks_at_8192_mac_per_clock\": {");
    for (int v = 0; v < 5; ++v)
    {
        std::printf("%s\"n%d\": %.0f", v ? ", " : "", chain_n[v], 128.0 * chain_n[v] * 32 / 8192.0);
    }
    std::printf("}, \"clocks_per_group_of_k_mmas_and_one_commit\": {");
    for (int v = 0; v < kGroupVariants; ++v)
    {
        std::printf("%s\"k%d_n%d\": %.1f", v ? ", " : "", group_k[v], group_n[v], h[kChainVariants + v]);
    }
    std::printf("}, \"clocks_per_instruction\": {");
    for (int v = 0; v < kOps; ++v)
    {
        std::printf("%s\"%s\": %.1f", v ? ", " : "", ops[v], h[kChainVariants + kGroupVariants + v]);
    }
    std::printf("}}\n");
    cudaFree(d_out);
    return 0;
}
