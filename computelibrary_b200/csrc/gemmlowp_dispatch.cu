// Chooses between the builds of the tensor-core kernels (four, eight or sixteen epilogue warps, see
// gemmlowp_tcgen05.cu).  The main loop of a 128 x 256 tile takes about 128 clocks per 32 bytes of K; its
// epilogue takes a fixed few thousand clocks with four warps.  Up to kShortK the epilogue is the longer of the
// two and gets eight warps; beyond it the main loop is, and extra resident warps only slow its single-thread
// producer and MMA loops down.
#include "kernels.cuh"

namespace cugl
{
namespace
{
constexpr int kShortK = 1024;

bool eight_epilogue_warps(const GemmOperands &op)
{
    if (op.epi_warps == 4 || op.epi_warps == 8)
    {
        return op.epi_warps == 8; // forced by the caller (tests, measurements)
    }
    return op.K <= kShortK;
}

// Tile width of the one-CTA kernels.  The widest tile N calls for moves the fewest operand bytes per output, but
// an output of fewer such tiles than SMs leaves SMs idle while each busy one walks all of K for a wide tile.
// Then the width is the one that minimises (waves of tiles over the SMs) x (128 + width), the operand bytes a
// CTA stages per K step; ties go to the wider tile.
int pick_block_n(const cugl_context *ctx, const GemmOperands &op)
{
    const int widest = op.N > 128 ? 256 : (op.N > 64 ? 128 : 64);
    if (op.block_n > 0)
    {
        return op.block_n < widest ? op.block_n : widest;
    }
    if (op.epi_warps == 16 || op.channel_major > 0)
    {
        return widest; // kernels the caller asked for by name: 256-column tiles only
    }
    const long long sms     = ctx->sm_count > 0 ? ctx->sm_count : 1;
    const long long m_tiles = (op.M + 127) / 128;
    if (m_tiles * ((op.N + widest - 1) / widest) >= sms)
    {
        return widest;
    }
    int       best      = widest;
    long long best_cost = -1;
    for (int bn = widest; bn >= 64; bn >>= 1)
    {
        const long long tiles = m_tiles * ((op.N + bn - 1) / bn);
        const long long cost  = ((tiles + sms - 1) / sms) * (128 + bn);
        if (best_cost < 0 || cost < best_cost)
        {
            best      = bn;
            best_cost = cost;
        }
    }
    return best;
}

// the SM-pair kernel works on 256 x 256 tiles, one per pair of SMs
bool pair_fills_the_device(const cugl_context *ctx, const GemmOperands &op)
{
    const long long tiles = static_cast<long long>((op.M + 255) / 256) * ((op.N + 255) / 256);
    return tiles >= ctx->sm_count / 2;
}
} // namespace

bool gemmlowp_conv_tma_supported(const GemmOperands &op)
{
    return gemmlowp_conv_tma_supported_epi4(op);
}

bool gemmlowp_tcgen05_supported(const GemmOperands &op)
{
    return gemmlowp_tcgen05_supported_epi4(op);
}

// The SM-pair kernel pays off once a tile spans both halves (more than 128 rows and more than 128 columns), the
// main loop is long enough to matter and there is a 256 x 256 tile for every pair of SMs.
bool gemmlowp_tcgen05_uses_pair(const cugl_context *ctx, const GemmOperands &op)
{
    return gemmlowp_tcgen05_uses_pair_epi4(op) && !eight_epilogue_warps(op) && pair_fills_the_device(ctx, op) &&
           (op.block_n == 0 || op.block_n == 256);
}

cugl_status launch_gemmlowp_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                    bool allow_pair)
{
    // The channel-major kernel (operand roles exchanged, output-stage terms in registers, stores through a byte
    // transpose in shared memory) against the row-major one with sixteen epilogue warps, paired drain and 256-bit
    // stores, measured: 802816 x 256 x 64: 189 us against 170 us; 200704 x 512 x 128: 102 / 94; 50176 x 1024 x 256:
    // 57 / 60; 12544 x 2048 x 512: 37 / 43.  It needs whole 128-channel blocks (N = 64: 110 / 78).
    GemmOperands o   = op;
    o.block_n        = pick_block_n(ctx, op); // before the automatic channel-major choice below
    if (ep.stage == CUGL_STAGE_NONE && (ep.out_f32 != 0 || ep.accumulate != 0) && o.channel_major == 0)
    {
        o.channel_major = -1; // read-modify-write of dst rows: the row-major epilogue does it with 128-bit accesses
    }
    if (o.channel_major == 0)
    {
        // with a fused residual too: 50176 x 1024 x 256 + residual 69 us against 79 us row-major, 12544 x 2048 x 512
        // 43 / 53; below K = 256 the two are level with a residual (200704 x 512 x 128: 125 / 128) and the row-major
        // kernel is ahead without one (102 / 94)
        // since the row-major epilogue stores through the TMA unit the two were measured again (batch 256, row-major /
        // channel-major): 256 -> 1024 at 14 x 14 45 / 45 us (with a residual 64 / 60), 256 -> 512 at 28 x 28 74 / 84,
        // 1024 -> 256 27 / 29, 512 -> 1024 53 / 49, 512 -> 2048 at 7 x 7 37 / 31, 1024 -> 2048 41 / 37
        o.channel_major = (o.K >= 512 && o.K <= kShortK && o.N >= 1024) ? 1 : -1;
    }
    const int widest = o.N > 128 ? 256 : (o.N > 64 ? 128 : 64);
    if (o.block_n < widest)
    {
        // a small output: narrower tiles on more SMs (the kernels of the complete builds only)
        o.channel_major = -1;
        return eight_epilogue_warps(o) ? launch_gemmlowp_tcgen05_epi8(ctx, o, ep, false)
                                       : launch_gemmlowp_tcgen05_epi4(ctx, o, ep, false);
    }
    allow_pair = allow_pair && pair_fills_the_device(ctx, o);
    // sixteen epilogue warps (256-column tiles only) buy another 4 - 7 % on short K with wide outputs
    // (up to K = 512, where its paired drain applies; above, eight warps -- whose single-tile drain stores through the
    // TMA unit -- measured faster: 50176 x 256 x 1024 25.5 against 27.6 us)
    if (o.N > 128 && (o.epi_warps == 16 || (o.epi_warps != 4 && o.epi_warps != 8 && o.K <= 512)))
    {
        return launch_gemmlowp_tcgen05_epi16(ctx, o, ep, false);
    }
    return eight_epilogue_warps(o) ? launch_gemmlowp_tcgen05_epi8(ctx, o, ep, false)
                                   : launch_gemmlowp_tcgen05_epi4(ctx, o, ep, allow_pair);
}

bool gemmlowp_conv_tcgen05_supported(const GemmOperands &op, const ConvOperands &cv)
{
    return gemmlowp_conv_tcgen05_supported_epi4(op, cv);
}

cugl_status launch_gemmlowp_conv_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                         const ConvOperands &cv)
{
    GemmOperands o = op;
    o.block_n      = pick_block_n(ctx, o);
    return eight_epilogue_warps(o) ? launch_gemmlowp_conv_tcgen05_epi8(ctx, o, ep, cv)
                                   : launch_gemmlowp_conv_tcgen05_epi4(ctx, o, ep, cv);
}
} // namespace cugl
