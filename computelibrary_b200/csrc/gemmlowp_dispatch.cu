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
} // namespace

bool gemmlowp_tcgen05_supported(const GemmOperands &op)
{
    return gemmlowp_tcgen05_supported_epi4(op);
}

// The SM-pair kernel pays off once a tile spans both halves (more than 128 rows and more than 128 columns) and
// the main loop is long enough to matter.
bool gemmlowp_tcgen05_uses_pair(const GemmOperands &op)
{
    return gemmlowp_tcgen05_uses_pair_epi4(op) && !eight_epilogue_warps(op);
}

cugl_status launch_gemmlowp_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                    bool allow_pair)
{
    // The channel-major kernel (operand roles exchanged, output-stage terms in registers, stores through a byte
    // transpose in shared memory) wins where the epilogue dominates and whole 128-channel blocks exist: measured
    // 802816 x 256 x 64: 209 us against 235 us row-major; 200704 x 512 x 128: 113 / 125; 50176 x 1024 x 256:
    // 63 / 70; 12544 x 2048 x 512: 39 / 47; but N = 64: 110 / 78 (half of the lanes idle).
    GemmOperands o = op;
    if (o.channel_major == 0)
    {
        // with a fused residual the row-major epilogue stays ahead (block-1 conv3 + add: 344 us against 377 us)
        o.channel_major = (o.K <= kShortK && o.N >= 256 && o.residual == nullptr) ? 1 : -1;
    }
    // sixteen epilogue warps (256-column tiles only) buy another 4 - 7 % on short K with wide outputs
    if (o.N > 128 && (o.epi_warps == 16 || (o.epi_warps != 4 && o.epi_warps != 8 && o.K <= kShortK)))
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
    return eight_epilogue_warps(op) ? launch_gemmlowp_conv_tcgen05_epi8(ctx, op, ep, cv)
                                    : launch_gemmlowp_conv_tcgen05_epi4(ctx, op, ep, cv);
}
} // namespace cugl
