// Chooses between the two builds of the tensor-core kernels (four or eight epilogue warps, see
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
    // The channel-major kernel (operand roles exchanged) runs only on request: its per-channel output-stage terms
    // live in registers, but its byte-wise transposed stores cost more than the shared-memory term reads of the
    // row-major epilogue save (802816 x 256 x 64: 256 us against 237 us).
    return eight_epilogue_warps(op) ? launch_gemmlowp_tcgen05_epi8(ctx, op, ep, false)
                                    : launch_gemmlowp_tcgen05_epi4(ctx, op, ep, allow_pair);
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
