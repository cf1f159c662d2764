// Launchers of every CUDA kernel in the library (defined in bandwidth_kernels.cu, gemmlowp_simt.cu
// and gemmlowp_tcgen05.cu).  All of them enqueue on ctx->stream and return without synchronising.
#pragma once

#include "common.cuh"

namespace cugl
{
cugl_status launch_reduce_rows(cugl_context *ctx, const void *d_a, bool is_signed, int M, int K, int64_t lda,
                               int32_t scalar, int32_t *d_out);
cugl_status launch_reduce_cols(cugl_context *ctx, const void *d_b, bool is_signed, int K, int N, int64_t ldb,
                               int32_t scalar, int32_t *d_out);
cugl_status launch_transpose_colsum(cugl_context *ctx, const void *d_b, bool is_signed, int K, int N, int64_t ldb,
                                    void *d_bt, int64_t ldbt, int32_t *d_colsum);
// batch matrices of rows x cols bytes, each transposed on its own (dense, back to back)
cugl_status launch_transpose_bytes(cugl_context *ctx, const void *d_src, int rows, int cols, void *d_dst, int batch = 1);
cugl_status launch_offset_contribution(cugl_context *ctx, int32_t *d_mm, int M, int N, int K, int64_t ld_bytes,
                                       const int32_t *d_colsum, const int32_t *d_rowsum, int32_t a_off,
                                       int32_t b_off);
cugl_status launch_output_stage(cugl_context *ctx, const int32_t *d_in, int64_t ld_in_bytes, const int32_t *d_bias,
                                void *d_out, int64_t ld_out_bytes, int M, int N, const int32_t *d_mults,
                                const int32_t *d_shifts, int32_t mult, int32_t shift, int32_t offset, int32_t lo,
                                int32_t hi, bool integer_stage = false, bool out16 = false);
// 2x2 space-to-depth lowering of stride-2 convolutions with <= 4 channels (see bandwidth_kernels.cu)
cugl_status launch_fold_input(cugl_context *ctx, const void *d_src, void *d_dst, int B, int H, int W, int C, int H2,
                              int W2, int zero_point);
cugl_status launch_fold_weights(cugl_context *ctx, const void *d_w, void *d_bt, int64_t ldbt, int OFM, int kh, int kw,
                                int C, int kh2, int kw2, int oy, int ox);
cugl_status launch_im2col_nhwc(cugl_context *ctx, const void *d_src, void *d_dst, int C, int W, int H, int B, int kw,
                               int kh, int sx, int sy, int pad_l, int pad_t, int dil_x, int dil_y, int Wo, int Ho,
                               int pad_value, int64_t row_stride);

// Operand description shared by both GEMM kernels.  B is always given K-major ("Bt": N rows of K
// contiguous bytes), which is what prepare() produces.
struct ConvOperands;
struct GemmOperands
{
    const void *a;   // [M][lda]   K contiguous
    const void *bt;  // [N][ldbt]  K contiguous
    void       *dst; // [M][ldd]   8-bit, or int32 when stage == NONE
    int64_t     lda, ldbt, ldd; // bytes
    int         M, N, K;
    bool        a_signed, b_signed;
    void       *extra_dst[7]; // tensor-core kernels only: further destinations that receive the same output
    int         n_extra_dst;  //   (peer GPUs' buffers in the push all-gather), same ldd as dst
    bool        generic_stage; // some shift is negative or some multiplier is INT32_MIN (decided on the host)
    bool        wide_stage;    // every shift in [2, 31], every multiplier in [0, 2^31), no row-sum term: the
                               // requantisation can use the one-multiply form (kStageWide)
    int         max_shift;     // largest right shift of the output stage (decides whether the offset fits kStagePack)
    int         pack_stage;    // < 0: never use the saturating-pack encoding (testing aid); else where it applies
    int         epi_warps;     // tensor-core kernels: 4, 8 or 16 forces that build, anything else lets the dispatcher choose
    // tensor-core kernels, 8-bit unsigned output only: dst = min(max(min(out + residual, 255), res_floor), res_cap)
    // with residual an [M][ldd] byte matrix (the fused residual addition of a convolution), or nullptr
    const void *residual;
    int         res_floor, res_cap;
    // > 0: run the GEMM with the operand roles exchanged (accumulator lanes = output channels); < 0: never;
    // 0: the dispatcher decides.  Ignored when a row-sum term or several destinations are present.
    int         channel_major;
    // SM-pair kernel: < 0 keeps every tile whole; otherwise the tiles of a short last wave are split in two
    int         split_tail;
    // one-CTA tensor-core kernels: tile width in columns (256, 128 or 64); 0 = the widest that N calls for.  Set by the
    // dispatcher, which narrows the tiles of an output too small to give every SM a wide one.
    int         block_n;
    // one-CTA tensor-core kernels with 256-column tiles: < 0 drains every accumulator buffer on its own; otherwise two
    // tiles of one column block are drained together wherever the output stage allows (see drain_accumulator_pair)
    int         pair_drain;
    // one-CTA row-major tensor-core kernels: not nullptr = implicit convolution, the A operand is read from the NHWC
    // tensor conv->src by im2col-mode TMA loads (a is ignored; M = B*Ho*Wo, K = kh*kw*C, C a multiple of 128, input
    // zero point 0)
    const ConvOperands *conv;
    // one-CTA row-major kernels, eight- and four-warp builds: < 0 keeps the epilogue on per-lane global stores; otherwise
    // a warp's 32 rows leave as one bulk tensor store from shared memory where the destination allows it
    int tma_store;
    // implicit convolution (gather): < 0 reloads the weights with every tile; otherwise they stay in shared memory for
    // the life of a CTA where one column block covers N and they fit beside the ring
    int resident_b;
    // the same kernels: < 0 keeps 128-row units of work; otherwise 256-row units (two tiles per hand-over) where the
    // output is large enough
    int double_tile;
};

// Geometry of an NHWC 8-bit convolution whose A operand is gathered on the fly (implicit GEMM).
// bytes of the zero-point pad buffer of the implicit convolution: 16 per gather thread
constexpr int kConvPadBytes = 16 * 256;

struct ConvOperands
{
    const void    *src;    // [B][H][W][C]
    const void    *pad;    // kConvPadBytes holding the input zero point (source of out-of-image taps)
    int            C, W, H, B, kw, kh, sx, sy, pad_l, pad_t, dil_x, dil_y, Wo, Ho;
};
bool        gemmlowp_conv_tcgen05_supported(const GemmOperands &op, const ConvOperands &cv);
// op.a / op.lda are unused: the A tile comes from cv.src.  M = B*Ho*Wo, K = kh*kw*C.
cugl_status launch_gemmlowp_conv_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                         const ConvOperands &cv);
// the two builds behind the dispatcher (four / eight epilogue warps)
bool        gemmlowp_conv_tcgen05_supported_epi4(const GemmOperands &op, const ConvOperands &cv);
bool        gemmlowp_conv_tcgen05_supported_epi8(const GemmOperands &op, const ConvOperands &cv);
cugl_status launch_gemmlowp_conv_tcgen05_epi4(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                              const ConvOperands &cv);
cugl_status launch_gemmlowp_conv_tcgen05_epi8(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                              const ConvOperands &cv);
bool        gemmlowp_tcgen05_supported_epi4(const GemmOperands &op);
bool        gemmlowp_conv_tma_supported_epi4(const GemmOperands &op); // op.conv set: im2col-mode route possible
bool        gemmlowp_conv_tma_supported(const GemmOperands &op);
bool        gemmlowp_tcgen05_supported_epi8(const GemmOperands &op);
bool        gemmlowp_tcgen05_uses_pair_epi4(const GemmOperands &op);
bool        gemmlowp_tcgen05_uses_pair_epi8(const GemmOperands &op);
cugl_status launch_gemmlowp_tcgen05_epi4(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                         bool allow_pair);
cugl_status launch_gemmlowp_tcgen05_epi8(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                         bool allow_pair);
// sixteen epilogue warps: 256-column one-CTA tiles only (op.N is not looked at)
cugl_status launch_gemmlowp_tcgen05_epi16(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                          bool allow_pair);

// Generic CUDA-core kernel: any shape, stride and alignment.
cugl_status launch_gemmlowp_simt(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep);

// TMA + tcgen05.mma.kind::i8 kernel.  Requires a, bt 16-byte aligned and lda, ldbt multiples of 16.
bool        gemmlowp_tcgen05_supported(const GemmOperands &op);
bool        gemmlowp_tcgen05_uses_pair(const cugl_context *ctx, const GemmOperands &op);
// allow_pair = false keeps to the one-CTA kernels (testing aid; all variants must agree bit for bit).
cugl_status launch_gemmlowp_tcgen05(cugl_context *ctx, const GemmOperands &op, const EpilogueParams &ep,
                                    bool allow_pair = true);
// The rules of cugl_gemmlowp_validate; returns nullptr (and *code = CUGL_SUCCESS) or the reason.
const char *validate_gemm_desc(const cugl_gemm_desc *d, cugl_status *code, bool need_host_vectors);
// QASYMM8 addition: true when the oracle's result equals min(max(min(a + b, 255), floor), cap) for every byte pair
// (proved by enumeration on the host, remembered per parameter set).
bool classify_add(float a_scale, int a_zp, float b_scale, int b_zp, float o_scale, int o_zp, int act, float act_a,
                  float act_b, int *floor_out, int *cap_out);
} // namespace cugl
