// Compute Library's OWN validation fixtures (tests/validation/fixtures/GEMMLowpFixture.h) instantiated with the CUDA
// backend's FunctionType / TensorType / AccessorType triple -- the way tests/validation/NEON/GEMMLowp.cpp:60-91
// instantiates them with NEGEMMLowpMatrixMultiplyCore / Tensor / Accessor -- and compared with the reference the
// fixture computes itself (reference::gemmlowp_matrix_multiply_core and the output-stage oracles).  The fixture
// headers are compiled from the Compute Library tree where they lie; nothing of them is copied here.
#include "arm_compute/runtime/CUDA/CUScheduler.h"
#include "arm_compute/runtime/CUDA/functions/CUGEMMLowpMatrixMultiplyCore.h"
#include "tests/cpp/CUAccessor.h"
#include "tests/validation/fixtures/GEMMLowpFixture.h"

#include <cstdio>

using namespace arm_compute;
using namespace arm_compute::test;
using namespace arm_compute::test::validation;

// the two globals tests/main.cpp:70-71 defines for the fixtures' seeded fills
namespace arm_compute
{
namespace test
{
std::unique_ptr<AssetsLibrary> library;
std::unique_ptr<AssetsLibrary> fixed_library;
} // namespace test
} // namespace arm_compute

namespace
{
int g_failures = 0;

// element-wise comparison of a target tensor with the fixture's reference, tolerance in units of T
template <typename T>
long mismatches(CUTensor &target, const SimpleTensor<T> &reference, double tolerance)
{
    CUAccessor acc(target);
    long       bad = 0;
    if (acc.shape() != reference.shape())
    {
        return -1;
    }
    for (int i = 0; i < reference.num_elements(); ++i)
    {
        const Coordinates c  = index2coord(reference.shape(), i);
        const T           tv = *reinterpret_cast<const T *>(acc(c));
        if (std::abs(static_cast<double>(tv) - static_cast<double>(reference[i])) > tolerance)
        {
            ++bad;
        }
    }
    return bad;
}

template <typename F>
struct Open : public F // the fixtures keep _target / _reference protected
{
    using F::_reference;
    using F::_target;
};

template <typename Fixture, typename T, typename... Args>
void run_case(const char *name, double tolerance, Args &&...args)
{
    Open<Fixture> f;
    f.setup(std::forward<Args>(args)...);
    const long bad = mismatches<T>(f._target, f._reference, tolerance);
    std::printf("%-64s %s (%ld mismatches)\n", name, bad == 0 ? "ok" : "FAILED", bad);
    g_failures += bad == 0 ? 0 : 1;
}
} // namespace

using CUCore          = GEMMLowpMatrixMultiplyCoreValidationFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore>;
using CUCoreTwice     = GEMMLowpMatrixMultiplyCoreValidationFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore, false, false, true>;
using CUCoreAccum     = GEMMLowpMatrixMultiplyAccumulateValidationFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore>;
using CUFused         = GEMMLowpMatrixMultiplyCoreFusedOffsetOutputValidationFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore>;
using CUFusedBatched  = GEMMLowpBatchedMatrixMultiplyCoreFusedOffsetOutputFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore>;
using CUDequantized   = GEMMLowpDequantizedMatrixMultiplyValidationFixture<CUTensor, CUAccessor, CUGEMMLowpMatrixMultiplyCore, float>;

int main()
{
    try
    {
        CUScheduler::get().default_init(0);
        // the framework's global asset library: only its seeded random fills are used (tests/main.cpp:82, fixed seed 1)
        library       = std::make_unique<AssetsLibrary>(".", 1);
        fixed_library = std::make_unique<AssetsLibrary>(".", 1);

        // S32 core: config-1 shape of examples/neon_gemm_qasymm8.cpp, shapes of tests/datasets/SmallGEMMLowpDataset.h:43-52
        run_case<CUCore, int32_t>("core 64x128x256 (config 1), offsets -128 / -120", 0, TensorShape(256U, 64U), TensorShape(128U, 256U),
                                  TensorShape(128U, 64U), -128, -120);
        run_case<CUCore, int32_t>("core 21x13x33, offsets 0 / 0", 0, TensorShape(21U, 13U), TensorShape(33U, 21U), TensorShape(33U, 13U), 0, 0);
        run_case<CUCore, int32_t>("core 52x13x33, offsets 0 / 4", 0, TensorShape(52U, 13U), TensorShape(33U, 52U), TensorShape(33U, 13U), 0, 4);
        run_case<CUCore, int32_t>("core 31x27x23, offsets 18 / 23", 0, TensorShape(31U, 27U), TensorShape(23U, 31U), TensorShape(23U, 27U), 18, 23);
        // tests/datasets/LargeGEMMLowpDataset.h:43-52 (K = 1021: no multiple of 16, a 16-byte-pitch copy of A keeps it on tcgen05)
        run_case<CUCore, int32_t>("core large dataset a(1021,973) b(221,1021), offsets 10 / 2", 0, TensorShape(1021U, 973U),
                                  TensorShape(221U, 1021U), TensorShape(221U, 973U), 10, 2);
        run_case<CUCoreTwice, int32_t>("core run twice with new data 32x72x17", 0, TensorShape(32U, 72U), TensorShape(17U, 32U),
                                       TensorShape(17U, 72U), -50, -30);
        run_case<CUCoreAccum, int32_t>("core accumulate 32x72x17", 0, TensorShape(32U, 72U), TensorShape(17U, 32U), TensorShape(17U, 72U), -9, 1);
        // fused offset contribution + fixed-point output stage (tolerance 1 in the reference's own NEON test: :361-384)
        run_case<CUFused, uint8_t>("fused QASYMM8 x QASYMM8 64x128x256", 0, TensorShape(256U, 64U), TensorShape(128U, 256U),
                                   TensorShape(128U, 64U), GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT, DataType::QASYMM8, true);
        run_case<CUFused, uint8_t>("fused QASYMM8 x QASYMM8 21x13x33, B constant", 0, TensorShape(21U, 13U), TensorShape(33U, 21U),
                                   TensorShape(33U, 13U), GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT, DataType::QASYMM8, true);
        run_case<CUFused, uint8_t>("fused QASYMM8 x QASYMM8 31x27x23, B variable", 0, TensorShape(31U, 27U), TensorShape(23U, 31U),
                                   TensorShape(23U, 27U), GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT, DataType::QASYMM8, false);
        run_case<CUFused, uint8_t>("fused QUANTIZE_DOWN (integer stage) 32x72x17", 0, TensorShape(32U, 72U), TensorShape(17U, 32U),
                                   TensorShape(17U, 72U), GEMMLowpOutputStageType::QUANTIZE_DOWN, DataType::QASYMM8, false);
        run_case<CUFusedBatched, uint8_t>("fused batched 21x13x33 x 3", 0, TensorShape(21U, 13U, 3U), TensorShape(33U, 21U, 3U),
                                          TensorShape(33U, 13U, 3U), GEMMLowpOutputStageType::QUANTIZE_DOWN_FIXEDPOINT, DataType::QASYMM8, false);
        // dequantised F32 output (tolerance 0.01 absolute in the reference's test, :570-581)
        run_case<CUDequantized, float>("dequantized F32 32x72x17", 0.0, TensorShape(32U, 72U), TensorShape(17U, 32U), TensorShape(17U, 72U), 5, 9,
                                       DataType::QASYMM8_SIGNED, DataType::QASYMM8_SIGNED, DataType::F32, false);
        run_case<CUDequantized, float>("dequantized F32 accumulate 32x72x17", 1e-5, TensorShape(32U, 72U), TensorShape(17U, 32U), TensorShape(17U, 72U),
                                       5, 9, DataType::QASYMM8_SIGNED, DataType::QASYMM8_SIGNED, DataType::F32, true);
    }
    catch (const std::exception &e)
    {
        std::printf("EXCEPTION: %s\n", e.what());
        return 2;
    }
    std::printf("%s (%d failing case%s)\n", g_failures == 0 ? "OK" : "FAILED", g_failures, g_failures == 1 ? "" : "s");
    return g_failures == 0 ? 0 : 1;
}
