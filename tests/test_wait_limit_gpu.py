"""The give-up path of the tensor-core kernels: every device-side wait on a barrier is bounded, and a wait that runs
out ends the launch with CUGL_RUNTIME_ERROR at the next synchronisation instead of hanging the GPU.  The wait is made
to run out on purpose and harmlessly: the limit is lowered to about a millisecond and one operand copy of CTA 0 is left
out (cugl_context_withhold_copy_once), so the MMA issuer's wait for it gives up, the other roles of the CTA see the
abort flag, tensor memory is freed and the kernel returns.  The following launch on the same context must be
bit-exact: it could not even start if tensor memory had leaked."""
import numpy as np
import pytest

from computelibrary_b200 import capi
from helpers import gpu_gemmlowp, q8_uniform

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,pair,want_kernel", [(512, 256, 2048, False, "tcgen05"), (2560, 2048, 2048, True, "tcgen05_2cta")])
@pytest.mark.parametrize("k_block", [0, 3])
def test_withheld_copy_gives_up_and_the_context_recovers(ctx, port, M, N, K, pair, want_kernel, k_block):
    import torch
    import computelibrary_b200 as cl
    r = np.random.default_rng(M + k_block)
    a, b = q8_uniform(r, (M, K), np.uint8), q8_uniform(r, (K, N), np.uint8)
    bias = r.integers(-2000, 2000, N).astype(np.int32)
    qm, sh = capi.calculate_quantized_multiplier(0.0004)
    # the rows of CTA 0's tile against the oracle, the whole output against an undisturbed launch on another context
    want_head = port.gemmlowp_fused(a[:256], b, bias, -3, -7, [qm], [sh], 10, 0, 255, np.uint8)
    want, kernel = gpu_gemmlowp(ctx, a, b, bias, -3, -7, qm, sh, 10, 0, 255, np.uint8, pair=pair)
    assert kernel == want_kernel
    assert np.array_equal(want[:256], want_head)
    ctx = cl.Context(0, torch.cuda.current_stream().cuda_stream)
    try:
        ctx.set_wait_limit_us(1000)
        ctx.withhold_copy_once(k_block)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        with pytest.raises(capi.CuglError) as err:
            gpu_gemmlowp(ctx, a, b, bias, -3, -7, qm, sh, 10, 0, 255, np.uint8, pair=pair)
        t1.record()
        torch.cuda.synchronize()
        assert err.value.status == capi.RUNTIME_ERROR
        assert "bounded wait ran out" in err.value.message
        assert t0.elapsed_time(t1) < 500.0  # the limit is a millisecond per wait, not the two-second default
        # the same context, straight afterwards: one shot is spent, status word cleared, tensor memory free again
        for _ in range(2):
            out, kernel = gpu_gemmlowp(ctx, a, b, bias, -3, -7, qm, sh, 10, 0, 255, np.uint8, pair=pair)
            assert kernel == want_kernel
            assert np.array_equal(out, want)
        ctx.set_wait_limit_us(0)
        out, _ = gpu_gemmlowp(ctx, a, b, bias, -3, -7, qm, sh, 10, 0, 255, np.uint8, pair=pair)
        assert np.array_equal(out, want)
    finally:
        ctx.close()


def test_withhold_argument_is_checked(ctx):
    with pytest.raises(capi.CuglError) as err:
        ctx.withhold_copy_once(-1)
    assert err.value.status == capi.INVALID_ARGUMENT
