"""The allocation-free entry point (cugl_gemmlowp_run_noalloc) against the planned entry point.

Who needs it: hosts that may not call cudaMalloc while they run -- a serving loop that gave all device memory
to its own arena, a plugin inside somebody else's process, work recorded into a stream capture.  The call
takes its workspace from a fixed array inside the library, so this file checks that (a) results are
bit-identical to cugl_gemmlowp_plan_create / prepare / run and to the CPU oracle, (b) a second call, with
different shapes and data, is not polluted by what the first call left in the shared array, (c) oversize
problems are refused, (d) a per-channel descriptor that carries no host copies of its vectors is accepted,
and (e) the status query reports no device-side time-out after each call.
It is collected last (file name) so that a run stopping at the first failure has already run everything else;
it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest

import oracle
from computelibrary_b200 import capi
from helpers import gpu_gemmlowp, q8_uniform

pytestmark = pytest.mark.gpu
CODE = {np.dtype(np.uint8): capi.U8, np.dtype(np.int8): capi.S8}


def run_noalloc(a, b, bias, a_off, b_off, mult, shift, offset, lo, hi, out_dtype, host_vectors=True):
    import torch
    M, K = a.shape
    N = b.shape[1]
    per_channel = np.ndim(mult) > 0
    desc, keep = capi.make_gemm_desc(M, N, K, CODE[a.dtype], CODE[b.dtype], CODE[np.dtype(out_dtype)], a_off, b_off,
                                     multiplier=0 if per_channel else int(mult),
                                     shift=0 if per_channel else int(shift),
                                     multipliers=mult if per_channel else None,
                                     shifts=shift if per_channel else None, offset=offset, min_bound=lo,
                                     max_bound=hi, has_bias=bias is not None)
    if per_channel and not host_vectors:  # the vectors exist on the device only
        desc.h_gemmlowp_multipliers = None
        desc.h_gemmlowp_shifts = None
    stream = torch.cuda.current_stream().cuda_stream
    d_a = torch.from_numpy(a.view(np.uint8)).cuda()
    d_b = torch.from_numpy(b.view(np.uint8)).cuda()
    d_bias = torch.from_numpy(bias).cuda() if bias is not None else None
    d_m = torch.from_numpy(np.asarray(mult, np.int32)).cuda() if per_channel else None
    d_s = torch.from_numpy(np.asarray(shift, np.int32)).cuda() if per_channel else None
    d_dst = torch.full((M, N), 0x5A, dtype=torch.uint8, device="cuda")
    capi.gemmlowp_run_noalloc(stream, desc, d_a, d_b, d_bias, d_m, d_s, d_dst)
    capi.gemmlowp_noalloc_status(stream)  # waits for the stream; raises if a bounded device wait ran out
    return d_dst.cpu().numpy().view(out_dtype)


def test_noalloc_matches_planned_entry_point_twice(ctx):
    rng = np.random.default_rng(42)
    # call 1: s8 x s8, per-channel, both kernels' favourite shape (SM-pair tensor-core kernel)
    a1, b1 = q8_uniform(rng, (384, 512), np.int8), q8_uniform(rng, (512, 320), np.int8, -127, 127)
    bias1 = rng.integers(-5000, 5001, 320).astype(np.int32)
    mult1 = rng.integers(2 ** 30, 2 ** 31 - 1, 320).astype(np.int32)
    shift1 = rng.integers(4, 12, 320).astype(np.int32)
    want1, _ = gpu_gemmlowp(ctx, a1, b1, bias1, 5, 0, mult1, shift1, 0, -128, 127, np.int8)
    got1 = run_noalloc(a1, b1, bias1, 5, 0, mult1, shift1, 0, -128, 127, np.int8)
    assert np.array_equal(got1, want1)
    port = oracle.port()
    assert np.array_equal(got1, port.gemmlowp_fused(a1, b1, bias1, 5, 0, mult1, shift1, 0, -128, 127, np.int8))
    # call 2, straight after: smaller u8 x u8 problem with both offsets (row sums + column sums from the same
    # array the first call used), per-tensor stage, odd sizes
    a2, b2 = q8_uniform(rng, (100, 144), np.uint8), q8_uniform(rng, (144, 77), np.uint8)
    bias2 = rng.integers(-2000, 2001, 77).astype(np.int32)
    want2, _ = gpu_gemmlowp(ctx, a2, b2, bias2, -128, -120, 1099511552, 8, 10, 0, 255, np.uint8)
    got2 = run_noalloc(a2, b2, bias2, -128, -120, 1099511552, 8, 10, 0, 255, np.uint8)
    assert np.array_equal(got2, want2)
    assert np.array_equal(got2, port.gemmlowp_fused(a2, b2, bias2, -128, -120, [1099511552], [8], 10, 0, 255, np.uint8))
    # and the first problem again: identical result a second time
    assert np.array_equal(run_noalloc(a1, b1, bias1, 5, 0, mult1, shift1, 0, -128, 127, np.int8), want1)


def test_noalloc_per_channel_vectors_on_the_device_only():
    """A caller that keeps its multipliers and shifts in device memory passes no host copies: the descriptor's
    h_ pointers are NULL."""
    rng = np.random.default_rng(7)
    a, b = q8_uniform(rng, (130, 96), np.uint8), q8_uniform(rng, (96, 72), np.int8, -127, 127)
    bias = rng.integers(-3000, 3001, 72).astype(np.int32)
    mult = rng.integers(2 ** 30, 2 ** 31 - 1, 72).astype(np.int32)
    shift = rng.integers(0, 12, 72).astype(np.int32)
    got = run_noalloc(a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8, host_vectors=False)
    assert np.array_equal(got, oracle.port().gemmlowp_fused(a, b, bias, -7, 0, mult, shift, 3, 0, 255, np.uint8))


def test_noalloc_rejects_oversize_problem():
    import torch
    d, keep = capi.make_gemm_desc(128, 8192, 1024, capi.S8, capi.S8, capi.S8, multiplier=2 ** 30, shift=3,
                                  min_bound=-128, max_bound=127)  # 8192 * 1024 = 8 MiB of B > 4 MiB
    x = torch.zeros(16, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.CuglError) as e:
        capi.gemmlowp_run_noalloc(0, d, x, x, None, None, None, x)
    assert e.value.status == 6 and "fixed workspace" in e.value.message
