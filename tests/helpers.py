"""Seeded synthetic inputs and small drivers shared by the tests (and by bench.py / smoke())."""
from __future__ import annotations

import numpy as np

from computelibrary_b200 import capi

NP_OF = {capi.U8: np.uint8, capi.S8: np.int8, capi.S32: np.int32, capi.F32: np.float32}
CODE_OF = {np.dtype(np.uint8): capi.U8, np.dtype(np.int8): capi.S8, np.dtype(np.int32): capi.S32,
           np.dtype(np.float32): capi.F32}


from computelibrary_b200.workloads import (config1, config2, config3, config5, q8_uniform,  # noqa: F401,E402
                                           type_range)


def f32_mults(port, i_scale, w_scales, o_scale):
    return port.calculate_quantized_multipliers(np.float32(i_scale), np.asarray(w_scales, np.float32),
                                                np.float32(o_scale))


# ---- GPU drivers (torch tensors as device buffers) ------------------------------------------------------
def gpu_gemmlowp(ctx, a, b, bias, a_off, b_off, mult, shift, offset, lo, hi, out_dtype, force_simt=False,
                 b_constant=True, runs=1, ldd_pad=0, pair=True, epi_warps=0, channel_major=0, integer_stage=False,
                 tile_columns=0, paired_drain=True, accumulate=False, dequantize_scale=0.0, dst_init=None,
                 temp_workspace=False, saturating_pack=True, tma_store=True):
    """Fused NEGEMMLowpMatrixMultiplyCore through the C ABI.  mult/shift scalars -> per-tensor; arrays ->
    per-channel.  out_dtype np.int32 -> output stage NONE.  Returns (numpy result, kernel name)."""
    import torch
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    batched = a.ndim == 3
    batch = a.shape[0] if batched else 1
    M, K = a.shape[-2:]
    N = b.shape[-1]
    out_dtype = np.dtype(out_dtype)
    dsz = out_dtype.itemsize
    per_channel = np.ndim(mult) > 0
    raw = out_dtype in (np.dtype(np.int32), np.dtype(np.float32))  # output stage NONE
    stage = capi.STAGE_NONE if raw else (capi.STAGE_QUANTIZE_DOWN if integer_stage else capi.STAGE_FIXEDPOINT)
    ldd = (N + ldd_pad) * dsz
    desc, keep = capi.make_gemm_desc(
        M, N, K, CODE_OF[a.dtype], CODE_OF[b.dtype], CODE_OF[out_dtype], a_off, b_off, stage,
        multiplier=0 if per_channel else int(mult), shift=0 if per_channel else int(shift),
        multipliers=mult if per_channel else None, shifts=shift if per_channel else None, offset=offset,
        min_bound=lo, max_bound=hi, has_bias=bias is not None, batch=batch, ldd=ldd,
        b_batch_stride=(K * N if b.ndim == 3 else 0), b_constant=b_constant, accumulate=accumulate,
        dequantize_scale=dequantize_scale)
    plan = capi.GemmPlan(ctx, desc, keep)
    try:
        ws = None
        if temp_workspace:  # the caller owns the temporary memory (what a MemoryGroup does for the C++ functions)
            nbytes = plan.temp_bytes
            ws = torch.full((max(nbytes, 1) + 64,), 0x77, dtype=torch.uint8, device="cuda")
            plan.bind_temp(ws, nbytes)
        if force_simt:
            plan.force_simt(True)
        if not pair:
            plan.allow_pair_kernel(False)
        if epi_warps:
            plan.set_epilogue_warps(epi_warps)
        if channel_major:
            plan.set_channel_major(channel_major)
        if tile_columns:
            plan.set_tile_columns(tile_columns)
        if not paired_drain:
            plan.set_paired_drain(False)
        if not saturating_pack:
            plan.set_saturating_pack(False)
        if not tma_store:
            plan.set_tma_store(False)
        da = torch.from_numpy(a.view(np.uint8)).cuda()
        db = torch.from_numpy(b.view(np.uint8)).cuda()
        dbias = torch.from_numpy(np.ascontiguousarray(bias, dtype=np.int32)).cuda() if bias is not None else None
        canary = 0xA5
        # guard regions of canary bytes on both sides of the destination: a store outside the matrix shows up
        guard = 4096
        whole = torch.full((guard + batch * M * ldd + guard,), canary, dtype=torch.uint8, device="cuda")
        dd = whole[guard:guard + batch * M * ldd]
        if dst_init is not None:  # accumulation starts from these values
            init = np.ascontiguousarray(dst_init, dtype=out_dtype).reshape(batch * M, N).view(np.uint8)
            dd.view(batch * M, ldd)[:, :N * dsz] = torch.from_numpy(init).cuda()
        if b_constant:
            plan.prepare(db)
        for _ in range(runs):
            plan.run(da, None if b_constant else db, dbias, dd)
        ctx.sync()
        everything = whole.cpu().numpy()
        assert (everything[:guard] == canary).all() and (everything[-guard:] == canary).all(), \
            "kernel wrote outside the destination matrix"
        raw = everything[guard:-guard].reshape(batch, M, ldd)
        if ldd_pad:
            bad = np.argwhere(raw[:, :, N * dsz:] != canary)
            assert bad.size == 0, f"kernel wrote into the row padding: {len(bad)} bytes, first (batch, row, byte) {bad[:4].tolist()}, bytes past the row {np.unique(bad[:, 2]).tolist()[:32]}"
        out = np.ascontiguousarray(raw[:, :, :N * dsz]).view(out_dtype).reshape(batch, M, N)
        kernel = plan.kernel
        if ws is not None:
            assert (ws[plan.temp_bytes:] == 0x77).all(), "the plan wrote past the bound temporary workspace"
    finally:
        plan.close()
    return (out if batched else out[0]), kernel


# ---- inputs of the committed golden fixtures (outputs live in tests/golden/*.npz) -------------------------
GOLDEN_GEMM_SHAPES = [(1, 1, 1), (21, 13, 33), (23, 31, 37), (32, 72, 4), (1, 129, 257), (130, 1, 40), (72, 33, 47),
                      (33, 67, 133)]
GOLDEN_GEMM_TYPES = [(np.uint8, np.uint8), (np.int8, np.int8), (np.uint8, np.int8)]


def golden_gemm_cases():
    """Yields dicts with the seeded inputs of every GEMMLowp golden case (odd M/N/K as in the reference's
    Small/LargeGEMMLowpDataset: M=1, N=1, K not a multiple of 16 or 32)."""
    for si, (M, N, K) in enumerate(GOLDEN_GEMM_SHAPES):
        for ci, (ad, bd) in enumerate(GOLDEN_GEMM_TYPES):
            r = np.random.default_rng(1000 + 10 * si + ci)
            a, b = q8_uniform(r, (M, K), ad), q8_uniform(r, (K, N), bd)
            ao, bo = int(r.integers(-255, 256)), int(r.integers(-255, 256))
            bias = r.integers(-3000, 3001, N).astype(np.int32)
            mult = r.integers(2 ** 30, 2 ** 31 - 1, N).astype(np.int32)
            shift = r.integers(0, 14, N).astype(np.int32)
            od = np.uint8 if ad == np.uint8 else np.int8
            lo, hi = type_range(od)
            yield dict(key=f"g{si}_{ci}", a=a, b=b, a_off=ao, b_off=bo, bias=bias, mult=mult, shift=shift,
                       out_dtype=od, lo=lo, hi=hi, pt_offset=3, pc_offset=-2)


def golden_int_stage(g):
    """Parameters of the QUANTIZE_DOWN (integer multiply) stage derived from a golden GEMM case: small multipliers,
    shifts in [0, 20), an offset, and bounds inside the type range."""
    r = np.random.default_rng(int(g["key"][1]) * 7 + 3)
    N = g["b"].shape[1]
    mult = r.integers(1, 400, N).astype(np.int32)
    shift = r.integers(8, 20, N).astype(np.int32)
    lo, hi = (20, 230) if g["out_dtype"] == np.uint8 else (-100, 110)
    return mult, shift, 1234, lo, hi


GOLDEN_CONV_GEOMS = [(3, 3, 1, 1, (1, 1, 1, 1)), (1, 1, 1, 1, (0, 0, 0, 0)), (3, 2, 2, 1, (0, 1, 1, 0)),
                     (5, 5, 2, 2, (2, 2, 2, 2)), (3, 3, 2, 2, (0, 1, 0, 1))]
GOLDEN_CONV_TYPES = [(np.uint8, np.uint8, False), (np.uint8, np.int8, True), (np.int8, np.int8, False),
                     (np.int8, np.int8, True)]
GOLDEN_CONV_SCALES = (np.float32(0.03), np.float32(0.4))  # input scale, output scale


def golden_conv_cases():
    """Seeded inputs of the convolution golden cases: NHWC src [2,9,8,C], weights [7,kh,kw,C]."""
    for ci, (kw, kh, sx, sy, pad) in enumerate(GOLDEN_CONV_GEOMS):
        for ti, (sd, wd, pc) in enumerate(GOLDEN_CONV_TYPES):
            r = np.random.default_rng(5000 + 10 * ci + ti)
            B, H, W, Cc, OFM = 2, 9, 8, (16 if ci % 2 == 0 else 5), 7
            src = q8_uniform(r, (B, H, W, Cc), sd)
            wgt = q8_uniform(r, (OFM, kh, kw, Cc), wd, np.iinfo(wd).min + 1)
            bias = r.integers(-500, 501, OFM).astype(np.int32)
            ws = r.uniform(2e-3, 8e-3, OFM if pc else 1).astype(np.float32)
            in_zp = int(r.integers(0, 256)) if sd == np.uint8 else int(r.integers(-128, 128))
            w_zp = 0 if pc else (int(r.integers(0, 256)) if wd == np.uint8 else int(r.integers(-128, 128)))
            out_zp = int(r.integers(0, 40)) if sd == np.uint8 else int(r.integers(-20, 20))
            yield dict(key=f"c{ci}_{ti}", src=src, weights=wgt, bias=bias, w_scales=ws, in_zp=in_zp, w_zp=w_zp,
                       out_zp=out_zp, stride=(sx, sy), pad=pad, kw=kw, kh=kh, per_channel=pc)


def golden_im2col_cases():
    for ci, (kw, kh, sx, sy, pad) in enumerate(GOLDEN_CONV_GEOMS):
        r = np.random.default_rng(7000 + ci)
        src = q8_uniform(r, (2, 9, 8, 16 if ci % 2 == 0 else 5), np.uint8)
        yield dict(key=f"im2col{ci}", src=src, kw=kw, kh=kh, stride=(sx, sy), pad=pad, zp=77)


# ---- QASYMM8 layers (pooling / addition / activation / softmax) -----------------------------------------
# (pool_type, size, stride, pad (l, r, t, b), exclude_padding, global)
GOLDEN_POOL_GEOMS = [
    ("max", (3, 3), (2, 2), (0, 1, 0, 1), False, False),   # ResNet-50 pool1
    ("max", (1, 1), (2, 2), (0, 0, 0, 0), True, False),    # ResNet-50 strided shortcut
    ("max", (2, 2), (2, 2), (0, 0, 0, 0), False, False),
    ("max", (3, 3), (1, 1), (1, 1, 1, 1), False, False),
    ("avg", (3, 3), (1, 1), (1, 1, 1, 1), False, False),
    ("avg", (3, 3), (2, 2), (1, 1, 1, 1), True, False),
    ("avg", (2, 2), (2, 1), (0, 1, 1, 0), False, False),
    ("avg", None, None, None, False, True),                # ResNet-50 pool5
]
GOLDEN_LAYER_QINFOS = [((0.05, 0), (0.05, 0)), ((0.03, 10), (0.07, 3)), ((0.5, 128), (0.25, 0))]
GOLDEN_ADD_QINFOS = [((0.05, 0), (0.05, 0), (0.05, 0)), ((0.03, 5), (0.07, 100), (0.09, 20)),
                     ((0.5, 128), (0.25, 0), (0.3, 7)), ((0.01, 3), (0.02, 250), (0.004, 128))]
GOLDEN_ACTS = [("relu", 0.0, 0.0), ("bounded_relu", 6.0, 0.0), ("lu_bounded_relu", 4.0, -2.0)]


def golden_pool_cases():
    for gi, geom in enumerate(GOLDEN_POOL_GEOMS):
        for si, shape in enumerate([(2, 9, 11, 5), (1, 8, 8, 32), (2, 7, 7, 48)]):
            for qi, (in_q, out_q) in enumerate(GOLDEN_LAYER_QINFOS):
                r = np.random.default_rng(9000 + 100 * gi + 10 * si + qi)
                yield dict(key=f"pool{gi}_{si}_{qi}", src=r.integers(0, 256, shape, dtype=np.uint8), geom=geom,
                           in_q=in_q, out_q=out_q)


def golden_add_cases():
    for qi, qs in enumerate(GOLDEN_ADD_QINFOS):
        for ni, n in enumerate([1, 15, 16, 4099, 65536]):
            r = np.random.default_rng(9500 + 10 * qi + ni)
            yield dict(key=f"add{qi}_{ni}", a=r.integers(0, 256, n, dtype=np.uint8),
                       b=r.integers(0, 256, n, dtype=np.uint8), q=qs)


def golden_act_cases():
    for ai, (act, a, b) in enumerate(GOLDEN_ACTS):
        for qi, (in_q, out_q) in enumerate(GOLDEN_LAYER_QINFOS + [((0.05, 100), (0.03, 80))]):
            r = np.random.default_rng(9700 + 10 * ai + qi)
            src = np.concatenate([np.arange(256, dtype=np.uint8), r.integers(0, 256, 4000 + ai, dtype=np.uint8)])
            yield dict(key=f"act{ai}_{qi}", src=src, act=act, a=a, b=b, in_q=in_q, out_q=out_q)


def golden_softmax_cases():
    for si, (rows, cols, beta, q) in enumerate([(7, 1000, 1.0, (0.05, 0)), (3, 10, 1.0, (0.1, 20)),
                                                (5, 257, 0.5, (0.02, 128)), (1, 1, 1.0, (0.05, 0))]):
        r = np.random.default_rng(9900 + si)
        yield dict(key=f"softmax{si}", src=r.integers(0, 256, (rows, cols), dtype=np.uint8), beta=beta, q=q)


def pool_with(oracle_obj, c):
    pt, size, stride, pad, excl, glob = c["geom"]
    return oracle_obj.pool_nhwc(c["src"], pt, size, stride, pad, c["in_q"], c["out_q"], exclude_padding=excl,
                                global_pool=glob)


# ---- QASYMM8 ResNet-50: the node list of computelibrary_b200.resnet50 interpreted by the CPU oracle ------
def run_graph_oracle(port, nodes, params, x, act_q=(0.05, 0)):
    """x: uint8 [B, image, image, 3].  Returns {node name: uint8 NHWC output}."""
    out = {"input": x}
    for n in nodes:
        src = [out[s] for s in n["inputs"]]
        if n["op"] == "conv":
            p = params[n["name"]]
            out[n["name"]] = port.conv2d_nhwc(src[0], p["weights"], p["bias"], (n["stride"],) * 2, (n["pad"],) * 4,
                                              act_q[1], 0, p["mult"], p["shift"], act_q[1],
                                              act_q[1] if n["relu"] else 0, 255)
        elif n["op"] == "maxpool":
            out[n["name"]] = port.pool_nhwc(src[0], "max", (n["k"],) * 2, (n["stride"],) * 2, n["pad"], act_q, act_q,
                                            exclude_padding=True)
        elif n["op"] == "avgpool_global":
            out[n["name"]] = port.pool_nhwc(src[0], "avg", None, None, None, act_q, act_q, global_pool=True)
        elif n["op"] == "add_relu":
            s = port.add_qasymm8(src[0], src[1], act_q, act_q, act_q)
            out[n["name"]] = port.activation_qasymm8(s, "relu", 0.0, 0.0, act_q, act_q)
        elif n["op"] == "softmax":
            B = src[0].shape[0]
            out[n["name"]] = port.softmax_qasymm8(src[0].reshape(B, -1), 1.0, act_q).reshape(src[0].shape)
        else:
            raise ValueError(n["op"])
    return out
