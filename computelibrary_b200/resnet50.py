"""QASYMM8 ResNet-50 v1 on the cugl C ABI.

The topology is that of Compute Library's ``examples/graph_resnet50.cpp`` (lines 80-121 and
``add_residual_block``, 141-240): conv1 7x7/2 -> max-pool 3x3/2 (pad 0,1,0,1) -> four blocks of bottleneck
units (64 x3, 128 x4, 256 x6, 512 x3; the LAST unit of blocks 1-3 strides its 3x3 convolution by 2 and
sub-samples its shortcut with a 1x1/2 max-pool; the first unit of every block has a 1x1 shortcut
convolution) -> global average pool -> 1x1 "logits" convolution -> flatten -> softmax.  As in the library's
own synthetic-type mode the batch normalisations are folded away (their shift becomes the convolution
bias) and every ReLU that follows a convolution is the clamp of its output stage.

``build_graph`` returns the node list (pure data, no GPU needed); ``synthetic_params`` draws seeded
weights; ``ResNet50`` turns the nodes into cugl plans and runs them in order on one GPU.  The same node list
is interpreted by the CPU oracle in the tests.
"""
from __future__ import annotations

import numpy as np

from . import capi

ACT_Q = (0.05, 0)            # quantization of every activation tensor, input image included
SOFTMAX_Q = (1.0 / 256, 0)   # fixed by the library for QASYMM8 softmax (src/core/Utils.cpp:421-439)


def build_graph(image: int = 224, num_classes: int = 1000):
    """Node list in execution order.  Every node: name, op, inputs (names), out shape (H, W, C) and
    op-specific fields.  ops: conv, maxpool, avgpool_global, add_relu, softmax."""
    nodes = []
    shapes = {"input": (image, image, 3)}

    def conv(name, src, ofm, k, stride, pad, relu):
        H, W, Cc = shapes[src]
        Ho = (H + 2 * pad - k) // stride + 1
        Wo = (W + 2 * pad - k) // stride + 1
        shapes[name] = (Ho, Wo, ofm)
        nodes.append(dict(name=name, op="conv", inputs=[src], ofm=ofm, k=k, stride=stride, pad=pad, relu=relu,
                          in_shape=(H, W, Cc), out_shape=shapes[name]))
        return name

    def maxpool(name, src, k, stride, pad):
        H, W, Cc = shapes[src]
        Ho = (H + pad[2] + pad[3] - k) // stride + 1
        Wo = (W + pad[0] + pad[1] - k) // stride + 1
        shapes[name] = (Ho, Wo, Cc)
        nodes.append(dict(name=name, op="maxpool", inputs=[src], k=k, stride=stride, pad=pad,
                          in_shape=(H, W, Cc), out_shape=shapes[name]))
        return name

    x = conv("conv1", "input", 64, 7, 2, 3, True)
    x = maxpool("pool1", x, 3, 2, (0, 1, 0, 1))
    for bi, (base, units, stride) in enumerate([(64, 3, 2), (128, 4, 2), (256, 6, 2), (512, 3, 1)], start=1):
        for ui in range(units):
            p = f"block{bi}/unit{ui + 1}/"
            middle = stride if ui == units - 1 else 1
            r = conv(p + "conv1", x, base, 1, 1, 0, True)
            r = conv(p + "conv2", r, base, 3, middle, 1, True)
            r = conv(p + "conv3", r, base * 4, 1, 1, 0, False)
            if ui == 0:
                left = conv(p + "shortcut", x, base * 4, 1, 1, 0, False)
            elif middle > 1:
                left = maxpool(p + "shortcut_pool", x, 1, middle, (0, 0, 0, 0))
            else:
                left = x
            shapes[p + "add"] = shapes[r]
            nodes.append(dict(name=p + "add", op="add_relu", inputs=[left, r], in_shape=shapes[r], out_shape=shapes[r]))
            x = p + "add"
    H, W, Cc = shapes[x]
    shapes["pool5"] = (1, 1, Cc)
    nodes.append(dict(name="pool5", op="avgpool_global", inputs=[x], in_shape=(H, W, Cc), out_shape=(1, 1, Cc)))
    x = conv("logits", "pool5", num_classes, 1, 1, 0, False)
    shapes["softmax"] = shapes[x]
    nodes.append(dict(name="softmax", op="softmax", inputs=[x], in_shape=shapes[x], out_shape=shapes[x]))
    return nodes


def graph_ops(nodes) -> float:
    """2 * MACs of all convolutions per image."""
    return float(sum(2.0 * n["out_shape"][0] * n["out_shape"][1] * n["ofm"] * n["k"] * n["k"] * n["in_shape"][2]
                     for n in nodes if n["op"] == "conv"))


def graph_bytes(nodes) -> float:
    """Bytes per image a layer-by-layer run has to move at least: every node reads its inputs and writes its output
    once (8-bit activations), the convolutions also read their weights once per batch (not counted per image)."""
    total = 0.0
    for n in nodes:
        ho, wo, co = n["out_shape"]
        hi, wi, ci = n["in_shape"]
        total += ho * wo * co                      # output written
        total += hi * wi * ci * len(n["inputs"])   # inputs read (the two operands of an addition have equal shapes)
    return float(total)


def synthetic_params(nodes, seed: int = 1, scale_range=(1e-3, 1e-2), bias_range: int = 5000, fan_in_scaled=False):
    """Seeded random parameters per convolution: int8 weights U[-127,127] [OFM,kh,kw,C], per-channel scales
    log-uniform in ``scale_range``, int32 bias U[-bias_range, bias_range].  ``fan_in_scaled`` divides the scales
    by sqrt(K)/8 so that deep stacks neither saturate nor die (used by the parity tests next to the plain
    distribution)."""
    params = {}
    for i, n in enumerate(nodes):
        if n["op"] != "conv":
            continue
        rng = np.random.default_rng(seed * 1000 + i)
        k, Cc, ofm = n["k"], n["in_shape"][2], n["ofm"]
        w = rng.integers(-127, 128, (ofm, k, k, Cc), dtype=np.int8)
        s = np.exp(rng.uniform(np.log(scale_range[0]), np.log(scale_range[1]), ofm)).astype(np.float32)
        if fan_in_scaled:
            s = (s / np.float32(np.sqrt(k * k * Cc) / 8.0)).astype(np.float32)
        b = rng.integers(-bias_range, bias_range + 1, ofm).astype(np.int32)
        mult, shift = capi.calculate_quantized_multipliers(ACT_Q[0], s, ACT_Q[0])
        params[n["name"]] = dict(weights=w, w_scales=s, bias=b, mult=mult, shift=shift)
    return params


class ResNet50:
    """One GPU's copy of the network: plans, device weights and activation buffers for a fixed batch."""

    def __init__(self, ctx: capi.Context, batch: int, params=None, image: int = 224, num_classes: int = 1000,
                 seed: int = 1, nodes=None, fuse_residual: bool = True):
        """``fuse_residual``: compute every ``add_relu`` node inside the epilogue of the convolution that produces
        its right-hand input (cugl_conv2d_run_residual); the convolution's own buffer is then never written."""
        import torch
        self.ctx, self.batch = ctx, batch
        self.fuse_residual = fuse_residual
        self.nodes = nodes if nodes is not None else build_graph(image, num_classes)
        self.params = params if params is not None else synthetic_params(self.nodes, seed)
        self.image = self.nodes[0]["in_shape"][0]
        self.steps = []      # (callable, launches)
        self.bufs = {}
        self._keep = []
        dev = torch.device("cuda", torch.cuda.current_device())
        for n in self.nodes:
            H, W, Cc = n["out_shape"]
            self.bufs[n["name"]] = torch.empty((batch, H, W, Cc), dtype=torch.uint8, device=dev)
        # a convolution whose only consumer is an add_relu node can absorb it, provided the other input of the
        # addition is produced earlier in the list (the shortcut convolution is moved ahead of it for that)
        order = list(self.nodes)
        self.fused = {}
        if fuse_residual:
            consumers = {}
            for n in order:
                for s in n["inputs"]:
                    consumers.setdefault(s, []).append(n["name"])
            by_name = {n["name"]: n for n in order}
            for add in [n for n in order if n["op"] == "add_relu"]:
                left, right = add["inputs"]
                conv = by_name.get(right)
                if conv is None or conv["op"] != "conv" or consumers[right] != [add["name"]]:
                    continue
                li, ci = (order.index(by_name[left]) if left in by_name else -1), order.index(conv)
                if li > ci:   # shortcut after the convolution: run it first (it does not depend on conv)
                    ln = order.pop(li)
                    order.insert(ci, ln)
                self.fused[conv["name"]] = add
        self.order = order
        for n in order:
            if n["op"] == "add_relu" and any(f is n for f in self.fused.values()):
                continue
            self._add_step(n, torch, dev)
        ctx.sync()

    def _add_step(self, n, torch, dev):
        ctx, B = self.ctx, self.batch
        H, W, Cc = n["in_shape"]
        dst = self.bufs[n["name"]]
        srcs = [None if s == "input" else self.bufs[s] for s in n["inputs"]]
        if n["op"] == "conv":
            p = self.params[n["name"]]
            desc, keep = capi.make_conv_desc(
                B, H, W, Cc, n["ofm"], n["k"], n["k"], (n["stride"],) * 2, (n["pad"],) * 4, (1, 1), capi.U8, capi.S8,
                ACT_Q[1], 0, multipliers=p["mult"], shifts=p["shift"], dst_zp=ACT_Q[1],
                min_bound=ACT_Q[1] if n["relu"] else 0, max_bound=255)
            plan = capi.ConvPlan(ctx, desc, keep)
            d_w = torch.from_numpy(p["weights"].view(np.uint8)).to(dev)
            d_b = torch.from_numpy(p["bias"]).to(dev)
            plan.prepare(d_w)
            self._keep += [plan, d_b]
            is_input = srcs[0] is None
            add = self.fused.get(n["name"])
            if add is not None:
                try:
                    plan.set_residual(ACT_Q[0], ACT_Q, ACT_Q, act=capi.ACT_RELU)
                except capi.CuglError:
                    add = None   # not a saturating addition for these quantizations: keep the separate kernel
                    del self.fused[n["name"]]
            if add is not None:
                res = self.bufs[[s for s in add["inputs"] if s != n["name"]][0]]
                out = self.bufs[add["name"]]
                self.steps.append((lambda x, plan=plan, d_b=d_b, out=out, s=srcs[0], res=res:
                                   plan.run_residual(s, d_b, res, out), plan, dict(n, name=n["name"] + "+add")))
            else:
                self.steps.append((lambda x, plan=plan, d_b=d_b, dst=dst, s=srcs[0], is_input=is_input:
                                   plan.run(x if is_input else s, d_b, dst), plan, n))
        elif n["op"] == "maxpool":
            desc = capi.make_pool_desc(B, H, W, Cc, capi.POOL_MAX, (n["k"],) * 2, (n["stride"],) * 2, n["pad"], ACT_Q, ACT_Q,
                                       exclude_padding=True)
            self.steps.append((lambda x, desc=desc, s=srcs[0], dst=dst: ctx.pool2d_nhwc(desc, s, dst), None, n))
        elif n["op"] == "avgpool_global":
            desc = capi.make_pool_desc(B, H, W, Cc, capi.POOL_AVG, in_q=ACT_Q, out_q=ACT_Q, global_pool=True)
            self.steps.append((lambda x, desc=desc, s=srcs[0], dst=dst: ctx.pool2d_nhwc(desc, s, dst), None, n))
        elif n["op"] == "add_relu":
            cnt = dst.numel()
            self.steps.append((lambda x, a=srcs[0], b=srcs[1], dst=dst, cnt=cnt:
                               ctx.add_qasymm8(a, b, dst, cnt, ACT_Q, ACT_Q, ACT_Q, act=capi.ACT_RELU), None, n))
        elif n["op"] == "softmax":
            cols = Cc * H * W
            self.steps.append((lambda x, s=srcs[0], dst=dst, cols=cols:
                               ctx.softmax_qasymm8(s, dst, B, cols, 1.0, ACT_Q), None, n))
        else:
            raise ValueError(n["op"])

    @property
    def launches(self) -> int:
        return sum(plan.launches if plan is not None else 1 for _, plan, _ in self.steps)

    def run(self, d_input):
        """d_input: uint8 [batch, image, image, 3] on the device.  Returns the softmax buffer (uint8 [batch,1,1,classes]);
        enqueues only, like every cugl run."""
        for fn, _, _ in self.steps:
            fn(d_input)
        return self.bufs["softmax"]

    def capture(self, d_input, torch_stream):
        """Records one pass over ``d_input`` into a CUDA graph and returns it (``graph.replay()`` re-runs the whole
        network with one launch; new images are copied into ``d_input`` beforehand).  ``torch_stream`` must be the
        torch stream the context was created on, and not the default stream.  One eager pass runs first so that
        nothing allocates or sets kernel attributes while the stream is capturing."""
        import torch
        assert torch_stream.cuda_stream == self.ctx.stream and torch_stream.cuda_stream != 0
        with torch.cuda.stream(torch_stream):
            self.run(d_input)
        self.ctx.sync()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=torch_stream):
            self.run(d_input)
        return graph

    def run_timed(self, d_input, stream=None):
        """Runs once with a CUDA event pair around every node; returns [(name, op, kernel, ms)].  ``stream`` is the
        torch stream the context enqueues on (default: torch's current stream)."""
        import torch
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(self.steps) + 1)]
        stream = stream if stream is not None else torch.cuda.current_stream()
        ev[0].record(stream)
        for i, (fn, _, _) in enumerate(self.steps):
            fn(d_input)
            ev[i + 1].record(stream)
        self.ctx.sync()
        return [(n["name"], n["op"], plan.kernel if plan is not None else n["op"], ev[i].elapsed_time(ev[i + 1]))
                for i, (_, plan, n) in enumerate(self.steps)]

    def close(self):
        for k in self._keep:
            if hasattr(k, "close"):
                k.close()
        self._keep = []
