"""QASYMM8 ResNet-50 (computelibrary_b200.resnet50): topology facts on CPU; on the GPU every node of a reduced
-size network (64x64 images, batch 2) against the CPU oracle interpreting the same node list, bit for bit
(softmax within one step)."""
import numpy as np
import pytest

from helpers import run_graph_oracle


def test_topology_matches_reference_example():
    from computelibrary_b200 import resnet50 as rn
    g = rn.build_graph()
    convs = [n for n in g if n["op"] == "conv"]
    assert len(convs) == 54                                   # 1 + 3*3+1 + 4*3+1 + 6*3+1 + 3*3+1 + logits
    assert abs(rn.graph_ops(g) - 6.96451072e9) < 1            # 3.482 GMAC per 224x224 image
    by = {n["name"]: n for n in g}
    assert by["conv1"]["out_shape"] == (112, 112, 64) and by["pool1"]["out_shape"] == (56, 56, 64)
    assert by["block1/unit3/conv2"]["stride"] == 2 and by["block1/unit3/add"]["out_shape"] == (28, 28, 256)
    assert by["block1/unit3/shortcut_pool"]["k"] == 1 and by["block1/unit3/shortcut_pool"]["stride"] == 2
    assert by["block4/unit3/conv2"]["stride"] == 1 and by["block4/unit3/add"]["out_shape"] == (7, 7, 2048)
    assert by["block2/unit1/shortcut"]["ofm"] == 512 and by["block2/unit2/add"]["inputs"][0] == "block2/unit1/add"
    assert by["logits"]["in_shape"] == (1, 1, 2048) and by["softmax"]["out_shape"] == (1, 1, 1000)
    assert sum(1 for n in g if n["op"] == "add_relu") == 16


def test_synthetic_params_are_seeded():
    from computelibrary_b200 import resnet50 as rn
    g = rn.build_graph(64, 10)
    a, b, c = rn.synthetic_params(g, 1), rn.synthetic_params(g, 1), rn.synthetic_params(g, 2)
    assert all(np.array_equal(a[k]["weights"], b[k]["weights"]) and np.array_equal(a[k]["mult"], b[k]["mult"]) for k in a)
    assert not np.array_equal(a["conv1"]["weights"], c["conv1"]["weights"])
    assert a["conv1"]["weights"].shape == (64, 7, 7, 3) and a["conv1"]["weights"].dtype == np.int8
    assert a["logits"]["bias"].shape == (10,) and int(a["conv1"]["shift"].min()) >= 0


@pytest.mark.gpu
@pytest.mark.parametrize("fuse_residual", [False, True])
@pytest.mark.parametrize("fan_in_scaled", [False, True])
def test_reduced_network_vs_oracle(ctx, port, fan_in_scaled, fuse_residual):
    import torch
    from computelibrary_b200 import resnet50 as rn
    g = rn.build_graph(64, 100)
    params = rn.synthetic_params(g, seed=3, fan_in_scaled=fan_in_scaled)
    x = np.random.default_rng(17).integers(0, 256, (2, 64, 64, 3), dtype=np.uint8)
    want = run_graph_oracle(port, g, params, x)
    net = rn.ResNet50(ctx, 2, params=params, nodes=g, fuse_residual=fuse_residual)
    assert len(net.fused) == (16 if fuse_residual else 0)
    net.run(torch.from_numpy(x).cuda())
    ctx.sync()
    for n in g:
        if n["name"] in net.fused:   # absorbed into the addition that follows: its own tensor is never written
            continue
        got = net.bufs[n["name"]].cpu().numpy()
        if n["op"] == "softmax":
            assert np.abs(got.astype(np.int32) - want[n["name"]].astype(np.int32)).max() <= 1
        else:
            np.testing.assert_array_equal(got, want[n["name"]], err_msg=n["name"])
    if fan_in_scaled:   # the twin exists so that deep layers carry mid-range values, not only 0 / 255
        deep = want["block3/unit2/add"]
        assert 0.02 < np.mean((deep > 0) & (deep < 255))
    assert net.launches >= len(g) - len(net.fused)
    net.close()


@pytest.mark.gpu
def test_graph_replay_equals_eager(port):
    """The node list captured into one CUDA graph gives the bytes of the eager pass, also on new images."""
    import torch
    import computelibrary_b200 as cl
    from computelibrary_b200 import resnet50 as rn
    torch.cuda.set_device(0)
    work = torch.cuda.Stream()
    ctx = cl.Context(0, work.cuda_stream)
    g = rn.build_graph(64, 100)
    params = rn.synthetic_params(g, seed=5, fan_in_scaled=True)
    rng = np.random.default_rng(23)
    x0, x1 = (rng.integers(0, 256, (2, 64, 64, 3), dtype=np.uint8) for _ in range(2))
    with torch.cuda.stream(work):
        net = rn.ResNet50(ctx, 2, params=params, nodes=g)
        d_in = torch.from_numpy(x0).cuda()
        graph = net.capture(d_in, work)
        for x in (x0, x1):
            d_in.copy_(torch.from_numpy(x).cuda())
            graph.replay()
            ctx.sync()
            got = {k: net.bufs[k].cpu().numpy() for k in ("block2/unit1/add", "logits")}
            want = run_graph_oracle(port, g, params, x)
            for k in got:
                np.testing.assert_array_equal(got[k], want[k], err_msg=k)
    net.close()
    ctx.close()


@pytest.mark.gpu
def test_full_size_network_vs_oracle_and_batch_invariance(ctx, port):
    """Config 4 at its real geometry (224x224x3, 1000 classes) on the specified parameter distribution: batch 3
    against the oracle node by node for the tensors that matter downstream, and the size-independent property
    the sharding relies on -- an image's result does not depend on which batch (rank) it travels in."""
    import torch
    from computelibrary_b200 import resnet50 as rn
    g = rn.build_graph(224, 1000)
    params = rn.synthetic_params(g, seed=1)
    x = np.random.default_rng(31).integers(0, 256, (3, 224, 224, 3), dtype=np.uint8)
    net = rn.ResNet50(ctx, 3, params=params, nodes=g)
    net.run(torch.from_numpy(x).cuda())
    ctx.sync()
    want = run_graph_oracle(port, g, params, x)
    for name in ("conv1", "pool1", "block1/unit1/add", "block1/unit3/add", "block2/unit4/add", "block3/unit6/add",
                 "block4/unit3/add", "pool5", "logits"):
        np.testing.assert_array_equal(net.bufs[name].cpu().numpy(), want[name], err_msg=name)
    sm = net.bufs["softmax"].cpu().numpy().astype(np.int32)
    assert np.abs(sm - want["softmax"].astype(np.int32)).max() <= 1
    full_logits = net.bufs["logits"].cpu().numpy().copy()
    net.close()
    single = rn.ResNet50(ctx, 1, params=params, nodes=g)
    for i in (0, 2):
        single.run(torch.from_numpy(x[i:i + 1]).cuda())
        ctx.sync()
        np.testing.assert_array_equal(single.bufs["logits"].cpu().numpy()[0], full_logits[i])
    single.close()
