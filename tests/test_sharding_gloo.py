"""Multi-rank host logic on CPU (gloo, world size 2): row / batch shards need no exchange, column shards are
all-gathered; the assembled result must equal the unsharded oracle result bit for bit."""
import os
import socket

import numpy as np
import pytest

from computelibrary_b200 import sharding


def test_split_even_properties():
    for total in (1, 7, 256, 1000, 4096, 14336):
        for world in (1, 2, 3, 4, 8):
            for align in (1, 16, 256):
                spans = [sharding.split_even(total, world, r, align) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == total
                for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                    assert e0 == b1 and b0 <= e0
                assert all(b % align == 0 or b == total for b, _ in spans)
    assert sharding.column_shard(14336, 8, 3) == (5376, 7168)   # 1792 columns per rank at G = 8
    with pytest.raises(ValueError):
        sharding.split_even(10, 2, 2)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = oracle.port()
    rng = np.random.default_rng(123)  # same data on every rank
    M, K, N = 96, 160, 600
    a = np.clip(np.rint(rng.normal(0, 30, (M, K))), -128, 127).astype(np.int8)
    b = rng.integers(-127, 128, (K, N)).astype(np.int8)
    ws = rng.uniform(1e-3, 5e-3, N).astype(np.float32)
    mult, shift = p.calculate_quantized_multipliers(np.float32(0.02), ws, np.float32(0.05))
    full = p.gemmlowp_fused(a, b, None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    # column sharding + all-gather (config 5)
    n0, n1 = sharding.column_shard(N, world, rank, align=256)
    local = p.gemmlowp_fused(a, np.ascontiguousarray(b[:, n0:n1]), None, 0, 0, mult[n0:n1], shift[n0:n1], 0, -128,
                             127, np.int8)
    got = sharding.allgather_columns(torch.from_numpy(local), N, world, rank, align=256).numpy()
    ok_cols = np.array_equal(got, full)
    # row sharding (config 2): no collective; every rank checks its own rows
    m0, m1 = sharding.row_shard(M, world, rank)
    rows = p.gemmlowp_fused(a[m0:m1], b, None, 0, 0, mult, shift, 0, -128, 127, np.int8)
    ok_rows = np.array_equal(rows, full[m0:m1])
    flags = torch.tensor([int(ok_cols), int(ok_rows)])
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{int(flags[0])} {int(flags[1])}")
    dist.destroy_process_group()


def test_column_and_row_sharding_two_ranks(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "result.txt").read_text() == "1 1"
