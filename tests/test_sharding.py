"""Row sharding of a quantised linear over ranks: partition arithmetic, raw-byte slicing and the
all-gather, run as world_size-2 (and 3) gloo process groups on CPU. The per-rank product is the CPU
checker, so the assembled result must equal the unsharded checker result bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_partition_covers_rows_once():
    from zignn_b200 import sharding
    for out_dim in (1, 15, 16, 17, 768, 50257, 262144):
        for world in (1, 2, 3, 4, 8):
            per = sharding.rows_per_rank(out_dim, world)
            assert per % sharding.ROW_ALIGN == 0 and per * world >= out_dim
            covered = []
            for r in range(world):
                lo, hi = sharding.row_range(out_dim, world, r)
                assert 0 <= lo <= hi <= out_dim and hi - lo <= per
                assert lo == min(r * per, out_dim)
                covered.extend(range(lo, hi)) if out_dim <= 1024 else covered.append((lo, hi))
            if out_dim <= 1024:
                assert covered == list(range(out_dim))
            else:
                assert covered[0][0] == 0 and covered[-1][1] == out_dim
                assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    with pytest.raises(ValueError):
        sharding.row_range(10, 2, 2)


def test_slice_rows_matches_block_geometry():
    from zignn_b200 import ggml, sharding
    for qt in (ggml.Q4_0, ggml.Q4_1, ggml.Q8_0):
        n, k = 40, 96
        raw = torch.arange(ggml.tensor_bytes(qt, n * k), dtype=torch.int64).to(torch.uint8)
        rb = ggml.tensor_bytes(qt, k)
        part = sharding.slice_rows(raw, qt, n, k, 16, 32)
        assert part.numel() == 16 * rb and torch.equal(part, raw[16 * rb:32 * rb])
        assert sharding.slice_rows(raw, qt, n, k, 40, 40).numel() == 0
        with pytest.raises(ValueError):
            sharding.slice_rows(raw[:-1], qt, n, k, 0, 1)
        with pytest.raises(ValueError):
            sharding.slice_rows(raw, qt, n, k, 8, 41)
    with pytest.raises(ValueError):
        sharding.slice_rows(torch.zeros(10, dtype=torch.uint8), ggml.Q4_0, 1, 48, 0, 1)


def _worker(rank, world, port, out_dim, in_dim, qt, m, act_mode, result_path):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import torch.distributed as dist
    import oracle
    from zignn_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # every rank draws the same full weight, as bench.py does
        w = (rng.standard_normal((out_dim, in_dim)) * 0.02).astype(np.float32)
        raw = oracle.quantize(qt, w)
        x = rng.standard_normal((m, in_dim)).astype(np.float32)

        def make_weight(part, t, rows, k):
            return part.numpy()

        def compute(xt, wpart, out):
            out.copy_(torch.from_numpy(oracle.linear(qt, wpart, xt.numpy(), out.shape[1], in_dim, act_mode)))

        lin = sharding.ShardedQuantLinear(torch.from_numpy(raw), qt, out_dim, in_dim, make_weight, compute)
        assert (lin.lo, lin.hi) == sharding.row_range(out_dim, world, rank)
        y = lin.forward(torch.from_numpy(x))
        full = oracle.linear(qt, raw, x, out_dim, in_dim, act_mode)
        assert y.shape == (m, out_dim)
        assert np.array_equal(y.numpy(), full), "rank %d: sharded result differs" % rank
        # a second call reuses the gather buffer
        y2 = lin.forward(torch.from_numpy(x))
        assert np.array_equal(y2.numpy(), full)
        if rank == 0:
            with open(result_path, "w") as f:
                f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,out_dim,m,act_mode", [
    (2, 96, 1, 0),     # even split
    (2, 100, 3, 1),    # ragged: rank 1 owns fewer rows, several activation rows, Q8 activations
    (3, 40, 2, 0),     # a rank with very few rows (48 per... 16-row alignment leaves rank 2 with 8)
    (2, 16, 1, 0),     # rank 1 owns nothing
])
def test_sharded_linear_gloo(tmp_path, oracle, world, out_dim, m, act_mode):
    from zignn_b200 import ggml
    result = tmp_path / "ok.txt"
    for qt in (ggml.Q4_0, ggml.Q8_0):
        if result.exists():
            result.unlink()
        mp.spawn(_worker, args=(world, _free_port(), out_dim, 64, qt, m, act_mode, str(result)), nprocs=world,
                 join=True)
        assert result.read_text() == "ok"
