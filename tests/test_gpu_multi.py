"""Row-sharded linear on two GPUs: the library's peer-store all-gather against NCCL's and against
the unsharded product. Needs two CUDA devices; skipped otherwise (the single-GPU run collects it)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dim, in_dim, m, result_path):
    sys.path.insert(0, REPO)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    import zignn_b200
    from zignn_b200 import api as zq, ggml, sharding
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator(device="cuda").manual_seed(11)  # same stream on every rank
        w = torch.randn(out_dim, in_dim, generator=g, device="cuda") * 0.02
        x = torch.randn(m, in_dim, generator=g, device="cuda")
        for qt in (ggml.Q4_0, ggml.Q8_0):
            raw = ggml.quantize(qt, w)
            full = zq.quant_matmul_no_grad(x, zq.QuantWeight(raw, qt, out_dim, in_dim))
            nccl = sharding.cuda_sharded_linear(raw, qt, out_dim, in_dim, gather="nccl")
            want = nccl.forward(x).clone()
            for tagged in (True, False):  # the fused exchange: words carrying the round number / counters after a fence
                peer = sharding.cuda_sharded_linear(raw, qt, out_dim, in_dim, gather="peer", m_rows=m)
                peer.peer.tagged = peer.peer.tagged and tagged
                for it in range(5):  # both result buffers, growing round numbers
                    got = peer.forward(x + float(it)) if it else peer.forward(x)
                    ref = nccl.forward(x + float(it)) if it else want
                    torch.cuda.synchronize()
                    if peer.fused:
                        # the fused kernel keeps whole rows per warp; the plain shard GEMV may split K over
                        # warps: same products, another summation order
                        e = float((got - ref).norm() / ref.norm())
                        assert e <= 2e-6, "rank %d type %d round %d: %g" % (rank, qt, it, e)
                    else:
                        assert torch.equal(got, ref), "rank %d type %d round %d" % (rank, qt, it)
            err = (want - full).norm() / full.norm()
            assert float(err) <= 2e-6, float(err)
            # the tagged exchange writing the gathered row straight into page-locked host memory
            if m == 1:
                tagged = sharding.cuda_sharded_linear(raw, qt, out_dim, in_dim, gather="peer", m_rows=1)
                ref = tagged.forward(x).clone()
                if tagged.fused and tagged.peer.tagged:
                    host_row = torch.zeros(tagged.world * tagged.per, dtype=torch.float32).pin_memory()
                    for it in range(3):
                        tagged.forward(x, out=host_row)
                        torch.cuda.synchronize()
                        assert torch.equal(host_row[:out_dim], ref[0].cpu()), (rank, qt, it)
                        host_row.zero_()
                    assert torch.equal(tagged.forward(x), ref)  # the library's own buffers still take their turns
            # greedy decoding: only the index of the first largest output crosses NVLink
            if m == 1:
                for it in range(4):
                    xi = x + float(it)
                    idx, val = peer.greedy(xi)
                    idx, val = idx.clone(), val.clone()
                    ref = peer.forward(xi).clone()  # the same kernel's rows: the same values bit for bit
                    torch.cuda.synchronize()
                    best = ref[0].max()
                    assert int(idx.item()) == int(torch.nonzero(ref[0] == best)[0, 0].item()), (rank, qt, it)
                    assert float(val.item()) == float(best.item())
        from zignn_b200 import _lib
        import ctypes as C
        v = C.c_uint()
        _lib.check(_lib.load().zq_device_error(C.byref(v), 0))
        assert v.value == 0, hex(v.value)
        dist.barrier()
        if rank == 0:
            with open(result_path, "w") as f:
                f.write("ok fused" if peer.fused else "ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("out_dim,m", [(4096, 1), (1000, 3), (2 * 148 * 8 * 16, 1)])  # small, ragged, fused-kernel size
def test_peer_gather_matches_nccl_two_gpus(tmp_path, out_dim, m):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    result = tmp_path / "ok.txt"
    mp.spawn(_worker, args=(2, _free_port(), out_dim, 1152, m, str(result)), nprocs=2, join=True)
    assert result.read_text() == ("ok fused" if out_dim >= 2 * 148 * 8 * 16 and m == 1 else "ok")
