"""Failure paths that must end with a status, not with a hang: a device-side wait that runs out, a missing
peer pointer, a many-row call without its workspace. Every wait here is bounded by a small poll count set
through zq_set_wait_limit; nothing faults, traps or spins for long."""
import ctypes as C

import numpy as np
import pytest
import torch

from zignn_b200 import ggml

pytestmark = pytest.mark.gpu

GATH = int.from_bytes(b"GATH", "big")
FGAT = int.from_bytes(b"FGAT", "big")


def ptr_array(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_peer_gather_wait_runs_out_and_the_library_stays_usable(zq):
    """world = 2 on ONE GPU: the 'peer' is a second local buffer whose owner never shows up, so the flag this
    rank waits for is never advanced. With a limit of 1024 polls the kernel returns, the device error word reads
    'GATH', zq_device_check reports ZQ_ERR_TIMEOUT once, and later calls work."""
    from zignn_b200 import _lib
    lib = _lib.load()
    assert _lib.device_error(clear=True) in (0, GATH, FGAT)
    n = 4096
    y = [torch.zeros(2 * n, device="cuda") for _ in range(2)]       # result buffers of rank 0 and of the absent rank 1
    flags = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(2)]
    y[0][:n] = 1.0
    lib.zq_set_wait_limit(1024)
    try:
        rc = lib.zq_peer_gather(ptr_array(y), ptr_array(flags), 2, 0, 0, n, 1, stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.all(y[1][:n] == 1.0)               # the slice was pushed to the peer's buffer
        assert int(flags[1][0].item()) == 8             # and published there (8 CTAs per peer)
        assert _lib.device_error(clear=False) == GATH   # the wait for the peer's slice gave up
        assert lib.zq_device_check(1) == 7              # ZQ_ERR_TIMEOUT, cleared by the call
        assert lib.zq_device_check(0) == 0
        # the same exchange with the peer's arrival supplied by hand completes without an error
        flags[0][1] = 16
        rc = lib.zq_peer_gather(ptr_array(y), ptr_array(flags), 2, 0, 0, n, 2, stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert lib.zq_device_check(1) == 0
    finally:
        lib.zq_set_wait_limit(0)
    # a missing peer pointer is a set-up error, reported before anything is launched
    bad = (C.c_void_p * 2)(y[0].data_ptr(), None)
    assert lib.zq_peer_gather(bad, ptr_array(flags), 2, 0, 0, n, 3, stream()) == 8  # ZQ_ERR_PEER


def test_fused_gather_wait_runs_out(zq, oracle):
    """The exchange fused into the GEMV epilogue, same set-up: the result rows are correct in this rank's own
    buffer and in the 'peer' buffer, the wait for the absent peer ends after the poll limit with 'FGAT'."""
    from zignn_b200 import _lib
    lib = _lib.load()
    _lib.device_error(clear=True)
    n, k = 148 * 2 * 8 * 16, 1152  # enough row tiles for the whole-rows kernel
    rng = np.random.default_rng(1)
    raw = oracle.quantize(ggml.Q4_0, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    qw = zq.QuantWeight(raw, ggml.Q4_0, n, k)
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float32)).cuda()
    want = zq.quant_matmul_no_grad(x, qw).reshape(-1)
    odd = [torch.zeros(2 * n, device="cuda") for _ in range(2)]
    even = [torch.zeros(2 * n, device="cuda") for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(2)]
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")
    lib.zq_set_wait_limit(1024)
    try:
        rc = lib.zq_matmul_gather(qw.handle, C.c_void_p(x.data_ptr()), None, ptr_array(odd), ptr_array(even),
                                  ptr_array(flags), 2, 0, 0, C.c_void_p(sync.data_ptr()), stream())
        assert rc == 0
        torch.cuda.synchronize()
        for buf in (odd[0], odd[1]):  # round 1 uses the odd buffers: this rank's own and the peer's
            assert torch.allclose(buf[:n], want, rtol=1e-5, atol=1e-7)
        assert _lib.device_error(clear=False) == FGAT
        assert lib.zq_device_check(1) == 7
    finally:
        lib.zq_set_wait_limit(0)
    assert torch.equal(zq.quant_matmul_no_grad(x, qw).reshape(-1), want)  # the library still works


def test_tagged_gather_wait_runs_out_and_completes_when_the_words_are_there(zq, oracle):
    """The tagged exchange (64-bit words carrying the round number), both 'ranks' on this GPU and no second rank
    running: round 1 stores this rank's rows and their words, the poll of the absent rank's words ends after the
    limit with 'FGAT'. Then the absent rank's words of round 2 are written by hand: round 2 completes without an
    error and unpacks them."""
    from zignn_b200 import _lib
    lib = _lib.load()
    _lib.device_error(clear=True)
    n, k = 148 * 2 * 8 * 16, 1152
    rng = np.random.default_rng(4)
    raw = oracle.quantize(ggml.Q4_0, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    qw = zq.QuantWeight(raw, ggml.Q4_0, n, k)
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float32)).cuda()
    want = zq.quant_matmul_no_grad(x, qw).reshape(-1)
    inbox_odd = [torch.zeros(2 * n, dtype=torch.int64, device="cuda") for _ in range(2)]
    inbox_even = [torch.zeros(2 * n, dtype=torch.int64, device="cuda") for _ in range(2)]
    y_odd, y_even = torch.zeros(2 * n, device="cuda"), torch.zeros(2 * n, device="cuda")
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")

    def call():
        return lib.zq_matmul_gather_tagged(qw.handle, C.c_void_p(x.data_ptr()), None, ptr_array(inbox_odd),
                                           ptr_array(inbox_even), C.c_void_p(y_odd.data_ptr()), C.c_void_p(y_even.data_ptr()),
                                           2, 0, C.c_void_p(sync.data_ptr()), stream())

    lib.zq_set_wait_limit(1024)
    try:
        assert call() == 0
        torch.cuda.synchronize()
        assert torch.allclose(y_odd[:n], want, rtol=1e-5, atol=1e-7)        # this rank's own rows
        words = inbox_odd[1][:n]                                             # what the 'peer' received
        assert torch.all((words >> 32) == 1)
        assert torch.equal((words & 0xFFFFFFFF).to(torch.int32).view(torch.float32), y_odd[:n])
        assert _lib.device_error(clear=False) == FGAT
        assert lib.zq_device_check(1) == 7
        assert int(sync[0].item()) == 1 and int(sync[1].item()) == 0        # the round still closed
        # round 2: the other rank's words are in this rank's even inbox before the call
        theirs = torch.arange(n, device="cuda", dtype=torch.float32) * 0.5
        inbox_even[0][n:] = (theirs.view(torch.int32).to(torch.int64) & 0xFFFFFFFF) | (2 << 32)
        assert call() == 0
        torch.cuda.synchronize()
        assert lib.zq_device_check(1) == 0
        assert torch.allclose(y_even[:n], want, rtol=1e-5, atol=1e-7)
        assert torch.equal(y_even[n:], theirs)
    finally:
        lib.zq_set_wait_limit(0)


def test_column_gather_on_one_gpu(zq):
    """zq_peer_gather_cols_step with both 'ranks' on this GPU: rank 1's [m][cols] block lands in columns
    [cols, 2 cols) of both row-major result buffers; nobody plays rank 0, so the wait ends with 'GATH'."""
    from zignn_b200 import _lib
    lib = _lib.load()
    _lib.device_error(clear=True)
    m, cols = 37, 200
    local = torch.arange(m * cols, device="cuda", dtype=torch.float32).reshape(m, cols)
    odd = [torch.zeros(m, 2 * cols, device="cuda") for _ in range(2)]
    even = [torch.zeros(m, 2 * cols, device="cuda") for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(2)]
    rnd = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.zq_set_wait_limit(1024)
    try:
        rc = lib.zq_peer_gather_cols_step(ptr_array(odd), ptr_array(even), ptr_array(flags), 2, 1, C.c_void_p(local.data_ptr()),
                                          m, 2 * cols, cols, cols, C.c_void_p(rnd.data_ptr()), stream())
        assert rc == 0
        torch.cuda.synchronize()
        for buf in odd:  # round 1: the odd buffers of both ranks
            assert torch.equal(buf[:, cols:], local) and torch.all(buf[:, :cols] == 0)
        assert int(flags[0][1].item()) == 32     # published on the other rank: 32 CTAs per destination
        assert _lib.device_error(clear=False) == GATH
        assert lib.zq_device_check(1) == 7
        flags[1][0] = 64                          # the other rank's arrivals of round 2, by hand
        rc = lib.zq_peer_gather_cols_step(ptr_array(odd), ptr_array(even), ptr_array(flags), 2, 1, C.c_void_p(local.data_ptr()),
                                          m, 2 * cols, cols, cols, C.c_void_p(rnd.data_ptr()), stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert lib.zq_device_check(1) == 0
        assert torch.equal(even[0][:, cols:], local)
    finally:
        lib.zq_set_wait_limit(0)


def test_argmax_exchange_on_one_gpu(zq, oracle):
    """zq_matmul_argmax. One rank: the index of the first largest output, also among equal values, with and without
    the outputs stored. Two 'ranks' with the other rank's words written by hand: the larger value wins, rank order
    decides between equal values, and without the other rank's words the poll ends with 'FGAT'."""
    from zignn_b200 import _lib
    lib = _lib.load()
    _lib.device_error(clear=True)
    n, k = 148 * 2 * 8 * 16, 1152
    rng = np.random.default_rng(6)
    raw = oracle.quantize(ggml.Q4_0, (rng.standard_normal((n, k)) * 0.02).astype(np.float32)).reshape(n, -1)
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float32)).cuda()
    y0 = zq.quant_matmul_no_grad(x, zq.QuantWeight(raw.reshape(-1), ggml.Q4_0, n, k)).reshape(-1)
    top = int(torch.argmax(y0).item())
    later, earlier = (top + 12345) % n, (top + n - 777) % n
    if later < top:
        later, earlier = earlier, later  # keep `later` above and `earlier` below the winning row
    index = torch.zeros(1, dtype=torch.int32, device="cuda")
    value = torch.zeros(1, device="cuda")
    y_local = torch.zeros(n, device="cuda")

    def run(qw, world=1, rank=0, inbox=None, sync=None, store=False):
        return lib.zq_matmul_argmax(qw.handle, C.c_void_p(x.data_ptr()), None, C.c_void_p(y_local.data_ptr()) if store else None,
                                    ptr_array(inbox[1]) if inbox else None, ptr_array(inbox[0]) if inbox else None,
                                    C.c_void_p(index.data_ptr()), C.c_void_p(value.data_ptr()), world, rank,
                                    C.c_void_p(sync.data_ptr()), stream())

    sync = torch.zeros(4096, dtype=torch.int32, device="cuda")
    qw = zq.QuantWeight(raw.reshape(-1), ggml.Q4_0, n, k)
    for store in (False, True, False):  # three rounds on the same counters
        assert run(qw, sync=sync, store=store) == 0
        torch.cuda.synchronize()
        assert int(index.item()) == top and float(value.item()) == float(y0[top].item())
        if store:
            assert torch.equal(y_local, y0)
    # the winning row's bytes copied to a later row: the first one still wins; to an earlier row: that one wins
    raw2 = raw.copy()
    raw2[later] = raw[top]
    assert run(zq.QuantWeight(raw2.reshape(-1), ggml.Q4_0, n, k), sync=sync) == 0
    torch.cuda.synchronize()
    assert int(index.item()) == min(top, later)
    raw2[earlier] = raw[top]
    assert run(zq.QuantWeight(raw2.reshape(-1), ggml.Q4_0, n, k), sync=sync) == 0
    torch.cuda.synchronize()
    assert int(index.item()) == min(top, later, earlier)

    # two ranks, the other one's words supplied by hand (inbox: two words per rank and round parity)
    def words(rnd, v, row):
        vb = int(np.float32(v).view(np.uint32))
        return torch.tensor([(rnd << 32) | vb, (rnd << 32) | row], dtype=torch.int64, device="cuda")

    best = float(y0[top].item())
    for rank, their_v, their_row, want in ((0, best * 2, n + 5, n + 5),      # the other rank's value is larger
                                            (0, best, n + 5, top),            # equal: the lower rank (this one) wins
                                            (1, best, 7, 7),                  # equal, the other rank is the lower one
                                            (1, best * 0.5, 7, n + top)):     # this rank's value is larger
        inbox = [[torch.zeros(4, dtype=torch.int64, device="cuda") for _ in range(2)] for _ in range(2)]
        sync2 = torch.zeros(4096, dtype=torch.int32, device="cuda")
        other = 1 - rank
        inbox[1][rank][2 * other: 2 * other + 2] = words(1, their_v, their_row)  # round 1 uses the odd inboxes
        assert run(qw, world=2, rank=rank, inbox=inbox, sync=sync2) == 0
        torch.cuda.synchronize()
        assert int(index.item()) == want, (rank, their_v, their_row, int(index.item()))
        sent = inbox[1][other][2 * rank: 2 * rank + 2]                           # what this rank sent
        assert int(sent[0].item()) >> 32 == 1 and int(sent[1].item()) & 0xFFFFFFFF == rank * n + top
        assert lib.zq_device_check(1) == 0
    lib.zq_set_wait_limit(1024)
    try:
        inbox = [[torch.zeros(4, dtype=torch.int64, device="cuda") for _ in range(2)] for _ in range(2)]
        sync2 = torch.zeros(4096, dtype=torch.int32, device="cuda")
        assert run(qw, world=2, rank=0, inbox=inbox, sync=sync2) == 0
        torch.cuda.synchronize()
        assert _lib.device_error(clear=False) == FGAT
        assert lib.zq_device_check(1) == 7
    finally:
        lib.zq_set_wait_limit(0)


def test_many_rows_without_workspace_is_refused(zq, oracle):
    from zignn_b200 import _lib
    import zignn_b200.structs as S
    lib = _lib.load()
    raw = oracle.quantize(ggml.Q4_0, np.zeros((64, 64), np.float32))
    qw = zq.QuantWeight(raw, ggml.Q4_0, 64, 64)
    x, y = torch.zeros(64, 64, device="cuda"), torch.zeros(64, 64, device="cuda")
    ep = S.Epilogue(None, 0, None, None)
    rc = lib.zq_matmul(qw.handle, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 64, zq.ACT_F32, C.byref(ep), None, 0,
                       stream())
    assert rc == 1  # ZQ_ERR_BAD_ARG: 49 rows or more need the workspace
    rc = lib.zq_matmul(qw.handle, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 48, zq.ACT_F32, C.byref(ep), None, 0,
                       stream())
    assert rc == 0


@pytest.mark.parametrize("m", [1, 64])
def test_rows_of_vanishing_magnitude_give_finite_results(zq, oracle, m):
    """A row whose largest magnitude is 1e-38 (a vanished gradient): the power-of-two row scale must not
    overflow; outputs are finite and zero at the accuracy of the path."""
    n, k = 128, 256
    raw = oracle.quantize(ggml.Q8_0, (np.random.default_rng(2).standard_normal((n, k)) * 0.02).astype(np.float32))
    qw = zq.QuantWeight(raw, ggml.Q8_0, n, k)
    x = np.random.default_rng(3).standard_normal((m, k)).astype(np.float32)
    x[0] = 1e-38
    got = zq.quant_matmul_no_grad(torch.from_numpy(x).cuda(), qw, zq.ACT_F32).cpu().numpy()
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got[0])) <= 1e-30
    if m > 1:
        want = oracle.linear(ggml.Q8_0, raw, x, n, k, act_mode=0, n_threads=2)
        err = np.linalg.norm(got[1:] - want[1:]) / np.linalg.norm(want[1:])
        assert err <= 6e-4
    go = torch.from_numpy(np.full((2, n), 1e-38, np.float32)).cuda()
    gx = zq.quant_matmul_transposed(go, qw).cpu().numpy()
    assert np.all(np.isfinite(gx)) and np.max(np.abs(gx)) <= 1e-30
