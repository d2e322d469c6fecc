"""Output-dimension sharding of a quantised linear layer over the ranks of one node.

A GGUF matrix is row-major: row r of [out_dim][in_dim] is in_dim/32 consecutive blocks. Rows are
independent dot products (zig-nn's own CPU pool splits the same way, src/gguf/thread_pool.zig:96-181),
so rank r keeps a contiguous slice of rows, computes its slice of y = x . W^T and the slices are
all-gathered. That all-gather is the only exchange on the path. This module holds the host logic
only: the partition, slicing of raw GGUF bytes, and the gather; the per-rank product is whatever
`compute` the caller passes (the CUDA path passes api.quant_matmul_no_grad).
"""
import torch

from . import ggml

ROW_ALIGN = 16  # one tensor-core row tile; keeps every shard's first row tile-aligned


def rows_per_rank(out_dim, world):
    """Rows each rank owns (the last ranks may own fewer, or none)."""
    per = -(-out_dim // world)
    return -(-per // ROW_ALIGN) * ROW_ALIGN


def row_range(out_dim, world, rank):
    """[lo, hi) of the rows rank `rank` owns."""
    if not 0 <= rank < world:
        raise ValueError("rank %d outside world of %d" % (rank, world))
    per = rows_per_rank(out_dim, world)
    lo = min(rank * per, out_dim)
    return lo, min(lo + per, out_dim)


def slice_rows(raw, quant_type, out_dim, in_dim, lo, hi):
    """The raw GGUF bytes of rows [lo, hi) of a [out_dim][in_dim] tensor (a view, no copy)."""
    if in_dim % ggml.BLOCK_SIZE:
        raise ValueError("in_dim must be a multiple of 32")
    row_bytes = ggml.tensor_bytes(quant_type, in_dim)
    flat = raw.reshape(-1)
    if flat.numel() != out_dim * row_bytes:
        raise ValueError("raw holds %d bytes, expected %d" % (flat.numel(), out_dim * row_bytes))
    if not 0 <= lo <= hi <= out_dim:
        raise ValueError("bad row range [%d, %d) for %d rows" % (lo, hi, out_dim))
    return flat[lo * row_bytes:hi * row_bytes]


class ShardedQuantLinear:
    """y[M][out_dim] = x[M][in_dim] . W^T with W's rows split over the process group.

    make_weight(raw_slice, quant_type, rows, in_dim) -> opaque weight for this rank (None if 0 rows)
    compute(x, weight, out)                          -> writes out[M][rows]
    Every rank calls forward() with the same x and gets the full y.
    """

    def __init__(self, raw, quant_type, out_dim, in_dim, make_weight, compute, group=None, rank=None, world=None):
        import torch.distributed as dist
        self.group = group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.out_dim, self.in_dim, self.quant_type = out_dim, in_dim, quant_type
        self.per = rows_per_rank(out_dim, self.world)
        self.lo, self.hi = row_range(out_dim, self.world, self.rank)
        self.rows = self.hi - self.lo
        part = slice_rows(raw, quant_type, out_dim, in_dim, self.lo, self.hi)
        self.weight = make_weight(part.contiguous(), quant_type, self.rows, in_dim) if self.rows else None
        self.compute = compute
        self._gathered = None

    def forward_local(self, x, out=None):
        """This rank's slice y[:, lo:hi] (shape [M][per]; columns past `rows` are zero)."""
        m = x.shape[0]
        if out is None:
            out = torch.zeros(m, self.per, dtype=torch.float32, device=x.device)
        if self.rows:
            if self.rows == self.per:
                self.compute(x, self.weight, out)
            else:
                tmp = torch.empty(m, self.rows, dtype=torch.float32, device=x.device)
                self.compute(x, self.weight, tmp)
                out[:, :self.rows] = tmp
        return out

    def gather(self, local):
        """All-gather the per-rank slices [M][per] into y[M][out_dim]."""
        m = local.shape[0]
        if self.world == 1:
            return local[:, :self.out_dim]
        import torch.distributed as dist
        if self._gathered is None or self._gathered.shape[0] != self.world * m or self._gathered.device != local.device:
            self._gathered = torch.empty(self.world * m, self.per, dtype=torch.float32, device=local.device)
        dist.all_gather_into_tensor(self._gathered, local.contiguous(), group=self.group)
        if m == 1:  # [world][per] is already y's memory order
            return self._gathered.reshape(1, self.world * self.per)[:, :self.out_dim]
        g = self._gathered.reshape(self.world, m, self.per)
        return g.permute(1, 0, 2).reshape(m, self.world * self.per)[:, :self.out_dim]

    def forward(self, x):
        return self.gather(self.forward_local(x))


class PeerGather:
    """The all-gather as peer stores over NVLink (csrc/peer_gather.cu) instead of a library collective.

    Result buffers and counters live in symmetric memory (torch.distributed._symmetric_memory supplies
    the allocation and the exchange of peer-mapped pointers; the copy and the flag protocol are the
    library's own kernel). Two result buffers alternate between rounds. Layout of a buffer:
    [world][m][per] f32, rank r's slice at r * m * per, the same layout all_gather_into_tensor produces.
    """

    def __init__(self, world, rank, m, per, device, group=None):
        import os
        import ctypes as C
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all we use
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self._lib, self._C = _lib, C
        self.world, self.rank, self.m, self.per = world, rank, m, per
        grp = group if group is not None else dist.group.WORLD
        n = world * m * per
        self.bufs, self._yptrs = [], []
        for _ in range(2):
            t = symm_mem.empty(n, dtype=torch.float32, device=device)
            t.zero_()
            h = symm_mem.rendezvous(t, grp)
            self.bufs.append(t)
            self._yptrs.append((C.c_void_p * world)(*[int(p) for p in h.buffer_ptrs]))
        self.flags = symm_mem.empty(world, dtype=torch.int32, device=device)
        self.flags.zero_()
        hf = symm_mem.rendezvous(self.flags, grp)
        self._fptrs = (C.c_void_p * world)(*[int(p) for p in hf.buffer_ptrs])
        self._handles = (h, hf)
        self.round = 0                                                     # host copy of the round number
        self.d_round = torch.zeros(1, dtype=torch.int32, device=device)    # the kernel's own copy
        # the fused GEMV + exchange keeps its own counters
        self.fflags = symm_mem.empty(world, dtype=torch.int32, device=device)
        self.fflags.zero_()
        hff = symm_mem.rendezvous(self.fflags, grp)
        self._ffptrs = (C.c_void_p * world)(*[int(p) for p in hff.buffer_ptrs])
        self._handles = self._handles + (hff,)
        self.d_sync = torch.zeros(2, dtype=torch.int32, device=device)
        # tagged form of the fused exchange (one activation row): an inbox of 64-bit words per round parity
        self._inptrs = None
        if m == 1 and per % 2 == 0:
            self.inboxes, self._inptrs = [], []
            for _ in range(2):
                t = symm_mem.empty(world * per, dtype=torch.int64, device=device)
                t.zero_()
                hi = symm_mem.rendezvous(t, grp)
                self.inboxes.append(t)
                self._inptrs.append((C.c_void_p * world)(*[int(p) for p in hi.buffer_ptrs]))
                self._handles = self._handles + (hi,)
        self.tagged = self._inptrs is not None
        # several activation rows: column slices written straight into the row-major result (own counters)
        self.cflags = symm_mem.empty(world, dtype=torch.int32, device=device)
        self.cflags.zero_()
        hcf = symm_mem.rendezvous(self.cflags, grp)
        self._cfptrs = (C.c_void_p * world)(*[int(p) for p in hcf.buffer_ptrs])
        self._handles = self._handles + (hcf,)
        self.d_round_cols = torch.zeros(1, dtype=torch.int32, device=device)
        self.round_cols = 0
        # arg-max form: two words per rank and round parity, its own counters and CTA slots
        self._amptrs = []
        for _ in range(2):
            t = symm_mem.empty(2 * world, dtype=torch.int64, device=device)
            t.zero_()
            ha = symm_mem.rendezvous(t, grp)
            self._amptrs.append((t, (C.c_void_p * world)(*[int(p) for p in ha.buffer_ptrs])))
            self._handles = self._handles + (ha,)
        self.d_sync_argmax = torch.zeros(4096, dtype=torch.int32, device=device)
        self.argmax_index = torch.zeros(1, dtype=torch.int32, device=device)
        self.argmax_value = torch.zeros(1, dtype=torch.float32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every rank's counters are zero before anybody adds to them

    def next_buffer(self):
        """The buffer this round's local slice goes into: [world][m][per], write row-block `rank`."""
        return self.bufs[(self.round + 1) & 1].view(self.world, self.m, self.per)

    def gather(self):
        """Publish this rank's slice of next_buffer() to all peers and wait for theirs; returns the buffer.
        The round number is kept on the device too, so a captured sequence with an even number of
        forward() calls can be replayed (call note_replayed() after each replay)."""
        self.round += 1
        which = self.round & 1
        C = self._C
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        n = self.m * self.per
        rc = self._lib.load().zq_peer_gather_step(self._yptrs[1], self._yptrs[0], self._fptrs, self.world, self.rank,
                                                  self.rank * n, n, C.c_void_p(self.d_round.data_ptr()), stream)
        self._lib.check(rc, "zq_peer_gather_step")
        return self.bufs[which].view(self.world, self.m, self.per)

    def gather_cols(self, local):
        """local: this rank's [m][per] block of columns. Stores it into place in every rank's row-major
        [m][world * per] result buffer and waits for the other ranks' blocks; returns that buffer."""
        C = self._C
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        n_total = self.world * self.per
        rc = self._lib.load().zq_peer_gather_cols_step(self._yptrs[1], self._yptrs[0], self._cfptrs, self.world, self.rank,
                                                       C.c_void_p(local.data_ptr()), self.m, n_total, self.rank * self.per,
                                                       self.per, C.c_void_p(self.d_round_cols.data_ptr()), stream)
        self._lib.check(rc, "zq_peer_gather_cols_step")
        self.round_cols += 1
        return self.bufs[self.round_cols & 1].view(self.m, n_total)

    def fused_matmul(self, x, weight, out=None):
        """x [1][in_dim] times this rank's weight rows with the exchange inside the GEMV kernel.
        Returns the gathered buffer, or None when the shard is too small for that kernel (nothing ran).
        out (tagged form only): a buffer of world * per floats that receives the row instead of the library's own,
        e.g. page-locked host memory, which the kernel then writes directly (peers never write result rows in
        this form, only inboxes, so one buffer serves every round)."""
        C = self._C
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        if self.tagged:  # words that carry their round number: nothing follows the peer stores
            y_odd = out.data_ptr() if out is not None else self.bufs[1].data_ptr()
            y_even = out.data_ptr() if out is not None else self.bufs[0].data_ptr()
            rc = self._lib.load().zq_matmul_gather_tagged(weight.handle, C.c_void_p(x.data_ptr()), None, self._inptrs[1],
                                                          self._inptrs[0], C.c_void_p(y_odd), C.c_void_p(y_even),
                                                          self.world, self.rank,
                                                          C.c_void_p(self.d_sync.data_ptr()), stream)
            if rc == 0 and out is not None:
                self.round += 1
                return out.view(self.world, self.m, self.per)
        else:
            rc = self._lib.load().zq_matmul_gather(weight.handle, C.c_void_p(x.data_ptr()), None, self._yptrs[1],
                                                   self._yptrs[0], self._ffptrs, self.world, self.rank,
                                                   self.rank * self.per, C.c_void_p(self.d_sync.data_ptr()), stream)
        if rc == 2:  # ZQ_ERR_UNSUPPORTED
            return None
        self._lib.check(rc, "zq_matmul_gather")
        self.round += 1
        return self.bufs[self.round & 1].view(self.world, self.m, self.per)

    def fused_argmax(self, x, weight):
        """Greedy decoding: x [1][in_dim] times this rank's weight rows; only the index of the first largest output
        over all ranks is exchanged (16 bytes per peer). Returns (index, value) device tensors of one element, the
        same on every rank, or None when the shard is too small for that kernel (nothing ran)."""
        C = self._C
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self._lib.load().zq_matmul_argmax(weight.handle, C.c_void_p(x.data_ptr()), None, None, self._amptrs[1][1],
                                               self._amptrs[0][1], C.c_void_p(self.argmax_index.data_ptr()),
                                               C.c_void_p(self.argmax_value.data_ptr()), self.world, self.rank,
                                               C.c_void_p(self.d_sync_argmax.data_ptr()), stream)
        if rc == 2:  # ZQ_ERR_UNSUPPORTED
            return None
        self._lib.check(rc, "zq_matmul_argmax")
        return self.argmax_index, self.argmax_value

    def check(self, clear=True):
        """Raises when a bounded device-side wait of an exchange ran out since the last check (a peer reached
        its call more than the wait limit later, or never): the buffers returned since then hold stale data.
        Synchronises the device; call it at the points where the host synchronises anyway."""
        self._lib.check(self._lib.load().zq_device_check(int(bool(clear))), "peer exchange")

    def note_replayed(self, n_calls):
        """A captured sequence containing `n_calls` (even) gather() calls has been replayed once."""
        if n_calls % 2:
            raise ValueError("a replayable sequence holds an even number of rounds")
        self.round += n_calls


class PeerShardedLinear(ShardedQuantLinear):
    """ShardedQuantLinear whose slices are exchanged by PeerGather: the local product is written straight
    into this rank's row-block of the symmetric result buffer, then pushed to the peers."""

    def __init__(self, *args, m_rows=1, device=None, **kw):
        super().__init__(*args, **kw)
        self.m_rows = m_rows
        self.fused = None  # None: not tried yet; True / False: the fused kernel does / does not take this shard
        self.cols_exchange = True  # several activation rows: column slices straight into the row-major result
        self._local = None
        self.peer = PeerGather(self.world, self.rank, m_rows, self.per, device, group=self.group)

    def greedy(self, x, weight=None):
        """Index (and value) of the first largest output of x [1][in_dim] over all ranks' rows, as one-element device
        tensors: the exchange carries 16 bytes per peer. Falls back to forward() + argmax for shards the fused kernel
        does not take."""
        w = weight if weight is not None else self.weight
        even = self.out_dim == self.world * self.per
        if x.shape[0] == 1 and even:
            r = self.peer.fused_argmax(x, w)
            if r is not None:
                return r
        y = self.forward(x, weight=weight)
        v, i = torch.max(y[0], dim=0)  # torch.max returns the first index among equal values on CUDA? not guaranteed:
        i = torch.nonzero(y[0] == v)[0, 0]  # take the lowest index explicitly
        return i.to(torch.int32).reshape(1), v.reshape(1)

    def forward(self, x, weight=None, out=None):
        """weight: another device copy of this rank's rows to use instead of the one built at construction.
        out: one activation row through the fused kernel in its tagged form only: the buffer (device or page-locked
        host memory, out_dim floats) that receives the row; ignored by the other routes."""
        m = x.shape[0]
        if m != self.m_rows:
            raise ValueError("built for %d activation rows, got %d" % (self.m_rows, m))
        w = weight if weight is not None else self.weight
        even = self.out_dim == self.world * self.per  # every rank owns `per` rows: all ranks take the same branch
        if m == 1 and self.fused is not False and even:
            direct = out if (out is not None and self.peer.tagged and out.numel() == self.world * self.per) else None
            g = self.peer.fused_matmul(x, w, out=direct)
            self.fused = g is not None
            if g is not None:
                return g.reshape(1, self.world * self.per)[:, :self.out_dim]
        if m > 1 and self.cols_exchange:
            # the block of columns goes straight into the row-major result on every rank: nothing to permute
            if self._local is None:
                self._local = torch.zeros(m, self.per, dtype=torch.float32, device=x.device)
            if self.rows == self.per:
                self.compute(x, w, self._local)
            elif self.rows:
                tmp = torch.empty(m, self.rows, dtype=torch.float32, device=x.device)
                self.compute(x, w, tmp)
                self._local[:, :self.rows] = tmp
            return self.peer.gather_cols(self._local)[:, :self.out_dim]
        buf = self.peer.next_buffer()
        if self.rows:
            if self.rows == self.per:
                self.compute(x, w, buf[self.rank])
            else:
                tmp = torch.empty(m, self.rows, dtype=torch.float32, device=x.device)
                self.compute(x, w, tmp)
                buf[self.rank][:, :self.rows] = tmp
        g = self.peer.gather()
        if m == 1:
            return g.reshape(1, self.world * self.per)[:, :self.out_dim]
        return g.permute(1, 0, 2).reshape(m, self.world * self.per)[:, :self.out_dim]


def cuda_sharded_linear(raw, quant_type, out_dim, in_dim, act_mode=0, group=None, gather="nccl", m_rows=1):
    """ShardedQuantLinear whose per-rank product is the CUDA kernel (raw: uint8 tensor on the device).
    gather: "nccl" (all_gather_into_tensor) or "peer" (the library's peer-store kernel)."""
    from . import api

    def make_weight(part, qt, rows, k):
        return api.QuantWeight(part, qt, rows, k)

    def compute(x, w, out):
        api.quant_matmul_no_grad(x, w, act_mode, out=out)

    if gather == "peer":
        return PeerShardedLinear(raw, quant_type, out_dim, in_dim, make_weight, compute, group=group,
                                 m_rows=m_rows, device=raw.device)
    return ShardedQuantLinear(raw, quant_type, out_dim, in_dim, make_weight, compute, group=group)
