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


def cuda_sharded_linear(raw, quant_type, out_dim, in_dim, act_mode=0, group=None):
    """ShardedQuantLinear whose per-rank product is the CUDA kernel (raw: uint8 tensor on the device)."""
    from . import api

    def make_weight(part, qt, rows, k):
        return api.QuantWeight(part, qt, rows, k)

    def compute(x, w, out):
        api.quant_matmul_no_grad(x, w, act_mode, out=out)

    return ShardedQuantLinear(raw, quant_type, out_dim, in_dim, make_weight, compute, group=group)
