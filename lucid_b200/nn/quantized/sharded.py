"""Output-channel (N) sharded W8A8 linear for one box of GPUs.

Rank ``r`` of ``w`` owns the contiguous rows ``[r*N/w, (r+1)*N/w)`` of the
``(N, K)`` weight with their scales and bias.  Activations (and their per-token
scales) are replicated, every rank's integer GEMM is independent, and one
exchange step -- an all-gather of the ``(M, N/w)`` output shards -- rebuilds the
``(M, N)`` result on every rank.  Sharding changes no number: each output
column is produced by exactly one rank with the 1-GPU arithmetic.

The reference has no distributed code; this module is new surface.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ... import _lib
from ...quantization import qint8, quantize_per_token
from . import functional as QF


def shard_bounds(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Row range of ``rank``: equal contiguous shards; ``n`` must divide evenly
    into ``world`` shards that are multiples of ``multiple``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if n % (world * multiple) != 0:
        raise _lib.ShapeMismatch(f"N={n} does not split into {world} shards of a multiple of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def gather_columns(local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather ``(M, n_local)`` column shards into ``(M, world * n_local)``.

    The collective lands shards as ``(world, M, n_local)``; one strided copy puts
    them side by side.  Works on any backend (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local
    m, n_local = local.shape
    stage = torch.empty((world * m, n_local), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(stage, local.contiguous(), group=group)
    stage = stage.view(world, m, n_local)
    if out is None:
        out = torch.empty((m, world * n_local), dtype=local.dtype, device=local.device)
    out.view(m, world, n_local).copy_(stage.permute(1, 0, 2))
    return out


class PeerOutputs:
    """Double-buffered `(rows, cols)` output that every rank of the group can write: the
    GEMM epilogue of each rank stores its column shard straight into all ranks' copies
    (symmetric memory, plain peer stores over NVLink), so the exchange step needs no separate
    all-gather kernel and no re-layout.  Two buffers alternate: a rank may start writing the
    other buffer while peers still read this one; the barrier after each GEMM orders the rest.

    Construction is collective (all ranks, same order)."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.bufs, self.ptrs, self.mc_ptrs = [], [], []
        for _ in range(2):
            t = symm_mem.empty((rows, cols), dtype=dtype, device=device)
            h = symm_mem.rendezvous(t, self.group)
            own = int(h.buffer_ptrs[self.rank])
            # this GPU's buffer first, then the peers'
            self.ptrs.append([own] + [int(p) for r, p in enumerate(h.buffer_ptrs) if r != self.rank])
            self.bufs.append(t)
            self.mc_ptrs.append(int(getattr(h, "multicast_ptr", 0) or 0))
            self._keep = getattr(self, "_keep", []) + [h]
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.turn = 0

    @property
    def has_multicast(self) -> bool:
        """The buffers are bound to an NVSwitch multicast object (one store reaches all ranks)."""
        return all(p != 0 for p in self.mc_ptrs)

    def next(self, multicast: bool = False):
        """(local tensor, destinations) of the buffer to fill now: the list of every rank's
        address (own first), or -- ``multicast=True`` -- the one multicast address."""
        i = self.turn
        self.turn ^= 1
        return self.bufs[i], (self.mc_ptrs[i] if multicast else self.ptrs[i])

    def fence(self) -> None:
        """All ranks' stores into the current buffer are complete and visible after this
        (stream-ordered): a 4-byte all-reduce follows each rank's GEMM on its stream."""
        dist.all_reduce(self._flag, group=self.group)


def shard_absmax(x_shard: torch.Tensor, group=None) -> torch.Tensor:
    """Per-token ``max |x|`` over all column shards: one range reduction of this rank's shard
    and a ``MAX`` all-reduce of ``rows`` floats (order-free, so bit-identical on every rank)."""
    from ...quantization.observer import minmax

    mn, mx = minmax(x_shard.reshape(-1, x_shard.shape[-1]), per_row=True)
    am = torch.maximum(mn.abs_(), mx.abs_())
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(am, op=dist.ReduceOp.MAX, group=group)
    return am


def quantize_shard_bcast(x_shard: torch.Tensor, row_absmax: torch.Tensor, dst_ptrs, ldo: int, col0: int,
                         out_scale: torch.Tensor | None = None, qdtype=qint8, eps: float = 1e-8):
    """Encode this rank's ``(rows, cols)`` shard with the global per-token scales and store
    the codes into columns ``[col0, col0 + cols)`` of every destination in ``dst_ptrs`` (raw
    device pointers of ``(rows, ldo)`` int8 buffers: own first, then the peers').  Returns the
    per-token scales."""
    import ctypes as C

    _lib.require_cuda(x_shard, "shard")
    x2 = x_shard.reshape(-1, x_shard.shape[-1]).contiguous()
    rows, cols = x2.shape
    if out_scale is None:
        out_scale = torch.empty(rows, dtype=torch.float32, device=x2.device)
    multicast = isinstance(dst_ptrs, int)  # an NVSwitch multicast address instead of a list
    plist = [dst_ptrs] if multicast else list(dst_ptrs)
    arr = (C.c_void_p * len(plist))(*[C.c_void_p(int(p)) for p in plist])
    with torch.cuda.device(x2.device):
        _lib.check(_lib.load().lq_quantize_rows_bcast(
            _lib.ptr(x2), _lib.code_of(x2.dtype), rows, cols, cols, _lib.ptr(row_absmax), qdtype.quant_min,
            qdtype.quant_max, C.c_float(eps), arr, -1 if multicast else len(plist), int(ldo), int(col0),
            _lib.ptr(out_scale), _lib.stream_ptr(x2.device)))
    return out_scale


class ColumnShardedLinear(torch.nn.Module):
    """This rank's shard of a per-token W8A8 linear plus the output all-gather."""

    def __init__(self, in_features: int, out_features: int, world: int, rank: int,
                 bias: bool = False, group=None) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.world, self.rank, self.group = world, rank, group
        self.n0, self.n1 = shard_bounds(out_features, world, rank)
        n_local = self.n1 - self.n0
        self.register_buffer("weight_int8", torch.zeros((n_local, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(n_local))
        if bias:
            self.register_buffer("bias", torch.zeros(n_local))
        else:
            self.bias = None

    @classmethod
    def from_full(cls, weight_int8: torch.Tensor, weight_scale: torch.Tensor, bias, world: int,
                  rank: int, group=None) -> "ColumnShardedLinear":
        n, k = weight_int8.shape
        m = cls(k, n, world, rank, bias is not None, group)
        m.weight_int8 = weight_int8[m.n0:m.n1].contiguous()
        m.weight_scale = weight_scale[m.n0:m.n1].contiguous()
        if bias is not None:
            m.bias = bias[m.n0:m.n1].contiguous()
        return m.to(weight_int8.device)

    def forward_codes(self, a: torch.Tensor, a_scale: torch.Tensor, out_dtype=torch.bfloat16,
                      gather: bool = True, act: int = _lib.ACT_NONE) -> torch.Tensor:
        """`exchange = "p2p"` (set by `use_peer_outputs`) fuses the exchange into the GEMM
        epilogue; otherwise the shards are all-gathered with NCCL."""
        n_local = self.weight_int8.shape[0] // (2 if act == _lib.ACT_SILU_GATE else 1)
        peer = getattr(self, "_peer", None)
        if gather and self.world > 1 and peer is not None:
            if a.shape[0] > peer.rows or peer.dtype != out_dtype:
                raise _lib.ShapeMismatch("peer output buffers were sized for fewer rows / another dtype")
            buf, ptrs = peer.next()
            QF.gemm_s8_bcast(a, self.weight_int8, ptrs, (peer.rows, peer.cols), self.rank * n_local,
                             out_dtype=out_dtype, a_scale=a_scale, b_scale=self.weight_scale,
                             bias=self.bias, act=act)
            peer.fence()
            return buf[: a.shape[0]]
        local = QF.gemm_s8(a, self.weight_int8, out_dtype=out_dtype, a_scale=a_scale,
                           b_scale=self.weight_scale, bias=self.bias, act=act)
        return gather_columns(local, self.group) if gather and self.world > 1 else local

    def use_peer_outputs(self, max_rows: int, dtype=torch.bfloat16, gated: bool = False) -> None:
        """Collective: allocate the symmetric output buffers for inputs of up to `max_rows`
        rows and switch the exchange step to epilogue peer stores."""
        cols = self.out_features // (2 if gated else 1)
        self._peer = PeerOutputs(max_rows, cols, dtype, self.weight_int8.device, self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        a, s = quantize_per_token(x.reshape(-1, self.in_features), qint8)
        y = self.forward_codes(a, s, x.dtype)
        return y.reshape(*lead, y.shape[-1])
