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


def _symmetric(shape, dtype, device, group):
    """A zero-filled tensor in symmetric memory and its rendezvous handle (collective)."""
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(shape, dtype=dtype, device=device)
    t.zero_()
    h = symm_mem.rendezvous(t, group)
    return t, h


class PeerFlags:
    """Step counters of one exchanged buffer, replacing a collective as the fence: rank ``r``
    publishes its step count to word ``r`` of every rank's flag array once its stores into the
    peers' buffers are complete (`signal`, or fused into the GEMM via `signal_arg`), and a
    consumer waits -- on its own stream, with a bounded device-side wait -- until all words have
    reached its own step count (`wait`).  All state lives on the device, so a step that uses
    these can be captured in a CUDA graph and replayed.  Construction is collective."""

    def __init__(self, device: torch.device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.flags, self._h = _symmetric((self.world,), torch.int32, device, self.group)
        # this rank's word on every rank (own included)
        self.flag_addrs = [int(p) + 4 * self.rank for p in self._h.buffer_ptrs]
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone signals

    @property
    def signal_arg(self):
        return self.flag_addrs, self.counter

    def signal(self) -> None:
        QF.peer_signal(self.flag_addrs, self.counter)

    def wait(self, timeout_cycles: int = 0) -> None:
        QF.peer_wait(self.flags, self.epoch, timeout_cycles)


class PeerOutputs:
    """Double-buffered `(rows, cols)` output that every rank of the group can write: the
    GEMM epilogue of each rank stores its column shard straight into all ranks' copies
    (symmetric memory, plain peer stores over NVLink), so the exchange step needs no separate
    all-gather kernel and no re-layout.  Two buffers alternate: a rank may start writing the
    other buffer while peers still read this one; `sync` (a `PeerFlags`) orders the rest.

    Construction is collective (all ranks, same order)."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, group=None,
                 buffers: int = 2):
        self.group = group if group is not None else dist.group.WORLD
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.bufs, self.ptrs, self.mc_ptrs, self._keep = [], [], [], []
        for _ in range(buffers):
            t, h = _symmetric((rows, cols), dtype, device, self.group)
            own = int(h.buffer_ptrs[self.rank])
            # this GPU's buffer first, then the peers'
            self.ptrs.append([own] + [int(p) for r, p in enumerate(h.buffer_ptrs) if r != self.rank])
            self.bufs.append(t)
            self.mc_ptrs.append(int(getattr(h, "multicast_ptr", 0) or 0))
            self._keep.append(h)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.sync = PeerFlags(device, self.group)
        self.turn = 0

    @property
    def has_multicast(self) -> bool:
        """The buffers are bound to an NVSwitch multicast object (one store reaches all ranks)."""
        return all(p != 0 for p in self.mc_ptrs)

    def next(self, multicast: bool = False):
        """(local tensor, destinations) of the buffer to fill now: the list of every rank's
        address (own first), or -- ``multicast=True`` -- the one multicast address."""
        i = self.turn
        self.turn = (self.turn + 1) % len(self.bufs)
        return self.bufs[i], (self.mc_ptrs[i] if multicast else self.ptrs[i])

    def fence(self) -> None:
        """Collective form of the fence (a 4-byte all-reduce after each rank's GEMM on its
        stream); `sync.wait()` after a signalling GEMM is the device-flag form."""
        dist.all_reduce(self._flag, group=self.group)


class TokenShardedEncoder:
    """Per-token int8 encode of a REPLICATED `(rows, cols)` activation, sharded over token rows:
    rank ``r`` encodes rows ``[r*rows/w, (r+1)*rows/w)`` and stores their codes and scales into
    every rank's operand buffers (peer stores, or one multicast store for the codes), so each
    rank encodes ``1/w`` of the tokens instead of all of them.  Bit-identical to the unsharded
    encode (rows are independent).  Construction is collective."""

    def __init__(self, rows: int, cols: int, device: torch.device, group=None):
        self.out = PeerOutputs(rows, cols, torch.int8, device, group, buffers=1)
        self.world, self.rank = self.out.world, self.out.rank
        if rows % self.world != 0:
            raise _lib.ShapeMismatch(f"{rows} token rows do not split over {self.world} ranks")
        self.rows, self.cols = rows, cols
        self.scale, self._sh = _symmetric((rows,), torch.float32, device, self.out.group)
        self.scale_ptrs = [int(self._sh.buffer_ptrs[self.rank])] + \
            [int(p) for r, p in enumerate(self._sh.buffer_ptrs) if r != self.rank]

    def __call__(self, x: torch.Tensor, multicast: bool = False, local: bool = False):
        """Encode this rank's rows of `x` -- the full replicated tensor, or with ``local=True``
        just this rank's `(rows / w, cols)` rows -- and exchange; returns (codes, scales) of all
        rows, valid after the wait that this call enqueues."""
        import ctypes as C

        per = self.rows // self.world
        r0 = self.rank * per
        shard = x.reshape(per, self.cols) if local else x.reshape(self.rows, self.cols)[r0:r0 + per]
        if not shard.is_contiguous():
            shard = shard.contiguous()
        codes, dst = self.out.next(multicast=multicast and self.out.has_multicast)
        mc = isinstance(dst, int)
        plist = self.out.ptrs[0] if mc else dst
        outs = (C.c_void_p * len(plist))(*[int(p) for p in plist])
        souts = (C.c_void_p * len(self.scale_ptrs))(*self.scale_ptrs)
        dev = x.device
        with torch.cuda.device(dev):
            _lib.check(_lib.load().lq_quantize_per_token_bcast(
                _lib.ptr(shard), _lib.code_of(x.dtype), per, self.cols, qint8.quant_min, qint8.quant_max,
                C.c_float(1e-8), outs, souts, len(plist), C.c_void_p(dst) if mc else None, r0,
                _lib.stream_ptr(dev)))
        self.out.sync.signal()
        self.out.sync.wait()
        return codes, self.scale


class HiddenExchange:
    """Exchange of a column-sharded hidden tensor as per-token int8 CODES: the ranks exchange
    the per-token abs-max of their shards (a `(world, rows)` table in symmetric memory, plain
    peer stores -- the max all-reduce of the encode), then each rank encodes its shard with the
    global scales and stores the codes into every rank's `(rows, cols)` operand buffer.  Scales
    and codes equal the single-GPU encode of the unsharded tensor bit for bit (max is
    order-free).  Construction is collective."""

    def __init__(self, rows: int, cols: int, device: torch.device, group=None):
        self.out = PeerOutputs(rows, cols, torch.int8, device, group, buffers=1)
        self.world, self.rank, self.rows, self.cols = self.out.world, self.out.rank, rows, cols
        self.table, self._th = _symmetric((self.world, rows), torch.float32, device, self.out.group)
        self.table_ptrs = [int(self._th.buffer_ptrs[self.rank])] + \
            [int(p) for r, p in enumerate(self._th.buffer_ptrs) if r != self.rank]
        self.table_sync = PeerFlags(device, self.out.group)
        self.scale = torch.empty(rows, dtype=torch.float32, device=device)

    def __call__(self, h_shard: torch.Tensor, multicast: bool = False):
        """`h_shard`: this rank's `(rows, cols / world)` columns.  Returns (codes, scales) of the
        full tensor, valid after the wait that this call enqueues."""
        import ctypes as C

        rows, n_local = h_shard.shape
        dev = h_shard.device
        lib = _lib.load()
        touts = (C.c_void_p * len(self.table_ptrs))(*self.table_ptrs)
        with torch.cuda.device(dev):
            _lib.check(lib.lq_absmax_rows_bcast(_lib.ptr(h_shard), _lib.code_of(h_shard.dtype), rows, n_local,
                                                h_shard.stride(0), touts, len(self.table_ptrs),
                                                self.rank * self.rows, _lib.stream_ptr(dev)))
        self.table_sync.signal()
        self.table_sync.wait()
        codes, dst = self.out.next(multicast=multicast and self.out.has_multicast)
        mc = isinstance(dst, int)
        plist = [dst] if mc else dst
        outs = (C.c_void_p * len(plist))(*[int(p) for p in plist])
        with torch.cuda.device(dev):
            _lib.check(lib.lq_quantize_rows_bcast(
                _lib.ptr(h_shard), _lib.code_of(h_shard.dtype), rows, n_local, h_shard.stride(0),
                _lib.ptr(self.table), self.world, self.rows, qint8.quant_min, qint8.quant_max, C.c_float(1e-8),
                outs, -1 if mc else len(plist), self.cols, self.rank * n_local, _lib.ptr(self.scale),
                _lib.stream_ptr(dev)))
        self.out.sync.signal()
        self.out.sync.wait()
        return codes, self.scale


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
            _lib.ptr(x2), _lib.code_of(x2.dtype), rows, cols, cols, _lib.ptr(row_absmax), 1, rows, qdtype.quant_min,
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
                             bias=self.bias, act=act, signal=peer.sync.signal_arg)
            peer.sync.wait()
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
