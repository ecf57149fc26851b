"""Output-column sharding of an NF4 / QLoRA linear across the GPUs of one node.

Each output column depends on one weight row (``W [d_out, d_in]``), its block scales and one row
of LoRA ``B``; ``x`` and LoRA ``A`` are replicated.  Rank ``r`` of ``g`` owns a contiguous range
of columns, computes ``y[:, range]`` with the single-GPU kernels, and the ranks exchange their
slabs with one all-gather (NCCL over NVLink on GPUs; any ``torch.distributed`` backend works,
which is how the host logic is tested on CPU with gloo).  The reference has no distributed
runtime; this partition is the one its path admits without touching the numerics: no
quantization block is split because blocks run along ``d_in``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ._lib import LAYOUT_OUT_IN

BLOCK_SIZE = 64


def column_shards(d_out: int, world: int, granule: int = 1) -> List[Tuple[int, int]]:
    """Contiguous column ranges ``[start, end)`` for ``world`` ranks, sizes differing by at most
    one ``granule`` (trailing ranks may be empty when ``d_out < world * granule``)."""
    if world < 1 or d_out < 0 or granule < 1:
        raise ValueError("column_shards: world, granule >= 1 and d_out >= 0 required")
    units = (d_out + granule - 1) // granule
    out = []
    for r in range(world):
        a = min((units * r) // world * granule, d_out)
        b = min((units * (r + 1)) // world * granule, d_out)
        out.append((a, b))
    return out


def shard_packed_rows(codes: torch.Tensor, scales: torch.Tensor, d_in: int,
                      rows: Tuple[int, int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Slice rows ``[start, end)`` out of a packed ``W [d_out, d_in]`` weight (``d_in % 64 == 0``).

    ``codes`` holds ``d_in / 2`` bytes per row and ``scales`` (f32 absmax or u8 scale codes)
    ``d_in / 64`` entries per row, so a row range is a contiguous byte range of both."""
    if d_in % BLOCK_SIZE != 0:
        raise ValueError("row sharding of a packed weight needs d_in % 64 == 0 "
                         "(otherwise a quantization block straddles two rows)")
    a, b = rows
    return (codes[a * (d_in // 2): b * (d_in // 2)].contiguous(),
            scales[a * (d_in // BLOCK_SIZE): b * (d_in // BLOCK_SIZE)].contiguous())


def gather_columns(y_local: torch.Tensor, shards: Sequence[Tuple[int, int]],
                   group: Optional[dist.ProcessGroup] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the ranks' column slabs ``y_local [rows, end - start]`` into ``y [rows, d_out]``.

    Equal slabs go through one ``all_gather_into_tensor`` (``[world, rows, width]``) followed by a
    permuting copy; unequal slabs are padded to the widest one first."""
    world = dist.get_world_size(group)
    if len(shards) != world:
        raise ValueError("gather_columns: one shard per rank expected")
    rows = y_local.shape[0]
    d_out = shards[-1][1]
    widths = [b - a for a, b in shards]
    wmax = max(widths)
    mine = widths[dist.get_rank(group)]
    if y_local.shape[1] != mine:
        raise ValueError(f"gather_columns: local slab has {y_local.shape[1]} columns, shard says {mine}")
    send = y_local.contiguous()
    if mine != wmax:
        send = torch.zeros(rows, wmax, dtype=y_local.dtype, device=y_local.device)
        send[:, :mine] = y_local
    flat = torch.empty(world * rows, wmax, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, send, group=group)  # slabs concatenated along dim 0
    stacked = flat.view(world, rows, wmax)
    y = out if out is not None else torch.empty(rows, d_out, dtype=y_local.dtype,
                                                device=y_local.device)
    if all(w == wmax for w in widths):
        y.view(rows, world, wmax).copy_(stacked.permute(1, 0, 2))
    else:
        for r, (a, b) in enumerate(shards):
            y[:, a:b] = stacked[r, :, : b - a]
    return y


class ShardedNf4Linear:
    """One rank's column shard of a QLoRA linear (``W [d_out, d_in]``, blocks along ``d_in``)."""

    def __init__(self, packed, d_in: int, d_out: int, shards: Sequence[Tuple[int, int]], rank: int,
                 bias: Optional[torch.Tensor] = None, lora_a: Optional[torch.Tensor] = None,
                 lora_b: Optional[torch.Tensor] = None, lora_scale: float = 0.0,
                 group: Optional[dist.ProcessGroup] = None):
        self.packed = packed          # PackedNf4Tensor of the local rows only
        self.d_in, self.d_out = d_in, d_out
        self.shards, self.rank, self.group = list(shards), rank, group
        self.bias, self.lora_a, self.lora_b, self.lora_scale = bias, lora_a, lora_b, lora_scale

    @staticmethod
    def from_full(packed_full, d_in: int, d_out: int, world: int, rank: int,
                  bias=None, lora_a=None, lora_b=None, lora_scale: float = 0.0, group=None,
                  granule: int = 1) -> "ShardedNf4Linear":
        """Cut rank ``rank``'s rows out of a full packed weight that every rank can see."""
        from .quantize import PackedNf4Tensor

        shards = column_shards(d_out, world, granule)
        a, b = shards[rank]
        dq = packed_full.is_double_quantized()
        scales = packed_full.scale_codes if dq else packed_full.absmax
        codes, sc = shard_packed_rows(packed_full.codes, scales, d_in, (a, b))
        local = PackedNf4Tensor(codes, (b - a) * d_in, None if dq else sc, sc if dq else None,
                                packed_full.scale_of_scales)
        return ShardedNf4Linear(local, d_in, d_out, shards, rank,
                                bias[a:b].contiguous() if bias is not None else None, lora_a,
                                lora_b[a:b].contiguous() if lora_b is not None else None,
                                lora_scale, group)

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        from .quantize import linear_forward

        a, b = self.shards[self.rank]
        return linear_forward(x, self.packed, self.d_in, b - a, LAYOUT_OUT_IN, bias=self.bias,
                              lora_a=self.lora_a, lora_b=self.lora_b, lora_scale=self.lora_scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y_local = self.forward_local(x)
        lead = y_local.shape[:-1]
        y = gather_columns(y_local.reshape(-1, y_local.shape[-1]), self.shards, self.group)
        return y.view(*lead, self.d_out)

    def peer_store_plan(self, x: torch.Tensor, **kw) -> "PeerStorePlan":
        """The decode-sized forward whose kernel stores into every rank's output (no collective)."""
        return PeerStorePlan(self, x, **kw)

    def plan(self, x: torch.Tensor) -> "ShardedForwardPlan":
        """Buffers and the argument block for repeated forwards of ``x``'s shape and storage: the
        serving loop's form of ``forward`` (nothing is allocated per call, so the calls can be
        captured in a CUDA graph)."""
        return ShardedForwardPlan(self, x)


class PeerStorePlan:
    """A sharded forward without a collective: ``run()`` enqueues this rank's forward and gets its
    columns into every rank's ``y [rows, d_out]`` over NVLink -- at decode sizes the kernel's own
    epilogue stores them there (``nf4_linear_forward_scatter_dev``), otherwise the forward writes
    them into this rank's ``y`` in place and ``nf4_peer_push_columns_dev`` pushes them to the
    peers -- and (with ``signal``) adds one arrival to every rank's counter
    ``arrivals[counter_index]`` when they are out; ``wait(n)`` enqueues the bounded wait for ``n``
    arrivals on this rank's own counter (one per rank and signalling forward).  Equal shards.  ``y`` and ``arrivals`` are allocated here, on every rank alike, and mapped into the
    peers with :func:`map_peer_tensors` (``arrivals`` may be shared between plans: pass the list
    a previous plan returned in ``peer_arrivals``)."""

    def __init__(self, lin: "ShardedNf4Linear", x: torch.Tensor, signal: bool = True, counter_index: int = 0,
                 peer_arrivals: Optional[List[torch.Tensor]] = None, wait_for: int = 0):
        import ctypes

        from . import _lib

        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2:
            raise ValueError("PeerStorePlan: x must be a contiguous bf16 [rows, d_in] tensor")
        world = dist.get_world_size(lin.group)
        widths = {e - s for s, e in lin.shards}
        if len(widths) != 1:
            raise ValueError("PeerStorePlan: the shards must be equal")
        width = widths.pop()
        self.lin, self.x, self.world = lin, x, world
        self.lib, self._check, self._vp = _lib.load(), _lib.check, ctypes.c_void_p
        rows, dev = x.shape[0], x.device
        self.y = torch.zeros(rows, lin.d_out, dtype=torch.bfloat16, device=dev)
        self.peer_y = map_peer_tensors(self.y, lin.group)
        if peer_arrivals is None:
            self.arrivals = torch.zeros(64, dtype=torch.int32, device=dev)
            peer_arrivals = map_peer_tensors(self.arrivals, lin.group)
        self.peer_arrivals = peer_arrivals
        self.arrivals = peer_arrivals[lin.rank]
        self.counter_index = counter_index
        rank = lin.lora_a.shape[0] if lin.lora_a is not None else 0
        ws_bytes = int(self.lib.nf4_linear_workspace_bytes(rows, lin.d_in, width, rank))
        self.ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        self.bias32 = lin.bias.to(torch.float32).contiguous() if lin.bias is not None else None
        self.la = lin.lora_a.to(torch.bfloat16).contiguous() if rank else None
        self.lb = lin.lora_b.to(torch.bfloat16).contiguous() if rank else None
        pk = lin.packed
        dq = pk.is_double_quantized()
        args = _lib.LinearArgs()
        args.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        args.layout, args.io_dtype = LAYOUT_OUT_IN, _lib.DTYPE_BF16
        args.rows, args.d_in, args.d_out = rows, lin.d_in, width
        args.x, args.packed = x.data_ptr(), pk.codes.data_ptr()
        args.absmax = None if dq else pk.absmax.data_ptr()
        args.scale_codes = pk.scale_codes.data_ptr() if dq else None
        args.scale_of_scales = pk.scale_of_scales.data_ptr() if dq else None
        args.bias = self.bias32.data_ptr() if self.bias32 is not None else None
        args.lora_a = self.la.data_ptr() if rank else None
        args.lora_b = self.lb.data_ptr() if rank else None
        args.lora_rank, args.lora_scale = rank, float(lin.lora_scale)
        args.workspace, args.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        # the decode kernel stores into the peers itself; other shapes write in place and push
        self.in_kernel = rows <= 16 and lin.d_in % 256 == 0 and lin.d_in <= 32768
        if not self.in_kernel:
            if wait_for:
                raise ValueError("PeerStorePlan: only the decode-sized forward waits inside the kernel")
            args.y = self.y.data_ptr() + lin.rank * width * 2
            args.ldy = lin.d_out
            self.push_word = torch.zeros(1, dtype=torch.int32, device=dev)
            self.rows, self.width = rows, width
        po = _lib.PeerOutputs()
        po.struct_bytes = ctypes.sizeof(_lib.PeerOutputs)
        po.world, po.rank, po.ldy_full = world, lin.rank, lin.d_out
        for r in range(world):
            po.y_full[r] = self.peer_y[r].data_ptr()
            po.arrivals[r] = peer_arrivals[r][counter_index:counter_index + 1].data_ptr()
        po.signal = 1 if signal else 0
        if wait_for:
            po.wait_arrivals = self.arrivals[counter_index:counter_index + 1].data_ptr()
            po.wait_expected = wait_for
        self.args, self.peers = args, po
        self._a, self._p = ctypes.byref(args), ctypes.byref(po)

    def run(self) -> torch.Tensor:
        stream = self._vp(torch.cuda.current_stream(self.x.device).cuda_stream)
        if self.in_kernel:
            self._check(self.lib.nf4_linear_forward_scatter_dev(self._a, self._p, stream))
        else:
            self._check(self.lib.nf4_linear_forward_dev(self._a, stream))
            self._check(self.lib.nf4_peer_push_columns_dev(self._p, self.rows, self.width, 2,
                                                           self._vp(self.push_word.data_ptr()), stream))
        return self.y

    def wait(self, arrivals: int, timeout_ns: int = 2_000_000_000) -> None:
        stream = self._vp(torch.cuda.current_stream(self.x.device).cuda_stream)
        ptr = self._vp(self.arrivals[self.counter_index:self.counter_index + 1].data_ptr())
        self._check(self.lib.nf4_peer_arrivals_wait_dev(ptr, arrivals, timeout_ns, stream))


class ShardedForwardPlan:
    """``ShardedNf4Linear.forward`` with everything allocated once: the local slab, the workspace,
    the gather buffer and the full output.  ``run()`` enqueues the local forward on the current
    stream, the all-gather of the slabs and the permuting copy into ``y [rows, d_out]``."""

    def __init__(self, lin: ShardedNf4Linear, x: torch.Tensor):
        import ctypes

        from . import _lib

        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2:
            raise ValueError("ShardedForwardPlan: x must be a contiguous bf16 [rows, d_in] tensor")
        self.lin, self.x = lin, x
        self.lib = _lib.load()
        self._check = _lib.check
        rows, dev = x.shape[0], x.device
        world = dist.get_world_size(lin.group)
        a, b = lin.shards[lin.rank]
        widths = [e - s for s, e in lin.shards]
        self.wmax, self.world, self.rows = max(widths), world, rows
        self.equal = all(w == self.wmax for w in widths)
        # the local slab is written straight into a [rows, wmax] send buffer (ldy = wmax)
        self.send = torch.zeros(rows, self.wmax, dtype=torch.bfloat16, device=dev)
        self.flat = torch.empty(world * rows, self.wmax, dtype=torch.bfloat16, device=dev)
        self.y = torch.empty(rows, lin.d_out, dtype=torch.bfloat16, device=dev)
        rank = lin.lora_a.shape[0] if lin.lora_a is not None else 0
        ws_bytes = int(self.lib.nf4_linear_workspace_bytes(rows, lin.d_in, b - a, rank))
        self.ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        self.bias32 = lin.bias.to(torch.float32).contiguous() if lin.bias is not None else None
        self.la = lin.lora_a.to(torch.bfloat16).contiguous() if rank else None
        self.lb = lin.lora_b.to(torch.bfloat16).contiguous() if rank else None
        pk = lin.packed
        dq = pk.is_double_quantized()
        args = _lib.LinearArgs()
        args.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        args.layout, args.io_dtype = LAYOUT_OUT_IN, _lib.DTYPE_BF16
        args.rows, args.d_in, args.d_out = rows, lin.d_in, b - a
        args.x, args.packed = x.data_ptr(), pk.codes.data_ptr()
        args.absmax = None if dq else pk.absmax.data_ptr()
        args.scale_codes = pk.scale_codes.data_ptr() if dq else None
        args.scale_of_scales = pk.scale_of_scales.data_ptr() if dq else None
        args.bias = self.bias32.data_ptr() if self.bias32 is not None else None
        args.lora_a = self.la.data_ptr() if rank else None
        args.lora_b = self.lb.data_ptr() if rank else None
        args.lora_rank, args.lora_scale = rank, float(lin.lora_scale)
        args.y, args.ldy = self.send.data_ptr(), self.wmax
        args.workspace, args.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        self.args = args
        self._byref = ctypes.byref(args)
        self._vp = ctypes.c_void_p
        self.empty_local = b == a

    def run_local(self) -> torch.Tensor:
        """The local slab only (no exchange); returns the [rows, wmax] send buffer."""
        if not self.empty_local:
            stream = self._vp(torch.cuda.current_stream(self.x.device).cuda_stream)
            self._check(self.lib.nf4_linear_forward_dev(self._byref, stream))
        return self.send

    def gather(self) -> torch.Tensor:
        """All-gather of the slabs and the permuting copy into ``y [rows, d_out]``."""
        dist.all_gather_into_tensor(self.flat, self.send, group=self.lin.group)
        stacked = self.flat.view(self.world, self.rows, self.wmax)
        if self.equal:
            self.y.view(self.rows, self.world, self.wmax).copy_(stacked.permute(1, 0, 2))
        else:
            for r, (a, b) in enumerate(self.lin.shards):
                self.y[:, a:b] = stacked[r, :, : b - a]
        return self.y

    def run(self) -> torch.Tensor:
        self.run_local()
        return self.gather()


def map_peer_tensors(t: torch.Tensor, group=None) -> List[torch.Tensor]:
    """Every rank's copy of ``t`` (same shape and dtype on every rank, each in its own GPU's
    memory) as tensors of THIS process: element ``r`` is rank ``r``'s allocation mapped into this
    rank's device through CUDA IPC, element ``rank`` is ``t`` itself.  Kernels of this rank can
    store into them over NVLink (``nf4_linear_forward_scatter_dev``).

    The handle is opened with the importing device current (as NCCL's peer transport does):
    opened under the exporting device, the mapping belongs to that device's context and kernels
    of this one fault.  Keep the returned tensors alive while kernels may touch them, and ``t``
    alive on every rank while any peer still holds its mapping."""
    if not t.is_cuda:
        raise ValueError("map_peer_tensors needs a CUDA tensor")
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    dev = t.device
    for r in range(world):
        if r != rank and not torch.cuda.can_device_access_peer(dev.index, r):
            raise RuntimeError(f"device {dev.index} cannot access device {r} as a peer")
    handles = [None] * world
    dist.all_gather_object(handles, t.untyped_storage()._share_cuda_(), group=group)
    out = []
    for r in range(world):
        if r == rank:
            out.append(t)
            continue
        st = torch.UntypedStorage._new_shared_cuda(dev.index, *handles[r][1:])
        out.append(torch.empty(0, dtype=t.dtype, device=dev).set_(st).view(t.shape))
    return out
