"""Host-side mirror of the reference's ``src/quantize.rs`` API over the B200 C ABI.

Same names, argument meaning and behaviour as the reference types
(``PackedNf4Tensor``, ``Nf4Tensor``, ``LoraConfig``, ``LoraAdapter``, ``QLoraLinear``,
``quantize_dequantize_tensor``, ``quantize_module``); storage is device memory held in
``torch`` tensors and every computation is a call into ``libnf4b200.so``.  ``torch`` is
used for memory and streams only.  There is no CPU path: without the CUDA library every
method raises.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import DTYPE_BF16, DTYPE_F32, LAYOUT_IN_OUT, LAYOUT_OUT_IN, LinearArgs

BLOCK_SIZE = 64  # src/quantize.rs:37


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{what} must live on a CUDA device (this package has no CPU path)")


def nf4_levels() -> torch.Tensor:
    """``NF4_LEVELS`` (src/quantize.rs:49-66) as a CPU f32 tensor."""
    buf = (ctypes.c_float * 16)()
    _lib.load().nf4_levels(buf)
    return torch.tensor(list(buf), dtype=torch.float32)


def _flat_f32(values: torch.Tensor) -> torch.Tensor:
    _require_cuda(values, "values")
    return values.detach().to(torch.float32).contiguous().view(-1)


class PackedNf4Tensor:
    """Packed 4-bit NF4 storage resident on the GPU (src/quantize.rs:248-400).

    Two codes per byte, low nibble first; one f32 absmax per 64-block, or 8-bit scale
    codes plus one f32 scale of scales after :meth:`with_double_quantization`.
    """

    def __init__(self, codes: torch.Tensor, length: int, absmax: Optional[torch.Tensor],
                 scale_codes: Optional[torch.Tensor] = None,
                 scale_of_scales: Optional[torch.Tensor] = None):
        self.codes = codes
        self._len = int(length)
        self._num_blocks = (self._len + BLOCK_SIZE - 1) // BLOCK_SIZE
        self.absmax = absmax
        self.scale_codes = scale_codes
        self.scale_of_scales = scale_of_scales  # 1-element f32 device tensor

    # -- construction ----------------------------------------------------------------
    @staticmethod
    def quantize(values: torch.Tensor) -> "PackedNf4Tensor":
        """``PackedNf4Tensor::quantize`` (src/quantize.rs:262-279) on the device."""
        v = _flat_f32(values)
        n = v.numel()
        dev = v.device
        codes = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
        absmax = torch.empty((n + BLOCK_SIZE - 1) // BLOCK_SIZE, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_quantize_dev(_ptr(v), n, _ptr(codes), _ptr(absmax),
                                                    _stream(dev)))
        return PackedNf4Tensor(codes, n, absmax)

    @staticmethod
    def quantize_transposed(weight: torch.Tensor) -> "PackedNf4Tensor":
        """Packed NF4 of ``weight.t()`` flattened row-major, for a 2-D f32 or bf16 ``weight`` on
        the GPU, without materialising the transpose: the reference's checkpoint load path
        (``transpose2d`` + ``PackedNf4Tensor::quantize``, src/qwennet.rs:1375-1390, 1709-1711)."""
        _require_cuda(weight, "weight")
        if weight.dim() != 2 or weight.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("weight must be a 2-D float32 or bfloat16 tensor")
        w = weight.contiguous()
        rows, cols = w.shape
        n = rows * cols
        dev = w.device
        codes = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
        absmax = torch.empty((n + BLOCK_SIZE - 1) // BLOCK_SIZE, dtype=torch.float32, device=dev)
        lib = _lib.load()
        ws_bytes = int(lib.nf4_quantize_transposed_workspace_bytes(rows, cols))
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.nf4_quantize_transposed_dev(
                _ptr(w), _lib.DTYPE_BF16 if w.dtype == torch.bfloat16 else _lib.DTYPE_F32, rows, cols,
                _ptr(codes), _ptr(absmax), _ptr(ws), ws.numel(), _stream(dev)))
        return PackedNf4Tensor(codes, n, absmax)

    def with_double_quantization(self) -> "PackedNf4Tensor":
        """src/quantize.rs:284-309; idempotent."""
        if self.is_double_quantized():
            return self
        dev = self.codes.device
        sc = torch.empty(max(self._num_blocks, 1), dtype=torch.uint8, device=dev)
        sos = torch.empty(1, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_double_quantize_dev(_ptr(self.absmax), self._num_blocks,
                                                           _ptr(sc), _ptr(sos), _stream(dev)))
        return PackedNf4Tensor(self.codes, self._len, None, sc[: self._num_blocks], sos)

    # -- queries -----------------------------------------------------------------------
    def is_double_quantized(self) -> bool:
        return self.scale_codes is not None

    def len(self) -> int:
        return self._len

    def __len__(self) -> int:
        return self._len

    def is_empty(self) -> bool:
        return self._len == 0

    def num_blocks(self) -> int:
        return self._num_blocks

    def dequantize(self) -> torch.Tensor:
        """src/quantize.rs:355-366: flat f32 device tensor of ``len()`` values."""
        dev = self.codes.device
        out = torch.empty(self._len, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_dequantize_dev(
                _ptr(self.codes), self._len, _ptr(self.absmax), _ptr(self.scale_codes),
                _ptr(self.scale_of_scales), _ptr(out), _stream(dev)))
        return out

    def resident_bytes(self) -> int:
        """src/quantize.rs:370-376."""
        scale_bytes = (self.scale_codes.numel() + 4) if self.is_double_quantized() \
            else 4 * self.absmax.numel()
        return self.codes.numel() + scale_bytes

    def bits_per_value(self) -> float:
        return 0.0 if self._len == 0 else 8.0 * self.resident_bytes() / self._len

    @staticmethod
    def estimated_resident_bytes(length: int, double_quantized: bool) -> int:
        """src/quantize.rs:391-399."""
        return int(_lib.load().nf4_estimated_resident_bytes(length, int(double_quantized)))

    def __eq__(self, other) -> bool:
        """Derived ``PartialEq`` of the reference: codes, len, num_blocks and scales."""
        if not isinstance(other, PackedNf4Tensor):
            return NotImplemented
        if (self._len, self._num_blocks, self.is_double_quantized()) != \
                (other._len, other._num_blocks, other.is_double_quantized()):
            return False
        if not torch.equal(self.codes, other.codes):
            return False
        if self.is_double_quantized():
            return torch.equal(self.scale_codes, other.scale_codes) and \
                torch.equal(self.scale_of_scales, other.scale_of_scales)
        return torch.equal(self.absmax, other.absmax)

    __hash__ = None


class Nf4Tensor:
    """The simulated one-code-per-byte form (src/quantize.rs:78-201)."""

    def __init__(self, codes, length, absmax, scale_codes=None, scale_of_scales=None):
        self.codes = codes
        self._len = int(length)
        self._num_blocks = (self._len + BLOCK_SIZE - 1) // BLOCK_SIZE
        self.absmax = absmax
        self.scale_codes = scale_codes
        self.scale_of_scales = scale_of_scales

    @staticmethod
    def quantize(values: torch.Tensor) -> "Nf4Tensor":
        v = _flat_f32(values)
        n = v.numel()
        dev = v.device
        codes = torch.empty(n, dtype=torch.uint8, device=dev)
        absmax = torch.empty((n + BLOCK_SIZE - 1) // BLOCK_SIZE, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_quantize_unpacked_dev(_ptr(v), n, _ptr(codes), _ptr(absmax),
                                                             _stream(dev)))
        return Nf4Tensor(codes, n, absmax)

    def with_double_quantization(self) -> "Nf4Tensor":
        dev = self.codes.device
        sc = torch.empty(max(self._num_blocks, 1), dtype=torch.uint8, device=dev)
        sos = torch.empty(1, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_double_quantize_dev(_ptr(self.absmax), self._num_blocks,
                                                           _ptr(sc), _ptr(sos), _stream(dev)))
        return Nf4Tensor(self.codes, self._len, self.absmax, sc[: self._num_blocks], sos)

    def is_double_quantized(self) -> bool:
        return self.scale_codes is not None

    def len(self) -> int:
        return self._len

    def is_empty(self) -> bool:
        return self._len == 0

    def num_blocks(self) -> int:
        return self._num_blocks

    def dequantize(self) -> torch.Tensor:
        dev = self.codes.device
        out = torch.empty(self._len, dtype=torch.float32, device=dev)
        dq = self.is_double_quantized()
        with torch.cuda.device(dev):
            _lib.check(_lib.load().nf4_dequantize_unpacked_dev(
                _ptr(self.codes), self._len, None if dq else _ptr(self.absmax),
                _ptr(self.scale_codes), _ptr(self.scale_of_scales), _ptr(out), _stream(dev)))
        return out

    def bits_per_value(self) -> float:
        """src/quantize.rs:190-200."""
        if self._len == 0:
            return 0.0
        scales = (8.0 * self._num_blocks + 32.0) if self.is_double_quantized() \
            else 32.0 * self._num_blocks
        return (4.0 * self._len + scales) / self._len


def quantize_dequantize_tensor(tensor: torch.Tensor, double_quantization: bool) -> torch.Tensor:
    """src/quantize.rs:404-416: the error a frozen NF4 weight carries, same shape back."""
    v = _flat_f32(tensor)
    n = v.numel()
    dev = v.device
    lib = _lib.load()
    out = torch.empty_like(v)
    ws_bytes = int(lib.nf4_quantize_dequantize_workspace_bytes(n))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_quantize_dequantize_dev(_ptr(v), n, int(double_quantization), _ptr(out),
                                                   _ptr(ws), ws_bytes, _stream(dev)))
    return out.view(tensor.shape)


def quantize_module(module: torch.nn.Module, double_quantization: bool,
                    skip: Sequence[str] = ()) -> Tuple[torch.nn.Module, int]:
    """src/quantize.rs:426-511: put every weight-shaped parameter on the NF4 grid in place.

    Parameters of rank < 2, with fewer than 64 values, or with a path component (a module or
    field name between the dots) that contains any entry of ``skip`` are left untouched, as
    ``Nf4Quantizer::is_skipped`` decides it (src/quantize.rs:454-458).  Returns the module and
    the number of values quantized."""
    count = 0
    with torch.no_grad():
        for name, param in module.named_parameters():
            skipped = any(needle in part for needle in skip for part in name.split("."))
            if param.dim() < 2 or param.numel() < BLOCK_SIZE or skipped:
                continue
            param.copy_(quantize_dequantize_tensor(param.data, double_quantization))
            param.requires_grad_(False)
            count += param.numel()
    return module, count


@dataclass
class LoraConfig:
    """src/quantize.rs:514-548."""

    in_features: int
    out_features: int
    rank: int
    alpha: float = None

    def __post_init__(self):
        self.rank = max(int(self.rank), 1)
        if self.alpha is None:
            self.alpha = float(self.rank)

    @staticmethod
    def new(in_features: int, out_features: int, rank: int) -> "LoraConfig":
        return LoraConfig(in_features, out_features, rank)

    def with_alpha(self, alpha: float) -> "LoraConfig":
        return LoraConfig(self.in_features, self.out_features, self.rank, float(alpha))

    def scaling(self) -> float:
        return self.alpha / max(self.rank, 1)

    def num_parameters(self) -> int:
        return self.rank * (self.in_features + self.out_features)


class LoraAdapter:
    """Low-rank update with ``A [in, rank] ~ N(0, 1/sqrt(rank))`` and ``B [rank, out] = 0``
    (src/quantize.rs:550-635).  ``forward`` is ``((x A) B) * scaling``."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, scaling: float):
        self._a, self._b, self._scaling = a, b, float(scaling)

    @staticmethod
    def new(config: LoraConfig, device, dtype=torch.float32, generator=None) -> "LoraAdapter":
        std = 1.0 / math.sqrt(max(config.rank, 1))
        a = torch.randn(config.in_features, config.rank, device=device, dtype=torch.float32,
                        generator=generator) * std
        b = torch.zeros(config.rank, config.out_features, device=device, dtype=torch.float32)
        return LoraAdapter(a.to(dtype), b.to(dtype), config.scaling())

    @staticmethod
    def from_parts(a: torch.Tensor, b: torch.Tensor, scaling: float) -> "LoraAdapter":
        return LoraAdapter(a.detach(), b.detach(), scaling)

    def a(self) -> torch.Tensor:
        return self._a

    def b(self) -> torch.Tensor:
        return self._b

    def in_features(self) -> int:
        return self._a.shape[0]

    def out_features(self) -> int:
        return self._b.shape[1]

    def rank(self) -> int:
        return self._a.shape[1]

    def scaling(self) -> float:
        return self._scaling

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``((x A) B) * scaling`` for ``x [rows, in]`` (src/quantize.rs:620-624)."""
        return lora_forward(x, self._a, self._b, self._scaling)

    def delta_weight(self) -> torch.Tensor:
        """``(A B) * scaling`` as f32 ``[in, out]`` (src/quantize.rs:629-634); for merging and
        verification, not for the forward path."""
        return lora_delta_weight(self._a, self._b, self._scaling)


def _io_dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"activations must be bf16 or f32, got {t.dtype}")


def lora_forward(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scaling: float) -> torch.Tensor:
    """``LoraAdapter::forward`` (src/quantize.rs:620-624) with the reference's factor shapes
    ``A [in, rank]``, ``B [rank, out]``, through ``nf4_lora_forward_dev``."""
    _require_cuda(x, "x")
    lib = _lib.load()
    d_in, rank = a.shape
    d_out = b.shape[1]
    x2 = x.contiguous().view(-1, d_in)
    rows, dev = x2.shape[0], x2.device
    a2, b2 = a.to(x2.dtype).contiguous(), b.to(x2.dtype).contiguous()
    y = torch.empty(rows, d_out, dtype=x2.dtype, device=dev)
    ws = torch.empty(max(int(lib.nf4_lora_workspace_bytes(rows, rank)), 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_lora_forward_dev(_ptr(x2), rows, d_in, d_out, _ptr(a2), _ptr(b2), rank,
                                            float(scaling), LAYOUT_IN_OUT, _io_dtype(x2), _ptr(y), d_out,
                                            _ptr(ws), ws.numel(), _stream(dev)))
    return y.view(*x.shape[:-1], d_out)


def lora_delta_weight(a: torch.Tensor, b: torch.Tensor, scaling: float) -> torch.Tensor:
    """``LoraAdapter::delta_weight`` (src/quantize.rs:629-634): f32 ``[in, out]``."""
    _require_cuda(a, "a")
    lib = _lib.load()
    d_in, rank = a.shape
    d_out = b.shape[1]
    dev = a.device
    a2 = a.contiguous()
    b2 = b.to(a2.dtype).contiguous()
    out = torch.empty(d_in, d_out, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_lora_delta_weight_dev(_ptr(a2), _ptr(b2), d_in, d_out, rank, float(scaling),
                                                 LAYOUT_IN_OUT, _io_dtype(a2), _ptr(out), _stream(dev)))
    return out


def qlora_merge(packed: "PackedNf4Tensor", d_in: int, d_out: int, a: torch.Tensor, b: torch.Tensor,
                scaling: float, layout: int = LAYOUT_IN_OUT) -> torch.Tensor:
    """``dequant(W) + (A B) * scaling`` in f32, in the weight's orientation
    (``QLoraLinear::merged``, src/quantize.rs:717-726)."""
    lib = _lib.load()
    dev = packed.codes.device
    rank = a.shape[1] if layout == LAYOUT_IN_OUT else a.shape[0]
    a2 = a.contiguous()
    b2 = b.to(a2.dtype).contiguous()
    shape = (d_in, d_out) if layout == LAYOUT_IN_OUT else (d_out, d_in)
    out = torch.empty(shape, dtype=torch.float32, device=dev)
    dq = packed.is_double_quantized()
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_qlora_merge_dev(
            _ptr(packed.codes), None if dq else _ptr(packed.absmax),
            _ptr(packed.scale_codes) if dq else None, _ptr(packed.scale_of_scales) if dq else None,
            d_in, d_out, layout, _ptr(a2), _ptr(b2), rank, float(scaling), _io_dtype(a2), _ptr(out),
            _stream(dev)))
    return out


def _linear_args(lib, x2: torch.Tensor, packed: PackedNf4Tensor, d_in: int, d_out: int, layout: int, bias, lora_a,
                 lora_b, lora_scale: float, out):
    """The argument block of one forward, its output, and the tensors that must outlive the launch."""
    dev = x2.device
    rows = x2.shape[0]
    rank = 0
    if lora_a is not None:
        rank = lora_a.shape[0] if layout == LAYOUT_OUT_IN else lora_a.shape[1]
        lora_a = lora_a.to(x2.dtype).contiguous()
        lora_b = lora_b.to(x2.dtype).contiguous()
    y = out if out is not None else torch.empty(rows, d_out, dtype=x2.dtype, device=dev)
    ws_bytes = int(lib.nf4_linear_workspace_bytes(rows, d_in, d_out, rank))
    # the decode kernel's flag words at the start of the workspace must start at zero; the rest
    # (tens of megabytes at prefill sizes) needs no initialisation
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    ws[:256].zero_()
    bias32 = bias.to(torch.float32).contiguous() if bias is not None else None
    a = LinearArgs()
    a.struct_bytes = ctypes.sizeof(LinearArgs)
    a.layout, a.io_dtype = layout, _io_dtype(x2)
    a.rows, a.d_in, a.d_out = rows, d_in, d_out
    a.x = x2.data_ptr()
    a.packed = packed.codes.data_ptr()
    a.absmax = packed.absmax.data_ptr() if not packed.is_double_quantized() else None
    a.scale_codes = packed.scale_codes.data_ptr() if packed.is_double_quantized() else None
    a.scale_of_scales = packed.scale_of_scales.data_ptr() if packed.is_double_quantized() else None
    a.bias = bias32.data_ptr() if bias32 is not None else None
    a.lora_a = lora_a.data_ptr() if rank else None
    a.lora_b = lora_b.data_ptr() if rank else None
    a.lora_rank, a.lora_scale = rank, float(lora_scale)
    a.y, a.ldy = y.data_ptr(), y.stride(0)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a, y, (ws, bias32, lora_a, lora_b, x2)


def linear_forward(x: torch.Tensor, packed: PackedNf4Tensor, d_in: int, d_out: int, layout: int,
                   bias: Optional[torch.Tensor] = None, lora_a: Optional[torch.Tensor] = None,
                   lora_b: Optional[torch.Tensor] = None, lora_scale: float = 0.0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One NF4 / QLoRA linear forward through ``nf4_linear_forward_dev``.

    ``x [..., d_in]`` (bf16 or f32); leading dims are flattened as the reference does
    (src/qwennet.rs:326-342).  ``layout`` selects ``W [d_out, d_in]`` (LAYOUT_OUT_IN, LoRA
    ``A [r, d_in]``, ``B [d_out, r]``) or the reference's ``W [d_in, d_out]``
    (LAYOUT_IN_OUT, ``A [d_in, r]``, ``B [r, d_out]``)."""
    _require_cuda(x, "x")
    lib = _lib.load()
    dev = x.device
    lead = x.shape[:-1]
    x2 = x.contiguous().view(-1, d_in)
    a, y, _alive = _linear_args(lib, x2, packed, d_in, d_out, layout, bias, lora_a, lora_b, lora_scale, out)
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_linear_forward_dev(ctypes.byref(a), _stream(dev)))
    return y.view(*lead, d_out) if out is None else y


def linear_forward_grouped(x: torch.Tensor, d_in: int, layout: int, projections) -> list:
    """Several projections of the same ``x`` through ``nf4_linear_forward_grouped_dev`` (one kernel
    launch where the shapes allow it).  ``projections``: up to four dicts with ``packed`` and
    ``d_out`` and optionally ``bias``, ``lora_a``, ``lora_b``, ``lora_scale``.  The outputs equal
    those of one ``linear_forward`` per projection, which is what the reference does
    (src/qwennet.rs:372-383 per projection)."""
    _require_cuda(x, "x")
    lib = _lib.load()
    dev = x.device
    lead = x.shape[:-1]
    x2 = x.contiguous().view(-1, d_in)
    block = (LinearArgs * len(projections))()
    ys, alive = [], []
    for i, pr in enumerate(projections):
        a, y, keep = _linear_args(lib, x2, pr["packed"], d_in, pr["d_out"], layout, pr.get("bias"),
                                  pr.get("lora_a"), pr.get("lora_b"), pr.get("lora_scale", 0.0), None)
        block[i] = a
        ys.append(y.view(*lead, pr["d_out"]))
        alive.append(keep)
    with torch.cuda.device(dev):
        _lib.check(lib.nf4_linear_forward_grouped_dev(block, len(projections), _stream(dev)))
    return ys


class QLoraLinear:
    """A linear layer with a frozen NF4-quantized base weight (held dequantized, on the
    grid) plus an adapter: the simulated form of src/quantize.rs:637-727."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], adapter: LoraAdapter,
                 quantized_values: int, double_quantized: bool):
        self.weight = weight  # [in, out] f32, already on the NF4 grid
        self.bias = bias
        self._adapter = adapter
        self.quantized_values = quantized_values
        self.double_quantized = double_quantized
        self._packed = None   # the packed form of `weight`, made once (the weight is frozen)

    @staticmethod
    def from_linear(weight: torch.Tensor, bias: Optional[torch.Tensor], config: LoraConfig,
                    double_quantization: bool, generator=None) -> "QLoraLinear":
        """``weight`` is ``[in_features, out_features]`` as Burn's ``Linear`` stores it."""
        q = quantize_dequantize_tensor(weight, double_quantization)
        adapter = LoraAdapter.new(config, weight.device, generator=generator)
        return QLoraLinear(q, bias, adapter, weight.numel(), double_quantization)

    @staticmethod
    def new(in_features: int, out_features: int, config: LoraConfig, double_quantization: bool,
            device, generator=None) -> "QLoraLinear":
        """A fresh quantized and adapted layer with a bias (src/quantize.rs:678-690): the base is
        initialised as Burn's ``LinearConfig`` does, uniform in ``+-1/sqrt(in_features)``."""
        bound = 1.0 / math.sqrt(in_features)
        w = (torch.rand(in_features, out_features, device=device, generator=generator) * 2 - 1) * bound
        b = (torch.rand(out_features, device=device, generator=generator) * 2 - 1) * bound
        return QLoraLinear.from_linear(w, b, config, double_quantization, generator=generator)

    def adapter(self) -> LoraAdapter:
        return self._adapter

    def packed(self) -> PackedNf4Tensor:
        """The frozen weight in packed form; quantizing a weight that is already on the NF4 grid
        (with the scales it was dequantized with) gives back its codes, so this is exact."""
        if self._packed is None:
            self._packed = PackedNf4Tensor.quantize(self.weight)
        return self._packed

    def base_forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_forward(x, self.packed(), self.weight.shape[0], self.weight.shape[1], LAYOUT_IN_OUT,
                              bias=self.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``base(x) + adapter(x)`` (src/quantize.rs:692-694) in one fused call."""
        return linear_forward(x, self.packed(), self.weight.shape[0], self.weight.shape[1], LAYOUT_IN_OUT,
                              bias=self.bias, lora_a=self._adapter.a(), lora_b=self._adapter.b(),
                              lora_scale=self._adapter.scaling())

    def resident_bits(self) -> Tuple[float, float]:
        """src/quantize.rs:701-712."""
        blocks = math.ceil(self.quantized_values / BLOCK_SIZE)
        scale_bits = 8.0 * blocks + 32.0 if self.double_quantized else 32.0 * blocks
        return 4.0 * self.quantized_values + scale_bits, 32.0 * self.quantized_values

    def merged(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``W + dW`` as a plain ``[in, out]`` f32 weight and the bias (src/quantize.rs:717-726)."""
        w = qlora_merge(self.packed(), self.weight.shape[0], self.weight.shape[1], self._adapter.a(),
                        self._adapter.b(), self._adapter.scaling(), LAYOUT_IN_OUT)
        return w, self.bias
