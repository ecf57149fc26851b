"""Host-side mirror of the NF4-resident modules of the reference's ``src/qwennet.rs``
(``Nf4Linear`` :168-242, ``Nf4Embedding`` :253-291, ``QloraLinear`` :318-345, ``QwenLinear``
:305-435) over the C ABI."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import LAYOUT_IN_OUT, LAYOUT_OUT_IN
from .quantize import LoraAdapter, LoraConfig, PackedNf4Tensor, linear_forward


class Nf4Linear:
    """A frozen NF4-resident linear.  ``forward`` is "dequantize, then matmul" fused into
    one kernel: the f32 weight is never materialised (the reference rebuilds it on every
    call, src/qwennet.rs:230-241).

    ``layout`` is ``LAYOUT_IN_OUT`` for the reference's ``[d_input, d_output]`` row-major
    weight (blocks along the flat index) or ``LAYOUT_OUT_IN`` for ``[d_output, d_input]``
    with blocks along ``d_input``."""

    def __init__(self, packed: PackedNf4Tensor, d_input: int, d_output: int,
                 bias: Optional[torch.Tensor] = None, layout: int = LAYOUT_IN_OUT):
        if packed.len() != d_input * d_output:
            raise ValueError(f"weight of shape [{d_input}, {d_output}] carries {packed.len()} values")
        self._packed, self._d_input, self._d_output = packed, d_input, d_output
        self.bias = bias
        self.layout = layout

    @staticmethod
    def from_packed(packed: PackedNf4Tensor, d_input: int, d_output: int,
                    bias: Optional[torch.Tensor] = None, layout: int = LAYOUT_IN_OUT) -> "Nf4Linear":
        return Nf4Linear(packed, d_input, d_output, bias, layout)

    @staticmethod
    def from_values(values: torch.Tensor, d_input: int, d_output: int,
                    layout: int = LAYOUT_IN_OUT, double_quantization: bool = True) -> "Nf4Linear":
        """src/qwennet.rs:198-205 (double-quantized there)."""
        packed = PackedNf4Tensor.quantize(values)
        if double_quantization:
            packed = packed.with_double_quantization()
        return Nf4Linear(packed, d_input, d_output, None, layout)

    @staticmethod
    def from_checkpoint(weight: torch.Tensor) -> "Nf4Linear":
        """A PyTorch-style ``[out, in]`` weight (f32 or bf16, on the GPU) -> the reference's
        ``[in, out]`` NF4 linear with double quantization, as its loader builds it
        (src/qwennet.rs:1687-1726): transpose and quantize fused on the device."""
        rows, cols = weight.shape
        packed = PackedNf4Tensor.quantize_transposed(weight).with_double_quantization()
        return Nf4Linear(packed, cols, rows, None, LAYOUT_IN_OUT)

    def d_input(self) -> int:
        return self._d_input

    def d_output(self) -> int:
        return self._d_output

    def resident_bytes(self) -> int:
        return self._packed.resident_bytes()

    def packed(self) -> PackedNf4Tensor:
        return self._packed

    def dequantized_weight(self) -> torch.Tensor:
        shape = (self._d_input, self._d_output) if self.layout == LAYOUT_IN_OUT \
            else (self._d_output, self._d_input)
        return self._packed.dequantize().view(shape)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_forward(x, self._packed, self._d_input, self._d_output, self.layout,
                              bias=self.bias)


class QloraLinear:
    """Frozen packed-NF4 base plus a trainable low-rank adapter (src/qwennet.rs:318-345).

    With ``LAYOUT_IN_OUT`` the adapter factors have the reference's shapes
    ``A [d_in, r]``, ``B [r, d_out]``; with ``LAYOUT_OUT_IN`` they are ``A [r, d_in]``,
    ``B [d_out, r]``."""

    def __init__(self, base: Nf4Linear, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float):
        self.base, self.lora_a, self.lora_b, self.scaling = base, lora_a, lora_b, float(scaling)

    @staticmethod
    def with_adapter(base: Nf4Linear, adapter: LoraAdapter) -> "QloraLinear":
        a, b = adapter.a(), adapter.b()
        if base.layout == LAYOUT_OUT_IN:
            a, b = a.t().contiguous(), b.t().contiguous()
        return QloraLinear(base, a, b, adapter.scaling())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_forward(x, self.base.packed(), self.base.d_input(), self.base.d_output(),
                              self.base.layout, bias=self.base.bias, lora_a=self.lora_a,
                              lora_b=self.lora_b, lora_scale=self.scaling)

    def backward(self, x: torch.Tensor, grad_y: torch.Tensor):
        """Gradients of ``forward`` with the base weight frozen, as the reference's autodiff sees
        the detached NF4 weight (src/qwennet.rs:226-241, used by src/qwentrain.rs:421-470):
        returns ``(grad_x, grad_a, grad_b)`` with the shapes of ``x``, ``lora_a``, ``lora_b``.

        ``grad_x = grad_y . W + s (grad_y . B) . A`` is one more NF4 linear over the SAME packed
        bytes read in the other orientation (a ``[d_out, d_in]`` weight is a ``[d_in', d_out']``
        weight with ``d_in' = d_out``), with the adapter factors swapping roles; the two adapter
        gradients are small dense products.  All of it runs in ``nf4_qlora_backward_dev``."""
        lib = _lib.load()
        d_in, d_out = self.base.d_input(), self.base.d_output()
        x2 = x.reshape(-1, d_in).contiguous()
        g2 = grad_y.reshape(-1, d_out).to(x2.dtype).contiguous()
        rows, dev = x2.shape[0], x2.device
        la, lb = self.lora_a.to(x2.dtype).contiguous(), self.lora_b.to(x2.dtype).contiguous()
        rank = la.shape[0] if self.base.layout == LAYOUT_OUT_IN else la.shape[1]
        gx = torch.empty(rows, d_in, dtype=x2.dtype, device=dev)
        ga, gb = torch.empty_like(la), torch.empty_like(lb)
        ws = torch.empty(max(int(lib.nf4_qlora_backward_workspace_bytes(rows, d_in, d_out, rank)), 256),
                         dtype=torch.uint8, device=dev)
        ws[:256].zero_()   # the flag words; the rest needs no initialisation
        pk = self.base.packed()
        dq = pk.is_double_quantized()
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout = self.base.layout
        a.io_dtype = _lib.DTYPE_BF16 if x2.dtype == torch.bfloat16 else _lib.DTYPE_F32
        a.rows, a.d_in, a.d_out = rows, d_in, d_out
        a.x, a.packed = x2.data_ptr(), pk.codes.data_ptr()
        a.absmax = None if dq else pk.absmax.data_ptr()
        a.scale_codes = pk.scale_codes.data_ptr() if dq else None
        a.scale_of_scales = pk.scale_of_scales.data_ptr() if dq else None
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), rank, self.scaling
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        vp = ctypes.c_void_p
        with torch.cuda.device(dev):
            _lib.check(lib.nf4_qlora_backward_dev(
                ctypes.byref(a), vp(g2.data_ptr()), vp(gx.data_ptr()), vp(ga.data_ptr()), vp(gb.data_ptr()),
                vp(torch.cuda.current_stream(dev).cuda_stream)))
        return gx.reshape(x.shape), ga.to(self.lora_a.dtype), gb.to(self.lora_b.dtype)

    def resident_bytes(self) -> int:
        """src/qwennet.rs:362-366."""
        r = self.lora_a.shape[0] if self.base.layout == LAYOUT_OUT_IN else self.lora_a.shape[1]
        return self.base.resident_bytes() + 4 * (self.base.d_input() + self.base.d_output()) * r


def with_lora(base: Nf4Linear, rank: int, alpha: float, generator=None) -> QloraLinear:
    """``QwenLinear::with_lora`` (src/qwennet.rs:419-434) on an NF4-resident base: attach a fresh
    zero-B adapter.  Rank 0 and non-finite alpha are refused as ``QwenLoraConfig::validate`` does."""
    if rank < 1:
        raise ValueError("LoRA rank must be at least 1")
    if not (alpha == alpha and abs(alpha) != float("inf")):
        raise ValueError("LoRA alpha must be finite")
    cfg = LoraConfig.new(base.d_input(), base.d_output(), rank).with_alpha(alpha)
    return QloraLinear.with_adapter(base, LoraAdapter.new(cfg, base.packed().codes.device,
                                                         generator=generator))


class QwenLinearError(RuntimeError):
    """The ``anyhow`` errors of ``QwenLinear::to_nf4`` / ``with_lora`` (src/qwennet.rs:378-435)."""


class QwenLinear:
    """Residency switch of one projection (src/qwennet.rs:305-435): an f32 weight, an NF4-resident
    weight, or an NF4-resident weight with an adapter.  ``forward`` gives the same function in all
    three; only the memory differs."""

    F32, NF4, QLORA = "F32", "Nf4", "Qlora"

    def __init__(self, kind: str, inner, bias: Optional[torch.Tensor] = None):
        self.kind, self.inner, self._f32_bias = kind, inner, bias

    @staticmethod
    def f32(weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "QwenLinear":
        """``weight [d_input, d_output]`` f32, as Burn's ``Linear`` stores it."""
        return QwenLinear(QwenLinear.F32, weight, bias)

    @staticmethod
    def nf4(linear: Nf4Linear) -> "QwenLinear":
        return QwenLinear(QwenLinear.NF4, linear)

    @staticmethod
    def qlora(linear: QloraLinear) -> "QwenLinear":
        return QwenLinear(QwenLinear.QLORA, linear)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.kind == QwenLinear.F32:
            # the f32 variant is Burn's own Linear, outside the NF4 path: plain framework matmul
            y = x.to(self.inner.dtype) @ self.inner
            return (y + self._f32_bias if self._f32_bias is not None else y).to(x.dtype)
        return self.inner.forward(x)

    def resident_bytes(self) -> int:
        """src/qwennet.rs:356-368."""
        if self.kind == QwenLinear.F32:
            return 4 * self.inner.numel()
        return self.inner.resident_bytes()

    def to_nf4(self) -> "QwenLinear":
        """Quantize an f32 weight into NF4 residency (src/qwennet.rs:378-413).  The in-memory
        weight is already ``[d_input, d_output]`` and is NOT transposed; a bias keeps its
        identity; an NF4 weight is returned as it is; a weight carrying an adapter is an error."""
        if self.kind == QwenLinear.F32:
            d_in, d_out = self.inner.shape
            if self.inner.numel() != d_in * d_out:
                raise QwenLinearError(f"weight of shape [{d_in}, {d_out}] carries {self.inner.numel()} values")
            lin = Nf4Linear.from_values(self.inner.contiguous().view(-1).float(), d_in, d_out)
            lin.bias = self._f32_bias  # the same tensor object: its identity is kept
            return QwenLinear.nf4(lin)
        if self.kind == QwenLinear.NF4:
            return self
        raise QwenLinearError("a weight carrying an adapter must be de-adapted before conversion")

    def with_lora(self, rank: int, alpha: float, generator=None) -> "QwenLinear":
        """Attach a fresh, exactly no-op adapter to an NF4-resident base (src/qwennet.rs:419-434);
        attaching to an f32 weight or twice is an error."""
        if rank < 1:
            raise QwenLinearError("LoRA rank must be at least 1")
        if not (alpha == alpha and abs(alpha) != float("inf")):
            raise QwenLinearError("LoRA alpha must be finite")
        if self.kind == QwenLinear.NF4:
            return QwenLinear.qlora(with_lora(self.inner, rank, alpha, generator))
        if self.kind == QwenLinear.F32:
            raise QwenLinearError("LoRA adapters attach to NF4-resident weights only")
        raise QwenLinearError("weight already carries a LoRA adapter")


class Nf4Embedding:
    """A frozen NF4-resident embedding table ``[n_embedding, d_model]`` (src/qwennet.rs:253-291).

    ``forward`` gathers and dequantizes only the rows the ids select; the reference rebuilds the
    whole f32 table on every call and then gathers.  The values are bit-identical."""

    def __init__(self, packed: PackedNf4Tensor, n_embedding: int, d_model: int):
        if packed.len() != n_embedding * d_model:
            raise ValueError(f"table of shape [{n_embedding}, {d_model}] carries {packed.len()} values")
        self._packed, self._n_embedding, self._d_model = packed, n_embedding, d_model

    @staticmethod
    def from_values(values: torch.Tensor, n_embedding: int, d_model: int) -> "Nf4Embedding":
        """Quantize a row-major table with double quantization (src/qwennet.rs:265-271)."""
        return Nf4Embedding(PackedNf4Tensor.quantize(values).with_double_quantization(),
                            n_embedding, d_model)

    def resident_bytes(self) -> int:
        return self._packed.resident_bytes()

    def dequantized_weight(self) -> torch.Tensor:
        return self._packed.dequantize().view(self._n_embedding, self._d_model)

    def forward(self, ids: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """``ids`` of any shape (integer) -> ``[*ids.shape, d_model]``."""
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        p = self._packed
        dev = p.codes.device
        flat = ids.to(device=dev, dtype=torch.int64).contiguous().view(-1)
        out = torch.empty(flat.numel(), self._d_model, dtype=dtype, device=dev)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
        _lib.check(_lib.load().nf4_embedding_gather_dev(
            ptr(p.codes), ptr(p.absmax), ptr(p.scale_codes), ptr(p.scale_of_scales),
            self._n_embedding, self._d_model, ptr(flat), flat.numel(), ptr(out),
            _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_F32,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
        return out.view(*ids.shape, self._d_model)
