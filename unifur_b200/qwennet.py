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
        gradients are small dense products."""
        d_in, d_out, s = self.base.d_input(), self.base.d_output(), self.scaling
        x2 = x.reshape(-1, d_in)
        g2 = grad_y.reshape(-1, d_out)
        if self.base.layout == LAYOUT_OUT_IN:
            # forward: y = x W^T + s (x A^T) B^T with W [d_out, d_in], A [r, d_in], B [d_out, r]
            gx = linear_forward(g2, self.base.packed(), d_out, d_in, LAYOUT_IN_OUT,
                                lora_a=self.lora_b, lora_b=self.lora_a, lora_scale=s)
            gb_t = g2.float().t() @ (x2.float() @ self.lora_a.float().t())   # [d_out, r]
            ga_t = (g2.float() @ self.lora_b.float()).t() @ x2.float()       # [r, d_in]
            ga, gb = s * ga_t, s * gb_t
        else:
            # forward: y = x W + s (x A) B with W [d_in, d_out], A [d_in, r], B [r, d_out]
            gx = linear_forward(g2, self.base.packed(), d_out, d_in, LAYOUT_OUT_IN,
                                lora_a=self.lora_b, lora_b=self.lora_a, lora_scale=s)
            ga = s * (x2.float().t() @ (g2.float() @ self.lora_b.float().t()))   # [d_in, r]
            gb = s * ((x2.float() @ self.lora_a.float()).t() @ g2.float())       # [r, d_out]
        return gx.reshape(x.shape), ga.to(self.lora_a.dtype), gb.to(self.lora_b.dtype)

    def resident_bytes(self) -> int:
        """src/qwennet.rs:362-366."""
        r = self.lora_a.shape[0] if self.base.layout == LAYOUT_OUT_IN else self.lora_a.shape[1]
        return self.base.resident_bytes() + 4 * (self.base.d_input() + self.base.d_output()) * r


def with_lora(base: Nf4Linear, rank: int, alpha: float, generator=None) -> QloraLinear:
    """``QwenLinear::with_lora`` (src/qwennet.rs:419-434): attach a fresh zero-B adapter.
    Rank 0 and non-finite alpha are refused as ``QwenLoraConfig::validate`` does."""
    if rank < 1:
        raise ValueError("LoRA rank must be at least 1")
    if not (alpha == alpha and abs(alpha) != float("inf")):
        raise ValueError("LoRA alpha must be finite")
    cfg = LoraConfig.new(base.d_input(), base.d_output(), rank).with_alpha(alpha)
    return QloraLinear.with_adapter(base, LoraAdapter.new(cfg, base.packed().codes.device,
                                                         generator=generator))


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
