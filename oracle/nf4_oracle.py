"""ctypes/numpy front-end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

The shared object built from ``nf4_oracle.c`` restates the reference crate's
``src/quantize.rs`` arithmetic; this module only marshals numpy arrays into it.
Nothing in the shipped package imports this file: the test-suite, the smoke
check and the CPU-baseline leg of the benchmark are its only users.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnf4oracle.so")

BLOCK_SIZE = 64


def build(force: bool = False) -> str:
    """Compile ``nf4_oracle.c`` into ``libnf4oracle.so`` (gcc, strict IEEE flags)."""
    src = os.path.join(_HERE, "nf4_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libnf4oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        c = ctypes
        vp, sz = c.c_void_p, c.c_size_t
        L.nf4o_levels.argtypes = [vp]
        L.nf4o_nearest_level_code.argtypes = [c.c_float]
        L.nf4o_nearest_level_code.restype = c.c_uint8
        L.nf4o_nearest_level_codes.argtypes = [vp, sz, vp]
        L.nf4o_num_blocks.argtypes = [sz]
        L.nf4o_num_blocks.restype = sz
        L.nf4o_quantize_simulated.argtypes = [vp, sz, vp, vp]
        L.nf4o_pack_codes.argtypes = [vp, sz, vp]
        L.nf4o_quantize_packed.argtypes = [vp, sz, vp, vp, vp]
        L.nf4o_double_quantize.argtypes = [vp, sz, vp, vp]
        L.nf4o_block_scale_dq.argtypes = [c.c_uint8, c.c_float]
        L.nf4o_block_scale_dq.restype = c.c_float
        L.nf4o_dequantize_packed.argtypes = [vp, sz, vp, vp, c.c_float, vp]
        L.nf4o_dequantize_simulated.argtypes = [vp, sz, vp, vp, c.c_float, vp]
        L.nf4o_estimated_resident_bytes.argtypes = [sz, c.c_int]
        L.nf4o_estimated_resident_bytes.restype = sz
        L.nf4o_bits_per_value_simulated.argtypes = [sz, c.c_int]
        L.nf4o_bits_per_value_simulated.restype = c.c_double
        L.nf4o_quantize_dequantize.argtypes = [vp, sz, c.c_int, vp, vp, vp, vp]
        L.nf4o_linear_in_out.argtypes = [vp, sz, sz, sz, vp, vp, vp]
        L.nf4o_linear_out_in.argtypes = [vp, sz, sz, sz, vp, vp, vp]
        L.nf4o_lora_forward.argtypes = [vp, sz, sz, sz, sz, vp, vp, c.c_double, vp]
        L.nf4o_lora_delta_weight.argtypes = [sz, sz, sz, vp, vp, c.c_double, vp]
        L.nf4o_lcg_fill.argtypes = [vp, vp, sz]
        L.nf4o_round_bf16.argtypes = [c.c_float]
        L.nf4o_round_bf16.restype = c.c_float
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def levels() -> np.ndarray:
    out = np.empty(16, np.float32)
    lib().nf4o_levels(_p(out))
    return out


def nearest_level_codes(v) -> np.ndarray:
    v = _f32(v).ravel()
    out = np.empty(v.size, np.uint8)
    lib().nf4o_nearest_level_codes(_p(v), v.size, _p(out))
    return out


def num_blocks(n: int) -> int:
    return (n + BLOCK_SIZE - 1) // BLOCK_SIZE


def quantize_simulated(values):
    """``Nf4Tensor::quantize``: (one code per byte, absmax per block)."""
    v = _f32(values).ravel()
    codes = np.empty(v.size, np.uint8)
    absmax = np.empty(num_blocks(v.size), np.float32)
    lib().nf4o_quantize_simulated(_p(v), v.size, _p(codes), _p(absmax))
    return codes, absmax


def quantize_packed(values):
    """``PackedNf4Tensor::quantize``: (ceil(len/2) packed bytes, absmax per block)."""
    v = _f32(values).ravel()
    packed = np.empty((v.size + 1) // 2, np.uint8)
    absmax = np.empty(num_blocks(v.size), np.float32)
    scratch = np.empty(v.size, np.uint8)
    lib().nf4o_quantize_packed(_p(v), v.size, _p(packed), _p(absmax), _p(scratch))
    return packed, absmax


def double_quantize(absmax):
    a = _f32(absmax).ravel()
    codes = np.empty(a.size, np.uint8)
    sos = np.zeros(1, np.float32)
    lib().nf4o_double_quantize(_p(a), a.size, _p(codes), _p(sos))
    return codes, np.float32(sos[0])


def block_scales_dq(scale_codes, scale_of_scales) -> np.ndarray:
    c = np.ascontiguousarray(scale_codes, np.uint8)
    return np.array([lib().nf4o_block_scale_dq(int(x), float(scale_of_scales)) for x in c],
                    dtype=np.float32)


def dequantize_packed(packed, n, absmax=None, scale_codes=None, scale_of_scales=0.0):
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.empty(n, np.float32)
    am = _f32(absmax) if absmax is not None else None
    sc = np.ascontiguousarray(scale_codes, np.uint8) if scale_codes is not None else None
    lib().nf4o_dequantize_packed(_p(packed), n, _p(am) if am is not None else None,
                                 _p(sc) if sc is not None else None,
                                 float(scale_of_scales), _p(out))
    return out


def dequantize_simulated(codes, n, absmax=None, scale_codes=None, scale_of_scales=0.0):
    codes = np.ascontiguousarray(codes, np.uint8)
    out = np.empty(n, np.float32)
    am = _f32(absmax) if absmax is not None else None
    sc = np.ascontiguousarray(scale_codes, np.uint8) if scale_codes is not None else None
    lib().nf4o_dequantize_simulated(_p(codes), n, _p(am) if am is not None else None,
                                    _p(sc) if sc is not None else None,
                                    float(scale_of_scales), _p(out))
    return out


def quantize_dequantize(values, double_quantization: bool) -> np.ndarray:
    v = _f32(values).ravel()
    nb = num_blocks(v.size)
    out = np.empty(v.size, np.float32)
    wc = np.empty(v.size, np.uint8)
    wa = np.empty(nb, np.float32)
    ws = np.empty(nb, np.uint8)
    lib().nf4o_quantize_dequantize(_p(v), v.size, int(double_quantization), _p(out), _p(wc),
                                   _p(wa), _p(ws))
    return out


def estimated_resident_bytes(n: int, double_quantized: bool) -> int:
    return int(lib().nf4o_estimated_resident_bytes(n, int(double_quantized)))


def bits_per_value_simulated(n: int, double_quantized: bool) -> float:
    return float(lib().nf4o_bits_per_value_simulated(n, int(double_quantized)))


def linear_in_out(x, w, bias=None) -> np.ndarray:
    """y = x @ W (+bias), W [d_in, d_out] as Burn's ``Linear`` stores it; f64 accumulate."""
    x = _f32(x)
    w = _f32(w)
    rows, d_in = x.shape
    d_out = w.shape[1]
    y = np.empty((rows, d_out), np.float64)
    b = _f32(bias) if bias is not None else None
    lib().nf4o_linear_in_out(_p(x), rows, d_in, d_out, _p(w), _p(b) if b is not None else None,
                             _p(y))
    return y


def linear_out_in(x, w, bias=None) -> np.ndarray:
    """y = x @ W^T (+bias), W [d_out, d_in]; f64 accumulate (plain C loops: small cases)."""
    x = _f32(x)
    w = _f32(w)
    rows, d_in = x.shape
    d_out = w.shape[0]
    y = np.empty((rows, d_out), np.float64)
    b = _f32(bias) if bias is not None else None
    lib().nf4o_linear_out_in(_p(x), rows, d_in, d_out, _p(w), _p(b) if b is not None else None,
                             _p(y))
    return y


def lora_forward(x, a, b, scaling: float) -> np.ndarray:
    """``LoraAdapter::forward``: ((x A) B) * scaling with A [d_in, r], B [r, d_out]."""
    x, a, b = _f32(x), _f32(a), _f32(b)
    rows, d_in = x.shape
    rank, d_out = b.shape
    y = np.empty((rows, d_out), np.float64)
    lib().nf4o_lora_forward(_p(x), rows, d_in, rank, d_out, _p(a), _p(b), float(scaling), _p(y))
    return y


def lora_delta_weight(a, b, scaling: float) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    d_in, rank = a.shape
    d_out = b.shape[1]
    dw = np.empty((d_in, d_out), np.float64)
    lib().nf4o_lora_delta_weight(d_in, rank, d_out, _p(a), _p(b), float(scaling), _p(dw))
    return dw


def lcg_fill(state: int, n: int):
    """The reference's fixture LCG (qwennet.rs:2567-2575); returns (values, new_state)."""
    st = np.array([state], np.uint64)
    out = np.empty(n, np.float32)
    lib().nf4o_lcg_fill(_p(st), _p(out), n)
    return out, int(st[0])


def round_bf16(x) -> np.ndarray:
    """f32 -> nearest-even bf16 grid, vectorised in numpy (same rule as nf4o_round_bf16)."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    special = (u & 0x7F800000) == 0x7F800000
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    r = np.where(special, u.astype(np.uint32), r)
    return r.view(np.float32).reshape(np.shape(x))


def qlora_forward_bnb(x, packed, absmax, d_out, d_in, lora_a=None, lora_b=None, scale=0.0,
                      bias=None, scale_codes=None, scale_of_scales=0.0) -> np.ndarray:
    """Measured-configuration forward: y = x W^T + s (x A^T) B^T with W [d_out, d_in]
    quantized along d_in, A [r, d_in], B [d_out, r].  Weights are the bit-exact
    dequantized f32 values; every product is accumulated in f64 (BLAS dgemm)."""
    w = dequantize_packed(packed, d_out * d_in, absmax, scale_codes, scale_of_scales)
    w = w.reshape(d_out, d_in).astype(np.float64)
    x64 = np.asarray(x, np.float64)
    y = x64 @ w.T
    if lora_a is not None:
        t = x64 @ np.asarray(lora_a, np.float64).T
        y = y + (t @ np.asarray(lora_b, np.float64).T) * float(np.float32(scale))
    if bias is not None:
        y = y + np.asarray(bias, np.float64)[None, :]
    return y


def qlora_forward_burn(x, packed, absmax, d_in, d_out, lora_a=None, lora_b=None, scale=0.0,
                       bias=None, scale_codes=None, scale_of_scales=0.0) -> np.ndarray:
    """Reference-orientation forward (qwennet.rs:230-241, 325-344): W [d_in, d_out] flat
    blocks, A [d_in, r], B [r, d_out]; y = x W + ((x A) B) s (+ bias)."""
    w = dequantize_packed(packed, d_in * d_out, absmax, scale_codes, scale_of_scales)
    w = w.reshape(d_in, d_out).astype(np.float64)
    x64 = np.asarray(x, np.float64)
    y = x64 @ w
    if lora_a is not None:
        y = y + ((x64 @ np.asarray(lora_a, np.float64)) @ np.asarray(lora_b, np.float64)) \
            * float(np.float32(scale))
    if bias is not None:
        y = y + np.asarray(bias, np.float64)[None, :]
    return y
