"""Helpers shared by the GPU parity tests: device buffers through torch, calls through the C ABI."""
import ctypes

import numpy as np
import torch

from unifur_b200 import _lib

DEV = "cuda:0"


def lib():
    return _lib.load()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


def quantize_dev(values_np, packed=True):
    """values (numpy f32, flat) -> (codes numpy u8, absmax numpy f32) through nf4_quantize*_dev."""
    L = lib()
    v = dev(np.asarray(values_np, np.float32).ravel())
    n = v.numel()
    nb = (n + 63) // 64
    codes = torch.full(((n + 1) // 2 if packed else n,), 0xEE, dtype=torch.uint8, device=DEV)
    absmax = torch.full((nb,), -7.0, dtype=torch.float32, device=DEV)
    fn = L.nf4_quantize_dev if packed else L.nf4_quantize_unpacked_dev
    _lib.check(fn(ptr(v), n, ptr(codes), ptr(absmax), None))
    torch.cuda.synchronize()
    return codes.cpu().numpy(), absmax.cpu().numpy()


def dequantize_dev(codes_np, n, absmax=None, scale_codes=None, sos=None, packed=True):
    L = lib()
    c = dev(np.asarray(codes_np, np.uint8))
    am = dev(np.asarray(absmax, np.float32)) if absmax is not None else None
    sc = dev(np.asarray(scale_codes, np.uint8)) if scale_codes is not None else None
    ss = dev(np.asarray([sos], np.float32)) if sos is not None else None
    out = torch.full((n,), 123.0, dtype=torch.float32, device=DEV)
    fn = L.nf4_dequantize_dev if packed else L.nf4_dequantize_unpacked_dev
    _lib.check(fn(ptr(c), n, ptr(am), ptr(sc), ptr(ss), ptr(out), None))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def double_quantize_dev(absmax_np):
    L = lib()
    am = dev(np.asarray(absmax_np, np.float32))
    nb = am.numel()
    sc = torch.full((max(nb, 1),), 0xEE, dtype=torch.uint8, device=DEV)
    ss = torch.full((1,), -1.0, dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_double_quantize_dev(ptr(am), nb, ptr(sc), ptr(ss), None))
    torch.cuda.synchronize()
    return sc.cpu().numpy()[:nb], np.float32(ss.cpu().numpy()[0])


def bits_equal(a, b):
    """Bit-for-bit equality.  For f32 arrays a NaN matches a NaN whatever its payload: the sign
    and payload of a generated NaN (0 * inf) differ between x86, ARM and the GPU, so the
    reference itself does not pin them."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype == np.float32 and (np.isnan(a).any() or np.isnan(b).any()):
        na, nb = np.isnan(a), np.isnan(b)
        return bool(np.array_equal(na, nb)) and a[~na].tobytes() == b[~nb].tobytes()
    return a.tobytes() == b.tobytes()


def student_t(rng, n, nu=4, scale=0.02):
    """0.02 * z / sqrt(chi2_nu / nu): heavy-tailed weights with outlier blocks."""
    z = rng.standard_normal(n)
    chi = (rng.standard_normal((nu, n)) ** 2).sum(0)
    return (scale * z / np.sqrt(chi / nu)).astype(np.float32)
