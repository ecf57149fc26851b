"""The allocation-free decode entry point gives what the ordinary entry point gives.

`nf4_linear_forward_noalloc_dev` serves callers that hold nothing but the device pointers they
were handed -- a plug-in inside another runtime's memory pool, an FFI shim without an allocator
-- and therefore cannot provide a workspace.  Its scratch is a fixed 4352-byte array inside the
library (two flag words and the adapter intermediate).  This file is collected last on purpose: a run that stops at the first failure has by
then exercised every other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import DEV, dev, lib  # noqa: E402
from unifur_b200 import _lib  # noqa: E402


def build_args(x, packed, absmax, la, lb, y, ws, rank, scale, rows, k, n):
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
    a.rows, a.d_in, a.d_out = rows, k, n
    a.x, a.packed, a.absmax = x.data_ptr(), packed.data_ptr(), absmax.data_ptr()
    if rank:
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), rank, scale
    a.y, a.ldy = y.data_ptr(), n
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def test_noalloc_entry_point_matches_the_workspace_entry_point(oracle):
    L = lib()
    assert L.nf4_linear_noalloc_scratch_bytes() == 4352
    rng = np.random.default_rng(2024)
    k, n = 1024, 512
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed_np, absmax_np = oracle.quantize_packed(w)
    packed, absmax = dev(packed_np), dev(absmax_np)
    # two calls in a row with different rows / rank: the second finds the first one's leftovers
    for rows, rank in ((16, 64), (3, 16), (5, 0)):
        x = dev(rng.standard_normal((rows, k)).astype(np.float32), torch.bfloat16)
        la = dev((rng.standard_normal((max(rank, 1), k)) * 0.05).astype(np.float32), torch.bfloat16)
        lb = dev((rng.standard_normal((n, max(rank, 1))) * 0.05).astype(np.float32), torch.bfloat16)
        ws = torch.zeros(max(int(L.nf4_linear_workspace_bytes(rows, k, n, rank)), 256),
                         dtype=torch.uint8, device=DEV)
        y_ref = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device=DEV)
        y_new = torch.full((rows, n), -7.0, dtype=torch.bfloat16, device=DEV)
        _lib.check(L.nf4_linear_forward_dev(
            ctypes.byref(build_args(x, packed, absmax, la, lb, y_ref, ws, rank, 2.0, rows, k, n)), None))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(L.nf4_linear_forward_noalloc_dev(
            ctypes.byref(build_args(x, packed, absmax, la, lb, y_new, None, rank, 2.0, rows, k, n)), None))
        torch.cuda.synchronize()
        # no allocation anywhere: the device's free memory is what it was
        assert torch.cuda.mem_get_info()[0] == free_before
        # The two entry points may run different decode kernels (the workspace one can use
        # the split-K tensor-memory kernel, which needs more scratch than the fixed array
        # holds), so they agree to the forward's tolerance rather than bit for bit: each is
        # within rel. L2 1e-3 of the exact result before its single bf16 rounding.
        a32, b32 = y_ref.float(), y_new.float()
        assert ((a32 - b32).norm() / a32.norm()).item() <= 2 * (1e-3 + 2.0 ** -9)
        assert bool(((a32 - b32).abs() <= 2.0 ** -6 * a32.abs() + 1e-3 * a32.abs().max()).all())
        # and both agree with the oracle within the forward's tolerance (bf16 output rounding added)
        ref = oracle.qlora_forward_bnb(x.float().cpu().numpy(), packed_np, absmax_np, n, k,
                                       la.float().cpu().numpy() if rank else None,
                                       lb.float().cpu().numpy() if rank else None, 2.0)
        got = y_new.float().cpu().numpy().astype(np.float64)
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-3 + 2.0 ** -9


def test_noalloc_entry_point_refuses_what_does_not_fit():
    L = lib()
    k, n = 256, 64
    packed = torch.full((n * k // 2,), 0x77, dtype=torch.uint8, device=DEV)
    absmax = torch.zeros(n * k // 64, dtype=torch.float32, device=DEV)
    la = torch.zeros(64, k, dtype=torch.bfloat16, device=DEV)
    lb = torch.zeros(n, 64, dtype=torch.bfloat16, device=DEV)
    # prefill-sized: not a decode shape
    x = torch.zeros(32, k, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(32, n, dtype=torch.bfloat16, device=DEV)
    st = L.nf4_linear_forward_noalloc_dev(
        ctypes.byref(build_args(x, packed, absmax, la, lb, y, None, 16, 1.0, 32, k, n)), None)
    assert st == -4 and b"decode shapes" in L.nf4_last_error()
    # rank beyond the scratch
    la2 = torch.zeros(128, k, dtype=torch.bfloat16, device=DEV)
    lb2 = torch.zeros(n, 128, dtype=torch.bfloat16, device=DEV)
    x = torch.zeros(16, k, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(16, n, dtype=torch.bfloat16, device=DEV)
    st = L.nf4_linear_forward_noalloc_dev(
        ctypes.byref(build_args(x, packed, absmax, la2, lb2, y, None, 128, 1.0, 16, k, n)), None)
    assert st == -1 and b"exceeds" in L.nf4_last_error()
    torch.cuda.synchronize()
