"""GPU tests of the reference-facing boundary beyond the plain forward: the adapter alone, its dense
update, the merge, the module quantizer, the residency switch with the reference's error cases,
the failure report, and the column-sharded forward through the C ABI.  Each test names the
reference test it restates (file:line within the reference crate)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import DEV, dev, lib  # noqa: E402
from unifur_b200 import _lib  # noqa: E402


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def test_lora_forward_matches_the_dense_update(oracle):
    # src/quantize.rs:1027-1047: factored x A B * s against x (s A B), < 1e-5, alpha / rank = 6 / 3
    from unifur_b200.quantize import LoraAdapter, LoraConfig

    g = torch.Generator(device=DEV).manual_seed(11)
    cfg = LoraConfig.new(12, 6, 3).with_alpha(6.0)
    ad = LoraAdapter.new(cfg, DEV, generator=g)
    ad = LoraAdapter.from_parts(ad.a(), torch.rand(3, 6, device=DEV, generator=g) - 0.5, ad.scaling())
    x = torch.rand(4, 12, device=DEV, generator=g) * 2 - 1
    factored = ad.forward(x)
    delta = ad.delta_weight()
    assert delta.shape == (12, 6) and delta.dtype == torch.float32
    dense = x.double() @ delta.double()
    assert (factored.double() - dense).abs().max().item() < 1e-5
    assert abs(ad.scaling() - 2.0) < 1e-12
    # and both against the oracle's restatement of src/quantize.rs:620-634, bit for bit in f32
    a_np, b_np, x_np = ad.a().cpu().numpy(), ad.b().cpu().numpy(), x.cpu().numpy()
    ref = oracle.lora_delta_weight(a_np, b_np, 2.0)
    assert np.allclose(delta.cpu().numpy(), ref, rtol=0, atol=1e-6)


@pytest.mark.parametrize("layout_name,dtype", [("in_out", "f32"), ("out_in", "f32"), ("out_in", "bf16")])
def test_lora_entry_points_in_both_orientations(layout_name, dtype):
    L = lib()
    rng = np.random.default_rng(77)
    rows, d_in, d_out, r, s = 7, 200, 136, 12, 1.5
    out_in = layout_name == "out_in"
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    a = dev((rng.standard_normal((r, d_in) if out_in else (d_in, r)) * 0.1).astype(np.float32), tdt)
    b = dev((rng.standard_normal((d_out, r) if out_in else (r, d_out)) * 0.1).astype(np.float32), tdt)
    x = dev(rng.standard_normal((rows, d_in)).astype(np.float32), tdt)
    A = (a.double().t() if out_in else a.double())      # [d_in, r]
    B = (b.double().t() if out_in else b.double())      # [r, d_out]
    lay = _lib.LAYOUT_OUT_IN if out_in else _lib.LAYOUT_IN_OUT
    io = _lib.DTYPE_F32 if dtype == "f32" else _lib.DTYPE_BF16
    y = torch.full((rows, d_out), 9.0, dtype=tdt, device=DEV)
    ws = torch.empty(max(int(L.nf4_lora_workspace_bytes(rows, r)), 256), dtype=torch.uint8, device=DEV)
    _lib.check(L.nf4_lora_forward_dev(_vp(x), rows, d_in, d_out, _vp(a), _vp(b), r, s, lay, io, _vp(y), d_out,
                                      _vp(ws), ws.numel(), None))
    ref = (x.double() @ A @ B) * s
    tol = 1e-5 if dtype == "f32" else 2.0 ** -8
    assert ((y.double() - ref).norm() / ref.norm()).item() < tol
    delta = torch.empty((d_out, d_in) if out_in else (d_in, d_out), dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_lora_delta_weight_dev(_vp(a), _vp(b), d_in, d_out, r, s, lay, io, _vp(delta), None))
    dref = (A @ B) * s
    dref = dref.t() if out_in else dref
    assert ((delta.double() - dref).norm() / dref.norm()).item() < 1e-6
    # bad arguments come back as a status, not as a fault
    assert L.nf4_lora_forward_dev(_vp(x), rows, d_in, d_out, None, _vp(b), r, s, lay, io, _vp(y), d_out,
                                  _vp(ws), ws.numel(), None) == -1
    assert L.nf4_lora_forward_dev(_vp(x), rows, d_in, d_out, _vp(a), _vp(b), r, s, lay, io, _vp(y), d_out,
                                  _vp(ws), 0, None) == -1


def test_qlora_merge_preserves_outputs():
    # src/quantize.rs:1083-1099: QLoraLinear::new (with a bias), a non-zero B, merged() gives the
    # same function to 1e-5
    from unifur_b200.quantize import BLOCK_SIZE, LoraAdapter, LoraConfig, QLoraLinear

    g = torch.Generator(device=DEV).manual_seed(5)
    cfg = LoraConfig.new(BLOCK_SIZE, 8, 2)
    q = QLoraLinear.new(BLOCK_SIZE, 8, cfg, False, DEV, generator=g)
    assert q.bias is not None and q.weight.shape == (BLOCK_SIZE, 8)
    q._adapter = LoraAdapter.from_parts(q.adapter().a(), (torch.rand(2, 8, device=DEV, generator=g) - 0.5) * 0.6,
                                        q.adapter().scaling())
    x = torch.rand(5, BLOCK_SIZE, device=DEV, generator=g) * 2 - 1
    before = q.forward(x)
    w, bias = q.merged()
    assert w.shape == (BLOCK_SIZE, 8) and w.dtype == torch.float32 and bias is q.bias
    after = x.double() @ w.double() + bias.double()
    assert (before.double() - after).abs().max().item() < 1e-5
    # merged = base weight + dense update, exactly that sum in f32
    assert torch.equal(w, q.weight + q.adapter().delta_weight())
    # the packed form of the frozen weight is made once
    assert q.packed() is q.packed()


@pytest.mark.parametrize("dq", [False, True])
def test_qlora_merge_entry_point_against_the_oracle(oracle, dq):
    L = lib()
    rng = np.random.default_rng(31)
    d_in, d_out, r, s = 96, 72, 5, 0.75
    w = (rng.standard_normal(d_in * d_out) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    wd = oracle.dequantize_packed(packed, w.size, None if dq else absmax, sc, sos if dq else 0.0)
    a = (rng.standard_normal((d_in, r)) * 0.2).astype(np.float32)
    b = (rng.standard_normal((r, d_out)) * 0.2).astype(np.float32)
    out = torch.empty(d_in, d_out, dtype=torch.float32, device=DEV)
    d_p, d_a, d_b = dev(packed), dev(a), dev(b)
    d_am = dev(absmax) if not dq else None
    d_sc = dev(sc) if dq else None
    d_ss = dev(np.asarray([sos], np.float32)) if dq else None
    _lib.check(L.nf4_qlora_merge_dev(_vp(d_p), _vp(d_am) if d_am is not None else None,
                                     _vp(d_sc) if dq else None, _vp(d_ss) if dq else None, d_in, d_out,
                                     _lib.LAYOUT_IN_OUT, _vp(d_a), _vp(d_b), r, s, _lib.DTYPE_F32, _vp(out), None))
    ref = wd.reshape(d_in, d_out).astype(np.float64) + (a.astype(np.float64) @ b.astype(np.float64)) * s
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() < 1e-6
    # where the update is zero the merged weight IS the dequantized weight, bit for bit
    _lib.check(L.nf4_qlora_merge_dev(_vp(d_p), _vp(d_am) if d_am is not None else None,
                                     _vp(d_sc) if dq else None, _vp(d_ss) if dq else None, d_in, d_out,
                                     _lib.LAYOUT_IN_OUT, _vp(d_a), _vp(torch.zeros_like(d_b)), r, s,
                                     _lib.DTYPE_F32, _vp(out), None))
    assert out.cpu().numpy().tobytes() == wd.reshape(d_in, d_out).tobytes()


def test_quantize_module_touches_only_weight_shaped_params(oracle):
    # src/quantize.rs:1101-1130: weights go onto the NF4 grid, rank-1 parameters and parameters
    # under a skipped module stay bit-identical; skip matches per path component
    # (Nf4Quantizer::is_skipped, src/quantize.rs:454-458)
    from unifur_b200.quantize import quantize_module

    torch.manual_seed(0)

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.label_embeddings = torch.nn.Embedding(10, 64)
            self.blocks = torch.nn.ModuleList([torch.nn.Linear(64, 32), torch.nn.Linear(32, 64)])
            self.norm = torch.nn.LayerNorm(64)
            self.small = torch.nn.Linear(4, 4)   # 16 values: fewer than one block

    m = Tiny().to(DEV)
    before = {k: v.detach().clone() for k, v in m.named_parameters()}
    m, count = quantize_module(m, True, ["label_embeddings"])
    after = dict(m.named_parameters())
    assert count == 64 * 32 + 32 * 64
    for name in ("label_embeddings.weight", "norm.weight", "norm.bias", "blocks.0.bias", "small.weight"):
        assert torch.equal(before[name], after[name]), name
    for name in ("blocks.0.weight", "blocks.1.weight"):
        w0 = before[name].cpu().numpy()
        ref = oracle.quantize_dequantize(w0.reshape(-1), True).reshape(w0.shape)
        assert after[name].detach().cpu().numpy().tobytes() == ref.tobytes(), name
        assert not after[name].requires_grad
    # a needle that only matches ACROSS a dot is not a path component: nothing is skipped by it
    m2 = Tiny().to(DEV)
    _, count2 = quantize_module(m2, False, ["blocks.0"])
    assert count2 == 64 * 32 + 32 * 64 + 10 * 64
    m3 = Tiny().to(DEV)
    _, count3 = quantize_module(m3, False, ["blocks"])
    assert count3 == 10 * 64


def test_qwen_linear_residency_switch_and_its_errors(oracle):
    # src/qwennet.rs:378-435 and the tests at src/qwennet.rs:3041-3047, src/qwentrain.rs:1089-1112
    from unifur_b200.qwennet import QwenLinear, QwenLinearError

    g = torch.Generator(device=DEV).manual_seed(9)
    d_in, d_out = 128, 96
    w = torch.randn(d_in, d_out, device=DEV, generator=g) * 0.02
    bias = torch.randn(d_out, device=DEV, generator=g)
    f32 = QwenLinear.f32(w, bias)
    assert f32.resident_bytes() == 4 * d_in * d_out
    with pytest.raises(QwenLinearError, match="NF4-resident weights only"):
        f32.with_lora(4, 8.0)
    nf4 = f32.to_nf4()
    assert nf4.kind == QwenLinear.NF4 and nf4.inner.bias is bias       # the bias keeps its identity
    assert nf4.to_nf4() is nf4                                          # already resident: unchanged
    assert nf4.inner.packed().is_double_quantized()
    # the in-memory [d_in, d_out] weight is not transposed: same function as the dequantized weight
    x = torch.randn(5, d_in, device=DEV, generator=g)
    y = nf4.forward(x)
    ref = x.double() @ nf4.inner.dequantized_weight().double() + bias.double()
    assert ((y.double() - ref).norm() / ref.norm()).item() < 1e-5
    # packed bytes are what the oracle packs for the flat [d_in, d_out] buffer
    p_ref, a_ref = oracle.quantize_packed(w.cpu().numpy().reshape(-1))
    assert np.array_equal(nf4.inner.packed().codes.cpu().numpy(), p_ref)
    with pytest.raises(QwenLinearError, match="rank"):
        nf4.with_lora(0, 8.0)
    with pytest.raises(QwenLinearError, match="finite"):
        nf4.with_lora(4, float("nan"))
    q = nf4.with_lora(4, 8.0, generator=g)
    assert q.kind == QwenLinear.QLORA
    assert torch.equal(q.forward(x), y)                                 # attaching is an exact no-op
    assert q.resident_bytes() == nf4.resident_bytes() + 4 * (d_in + d_out) * 4
    with pytest.raises(QwenLinearError, match="already carries"):
        q.with_lora(4, 8.0)
    with pytest.raises(QwenLinearError, match="de-adapted"):
        q.to_nf4()


def test_device_status_is_clean_and_a_bounded_wait_reports_a_timeout():
    L = lib()
    d, d2, pf = ctypes.c_int32(-1), ctypes.c_int32(-1), ctypes.c_int32(-1)
    assert L.nf4_device_status(ctypes.byref(d), ctypes.byref(d2), ctypes.byref(pf)) == 0
    assert (d.value, d2.value, pf.value) == (0, 0, 0)
    # a wait that nothing will ever satisfy, with a one-millisecond limit: the kernel comes back,
    # the status says timeout, the flag is cleared and the context is usable afterwards
    waited_ns = ctypes.c_uint64(0)
    st = L.nf4_selftest_bounded_wait(1_000_000, ctypes.byref(waited_ns))
    assert st == -5 and b"wait" in L.nf4_last_error()
    assert 1_000_000 <= waited_ns.value < 500_000_000
    assert L.nf4_device_status(None, None, None) == 0
    t = torch.ones(4, device=DEV)
    assert float(t.sum().item()) == 4.0


def _nccl():
    import os

    import torch as _t

    path = os.path.join(os.path.dirname(_t.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so.2")
    return ctypes.CDLL(path if os.path.exists(path) else "libnccl.so.2", mode=ctypes.RTLD_GLOBAL)


class _NcclId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def test_sharded_forward_through_the_c_abi_with_a_one_rank_communicator(oracle):
    # The exchange below the C ABI with a world of one (what a single GPU can run): local forward,
    # ncclAllGather, placement into y_full.  Two and more ranks run in tests/test_gpu_multi.py.
    L = lib()
    nccl = _nccl()
    uid = _NcclId()
    assert nccl.ncclGetUniqueId(ctypes.byref(uid)) == 0
    comm = ctypes.c_void_p()
    torch.cuda.set_device(0)
    nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _NcclId, ctypes.c_int]
    assert nccl.ncclCommInitRank(ctypes.byref(comm), 1, uid, 0) == 0
    try:
        rng = np.random.default_rng(8)
        rows, k, n, r = 4, 512, 256, 8
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        packed_np, absmax_np = oracle.quantize_packed(w)
        x = dev(rng.standard_normal((rows, k)).astype(np.float32), torch.bfloat16)
        la = dev((rng.standard_normal((r, k)) * 0.05).astype(np.float32), torch.bfloat16)
        lb = dev((rng.standard_normal((n, r)) * 0.05).astype(np.float32), torch.bfloat16)
        packed, absmax = dev(packed_np), dev(absmax_np)
        slab = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
        y_full = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
        gb = int(L.nf4_sharded_gather_bytes(rows, n, 1, _lib.DTYPE_BF16, 0))
        assert gb == rows * n * 2
        gbuf = torch.zeros(gb, dtype=torch.uint8, device=DEV)
        ws = torch.zeros(max(int(L.nf4_linear_workspace_bytes(rows, k, n, r)), 256), dtype=torch.uint8, device=DEV)
        a = _lib.LinearArgs()
        a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
        a.layout, a.io_dtype = _lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16
        a.rows, a.d_in, a.d_out = rows, k, n
        a.x, a.packed, a.absmax = x.data_ptr(), packed.data_ptr(), absmax.data_ptr()
        a.lora_a, a.lora_b, a.lora_rank, a.lora_scale = la.data_ptr(), lb.data_ptr(), r, 2.0
        a.y, a.ldy = slab.data_ptr(), n
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L.nf4_sharded_linear_forward_dev(ctypes.byref(a), comm, 0, 1, _vp(gbuf), gb, _vp(y_full), n, None))
        torch.cuda.synchronize()
        assert torch.equal(y_full, slab)
        ref = oracle.qlora_forward_bnb(x.float().cpu().numpy(), packed_np, absmax_np, n, k,
                                       la.float().cpu().numpy(), lb.float().cpu().numpy(), 2.0)
        got = y_full.float().cpu().numpy().astype(np.float64)
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-3 + 2.0 ** -9
        assert L.nf4_sharded_linear_forward_dev(ctypes.byref(a), None, 0, 1, _vp(gbuf), gb, _vp(y_full), n, None) == -1
    finally:
        nccl.ncclCommDestroy(comm)


@pytest.mark.parametrize("m,k,widths,ranks,dq", [
    (8, 3584, (3584, 512, 512), (16, 16, 16), False),   # q | k | v of the Qwen2-7B-shaped block
    (1, 3584, (18944, 18944), (16, 16), False),         # gate | up
    (16, 4096, (1024, 160, 48, 2048), (64, 0, 8, 16), True),
    (4, 2048, (320, 64), (16, 32), False),              # two groups of warps per CTA
    (8, 18944, (512, 256), (16, 16), False),            # d_in above 4096: falls back to one launch each
    (40, 1024, (256, 384), (8, 8), False),              # more than 16 rows: one launch each (tensor-core GEMM)
])
def test_grouped_forward_equals_one_call_per_projection(m, k, widths, ranks, dq):
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward, linear_forward_grouped

    g = torch.Generator(device=DEV).manual_seed(500 + m + k)
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    projections = []
    for n, r in zip(widths, ranks):
        w = torch.randn(n * k, device=DEV, generator=g) * 0.02
        packed = PackedNf4Tensor.quantize(w)
        pr = {"packed": packed.with_double_quantization() if dq else packed, "d_out": n,
              "bias": torch.randn(n, device=DEV, generator=g) * 0.1 if n % 3 == 0 else None}
        if r:
            pr["lora_a"] = (torch.randn(r, k, device=DEV, generator=g) * 0.01).bfloat16()
            pr["lora_b"] = (torch.randn(n, r, device=DEV, generator=g) * 0.01).bfloat16()
            pr["lora_scale"] = 2.0
        projections.append(pr)
    lib = _lib.load()
    before = _lib.launch_count()
    ys = linear_forward_grouped(x, k, _lib.LAYOUT_OUT_IN, projections)
    launches = _lib.launch_count() - before
    torch.cuda.synchronize()
    fits = m <= 16 and k <= 4096
    assert launches == 1 if fits else launches >= len(widths)
    for pr, y in zip(projections, ys):
        one = linear_forward(x, pr["packed"], k, pr["d_out"], _lib.LAYOUT_OUT_IN, bias=pr.get("bias"),
                             lora_a=pr.get("lora_a"), lora_b=pr.get("lora_b"), lora_scale=pr.get("lora_scale", 0.0))
        torch.cuda.synchronize()
        if m <= 16:
            assert torch.equal(y, one)   # the decode kernels add in a fixed order
        else:
            tol = one.float().abs() * 2.0 ** -7 + 4e-6 * float(one.float().abs().max())
            assert bool(((y.float() - one.float()).abs() <= tol).all())
    d0, d1, d2 = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    assert lib.nf4_device_status(ctypes.byref(d0), ctypes.byref(d1), ctypes.byref(d2)) == 0


def test_reserved_sms_do_not_change_results():
    # nf4_reserve_sms shrinks the decode kernel's grid (fewer CTAs, other row ranges): same bits
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    L = _lib.load()
    g = torch.Generator(device=DEV).manual_seed(77)
    m, k, n, r = 4, 4096, 11008, 16
    w = torch.randn(n * k, device=DEV, generator=g) * 0.02
    packed = PackedNf4Tensor.quantize(w)
    la = (torch.randn(r, k, device=DEV, generator=g) * 0.01).bfloat16()
    lb = (torch.randn(n, r, device=DEV, generator=g) * 0.01).bfloat16()
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    base = linear_forward(x, packed, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=2.0)
    try:
        for count in (4, 20, 74):
            _lib.check(L.nf4_reserve_sms(count))
            y = linear_forward(x, packed, k, n, _lib.LAYOUT_OUT_IN, lora_a=la, lora_b=lb, lora_scale=2.0)
            assert torch.equal(y, base), count
        assert L.nf4_reserve_sms(75) == -1 and L.nf4_reserve_sms(-1) == -1
    finally:
        _lib.check(L.nf4_reserve_sms(0))


@pytest.mark.parametrize("m,k,n", [(4, 4096, 512), (8, 4128, 256), (64, 1024, 256)])
def test_adapter_views_at_odd_offsets_take_the_general_kernel(m, k, n):
    # LoRA factors that are views two bytes into a buffer (an ordinary slice) cannot be read with
    # the tuned kernels' 16-byte loads: the forward must neither fault nor differ
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    g = torch.Generator(device=DEV).manual_seed(91 + k)
    r = 16
    w = torch.randn(n * k, device=DEV, generator=g) * 0.02
    packed = PackedNf4Tensor.quantize(w)
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    la_buf = (torch.randn(r * k + 8, device=DEV, generator=g) * 0.01).bfloat16()
    lb_buf = (torch.randn(n * r + 8, device=DEV, generator=g) * 0.01).bfloat16()
    la_odd, lb_odd = la_buf[1:1 + r * k].view(r, k), lb_buf[1:1 + n * r].view(n, r)
    assert la_odd.data_ptr() % 16 != 0 and lb_odd.data_ptr() % 16 != 0
    y_odd = linear_forward(x, packed, k, n, _lib.LAYOUT_OUT_IN, lora_a=la_odd, lora_b=lb_odd, lora_scale=2.0)
    y_ref = linear_forward(x, packed, k, n, _lib.LAYOUT_OUT_IN, lora_a=la_odd.clone(), lora_b=lb_odd.clone(),
                           lora_scale=2.0)
    torch.cuda.synchronize()
    # the general kernel multiplies exactly dequantized weights in f32, the tuned ones f16 operands:
    # both are within 1e-3 of the exact product, and each output is rounded to bf16 once
    err = (y_odd.float() - y_ref.float()).norm() / y_ref.float().norm()
    assert float(err) <= 2e-3 + 2.0 ** -8
