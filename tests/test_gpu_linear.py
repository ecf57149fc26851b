"""GPU parity of the NF4 / QLoRA linear forward with the CPU oracle, through the C ABI.

Tolerance (stated by the task's north star): relative L2 error <= 1e-3 against the oracle's
f64 accumulation over the bit-exact dequantized f32 weights, for bf16 activations with f32
accumulation.  f32 activations on the general kernel are held to 1e-5."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import DEV, dev, lib, ptr  # noqa: E402
from unifur_b200 import _lib  # noqa: E402

REL_L2_BF16 = 1e-3
REL_L2_F32 = 1e-5


def bf16_round(oracle, a):
    return oracle.round_bf16(np.asarray(a, np.float32))


def rel_l2(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30))


def run_forward(layout, dtype, x, packed, absmax, d_in, d_out, bias=None, lora_a=None, lora_b=None,
                scale=0.0, scale_codes=None, sos=None, y_f32=False, calls=1):
    L = lib()
    tdt = torch.bfloat16 if dtype == _lib.DTYPE_BF16 else torch.float32
    rows = x.shape[0]
    d_x = dev(x, tdt)
    d_p = dev(packed)
    d_am = dev(absmax) if absmax is not None else None
    d_sc = dev(scale_codes) if scale_codes is not None else None
    d_ss = dev(np.asarray([sos], np.float32)) if sos is not None else None
    d_b = dev(bias) if bias is not None else None
    rank = 0
    d_la = d_lb = None
    if lora_a is not None:
        rank = lora_a.shape[0] if layout == _lib.LAYOUT_OUT_IN else lora_a.shape[1]
        d_la, d_lb = dev(lora_a, tdt), dev(lora_b, tdt)
    y = torch.full((rows, d_out), 777.0, dtype=torch.float32 if y_f32 else tdt, device=DEV)
    wsb = int(L.nf4_linear_workspace_bytes(rows, d_in, d_out, rank))
    ws = torch.zeros(max(wsb, 256), dtype=torch.uint8, device=DEV)
    a = _lib.LinearArgs()
    a.struct_bytes = ctypes.sizeof(_lib.LinearArgs)
    a.layout, a.io_dtype, a.y_f32 = layout, dtype, int(y_f32)
    a.rows, a.d_in, a.d_out = rows, d_in, d_out
    a.x, a.packed = d_x.data_ptr(), d_p.data_ptr()
    a.absmax = d_am.data_ptr() if d_am is not None else None
    a.scale_codes = d_sc.data_ptr() if d_sc is not None else None
    a.scale_of_scales = d_ss.data_ptr() if d_ss is not None else None
    a.bias = d_b.data_ptr() if d_b is not None else None
    a.lora_a = d_la.data_ptr() if rank else None
    a.lora_b = d_lb.data_ptr() if rank else None
    a.lora_rank, a.lora_scale = rank, scale
    a.y, a.ldy = y.data_ptr(), d_out
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    for i in range(calls):  # the same arguments and workspace again: what a call leaves must serve the next
        if i:
            y.fill_(777.0)
        _lib.check(L.nf4_linear_forward_dev(ctypes.byref(a), None))
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


def make_case(oracle, seed, M, K, N, r, dq=False, bias=False, w_std=0.02, ab_std=0.01):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * w_std).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    x = bf16_round(oracle, rng.standard_normal((M, K)))
    la = lb = None
    if r:
        la = bf16_round(oracle, rng.standard_normal((r, K)) * ab_std)
        lb = bf16_round(oracle, rng.standard_normal((N, r)) * ab_std)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32) if bias else None
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    return dict(x=x, packed=packed, absmax=None if dq else absmax, sc=sc, sos=sos, la=la, lb=lb, bias=b)


def check_out_in(oracle, c, M, K, N, scale, tol=REL_L2_BF16):
    """bf16 activations, W [N, K].  The kernel's own error is measured on its f32 output (bar:
    rel. L2 <= 1e-3); the bf16 output must then be that result rounded once to bf16, up to one
    bf16 ulp where the f32 sums differ in their last bits (the decode kernel's split-K shapes
    add partial sums in another order than one pass over K would)."""
    ref = oracle.qlora_forward_bnb(c["x"], c["packed"], c["absmax"], N, K, c["la"], c["lb"], scale,
                                   c["bias"], c["sc"], c["sos"] if c["sos"] is not None else 0.0)
    kw = dict(bias=c["bias"], lora_a=c["la"], lora_b=c["lb"], scale=scale, scale_codes=c["sc"],
              sos=c["sos"])
    y32 = run_forward(_lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16, c["x"], c["packed"], c["absmax"], K, N,
                      y_f32=True, **kw)
    err = rel_l2(y32, ref)
    assert err <= tol, err
    y16 = run_forward(_lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16, c["x"], c["packed"], c["absmax"], K, N,
                      **kw)
    once = torch.from_numpy(y32).bfloat16().float().numpy()
    # one bf16 ulp, plus the f32 reassociation noise of a sum whose terms are ~max|y| (matters
    # only for outputs that cancel to almost zero)
    ulp = np.abs(once) * 2.0 ** -7 + 4e-6 * np.abs(once).max()
    assert np.all(np.abs(y16 - once) <= ulp)
    assert np.mean(y16 != once) < 0.02
    return y16, ref


@pytest.mark.parametrize("M", [1, 4, 16])
def test_decode_config_shapes(oracle, M):
    # config 2 at full size: K = 4096, N = 11008, rank 16, scale 2.0
    K, N, r = 4096, 11008, 16
    c = make_case(oracle, 2, M, K, N, r)
    check_out_in(oracle, c, M, K, N, 2.0)


@pytest.mark.parametrize("M,K,N,r,dq,bias", [
    (1, 64, 16, 0, False, False),
    (2, 128, 48, 4, False, True),
    (3, 512, 200, 8, True, False),
    (8, 3584, 512, 16, False, False),     # Qwen2-7B k/v projection
    (8, 3584, 448, 16, True, True),       # one 8-GPU shard of q/o
    (5, 1024, 1000, 16, False, True),     # ragged N
    (16, 4096, 160, 64, True, True),
    (9, 2048, 64, 1, False, False),
    (7, 192, 24, 3, False, False),        # odd rank and tiny N: general kernel
])
def test_decode_edge_shapes(oracle, M, K, N, r, dq, bias):
    c = make_case(oracle, 1000 + M + K + N, M, K, N, r, dq=dq, bias=bias)
    check_out_in(oracle, c, M, K, N, 1.5)


def test_lora_only_and_base_only_terms(oracle):
    M, K, N, r = 4, 1024, 256, 16
    c = make_case(oracle, 77, M, K, N, r, ab_std=0.3)
    # zero base weight: y is the LoRA term alone and must still meet the bar
    z = dict(c)
    z["packed"] = np.full_like(c["packed"], 0x77)
    z["absmax"] = np.zeros_like(c["absmax"])
    check_out_in(oracle, z, M, K, N, 2.0)
    # zero B: attaching the adapter is an exact no-op (qwentrain.rs:1089-1112)
    nb = dict(c)
    nb["lb"] = np.zeros_like(c["lb"])
    with_adapter, _ = check_out_in(oracle, nb, M, K, N, 2.0)
    nb["la"] = nb["lb"] = None
    without, _ = check_out_in(oracle, nb, M, K, N, 0.0)
    assert np.array_equal(with_adapter, without)


def test_general_kernel_in_out_layout_f32(oracle):
    # the reference's own orientation and types: W [d_in, d_out] flat blocks, f32 everywhere
    # (qwennet.rs:2518-2562), including d_out = 48 whose blocks straddle rows
    rng = np.random.default_rng(5)
    for rows, d_in, d_out, r, dq in ((3, 8, 6, 0, True), (4, 96, 48, 4, True), (5, 64, 8, 2, False),
                                     (17, 130, 70, 3, False)):
        w = rng.standard_normal((d_in, d_out)).astype(np.float32)
        packed, absmax = oracle.quantize_packed(w)
        sc = sos = None
        if dq:
            sc, sos = oracle.double_quantize(absmax)
        x = rng.uniform(-1, 1, (rows, d_in)).astype(np.float32)
        la = lb = None
        if r:
            la = rng.standard_normal((d_in, r)).astype(np.float32)
            lb = rng.uniform(-0.5, 0.5, (r, d_out)).astype(np.float32)
        bias = rng.standard_normal(d_out).astype(np.float32)
        ref = oracle.qlora_forward_burn(x, packed, None if dq else absmax, d_in, d_out, la, lb, 2.0,
                                        bias, sc, sos if dq else 0.0)
        got = run_forward(_lib.LAYOUT_IN_OUT, _lib.DTYPE_F32, x, packed, None if dq else absmax,
                          d_in, d_out, bias=bias, lora_a=la, lora_b=lb, scale=2.0,
                          scale_codes=sc, sos=sos)
        assert rel_l2(got, ref) <= REL_L2_F32


@pytest.mark.parametrize("rows,d_in,d_out,r,dq,f32", [
    (1, 4096, 11008, 16, False, True),     # the decode configuration in the reference's orientation and types
    (4, 4096, 11008, 16, True, False),     # bf16 activations, double-quantized scales
    (16, 1024, 4096, 8, False, True),      # two launches of eight activation rows
    (40, 512, 320, 3, True, True),         # five launches (rank 3: not for the tensor-core path); strip narrower than 256 columns at the end
    (3, 100, 64, 0, False, True),          # one strip, K shorter than two pieces
    (8, 18944, 3584, 16, False, False),    # the block's down projection
])
def test_reference_orientation_at_decode_sizes(oracle, rows, d_in, d_out, r, dq, f32):
    # W [d_in, d_out] with d_out a multiple of 64 and few activation rows: the strip kernel (f32
    # dequantisation as the reference does it, f32 sums; pieces of K added in a fixed order)
    rng = np.random.default_rng(700 + rows + d_in + d_out)
    w = (rng.standard_normal((d_in, d_out)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    x = rng.uniform(-1, 1, (rows, d_in)).astype(np.float32)
    la = lb = None
    if r:
        la = (rng.standard_normal((d_in, r)) * 0.05).astype(np.float32)
        lb = rng.uniform(-0.5, 0.5, (r, d_out)).astype(np.float32)
    bias = rng.standard_normal(d_out).astype(np.float32)
    if not f32:
        x, bias = bf16_round(oracle, x), bias
        if r:
            la, lb = bf16_round(oracle, la), bf16_round(oracle, lb)
    ref = oracle.qlora_forward_burn(x, packed, None if dq else absmax, d_in, d_out, la, lb, 2.0, bias, sc,
                                    sos if dq else 0.0)
    dt = _lib.DTYPE_F32 if f32 else _lib.DTYPE_BF16
    kw = dict(bias=bias, lora_a=la, lora_b=lb, scale=2.0, scale_codes=sc, sos=sos)
    got = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, y_f32=True, calls=2, **kw)
    assert rel_l2(got, ref) <= REL_L2_F32   # f32 products and sums of exactly dequantized weights
    again = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, y_f32=True, **kw)
    assert np.array_equal(got, again)       # bit-reproducible
    if not f32:
        y16 = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, **kw)
        assert np.array_equal(y16, torch.from_numpy(got).bfloat16().float().numpy())


@pytest.mark.parametrize("rows,d_in,d_out,r,dq,f32,bias", [
    (17, 128, 64, 0, False, True, False),     # the smallest shape: one tile, half of its weight rows empty
    (200, 512, 320, 4, True, True, True),     # d_out = 2.5 tiles; f32 factors enter as rank 8
    (300, 1024, 768, 8, False, False, True),  # bf16 activations and factors
    (257, 4096, 1024, 64, False, True, False),  # rank 64 in f32: two 64-rank chunks per half of T
    (1000, 2048, 2048, 16, True, False, False),
])
def test_reference_orientation_at_prefill_sizes(oracle, rows, d_in, d_out, r, dq, f32, bias):
    # W [d_in, d_out] at more than 16 activation rows: nibbles and scales are repacked into the
    # workspace and the tensor-core GEMM multiplies (f16 operands, f32 sums): rel. L2 <= 1e-3
    rng = np.random.default_rng(800 + rows + d_in + d_out)
    w = (rng.standard_normal((d_in, d_out)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    x = rng.standard_normal((rows, d_in)).astype(np.float32)
    x[3] *= 2.0 ** 18      # rows outside f16's range on both sides
    x[5] *= 2.0 ** -22
    la = lb = None
    if r:
        la = (rng.standard_normal((d_in, r)) * 0.05).astype(np.float32)
        lb = rng.uniform(-0.5, 0.5, (r, d_out)).astype(np.float32)   # an adapter term as large as the base term
    b = rng.standard_normal(d_out).astype(np.float32) if bias else None
    if not f32:
        x = bf16_round(oracle, x)
        if r:
            la, lb = bf16_round(oracle, la), bf16_round(oracle, lb)
    ref = oracle.qlora_forward_burn(x, packed, None if dq else absmax, d_in, d_out, la, lb, 2.0, b, sc,
                                    sos if dq else 0.0)
    dt = _lib.DTYPE_F32 if f32 else _lib.DTYPE_BF16
    kw = dict(bias=b, lora_a=la, lora_b=lb, scale=2.0, scale_codes=sc, sos=sos)
    got = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, y_f32=True, calls=2, **kw)
    assert rel_l2(got, ref) <= 1e-3
    for rows_ in (slice(0, 3), slice(3, 4), slice(5, 6), slice(rows - 1, rows)):   # every row on its own scale
        assert rel_l2(got[rows_], ref[rows_]) <= 1e-3, rows_
    again = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, y_f32=True, **kw)
    assert np.array_equal(got, again)   # every sum in a fixed order: the same bits from run to run
    if not f32:
        y16 = run_forward(_lib.LAYOUT_IN_OUT, dt, x, packed, None if dq else absmax, d_in, d_out, **kw)
        assert rel_l2(y16, ref) <= REL_L2_BF16 + 2.0 ** -9


@pytest.mark.parametrize("rows,d_in,d_out,r,dq,bias", [
    (33, 256, 200, 4, False, True),      # d_out no multiple of the tile: the last tile's rows beyond N
    (500, 1024, 1536, 16, True, False),
    (257, 4096, 640, 64, False, False),  # f32 factors of rank 64 enter as rank 128: two chunks per half of T
])
def test_f32_tensors_at_prefill_sizes(oracle, rows, d_in, d_out, r, dq, bias):
    # W [d_out, d_in] with f32 activations and factors (the reference's tensor type) at more than 16
    # rows: activations to f16 per row, factors converted into the workspace, the tensor-core GEMM
    rng = np.random.default_rng(860 + rows + d_in + d_out)
    w = (rng.standard_normal((d_out, d_in)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    x = rng.standard_normal((rows, d_in)).astype(np.float32)
    x[1] *= 2.0 ** 19
    x[2] *= 2.0 ** -21
    la = (rng.standard_normal((r, d_in)) * 0.05).astype(np.float32)
    lb = rng.uniform(-0.5, 0.5, (d_out, r)).astype(np.float32)
    b = rng.standard_normal(d_out).astype(np.float32) if bias else None
    ref = oracle.qlora_forward_bnb(x, packed, None if dq else absmax, d_out, d_in, la, lb, 2.0, b, sc,
                                   sos if dq else 0.0)
    kw = dict(bias=b, lora_a=la, lora_b=lb, scale=2.0, scale_codes=sc, sos=sos)
    got = run_forward(_lib.LAYOUT_OUT_IN, _lib.DTYPE_F32, x, packed, None if dq else absmax, d_in, d_out, calls=2, **kw)
    assert rel_l2(got, ref) <= 1e-3
    for rows_ in (slice(0, 1), slice(1, 2), slice(2, 3), slice(rows - 1, rows)):
        assert rel_l2(got[rows_], ref[rows_]) <= 1e-3, rows_


@pytest.mark.parametrize("rows,d_in,d_out,r,dq,bias", [
    (1, 4096, 11008, 16, False, False),    # the decode configuration with f32 tensors
    (5, 4096, 11008, 16, True, True),
    (16, 1024, 768, 12, False, True),      # two passes of eight rows; a rank the decode kernel itself would refuse
    (3, 18944, 512, 8, False, False),      # K in parts
    (2, 320, 192, 4, False, True),         # d_in no multiple of 256: the split-K tensor-core kernel
])
def test_f32_tensors_at_decode_sizes(oracle, rows, d_in, d_out, r, dq, bias):
    # W [d_out, d_in] with f32 activations and factors at up to 16 rows: every row goes through the
    # decode kernel as two bf16 rows (high and low part), the adapter term is added in f32
    rng = np.random.default_rng(870 + rows + d_in + d_out)
    w = (rng.standard_normal((d_out, d_in)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    sc = sos = None
    if dq:
        sc, sos = oracle.double_quantize(absmax)
    x = rng.standard_normal((rows, d_in)).astype(np.float32)
    x[0] *= 2.0 ** 19
    if rows > 1:
        x[1] *= 2.0 ** -21
    la = (rng.standard_normal((r, d_in)) * 0.05).astype(np.float32)
    lb = rng.uniform(-0.5, 0.5, (d_out, r)).astype(np.float32)
    b = rng.standard_normal(d_out).astype(np.float32) if bias else None
    ref = oracle.qlora_forward_bnb(x, packed, None if dq else absmax, d_out, d_in, la, lb, 2.0, b, sc,
                                   sos if dq else 0.0)
    kw = dict(bias=b, lora_a=la, lora_b=lb, scale=2.0, scale_codes=sc, sos=sos)
    got = run_forward(_lib.LAYOUT_OUT_IN, _lib.DTYPE_F32, x, packed, None if dq else absmax, d_in, d_out, calls=2, **kw)
    assert rel_l2(got, ref) <= 1e-3
    for i in range(rows):
        assert rel_l2(got[i:i + 1], ref[i:i + 1]) <= 1e-3, i


def test_layout_kat_minus_three(oracle):
    # qwennet.rs:2196-2211: y[o] = sum_i x[i] W[i][o] with W = [[1,2,3],[4,5,6]] (values on a
    # grid NF4 cannot hold exactly, so compare against the oracle's own dequantized weight)
    w = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    packed, absmax = oracle.quantize_packed(w)
    x = np.array([[1.0, -1.0]], np.float32)
    ref = oracle.qlora_forward_burn(x, packed, absmax, 2, 3)
    got = run_forward(_lib.LAYOUT_IN_OUT, _lib.DTYPE_F32, x, packed, absmax, 2, 3)
    assert np.allclose(got, ref, atol=1e-6)
    deq = oracle.dequantize_packed(packed, 6, absmax).reshape(2, 3)
    assert np.allclose(got[0], deq[0] - deq[1], atol=1e-6)


def test_host_weight_handle_forward(oracle):
    # the path Nf4Linear::from_values + forward takes from host memory (qwennet.rs:198-241)
    L = lib()
    rng = np.random.default_rng(8)
    M, K, N, r = 4, 1024, 512, 16
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    h = ctypes.c_void_p()
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    _lib.check(L.nf4_weight_from_values_host(vp(w), K, N, _lib.LAYOUT_OUT_IN, 1, ctypes.byref(h)))
    try:
        packed, absmax = oracle.quantize_packed(w)
        sc, sos = oracle.double_quantize(absmax)
        assert L.nf4_weight_resident_bytes(h) == oracle.estimated_resident_bytes(N * K, True)
        got_p = np.zeros_like(packed)
        got_sc = np.zeros_like(sc)
        got_sos = np.zeros(1, np.float32)
        _lib.check(L.nf4_weight_download_host(h, vp(got_p), None, vp(got_sc), vp(got_sos)))
        assert np.array_equal(got_p, packed) and np.array_equal(got_sc, sc) and got_sos[0] == sos
        deq = np.zeros(N * K, np.float32)
        _lib.check(L.nf4_weight_dequantize_host(h, vp(deq)))
        assert deq.tobytes() == oracle.dequantize_packed(packed, N * K, None, sc, sos).tobytes()
        x = bf16_round(oracle, rng.standard_normal((M, K)))
        la = bf16_round(oracle, rng.standard_normal((r, K)) * 0.01)
        lb = bf16_round(oracle, rng.standard_normal((N, r)) * 0.01)
        to_bf16 = lambda a: torch.from_numpy(a).bfloat16().view(torch.int16).numpy()
        xb, lab, lbb = to_bf16(x), to_bf16(la), to_bf16(lb)
        yb = np.zeros((M, N), np.int16)
        _lib.check(L.nf4_weight_linear_forward_host(h, vp(xb), M, _lib.DTYPE_BF16, None, vp(lab),
                                                    vp(lbb), r, 2.0, vp(yb)))
        got = torch.from_numpy(yb).view(torch.bfloat16).float().numpy()
        ref = oracle.qlora_forward_bnb(x, packed, None, N, K, la, lb, 2.0, None, sc, sos)
        # the result has been rounded to bf16 once (2^-9 relative at most per element)
        assert rel_l2(got, ref) <= REL_L2_BF16 + 2.0 ** -9
        # a page-locked output is written by the kernel itself (no copy back): the same bits
        y_locked = torch.full((M, N), 7.0, dtype=torch.bfloat16).pin_memory()
        x_locked = torch.from_numpy(x).bfloat16().pin_memory()
        for _ in range(2):
            _lib.check(L.nf4_weight_linear_forward_host(h, ctypes.c_void_p(x_locked.data_ptr()), M, _lib.DTYPE_BF16, None,
                                                        vp(lab), vp(lbb), r, 2.0, ctypes.c_void_p(y_locked.data_ptr())))
            assert np.array_equal(y_locked.view(torch.int16).numpy(), yb)
            y_locked.fill_(7.0)
    finally:
        L.nf4_weight_free(h)


def test_python_mirror_reads_like_the_reference(oracle):
    # test_qlora_linear_is_the_base_layer_at_init / test_lora_starts_as_an_exact_identity
    # (quantize.rs:1011-1081) through the host-side mirror
    from unifur_b200.quantize import LoraAdapter, LoraConfig, PackedNf4Tensor, QLoraLinear

    g = torch.Generator(device=DEV).manual_seed(3)
    cfg = LoraConfig.new(16, 8, 4)
    adapter = LoraAdapter.new(cfg, DEV, generator=g)
    x = torch.rand(3, 16, device=DEV, generator=g) * 2 - 1
    assert adapter.forward(x).abs().max().item() == 0.0
    assert adapter.delta_weight().abs().max().item() == 0.0
    assert adapter.rank() == 4 and abs(adapter.scaling() - 1.0) < 1e-12
    assert abs(LoraConfig.new(12, 6, 3).with_alpha(6.0).scaling() - 2.0) < 1e-12
    w = torch.randn(64, 8, device=DEV, generator=g)
    bias = torch.randn(8, device=DEV, generator=g)
    q = QLoraLinear.from_linear(w, bias, LoraConfig.new(64, 8, 2), True, generator=g)
    x = torch.rand(2, 64, device=DEV, generator=g) * 2 - 1
    assert (q.forward(x) - q.base_forward(x)).abs().max().item() == 0.0
    nf4_bits, f32_bits = q.resident_bits()
    assert nf4_bits * 7.0 < f32_bits
    p1 = PackedNf4Tensor.quantize(w)
    p2 = PackedNf4Tensor.quantize(w)
    assert p1 == p2 and p1.with_double_quantization() == p2.with_double_quantization()
    assert p1.resident_bytes() == 64 * 8 // 2 + 8 * 4


QWEN2_7B_BLOCK = [  # name, d_in, d_out  (configuration 5: all seven projections NF4, rank 16)
    ("q", 3584, 3584), ("k", 3584, 512), ("v", 3584, 512), ("o", 3584, 3584),
    ("gate", 3584, 18944), ("up", 3584, 18944), ("down", 18944, 3584),
]


@pytest.mark.parametrize("M,K,N,r,dq,bias", [
    (1, 8192, 384, 16, False, False),     # two parts of sixteen slices
    (8, 4352, 96, 8, True, True),         # seventeen slices: parts of nine and eight
    (16, 18944, 512, 64, False, True),    # five parts, the last one slice shorter
    (3, 12288, 1000, 0, False, True),     # no adapter, ragged N, three parts
    (5, 32768, 48, 32, True, False),      # the longest K the kernel takes: eight parts
])
def test_decode_long_k_shared_out_between_ctas(oracle, M, K, N, r, dq, bias):
    # d_in above 4096: groups of CTAs multiply parts of K and the last to arrive for a range of
    # rows adds the parts' sums in a fixed order
    c = make_case(oracle, 3000 + M + K + N, M, K, N, r, dq=dq, bias=bias)
    y1, _ = check_out_in(oracle, c, M, K, N, 1.5)
    # three calls on one workspace: the flag words and counters re-arm, the result is the same
    y3 = run_forward(_lib.LAYOUT_OUT_IN, _lib.DTYPE_BF16, c["x"], c["packed"], c["absmax"], K, N, bias=c["bias"],
                     lora_a=c["la"], lora_b=c["lb"], scale=1.5, scale_codes=c["sc"], sos=c["sos"], calls=3)
    assert np.array_equal(y1, y3)


@pytest.mark.parametrize("dq", [False, True])
def test_qwen2_7b_block_decode_batch_8(oracle, dq):
    # The seven projections at full size, decode batch 8, chained the way a decoder block feeds
    # them.  The reference has no Qwen2 block, so the glue between the projections is a cheap
    # stand-in (attention replaced by v broadcast over the query groups, SiLU(gate) * up for the
    # MLP); every projection is checked on its own input against the oracle.
    M, r, scale = 8, 16, 2.0
    rng = np.random.default_rng(200)
    x = bf16_round(oracle, rng.standard_normal((M, 3584)))
    outs = {}
    for i, (name, K, N) in enumerate(QWEN2_7B_BLOCK):
        if name in ("q", "k", "v", "gate", "up"):
            inp = x
        elif name == "o":
            inp = bf16_round(oracle, np.tile(outs["v"], (1, 7)))
        else:
            g = outs["gate"].astype(np.float64)
            inp = bf16_round(oracle, g / (1.0 + np.exp(-g)) * outs["up"])
        c = make_case(oracle, 200 + i, M, K, N, r, dq=dq)
        c["x"] = inp
        outs[name], _ = check_out_in(oracle, c, M, K, N, scale)
        if name == "o":
            x = bf16_round(oracle, x + outs["o"])  # residual; feeds gate/up


# ------------------------------------------------------------------ prefill (tcgen05) path
@pytest.mark.parametrize("M,K,N,r,dq,bias", [
    (256, 256, 128, 0, False, False),     # one tile, four k-stages
    (17, 64, 8, 0, False, False),         # smallest shape the tensor-core path takes
    (300, 512, 200, 16, False, True),     # ragged in both M and N, adapter narrower than a chunk
    (512, 1024, 384, 64, True, True),     # double-quantized scales, full-chunk adapter
    (257, 192, 136, 80, False, False),    # adapter wider than one 64-chunk
    (128, 3584, 512, 16, True, False),    # Qwen2-7B k/v projection
    (40, 128, 72, 12, False, True),       # rank not a multiple of 8: LoRA B is not TMA-readable, general kernel
    (520, 256, 304, 8, False, False),     # three activation tiles x three weight tiles, narrow adapter
    (512, 4096, 256, 16, False, True),    # four tiles over ten CTAs: a tile's k-stages split three ways
    (300, 3072, 200, 64, True, True),     # four ragged tiles over eight CTAs, adapter stages on the finishing CTA only
    (768, 1536, 6400, 16, False, False),  # 150 tiles on 148 CTAs: every CTA takes a little more than one tile
])
def test_prefill_shapes(oracle, M, K, N, r, dq, bias):
    c = make_case(oracle, 5000 + M + K + N, M, K, N, r, dq=dq, bias=bias)
    check_out_in(oracle, c, M, K, N, 2.0)


def test_prefill_config3_slice(oracle):
    # config 3 (M = 2048, K = 4096, rank 64) on a 1024-column slice of its N = 14336: several
    # persistent tiles per CTA, the full K loop and the fused adapter
    M, K, N, r = 2048, 4096, 1024, 64
    c = make_case(oracle, 5, M, K, N, r)
    check_out_in(oracle, c, M, K, N, 2.0)


def test_prefill_linearity_at_full_config3_size(oracle):
    # size-independent property at the full config-3 size (N = 14336): the forward is linear
    # in x, so y(x1 + x2) = y(x1) + y(x2) up to rounding, and y(0) = bias-free zero
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    M, K, N, r = 2048, 4096, 14336, 64
    g = torch.Generator(device=DEV).manual_seed(5)
    w = torch.randn(N * K, device=DEV, generator=g) * 0.02
    packed = PackedNf4Tensor.quantize(w)
    del w
    a = (torch.randn(r, K, device=DEV, generator=g) * 0.01).bfloat16()
    b = (torch.randn(N, r, device=DEV, generator=g) * 0.01).bfloat16()
    x1 = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    x2 = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    xs = (x1.float() + x2.float()).bfloat16()
    y = lambda x: linear_forward(x, packed, K, N, _lib.LAYOUT_OUT_IN, lora_a=a, lora_b=b,
                                 lora_scale=2.0).float()
    y1, y2, ys = y(x1), y(x2), y(xs)
    # x1 + x2 was itself rounded to bf16, so compare against the forward of the exact residual
    resid = (xs.float() - x1.float() - x2.float()).bfloat16()
    yr = y(resid)
    err = (ys - y1 - y2 - yr).norm() / ys.norm()
    assert err.item() < 6e-3  # four bf16 output roundings
    assert y(torch.zeros_like(x1)).abs().max().item() == 0.0
    # a slice of rows against the oracle (f64) to pin absolute values at this size
    rows = slice(1000, 1016)
    deq = packed.dequantize().view(N, K)[:256].double()
    ref = x1[rows].double() @ deq.t() + 2.0 * (x1[rows].double() @ a.double().t()) @ b[:256].double().t()
    got = y1[rows, :256].double()
    assert ((got - ref).norm() / ref.norm()).item() < 1e-3 + 2.0 ** -9
    # the last 128 weight rows belong to the tiles of the last, partly filled round
    for rows in (slice(1000, 1016), slice(1080, 1096), slice(2040, 2048)):
        deq = packed.dequantize().view(N, K)[N - 128:].double()
        ref = x1[rows].double() @ deq.t() + 2.0 * (x1[rows].double() @ a.double().t()) @ b[N - 128:].double().t()
        got = y1[rows, N - 128:].double()
        assert ((got - ref).norm() / ref.norm()).item() < 1e-3 + 2.0 ** -9


@pytest.mark.parametrize("layout_name,M,K,N,r", [("out_in", 300, 448, 576, 24), ("in_out", 130, 320, 200, 72),
                                                 ("out_in", 9, 200, 100, 5)])   # the last: shapes the MMA product declines
def test_qlora_backward_bf16(oracle, layout_name, M, K, N, r):
    # bf16 tensors: the adapter intermediates come from warp MMAs (exact products, f32 sums), grad_x at
    # more than 16 rows from the tensor-core GEMM; outputs are bf16 (one rounding: 2^-9)
    from unifur_b200.quantize import PackedNf4Tensor
    from unifur_b200.qwennet import Nf4Linear, QloraLinear

    rng = np.random.default_rng(950 + M + K + N)
    out_in = layout_name == "out_in"
    w = (rng.standard_normal((N, K) if out_in else (K, N)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    wd = oracle.dequantize_packed(packed, w.size, absmax).reshape(w.shape).astype(np.float64)
    a = bf16_round(oracle, rng.standard_normal((r, K) if out_in else (K, r)) * 0.1)
    b = bf16_round(oracle, rng.standard_normal((N, r) if out_in else (r, N)) * 0.1)
    x = bf16_round(oracle, rng.standard_normal((M, K)))
    gy = bf16_round(oracle, rng.standard_normal((M, N)))
    s = 1.5
    X, GY, A, B = (t.astype(np.float64) for t in (x, gy, a, b))
    if out_in:
        gx_ref = GY @ wd + s * (GY @ B) @ A
        ga_ref = s * (GY @ B).T @ X
        gb_ref = s * GY.T @ (X @ A.T)
    else:
        gx_ref = GY @ wd.T + s * (GY @ B.T) @ A.T
        ga_ref = s * X.T @ (GY @ B.T)
        gb_ref = s * (X @ A).T @ GY
    lay = _lib.LAYOUT_OUT_IN if out_in else _lib.LAYOUT_IN_OUT
    bf = lambda t: torch.from_numpy(t).to(DEV).bfloat16()
    base = Nf4Linear(PackedNf4Tensor.quantize(torch.from_numpy(w.reshape(-1)).to(DEV)), K, N, None, lay)
    q = QloraLinear(base, bf(a), bf(b), s)
    gx, ga, gb = q.backward(bf(x), bf(gy))
    assert gx.dtype == torch.bfloat16
    tol = 1e-3 + 2.0 ** -8
    assert rel_l2(gx.float().cpu().numpy(), gx_ref) <= tol
    assert rel_l2(ga.float().cpu().numpy(), ga_ref) <= tol
    assert rel_l2(gb.float().cpu().numpy(), gb_ref) <= tol


@pytest.mark.parametrize("layout_name,M,K,N,r", [("out_in", 8, 256, 192, 16), ("out_in", 40, 512, 320, 8),
                                                 ("in_out", 6, 128, 96, 4),
                                                 ("out_in", 300, 448, 576, 24),   # several pieces of rows, ragged tiles of columns
                                                 ("in_out", 130, 320, 200, 72)])  # more than 64 ranks: two passes over them
def test_qlora_backward_matches_f64_reference(oracle, layout_name, M, K, N, r):
    # Gradients with the NF4 base frozen (what the reference's autodiff sees through the detached
    # weight, src/qwennet.rs:226-241): grad_x runs through the NF4 kernels on the same packed
    # bytes in the other orientation, grad_a / grad_b are dense.  f32 activations: 1e-5 (grad_x at
    # more than 16 rows: 1e-3).
    from unifur_b200.quantize import PackedNf4Tensor
    from unifur_b200.qwennet import Nf4Linear, QloraLinear

    rng = np.random.default_rng(900 + M + K + N)
    out_in = layout_name == "out_in"
    w = (rng.standard_normal((N, K) if out_in else (K, N)) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    wd = oracle.dequantize_packed(packed, w.size, absmax).reshape(w.shape).astype(np.float64)
    a = (rng.standard_normal((r, K) if out_in else (K, r)) * 0.1).astype(np.float32)
    b = (rng.standard_normal((N, r) if out_in else (r, N)) * 0.1).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    gy = rng.standard_normal((M, N)).astype(np.float32)
    s = 1.5
    X, GY, A, B = (t.astype(np.float64) for t in (x, gy, a, b))
    if out_in:
        gx_ref = GY @ wd + s * (GY @ B) @ A
        ga_ref = s * (GY @ B).T @ X
        gb_ref = s * GY.T @ (X @ A.T)
    else:
        gx_ref = GY @ wd.T + s * (GY @ B.T) @ A.T
        ga_ref = s * X.T @ (GY @ B.T)
        gb_ref = s * (X @ A).T @ GY
    lay = _lib.LAYOUT_OUT_IN if out_in else _lib.LAYOUT_IN_OUT
    base = Nf4Linear(PackedNf4Tensor.quantize(torch.from_numpy(w.reshape(-1)).to(DEV)), K, N, None, lay)
    q = QloraLinear(base, torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV), s)
    gx, ga, gb = q.backward(torch.from_numpy(x).to(DEV), torch.from_numpy(gy).to(DEV))
    # more than 16 rows: grad_x of the out_in layout is a forward in the other orientation on the tensor cores
    assert rel_l2(gx.cpu().numpy(), gx_ref) <= (1e-3 if (out_in and M > 16) else REL_L2_F32)
    assert rel_l2(ga.cpu().numpy(), ga_ref) <= REL_L2_F32
    assert rel_l2(gb.cpu().numpy(), gb_ref) <= REL_L2_F32
    if M > 16:
        return   # the forward of more than 16 rows rounds the activations to f16: too coarse for a difference quotient
    # and the forward it differentiates: finite differences along one direction
    dx = rng.standard_normal((M, K)).astype(np.float32) * 1e-2
    y0 = q.forward(torch.from_numpy(x).to(DEV)).double().cpu().numpy()
    y1 = q.forward(torch.from_numpy(x + dx).to(DEV)).double().cpu().numpy()
    lhs = float(np.sum((y1 - y0) * gy))
    rhs = float(np.sum(gx.double().cpu().numpy() * dx))
    # (the forward of f32 rows on the decode kernels carries sixteen bits of the activations)
    assert abs(lhs - rhs) <= 5e-3 * max(abs(lhs), abs(rhs), 1e-6)
