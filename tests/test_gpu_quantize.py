"""GPU parity of quantize / double-quantize / dequantize with the CPU oracle: bit-exact codes,
packed bytes, absmax and dequantized f32, through the C ABI.  Edge cases follow the reference's
own tests (src/quantize.rs:755-1009, src/verify.rs:1042-1120)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import (DEV, bits_equal, dequantize_dev, dev, double_quantize_dev, lib, ptr,  # noqa: E402
                      quantize_dev, student_t)
from unifur_b200 import _lib  # noqa: E402


def check_roundtrip(oracle, values, label=""):
    values = np.asarray(values, np.float32).ravel()
    n = values.size
    o_packed, o_absmax = oracle.quantize_packed(values)
    o_codes, _ = oracle.quantize_simulated(values)
    g_packed, g_absmax = quantize_dev(values, packed=True)
    g_codes, g_absmax2 = quantize_dev(values, packed=False)
    assert bits_equal(g_absmax, o_absmax), f"absmax {label}"
    assert bits_equal(g_absmax2, o_absmax), f"absmax (unpacked) {label}"
    assert bits_equal(g_packed, o_packed), f"packed bytes {label}"
    assert bits_equal(g_codes, o_codes), f"codes {label}"
    # plain dequantize
    o_deq = oracle.dequantize_packed(o_packed, n, o_absmax)
    assert bits_equal(dequantize_dev(g_packed, n, absmax=g_absmax), o_deq), f"dequant {label}"
    assert bits_equal(dequantize_dev(g_codes, n, absmax=g_absmax, packed=False), o_deq)
    # double quantization
    o_sc, o_sos = oracle.double_quantize(o_absmax)
    g_sc, g_sos = double_quantize_dev(g_absmax)
    assert bits_equal(g_sc, o_sc) and bits_equal(np.float32(g_sos), np.float32(o_sos)), f"dq {label}"
    o_deq2 = oracle.dequantize_packed(o_packed, n, None, o_sc, o_sos)
    assert bits_equal(dequantize_dev(g_packed, n, scale_codes=g_sc, sos=g_sos), o_deq2)
    assert bits_equal(dequantize_dev(g_codes, n, scale_codes=g_sc, sos=g_sos, packed=False), o_deq2)


def test_reference_known_answers_on_gpu(oracle):
    lv = oracle.levels()
    # quantize.rs:868-879
    packed, absmax = quantize_dev(lv * np.float32(0.75))
    assert list(packed) == [(2 * i) | ((2 * i + 1) << 4) for i in range(8)]
    # quantize.rs:881-894
    v = np.full(64, 0.01, np.float32)
    v[7], v[9] = -4.25, 2.0
    packed, absmax = quantize_dev(v)
    assert absmax[0] == np.float32(4.25)
    assert dequantize_dev(packed, 64, absmax=absmax)[7] == np.float32(-4.25)
    # quantize.rs:957-964 and verify.rs:1070-1078
    packed, absmax = quantize_dev(np.zeros(128, np.float32))
    assert np.all(packed == 0x77) and np.all(absmax == 0)
    assert np.all(dequantize_dev(packed, 128, absmax=absmax) == 0.0)
    # quantize.rs:966-973
    packed, absmax = quantize_dev(np.arange(69, dtype=np.float32) * np.float32(0.01))
    assert packed.size == 35 and absmax.size == 2 and (packed[-1] >> 4) == 0


@pytest.mark.parametrize("n", [1, 2, 63, 64, 65, 69, 127, 128, 129, 384, 1000, 2048, 4097, 65536 + 7])
def test_ragged_and_small_lengths(oracle, n):
    rng = np.random.default_rng(n)
    v = (rng.standard_normal(n) * 1.7).astype(np.float32)
    if n >= 192:
        v[64:128] = 0.0  # an all-zero block in the middle (quantize.rs:769-774)
    check_roundtrip(oracle, v, f"n={n}")


def test_empty_input_is_a_noop():
    L = lib()
    assert L.nf4_quantize_dev(None, 0, None, None, None) == 0
    assert L.nf4_dequantize_dev(None, 0, None, None, None, None, None) == 0
    ss = torch.full((1,), -1.0, device=DEV)
    assert L.nf4_double_quantize_dev(None, 0, None, ptr(ss), None) == 0
    assert ss.item() == 0.0


def test_config1_4096x4096_normal_weights(oracle):
    rng = np.random.default_rng(1)
    w = (rng.standard_normal(4096 * 4096) * 0.02).astype(np.float32)
    check_roundtrip(oracle, w, "cfg1")


def test_heavy_tailed_student_t_matrices(oracle):
    # the batch-sweep distribution: Student-t(4) * 0.02 with outlier blocks; two of its shapes
    for seed, shape in ((100, (1024, 4096)), (101, (4096, 4096))):
        v = student_t(np.random.default_rng(seed), shape[0] * shape[1])
        check_roundtrip(oracle, v, f"student-t {shape}")


def test_nan_inf_subnormal_and_signed_zero_blocks(oracle):
    rng = np.random.default_rng(3)
    v = rng.standard_normal(64 * 12).astype(np.float32)
    v[5] = np.nan                      # NaN inside a normal block
    v[64:128] = np.nan                 # all-NaN block -> absmax 0, code 7
    v[130] = np.inf                    # +inf makes the block's absmax inf
    v[200] = -np.inf
    v[256:320] = 1e-42                 # subnormal block
    v[320:384] = -0.0
    v[384:448] = np.float32(3.0e38)    # near-overflow block
    v[448] = np.float32(1e-45)
    v[512:576] = np.float32(-7.25)     # constant block: every value is -absmax
    check_roundtrip(oracle, v, "specials")


def test_values_on_and_next_to_every_decision_boundary(oracle):
    lv = oracle.levels()
    mids = (lv[:-1].astype(np.float64) + lv[1:].astype(np.float64)) / 2
    pts = []
    for c in np.concatenate([lv, mids.astype(np.float32)]):
        b = int(np.array([c], np.float32).view(np.int32)[0])
        pts.append((np.arange(-32, 33) + b).astype(np.int32).view(np.float32))
    cand = np.concatenate(pts)
    cand = cand[np.abs(cand) <= 1.0]
    for scale in (1.0, 0.75, 3.1415927, 1e-3):
        blocks = []
        for i in range(0, cand.size, 63):
            blk = np.concatenate([[np.float32(1.0)], cand[i:i + 63]]).astype(np.float32)
            blk = np.pad(blk, (0, 64 - blk.size))
            blocks.append(blk * np.float32(scale))
        check_roundtrip(oracle, np.concatenate(blocks), f"boundaries x{scale}")


def test_code_selection_matches_the_literal_scan_for_all_f32():
    # 2^32 bit patterns: the kernels' bisection against the sixteen-way scan, on the device
    bad = ctypes.c_uint64(99)
    _lib.check(lib().nf4_selfcheck_code_selection(0, 1 << 32, ctypes.byref(bad)))
    assert bad.value == 0


@pytest.mark.parametrize("absmax", [1.0, 0.75, 3.1415927, 0.0517, 1e-3, 6.1e-5, 1e-38, 3e38,
                                    1.0000001, 0.99999994, 1e-31, 1e31, 0.0, float("inf")])
def test_division_free_fast_path_equals_exact_division_for_all_x(absmax):
    # every f32 x with |x| <= absmax (2^32 bit patterns walked), per block scale
    bad = ctypes.c_uint64(99)
    _lib.check(lib().nf4_selfcheck_quantize_fast_path(0, 1 << 32, absmax, ctypes.byref(bad)))
    assert bad.value == 0


def test_quantization_is_deterministic(oracle):
    # qwennet.rs:3041-3047: resume re-quantizes and expects identical bytes
    v = (np.random.default_rng(9).standard_normal(1 << 20) * 0.02).astype(np.float32)
    a = quantize_dev(v)
    b = quantize_dev(v)
    assert bits_equal(a[0], b[0]) and bits_equal(a[1], b[1])


def test_unaligned_device_pointers_take_the_generic_path(oracle):
    L = lib()
    v = (np.random.default_rng(21).standard_normal(1000) * 0.5).astype(np.float32)
    buf = torch.zeros(1001, dtype=torch.float32, device=DEV)
    buf[1:] = torch.from_numpy(v).to(DEV)
    codes = torch.zeros(501 + 16, dtype=torch.uint8, device=DEV)
    absmax = torch.zeros(16, dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_quantize_dev(ctypes.c_void_p(buf.data_ptr() + 4), 1000,
                                  ctypes.c_void_p(codes.data_ptr() + 1), ptr(absmax), None))
    torch.cuda.synchronize()
    o_packed, o_absmax = oracle.quantize_packed(v)
    assert bits_equal(codes.cpu().numpy()[1:501], o_packed)
    assert bits_equal(absmax.cpu().numpy(), o_absmax)
    out = torch.zeros(1001, dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_dequantize_dev(ctypes.c_void_p(codes.data_ptr() + 1), 1000, ptr(absmax), None,
                                    None, ctypes.c_void_p(out.data_ptr() + 4), None))
    torch.cuda.synchronize()
    assert bits_equal(out.cpu().numpy()[1:], oracle.dequantize_packed(o_packed, 1000, o_absmax))


@pytest.mark.parametrize("dq", [False, True])
def test_quantize_dequantize_roundtrip_entry_points(oracle, dq):
    # quantize.rs:404-416
    L = lib()
    v = (np.random.default_rng(33).standard_normal(4096 * 3 + 17)).astype(np.float32)
    expect = oracle.quantize_dequantize(v, dq)
    n = v.size
    ws_bytes = L.nf4_quantize_dequantize_workspace_bytes(n)
    d_v, d_o = dev(v), torch.zeros(n, dtype=torch.float32, device=DEV)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    _lib.check(L.nf4_quantize_dequantize_dev(ptr(d_v), n, int(dq), ptr(d_o), ptr(ws), ws_bytes, None))
    torch.cuda.synchronize()
    assert bits_equal(d_o.cpu().numpy(), expect)
    out = np.zeros(n, np.float32)
    _lib.check(L.nf4_quantize_dequantize_host(v.ctypes.data_as(ctypes.c_void_p), n, int(dq),
                                              out.ctypes.data_as(ctypes.c_void_p)))
    assert bits_equal(out, expect)


def test_host_pointer_entry_points(oracle):
    L = lib()
    v = (np.random.default_rng(44).standard_normal(100_003) * 0.02).astype(np.float32)
    n = v.size
    packed = np.zeros((n + 1) // 2, np.uint8)
    absmax = np.zeros((n + 63) // 64, np.float32)
    vp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    _lib.check(L.nf4_quantize_host(vp(v), n, vp(packed), vp(absmax)))
    o_packed, o_absmax = oracle.quantize_packed(v)
    assert bits_equal(packed, o_packed) and bits_equal(absmax, o_absmax)
    sc = np.zeros(absmax.size, np.uint8)
    sos = np.zeros(1, np.float32)
    _lib.check(L.nf4_double_quantize_host(vp(absmax), absmax.size, vp(sc), vp(sos)))
    o_sc, o_sos = oracle.double_quantize(o_absmax)
    assert bits_equal(sc, o_sc) and sos[0] == o_sos
    out = np.zeros(n, np.float32)
    _lib.check(L.nf4_dequantize_host(vp(packed), n, vp(absmax), None, None, vp(out)))
    assert bits_equal(out, oracle.dequantize_packed(o_packed, n, o_absmax))
    _lib.check(L.nf4_dequantize_host(vp(packed), n, None, vp(sc), vp(sos), vp(out)))
    assert bits_equal(out, oracle.dequantize_packed(o_packed, n, None, o_sc, o_sos))


def test_encode_erase_nothing_decode_is_idempotent(oracle):
    # size-independent property at full config-1 size: quantizing the dequantized matrix
    # reproduces the same codes and absmax (the grid is a fixed point), entirely on the GPU
    L = lib()
    n = 4096 * 4096
    g = torch.Generator(device=DEV).manual_seed(1)
    w = torch.randn(n, device=DEV, generator=g) * 0.02
    nb = n // 64
    p1 = torch.zeros(n // 2, dtype=torch.uint8, device=DEV)
    a1 = torch.zeros(nb, dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_quantize_dev(ptr(w), n, ptr(p1), ptr(a1), None))
    d1 = torch.zeros(n, dtype=torch.float32, device=DEV)
    _lib.check(L.nf4_dequantize_dev(ptr(p1), n, ptr(a1), None, None, ptr(d1), None))
    p2, a2 = torch.zeros_like(p1), torch.zeros_like(a1)
    _lib.check(L.nf4_quantize_dev(ptr(d1), n, ptr(p2), ptr(a2), None))
    torch.cuda.synchronize()
    assert torch.equal(a1, a2)
    assert torch.equal(p1, p2)
    # absmax equals the true block maxima, and every value sits within half the widest gap
    assert torch.equal(a1, w.view(nb, 64).abs().amax(1))
    lv = torch.from_numpy(oracle.levels()).to(DEV)
    gap = (lv[1:] - lv[:-1]).max()
    err = (d1 - w).view(nb, 64).abs()
    assert bool((err <= 0.5 * gap * a1[:, None] + 1e-6).all())


@pytest.mark.parametrize("n_embedding,d_model,dq", [(1000, 64, True), (257, 136, True), (97, 100, False),
                                                    (5000, 1024, True), (33, 7, False)])
def test_embedding_gather_equals_dequantize_then_gather(oracle, n_embedding, d_model, dq):
    # src/qwennet.rs:285-291 dequantizes the whole table and gathers; the kernel gathers and
    # dequantizes only the selected rows.  Same values, bit for bit (blocks straddle rows when
    # d_model is not a multiple of 64).
    from unifur_b200.qwennet import Nf4Embedding
    from unifur_b200.quantize import PackedNf4Tensor

    rng = np.random.default_rng(n_embedding + d_model)
    table = (rng.standard_normal(n_embedding * d_model) * 0.02).astype(np.float32)
    packed, absmax = oracle.quantize_packed(table)
    if dq:
        sc, sos = oracle.double_quantize(absmax)
        ref_table = oracle.dequantize_packed(packed, table.size, None, sc, sos)
    else:
        ref_table = oracle.dequantize_packed(packed, table.size, absmax)
    ref_table = ref_table.reshape(n_embedding, d_model)
    ids = rng.integers(0, n_embedding, size=(3, 41))
    ids[0, 0], ids[2, 40] = 0, n_embedding - 1
    pt = PackedNf4Tensor.quantize(torch.from_numpy(table).to(DEV))
    if dq:
        pt = pt.with_double_quantization()
    emb = Nf4Embedding(pt, n_embedding, d_model)
    got = emb.forward(torch.from_numpy(ids)).cpu().numpy()
    assert got.shape == (3, 41, d_model)
    assert bits_equal(got, ref_table[ids])
    got16 = emb.forward(torch.from_numpy(ids), dtype=torch.bfloat16).float().cpu().numpy()
    assert bits_equal(got16, oracle.round_bf16(ref_table[ids].astype(np.float32)))
    bad = emb.forward(torch.tensor([[-1, n_embedding]]))
    assert torch.isnan(bad).all()


@pytest.mark.parametrize("rows,cols,bf16", [(64, 64, False), (128, 200, True), (256, 1024, True),
                                            (192, 36, False), (100, 72, True), (65, 7, False)])
def test_load_path_quantize_of_the_transpose(oracle, rows, cols, bf16):
    # src/qwennet.rs:1709-1711: transpose2d([out, in]) then PackedNf4Tensor::quantize (+ double
    # quantization).  The fused kernel (rows % 64 == 0) and the workspace route must both give
    # the oracle's bytes for the transposed buffer.
    from unifur_b200.quantize import PackedNf4Tensor
    from unifur_b200.qwennet import Nf4Linear

    rng = np.random.default_rng(rows * 1000 + cols)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    w[0, 0], w[rows - 1, cols - 1] = 0.5, -0.75  # outliers in the first and last block
    if bf16:
        w = oracle.round_bf16(w)
    wt = np.ascontiguousarray(w.T).reshape(-1)
    o_packed, o_absmax = oracle.quantize_packed(wt)
    src = torch.from_numpy(w).to(DEV)
    if bf16:
        src = src.bfloat16()
    p = PackedNf4Tensor.quantize_transposed(src)
    assert np.array_equal(p.codes.cpu().numpy(), o_packed)
    assert bits_equal(p.absmax.cpu().numpy(), o_absmax)
    lin = Nf4Linear.from_checkpoint(src)
    assert (lin.d_input(), lin.d_output()) == (cols, rows)
    o_sc, o_sos = oracle.double_quantize(o_absmax)
    assert np.array_equal(lin.packed().scale_codes.cpu().numpy(), o_sc)
    assert bits_equal(lin.packed().scale_of_scales.cpu().numpy(), np.asarray([o_sos], np.float32))
