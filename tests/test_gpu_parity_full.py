"""GPU parity at the full sizes of the named configurations, against the CPU oracle.

The forwards run at full size on the GPU; the oracle (C restatement of the reference, f64
accumulation over its own bit-exact dequantized weights) is evaluated on scattered slices of the
output, so that the CPU side stays within seconds.  Tolerance of the forward (the north star's):
relative L2 <= 1e-3 for bf16 activations with f32 accumulation, plus the single bf16 rounding of
the output (2^-9)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import DEV, bits_equal, dev, lib, quantize_dev, student_t  # noqa: E402
from unifur_b200 import _lib  # noqa: E402

TOL = 1e-3 + 2.0 ** -9

QWEN2_7B_BLOCK = [("q", 3584, 3584), ("k", 3584, 512), ("v", 3584, 512), ("o", 3584, 3584),
                  ("gate", 3584, 18944), ("up", 3584, 18944), ("down", 18944, 3584)]


def _forward_full(m, k, n, r, seed, scale=2.0):
    """Seeded full-size QLoRA forward on the GPU; returns everything a slice check needs."""
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    g = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randn(n * k, device=DEV, generator=g) * 0.02
    packed = PackedNf4Tensor.quantize(w)
    del w
    a = (torch.randn(r, k, device=DEV, generator=g) * 0.01).bfloat16()
    b = (torch.randn(n, r, device=DEV, generator=g) * 0.01).bfloat16()
    x = torch.randn(m, k, device=DEV, generator=g).bfloat16()
    y = linear_forward(x, packed, k, n, _lib.LAYOUT_OUT_IN, lora_a=a, lora_b=b, lora_scale=scale)
    torch.cuda.synchronize()
    return packed, a, b, x, y


def _check_slices(oracle, packed, a, b, x, y, k, n, col_starts, row_sets, width=128, scale=2.0):
    """y[rows, c0:c0+width] against the oracle: the slice's packed rows are dequantized by the
    oracle's C code (not by the library), then multiplied in f64."""
    a64, x_all = a.double().cpu().numpy(), x.double().cpu().numpy()
    for c0 in col_starts:
        c1 = min(c0 + width, n)
        codes = packed.codes[c0 * (k // 2): c1 * (k // 2)].cpu().numpy()
        absmax = packed.absmax[c0 * (k // 64): c1 * (k // 64)].cpu().numpy()
        wd = oracle.dequantize_packed(codes, (c1 - c0) * k, absmax).reshape(c1 - c0, k).astype(np.float64)
        b64 = b[c0:c1].double().cpu().numpy()
        for rows in row_sets:
            xs = x_all[rows]
            ref = xs @ wd.T + scale * (xs @ a64.T) @ b64.T
            got = y[rows, c0:c1].double().cpu().numpy()
            err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
            assert err <= TOL, (c0, rows, err)


def test_config3_prefill_full_width_against_the_oracle(oracle):
    # x [2048, 4096], W [14336, 4096], rank 64: eight scattered 128-column slices, among them
    # the first and the last columns, three sets of activation rows
    m, k, n, r = 2048, 4096, 14336, 64
    packed, a, b, x, y = _forward_full(m, k, n, r, seed=5)
    cols = [0, 1792, 3584 + 64, 5000, 7168 - 64, 9999, 12800, n - 128]
    _check_slices(oracle, packed, a, b, x, y, k, n, cols, [slice(0, 16), slice(1000, 1016), slice(2040, 2048)])


@pytest.mark.parametrize("name,k,n", QWEN2_7B_BLOCK)
def test_config5_prefill_4096_tokens_every_projection(oracle, name, k, n):
    # the seven projections of the Qwen2-7B-shaped block at 4096 tokens, rank 16 (the down
    # projection walks 296 k-stages per tile)
    m, r = 4096, 16
    packed, a, b, x, y = _forward_full(m, k, n, r, seed=200 + len(name) + k % 97)
    cols = sorted({0, (n // 2) // 128 * 128, n - 128})
    _check_slices(oracle, packed, a, b, x, y, k, n, cols, [slice(0, 8), slice(2048, 2056), slice(4088, 4096)])


@pytest.mark.parametrize("k,n", [(18944, 1792), (3584, 9472), (3584, 256), (18944, 896), (18944, 448), (3584, 2368)])
def test_config5_prefill_4096_tokens_shards(oracle, k, n):
    # the column shards a GPU owns when the block is split over two, four or eight GPUs (down, gate / up, k / v):
    # other tile counts than the whole projections, so other splits of the tiles between the CTAs
    m, r = 4096, 16
    packed, a, b, x, y = _forward_full(m, k, n, r, seed=300 + n % 89)
    cols = sorted({0, (n // 2) // 128 * 128, n - 128})
    _check_slices(oracle, packed, a, b, x, y, k, n, cols, [slice(0, 8), slice(2048, 2056), slice(4088, 4096)])


@pytest.mark.parametrize("f32", [True, False])
def test_config3_in_the_reference_orientation(oracle, f32):
    # the prefill configuration as the reference itself would hold it: x [2048, 4096], W [4096, 14336]
    # with the 64-blocks along d_out, A [4096, 64], B [64, 14336], f32 (its own types) or bf16.  The
    # oracle dequantizes the whole weight; scattered column slices are multiplied in f64.
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    m, k, n, r = 2048, 4096, 14336, 64
    tdt = torch.float32 if f32 else torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(31)
    w = torch.randn(k * n, device=DEV, generator=g) * 0.02
    packed = PackedNf4Tensor.quantize(w)
    del w
    a = (torch.randn(k, r, device=DEV, generator=g) * 0.01).to(tdt)
    b = (torch.randn(r, n, device=DEV, generator=g) * 0.01).to(tdt)
    x = torch.randn(m, k, device=DEV, generator=g).to(tdt)
    y = linear_forward(x, packed, k, n, _lib.LAYOUT_IN_OUT, lora_a=a, lora_b=b, lora_scale=2.0)
    torch.cuda.synchronize()
    wd = oracle.dequantize_packed(packed.codes.cpu().numpy(), k * n, packed.absmax.cpu().numpy()).reshape(k, n)
    a64, b64 = a.double().cpu().numpy(), b.double().cpu().numpy()
    tol = 1e-3 if f32 else TOL
    for rows in (slice(0, 16), slice(1000, 1016), slice(2040, 2048)):
        xs = x[rows].double().cpu().numpy()
        t = xs @ a64
        for c0 in (0, 1792, 5000, 7168 - 64, 9999, n - 128):
            ref = xs @ wd[:, c0:c0 + 128].astype(np.float64) + 2.0 * t @ b64[:, c0:c0 + 128]
            got = y[rows, c0:c0 + 128].double().cpu().numpy()
            err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
            assert err <= tol, (rows, c0, err)


@pytest.mark.parametrize("rows,cols", [(4096, 14336), (14336, 4096)])
def test_config4_the_two_long_matrices_bit_exact(oracle, rows, cols):
    # the 58.7 M-element members of the sweep, heavy-tailed values: codes and absmax bit-exact
    rng = np.random.default_rng(100 + rows % 7)
    v = student_t(rng, rows * cols)
    codes, absmax = quantize_dev(v, packed=True)
    ref_c, ref_a = oracle.quantize_packed(v)
    assert np.array_equal(codes, ref_c)
    assert bits_equal(absmax, ref_a)


def _decode_case(oracle, m, k, n, r, x_scale_rows, seed):
    from test_gpu_linear import check_out_in, make_case

    c = make_case(oracle, seed, m, k, n, r)
    x = c["x"].astype(np.float64)
    for row, s in x_scale_rows.items():
        if row < m:
            x[row] *= s
    c["x"] = oracle.round_bf16(x.astype(np.float32))
    check_out_in(oracle, c, m, k, n, 2.0)


@pytest.mark.parametrize("m", [1, 5, 16])
def test_decode_activations_far_outside_f16_range(oracle, m):
    # bf16 activations the f16 operand type cannot hold: rows scaled by 2^17 (overflow), by 2^-20
    # (below f16's normal range) and mixed rows; the kernel rescales each warp's slice by a power
    # of two, so the tolerance is the usual one
    k, n, r = 4096, 1024, 16
    _decode_case(oracle, m, k, n, r, {i: 2.0 ** 17 for i in range(16)}, 71)
    _decode_case(oracle, m, k, n, r, {i: 2.0 ** -20 for i in range(16)}, 72)
    _decode_case(oracle, m, k, n, r, {0: 2.0 ** 17, 1: 2.0 ** -20, 3: 2.0 ** 30, 9: 2.0 ** -40}, 73)


def test_decode_block_scales_at_both_ends(oracle):
    # the decode kernel multiplies by the f32 block scale after the MMA: weights of any magnitude
    from test_gpu_linear import check_out_in, make_case

    for w_std, seed in ((1e-5, 81), (1e4, 82)):
        c = make_case(oracle, seed, 4, 2048, 512, 16, w_std=w_std)
        check_out_in(oracle, c, 4, 2048, 512, 2.0)


@pytest.mark.parametrize("w_std", [1e-5, 3e3])
def test_prefill_block_scales_at_both_ends(oracle, w_std):
    # The tensor-core GEMM scales the expanded weights in f16: block scales below f16's normal range
    # (6.1e-5) or above 65504 would lose bits there, so the kernel divides all scales by a power of
    # two taken from the largest one (exact) and multiplies the outputs back.
    from test_gpu_linear import check_out_in, make_case

    c = make_case(oracle, 91, 256, 512, 384, 16, w_std=w_std)
    check_out_in(oracle, c, 256, 512, 384, 2.0)
