"""Pins the CPU oracle against the deterministic known-answer tests of the reference
(src/quantize.rs tests, src/verify.rs quantize certificates, src/qwennet.rs layout KAT).
Each test names the reference test it restates."""
import numpy as np

PUBLISHED = [
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
]


def test_levels_are_the_published_nf4_codebook(oracle):
    # quantize.rs:839-866
    lv = oracle.levels()
    assert lv.dtype == np.float32 and lv.shape == (16,)
    for ours, theirs in zip(lv, PUBLISHED):
        assert ours == np.float32(theirs)


def test_levels_are_sorted_symmetric_and_contain_zero(oracle):
    # quantize.rs:824-837
    lv = oracle.levels()
    assert np.all(lv[:-1] < lv[1:])
    assert lv[0] == -1.0 and lv[-1] == 1.0 and 0.0 in lv and len(lv) == 16


def test_exact_values_survive_a_roundtrip(oracle):
    # quantize.rs:868-879
    values = oracle.levels() * np.float32(0.75)
    codes, absmax = oracle.quantize_simulated(values)
    restored = oracle.dequantize_simulated(codes, values.size, absmax)
    assert np.all(np.abs(restored - values) < 1e-6)
    assert list(codes) == list(range(16))


def test_absmax_endpoints_are_exact(oracle):
    # quantize.rs:881-894
    values = np.full(64, 0.01, np.float32)
    values[7] = -4.25
    values[9] = 2.0
    codes, absmax = oracle.quantize_simulated(values)
    restored = oracle.dequantize_simulated(codes, 64, absmax)
    assert absmax[0] == np.float32(4.25)
    assert codes[7] == 0 and restored[7] == np.float32(-4.25)


def test_all_zero_block_is_exact(oracle):
    # quantize.rs:957-964, verify.rs:1070-1078
    for n in (64, 128):
        codes, absmax = oracle.quantize_simulated(np.zeros(n, np.float32))
        assert np.all(codes == 7) and np.all(absmax == 0.0)
        assert np.all(oracle.dequantize_simulated(codes, n, absmax) == 0.0)
    v = np.zeros(64, np.float32)
    v[3] = 2.5
    codes, absmax = oracle.quantize_simulated(v)
    out = oracle.dequantize_simulated(codes, 64, absmax)
    assert out[0] == 0.0 and out[3] == np.float32(2.5)


def test_ragged_last_block(oracle):
    # quantize.rs:966-973
    values = np.arange(69, dtype=np.float32) * np.float32(0.01)
    codes, absmax = oracle.quantize_simulated(values)
    assert absmax.size == 2 and codes.size == 69
    packed, am2 = oracle.quantize_packed(values)
    assert packed.size == 35 and np.array_equal(absmax, am2)
    assert packed[-1] >> 4 == 0  # odd tail leaves the high nibble clear
    assert oracle.dequantize_packed(packed, 69, absmax).size == 69


def test_packed_nf4_actually_packs(oracle):
    # quantize.rs:793-822 -- residency formulae
    n = 640
    assert oracle.estimated_resident_bytes(n, False) == n // 2 + 10 * 4
    assert oracle.estimated_resident_bytes(n, True) == n // 2 + 10 + 4
    assert abs(8.0 * oracle.estimated_resident_bytes(n, False) / n - 4.5) < 1e-9
    assert 8.0 * oracle.estimated_resident_bytes(n, True) / n < 4.2
    assert abs(oracle.bits_per_value_simulated(64 * 64, False) - 4.5) < 1e-9
    assert oracle.bits_per_value_simulated(64 * 64, True) < 4.2


def test_packed_nf4_roundtrip_matches_simulated_exactly(oracle):
    # quantize.rs:755-791, verify.rs:1086-1120
    rng = np.random.default_rng(7)
    for n in (1000, 63, 384, 2048):
        values = (rng.standard_normal(n) * 1.7).astype(np.float32)
        if n >= 192:
            values[64:128] = 0.0
        codes, absmax = oracle.quantize_simulated(values)
        packed, am2 = oracle.quantize_packed(values)
        assert np.array_equal(absmax, am2)
        a = oracle.dequantize_packed(packed, n, absmax)
        b = oracle.dequantize_simulated(codes, n, absmax)
        assert a.tobytes() == b.tobytes()
        sc, sos = oracle.double_quantize(absmax)
        a = oracle.dequantize_packed(packed, n, None, sc, sos)
        b = oracle.dequantize_simulated(codes, n, None, sc, sos)
        assert a.tobytes() == b.tobytes()


def test_quantization_error_is_bounded_by_half_the_level_gap(oracle):
    # quantize.rs:896-955, verify.rs:1048-1066
    lv = oracle.levels()
    max_gap = np.max(lv[1:] - lv[:-1])
    rng = np.random.default_rng(11)
    values = rng.standard_normal(64 * 32).astype(np.float32)
    codes, absmax = oracle.quantize_simulated(values)
    restored = oracle.dequantize_simulated(codes, values.size, absmax)
    bound = 0.5 * max_gap * np.repeat(absmax, 64) + 1e-6
    assert np.all(np.abs(restored - values) <= bound)
    step = 2.0 * np.repeat(absmax, 64) / 15.0
    am = np.repeat(absmax, 64)
    uniform = np.round((values + am) / step) * step - am
    assert np.sum((values - restored) ** 2) < np.sum((values - uniform) ** 2)


def test_double_quantization_shrinks_overhead_and_keeps_accuracy(oracle):
    # quantize.rs:975-1009
    rng = np.random.default_rng(13)
    values = rng.standard_normal(64 * 64).astype(np.float32)
    plain = oracle.quantize_dequantize(values, False)
    double = oracle.quantize_dequantize(values, True)
    e_plain = np.sum((plain - values) ** 2)
    e_double = np.sum((double - values) ** 2)
    assert e_double < e_plain * 1.1


def test_double_quantization_formula(oracle):
    # quantize.rs:300 and :348 -- divide, multiply, round half away; decode divides first
    absmax = np.array([0.0, 1.0, 0.5, 0.25, 0.3, 1e-3], np.float32)
    sc, sos = oracle.double_quantize(absmax)
    assert sos == np.float32(1.0)
    expect = [0, 255, 128, 64, 77, 0]  # 127.5 -> 128 (half away), 63.75 -> 64, 76.5 -> 77
    assert list(sc) == expect
    sc0, sos0 = oracle.double_quantize(np.zeros(4, np.float32))
    assert sos0 == 0.0 and np.all(sc0 == 0)
    dec = oracle.block_scales_dq(sc, sos)
    assert dec[1] == np.float32(1.0) and dec[2] == np.float32(np.float32(128) / np.float32(255))


def test_quantized_weights_stay_on_the_grid(oracle):
    # quantize.rs:1132-1163
    rng = np.random.default_rng(17)
    values = rng.standard_normal(4 * 64).astype(np.float32)
    restored = oracle.quantize_dequantize(values, False)
    lv = oracle.levels()
    for b in range(4):
        am = np.max(np.abs(values[b * 64:(b + 1) * 64]))
        grid = lv * am
        for r in restored[b * 64:(b + 1) * 64]:
            assert np.any(np.abs(grid - r) <= 1e-6 * max(am, 1.0))


def test_nearest_level_tie_and_specials(oracle):
    # quantize.rs:208-219 -- strict '<': ties keep the lower index; NaN and inf give code 0
    lv = oracle.levels()
    assert oracle.nearest_level_codes([np.nan, np.inf, -np.inf])[0] == 0
    assert list(oracle.nearest_level_codes([np.inf, -np.inf])) == [0, 0]
    assert list(oracle.nearest_level_codes(lv)) == list(range(16))
    assert list(oracle.nearest_level_codes([0.0, -0.0, 2.0, -2.0])) == [7, 7, 15, 0]
    # an exact f32 tie between two neighbours: 0.5 lies between levels 12 and 13
    mid = np.float32(0.5) * (lv[7] + lv[8])  # exact: halving is exact in binary
    d_lo = abs(np.float32(mid - lv[7]))
    d_hi = abs(np.float32(mid - lv[8]))
    if d_lo == d_hi:
        assert oracle.nearest_level_codes([mid])[0] == 7


def test_nan_and_inf_blocks(oracle):
    # quantize.rs:103 (maxNum ignores NaN), :109-112
    v = np.full(64, 0.5, np.float32)
    v[5] = np.nan
    codes, absmax = oracle.quantize_simulated(v)
    assert absmax[0] == np.float32(0.5) and codes[5] == 0 and codes[0] == 15
    v = np.full(64, np.nan, np.float32)
    codes, absmax = oracle.quantize_simulated(v)
    assert absmax[0] == 0.0 and np.all(codes == 7)
    v = np.full(64, 1.0, np.float32)
    v[0] = np.inf
    codes, absmax = oracle.quantize_simulated(v)
    assert np.isinf(absmax[0]) and codes[0] == 0 and np.all(codes[1:] == 7)


def test_linear_weight_layout_is_in_times_out(oracle):
    # qwennet.rs:2196-2211
    w = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    y = oracle.linear_in_out(np.array([[1.0, -1.0]], np.float32), w)
    assert np.allclose(y, [[-3.0, -3.0, -3.0]], atol=1e-6)


def test_lora_identity_and_dense_update(oracle):
    # quantize.rs:1011-1047, verify.rs:1080-1084
    rng = np.random.default_rng(19)
    a = rng.standard_normal((16, 4)).astype(np.float32)
    x = rng.uniform(-1, 1, (3, 16)).astype(np.float32)
    assert np.all(oracle.lora_forward(x, a, np.zeros((4, 8), np.float32), 1.0) == 0.0)
    a = rng.standard_normal((12, 3)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, (3, 6)).astype(np.float32)
    x = rng.uniform(-1, 1, (4, 12)).astype(np.float32)
    factored = oracle.lora_forward(x, a, b, 2.0)
    dense = x.astype(np.float64) @ oracle.lora_delta_weight(a, b, 2.0)
    assert np.max(np.abs(factored - dense)) < 1e-5


def test_lcg_fixture_generator(oracle):
    # qwennet.rs:2567-2575 -- first values from state 1, computed by hand in integers
    vals, _ = oracle.lcg_fill(1, 3)
    s = 1
    exp = []
    for _ in range(3):
        s = (s * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        bits = s >> 48
        exp.append((np.float32(bits) / np.float32(65535) - np.float32(0.5)) * np.float32(0.1))
    assert [np.float32(v) for v in vals] == exp


def test_bf16_rounding(oracle):
    # precision.rs:95-127 -- nearest-even on the 8-bit significand
    x = np.array([1.0, 1.00390625, 1.01171875, 3.14159265, -2.71828183, 0.0], np.float32)
    r = oracle.round_bf16(x)
    assert r[0] == 1.0
    assert r[1] == np.float32(1.0)          # 1 + 2^-8 ties to even (1.0)
    assert r[2] == np.float32(1.015625)     # 1 + 3*2^-8 ties to even (1 + 2^-6)
    import torch
    t = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(r, t)
