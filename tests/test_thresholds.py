"""The fifteen decision thresholds baked into the CUDA code (csrc/nf4_tables.inc) agree
with the reference's sixteen-way scan as restated by the oracle."""
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def read_tables():
    text = open(os.path.join(ROOT, "unifur_b200", "csrc", "nf4_tables.inc")).read()
    lv = re.search(r"NF4_LEVEL_BITS_LIST \\\n(.*)\n", text).group(1)
    th = re.search(r"NF4_THRESHOLD_BITS_LIST \\\n(.*)\n", text).group(1)
    conv = lambda s: np.array([int(x.strip().rstrip("u"), 16) for x in s.split(",")],
                              dtype=np.uint32).view(np.float32)
    return conv(lv), conv(th)


def code_by_thresholds(v, th):
    v = np.asarray(v, np.float32)
    with np.errstate(invalid="ignore"):
        return (v[:, None] >= th[None, :]).sum(1).astype(np.uint8)


def test_level_table_matches_the_oracle(oracle):
    lv, _ = read_tables()
    assert lv.tobytes() == oracle.levels().tobytes()


def test_thresholds_are_exact_boundaries(oracle):
    _, th = read_tables()
    assert th.size == 15 and np.all(th[:-1] < th[1:])
    for i, t in enumerate(th):
        below = np.nextafter(t, np.float32(-np.inf), dtype=np.float32)
        assert oracle.nearest_level_codes([below])[0] == i
        assert oracle.nearest_level_codes([t])[0] == i + 1


def test_threshold_count_equals_scan_near_every_boundary(oracle):
    lv, th = read_tables()
    pts = []
    for c in np.concatenate([lv, th, np.float32([0.5 * (a + b) for a, b in zip(lv[:-1], lv[1:])])]):
        bits = np.array([c], np.float32).view(np.int32)[0]
        neigh = (np.arange(-300, 301, dtype=np.int64) + int(bits)).astype(np.int32)
        pts.append(neigh.view(np.float32))
    v = np.concatenate(pts)
    v = v[np.isfinite(v)]
    assert np.array_equal(code_by_thresholds(v, th), oracle.nearest_level_codes(v))


def test_threshold_count_equals_scan_on_random_and_special_values(oracle):
    _, th = read_tables()
    rng = np.random.default_rng(5)
    v = np.concatenate([
        rng.uniform(-1, 1, 2_000_000).astype(np.float32),
        rng.standard_normal(500_000).astype(np.float32),
        rng.integers(0, 2**32, 1_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32),
        np.float32([0.0, -0.0, 1.0, -1.0, 2.0, -2.0, 1e-45, -1e-45, 65536.0, -65536.0, np.nan]),
    ])
    # domain of the bisection: NaN and |v| <= 65536 (a normalised value never exceeds 1)
    v = v[np.isnan(v) | (np.abs(v) <= 65536.0)]
    assert np.array_equal(code_by_thresholds(v, th), oracle.nearest_level_codes(v))
