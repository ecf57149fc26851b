"""Writes tests/golden/nf4_golden.npz: inputs and expected outputs of the NF4 path.

The reference is Rust and cannot be run where this repository is built, so the expected values
come from the CPU oracle (oracle/nf4_oracle.c), which tests/test_oracle_kat.py pins to every
deterministic known answer the reference's own tests hold (src/quantize.rs:755-1163,
src/qwennet.rs:2196-2211, 2567-2575).  The inputs are those known-answer inputs plus seeded
samples of the benchmark configurations' distributions.  The file lets the CUDA path be checked
without the oracle at hand, and lets a change of the oracle itself be noticed.

Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import nf4_oracle as o  # noqa: E402


def case(values):
    values = np.ascontiguousarray(values, np.float32)
    packed, absmax = o.quantize_packed(values)
    sc, sos = o.double_quantize(absmax)
    return {
        "values": values,
        "packed": packed,
        "absmax_bits": absmax.view(np.uint32),
        "scale_codes": sc,
        "scale_of_scales_bits": np.asarray([sos], np.float32).view(np.uint32),
        "deq_bits": o.dequantize_packed(packed, values.size, absmax).view(np.uint32),
        "deq_dq_bits": o.dequantize_packed(packed, values.size, None, sc, sos).view(np.uint32),
    }


def main():
    out = {}
    levels = o.levels()
    kat_block = np.full(64, 0.01, np.float32)
    kat_block[7], kat_block[9] = -4.25, 2.0
    rng = np.random.default_rng(1)
    t_rng = np.random.default_rng(100)
    z = t_rng.standard_normal(4096)
    chi = np.sqrt((t_rng.standard_normal((4, 4096)) ** 2).sum(0) / 4.0)
    specials = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e-45, -1e-45, 3e38, -3e38] + [0.5] * 55
                        + [np.nan] * 64 + [np.inf] + [1.0] * 63, np.float32)
    cases = {
        "levels_x_0p75": levels * np.float32(0.75),               # src/quantize.rs:868-879
        "absmax_endpoints": kat_block,                             # src/quantize.rs:881-894
        "zeros": np.zeros(64, np.float32),                         # src/quantize.rs:957-964
        "ragged_69": np.arange(69, dtype=np.float32) * np.float32(0.01),  # src/quantize.rs:966-973
        "lcg_640": o.lcg_fill(1, 640)[0],                         # src/qwennet.rs:2567-2575
        "normal_0p02_seed1": (rng.standard_normal(4096) * 0.02).astype(np.float32),
        "student_t4_seed100": (0.02 * z / chi).astype(np.float32),
        "specials": specials,
    }
    for name, v in cases.items():
        for k, a in case(v).items():
            out[f"{name}/{k}"] = a
    # one small QLoRA forward (bf16-rounded activations and adapter, f64 accumulation)
    g = np.random.default_rng(7)
    M, K, N, r = 3, 128, 40, 4
    w = (g.standard_normal((N, K)) * 0.02).astype(np.float32)
    packed, absmax = o.quantize_packed(w)
    x = o.round_bf16((g.standard_normal((M, K))).astype(np.float32))
    a = o.round_bf16((g.standard_normal((r, K)) * 0.01).astype(np.float32))
    b = o.round_bf16((g.standard_normal((N, r)) * 0.01).astype(np.float32))
    y = o.qlora_forward_bnb(x, packed, absmax, N, K, a, b, 2.0, None, None, 0.0)
    out.update({"forward/x": x, "forward/packed": packed, "forward/absmax": absmax, "forward/a": a,
                "forward/b": b, "forward/y_f64": np.asarray(y, np.float64),
                "forward/shape": np.asarray([M, K, N, r], np.int64)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nf4_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes, sha256",
          hashlib.sha256(open(path, "rb").read()).hexdigest()[:16])


if __name__ == "__main__":
    main()
