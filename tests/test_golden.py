"""The committed fixtures of tests/golden/nf4_golden.npz (made by tests/golden/make_golden.py).

CPU: the oracle still produces them (a change of the oracle is noticed).  GPU: the CUDA path
produces them through the C ABI with no oracle involved."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nf4_golden.npz")
CASES = ["levels_x_0p75", "absmax_endpoints", "zeros", "ragged_69", "lcg_640", "normal_0p02_seed1",
         "student_t4_seed100", "specials"]


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def same_bits(a, b):
    """Bit equality, with any NaN equal to any NaN (payloads differ between CPU and GPU)."""
    a, b = np.asarray(a, np.uint32), np.asarray(b, np.uint32)
    nan = lambda u: (u & 0x7fffffff) > 0x7f800000
    return a.shape == b.shape and bool(np.all((a == b) | (nan(a) & nan(b))))


@pytest.mark.parametrize("name", CASES)
def test_oracle_reproduces_the_golden_vectors(oracle, golden, name):
    v = golden[f"{name}/values"]
    packed, absmax = oracle.quantize_packed(v)
    assert np.array_equal(packed, golden[f"{name}/packed"])
    assert same_bits(absmax.view(np.uint32), golden[f"{name}/absmax_bits"])
    sc, sos = oracle.double_quantize(absmax)
    assert np.array_equal(sc, golden[f"{name}/scale_codes"])
    assert same_bits(np.asarray([sos], np.float32).view(np.uint32), golden[f"{name}/scale_of_scales_bits"])
    assert same_bits(oracle.dequantize_packed(packed, v.size, absmax).view(np.uint32),
                     golden[f"{name}/deq_bits"])
    assert same_bits(oracle.dequantize_packed(packed, v.size, None, sc, sos).view(np.uint32),
                     golden[f"{name}/deq_dq_bits"])


def test_known_answers_inside_the_golden_file(golden):
    # src/quantize.rs:868-879: the sixteen levels x 0.75 quantize to codes 0..15 with absmax 0.75
    assert golden["levels_x_0p75/packed"].tolist() == [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]
    assert golden["levels_x_0p75/absmax_bits"].view(np.float32).tolist() == [0.75]
    # src/quantize.rs:881-894: absmax of the block is 4.25 and both outliers survive exactly
    deq = golden["absmax_endpoints/deq_bits"].view(np.float32)
    assert golden["absmax_endpoints/absmax_bits"].view(np.float32)[0] == 4.25
    assert deq[7] == -4.25 and abs(deq[9] - 2.0) < 0.5 * 0.34 * 4.25
    # src/quantize.rs:957-964 and :966-973
    assert not golden["zeros/deq_bits"].any()
    assert golden["ragged_69/packed"].size == 35 and golden["ragged_69/absmax_bits"].size == 2


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_path_reproduces_the_golden_vectors(golden, name):
    torch = pytest.importorskip("torch")
    from unifur_b200.quantize import PackedNf4Tensor

    dev = torch.device("cuda", 0)
    v = torch.from_numpy(golden[f"{name}/values"]).to(dev)
    p = PackedNf4Tensor.quantize(v)
    assert np.array_equal(p.codes.cpu().numpy(), golden[f"{name}/packed"])
    assert same_bits(p.absmax.cpu().numpy().view(np.uint32), golden[f"{name}/absmax_bits"])
    assert same_bits(p.dequantize().cpu().numpy().view(np.uint32), golden[f"{name}/deq_bits"])
    q = p.with_double_quantization()
    assert np.array_equal(q.scale_codes.cpu().numpy(), golden[f"{name}/scale_codes"])
    assert same_bits(q.scale_of_scales.cpu().numpy().view(np.uint32), golden[f"{name}/scale_of_scales_bits"])
    assert same_bits(q.dequantize().cpu().numpy().view(np.uint32), golden[f"{name}/deq_dq_bits"])


@pytest.mark.gpu
def test_cuda_forward_reproduces_the_golden_output(golden):
    torch = pytest.importorskip("torch")
    from unifur_b200 import _lib
    from unifur_b200.quantize import PackedNf4Tensor, linear_forward

    dev = torch.device("cuda", 0)
    M, K, N, r = (int(t) for t in golden["forward/shape"])
    p = PackedNf4Tensor(torch.from_numpy(golden["forward/packed"]).to(dev), N * K,
                        torch.from_numpy(golden["forward/absmax"]).to(dev))
    x = torch.from_numpy(golden["forward/x"]).to(dev).bfloat16()
    a = torch.from_numpy(golden["forward/a"]).to(dev).bfloat16()
    b = torch.from_numpy(golden["forward/b"]).to(dev).bfloat16()
    y = linear_forward(x, p, K, N, _lib.LAYOUT_OUT_IN, lora_a=a, lora_b=b, lora_scale=2.0)
    ref = golden["forward/y_f64"]
    err = np.linalg.norm(y.double().cpu().numpy() - ref) / np.linalg.norm(ref)
    assert err <= 1e-3 + 2.0 ** -9  # the north star's bar plus the bf16 rounding of the output
