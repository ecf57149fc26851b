"""The C-ABI shared library builds, loads and exports every symbol include/nf4_b200.h declares.
No compute call is made here (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from unifur_b200 import build

    build.build()
    from unifur_b200 import _lib

    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nf4_b200.h")).read()
    return sorted(set(re.findall(r"NF4_API[^;(]*?\b(nf4_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert len(names) >= 25
    for must in ("nf4_quantize_dev", "nf4_dequantize_dev", "nf4_double_quantize_dev",
                 "nf4_linear_forward_dev", "nf4_weight_linear_forward_host", "nf4_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_python_binding_covers_the_header(lib):
    from unifur_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_struct_layout_matches_the_header(lib):
    from unifur_b200 import _lib

    # 4 x 4-byte + 3 x 8 + 8 pointers + (4 + 4) + pointer + 8 + pointer + 8
    assert ctypes.sizeof(_lib.LinearArgs) == 16 + 24 + 64 + 8 + 8 + 8 + 8 + 8


def test_pure_host_helpers(lib):
    assert lib.nf4_version() >= 100
    assert lib.nf4_num_blocks(69) == 2 and lib.nf4_packed_bytes(69) == 35
    assert lib.nf4_estimated_resident_bytes(640, 0) == 320 + 40      # quantize.rs:804
    assert lib.nf4_estimated_resident_bytes(640, 1) == 320 + 10 + 4  # quantize.rs:807-811
    import numpy as np

    lv = np.zeros(16, np.float32)
    lib.nf4_levels(lv.ctypes.data_as(ctypes.c_void_p))
    from oracle import nf4_oracle

    assert lv.tobytes() == nf4_oracle.levels().tobytes()


def test_workspace_sizes_cover_every_route(lib):
    # host arithmetic only: what nf4_linear_workspace_bytes reports must hold the scratch of every
    # kernel a call of these sizes can be routed to, in either orientation and tensor type
    ws = lambda rows, k, n, r: int(lib.nf4_linear_workspace_bytes(rows, k, n, r))
    k, n, r = 4096, 11008, 16
    # more than 16 rows: the f16 copy of x, T, and for the reference's orientation the weight's
    # nibbles transposed plus its scales as f16 [n / 64][k]
    big = ws(2048, k, n, r)
    assert big >= 2048 * k * 2 + k * n // 2 + (n // 64) * k * 2
    # ... which a d_out that is no multiple of 64 cannot use
    assert ws(2048, k, n + 8, r) < ws(2048, k, n, r)
    # at most 16 rows: flag words, T, and the halves / results of f32 rows (16 x k bf16, 16 x n f32)
    small = ws(4, k, n, r)
    assert small >= 256 + 16 * k * 2 + 16 * n * 4
    assert small < 4 * 1024 * 1024
    # d_in beyond 4096 at decode sizes: the parts' partial sums
    assert ws(8, 18944, 3584, 16) >= 5 * 8 * 3584 * 4
    # sizes grow with the rank, and a multiple of 256 bytes comes back
    assert ws(2048, k, n, 64) > ws(2048, k, n, 16) and big % 256 == 0 and small % 256 == 0
    # the backward holds a forward with d_in and d_out exchanged, two [rows][rank] f32 intermediates
    # and one factor transposed
    bw = int(lib.nf4_qlora_backward_workspace_bytes(2048, k, n, r))
    assert bw >= ws(2048, n, k, r) + 2 * 2048 * r * 4 + r * n * 2


def test_invalid_arguments_are_reported_not_fatal(lib):
    from unifur_b200 import _lib

    a = _lib.LinearArgs()
    a.struct_bytes = 3
    st = lib.nf4_linear_forward_dev(ctypes.byref(a), None)
    assert st == -1 and b"struct_bytes" in lib.nf4_last_error()
    assert lib.nf4_linear_forward_dev(None, None) == -1
    out = ctypes.c_void_p()
    assert lib.nf4_weight_from_values_host(None, 4, 4, 0, 1, ctypes.byref(out)) == -1
    assert lib.nf4_quantize_host(None, 10, None, None) == -1
    assert lib.nf4_quantize_host(None, 0, None, None) == 0  # empty input is a no-op
