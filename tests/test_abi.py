"""CPU tests of the boundary: the library loads, exports every declared symbol, and the host
logic (geometry, shape and argument errors, graph building) behaves like the reference's."""
import ctypes as C
import os
import re

import pytest

import rlx_b200 as R
from rlx_b200._lib import LIB_PATH, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for h in ("rlxq.h", "rlxq_session.h", "rlxq_tp.h", "rlxq_lm.h", "rlxq_moe.h", "rlxq_gguf.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        names += re.findall(r"^RLXQ_API [^;(]*?\b(rlxq_[a-z0-9_]+)\(", text, flags=re.M)
    return names


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 25
    raw = C.CDLL(LIB_PATH)
    for nm in names:
        assert hasattr(raw, nm), f"{nm} declared in include/ but not exported by librlxq.so"


def test_version_and_status_strings():
    assert lib.rlxq_version() >= 100
    assert lib.rlxq_status_string(0) == b"ok"
    assert b"shape" in lib.rlxq_status_string(-2)


def test_geometry_matches_reference_table():
    # rlx-ir/src/quant.rs:138-164
    assert R.scheme_geometry(R.QuantScheme.GgufQ4K) == (256, 144)
    assert R.scheme_geometry(R.QuantScheme.GgufQ6K) == (256, 210)
    assert R.scheme_geometry(R.QuantScheme.GgufQ4_0) == (32, 18)
    assert R.scheme_geometry(R.QuantScheme.GgufQ8_0) == (32, 34)
    assert R.scheme_geometry(R.QuantScheme.GgufQ5K) == (256, 176)
    assert R.scheme_geometry(R.QuantScheme.GgufQ8K) == (256, 292)
    assert R.scheme_geometry(R.QuantScheme.GgufQ2K) == (256, 84)
    assert R.scheme_geometry(R.QuantScheme.GgufQ3K) == (256, 110)
    assert R.scheme_geometry(8) == (32, 20) and R.scheme_geometry(9) == (32, 22) and R.scheme_geometry(10) == (32, 24)
    for bad in (11, 12, 100):
        with pytest.raises(R.RlxqError) as e:
            R.scheme_geometry(bad)
        assert e.value.status == -1


def test_packed_bytes_of_benchmark_shapes():
    assert R.packed_bytes(7, 4096, 4096) == 17_825_792
    assert R.packed_bytes(6, 4096, 11008) == 25_362_432
    assert R.packed_bytes(6, 11008, 4096) == 25_362_432
    assert R.packed_bytes(0, 4096, 14336) == 33_030_144
    assert R.packed_bytes(2, 14336, 4096) == 48_168_960
    assert R.packed_bytes(0, 8192, 28672) == 132_120_576
    assert R.packed_bytes(7, 8192, 28672) == 249_561_088
    with pytest.raises(R.RlxqError) as e:
        R.packed_bytes(0, 128, 4)
    assert e.value.status == -2


def test_argument_errors_without_a_device():
    st = lib.rlxq_matmul(None, 99, None, 0, None, None, 0, 1, 32, 1, None, 0)
    assert st == -1
    st = lib.rlxq_matmul(None, 6, None, 5, None, None, 0, 1, 32, 1, None, 0)
    assert st == -4
    st = lib.rlxq_matmul(None, 6, None, 0, None, None, 0, 1, 33, 1, None, 0)
    assert st == -2
    assert lib.rlxq_matmul(None, 6, None, 0, None, None, 0, 0, 32, 5, None, 0) == 0   # m = 0: empty
    assert lib.rlxq_matmul(None, 6, None, 0, None, None, 0, 1, 32, 1, None, 0) == -3  # y null
    assert lib.rlxq_dequant_f32(None, 6, None, 0, None) == 0
    assert lib.rlxq_dequant_f32(None, 6, None, 31, None) == -2
    assert lib.rlxq_dequant_f32(None, 6, None, 32, None) == -3


def test_options_roundtrip():
    R.set_option("gemv_kernel", 1)
    assert R.get_option("gemv_kernel") == 1
    R.set_option("gemv_kernel", 0)
    with pytest.raises(R.RlxqError):
        R.set_option("no_such_key", 1)


def test_graph_building_errors_mirror_the_reference():
    g = R.Graph("t")
    x = g.input("x", [2, 256])
    w = g.param("w_packed", [R.packed_bytes(0, 256, 4)])
    y = g.dequant_matmul_packed(x, w, R.QuantScheme.GgufQ4K, 4)
    g.set_outputs([y])
    # a param of the wrong size is rejected when the node is built
    bad = g.param("w_bad", [100])
    with pytest.raises(R.RlxqError) as e:
        g.dequant_matmul_packed(x, bad, R.QuantScheme.GgufQ4K, 4)
    assert e.value.status == -2
    with pytest.raises(R.RlxqError):
        g.dequant_matmul_packed(x, x, R.QuantScheme.GgufQ4K, 4)   # weight must be a U8 param
    with pytest.raises(R.RlxqError):
        g.set_outputs([w])


def test_session_needs_a_cuda_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    g = R.Graph("t")
    x = g.input("x", [1, 256])
    w = g.param("w", [R.packed_bytes(7, 256, 4)])
    g.set_outputs([g.dequant_matmul_packed(x, w, R.QuantScheme.GgufQ8_0, 4)])
    with pytest.raises(R.RlxqError) as e:
        R.Session(R.Device.Cuda).compile(g)
    assert e.value.status == -6 and "no CUDA device" in str(e.value)   # loud, no CPU fallback


def test_workspace_bytes_are_modest():
    """The reference reserves k*n*4 bytes of f32 scratch (rlx-cuda/src/gguf_gpu.rs:35-59); the GEMV
    paths need the quantised activations and a few partial tiles only."""
    for s, m, k, n in ((6, 1, 4096, 11008), (6, 1, 11008, 4096), (6, 8, 11008, 4096), (0, 1, 28672, 8192)):
        ws = R.workspace_bytes(s, m, k, n)
        assert ws % 16 == 0 and ws < k * n * 4 // 100
