"""GPU parity for the GGUF schemes beyond the four benchmark formats: Q5_K, Q8_K, Q2_K, Q3_K, and the 32-weight
container types Q4_1, Q5_0, Q5_1 that the reference decodes only when a file is loaded (rlx-gguf/src/lib.rs:635-729).

They complete QuantScheme::is_gguf (rlx-ir/src/quant.rs:170-182): with them every scheme the reference's
`Op::DequantMatMul` accepts runs on the GPU (the reference sends all of them to a host fallback or to its
dequantise-everything kernel).  Dequantisation is bit-exact against the oracle; the matmul goes through the integer-MMA units where the shape allows (Q5_K, Q8_K, Q2_K, Q3_K), else the
general kernel (f32 accumulation in a different order from the CPU's) and is held to 2e-5 * |x| * |w_row|.
Q5_K also has the integer streaming GEMV (batch 1-2); Q5_K, Q2_K and Q3_K the tensor-core GEMM (batch > 8, k a multiple of
256 / 1024 / 2048, Q8_K 1024; f32 activations as two bf16 halves).
"""
import json
import os

import numpy as np
import pytest

import rlx_b200 as R
from oracle import oracle as O
from tests.helpers import assert_within_tolerance, bound, make_case, reference

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
NEW = ["q5_k", "q8_k", "q2_k", "q3_k", "q4_1", "q5_0", "q5_1"]


def _gpu_dequant(scheme, w, n_elems):
    import torch
    out = R.dequant_f32(torch.from_numpy(w).cuda(), scheme, n_elems)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _gpu_matmul(scheme, w, x, n, x_bf16=False):
    import torch
    xd = torch.from_numpy(x).cuda()
    if x_bf16:
        xd = xd.to(torch.bfloat16)
    y = R.matmul(xd, torch.from_numpy(w).cuda(), scheme, n)
    R.device_status()
    return y.cpu().numpy()


@pytest.mark.parametrize("sch", NEW)
@pytest.mark.parametrize("nblk", [1, 3, 257, 5000])
def test_dequant_bit_exact_seeded(sch, nblk):
    s = O.SCHEMES[sch]
    w = O.fill_blocks(s, 200 + nblk, nblk)
    be = O.GEOMETRY[s][0]
    got = _gpu_dequant(s, w, nblk * be)
    exp = O.dequant(s, w, nblk * be)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


@pytest.mark.parametrize("sch", NEW)
def test_dequant_arbitrary_bytes_and_special_scales(sch):
    """Every byte random (all scale / mask / quant patterns), plus subnormal, zero, negative and huge d."""
    s = O.SCHEMES[sch]
    _, bb = O.GEOMETRY[s]
    rng = np.random.default_rng(17)
    w = rng.integers(0, 256, 96 * bb, dtype=np.uint8).reshape(96, bb)
    specials16 = [0x0001, 0x03FF, 0x0000, 0x8000, 0xBC00, 0x7BFF, 0x8001, 0x3C00]
    specials32 = [0x00000001, 0x007FFFFF, 0x00000000, 0x80000000, 0xBF800000, 0x7F7FFFFF, 0x3F800000, 0x80000001]
    for i in range(64, 96):
        if s == O.Q8_K:
            w[i, 0:4] = np.frombuffer(np.uint32(specials32[i % 8]).tobytes(), np.uint8)
        else:
            v = specials16[i % 8]
            w[i, 0], w[i, 1] = v & 0xFF, v >> 8
    # random d bytes can be NaN / Inf: compare bit patterns, NaN payloads included
    w = w.ravel()
    be = O.GEOMETRY[s][0]
    got = _gpu_dequant(s, w, 96 * be)
    exp = O.dequant(s, w, 96 * be)
    same = got.view(np.uint32) == exp.view(np.uint32)
    both_nan = np.isnan(got) & np.isnan(exp)
    assert np.all(same | both_nan)


def test_reference_known_answers_on_the_gpu():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = [c for c in json.load(f) if c["scheme"] in NEW]
    assert len(cases) >= 5          # the reference holds none for Q4_1 / Q5_0 / Q5_1 (cross-checked decoders only)
    for case in cases:
        s = O.SCHEMES[case["scheme"]]
        w = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8).copy()
        if case.get("finite_only"):
            assert np.isfinite(_gpu_dequant(s, w, case["n_elems"])).all(), case["name"]
        if "expected" in case:
            got = _gpu_dequant(s, w, case["n_elems"])
            assert np.max(np.abs(got - np.array(case["expected"], np.float32))) <= case["tol"], case["name"]
        if "matmul" in case:
            mm = case["matmul"]
            x = np.array(mm["x"], np.float32).reshape(mm["m"], mm["k"])
            y = _gpu_matmul(s, w, x, mm["n"]).ravel()
            exp = np.array(mm["expected"], np.float32)
            if "rel_tol" in mm:
                assert np.all(np.abs(y - exp) / np.maximum(np.abs(exp), 1.0) < mm["rel_tol"]), case["name"]
            else:
                assert np.all(np.abs(y - exp) < mm["abs_tol"]), case["name"]


@pytest.mark.parametrize("sch", NEW)
@pytest.mark.parametrize("m,k,n,x_bf16", [(1, 256, 1, False), (1, 4096, 130, False), (2, 2048, 33, True),
                                          (8, 512, 17, False), (20, 768, 40, False), (64, 1024, 96, True)])
def test_matmul_matches_oracle(sch, m, k, n, x_bf16):
    s = O.SCHEMES[sch]
    w, x = make_case(s, m, k, n, seed=2000 + m + n, x_bf16=x_bf16)
    y = _gpu_matmul(s, w, x, n, x_bf16=x_bf16)
    tol = 2e-5
    gemm_k = {"q5_k": 256, "q2_k": 1024, "q3_k": 2048, "q8_k": 1024, "q4_1": 256, "q5_0": 256, "q5_1": 256}.get(sch)
    if gemm_k and m > 8 and k % gemm_k == 0:    # tensor-core GEMM (f32 activations as two bf16 halves): weights rounded once to bf16
        tol = min(1e-3, (24e-3 if sch in ("q2_k", "q3_k", "q4_1", "q5_1") else 12e-3) / np.sqrt(k))   # few distinct values per sub-block: rounding errors repeat
    assert_within_tolerance(y, reference(s, w, x, n), bound(s, w, x, n), tol=tol, what=f"{sch} {m}x{k}x{n}")


def test_committed_fixtures_of_the_new_formats():
    z = np.load(os.path.join(GOLDEN, "seeded_small.npz"))
    seen = 0
    for nm in sorted({k.split(".")[0] for k in z.files}):
        s, m, k, n, _ = (int(v) for v in z[f"{nm}.meta"])
        if s not in (O.Q5_K, O.Q8_K, O.Q2_K, O.Q3_K):
            continue
        seen += 1
        got = _gpu_dequant(s, z[f"{nm}.w"], k * n)
        assert np.array_equal(got.view(np.uint32), z[f"{nm}.deq"].view(np.uint32)), nm
        y = _gpu_matmul(s, z[f"{nm}.w"], z[f"{nm}.x"], n)
        assert_within_tolerance(y, z[f"{nm}.y"], bound(s, z[f"{nm}.w"], z[f"{nm}.x"], n), tol=2e-5, what=nm)
    assert seen == 4


def test_shape_and_session_errors_for_new_formats():
    import torch
    s = O.Q3_K
    wd = torch.from_numpy(O.fill_weights(s, 1, 256, 8)).cuda()
    with pytest.raises(R.RlxqError) as e:
        R.matmul(torch.zeros((1, 128), device="cuda"), wd, s, 8)      # k not a multiple of 256
    assert e.value.status == -2
    # through the Graph / Session mirror
    g = R.Graph("q5k")
    k, n, m = 512, 12, 3
    w, x = make_case(O.Q5_K, m, k, n, seed=5)
    xi = g.input("x", [m, k])
    p = g.param("w", [w.size])
    g.set_outputs([g.dequant_matmul_packed(xi, p, R.QuantScheme.GgufQ5K, n)])
    c = R.Session(R.Device.Cuda).compile(g)
    c.set_param_typed("w", w, R.DType.U8)
    y = c.run([("x", x)], (m, n))
    assert_within_tolerance(y, reference(O.Q5_K, w, x, n), bound(O.Q5_K, w, x, n), tol=2e-5, what="session q5_k")
