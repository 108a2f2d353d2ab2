"""GPU parity of rlxq_matmul (through the C ABI) against the CPU oracle.

Tolerance (stated by the path's specification): |y - y_ref| <= 1e-3 * ||x_row|| * ||w_row|| per
element with f32 accumulation.  The kernels are far inside it; the tests also pin the much
tighter bounds the two kernels are designed to: 2e-5 for the f32 generic kernel and 3e-4 for the
staged GEMV (whose only extra rounding is x -> fp16, relative 2^-12).
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


@pytest.fixture(autouse=True)
def _reset_options():
    yield
    R.set_option("gemv_kernel", 0)
    R.set_option("gemm_kernel", 0)
    R.set_option("gemv_kslices", 0)
    R.set_option("gemv_inline_q", 0)


def _run(scheme, w, x, n, x_bf16=False, y_bf16=False):
    import torch
    wd = torch.from_numpy(w).cuda()
    xd = torch.from_numpy(x).cuda()
    if x_bf16:
        xd = xd.to(torch.bfloat16)
    y = R.matmul(xd, wd, scheme, n, out_dtype=torch.bfloat16 if y_bf16 else torch.float32)
    R.device_status()
    return y.float().cpu().numpy()


GENERIC_SHAPES = [("q8_0", 1, 32, 1), ("q8_0", 3, 96, 7), ("q4_0", 1, 32, 5), ("q4_0", 8, 512, 17),
                  ("q4_k", 1, 256, 1), ("q4_k", 5, 256, 33), ("q6_k", 2, 512, 9), ("q6_k", 1, 256, 3),
                  ("q4_0", 20, 160, 11), ("q8_0", 9, 64, 4)]


@pytest.mark.parametrize("sch,m,k,n", GENERIC_SHAPES)
def test_generic_kernel_matches_oracle(sch, m, k, n):
    s = O.SCHEMES[sch]
    R.set_option("gemv_kernel", 1)
    w, x = make_case(s, m, k, n, seed=50 + m + n)
    y = _run(s, w, x, n)
    ref = reference(s, w, x, n, serial=True)
    assert_within_tolerance(y, ref, bound(s, w, x, n), tol=2e-5, what=f"generic {sch} {m}x{k}x{n}")


def _kernels_for(s, m, k):
    """Kernel selectors that accept this shape: 1 generic, 2 staged tensor mode, 3 staged integer, 0 auto."""
    unit = 2048 if s == O.Q6_K else 256
    ks = [1, 0]
    if s in (O.Q4_0, O.Q8_0, O.Q4_K, O.Q6_K) and k % unit == 0 and m <= 8:
        ks.append(2)
        if m <= 4:
            ks.append(3)
    if s == O.Q5_K and k % 256 == 0 and m <= 4:      # integer kernel only
        ks.append(3)
    return ks


def test_committed_fixtures_all_kernels():
    z = np.load(os.path.join(GOLDEN, "seeded_small.npz"))
    for nm in sorted({k.split(".")[0] for k in z.files}):
        s, m, k, n, _ = (int(v) for v in z[f"{nm}.meta"])
        w, x, ref = z[f"{nm}.w"], z[f"{nm}.x"], z[f"{nm}.y"]
        for kern in _kernels_for(s, m, k):
            R.set_option("gemv_kernel", kern)
            y = _run(s, w, x, n)
            assert_within_tolerance(y, ref, bound(s, w, x, n), tol=3e-4, what=f"{nm} kernel={kern}")


def test_reference_known_answer_matmuls():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = [c for c in json.load(f) if "matmul" in c]
    assert len(cases) == 4
    for case in cases:
        s = O.SCHEMES[case["scheme"]]
        mm = case["matmul"]
        w = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8).copy()
        x = (np.ones((mm["m"], mm["k"]), np.float32) if mm["x"] == "ones"
             else np.array(mm["x"], np.float32).reshape(mm["m"], mm["k"]))
        for kern in _kernels_for(s, mm["m"], mm["k"]):
            R.set_option("gemv_kernel", kern)
            y = _run(s, w, x, mm["n"]).ravel()
            exp = np.array(mm["expected"], np.float32)
            if "rel_tol" in mm:
                assert np.all(np.abs(y - exp) / np.maximum(np.abs(exp), 1.0) < mm["rel_tol"]), case["name"]
            else:
                assert np.all(np.abs(y - exp) < mm["abs_tol"]), case["name"]


def test_layout_regression_shape_distinct_rows():
    """The n=4, m=2, k=256 shape of rlx-runtime/tests/dequant_matmul_gguf.rs:176-241: rows of W
    differ, so an [n,k] / [k,n] mix-up (the reference's CUDA path has one) cannot pass."""
    for sch in ("q8_0", "q4_k"):
        s = O.SCHEMES[sch]
        w = O.fill_weights(s, 77, 256, 4)
        x = (0.01 * (np.arange(512, dtype=np.float32) + 1.0)).reshape(2, 256)
        ref = reference(s, w, x, 4, serial=True)
        bnd = bound(s, w, x, 4)
        for kern in (1, 2, 3, 0):
            R.set_option("gemv_kernel", kern)
            y = _run(s, w, x, 4)
            rel = np.abs(y - ref) / np.maximum(np.abs(ref), 1.0)
            # 1e-4 is the reference's own bar for its f32 backends; the f32 generic kernel and the
            # integer kernel meet it.  The tensor-mode kernel rounds x to fp16 (2^-12), which this
            # all-positive ramp turns into 1e-3 relative; it is held to the path's bound instead.
            if kern == 1:
                assert rel.max() < 1e-4, (sch, kern, rel.max())
            else:
                assert_within_tolerance(y, ref, bnd, tol=3e-4, what=f"layout {sch} kernel {kern}")
                assert rel.max() < 5e-3


STAGED_SHAPES = [
    ("q4_0", 1, 256, 16), ("q4_0", 1, 256, 24), ("q4_0", 2, 1024, 17), ("q4_0", 8, 2304, 50), ("q4_0", 5, 4096, 130),
    ("q8_0", 1, 256, 16), ("q8_0", 3, 768, 33), ("q8_0", 8, 1280, 64), ("q8_0", 1, 4096, 100),
    ("q4_k", 1, 256, 1), ("q4_k", 1, 512, 19), ("q4_k", 4, 1280, 40), ("q4_k", 8, 2048, 48), ("q4_k", 7, 4096, 31),
    ("q6_k", 1, 2048, 9), ("q6_k", 2, 2048, 16), ("q6_k", 8, 4096, 37), ("q6_k", 3, 6144, 20),
]


@pytest.mark.parametrize("sch,m,k,n", STAGED_SHAPES)
@pytest.mark.parametrize("x_bf16", [False, True])
def test_staged_gemv_matches_oracle(sch, m, k, n, x_bf16):
    s = O.SCHEMES[sch]
    R.set_option("gemv_kernel", 2)
    w, x = make_case(s, m, k, n, seed=300 + m + n, x_bf16=x_bf16)
    y = _run(s, w, x, n, x_bf16=x_bf16)
    ref = reference(s, w, x, n)
    assert_within_tolerance(y, ref, bound(s, w, x, n), tol=3e-4, what=f"staged {sch} {m}x{k}x{n}")


INT_SHAPES = [
    ("q4_0", 1, 256, 16), ("q4_0", 1, 1024, 17), ("q4_0", 2, 2304, 50), ("q4_0", 1, 4096, 130), ("q4_0", 2, 11008, 33),
    ("q8_0", 1, 256, 16), ("q8_0", 2, 768, 33), ("q8_0", 1, 4096, 100),
    ("q4_k", 1, 256, 1), ("q4_k", 1, 512, 19), ("q4_k", 2, 1280, 40), ("q4_k", 1, 4096, 31),
    ("q6_k", 1, 2048, 9), ("q6_k", 2, 2048, 16), ("q6_k", 1, 6144, 37),
    ("q5_k", 1, 256, 1), ("q5_k", 1, 768, 19), ("q5_k", 2, 1280, 40), ("q5_k", 1, 4096, 131), ("q5_k", 4, 2048, 50),
    # three and four rows: the four-row kernel (one CTA per SM, activations of a block in registers for Q4_0)
    ("q4_0", 4, 4096, 130), ("q4_0", 3, 2304, 50), ("q4_0", 4, 11008, 33), ("q8_0", 4, 1024, 77), ("q8_0", 3, 4096, 40),
    ("q4_k", 4, 4096, 31), ("q4_k", 3, 1280, 100), ("q6_k", 4, 2048, 16), ("q6_k", 3, 6144, 37),
]


@pytest.mark.parametrize("sch,m,k,n", INT_SHAPES)
@pytest.mark.parametrize("x_bf16", [False, True])
def test_integer_gemv_matches_oracle(sch, m, k, n, x_bf16):
    s = O.SCHEMES[sch]
    R.set_option("gemv_kernel", 3)
    w, x = make_case(s, m, k, n, seed=500 + m + n, x_bf16=x_bf16)
    y = _run(s, w, x, n, x_bf16=x_bf16)
    ref = reference(s, w, x, n)
    # 15-bit activations: worst case 1.7e-4, typically 1e-6; 2e-5 leaves room for f32 accumulation
    assert_within_tolerance(y, ref, bound(s, w, x, n), tol=2e-5, what=f"integer {sch} {m}x{k}x{n}")


@pytest.mark.parametrize("sch,m,k,n", [("q4_0", 1, 4096, 2000), ("q4_0", 2, 2304, 5000), ("q8_0", 1, 1024, 4100),
                                       ("q4_k", 2, 4096, 3000), ("q6_k", 1, 2048, 4500), ("q4_0", 1, 11008, 700)])
@pytest.mark.parametrize("fill", [0x00, 0xFF, 0x5A])
def test_integer_gemv_one_and_two_kernel_modes_agree_on_any_workspace(sch, m, k, n, fill):
    """The integer GEMV runs as one kernel (activations quantised by the streaming kernel, shared tiles
    completed through a token exchange) or as two (a quantiser kernel in front).  Both quantise the same
    way, so they must agree to the last bit whatever the workspace held, call after call."""
    import torch
    s = O.SCHEMES[sch]
    R.set_option("gemv_kernel", 3)
    w, x = make_case(s, m, k, n, seed=1300 + m + n)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    ws = torch.full((R.workspace_bytes(s, m, k, n) + 16,), fill, dtype=torch.uint8, device="cuda")
    outs = []
    for mode in (1, 2, 2, 1, 2):
        R.set_option("gemv_inline_q", mode)
        outs.append(R.matmul(xd, wd, s, n, workspace=ws).cpu().numpy())
        R.device_status()
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    assert_within_tolerance(outs[0], reference(s, w, x, n), bound(s, w, x, n), tol=2e-5, what=f"integer {sch} modes")


def test_integer_gemv_single_kernel_mode_replays_in_a_cuda_graph():
    """A captured launch carries the same token on every replay; the kernel leaves the rendezvous words clean."""
    import torch
    s, m, k, n = O.Q4_0, 1, 4096, 5000
    R.set_option("gemv_kernel", 3)
    R.set_option("gemv_inline_q", 2)
    w, x = make_case(s, m, k, n, seed=77)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    ws = torch.full((R.workspace_bytes(s, m, k, n) + 16,), 0xC3, dtype=torch.uint8, device="cuda")
    y = torch.empty((m, n), device="cuda")
    R.matmul(xd, wd, s, n, out=y, workspace=ws)
    torch.cuda.synchronize()
    want = y.cpu().numpy().copy()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(3):
            R.matmul(xd, wd, s, n, out=y, workspace=ws)
    for _ in range(4):
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(y.cpu().numpy(), want)
    R.device_status()


@pytest.mark.parametrize("sch,k", [("q4_0", 2048), ("q8_0", 1536), ("q4_k", 2560), ("q6_k", 8192)])
@pytest.mark.parametrize("ksl", [1, 2, 3])
@pytest.mark.parametrize("kern,m", [(2, 3), (3, 2)])
def test_staged_gemv_split_k_is_deterministic_and_correct(sch, k, ksl, kern, m):
    s = O.SCHEMES[sch]
    R.set_option("gemv_kernel", kern)
    R.set_option("gemv_kslices", ksl)
    n = 77
    w, x = make_case(s, m, k, n, seed=900 + ksl)
    y1 = _run(s, w, x, n)
    y2 = _run(s, w, x, n)
    assert np.array_equal(y1, y2)   # fixed reduction order
    assert_within_tolerance(y1, reference(s, w, x, n), bound(s, w, x, n), tol=3e-4, what=f"{sch} ksl={ksl}")


def test_bf16_output_is_rne_of_f32_output():
    import torch
    s = O.Q4_0
    w, x = make_case(s, 4, 1024, 64, seed=5)
    yf = _run(s, w, x, 64)
    yb = _run(s, w, x, 64, y_bf16=True)
    exp = torch.from_numpy(yf).to(torch.bfloat16).float().numpy()
    assert np.array_equal(yb, exp)


def test_activation_range_is_rescaled():
    """Rows far outside fp16's range (1e-30 .. 1e30) must come out as accurately as O(1) rows."""
    s = O.Q8_0
    w, x = make_case(s, 4, 1024, 48, seed=6)
    x = (x * np.array([[1e-30], [1.0], [1e20], [3e4]], np.float32)).astype(np.float32)
    R.set_option("gemv_kernel", 2)
    y = _run(s, w, x, 48)
    assert_within_tolerance(y, reference(s, w, x, 48), bound(s, w, x, 48), tol=3e-4, what="range")
    # the integer kernel scales per 32-value block, so it does not care about the row's range either
    R.set_option("gemv_kernel", 3)
    for rows in ((0, 2), (2, 4)):
        xs = np.ascontiguousarray(x[rows[0]:rows[1]])
        y = _run(s, w, xs, 48)
        assert_within_tolerance(y, reference(s, w, xs, 48), bound(s, w, xs, 48), tol=2e-5, what="range int")


def test_one_hot_activation_reproduces_the_weight_column():
    """Size-independent property: x = e_p gives y[j] = W[j,p], checked against the bit-exact
    decoder at a full benchmark size (Q4_0 11008 -> 4096)."""
    import torch
    s, k, n = O.Q4_0, 11008, 4096
    w = O.fill_weights(s, 31, k, n)
    wd = torch.from_numpy(w).cuda()
    deq = R.dequant_f32(wd, s, k * n).view(n, k)
    for p in (0, 17, 5000, 11007):
        x = torch.zeros((1, k), dtype=torch.float32, device="cuda")
        x[0, p] = 1.0
        R.set_option("gemv_kernel", 2)       # tensor mode: exact (power-of-two rescale, one rounding)
        y = R.matmul(x, wd, s, n)
        assert torch.equal(y[0], deq[:, p]), p
        R.set_option("gemv_kernel", 0)       # integer mode: d * s_b and the product round separately
        y = R.matmul(x, wd, s, n)
        assert torch.all((y[0] - deq[:, p]).abs() <= 4e-7 * deq[:, p].abs()), p


def test_zero_activation_gives_zero():
    import torch
    for s, k in ((O.Q4_K, 4096), (O.Q6_K, 4096)):
        wd = torch.from_numpy(O.fill_weights(s, 3, k, 256)).cuda()
        y = R.matmul(torch.zeros((2, k), device="cuda"), wd, s, 256)
        assert torch.count_nonzero(y).item() == 0


FULL = [("q8_0", 1, 4096, 4096, False), ("q4_0", 1, 4096, 11008, False), ("q4_0", 4, 4096, 11008, False),
        ("q4_0", 8, 4096, 11008, False), ("q4_0", 1, 11008, 4096, False), ("q4_0", 4, 11008, 4096, False),
        ("q4_0", 8, 11008, 4096, False), ("q4_k", 1, 4096, 14336, True), ("q6_k", 1, 14336, 4096, True)]


@pytest.mark.parametrize("sch,m,k,n,x_bf16", FULL)
def test_benchmark_configurations_full_size(sch, m, k, n, x_bf16):
    """Configurations 0, 1 and the decode half of 2 at their real sizes, every output checked."""
    s = O.SCHEMES[sch]
    w, x = make_case(s, m, k, n, seed=1, x_bf16=x_bf16)
    y = _run(s, w, x, n, x_bf16=x_bf16)
    worst = assert_within_tolerance(y, reference(s, w, x, n), bound(s, w, x, n), what=f"cfg {sch} m={m}")
    assert worst < 3e-4


def test_matmul_edge_cases():
    import torch
    s = O.Q4_0
    wd = torch.from_numpy(O.fill_weights(s, 1, 64, 8)).cuda()
    # m = 0 and n = 0 are empty outputs, not errors
    assert R.matmul(torch.zeros((0, 64), device="cuda"), wd, s, 8).shape == (0, 8)
    # k not a multiple of the block
    with pytest.raises(R.RlxqError) as e:
        R.matmul(torch.zeros((1, 48), device="cuda"), wd, s, 8)
    assert e.value.status == -2
    # forcing the staged kernel on a shape it cannot take is an error, not a silent fallback
    R.set_option("gemv_kernel", 2)
    with pytest.raises(R.RlxqError):
        R.matmul(torch.zeros((1, 64), device="cuda"), wd, s, 8)


def test_launch_counter_counts_kernels():
    import torch
    s = O.Q8_0
    wd = torch.from_numpy(O.fill_weights(s, 1, 256, 16)).cuda()
    x = torch.zeros((1, 256), device="cuda")
    R.set_option("gemv_kernel", 1)
    before = R.launch_count()
    R.matmul(x, wd, s, 16)
    assert R.launch_count() == before + 1      # generic kernel: one launch
    R.set_option("gemv_kernel", 3)
    R.set_option("gemv_inline_q", 1)
    before = R.launch_count()
    R.matmul(x, wd, s, 16)
    assert R.launch_count() == before + 2      # integer GEMV: activation quantiser + streaming kernel
    R.set_option("gemv_inline_q", 2)
    before = R.launch_count()
    R.matmul(x, wd, s, 16)
    assert R.launch_count() == before + 1      # integer GEMV, single-kernel mode


# ------------------------------------------------------------------ the tcgen05 GEMV (opt-in, gemv_kernel = 4)
TC_GEMV_SHAPES = [("q8_0", 1, 256, 128, False, False), ("q8_0", 1, 256, 100, False, False), ("q4_0", 2, 1024, 300, False, False),
                  ("q4_k", 3, 2048, 1000, False, False), ("q4_0", 1, 4096, 11008, False, False),
                  ("q4_0", 8, 11008, 4096, False, False), ("q8_0", 5, 4096, 4096, True, False),
                  ("q4_k", 1, 4096, 14336, True, False), ("q4_k", 7, 8192, 3000, False, True),
                  ("q4_0", 4, 4096, 11008, True, True)]


@pytest.mark.parametrize("ctas", [2, 1])
@pytest.mark.parametrize("sch,m,k,n,x_bf16,y_bf16", TC_GEMV_SHAPES)
def test_tensor_core_gemv_matches_oracle(sch, m, k, n, x_bf16, y_bf16, ctas):
    """The tcgen05 decode GEMV: weights as fp16(d * q) in tensor memory (one rounding of 2^-12 per weight),
    activations as two fp16 limbs.  Held to min(1e-3, 4e-3 / sqrt(k)) of ||x|| ||w_row|| (1e-3 with a bf16
    output); both CTA counts per SM, so short ranges (direct activation loads) and long ones (staging ring)
    and tiles cut between two and many contributors are all exercised, twice in a row on the same scratch."""
    import torch
    s = O.SCHEMES[sch]
    w, x = make_case(s, m, k, n, seed=900 + n + m, x_bf16=x_bf16)
    R.set_option("gemv_kernel", 4)
    R.set_option("gemv_tc_ctas", ctas)
    try:
        wd = torch.from_numpy(w).cuda()
        xd = torch.from_numpy(x).cuda()
        if x_bf16:
            xd = xd.to(torch.bfloat16)
        ws = torch.empty(R.workspace_bytes(s, m, k, n, 1 if x_bf16 else 0, 1 if y_bf16 else 0) + 16, dtype=torch.uint8, device="cuda")
        outs = []
        for _ in range(2):
            before = R.launch_count()
            y = R.matmul(xd, wd, s, n, out_dtype=torch.bfloat16 if y_bf16 else torch.float32, workspace=ws)
            assert R.launch_count() - before == 1                 # one kernel, no prepass
            outs.append(y.float().cpu().numpy())
        R.device_status()
    finally:
        R.set_option("gemv_tc_ctas", 2)
    assert np.array_equal(outs[0], outs[1])                       # same bits from run to run
    ref = reference(s, w, x, n)
    tol = 1e-3 if y_bf16 else min(1e-3, 4e-3 / np.sqrt(k))       # a bf16 output carries its own rounding of |y| * 2^-9
    assert_within_tolerance(outs[0], ref, bound(s, w, x, n), tol=tol, what=f"tcgen05 gemv {sch} m={m} k={k} n={n}")


def test_tensor_core_gemv_refuses_what_it_cannot_run():
    import torch
    R.set_option("gemv_kernel", 4)
    s = O.Q6_K                                                   # no decoder for this format in this kernel
    w, x = make_case(s, 1, 2048, 16, seed=3)
    with pytest.raises(R.RlxqError) as e:
        R.matmul(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), s, 16)
    assert e.value.status == -2


# ------------------------------------------------------------------ the integer-MMA units (batch 3-8 by default)
IMMA_SHAPES = [("q4_0", 3, 256, 100, False, False), ("q4_0", 4, 4096, 11008, False, False), ("q4_0", 4, 11008, 4096, False, False),
               ("q4_0", 8, 4096, 11008, False, False), ("q4_0", 7, 8192, 4096, True, False), ("q4_0", 1, 2048, 1000, False, False),
               ("q8_0", 3, 256, 100, False, False), ("q8_0", 8, 4096, 4096, False, False), ("q8_0", 5, 4096, 4096, True, True),
               ("q4_k", 3, 256, 100, False, False), ("q4_k", 4, 4096, 14336, False, False), ("q4_k", 8, 2048, 1000, False, False),
               ("q4_k", 3, 14336, 4096, False, False), ("q4_k", 6, 8192, 3000, True, False), ("q4_k", 2, 1024, 300, False, True),
               ("q6_k", 3, 2048, 100, False, False), ("q6_k", 4, 14336, 4096, False, False), ("q6_k", 8, 4096, 3000, False, False),
               ("q6_k", 5, 6144, 256, True, True), ("q6_k", 2, 4096, 14336, False, False),
               ("q5_k", 3, 256, 100, False, False), ("q5_k", 4, 4096, 14336, False, False), ("q5_k", 8, 2048, 1000, True, False),
               ("q5_k", 2, 14336, 520, False, True), ("q5_k", 6, 28672, 300, False, False),
               ("q8_k", 1, 1024, 100, False, False), ("q8_k", 4, 4096, 4096, False, False), ("q8_k", 8, 2048, 1000, True, False),
               ("q8_k", 6, 28672, 300, False, True),
               ("q2_k", 1, 1024, 100, False, False), ("q2_k", 3, 4096, 4096, False, False), ("q2_k", 8, 2048, 1000, True, False),
               ("q2_k", 5, 28672, 300, False, False), ("q2_k", 2, 5120, 777, False, True),
               ("q3_k", 1, 2048, 100, False, False), ("q3_k", 4, 4096, 4096, False, False), ("q3_k", 8, 2048, 1000, True, False),
               ("q3_k", 7, 28672, 300, False, False), ("q3_k", 2, 6144, 777, False, True),
               ("q4_1", 1, 256, 100, False, False), ("q4_1", 4, 4096, 1000, False, False), ("q4_1", 8, 2048, 300, True, False),
               ("q5_0", 1, 512, 100, False, False), ("q5_0", 3, 4096, 1000, False, False), ("q5_0", 8, 11008, 256, False, True),
               ("q5_1", 2, 256, 100, False, False), ("q5_1", 5, 4096, 777, False, False), ("q5_1", 8, 14336, 300, True, False),
               # fragments of all rows do not fit in shared memory: they stream through the ring beside the weights
               ("q4_0", 8, 11008, 4096, False, False), ("q6_k", 8, 8192, 1000, False, False), ("q4_k", 4, 28672, 2048, False, False),
               ("q8_0", 8, 14336, 777, True, True), ("q4_k", 7, 28672, 520, True, False)]


@pytest.mark.parametrize("inline_q", [0, 1])
@pytest.mark.parametrize("sch,m,k,n,x_bf16,y_bf16", IMMA_SHAPES)
def test_integer_mma_gemv_matches_oracle(sch, m, k, n, x_bf16, y_bf16, inline_q):
    """The integer GEMV with its MMA units (gemv_kernel = 5): same integer products as the dp4a units, so the
    same bound.  Both ways to quantise the activations (inside the streaming kernel where the shape allows it,
    and as a kernel of its own), ragged n, whole and cut tiles, twice in a row on the same scratch."""
    import torch
    s = O.SCHEMES[sch]
    w, x = make_case(s, m, k, n, seed=700 + n + m, x_bf16=x_bf16)
    R.set_option("gemv_kernel", 5)
    R.set_option("gemv_inline_q", inline_q)
    try:
        wd = torch.from_numpy(w).cuda()
        xd = torch.from_numpy(x).cuda()
        if x_bf16:
            xd = xd.to(torch.bfloat16)
        ws = torch.empty(R.workspace_bytes(s, m, k, n, 1 if x_bf16 else 0, 1 if y_bf16 else 0) + 16, dtype=torch.uint8, device="cuda")
        outs = []
        for _ in range(2):
            y = R.matmul(xd, wd, s, n, out_dtype=torch.bfloat16 if y_bf16 else torch.float32, workspace=ws)
            outs.append(y.float().cpu().numpy())
        R.device_status()
    finally:
        R.set_option("gemv_inline_q", 0)
        R.set_option("gemv_kernel", 0)
    assert np.array_equal(outs[0], outs[1])                       # same bits from run to run
    ref = reference(s, w, x, n)
    assert_within_tolerance(outs[0], ref, bound(s, w, x, n), tol=1e-3 if y_bf16 else 2e-4,
                            what=f"integer-MMA gemv {sch} m={m} k={k} n={n}")


def test_integer_mma_gemv_is_the_default_for_batch_3_to_8():
    """Automatic dispatch and the forced kernel give the same bits for a batch the MMA units take by default."""
    import torch
    s = O.Q4_0
    w, x = make_case(s, 4, 4096, 512, seed=41)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    y_auto = R.matmul(xd, wd, s, 512).cpu().numpy()
    R.set_option("gemv_kernel", 5)
    try:
        y_forced = R.matmul(xd, wd, s, 512).cpu().numpy()
    finally:
        R.set_option("gemv_kernel", 0)
    R.device_status()
    assert np.array_equal(y_auto, y_forced)


def test_integer_mma_gemv_refuses_what_it_cannot_run():
    import torch
    R.set_option("gemv_kernel", 5)
    try:
        s = O.Q2_K                                               # rows of 84-byte super-blocks: k a multiple of 1024
        w, x = make_case(s, 4, 768, 16, seed=3)
        with pytest.raises(R.RlxqError) as e:
            R.matmul(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), s, 16)
        assert e.value.status == -2
        s = O.Q4_0                                               # k must be a multiple of 256
        w, x = make_case(s, 4, 288, 16, seed=4)
        with pytest.raises(R.RlxqError) as e:
            R.matmul(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), s, 16)
        assert e.value.status == -2
    finally:
        R.set_option("gemv_kernel", 0)


# ------------------------------------------------------------------ rlxq_matmul_chain
def _chain_reference(s, x, ws, spec):
    cur = x.astype(np.float32)
    for w, (k, n, sw) in zip(ws, spec):
        if sw:
            g, u = cur[:, :k].astype(np.float64), cur[:, k:].astype(np.float64)
            cur = (u * (g / (1.0 + np.exp(-g)))).astype(np.float32)
        cur = O.matmul_bt_mt(np.ascontiguousarray(cur), w, cur.shape[0], k, n, s).astype(np.float32)
    return cur


CHAIN_CASES = [("q4_0", 1, [(256, 512, 0), (512, 256, 0)]), ("q4_0", 1, [(4096, 11008, 0), (11008, 4096, 0)]),
               ("q4_0", 2, [(4096, 11008, 0), (11008, 4096, 0)]), ("q4_k", 1, [(4096, 2 * 7168, 0), (7168, 8192, 1)]),
               ("q6_k", 1, [(2048, 8192, 0), (8192, 6144, 0), (6144, 4800, 0)]), ("q8_0", 2, [(1024, 2 * 4096, 0), (4096, 5000, 1)]),
               ("q4_k", 4, [(2048, 2 * 1024, 0), (1024, 512, 1)]), ("q5_k", 1, [(512, 300, 0)])]


@pytest.mark.parametrize("fused", [0, 1])
@pytest.mark.parametrize("sch,m,spec", CHAIN_CASES)
def test_matmul_chain_matches_the_layers_run_on_the_oracle(sch, m, spec, fused):
    """rlxq_matmul_chain layer by layer (the default) and as one cooperative kernel (option gemv_chain = 1, where
    the shapes allow it; the call falls back by itself elsewhere): plain layers, SwiGLU layers, two and three
    layers, twice in a row on the same workspace."""
    import torch
    s = O.SCHEMES[sch]
    ws = [O.fill_weights(s, 300 + 7 * i + m, k, n) for i, (k, n, sw) in enumerate(spec)]
    x = O.fill_normal(301 + m, m * spec[0][0]).reshape(m, -1)
    wd = [torch.from_numpy(w).cuda() for w in ws]
    xd = torch.from_numpy(x).cuda()
    layers = [(w, n, sw) for w, (k, n, sw) in zip(wd, spec)]
    need = R.chain_workspace_bytes(s, spec, m)
    wsb = torch.full((need + 256,), 0xA5, dtype=torch.uint8, device="cuda")      # contents irrelevant on entry
    R.set_option("gemv_chain", fused)
    try:
        before = R.launch_count()
        y1 = R.matmul_chain(xd, layers, s, workspace=wsb).cpu().numpy()
        launches = R.launch_count() - before
        y2 = R.matmul_chain(xd, layers, s, workspace=wsb).cpu().numpy()
        R.device_status()
    finally:
        R.set_option("gemv_chain", 0)
    assert np.array_equal(y1, y2)
    if fused and sch == "q4_0" and m <= 2:
        assert launches == 1                                   # one kernel for the whole chain
    ref = _chain_reference(s, x, ws, spec)
    assert np.isfinite(y1).all()
    assert np.abs(y1 - ref).max() <= 1e-3 * (np.abs(ref).max() + 1e-30)


def test_matmul_chain_rejects_layers_that_do_not_fit_together():
    s = O.Q4_0
    with pytest.raises(R.RlxqError) as e:
        R.chain_workspace_bytes(s, [(256, 64, 0), (256, 32, 0)], 1)      # layer 1 takes 256 values, layer 0 yields 64
    assert e.value.status == -2
    with pytest.raises(R.RlxqError) as e:
        R.chain_workspace_bytes(s, [(256, 64, 1)], 1)                    # the first layer has nothing to combine
    assert e.value.status == -2
    with pytest.raises(R.RlxqError) as e:
        R.chain_workspace_bytes(s, [(256, 64, 0), (32, 16, 0)], 1)       # SwiGLU flag missing: 64 != 32
    assert e.value.status == -2
    assert R.chain_workspace_bytes(s, [(256, 64, 0), (32, 16, 1)], 1) > 0


# ------------------------------------------------------------------ seeded random shapes through the automatic dispatch
def _random_gemv_cases(count=110, seed=20240611):
    rng = np.random.default_rng(seed)
    cases = []
    while len(cases) < count:
        sch = ["q4_0", "q8_0", "q4_k", "q5_k", "q6_k", "q8_k", "q2_k", "q3_k", "q4_1", "q5_0", "q5_1"][int(rng.integers(0, 11))]
        unit = {"q6_k": 2048, "q3_k": 2048, "q8_k": 1024, "q2_k": 1024}.get(sch, 256)
        k = unit * int(rng.integers(1, 32768 // unit + 1))
        m = int(rng.integers(1, 9))
        nmax = max(1, min(6000, 24_000_000 // k))
        n = int(rng.integers(1, nmax + 1))
        cases.append((sch, m, k, n, bool(rng.integers(0, 2)), bool(rng.integers(0, 4) == 0), int(rng.integers(0, 2))))
    return cases


@pytest.mark.parametrize("sch,m,k,n,x_bf16,y_bf16,two_kernel", _random_gemv_cases())
def test_decode_gemv_random_shapes(sch, m, k, n, x_bf16, y_bf16, two_kernel):
    """Whatever the plan makes of a shape (ring depth, CTAs per SM, tiles cut once or many times, activations
    resident or streamed, quantised in the kernel or in front of it), the result is the oracle's."""
    import torch
    s = O.SCHEMES[sch]
    w, x = make_case(s, m, k, n, seed=31 * k + n + m, x_bf16=x_bf16)
    R.set_option("gemv_inline_q", 1 if two_kernel else 0)
    try:
        wd = torch.from_numpy(w).cuda()
        xd = torch.from_numpy(x).cuda()
        if x_bf16:
            xd = xd.to(torch.bfloat16)
        y = R.matmul(xd, wd, s, n, out_dtype=torch.bfloat16 if y_bf16 else torch.float32).float().cpu().numpy()
        R.device_status()
    finally:
        R.set_option("gemv_inline_q", 0)
    assert_within_tolerance(y, reference(s, w, x, n), bound(s, w, x, n), tol=1e-3 if y_bf16 else 2e-4,
                            what=f"random {sch} m={m} k={k} n={n}")
