"""Op::DequantGroupedMatMul (MoE expert stacks): y[i] = x[i] . W_{expert_idx[i]}^T.

CPU part: the oracle against the reference's graph test (restated in tests/golden/grouped_matmul_case.json).
GPU part: rlxq_grouped_matmul through the C ABI against the oracle, every scheme, ragged routings.
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _case():
    with open(os.path.join(GOLDEN, "grouped_matmul_case.json")) as f:
        c = json.load(f)
    w = np.frombuffer(bytes.fromhex(c["bytes"]), np.uint8).copy()
    x = np.array(c["x"], np.float32).reshape(c["m"], c["k"])
    idx = np.array(c["expert_idx"], np.float32)
    return c, w, x, idx


def _close(y, c):
    exp = np.array(c["expected"], np.float32)
    return np.all(np.abs(y.ravel() - exp) / np.maximum(np.abs(exp), 1.0) < c["rel_tol"])


def test_oracle_reproduces_the_reference_grouped_test():
    c, w, x, idx = _case()
    y = O.grouped_matmul_bt(x, w, idx, c["m"], c["k"], c["n"], c["num_experts"], O.SCHEMES[c["scheme"]])
    assert _close(y, c)
    # routing to the wrong expert would be off by the ratio of the scales
    wrong = O.grouped_matmul_bt(x, w, np.roll(idx, 1), c["m"], c["k"], c["n"], c["num_experts"], O.SCHEMES[c["scheme"]])
    assert not _close(wrong, c)


def test_oracle_reads_expert_ids_as_the_reference_cast_does():
    """`expert_idx[i] as usize` (rlx-cpu/src/gguf_matmul.rs:187,198) saturates: NaN, negatives and fractions
    below 1 select expert 0, 2.7 selects 2; ids of num_experts and above stay zero rows here."""
    s, m, k, n, E = O.Q4_0, 6, 256, 5, 3
    w = O.fill_weights(s, 13, k, n * E)
    x = O.fill_normal(14, m * k).reshape(m, k)
    idx = np.array([np.nan, -3.0, 0.9, 2.7, 3.0, 1e30], np.float32)
    y = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    slab = w.size // E
    for i, e in enumerate((0, 0, 0, 2)):
        assert np.array_equal(y[i], O.matmul_bt(x[i:i + 1], w[e * slab:(e + 1) * slab], 1, k, n, s).ravel())
    assert np.all(y[4:] == 0)


def test_oracle_grouped_equals_per_row_matmul():
    s, m, k, n, E = O.Q4_K, 7, 512, 9, 4
    w = O.fill_weights(s, 3, k, n * E)          # E slabs of [n, k] back to back
    x = O.fill_normal(5, m * k).reshape(m, k)
    idx = np.array([3, 0, 0, 2, 3, 3, 0], np.float32)
    y = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    slab = w.size // E
    for i in range(m):
        e = int(idx[i])
        ref = O.matmul_bt(x[i:i + 1], w[e * slab:(e + 1) * slab], 1, k, n, s)
        assert np.array_equal(y[i], ref.ravel())


# ------------------------------------------------------------------ GPU
def _gpu(x, w, idx, s, n, E, x_bf16=False, y_bf16=False):
    import torch
    import rlx_b200 as R
    xd = torch.from_numpy(x).cuda()
    if x_bf16:
        xd = xd.to(torch.bfloat16)
    y = R.grouped_matmul(xd, torch.from_numpy(w).cuda(), torch.from_numpy(idx).cuda(), s, n, E,
                         out_dtype=torch.bfloat16 if y_bf16 else torch.float32)
    R.device_status()
    return y.float().cpu().numpy()


@pytest.mark.gpu
def test_gpu_reference_grouped_test():
    c, w, x, idx = _case()
    y = _gpu(x, w, idx, O.SCHEMES[c["scheme"]], c["n"], c["num_experts"])
    assert _close(y, c)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["stream", "graph"])
def test_gpu_reference_grouped_test_through_the_graph_api(mode):
    """The reference's test as it is written there: Graph -> Session -> set_param_typed -> run with two inputs."""
    import rlx_b200 as R
    c, w, x, idx = _case()
    g = R.Graph("dq_grouped_matmul_q8k")
    x_in = g.input("x", [c["m"], c["k"]], R.DType.F32)
    w_packed = g.param("w_packed", [w.size], R.DType.U8)
    idx_in = g.input("expert_idx", [c["m"], 1], R.DType.F32)
    y = g.dequant_grouped_matmul_packed(x_in, w_packed, idx_in, R.QuantScheme.GgufQ8K, c["n"], c["num_experts"])
    g.set_outputs([y])
    compiled = R.Session(R.Device.Cuda, exec_mode=mode).compile(g)
    compiled.set_param_typed("w_packed", w, R.DType.U8)
    for _ in range(2):
        actual = compiled.run([("x", x), ("expert_idx", idx)], (c["m"], c["n"]))
        assert _close(actual, c)
    # a param that does not hold num_experts slabs is rejected when the node is built
    bad = g.param("w_bad", [w.size - 292], R.DType.U8)
    with pytest.raises(R.RlxqError) as e:
        g.dequant_grouped_matmul_packed(x_in, bad, idx_in, R.QuantScheme.GgufQ8K, c["n"], c["num_experts"])
    assert e.value.status == -2


@pytest.mark.gpu
@pytest.mark.parametrize("sch", ["q4_0", "q8_0", "q4_k", "q6_k", "q5_k", "q8_k", "q2_k", "q3_k"])
@pytest.mark.parametrize("m,k,n,E,x_bf16", [(1, 256, 5, 1, False), (8, 512, 33, 8, False), (37, 1024, 20, 5, True),
                                            (64, 2048, 130, 16, False)])
def test_gpu_grouped_matches_oracle(sch, m, k, n, E, x_bf16):
    from tests.helpers import assert_within_tolerance
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 40 + m, k, n * E)
    x = O.fill_normal(41 + m, m * k).reshape(m, k)
    if x_bf16:
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).reshape(m, k)
    rng = np.random.default_rng(m + E)
    idx = rng.integers(0, E, m).astype(np.float32)            # ragged: some experts get no rows, some many
    y = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16)
    ref = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    slab = w.size // E
    wn = np.stack([O.row_norms(s, w[e * slab:(e + 1) * slab], k, n) for e in range(E)])    # [E, n]
    xn = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
    bnd = xn[:, None] * wn[idx.astype(np.int64)]
    # 32 rows and more of a format and shape the tensor-core GEMM takes run there (weights rounded to bf16)
    gemm_k = {"q4_0": 256, "q8_0": 256, "q4_k": 256, "q5_k": 256, "q6_k": 2048, "q2_k": 1024, "q3_k": 2048, "q8_k": 1024,
              "q4_1": 256, "q5_0": 256, "q5_1": 256}.get(sch)
    on_gemm = m >= 32 and gemm_k is not None and k % gemm_k == 0
    # (Q2_K / Q3_K: few distinct values per sub-block, so the bf16 rounding errors repeat: twice the allowance)
    tol = min(1e-3, (24e-3 if sch in ("q2_k", "q3_k", "q4_1", "q5_1") else 12e-3) / np.sqrt(k)) if on_gemm else 2e-5
    assert_within_tolerance(y, ref, bnd, tol=tol, what=f"grouped {sch} m={m} E={E}")
    if on_gemm:
        import rlx_b200 as R
        R.set_option("gemm_kernel", 1)                        # the general kernel stays available, and is tighter
        try:
            y = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16)
        finally:
            R.set_option("gemm_kernel", 0)
        assert_within_tolerance(y, ref, bnd, tol=2e-5, what=f"grouped, general kernel {sch} m={m} E={E}")


@pytest.mark.gpu
@pytest.mark.parametrize("sch,m,k,n,E,x_bf16,y_bf16", [("q4_k", 300, 1024, 200, 8, False, False), ("q4_0", 700, 512, 136, 3, True, False),
                                                       ("q8_0", 96, 256, 64, 24, False, True), ("q6_k", 260, 2048, 130, 4, False, False),
                                                       ("q5_k", 1000, 512, 128, 5, True, True)])
def test_gpu_prefill_sized_batches_take_the_tensor_core_gemm(sch, m, k, n, E, x_bf16, y_bf16):
    """Sort, tile table, gather (f32 rows as bf16 hi + lo), one grouped GEMM launch over all experts, scatter:
    five launches.  Ragged groups: experts with no rows, with a few, with several 128-row tiles; ids out of range."""
    import torch
    import rlx_b200 as R
    from tests.helpers import assert_within_tolerance
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 70 + m, k, n * E)
    x = O.fill_normal(71 + m, m * k).reshape(m, k)
    if x_bf16:
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).reshape(m, k)
    rng = np.random.default_rng(m + E)
    p = rng.random(E) ** 3
    p[rng.integers(0, E)] = 0.0                                # at least one expert without rows
    idx = rng.choice(E, size=m, p=p / p.sum()).astype(np.float32)
    idx[5], idx[17] = float(E), float(E + 3)                   # in no group: zero rows
    before = R.launch_count()
    y = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16, y_bf16=y_bf16)
    assert R.launch_count() - before == 5
    y_again = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16, y_bf16=y_bf16)
    assert np.array_equal(y, y_again)
    ref = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    assert np.all(y[5] == 0) and np.all(y[17] == 0) and np.all(ref[5] == 0)
    slab = w.size // E
    wn = np.stack([O.row_norms(s, w[e * slab:(e + 1) * slab], k, n) for e in range(E)])
    xn = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
    bnd = xn[:, None] * wn[np.minimum(idx.astype(np.int64), E - 1)]
    tol = 1e-3 if y_bf16 else min(1e-3, 12e-3 / np.sqrt(k))
    assert_within_tolerance(y, ref, bnd, tol=tol, what=f"grouped GEMM {sch} m={m} E={E}")


@pytest.mark.gpu
@pytest.mark.parametrize("sch", ["q4_0", "q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("m,k,n,E,x_bf16", [(1, 4096, 4800, 4, False), (2, 2048, 4100, 8, True), (8, 4096, 4736, 3, False),
                                            (5, 6144, 4800, 2, False)])
def test_gpu_decode_rows_take_the_streaming_gemv(sch, m, k, n, E, x_bf16):
    """Up to eight rows: one expert-indirect launch of the integer GEMV per row (k a multiple of 2048 here so
    that Q6_K qualifies too); the general grouped kernel must agree with it to the path's tolerance."""
    import rlx_b200 as R
    from tests.helpers import assert_within_tolerance
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 60 + m, k, n * E)
    x = O.fill_normal(61 + m, m * k).reshape(m, k)
    if x_bf16:
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).reshape(m, k)
    idx = np.array([(3 * i + 1) % E for i in range(m)], np.float32)
    if m >= 5:
        idx[2] = idx[0]                                    # two rows on the same expert
        idx[4] = float(E)                                  # out of range: a zero row
    before = R.launch_count()
    y = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16)
    assert R.launch_count() - before == m                  # one kernel per row, no sort kernel
    ref = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    slab = w.size // E
    wn = np.stack([O.row_norms(s, w[e * slab:(e + 1) * slab], k, n) for e in range(E)])
    xn = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
    bnd = xn[:, None] * wn[np.minimum(idx, E - 1).astype(np.int64)]
    assert_within_tolerance(y, ref, bnd, tol=2e-5, what=f"moe decode {sch} m={m}")
    if m >= 5:
        assert np.all(y[4] == 0)
    R.set_option("gemv_kernel", 1)                         # the general grouped kernel on the same inputs
    try:
        y2 = _gpu(x, w, idx, s, n, E, x_bf16=x_bf16)
    finally:
        R.set_option("gemv_kernel", 0)
    assert_within_tolerance(y2, ref, bnd, tol=2e-5, what=f"moe general {sch} m={m}")


@pytest.mark.gpu
def test_gpu_grouped_routing_edges():
    import torch
    import rlx_b200 as R
    s, m, k, n, E = O.Q8_0, 20, 256, 12, 6
    w = O.fill_weights(s, 2, k, n * E)
    x = O.fill_normal(3, m * k).reshape(m, k)
    # all rows to one expert (more than eight: several passes), and ids out of range / NaN -> zero rows
    idx = np.full(m, 4, np.float32)
    y = _gpu(x, w, idx, s, n, E)
    ref = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    assert np.allclose(y, ref, rtol=0, atol=2e-5 * np.abs(ref).max() + 1e-6)
    # the reference's `as usize` cast: negative, fractional and NaN ids mean expert 0; E and above is out of range
    idx[3], idx[7], idx[11], idx[12], idx[13] = 6.0, -1.0, np.nan, 0.5, 5.9
    y = _gpu(x, w, idx, s, n, E)
    ref = O.grouped_matmul_bt(x, w, idx, m, k, n, E, s)
    slab = w.size // E
    for row, e in ((7, 0), (11, 0), (12, 0), (13, 5)):
        assert np.array_equal(ref[row], O.matmul_bt(x[row:row + 1], w[e * slab:(e + 1) * slab], 1, k, n, s).ravel())
    assert np.all(y[3] == 0) and np.all(ref[3] == 0) and np.any(y[4] != 0)
    assert np.allclose(y, ref, rtol=0, atol=2e-5 * np.abs(ref).max() + 1e-6)
    # bf16 output is the rounding of the f32 output
    idx = (np.arange(m) % E).astype(np.float32)
    yf = _gpu(x, w, idx, s, n, E)
    yb = _gpu(x, w, idx, s, n, E, y_bf16=True)
    assert np.array_equal(yb, torch.from_numpy(yf).to(torch.bfloat16).float().numpy())
    # errors
    from rlx_b200._lib import lib
    assert lib.rlxq_grouped_matmul(None, s, None, 0, None, None, None, 0, 4, 100, 4, 2, None, 0) == -2   # k % 32
    assert lib.rlxq_grouped_matmul(None, s, None, 0, None, None, None, 0, 4, 256, 4, 0, None, 0) == -11  # no experts
    assert lib.rlxq_grouped_matmul(None, 99, None, 0, None, None, None, 0, 4, 256, 4, 2, None, 0) == -1
