"""The reference's graph-level tests for this path, run through the Graph / Session mirror with
host buffers (rlx-runtime/tests/dequant_matmul_gguf.rs, rlx-cuda/tests/basic.rs:200-248)."""
import json
import os

import numpy as np
import pytest

import rlx_b200 as R
from rlx_b200 import DType, Device, Graph, QuantScheme, Session
from oracle import oracle as O
from tests.helpers import assert_within_tolerance, bound, make_case, reference

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _single(scheme, m, k, n, packed, x, exec_mode="graph"):
    g = Graph("case")
    x_in = g.input("x", [m, k], DType.F32)
    w_packed = g.param("w_packed", [len(packed)], DType.U8)
    y = g.dequant_matmul_packed(x_in, w_packed, scheme, n)
    g.set_outputs([y])
    compiled = Session(Device.Cuda, exec_mode=exec_mode).compile(g)
    compiled.set_param_typed("w_packed", packed, DType.U8)
    return compiled.run([("x", x)], (m, n))


@pytest.mark.parametrize("exec_mode", ["stream", "graph"])
def test_layout_case_n4(exec_mode):
    """run_q8k_layout_case (dequant_matmul_gguf.rs:176-241) with a scheme this path covers."""
    k, n, m = 256, 4, 2
    for scheme, s in ((QuantScheme.GgufQ8_0, O.Q8_0), (QuantScheme.GgufQ4K, O.Q4_K)):
        packed = O.fill_weights(s, 42, k, n)
        x = (0.01 * (np.arange(m * k, dtype=np.float32) + 1.0)).reshape(m, k)
        w_ref = O.dequant(s, packed, k * n).reshape(n, k)
        expected = np.zeros((m, n), np.float32)
        for r in range(m):
            for c in range(n):
                acc = np.float32(0)
                for i in range(k):
                    acc = np.float32(acc + np.float32(x[r, i] * w_ref[c, i]))
                expected[r, c] = acc
        actual = _single(scheme, m, k, n, packed, x, exec_mode)
        rel = np.abs(actual - expected) / np.maximum(np.abs(expected), 1.0)
        assert rel.max() < 1e-4


def test_known_answer_graphs():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = [c for c in json.load(f) if "matmul" in c]
    for case in cases:
        mm = case["matmul"]
        packed = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8).copy()
        scheme = QuantScheme(O.SCHEMES[case["scheme"]])
        x = (np.ones((mm["m"], mm["k"]), np.float32) if mm["x"] == "ones"
             else np.array(mm["x"], np.float32).reshape(mm["m"], mm["k"]))
        y = _single(scheme, mm["m"], mm["k"], mm["n"], packed, x).ravel()
        exp = np.array(mm["expected"], np.float32)
        if "rel_tol" in mm:
            assert np.all(np.abs(y - exp) / np.maximum(np.abs(exp), 1.0) < mm["rel_tol"]), case["name"]
        else:
            assert np.all(np.abs(y - exp) < mm["abs_tol"]), case["name"]


def test_decode_shapes_through_the_session():
    for sch, m, k, n in (("q4_0", 1, 4096, 512), ("q8_0", 8, 1024, 300), ("q6_k", 1, 2048, 64)):
        s = O.SCHEMES[sch]
        w, x = make_case(s, m, k, n, seed=12)
        y = _single(QuantScheme(s), m, k, n, w, x)
        assert_within_tolerance(y, reference(s, w, x, n), bound(s, w, x, n), what=sch)


def test_run_typed_bf16_in_bf16_out():
    s, m, k, n = O.Q4_K, 2, 1024, 96
    w, x = make_case(s, m, k, n, seed=13, x_bf16=True)
    g = Graph("typed")
    xi = g.input("x", [m, k], DType.BF16)
    wp = g.param("w", [len(w)], DType.U8)
    g.set_outputs([g.dequant_matmul_packed(xi, wp, QuantScheme.GgufQ4K, n, DType.BF16)])
    c = Session(Device.Cuda).compile(g)
    c.set_param_typed("w", w, DType.U8)
    yb = c.run_typed([("x", O.f32_to_bf16_bits(x), DType.BF16)], (m, n), DType.BF16)
    y = O.bf16_bits_to_f32(yb)
    ref = reference(s, w, x, n)
    # the output is the f32 accumulator rounded once to bf16: half an ulp of bf16 on top of the bound
    bnd = bound(s, w, x, n)
    err = np.abs(y.astype(np.float64) - ref)
    assert np.all(err <= 1e-3 * bnd + np.abs(ref) * 2.0 ** -8)


def test_swiglu_ffn_graph_matches_oracle():
    """down(up(x) * silu(gate(x))) — rlx-flow/src/blocks/swiglu.rs:48-52 — as a five-node graph."""
    dm, df, m = 512, 1024, 2
    gw = O.fill_weights(O.Q4_K, 1, dm, df)
    uw = O.fill_weights(O.Q4_K, 2, dm, df)
    dw = O.fill_weights(O.Q4_K, 3, df, dm)
    x = O.fill_normal(4, m * dm).reshape(m, dm)
    g = Graph("ffn")
    xi = g.input("x", [m, dm])
    pg, pu, pd = g.param("gate", [len(gw)]), g.param("up", [len(uw)]), g.param("down", [len(dw)])
    gate = g.dequant_matmul_packed(xi, pg, QuantScheme.GgufQ4K, df)
    up = g.dequant_matmul_packed(xi, pu, QuantScheme.GgufQ4K, df)
    h = g.swiglu_mul(gate, up)
    g.set_outputs([g.dequant_matmul_packed(h, pd, QuantScheme.GgufQ4K, dm)])
    c = Session(Device.Cuda).compile(g)
    for nm, arr in (("gate", gw), ("up", uw), ("down", dw)):
        c.set_param_typed(nm, arr, DType.U8)
    y = c.run([("x", x)], (m, dm))
    y_ref, h_ref = O.ffn_swiglu(x, gw, uw, dw, m, dm, df, O.Q4_K, O.Q4_K, want_h=True)
    bnd = bound(O.Q4_K, dw, h_ref, dm)
    # two chained matmuls: allow the first layer's error to propagate (still the 1e-3 form)
    assert_within_tolerance(y, y_ref, bnd, what="ffn")


@pytest.mark.parametrize("m,dm,df,x_bf16", [(1, 8192, 28672, True), (2, 1024, 4096, False), (1, 512, 1024, False), (16, 1024, 2048, True)])
def test_swiglu_ffn_graph_is_fused_and_matches_the_unfused_graph(m, dm, df, x_bf16):
    """The five-node FFN is lowered to the fused form: fewer kernels per run, and both lowerings agree with the
    oracle FFN to the path's tolerance; the 70B-shaped layer of the tensor-parallel configuration included."""
    gw = O.fill_weights(O.Q4_K, 11, dm, df)
    uw = O.fill_weights(O.Q4_K, 12, dm, df)
    dw = O.fill_weights(O.Q4_K, 13, df, dm)
    x = O.fill_normal(14, m * dm).reshape(m, dm)
    if x_bf16:
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).reshape(m, dm)

    def build():
        g = Graph("ffn")
        xi = g.input("x", [m, dm], DType.BF16 if x_bf16 else DType.F32)
        pg, pu, pd = g.param("gate", [len(gw)]), g.param("up", [len(uw)]), g.param("down", [len(dw)])
        gate = g.dequant_matmul_packed(xi, pg, QuantScheme.GgufQ4K, df)
        up = g.dequant_matmul_packed(xi, pu, QuantScheme.GgufQ4K, df)
        g.set_outputs([g.dequant_matmul_packed(g.swiglu_mul(gate, up), pd, QuantScheme.GgufQ4K, dm)])
        c = Session(Device.Cuda, exec_mode="graph").compile(g)
        for nm, arr in (("gate", gw), ("up", uw), ("down", dw)):
            c.set_param_typed(nm, arr, DType.U8)
        return c

    def run(c):
        xin = O.f32_to_bf16_bits(x) if x_bf16 else x
        before = R.launch_count()
        y = c.run_typed([("x", xin, DType.BF16 if x_bf16 else DType.F32)], (m, dm), DType.F32)
        return y, R.launch_count() - before

    fused = build()
    assert fused.fused_ffn_count() == 1
    y_f, launches_f = run(fused)
    R.set_option("graph_fuse_ffn", 0)
    try:
        plain = build()
    finally:
        R.set_option("graph_fuse_ffn", 1)
    assert plain.fused_ffn_count() == 0
    y_p, launches_p = run(plain)
    R.device_status()
    assert launches_f < launches_p, (launches_f, launches_p)
    y_ref, h_ref = O.ffn_swiglu(x, gw, uw, dw, m, dm, df, O.Q4_K, O.Q4_K, want_h=True)
    bnd = bound(O.Q4_K, dw, h_ref, dm)
    assert_within_tolerance(y_f, y_ref, bnd, what="fused ffn")
    assert_within_tolerance(y_p, y_ref, bnd, what="unfused ffn")


def test_ffn_pattern_is_not_fused_when_an_intermediate_value_is_used_elsewhere():
    dm, df, m = 512, 1024, 1
    g = Graph("ffn2")
    xi = g.input("x", [m, dm])
    pg, pu = g.param("gate", [R.packed_bytes(0, dm, df)]), g.param("up", [R.packed_bytes(0, dm, df)])
    gate = g.dequant_matmul_packed(xi, pg, QuantScheme.GgufQ4K, df)
    up = g.dequant_matmul_packed(xi, pu, QuantScheme.GgufQ4K, df)
    h = g.swiglu_mul(gate, up)
    g.set_outputs([h])                       # the product itself is the output: nothing to fuse into
    c = Session(Device.Cuda).compile(g)
    assert c.fused_ffn_count() == 0


def test_run_errors():
    s, m, k, n = O.Q8_0, 1, 256, 8
    w, x = make_case(s, m, k, n, seed=2)
    g = Graph("err")
    xi = g.input("x", [m, k])
    wp = g.param("w", [len(w)])
    g.set_outputs([g.dequant_matmul_packed(xi, wp, QuantScheme.GgufQ8_0, n)])
    c = Session(Device.Cuda).compile(g)
    with pytest.raises(R.RlxqError):
        c.set_param_typed("w", w[:-1], DType.U8)          # wrong byte count
    with pytest.raises(R.RlxqError):
        c.set_param_typed("nope", w, DType.U8)
    c.set_param_typed("w", w, DType.U8)
    with pytest.raises(R.RlxqError):
        c.run([("y", x)], (m, n))                          # input name not in the graph
    with pytest.raises(R.RlxqError):
        c.run([("x", x[:, :128])], (m, n))                 # wrong size
    assert c.arena_bytes < 4 * (len(w) + 4096)             # byte-accurate slots, no 4x inflation
