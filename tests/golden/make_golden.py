"""Regenerates the committed fixtures in this directory.

known_answers.json
    The reference's own known-answer vectors for this path, rebuilt from the byte
    recipes and assertions in its unit tests (read as text; the reference is Rust and
    cannot be executed in this image).  Each entry names the test it restates.

grouped_matmul_case.json
    The reference's MoE grouped-matmul graph test (rlx-runtime/tests/dequant_grouped_matmul_gguf.rs).

lm_head_cases.json
    The reference's LM-head unit tests (rlx-cpu/src/lm_head.rs:254-335), restated the same way.

seeded_small.npz
    Seeded block bytes and activations at small shapes together with the CPU oracle's
    dequantised weights and matmul outputs.  These are ORACLE-generated (a regression
    pin for the oracle and a fixed comparison target for the CUDA path), not reference
    outputs.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle as O  # noqa: E402


def f16_bytes(v: float) -> bytes:
    return struct.pack("<e", v)


def known_answers() -> list[dict]:
    out = []

    # rlx-gguf/src/lib.rs:1188-1202  dequant_q8_0_block: d = 0.5, q[i] = i - 16
    qs = [(i - 16) for i in range(32)]
    b = f16_bytes(0.5) + bytes((q & 0xFF) for q in qs)
    out.append(dict(name="q8_0_d_half_ramp", cite="rlx-gguf/src/lib.rs:1188-1202", scheme="q8_0",
                    n_elems=32, bytes=b.hex(), expected=[0.5 * q for q in qs], tol=1e-6))

    # rlx-gguf/src/lib.rs:1205-1221  dequant_q4_0_block: d = 1, byte i = i | i << 4
    b = f16_bytes(1.0) + bytes(((i & 15) | ((i & 15) << 4)) for i in range(16))
    exp = [float(i) - 8.0 for i in range(16)] * 2
    out.append(dict(name="q4_0_nibble_order", cite="rlx-gguf/src/lib.rs:1205-1221", scheme="q4_0",
                    n_elems=32, bytes=b.hex(), expected=exp, tol=0.0))

    # rlx-gguf/src/lib.rs:1224-1264  Q4_K: d = dmin = 1, scales[0..4] = 1, rest 0, qs = 0x77.
    # The test asserts the first 128 outputs are 7.0; the last 128 follow from
    # get_scale_min_k4 (:743-751): sc = m = 0 for j >= 4, hence 0.0 (not asserted upstream).
    scales = bytes([1, 1, 1, 1] + [0] * 8)
    b = f16_bytes(1.0) + f16_bytes(1.0) + scales + bytes([0x77] * 128)
    out.append(dict(name="q4_k_first_half_sevens", cite="rlx-gguf/src/lib.rs:1224-1264",
                    scheme="q4_k", n_elems=256, bytes=b.hex(),
                    expected=[7.0] * 128 + [0.0] * 128, tol=1e-5, asserted_prefix=128))

    # rlx-gguf/src/lib.rs:1267-1291  Q6_K: ql = 0, qh = 0xAA, sc = 1, d = 1 -> all zeros
    b = bytes([0] * 128) + bytes([0xAA] * 64) + bytes([1] * 16) + f16_bytes(1.0)
    out.append(dict(name="q6_k_all_zero", cite="rlx-gguf/src/lib.rs:1267-1291", scheme="q6_k",
                    n_elems=256, bytes=b.hex(), expected=[0.0] * 256, tol=1e-5))

    # rlx-runtime/tests/dequant_matmul_gguf.rs:249-303  Q4_K through the graph: the same
    # block as above, x = 1 over k = 256, n = 1 -> y = 128 * 7 = 896 (rel 1e-3 upstream).
    out.append(dict(name="q4_k_matmul_ones", cite="rlx-runtime/tests/dequant_matmul_gguf.rs:249-303",
                    scheme="q4_k", n_elems=256, bytes=b"".join(
                        [f16_bytes(1.0), f16_bytes(1.0), scales, bytes([0x77] * 128)]).hex(),
                    matmul=dict(m=1, k=256, n=1, x="ones", expected=[896.0], rel_tol=1e-3)))

    # rlx-runtime/tests/dequant_matmul_gguf.rs:131-174  Q6_K zero block, x = 1 -> y = 0
    out.append(dict(name="q6_k_matmul_zero", cite="rlx-runtime/tests/dequant_matmul_gguf.rs:131-174",
                    scheme="q6_k", n_elems=256, bytes=b.hex(),
                    matmul=dict(m=1, k=256, n=1, x="ones", expected=[0.0], abs_tol=1e-4)))

    # ---- the other GGUF schemes of QuantScheme::is_gguf ----
    # rlx-gguf/src/lib.rs:1293-1306  Q2_K: d = 1, min = 0, every scale byte 0x01, every 2-bit field 3 -> 3.0
    b = f16_bytes(1.0) + f16_bytes(0.0) + bytes([0x01] * 16) + bytes([0xFF] * 64)
    out.append(dict(name="q2_k_constant_three", cite="rlx-gguf/src/lib.rs:1293-1306", scheme="q2_k",
                    n_elems=256, bytes=b.hex(), expected=[3.0] * 256, tol=1e-4))

    # rlx-gguf/src/lib.rs:1308-1315  Q3_K: an all-zero block decodes to finite values
    out.append(dict(name="q3_k_zero_block_is_finite", cite="rlx-gguf/src/lib.rs:1308-1315", scheme="q3_k",
                    n_elems=256, bytes=bytes(110).hex(), finite_only=True))

    # rlx-gguf/src/lib.rs:1317-1334  Q8_K: d = 0.25 (f32), q[i] = i - 128, zero block sums
    q8 = [(i - 128) for i in range(256)]
    b = struct.pack("<f", 0.25) + bytes((q & 0xFF) for q in q8) + bytes(32)
    out.append(dict(name="q8_k_quarter_ramp", cite="rlx-gguf/src/lib.rs:1317-1334", scheme="q8_k",
                    n_elems=256, bytes=b.hex(), expected=[0.25 * q for q in q8], tol=1e-6))

    def seq_dot(xrow, wrow):     # the tests' own reference: f32 accumulate in order
        acc = np.float32(0.0)
        for a, w in zip(xrow, wrow):
            acc = np.float32(acc + np.float32(a * w))
        return float(acc)

    # rlx-runtime/tests/dequant_matmul_gguf.rs:43-127 and rlx-cuda/tests/basic.rs:200-247
    # Q8_K through the graph: scale 0.0625, q[i] = i - 128, m = 2, k = 256, n = 1,
    # x[i] = i * 0.001 - 0.5 (f32), expected = in-order f32 dot with scale * q; |diff| < 1e-3
    b = struct.pack("<f", 0.0625) + bytes((q & 0xFF) for q in q8) + bytes(32)
    x = [np.float32(np.float32(i) * np.float32(0.001)) - np.float32(0.5) for i in range(2 * 256)]
    wref = [np.float32(np.float32(0.0625) * np.float32(q)) for q in q8]
    out.append(dict(name="q8_k_matmul_ramp", cite="rlx-runtime/tests/dequant_matmul_gguf.rs:43-127; rlx-cuda/tests/basic.rs:200-247",
                    scheme="q8_k", n_elems=256, bytes=b.hex(),
                    matmul=dict(m=2, k=256, n=1, x=[float(v) for v in x],
                                expected=[seq_dot(x[r * 256:(r + 1) * 256], wref) for r in range(2)], abs_tol=1e-3)))

    # rlx-runtime/tests/dequant_matmul_gguf.rs:176-241  layout regression: n = 4 distinct rows,
    # scale 1, q = clamp(1000 j + i - 128), x[i] = 0.01 (i + 1); relative error < 1e-4
    blocks, wrows = b"", []
    for j in range(4):
        qj = [max(-128, min(127, j * 1000 + i - 128)) for i in range(256)]
        blocks += struct.pack("<f", 1.0) + bytes((q & 0xFF) for q in qj) + bytes(32)
        wrows.append([np.float32(q) for q in qj])
    x = [np.float32(np.float32(0.01) * np.float32(np.float32(i) + np.float32(1.0))) for i in range(2 * 256)]
    out.append(dict(name="q8_k_layout_n4", cite="rlx-runtime/tests/dequant_matmul_gguf.rs:176-241",
                    scheme="q8_k", n_elems=1024, bytes=blocks.hex(),
                    matmul=dict(m=2, k=256, n=4, x=[float(v) for v in x],
                                expected=[seq_dot(x[r * 256:(r + 1) * 256], wrows[c]) for r in range(2) for c in range(4)],
                                rel_tol=1e-4)))
    return out


def grouped_case() -> dict:
    """rlx-runtime/tests/dequant_grouped_matmul_gguf.rs:82-128: three Q8_K experts with scales 0.25, 0.5, 1
    (every block q[i] = i - 128), k = 256, n = 4, m = 5 rows routed [1, 0, 2, 1, 0], x[i] = 0.01 (i + 1);
    expected = per-row in-order f32 dot with the routed expert's dequantised rows; relative error < 1e-4."""
    k, n, m, scales, route = 256, 4, 5, [0.25, 0.5, 1.0], [1, 0, 2, 1, 0]
    q = [i - 128 for i in range(256)]
    packed = b""
    for sc in scales:
        for _ in range(n):
            packed += struct.pack("<f", sc) + bytes((v & 0xFF) for v in q) + bytes(32)
    x = [np.float32(np.float32(0.01) * np.float32(np.float32(i) + np.float32(1.0))) for i in range(m * k)]
    exp = []
    for r in range(m):
        wrow = [np.float32(np.float32(scales[route[r]]) * np.float32(v)) for v in q]
        acc = np.float32(0.0)
        for a, w in zip(x[r * k:(r + 1) * k], wrow):
            acc = np.float32(acc + np.float32(a * w))
        exp += [float(acc)] * n
    return dict(name="grouped_q8k_three_experts", cite="rlx-runtime/tests/dequant_grouped_matmul_gguf.rs:82-128",
                scheme="q8_k", m=m, k=k, n=n, num_experts=3, expert_idx=[float(v) for v in route],
                bytes=packed.hex(), x=[float(v) for v in x], expected=exp, rel_tol=1e-4)


def lm_head_cases() -> list[dict]:
    """The reference's LM-head unit tests (rlx-cpu/src/lm_head.rs:254-335) restated: Q8_K rows with
    scale 1 and q = clamp(10 j + i - 128), hidden[i] = 0.01 i.  Expected logits are computed here with
    plain f32 in-order arithmetic, not with the oracle."""
    def build(n):
        blocks, rows = b"", []
        for j in range(n):
            qj = [max(-128, min(127, j * 10 + i - 128)) for i in range(256)]
            blocks += struct.pack("<f", 1.0) + bytes((q & 0xFF) for q in qj) + bytes(32)
            rows.append([np.float32(q) for q in qj])
        return blocks, rows
    hidden = [np.float32(np.float32(0.01) * np.float32(i)) for i in range(256)]

    def seq_dot(wrow):
        acc = np.float32(0.0)
        for a, w in zip(hidden, wrow):
            acc = np.float32(acc + np.float32(a * w))
        return float(acc)

    out = []
    # lm_head.rs:308-335 argmax_matches_matmul_on_q8k: n = 8, the argmax equals the matmul's, |val - logit| < 1e-3
    blocks, rows = build(8)
    logits = [seq_dot(r) for r in rows]
    out.append(dict(name="lm_argmax_q8k_n8", cite="rlx-cpu/src/lm_head.rs:308-335", scheme="q8_k", n_embd=256,
                    n_vocab=8, bytes=blocks.hex(), hidden=[float(h) for h in hidden], logits=logits,
                    argmax=int(np.argmax(np.array(logits, np.float32))), val_tol=1e-3))
    # lm_head.rs:277-305 topk_early_exit_matches_full_sort_gguf: n = 64, cap = 8; rows 26..63 saturate to
    # all-127 and tie for the best score, so any eight of them are a correct answer; scores must be equal
    blocks, rows = build(64)
    logits = [seq_dot(r) for r in rows]
    out.append(dict(name="lm_topk_q8k_n64_cap8", cite="rlx-cpu/src/lm_head.rs:277-305", scheme="q8_k", n_embd=256,
                    n_vocab=64, cap=8, bytes=blocks.hex(), hidden=[float(h) for h in hidden], logits=logits,
                    top_scores=sorted(logits, reverse=True)[:8]))
    return out


SEEDED = [
    # (name, scheme, m, k, n, seed) — small enough to commit, ragged on purpose
    ("q8_0_m1", "q8_0", 1, 256, 24, 11),
    ("q8_0_m3", "q8_0", 3, 96, 7, 12),
    ("q4_0_m1", "q4_0", 1, 256, 24, 21),
    ("q4_0_m8", "q4_0", 8, 512, 17, 22),
    ("q4_k_m1", "q4_k", 1, 512, 19, 31),
    ("q4_k_m5", "q4_k", 5, 256, 33, 32),
    ("q6_k_m1", "q6_k", 1, 512, 19, 41),
    ("q6_k_m2", "q6_k", 2, 2048, 9, 42),
    ("q5_k_m2", "q5_k", 2, 512, 11, 51),
    ("q8_k_m1", "q8_k", 1, 256, 13, 61),
    ("q2_k_m3", "q2_k", 3, 512, 9, 71),
    ("q3_k_m2", "q3_k", 2, 768, 7, 81),
]


def seeded() -> dict[str, np.ndarray]:
    arrs: dict[str, np.ndarray] = {}
    for name, sch, m, k, n, seed in SEEDED:
        s = O.SCHEMES[sch]
        w = O.fill_weights(s, seed, k, n)
        x = O.fill_normal(seed + 1000, m * k).reshape(m, k)
        arrs[f"{name}.w"] = w
        arrs[f"{name}.x"] = x
        arrs[f"{name}.deq"] = O.dequant(s, w, k * n)
        arrs[f"{name}.y"] = O.matmul_bt(x, w, m, k, n, s)
        arrs[f"{name}.meta"] = np.array([s, m, k, n, seed], np.int64)
    return arrs


def main() -> None:
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(known_answers(), f, indent=1)
    with open(os.path.join(HERE, "lm_head_cases.json"), "w") as f:
        json.dump(lm_head_cases(), f, indent=1)
    with open(os.path.join(HERE, "grouped_matmul_case.json"), "w") as f:
        json.dump(grouped_case(), f, indent=1)
    np.savez_compressed(os.path.join(HERE, "seeded_small.npz"), **seeded())
    print("wrote known_answers.json and seeded_small.npz")


if __name__ == "__main__":
    main()
