"""Regenerates the committed fixtures in this directory.

known_answers.json
    The reference's own known-answer vectors for this path, rebuilt from the byte
    recipes and assertions in its unit tests (read as text; the reference is Rust and
    cannot be executed in this image).  Each entry names the test it restates.

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
    np.savez_compressed(os.path.join(HERE, "seeded_small.npz"), **seeded())
    print("wrote known_answers.json and seeded_small.npz")


if __name__ == "__main__":
    main()
