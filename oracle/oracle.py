"""ctypes wrapper around the CPU oracle (librlxq_oracle.so).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this
module; the shipped package (rlx_b200/) never does.  The oracle restates the reference's
CPU path (rlx-gguf/src/lib.rs decoders, rlx-cpu/src/gguf_matmul.rs:40-95); see
rlxq_oracle.h for the line-by-line citations and the parity status.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librlxq_oracle.so")

Q4_K, Q5_K, Q6_K, Q8_K, Q2_K, Q3_K, Q4_0, Q8_0, Q4_1, Q5_0, Q5_1 = 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10
SCHEMES = {"q4_k": Q4_K, "q5_k": Q5_K, "q6_k": Q6_K, "q8_k": Q8_K, "q2_k": Q2_K, "q3_k": Q3_K,
           "q4_0": Q4_0, "q8_0": Q8_0, "q4_1": Q4_1, "q5_0": Q5_0, "q5_1": Q5_1}
GEOMETRY = {Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), Q8_K: (256, 292), Q2_K: (256, 84),
            Q3_K: (256, 110), Q4_0: (32, 18), Q8_0: (32, 34), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24)}


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile if the .so is missing or stale."""
    src = os.path.join(_HERE, "rlxq_oracle.c")
    hdr = os.path.join(_HERE, "rlxq_oracle.h")
    stale = (not os.path.exists(_SO)) or any(
        os.path.getmtime(p) > os.path.getmtime(_SO) for p in (src, hdr))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "librlxq_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u8p, f32p = C.POINTER(C.c_uint8), C.POINTER(C.c_float)
        L.rlxo_scheme_geometry.argtypes = [C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.rlxo_f16_to_f32.argtypes = [C.c_uint16]
        L.rlxo_f16_to_f32.restype = C.c_float
        L.rlxo_f32_to_f16.argtypes = [C.c_float]
        L.rlxo_f32_to_f16.restype = C.c_uint16
        L.rlxo_bf16_to_f32.argtypes = [C.c_uint16]
        L.rlxo_bf16_to_f32.restype = C.c_float
        L.rlxo_f32_to_bf16.argtypes = [C.c_float]
        L.rlxo_f32_to_bf16.restype = C.c_uint16
        L.rlxo_dequant.argtypes = [C.c_uint32, u8p, C.c_uint64, f32p]
        L.rlxo_dequant_q6k_unsigned.argtypes = [u8p, C.c_uint64, f32p]
        L.rlxo_matmul_bt.argtypes = [f32p, u8p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32]
        L.rlxo_matmul_bt_mt.argtypes = [f32p, u8p, f32p, C.c_uint64, C.c_uint64, C.c_uint64,
                                        C.c_uint32, C.c_uint64, C.c_uint64, C.c_int]
        L.rlxo_silu.argtypes = [C.c_float]
        L.rlxo_silu.restype = C.c_float
        L.rlxo_ffn_swiglu.argtypes = [f32p, u8p, u8p, u8p, f32p, f32p, C.c_uint64, C.c_uint64,
                                      C.c_uint64, C.c_uint32, C.c_uint32, C.c_int]
        L.rlxo_allreduce_sum.argtypes = [f32p, C.c_uint64, C.c_uint64, f32p]
        L.rlxo_allreduce_sum.restype = None
        L.rlxo_fill_blocks.argtypes = [C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64, u8p]
        L.rlxo_fill_normal_f32.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        L.rlxo_fill_normal_f32.restype = None
        L.rlxo_q4k_pack_scales.argtypes = [u8p, u8p, u8p]
        L.rlxo_q4k_pack_scales.restype = None
        L.rlxo_q4k_unpack_scale_min.argtypes = [C.c_int, u8p, u8p, u8p]
        L.rlxo_q4k_unpack_scale_min.restype = None
        _lib = L
    return _lib


def _u8(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_uint8))


def _f32(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_float))


def packed_bytes(scheme: int, k: int, n: int) -> int:
    be, bb = GEOMETRY[scheme]
    assert (k * n) % be == 0
    return k * n // be * bb


def dequant(scheme: int, blocks: np.ndarray, n_elems: int) -> np.ndarray:
    out = np.empty(n_elems, np.float32)
    rc = lib().rlxo_dequant(scheme, _u8(blocks), n_elems, _f32(out))
    if rc:
        raise ValueError(f"rlxo_dequant rc={rc}")
    return out


def dequant_q6k_unsigned(blocks: np.ndarray, n_elems: int) -> np.ndarray:
    out = np.empty(n_elems, np.float32)
    rc = lib().rlxo_dequant_q6k_unsigned(_u8(blocks), n_elems, _f32(out))
    if rc:
        raise ValueError(f"rc={rc}")
    return out


def matmul_bt(x: np.ndarray, w: np.ndarray, m: int, k: int, n: int, scheme: int) -> np.ndarray:
    """The reference's serial fused matmul, exact accumulation order."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty((m, n), np.float32)
    rc = lib().rlxo_matmul_bt(_f32(x), _u8(w), _f32(out), m, k, n, scheme)
    if rc:
        raise ValueError(f"rlxo_matmul_bt rc={rc}")
    return out


def matmul_bt_mt(x, w, m, k, n, scheme, n0=0, n1=None, threads=None) -> np.ndarray:
    """Row-parallel version (bit-identical outputs); computes columns [n0, n1) of out."""
    x = np.ascontiguousarray(x, np.float32)
    n1 = n if n1 is None else n1
    threads = threads or (os.cpu_count() or 1)
    out = np.zeros((m, n), np.float32)
    rc = lib().rlxo_matmul_bt_mt(_f32(x), _u8(w), _f32(out), m, k, n, scheme, n0, n1, threads)
    if rc:
        raise ValueError(f"rlxo_matmul_bt_mt rc={rc}")
    return out


def ffn_swiglu(x, gate, up, down, m, d_model, d_ffn, scheme_gu, scheme_down, threads=None,
               want_h=False):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty((m, d_model), np.float32)
    h = np.empty((m, d_ffn), np.float32) if want_h else None
    threads = threads or (os.cpu_count() or 1)
    rc = lib().rlxo_ffn_swiglu(_f32(x), _u8(gate), _u8(up), _u8(down), _f32(y),
                               _f32(h) if want_h else None, m, d_model, d_ffn,
                               scheme_gu, scheme_down, threads)
    if rc:
        raise ValueError(f"rlxo_ffn_swiglu rc={rc}")
    return (y, h) if want_h else y


def allreduce_sum(parts: np.ndarray) -> np.ndarray:
    parts = np.ascontiguousarray(parts, np.float32)
    ranks, elems = parts.shape[0], int(np.prod(parts.shape[1:]))
    out = np.empty(parts.shape[1:], np.float32)
    lib().rlxo_allreduce_sum(_f32(parts), ranks, elems, _f32(out))
    return out


def fill_blocks(scheme: int, seed: int, n_blocks: int, first_block: int = 0) -> np.ndarray:
    be, bb = GEOMETRY[scheme]
    out = np.empty(n_blocks * bb, np.uint8)
    rc = lib().rlxo_fill_blocks(scheme, seed, first_block, n_blocks, _u8(out))
    if rc:
        raise ValueError(f"rlxo_fill_blocks rc={rc}")
    return out


def fill_weights(scheme: int, seed: int, k: int, n: int) -> np.ndarray:
    be, _ = GEOMETRY[scheme]
    return fill_blocks(scheme, seed, k * n // be)


def fill_normal(seed: int, count: int, first: int = 0) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().rlxo_fill_normal_f32(seed, first, count, _f32(out))
    return out


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrowing, vectorised restatement of rlxo_f32_to_bf16."""
    x = np.ascontiguousarray(a, np.float32).view(np.uint32)
    nan = (x & 0x7FFFFFFF) > 0x7F800000
    rb = np.uint32(0x8000)
    up = ((x & rb) != 0) & ((x & np.uint32(0x17FFF)) != 0)
    r = (x >> 16) + up.astype(np.uint32)
    r = np.where(nan, (x >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def grouped_matmul_bt(x: np.ndarray, w: np.ndarray, expert_idx: np.ndarray, m: int, k: int, n: int,
                      num_experts: int, scheme: int) -> np.ndarray:
    """gguf_grouped_matmul_bt (rlx-cpu/src/gguf_matmul.rs:102-139): counting-sort the rows by expert
    (grouped_moe_sort_plan, :178-205), one fused matmul per expert over its slab, unpermute (:207-218).
    The arithmetic is the C oracle's matmul; only the routing is done here.  Ids are read as `expert_idx[i] as
    usize` reads them (:187,198): a saturating cast, so NaN, negative values and fractions go to expert 0.  An id of
    num_experts or more indexes out of bounds in the reference (a panic); such rows stay zero here."""
    be, bb = GEOMETRY[scheme]
    slab = k * n // be * bb
    assert w.size == num_experts * slab and expert_idx.size == m
    x = np.ascontiguousarray(x, np.float32).reshape(m, k)
    raw = expert_idx.astype(np.float32)
    ids = np.where(raw >= 1.0, np.floor(np.minimum(raw, np.float32(2.0 ** 31))), 0.0).astype(np.int64)   # NaN compares false
    out = np.zeros((m, n), np.float32)
    for e in range(num_experts):
        rows = np.flatnonzero(ids == e) if m else np.array([], np.int64)
        if rows.size == 0:
            continue
        out[rows] = matmul_bt_mt(np.ascontiguousarray(x[rows]), np.ascontiguousarray(w[e * slab:(e + 1) * slab]),
                                 rows.size, k, n, scheme)
    return out


def lm_logits(hidden: np.ndarray, w: np.ndarray, n_embd: int, n_vocab: int, scheme: int) -> np.ndarray:
    """hidden . W[j,:] for every row j with row_dot_gguf's arithmetic (rlx-cpu/src/lm_head.rs:46-76): the same
    in-order f32 multiply-then-add as gguf_matmul_bt with m = 1, so that function is reused."""
    h = np.ascontiguousarray(hidden, np.float32).reshape(1, n_embd)
    return matmul_bt_mt(h, w, 1, n_embd, n_vocab, scheme).ravel()


def lm_argmax(hidden: np.ndarray, w: np.ndarray, n_embd: int, n_vocab: int, scheme: int):
    """gguf_tied_lm_argmax (rlx-cpu/src/lm_head.rs:223-251): strict '>' scan from (0, -inf)."""
    logits = lm_logits(hidden, w, n_embd, n_vocab, scheme)
    best_idx, best_val = 0, np.float32(-np.inf)
    v = np.where(np.isnan(logits), -np.inf, logits)
    j = int(np.argmax(v))                      # first maximum, as the scan finds it
    if v[j] > best_val:
        best_idx, best_val = j, logits[j]
    return best_idx, np.float32(best_val), logits


def lm_topk(hidden: np.ndarray, w: np.ndarray, n_embd: int, n_vocab: int, scheme: int, cap: int):
    """gguf_tied_lm_topk (rlx-cpu/src/lm_head.rs:172-199): the cap best (id, logit), best first.  The
    reference leaves the order of equal logits to an unstable selection; here equal logits are ordered
    by token id, which is one of the orders it may produce."""
    logits = lm_logits(hidden, w, n_embd, n_vocab, scheme)
    cap = max(1, min(cap, n_vocab))
    ok = np.flatnonzero(~np.isnan(logits))
    order = ok[np.lexsort((ok, -logits[ok].astype(np.float64)))][:cap]
    return [(int(j), np.float32(logits[j])) for j in order], logits


def row_norms(scheme: int, w: np.ndarray, k: int, n: int) -> np.ndarray:
    """||w_row||_2 per output row, in float64, for the matmul tolerance."""
    wf = dequant(scheme, w, k * n).reshape(n, k).astype(np.float64)
    return np.sqrt((wf * wf).sum(axis=1))
