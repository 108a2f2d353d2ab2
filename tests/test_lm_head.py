"""Tied LM head: greedy argmax and top-k over a GGUF-packed embedding.

CPU part: the oracle against the reference's own LM-head unit tests (restated in
tests/golden/lm_head_cases.json).  GPU part: rlxq_lm_head_argmax / rlxq_lm_head_topk through the C ABI.
With RLXQ_LM_EXACT the chosen tokens must equal the oracle's and the logits must be bit-identical (the
winners are re-evaluated in the reference's arithmetic); without it the logits carry the streaming GEMV's
rounding and the choice may differ only between rows that close.
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _cases():
    with open(os.path.join(GOLDEN, "lm_head_cases.json")) as f:
        return json.load(f)


def _unpack(c):
    s = O.SCHEMES[c["scheme"]]
    w = np.frombuffer(bytes.fromhex(c["bytes"]), np.uint8).copy()
    h = np.array(c["hidden"], np.float32)
    return s, w, h


@pytest.mark.parametrize("c", _cases(), ids=lambda c: c["name"])
def test_oracle_reproduces_the_reference_lm_head_tests(c):
    s, w, h = _unpack(c)
    logits = O.lm_logits(h, w, c["n_embd"], c["n_vocab"], s)
    assert np.array_equal(logits, np.array(c["logits"], np.float32))
    if "argmax" in c:
        idx, val, _ = O.lm_argmax(h, w, c["n_embd"], c["n_vocab"], s)
        assert idx == c["argmax"] and abs(float(val) - c["logits"][idx]) < c["val_tol"]
    else:
        top, _ = O.lm_topk(h, w, c["n_embd"], c["n_vocab"], s, c["cap"])
        assert [float(v) for _, v in top] == c["top_scores"]
        assert all(c["logits"][j] == float(v) for j, v in top)


def test_oracle_argmax_edge_semantics():
    """First maximum wins; (0, -inf) when nothing exceeds -inf (rlx-cpu/src/lm_head.rs:236-250)."""
    s = O.Q8_0
    w = O.fill_weights(s, 3, 64, 6)
    w = np.concatenate([w[:2 * 68], w[:2 * 68], w[4 * 68:]])        # rows 2,3 duplicate rows 0,1
    h = O.fill_normal(9, 64)
    idx, val, logits = O.lm_argmax(h, w, 64, 6, s)
    assert logits[0] == logits[2] and logits[1] == logits[3]
    assert idx == int(np.argmax(logits)) and idx not in (2, 3) or logits[idx] > logits[idx % 2]
    hn = h.copy()
    hn[5] = np.nan
    assert O.lm_argmax(hn, w, 64, 6, s)[:2] == (0, np.float32(-np.inf))


# ------------------------------------------------------------------ GPU
def _gpu(h, w, n_embd, n_vocab, s, cap=None, exact=True, bf16=False):
    import torch
    import rlx_b200 as R
    hd = torch.from_numpy(h).cuda()
    if bf16:
        hd = hd.to(torch.bfloat16)
    wd = torch.from_numpy(w).cuda()
    if cap is None:
        i, v = R.gguf_tied_lm_argmax(hd, wd, n_embd, n_vocab, s, exact=exact)
    else:
        i, v = R.gguf_tied_lm_topk(hd, wd, n_embd, n_vocab, s, cap, exact=exact)
    R.device_status()
    return i.cpu().numpy(), v.cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("c", _cases(), ids=lambda c: c["name"])
def test_gpu_reference_lm_head_tests(c):
    s, w, h = _unpack(c)
    if "argmax" in c:
        for exact in (True, False):
            i, v = _gpu(h, w, c["n_embd"], c["n_vocab"], s, exact=exact)
            assert int(i[0]) == c["argmax"]
            assert abs(float(v[0]) - c["logits"][c["argmax"]]) < c["val_tol"]
        i, v = _gpu(h, w, c["n_embd"], c["n_vocab"], s, exact=True)
        assert np.float32(v[0]) == np.float32(c["logits"][c["argmax"]])
    else:
        i, v = _gpu(h, w, c["n_embd"], c["n_vocab"], s, cap=c["cap"], exact=True)
        assert [float(x) for x in v] == c["top_scores"]
        assert all(np.float32(c["logits"][int(j)]) == x for j, x in zip(i, v))
        # 38 rows tie for the best score: ties go to the lowest token ids
        assert list(i) == sorted(i) and len(set(i.tolist())) == c["cap"]


SCHEMES = ["q4_0", "q8_0", "q4_k", "q6_k", "q5_k", "q8_k", "q2_k", "q3_k"]


@pytest.mark.gpu
@pytest.mark.parametrize("sch", SCHEMES)
@pytest.mark.parametrize("n_embd,n_vocab,bf16", [(2048, 5000, False), (4096, 2049, True), (6144, 300, False)])
def test_gpu_exact_mode_matches_oracle_bit_for_bit(sch, n_embd, n_vocab, bf16):
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 31 + n_vocab, n_embd, n_vocab)
    h = O.fill_normal(77 + n_embd, n_embd)
    if bf16:
        h = O.bf16_bits_to_f32(O.f32_to_bf16_bits(h)).ravel()
    idx, val, logits = O.lm_argmax(h, w, n_embd, n_vocab, s)
    gi, gv = _gpu(h, w, n_embd, n_vocab, s, exact=True, bf16=bf16)
    assert int(gi[0]) == idx and np.float32(gv[0]).view(np.uint32) == np.float32(val).view(np.uint32)
    for cap in (5, 40):
        top, _ = O.lm_topk(h, w, n_embd, n_vocab, s, cap)
        gi, gv = _gpu(h, w, n_embd, n_vocab, s, cap=cap, exact=True, bf16=bf16)
        assert [int(j) for j in gi] == [j for j, _ in top]
        assert np.array_equal(gv.view(np.uint32), np.array([v for _, v in top], np.float32).view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("sch", ["q4_0", "q4_k", "q6_k", "q3_k"])
def test_gpu_fast_mode_is_within_the_gemv_tolerance(sch):
    from tests.helpers import bound
    s = O.SCHEMES[sch]
    n_embd, n_vocab = 4096, 3000
    w = O.fill_weights(s, 5, n_embd, n_vocab)
    h = O.fill_normal(6, n_embd)
    idx, val, logits = O.lm_argmax(h, w, n_embd, n_vocab, s)
    bnd = bound(s, w, h.reshape(1, -1), n_vocab).ravel()
    gi, gv = _gpu(h, w, n_embd, n_vocab, s, exact=False)
    j = int(gi[0])
    assert abs(float(gv[0]) - float(logits[j])) <= 2e-5 * bnd[j]
    assert j == idx or float(logits[idx]) - float(logits[j]) <= 4e-5 * max(bnd[j], bnd[idx])
    gi, gv = _gpu(h, w, n_embd, n_vocab, s, cap=16, exact=False)
    assert len(set(gi.tolist())) == 16 and np.all(np.diff(gv) <= 0)
    assert np.all(np.abs(gv - logits[gi]) <= 2e-5 * bnd[gi])
    assert float(np.sort(logits)[-16]) - float(logits[gi].min()) <= 4e-5 * bnd.max()


@pytest.mark.gpu
def test_gpu_ties_nan_small_vocab_and_errors():
    import torch
    import rlx_b200 as R
    s = O.Q8_0
    n_embd = 256
    base = O.fill_weights(s, 3, n_embd, 4)
    rb = n_embd // 32 * 34
    w = np.concatenate([base, base[:2 * rb]])                  # rows 4, 5 repeat rows 0, 1
    h = O.fill_normal(9, n_embd)
    top, logits = O.lm_topk(h, w, n_embd, 6, s, 6)
    gi, gv = _gpu(h, w, n_embd, 6, s, cap=6)
    assert [int(j) for j in gi] == [j for j, _ in top]          # equal logits: lower id first
    assert np.array_equal(gv, np.array([v for _, v in top], np.float32))
    # cap larger than the vocabulary is clamped (rlx-cpu/src/lm_head.rs:181)
    gi2, _ = _gpu(h, w, n_embd, 6, s, cap=50)
    assert len(gi2) == 6
    # a NaN activation makes every logit NaN: nothing can be chosen
    hn = h.copy()
    hn[7] = np.nan
    gi, gv = _gpu(hn, w, n_embd, 6, s)
    assert int(gi[0]) == 0 and gv[0] == -np.inf
    gi, gv = _gpu(hn, w, n_embd, 6, s, cap=3)
    assert list(gi) == [-1] * 3 and np.all(gv == -np.inf)
    # errors: cap out of range, workspace too small
    from rlx_b200._lib import lib
    hd, wd = torch.from_numpy(h).cuda(), torch.from_numpy(w).cuda()
    out_i = torch.empty(4, dtype=torch.int32, device="cuda")
    out_v = torch.empty(4, dtype=torch.float32, device="cuda")
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    assert lib.rlxq_lm_head_topk(None, s, hd.data_ptr(), 0, wd.data_ptr(), n_embd, 6, 0, 1, ws.data_ptr(), ws.numel(),
                                 out_i.data_ptr(), out_v.data_ptr()) == -10
    assert lib.rlxq_lm_head_topk(None, s, hd.data_ptr(), 0, wd.data_ptr(), n_embd, 6, 65, 1, ws.data_ptr(), ws.numel(),
                                 out_i.data_ptr(), out_v.data_ptr()) == -10
    assert lib.rlxq_lm_head_argmax(None, s, hd.data_ptr(), 0, wd.data_ptr(), n_embd, 6, 1, ws.data_ptr(), 64,
                                   out_i.data_ptr(), out_v.data_ptr()) == -5
    assert lib.rlxq_lm_head_argmax(None, s, hd.data_ptr(), 0, wd.data_ptr(), 100, 6, 1, ws.data_ptr(), ws.numel(),
                                   out_i.data_ptr(), out_v.data_ptr()) == -2


@pytest.mark.gpu
def test_gpu_llama3_sized_vocabulary():
    """128256 x 4096 Q4_K: the tied embedding of an 8B model (295 MB of blocks)."""
    s, n_embd, n_vocab = O.Q4_K, 4096, 128256
    w = O.fill_weights(s, 11, n_embd, n_vocab)
    h = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(12, n_embd))).ravel()
    idx, val, _ = O.lm_argmax(h, w, n_embd, n_vocab, s)
    gi, gv = _gpu(h, w, n_embd, n_vocab, s, exact=True, bf16=True)
    assert int(gi[0]) == idx and np.float32(gv[0]) == np.float32(val)
    top, _ = O.lm_topk(h, w, n_embd, n_vocab, s, 10)
    gi, gv = _gpu(h, w, n_embd, n_vocab, s, cap=10, exact=True, bf16=True)
    assert [int(j) for j in gi] == [j for j, _ in top]
    assert np.array_equal(gv, np.array([v for _, v in top], np.float32))
