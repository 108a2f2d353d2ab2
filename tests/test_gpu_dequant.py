"""GPU parity: rlxq_dequant_f32 must be bit-identical to the CPU oracle."""
import json
import os

import numpy as np
import pytest

import rlx_b200 as R
from oracle import oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _gpu_dequant(scheme, w, n_elems):
    import torch
    wd = torch.from_numpy(w).cuda()
    out = R.dequant_f32(wd, scheme, n_elems)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("sch", ["q8_0", "q4_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("nblk", [1, 3, 257, 5000])
def test_dequant_bit_exact_seeded(sch, nblk):
    s = O.SCHEMES[sch]
    be, _ = O.GEOMETRY[s]
    w = O.fill_blocks(s, 100 + nblk, nblk)
    got = _gpu_dequant(s, w, nblk * be)
    exp = O.dequant(s, w, nblk * be)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


def test_dequant_known_answers_from_the_reference_tests():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = json.load(f)
    for case in cases:
        if "expected" not in case:
            continue
        s = O.SCHEMES[case["scheme"]]
        w = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8).copy()
        got = _gpu_dequant(s, w, case["n_elems"])
        exp = np.array(case["expected"], np.float32)
        assert np.max(np.abs(got - exp)) <= case["tol"], case["name"]


def test_dequant_committed_fixtures():
    z = np.load(os.path.join(GOLDEN, "seeded_small.npz"))
    for nm in sorted({k.split(".")[0] for k in z.files}):
        s, m, k, n, _ = (int(v) for v in z[f"{nm}.meta"])
        got = _gpu_dequant(s, z[f"{nm}.w"], k * n)
        assert np.array_equal(got.view(np.uint32), z[f"{nm}.deq"].view(np.uint32)), nm


def test_dequant_special_scales():
    # subnormal, zero, negative, largest finite fp16 scales; arbitrary bytes elsewhere
    rng = np.random.default_rng(5)
    for s in (O.Q8_0, O.Q4_0, O.Q4_K, O.Q6_K):
        be, bb = O.GEOMETRY[s]
        w = rng.integers(0, 256, 64 * bb, dtype=np.uint8).reshape(64, bb)
        specials = [0x0001, 0x03FF, 0x0000, 0x8000, 0xBC00, 0x7BFF, 0x8001, 0x3C00]
        for i in range(64):
            v = specials[i % len(specials)]
            pos = 208 if s == O.Q6_K else 0
            w[i, pos], w[i, pos + 1] = v & 0xFF, v >> 8
            if s == O.Q4_K:
                v2 = specials[(i // 8) % len(specials)]
                w[i, 2], w[i, 3] = v2 & 0xFF, v2 >> 8
        w = w.ravel()
        got = _gpu_dequant(s, w, 64 * be)
        exp = O.dequant(s, w, 64 * be)
        assert np.array_equal(got.view(np.uint32), exp.view(np.uint32)), s


@pytest.mark.parametrize("sch,k,n", [("q8_0", 4096, 4096), ("q4_0", 4096, 11008), ("q4_0", 11008, 4096),
                                     ("q4_k", 4096, 14336), ("q6_k", 14336, 4096)])
def test_dequant_bit_exact_benchmark_weights(sch, k, n):
    """Every weight of configurations 0-2, full size."""
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 7, k, n)
    got = _gpu_dequant(s, w, k * n)
    exp = O.dequant(s, w, k * n)
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


@pytest.mark.parametrize("sch,k,n", [("q4_k", 8192, 28672), ("q8_0", 8192, 28672), ("q4_0", 8192, 28672)])
def test_dequant_bit_exact_large_weights_by_slices(sch, k, n):
    """Configurations 3 and 4: the whole tensor is decoded on the GPU; the oracle checks the
    first, a middle and the last 4 Mi-element slice, and a checksum-of-slices covers the rest
    against a second GPU decode of independently uploaded slices."""
    import torch
    s = O.SCHEMES[sch]
    be, bb = O.GEOMETRY[s]
    w = O.fill_weights(s, 8, k, n)
    wd = torch.from_numpy(w).cuda()
    full = R.dequant_f32(wd, s, k * n)
    sl = 4 << 20
    total = k * n
    for start in (0, (total // 2 // sl) * sl, total - sl):
        exp = O.dequant(s, w[start // be * bb:(start + sl) // be * bb], sl)
        got = full[start:start + sl].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), exp.view(np.uint32)), (sch, start)
    # slice-wise decode of separately uploaded pieces must reproduce the whole-tensor decode
    for start in range(0, total, 32 << 20):
        cnt = min(32 << 20, total - start)
        piece = torch.from_numpy(w[start // be * bb:(start + cnt) // be * bb]).cuda()
        part = R.dequant_f32(piece, s, cnt)
        assert torch.equal(part.view(torch.int32), full[start:start + cnt].view(torch.int32))


def test_dequant_empty_and_errors():
    import torch
    w = torch.zeros(18, dtype=torch.uint8, device="cuda")
    out = R.dequant_f32(w, O.Q4_0, 0)
    assert out.numel() == 0
    with pytest.raises(R.RlxqError):
        R.dequant_f32(w, O.Q4_0, 16)
