"""CPU tests of the oracle: the reference's known-answer vectors, an independent
formula-level decoder, and the properties the reference's own tests assert."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load_known():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", _load_known(), ids=lambda c: c["name"])
def test_reference_known_answers(case):
    s = O.SCHEMES[case["scheme"]]
    blocks = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8).copy()
    if case.get("finite_only"):
        assert np.isfinite(O.dequant(s, blocks, case["n_elems"])).all()
    if "expected" in case:
        got = O.dequant(s, blocks, case["n_elems"])
        exp = np.array(case["expected"], np.float32)
        if case["tol"] == 0.0:
            assert np.array_equal(got, exp)
        else:
            assert np.max(np.abs(got - exp)) < case["tol"]
    if "matmul" in case:
        mm = case["matmul"]
        x = (np.ones((mm["m"], mm["k"]), np.float32) if mm["x"] == "ones"
             else np.array(mm["x"], np.float32).reshape(mm["m"], mm["k"]))
        y = O.matmul_bt(x, blocks, mm["m"], mm["k"], mm["n"], s).ravel()
        exp = np.array(mm["expected"], np.float32)
        if "rel_tol" in mm:
            assert np.all(np.abs(y - exp) / np.maximum(np.abs(exp), 1.0) < mm["rel_tol"])
        else:
            assert np.all(np.abs(y - exp) < mm["abs_tol"])


# ---- independent decoder written from the format description in the benchmark configs ----
def _f16(b):
    return np.frombuffer(bytes(b), "<f2").astype(np.float32)


def formula_decode(scheme, blocks, n_elems):
    be, bb = O.GEOMETRY[scheme]
    nb = n_elems // be
    B = blocks.reshape(nb, bb)
    f = np.float32
    if scheme == O.Q8_0:
        d = B[:, :2].copy().view("<f2").astype(f)
        q = B[:, 2:].view(np.int8).astype(f)
        return (d * q).ravel()
    if scheme == O.Q4_0:
        d = B[:, :2].copy().view("<f2").astype(f)
        qs = B[:, 2:]
        q = np.concatenate([qs & 15, qs >> 4], axis=1).astype(np.int32) - 8
        return (d * q.astype(f)).ravel()
    if scheme == O.Q4_K:
        d = B[:, 0:2].copy().view("<f2").astype(f)
        dmin = B[:, 2:4].copy().view("<f2").astype(f)
        s = B[:, 4:16].astype(np.uint32)
        sc = np.zeros((nb, 8), np.uint32)
        mn = np.zeros((nb, 8), np.uint32)
        for j in range(8):
            if j < 4:
                sc[:, j] = s[:, j] & 63
                mn[:, j] = s[:, j + 4] & 63
            else:
                sc[:, j] = (s[:, j + 4] & 15) | ((s[:, j - 4] >> 6) << 4)
                mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
        qs = B[:, 16:].reshape(nb, 4, 32)
        q = np.stack([qs & 15, qs >> 4], axis=2).reshape(nb, 8, 32).astype(f)  # sub-block major
        dsc = (d * sc.astype(f))[:, :, None]
        dm = (dmin * mn.astype(f))[:, :, None]
        return ((dsc * q).astype(f) - dm).astype(f).ravel()
    if scheme == O.Q6_K:
        ql = B[:, :128].reshape(nb, 2, 2, 32).astype(np.int32)   # half, (l | l+32), l
        qh = B[:, 128:192].reshape(nb, 2, 32).astype(np.int32)
        sc = B[:, 192:208].copy().view(np.int8).reshape(nb, 2, 8).astype(f)
        d = B[:, 208:210].copy().view("<f2").astype(f).reshape(nb, 1, 1)
        out = np.zeros((nb, 2, 4, 32), f)
        for g in range(4):
            lo = (ql[:, :, g & 1, :] >> (4 * (g >> 1))) & 15
            hi = (qh >> (2 * g)) & 3
            q = ((lo | (hi << 4)) - 32).astype(f)
            # scale index within the half: is + 2g with is = l // 16
            idx = (np.arange(32) // 16)[None, None, :] + 2 * g
            scg = np.take_along_axis(sc, np.broadcast_to(idx, (nb, 2, 32)), axis=2)
            out[:, :, g, :] = ((d * scg).astype(f) * q).astype(f)
        return out.ravel()
    if scheme == O.Q5_K:
        # d, dmin, 12 scale bytes (as Q4_K), 32 bytes of fifth bits (bit j of byte l belongs to
        # weight l of sub-block j), 128 nibble bytes (as Q4_K)
        d = B[:, 0:2].copy().view("<f2").astype(f)
        dmin = B[:, 2:4].copy().view("<f2").astype(f)
        s = B[:, 4:16].astype(np.uint32)
        sc = np.zeros((nb, 8), np.uint32)
        mn = np.zeros((nb, 8), np.uint32)
        for j in range(8):
            if j < 4:
                sc[:, j], mn[:, j] = s[:, j] & 63, s[:, j + 4] & 63
            else:
                sc[:, j] = (s[:, j + 4] & 15) | ((s[:, j - 4] >> 6) << 4)
                mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
        qh = B[:, 16:48].astype(np.uint32)                                  # [nb, 32]
        fifth = np.stack([(qh >> j) & 1 for j in range(8)], axis=1) * 16    # [nb, 8, 32]
        qs = B[:, 48:].reshape(nb, 4, 32)
        q = (np.stack([qs & 15, qs >> 4], axis=2).reshape(nb, 8, 32) + fifth).astype(f)
        dsc = (d * sc.astype(f))[:, :, None]
        dm = (dmin * mn.astype(f))[:, :, None]
        return ((dsc * q).astype(f) - dm).astype(f).ravel()
    if scheme == O.Q8_K:
        d = B[:, 0:4].copy().view("<f4")
        q = B[:, 4:260].copy().view(np.int8).astype(f)
        return (d * q).astype(f).ravel()
    if scheme == O.Q2_K:
        # d, dmin, 16 bytes (scale | min << 4) for 16-weight groups, 64 quant bytes: two halves of
        # 32 bytes, each holding four 2-bit planes; group g of a half = plane g // 2, bytes 16 (g % 2) ..
        d = B[:, 0:2].copy().view("<f2").astype(f)
        mn = B[:, 2:4].copy().view("<f2").astype(f)
        scb = B[:, 4:20].astype(np.uint32).reshape(nb, 2, 4, 2)             # half, plane, sub
        q = B[:, 20:84].astype(np.uint32).reshape(nb, 2, 1, 2, 16)          # half, -, sub, l
        planes = (q >> (2 * np.arange(4, dtype=np.uint32))[None, None, :, None, None]) & 3   # [nb,2,4,2,16]
        dl = (d[:, :, None, None] * (scb & 15).astype(f))[..., None]
        ml = (mn[:, :, None, None] * (scb >> 4).astype(f))[..., None]
        return ((dl * planes.astype(f)).astype(f) - ml).astype(f).ravel()
    if scheme == O.Q3_K:
        # d, 12 scale bytes, 32 mask bytes, 64 quant bytes.  Scale i (0..15): low nibble field from
        # bytes 0..7 (i < 8: low nibble of byte i, else high nibble of byte i - 8), two more bits from
        # bytes 8..11 (bits 2 (i // 4) of byte 8 + i % 4); value = field - 32.
        d = B[:, 0:2].copy().view("<f2").astype(f)
        sb = B[:, 2:14].astype(np.int32)
        sc = np.zeros((nb, 16), np.int32)
        for i in range(16):
            low = (sb[:, i] & 15) if i < 8 else (sb[:, i - 8] >> 4)
            high = (sb[:, 8 + i % 4] >> (2 * (i // 4))) & 3
            sc[:, i] = (low | (high << 4)) - 32
        hm = B[:, 14:46].astype(np.int32).reshape(nb, 1, 1, 2, 16)          # -, -, sub, l
        q = B[:, 46:110].astype(np.int32).reshape(nb, 2, 1, 2, 16)          # half, -, sub, l
        plane = np.arange(4).reshape(1, 1, 4, 1, 1)
        half = np.arange(2).reshape(1, 2, 1, 1, 1)
        two = (q >> (2 * plane)) & 3
        bit = (hm >> (4 * half + plane)) & 1
        val = (two - 4 * (1 - bit)).astype(f)                                # [nb, 2, 4, 2, 16]
        dl = (d[:, :, None, None] * sc.reshape(nb, 2, 4, 2).astype(f))[..., None]
        return (dl * val).astype(f).ravel()
    if scheme in (O.Q4_1, O.Q5_0, O.Q5_1):
        # 32-weight blocks: f16 d [, f16 m] [, u32 of fifth bits], 16 bytes of nibbles; weight j is the low nibble of
        # byte j, weight 16 + j the high nibble, bit j (16 + j) of the u32 its fifth bit.
        d = B[:, 0:2].copy().view("<f2").astype(f)
        off = 2
        mn = None
        if scheme != O.Q5_0:
            mn = B[:, 2:4].copy().view("<f2").astype(f)
            off = 4
        fifth = np.zeros((nb, 32), np.uint32)
        if scheme != O.Q4_1:
            qh = B[:, off:off + 4].copy().view("<u4")                          # [nb, 1]
            fifth = ((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1) << 4
            off += 4
        qs = B[:, off:off + 16].astype(np.uint32)
        q = np.concatenate([qs & 15, qs >> 4], axis=1) | fifth                # [nb, 32]
        if scheme == O.Q5_0:
            return (d * (q.astype(np.int32) - 16).astype(f)).astype(f).ravel()
        return ((d * q.astype(f)).astype(f) + mn).astype(f).ravel()
    raise ValueError(scheme)


@pytest.mark.parametrize("sch", ["q8_0", "q4_0", "q4_k", "q6_k", "q5_k", "q8_k", "q2_k", "q3_k", "q4_1", "q5_0", "q5_1"])
def test_oracle_matches_formula_decoder_bit_exact(sch):
    s = O.SCHEMES[sch]
    be, _ = O.GEOMETRY[s]
    nblk = 300
    w = O.fill_blocks(s, 1234, nblk)
    a = O.dequant(s, w, nblk * be)
    b = formula_decode(s, w, nblk * be)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q4k_upper_subblocks_and_scale_roundtrip():
    rng = np.random.default_rng(7)
    import ctypes as C
    for _ in range(50):
        sc = rng.integers(0, 64, 8).astype(np.uint8)
        mn = rng.integers(0, 64, 8).astype(np.uint8)
        packed = np.zeros(12, np.uint8)
        O.lib().rlxo_q4k_pack_scales(O._u8(sc), O._u8(mn), O._u8(packed))
        for j in range(8):
            a, b = C.c_uint8(), C.c_uint8()
            O.lib().rlxo_q4k_unpack_scale_min(j, O._u8(packed), C.byref(a), C.byref(b))
            assert (a.value, b.value) == (sc[j], mn[j])


def test_q6k_negative_scales_signed_vs_unsigned_decoder():
    w = O.fill_blocks(O.Q6_K, 5, 4)
    signed = O.dequant(O.Q6_K, w, 1024)
    unsigned = O.dequant_q6k_unsigned(w, 1024)
    sc = w.reshape(4, 210)[:, 192:208].view(np.int8)
    assert (sc < 0).any()
    assert not np.array_equal(signed, unsigned)          # the two upstream decoders differ
    # where every sub-scale is non-negative they agree
    w2 = w.copy().reshape(4, 210)
    w2[:, 192:208] &= 0x3F
    w2 = w2.ravel()
    assert np.array_equal(O.dequant(O.Q6_K, w2, 1024), O.dequant_q6k_unsigned(w2, 1024))


def test_special_scales_subnormal_zero_negative():
    # fp16 d: subnormal, zero, negative, largest finite
    for bits in (0x0001, 0x03FF, 0x0000, 0x8000, 0xBC00, 0x7BFF):
        blk = np.zeros(34, np.uint8)
        blk[0], blk[1] = bits & 0xFF, bits >> 8
        blk[2:] = np.arange(-16, 16).astype(np.int8).view(np.uint8)
        d = np.array([bits], np.uint16).view(np.float16).astype(np.float32)[0]
        got = O.dequant(O.Q8_0, blk, 32)
        exp = (d * np.arange(-16, 16).astype(np.float32)).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))


def test_f16_bf16_conversions():
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([O.lib().rlxo_f16_to_f32(int(h)) for h in allh[::7]], np.float32)
    r = ref[::7]
    ok = (got.view(np.uint32) == r.view(np.uint32)) | (np.isnan(got) & np.isnan(r))
    assert ok.all()
    rng = np.random.default_rng(3)
    f = np.concatenate([rng.standard_normal(5000).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 5000),
                        np.array([0.0, -0.0, 1e-3, 1e-2, 65504.0, 1e-8, np.inf], np.float32)])
    h = np.array([O.lib().rlxo_f32_to_f16(float(v)) for v in f], np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(h, f.astype(np.float16).view(np.uint16))
    import torch
    tb = torch.from_numpy(f).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(f), tb)
    hb = np.array([O.lib().rlxo_f32_to_bf16(float(v)) for v in f], np.uint16)
    assert np.array_equal(hb, tb)
    assert np.array_equal(O.bf16_bits_to_f32(tb), torch.from_numpy(f).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("sch,m,k,n", [("q8_0", 1, 256, 4), ("q4_0", 2, 256, 4), ("q4_k", 2, 256, 4),
                                       ("q6_k", 3, 512, 5), ("q4_0", 8, 96, 3)])
def test_fused_equals_dequant_then_dot(sch, m, k, n):
    """rlx-cpu/src/gguf_matmul.rs:238-277 (1e-4) and the n=4 layout-regression shape of
    rlx-runtime/tests/dequant_matmul_gguf.rs:176-241 (distinct rows, m=2, k=256)."""
    s = O.SCHEMES[sch]
    w = O.fill_weights(s, 99, k, n)
    x = (0.01 * (np.arange(m * k, dtype=np.float32) + 1.0)).reshape(m, k)
    y = O.matmul_bt(x, w, m, k, n, s)
    wf = O.dequant(s, w, k * n).reshape(n, k)
    exp = np.zeros((m, n), np.float32)
    for r in range(m):
        for c in range(n):
            acc = np.float32(0)
            for i in range(k):
                acc = np.float32(acc + np.float32(x[r, i] * wf[c, i]))
            exp[r, c] = acc
    assert np.array_equal(y, exp)   # same order, so bit-identical (upstream asks 1e-4)
    y_mt = O.matmul_bt_mt(x, w, m, k, n, s, threads=3)
    assert np.array_equal(y, y_mt)


def test_seeded_fixtures_reproduce():
    z = np.load(os.path.join(GOLDEN, "seeded_small.npz"))
    names = sorted({k.split(".")[0] for k in z.files})
    assert len(names) == 12
    for nm in names:
        s, m, k, n, seed = (int(v) for v in z[f"{nm}.meta"])
        w = O.fill_weights(s, seed, k, n)
        assert np.array_equal(w, z[f"{nm}.w"])
        x = O.fill_normal(seed + 1000, m * k).reshape(m, k)
        assert np.array_equal(x, z[f"{nm}.x"])
        assert np.array_equal(O.dequant(s, w, k * n), z[f"{nm}.deq"])
        assert np.array_equal(O.matmul_bt(x, w, m, k, n, s), z[f"{nm}.y"])


def test_generator_distributions():
    w = O.fill_blocks(O.Q8_0, 1, 4000).reshape(-1, 34)
    q = w[:, 2:].view(np.int8)
    assert q.min() == -127 and q.max() == 127
    d = w[:, :2].copy().view("<f2").astype(np.float32)
    assert d.min() >= 1e-3 * 0.999 and d.max() <= 1e-2 * 1.001
    w6 = O.fill_blocks(O.Q6_K, 2, 2000).reshape(-1, 210)
    sc = w6[:, 192:208].view(np.int8)
    assert sc.min() == -64 and sc.max() == 63
    x = O.fill_normal(3, 200000)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    # counter-based: a sub-range equals the slice of the full stream
    assert np.array_equal(O.fill_normal(3, 100, first=777), x[777:877])
    assert np.array_equal(O.fill_blocks(O.Q4_K, 9, 5, first_block=3),
                          O.fill_blocks(O.Q4_K, 9, 8)[3 * 144:])


def test_ffn_and_allreduce_semantics():
    dm, df, m = 256, 512, 2
    g = O.fill_weights(O.Q4_K, 1, dm, df)
    u = O.fill_weights(O.Q4_K, 2, dm, df)
    dn = O.fill_weights(O.Q4_K, 3, df, dm)
    x = O.fill_normal(4, m * dm).reshape(m, dm)
    y, h = O.ffn_swiglu(x, g, u, dn, m, dm, df, O.Q4_K, O.Q4_K, threads=2, want_h=True)
    gg = O.matmul_bt(x, g, m, dm, df, O.Q4_K)
    uu = O.matmul_bt(x, u, m, dm, df, O.Q4_K)
    silu = np.array([O.lib().rlxo_silu(float(v)) for v in gg.ravel()], np.float32).reshape(gg.shape)
    hh = (uu * silu).astype(np.float32)
    assert np.array_equal(h, hh)
    assert np.array_equal(y, O.matmul_bt(hh, dn, m, df, dm, O.Q4_K))
    parts = np.array([[1e8, 1.0], [1.0, 2.0], [-1e8, 3.0]], np.float32)
    out = O.allreduce_sum(parts)
    assert out[0] == np.float32(np.float32(np.float32(0 + 1e8) + 1.0) - 1e8) and out[1] == 6.0
