"""GGUF container reader and file -> device upload (include/rlxq_gguf.h).

The files are written here byte by byte, as the reference's own tests do (rlx-gguf/src/lib.rs:1149-1186,
1336-1362): magic, version, counts, metadata pairs, tensor table, padding to the alignment, data.
"""
import os
import struct

import numpy as np
import pytest

import rlx_b200 as R
from oracle import oracle as O

MAGIC = 0x46554747
F32, F16, Q4_0, Q8_0, Q2K, Q3K, Q4K, Q5K, Q6K, Q8K, BF16 = 0, 1, 2, 8, 10, 11, 12, 13, 14, 15, 30


def _s(text, version=3):
    b = text.encode()
    return struct.pack("<I" if version == 1 else "<Q", len(b)) + b


def write_gguf(path, tensors, meta=(), version=3, alignment=None):
    """tensors: [(name, dims (innermost first), ggml_type, bytes)], meta: [(key, type_id, packed_value_bytes)]."""
    cnt = "<I" if version == 1 else "<Q"
    meta = list(meta)
    if alignment is not None:
        meta.append(("general.alignment", 4, struct.pack("<I", alignment)))
    buf = struct.pack("<II", MAGIC, version) + struct.pack(cnt, len(tensors)) + struct.pack(cnt, len(meta))
    for key, ty, val in meta:
        buf += _s(key, version) + struct.pack("<I", ty) + val
    al = alignment or 32
    off, offsets = 0, []
    for _, _, _, data in tensors:
        offsets.append(off)
        off = (off + len(data) + al - 1) // al * al
    for (name, dims, ty, _), o in zip(tensors, offsets):
        buf += _s(name, version) + struct.pack("<I", len(dims))
        buf += b"".join(struct.pack(cnt, d) for d in dims) + struct.pack("<IQ", ty, o)
    buf += bytes((-len(buf)) % al)
    data_seg = bytearray(off)
    for (_, _, _, data), o in zip(tensors, offsets):
        data_seg[o:o + len(data)] = data
    with open(path, "wb") as f:
        f.write(buf + bytes(data_seg))


def test_reference_roundtrip_f32_v3(tmp_path):
    """rlx-gguf/src/lib.rs:1149-1178: one F32 tensor 'w' of four values, no metadata."""
    data = np.array([1.0, -2.0, 3.5, 0.0], np.float32)
    p = tmp_path / "a.gguf"
    write_gguf(p, [("w", [4], F32, data.tobytes())])
    f = R.GgufFile(p)
    assert f.version == 3 and len(f.tensors) == 1
    t = f.get("w")
    assert t.shape == (4,) and t.ggml_type == F32 and t.scheme == -1 and t.nbytes == 16
    assert np.array_equal(f.tensor_bytes("w").view(np.float32), data)


def test_reference_rejects_wrong_magic(tmp_path):
    """rlx-gguf/src/lib.rs:1180-1185."""
    p = tmp_path / "bad.gguf"
    p.write_bytes(bytes(16))
    with pytest.raises(R.RlxqError) as e:
        R.GgufFile(p)
    assert e.value.status == -10 and "not a GGUF file" in str(e.value)
    with pytest.raises(R.RlxqError):
        R.GgufFile(tmp_path / "missing.gguf")


def test_reference_metadata_roundtrip(tmp_path):
    """rlx-gguf/src/lib.rs:1336-1362: general.architecture = "llama", no tensors."""
    p = tmp_path / "m.gguf"
    write_gguf(p, [], meta=[("general.architecture", 8, _s("llama"))])
    f = R.GgufFile(p)
    assert f.meta_str("general.architecture") == "llama" and len(f.tensors) == 0
    with pytest.raises(R.RlxqError):
        f.meta_str("no.such.key")


@pytest.mark.parametrize("version", [1, 2, 3])
def test_tensor_table_metadata_kinds_and_alignment(tmp_path, version):
    k, n = 512, 6
    blobs = {
        "blk.0.ffn_up.weight": (Q4K, O.fill_weights(O.Q4_K, 1, k, n)),
        "blk.0.ffn_down.weight": (Q6K, O.fill_weights(O.Q6_K, 2, k, n)),
        "blk.0.attn_q.weight": (Q8_0, O.fill_weights(O.Q8_0, 3, k, n)),
        "blk.0.attn_k.weight": (Q4_0, O.fill_weights(O.Q4_0, 4, k, n)),
        "a.q5": (Q5K, O.fill_weights(O.Q5_K, 5, k, n)),
        "a.q8k": (Q8K, O.fill_weights(O.Q8_K, 6, k, n)),
        "a.q2": (Q2K, O.fill_weights(O.Q2_K, 7, k, n)),
        "a.q3": (Q3K, O.fill_weights(O.Q3_K, 8, k, n)),
        "a.q41": (3, O.fill_weights(O.Q4_1, 9, k, n)),
        "a.q50": (6, O.fill_weights(O.Q5_0, 10, k, n)),
        "a.q51": (7, O.fill_weights(O.Q5_1, 11, k, n)),
    }
    tensors = [(nm, [k, n], ty, w.tobytes()) for nm, (ty, w) in blobs.items()]
    tensors.append(("output_norm.weight", [k], F32, np.arange(k, dtype=np.float32).tobytes()))
    tensors.append(("half.weight", [8], BF16, bytes(16)))
    cnt = "<I" if version == 1 else "<Q"
    arr_u32 = struct.pack("<I", 4) + struct.pack(cnt, 3) + struct.pack("<III", 7, 8, 9)
    arr_str = struct.pack("<I", 8) + struct.pack(cnt, 2) + _s("a", version) + _s("bc", version)
    meta = [("general.architecture", 8, _s("llama", version)), ("llama.block_count", 4, struct.pack("<I", 32)),
            ("x.u8", 0, b"\x07"), ("x.i8", 1, b"\xff"), ("x.u16", 2, struct.pack("<H", 65535)),
            ("x.i16", 3, struct.pack("<h", -3)), ("x.i32", 5, struct.pack("<i", 12)), ("x.f32", 6, struct.pack("<f", 1.5)),
            ("x.bool", 7, b"\x01"), ("x.u64", 10, struct.pack("<Q", 1 << 40)), ("x.i64", 11, struct.pack("<q", -1)),
            ("x.f64", 12, struct.pack("<d", 2.5)), ("tokenizer.ggml.token_type", 9, arr_u32),
            ("tokenizer.ggml.tokens", 9, arr_str)]
    p = tmp_path / f"v{version}.gguf"
    write_gguf(p, tensors, meta=meta, version=version, alignment=64)
    f = R.GgufFile(p)
    assert f.version == version and f.alignment == 64 and f.data_start % 64 == 0
    assert list(f.keys()) == [t[0] for t in tensors]            # file order
    assert f.meta_str("general.architecture") == "llama" and f.meta_u64("llama.block_count") == 32
    assert f.meta_u64("x.u8") == 7 and f.meta_u64("x.u16") == 65535 and f.meta_u64("x.i32") == 12
    assert f.meta_u64("x.u64") == 1 << 40 and f.meta_u64("x.bool") == 1
    for key in ("x.i8", "x.i16", "x.i64", "x.f32", "x.f64", "tokenizer.ggml.tokens"):
        with pytest.raises(R.RlxqError):
            f.meta_u64(key)                                     # negative, float, or a skipped array
    want = {"blk.0.ffn_up.weight": 0, "blk.0.ffn_down.weight": 2, "blk.0.attn_q.weight": 7, "blk.0.attn_k.weight": 6,
            "a.q5": 1, "a.q8k": 3, "a.q2": 4, "a.q3": 5, "a.q41": 8, "a.q50": 9, "a.q51": 10, "output_norm.weight": -1,
            "half.weight": -1}
    for nm, (ty, w) in blobs.items():
        t = f.get(nm)
        assert t.shape == (k, n) and t.ggml_type == ty and t.scheme == want[nm] and t.nbytes == w.size
        assert t.offset % 64 == 0
        assert np.array_equal(f.tensor_bytes(nm), w)
        assert R.packed_bytes(t.scheme, k, n) == t.nbytes       # the slot rlxq_matmul expects
    assert f.get("half.weight").nbytes == 16 and f.get("nope") is None


def test_malformed_files_are_rejected(tmp_path):
    good = tmp_path / "g.gguf"
    w = O.fill_weights(O.Q4_K, 1, 256, 2)
    write_gguf(good, [("w", [256, 2], Q4K, w.tobytes())])
    raw = good.read_bytes()
    cases = {
        "version": raw[:4] + struct.pack("<I", 4) + raw[8:],                       # unsupported version
        "trunc": raw[:30],                                                         # header cut short
        "type": raw.replace(struct.pack("<IQ", Q4K, 0), struct.pack("<IQ", 33, 0)),  # ggml type the reference rejects
    }
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(data)
        with pytest.raises(R.RlxqError) as e:
            R.GgufFile(p)
        assert e.value.status == -10, name
    # a tensor that reaches past the end of the file, and one whose element count is not whole blocks
    short = tmp_path / "short.gguf"
    short.write_bytes(raw[:-10])
    f = R.GgufFile(short)
    with pytest.raises(R.RlxqError) as e:
        f.tensor_bytes("w")
    assert e.value.status == -2
    odd = tmp_path / "odd.gguf"
    write_gguf(odd, [("w", [100, 2], Q4K, bytes(288))])
    f = R.GgufFile(odd)
    assert f.get("w").nbytes == 0
    with pytest.raises(R.RlxqError):
        f.tensor_bytes("w")
    with pytest.raises(R.RlxqError):
        R.GgufFile(good).tensor_bytes("missing")


def test_header_sizes_that_wrap_64_bits_are_rejected(tmp_path):
    """A crafted count must not wrap the size arithmetic: 2^61 u64 elements are 2^64 bytes = 0 mod 2^64, and
    dimensions whose product wraps would record a small tensor.  Both are malformed headers."""
    w = O.fill_weights(O.Q4_K, 1, 256, 2)
    arr = tmp_path / "arr.gguf"
    write_gguf(arr, [("w", [256, 2], Q4K, w.tobytes())],
               meta=[("big", 9, struct.pack("<IQ", 10, 1 << 61))])                   # array of 2^61 u64
    dims = tmp_path / "dims.gguf"
    write_gguf(dims, [("w", [1 << 33, 1 << 33], Q4K, w.tobytes())])                  # 2^66 elements
    for p in (arr, dims):
        with pytest.raises(R.RlxqError) as e:
            R.GgufFile(p)
        assert e.value.status == -10, p.name


def test_a_repeated_tensor_name_is_listed_once(tmp_path):
    a = np.arange(4, dtype=np.float32)
    b = np.arange(4, 8, dtype=np.float32)
    p = tmp_path / "dup.gguf"
    write_gguf(p, [("t", [4], F32, a.tobytes()), ("t", [4], F32, b.tobytes())])
    f = R.GgufFile(p)
    assert list(f.keys()) == ["t"] and int(R._lib.lib.rlxq_gguf_tensor_count(f._h)) == 1
    assert np.array_equal(np.frombuffer(f.tensor_bytes("t"), np.float32), b)     # the later entry wins, as in a map insert


@pytest.mark.gpu
def test_upload_and_matmul_from_a_gguf_file(tmp_path):
    """File -> pinned staging -> device (several staging chunks), then the matmul on the uploaded bytes."""
    import torch
    from tests.helpers import assert_within_tolerance, bound, reference
    k, n = 4096, 9000                                  # 20.7 MB of Q4_K: more than one 16 MiB staging buffer
    w = O.fill_weights(O.Q4_K, 21, k, n)
    small = O.fill_weights(O.Q6_K, 22, 2048, 8)
    p = tmp_path / "model.gguf"
    write_gguf(p, [("blk.0.ffn_up.weight", [k, n], Q4K, w.tobytes()), ("tiny", [2048, 8], Q6K, small.tobytes())])
    f = R.GgufFile(p)
    wd = f.upload("blk.0.ffn_up.weight")
    sd = f.upload("tiny")
    torch.cuda.synchronize()
    assert np.array_equal(wd.cpu().numpy(), w) and np.array_equal(sd.cpu().numpy(), small)
    x = O.fill_normal(5, k).reshape(1, k)
    y = R.matmul(torch.from_numpy(x).cuda(), wd, f.get("blk.0.ffn_up.weight").scheme, n).cpu().numpy()
    R.device_status()
    assert_within_tolerance(y, reference(O.Q4_K, w, x, n), bound(O.Q4_K, w, x, n), tol=2e-5, what="gguf upload matmul")
    with pytest.raises(R.RlxqError):
        f.upload("nope")


@pytest.mark.gpu
def test_upload_of_a_large_tensor_uses_several_readers(tmp_path):
    """64 MiB and more: four threads read interleaved 8 MiB chunks; every byte must land where it belongs."""
    import torch
    rng = np.random.default_rng(3)
    big = rng.integers(0, 256, 75 * 144 * 7000 + 0, dtype=np.uint8)          # 75.6 MB = 525000 Q4_K blocks, ragged last chunk
    p = tmp_path / "big.gguf"
    write_gguf(p, [("pad", [32], F32, bytes(128)), ("big", [256 * 75, 7000], Q4K, big.tobytes())])
    f = R.GgufFile(p)
    assert f.get("big").nbytes == big.size
    for _ in range(2):                                                        # staging buffers are reused
        d = f.upload("big")
        torch.cuda.synchronize()
        assert np.array_equal(d.cpu().numpy(), big)
