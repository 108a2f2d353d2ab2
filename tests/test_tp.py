"""Tensor-parallel FFN: shard planner and k-slicing on the CPU (incl. a world-size-2 gloo run whose
per-rank arithmetic is the oracle), and the per-rank CUDA path on one GPU."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as O
from rlx_b200 import tp
import rlx_b200 as R


def _weights(dm, df, seed=1):
    return (O.fill_weights(O.Q4_K, seed, dm, df), O.fill_weights(O.Q4_K, seed + 1, dm, df),
            O.fill_weights(O.Q4_K, seed + 2, df, dm))


def _oracle_partial(x, gate_up, down, dm, f):
    m = x.shape[0]
    gu = O.matmul_bt_mt(x, gate_up, m, dm, 2 * f, O.Q4_K)
    g, u = gu[:, :f], gu[:, f:]
    with np.errstate(over="ignore"):
        silu = (g / (1.0 + np.exp(-g.astype(np.float32)))).astype(np.float32)
    h = (u * silu).astype(np.float32)
    return O.matmul_bt_mt(h, down, m, f, dm, O.Q4_K)


def test_shard_plan_geometry():
    p = tp.shard_plan(O.Q4_K, 8192, 28672, 8, 3)
    assert (p.ffn_local, p.ffn_begin) == (3584, 10752)
    assert p.gate_up_row_bytes == 4608 and p.gate_up_bytes == 3584 * 4608
    assert p.down_row_bytes_local == 14 * 144 and p.down_row_byte_offset == 42 * 144
    assert p.down_bytes == 8192 * 2016
    with pytest.raises(R.RlxqError):
        tp.shard_plan(O.Q4_K, 8192, 28672, 3, 0)         # 28672 / 3 is not whole 256-weight groups
    with pytest.raises(R.RlxqError):
        tp.shard_plan(O.Q4_K, 8192, 28672, 4, 4)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_shards_partition_the_weights_and_sum_to_the_full_ffn(world):
    dm, df, m = 512, 2048, 2
    gate, up, down = _weights(dm, df)
    x = O.fill_normal(9, m * dm).reshape(m, dm)
    y_ref = O.ffn_swiglu(x, gate, up, down, m, dm, df, O.Q4_K, O.Q4_K)
    parts, covered = [], np.zeros(len(down), bool)
    for r in range(world):
        gu, dn, p = tp.shard_weights(O.Q4_K, gate, up, down, dm, df, world, r)
        # the k-slice of down decodes to the matching columns of the full matrix
        full = O.dequant(O.Q4_K, down, dm * df).reshape(dm, df)
        assert np.array_equal(O.dequant(O.Q4_K, dn, dm * p.ffn_local).reshape(dm, p.ffn_local),
                              full[:, p.ffn_begin:p.ffn_begin + p.ffn_local])
        parts.append(_oracle_partial(x, gu, dn, dm, p.ffn_local))
    y = O.allreduce_sum(np.stack(parts))
    wn = O.row_norms(O.Q4_K, down, df, dm)
    h = O.ffn_swiglu(x, gate, up, down, m, dm, df, O.Q4_K, O.Q4_K, want_h=True)[1]
    bnd = np.sqrt((h.astype(np.float64) ** 2).sum(1))[:, None] * wn[None, :]
    assert np.max(np.abs(y - y_ref) / bnd) < 1e-5        # only the f32 summation order differs


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _gloo_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dm, df, m = 512, 2048, 1
    gate, up, down = _weights(dm, df)
    x = O.fill_normal(9, m * dm).reshape(m, dm)
    gu, dn, p = tp.shard_weights(O.Q4_K, gate, up, down, dm, df, world, rank)
    y = torch.from_numpy(_oracle_partial(x, gu, dn, dm, p.ffn_local))
    dist.all_reduce(y)                                    # the exchange step of the path
    if rank == 0:
        q.put(y.numpy())
    dist.destroy_process_group()


def test_world_size_two_gloo_all_reduce():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), _free_port()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    y = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    dm, df = 512, 2048
    gate, up, down = _weights(dm, df)
    x = O.fill_normal(9, dm).reshape(1, dm)
    y_ref = O.ffn_swiglu(x, gate, up, down, 1, dm, df, O.Q4_K, O.Q4_K)
    assert np.max(np.abs(y - y_ref)) < 1e-4 * np.max(np.abs(y_ref))


@pytest.mark.gpu
@pytest.mark.parametrize("m,world", [(1, 1), (1, 2), (2, 4), (8, 2), (64, 2)])
def test_per_rank_cuda_partials_sum_to_the_oracle_ffn(m, world):
    """All ranks' shards run one after the other on one GPU; partials are summed in rank order."""
    import torch
    dm, df = 1024, 4096
    gate, up, down = _weights(dm, df, seed=4)
    x = O.fill_normal(11, m * dm).reshape(m, dm)
    xb = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x)).reshape(m, dm)
    xd = torch.from_numpy(xb).cuda().to(torch.bfloat16)
    parts = []
    for r in range(world):
        ffn = tp.TensorParallelFFN(O.Q4_K, dm, df, rank=r, world=world)
        ffn.load(gate, up, down)
        parts.append(ffn.partial(xd).cpu().numpy())
    R.device_status()
    y = O.allreduce_sum(np.stack(parts))
    y_ref, h = O.ffn_swiglu(xb, gate, up, down, m, dm, df, O.Q4_K, O.Q4_K, want_h=True)
    bnd = np.sqrt((h.astype(np.float64) ** 2).sum(1))[:, None] * O.row_norms(O.Q4_K, down, df, dm)[None, :]
    assert np.max(np.abs(y - y_ref) / bnd) < 1e-3        # the path's bound, both layers chained


# ------------------------------------------------------------------ configuration 3 at its real shape
_CFG3 = {}


def _cfg3():
    """The 70B-shaped FFN of configuration 3 (d_model 8192, d_ffn 28672, Q4_K), generated once per test run
    with the oracle results the cases share: the full FFN for one token and for four sampled rows of a
    256-token batch."""
    if not _CFG3:
        dm, df = 8192, 28672
        gate, up, down = _weights(dm, df, seed=2000)
        wn = O.row_norms(O.Q4_K, down, df, dm)
        x256 = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(78, 256 * dm))).reshape(256, dm)
        rows = np.array([0, 85, 170, 255])
        ref = {}
        for m, xs in ((1, x256[:1]), (256, x256[rows])):
            y, h = O.ffn_swiglu(np.ascontiguousarray(xs), gate, up, down, xs.shape[0], dm, df, O.Q4_K, O.Q4_K, want_h=True)
            ref[m] = (y, np.sqrt((h.astype(np.float64) ** 2).sum(1))[:, None] * wn[None, :])
        _CFG3.update(dm=dm, df=df, gate=gate, up=up, down=down, x=x256, rows=rows, ref=ref)
    return _CFG3


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("m", [1, 256])
def test_cfg3_real_shape_shards_sum_to_the_oracle_ffn(m, world):
    """Q4_K, d_model 8192, d_ffn 28672, one token and 256 tokens, split 1 / 2 / 4 / 8 ways: every rank's shard
    runs through rlxq_tp_ffn_partial on this GPU, the partials are summed in rank order
    (rlx-driver/src/collective.rs:107-127) and compared with the oracle FFN -- every output for one token,
    four sampled token rows (rows are independent) for 256.  The 8-way down projection has k = 3584."""
    import torch
    c = _cfg3()
    dm, df = c["dm"], c["df"]
    x = c["x"][:m]
    xd = torch.from_numpy(np.ascontiguousarray(x)).cuda().to(torch.bfloat16)
    parts = []
    for r in range(world):
        ffn = tp.TensorParallelFFN(O.Q4_K, dm, df, rank=r, world=world)
        ffn.load(c["gate"], c["up"], c["down"])
        parts.append(ffn.partial(xd).cpu().numpy())
        del ffn
    R.device_status()
    y = O.allreduce_sum(np.stack(parts))
    y_ref, bnd = c["ref"][m]
    sel = np.arange(1) if m == 1 else c["rows"]
    assert np.isfinite(y).all()
    assert np.max(np.abs(y[sel].astype(np.float64) - y_ref) / bnd) < 1e-3   # the path's bound, both layers chained


# ------------------------------------------------------------------ peer-memory all-reduce (needs two GPUs)
def _peer_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        pr = tp.PeerAllReduce(rank, world)
        assert pr.available, "peer mapping could not be set up"
        results = {}
        for step, n in enumerate((8192, 16, 65536, 8192)):
            part = O.fill_normal(100 * step + rank, n)
            t = torch.from_numpy(part).cuda()
            pr(t)
            torch.cuda.synchronize()
            results[f"eager{step}"] = t.cpu().numpy()
        # captured once, replayed: the step counter lives on the device
        part = O.fill_normal(900 + rank, 8192)
        src = torch.from_numpy(part).cuda()
        t = torch.empty_like(src)
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            t.copy_(src); pr(t)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                t.copy_(src)
                pr(t)
                t.mul_(1.0)
        for rep in range(3):
            g.replay()
            torch.cuda.synchronize()
            results[f"graph{rep}"] = t.cpu().numpy()
        R.device_status()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
        dist.barrier()
        pr.close()
    finally:
        os._exit(0)      # tearing the NCCL group down after graph capture can block for minutes


@pytest.mark.gpu
def test_peer_memory_all_reduce_two_gpus(tmp_path):
    """rlxq_tp_allreduce_sum on two GPUs: bit-identical on both ranks and equal to the sum in rank order
    (rlx-driver/src/collective.rs:107-127), eager and through a replayed CUDA graph."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    for step, n in enumerate((8192, 16, 65536, 8192)):
        parts = np.stack([O.fill_normal(100 * step + r, n) for r in range(world)])
        want = O.allreduce_sum(parts)
        for r in range(world):
            assert np.array_equal(got[r][f"eager{step}"], want), (step, r)
    parts = np.stack([O.fill_normal(900 + r, 8192) for r in range(world)])
    want = O.allreduce_sum(parts)
    for rep in range(3):
        for r in range(world):
            assert np.array_equal(got[r][f"graph{rep}"], want), (rep, r)


# ------------------------------------------------------------------ a bounded wait that runs out (one GPU)
@pytest.mark.gpu
def test_peer_all_reduce_wait_runs_out_and_the_context_stays_usable():
    """rlxq_tp_allreduce_sum with world = 2 where the "peer" is a second buffer on the same GPU that nobody writes:
    with a short poll limit the kernel gives up, leaves dst alone and records 40 + peer rank; rlxq_device_status turns
    that into RLXQ_E_TIMEOUT, and the next call (the peer's tagged words now written by the host, as a live peer would
    push them) completes normally.  Nothing faults and nothing hangs: the wait is a counted loop of plain loads."""
    import ctypes as C
    import torch
    from rlx_b200._lib import lib
    from tests.helpers import copy_to_device
    n = 1024
    bufs = []
    for _ in range(2):
        p = C.c_void_p()
        assert lib.rlxq_tp_comm_alloc(n, C.byref(p)) == 0
        bufs.append(p.value)
    arr = (C.c_void_p * 2)(*bufs)
    src = torch.from_numpy(O.fill_normal(1, n)).cuda()
    dst = torch.full((n,), 7.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    code = C.c_int(0)
    assert lib.rlxq_device_status(C.byref(code)) == 0          # clean before
    R.set_option("tp_spin_limit", 1 << 12)
    try:
        assert lib.rlxq_tp_allreduce_sum(stream, 0, 2, arr, n, src.data_ptr(), dst.data_ptr(), n) == 0
        st = lib.rlxq_device_status(C.byref(code))
        assert st == -8 and code.value == 41, (st, code.value)  # RLXQ_E_TIMEOUT, waiting for rank 1
        assert torch.all(dst == 7.0)                             # the sum never ran
        assert lib.rlxq_device_status(C.byref(code)) == 0 and code.value == 0   # reported once, then clear
        # now play the peer from the host, as a live peer would push: rank 1's partial as 8-byte words {value, step tag}
        # into rank 1's slot of rank 0's buffer ([header][parity][rank slot of n words, 8 of them]).  The call above
        # was step 1 of every part, the next is step 2: parity 0, tag 0x80000002.
        peer = O.fill_normal(2, n)
        words = np.empty((n, 2), np.uint32)
        words[:, 0] = peer.view(np.uint32)
        words[:, 1] = 0x80000002
        copy_to_device(bufs[0] + 1024 + (0 * 8 + 1) * n * 8, words.ravel())
        assert lib.rlxq_tp_allreduce_sum(stream, 0, 2, arr, n, src.data_ptr(), dst.data_ptr(), n) == 0
        assert lib.rlxq_device_status(C.byref(code)) == 0 and code.value == 0
        want = O.allreduce_sum(np.stack([src.cpu().numpy(), peer]))
        assert np.array_equal(dst.cpu().numpy(), want)
    finally:
        R.set_option("tp_spin_limit", 1 << 24)
        for b in bufs:
            lib.rlxq_tp_comm_free(b)


# ------------------------------------------------------------------ the C-ABI lifecycle: create / load / run / destroy
def test_tp_create_without_a_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(R.RlxqError) as e:
        tp.TensorParallelGroup(ndev=1)
    assert e.value.status == -6                      # RLXQ_E_CUDA: there is no CPU path behind this entry point
    with pytest.raises(R.RlxqError) as e:
        tp.TensorParallelGroup(ndev=9)
    assert e.value.status == -10


def _group_case(world, dm, df, ms):
    gate, up, down = _weights(dm, df, seed=40)
    g = tp.TensorParallelGroup(ndev=world)
    assert g.world == world
    g.load(O.Q4_K, gate, up, down, dm, df)
    wn = O.row_norms(O.Q4_K, down, df, dm)
    for m in ms:
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(50 + m, m * dm))).reshape(m, dm)
        for bf16 in (False, True):
            y = g.run(O.f32_to_bf16_bits(x).reshape(m, dm) if bf16 else x, bf16=bf16)
            g.status()
            y_ref, h = O.ffn_swiglu(x, gate, up, down, m, dm, df, O.Q4_K, O.Q4_K, want_h=True)
            bnd = np.sqrt((h.astype(np.float64) ** 2).sum(1))[:, None] * wn[None, :]
            assert np.isfinite(y).all()
            assert np.max(np.abs(y - y_ref) / bnd) < 1e-3, (world, m, bf16)
        y2 = g.run(x)                                 # the same bits from run to run
        assert np.array_equal(y2, g.run(x))
    g.close()


@pytest.mark.gpu
def test_tp_lifecycle_one_device():
    """rlxq_tp_create / ffn_load / ffn_run / destroy with a single device: host buffers in and out, no collective."""
    _group_case(1, 1024, 4096, (1, 2, 16))


@pytest.mark.gpu
def test_tp_lifecycle_two_devices():
    """Two GPUs driven from this process: one token and 64 tokens take the peer-memory all-reduce (m * d_model up to
    65536 values), 128 tokens NCCL's."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _group_case(2, 1024, 4096, (1, 64, 128))


# ------------------------------------------------------------------ the step with the exchange inside the down projection
@pytest.mark.gpu
@pytest.mark.parametrize("dm,df,m", [(1024, 4096, 1), (1024, 4096, 2), (2048, 8192, 4), (4096, 14336, 8)])
def test_ffn_step_pushes_and_sums_inside_the_down_projection(dm, df, m):
    """rlxq_tp_ffn_step with world = 1 (the one rank is its own peer: it pushes its tiles into its own exchange buffer,
    counts its CTAs in and sums one slot): the same bits as rlxq_tp_ffn_partial, one launch fewer than partial +
    all-reduce, step after step on the same buffers (the two sets of slots alternate), fused and not."""
    import ctypes as C
    import torch
    from rlx_b200._lib import lib
    s = O.Q4_K
    gate, up, down = _weights(dm, df, seed=70 + m)
    f = tp.TensorParallelFFN(s, dm, df, rank=0, world=1, device=torch.device("cuda", 0))
    f.load(gate, up, down)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(71 + m, m * dm))).reshape(m, dm)
    xd = torch.from_numpy(x).cuda()
    want = f.partial(xd).cpu().numpy()
    buf = C.c_void_p()
    assert lib.rlxq_tp_comm_alloc(65536, C.byref(buf)) == 0
    bufs = (C.c_void_p * 1)(buf.value)
    ws = f._workspace(m, 0)
    base = (ws.data_ptr() + 255) // 256 * 256
    stream = torch.cuda.current_stream().cuda_stream
    counts = {}
    try:
        for fused in (1, 0, 1):
            R.set_option("tp_fused", fused)
            for _ in range(3):
                y = torch.full((m, dm), 9.0, device="cuda")
                before = R.launch_count()
                rc = lib.rlxq_tp_ffn_step(stream, s, s, xd.data_ptr(), 0, f.gate_up.data_ptr(), f.down.data_ptr(),
                                          y.data_ptr(), m, dm, f.plan.ffn_local, base, ws.numel() - (base - ws.data_ptr()),
                                          0, 1, bufs, 65536)
                assert rc == 0
                launches = R.launch_count() - before
                R.device_status()
                assert np.array_equal(y.cpu().numpy(), want), (fused, m)
            counts[fused] = launches
        assert counts[1] == counts[0] - 1          # the pushing down projection replaces GEMV + all-reduce
    finally:
        R.set_option("tp_fused", 0)
        lib.rlxq_tp_comm_free(buf.value)
    y_ref, h = O.ffn_swiglu(x, gate, up, down, m, dm, df, s, s, want_h=True)
    wn = O.row_norms(s, down, df, dm)
    bnd = np.sqrt((h.astype(np.float64) ** 2).sum(1))[:, None] * wn[None, :]
    assert np.max(np.abs(want - y_ref) / bnd) < 1e-3
