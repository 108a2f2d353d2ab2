"""Tensor-parallel SwiGLU FFN over packed GGUF weights: one process per GPU.

`shard_plan` / `shard_weights` are host logic (rlxq_tp_shard_plan, rlxq_tp_slice_k_host).
`TensorParallelFFN` holds one rank's shards on its GPU and runs
    y = all_reduce_sum( down_r( up_r(x) * silu(gate_r(x)) ) )
with the per-rank part in the C-ABI call rlxq_tp_ffn_partial and the sum through the process
group the ranks already share (torch.distributed, NCCL on GPUs).  The reference has no device
collective (rlx-driver/src/collective.rs:79-128 emulates them on the host); the FFN is
rlx-flow/src/blocks/swiglu.rs:48-52.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib


class Shard(C.Structure):
    _fields_ = [("ffn_local", C.c_uint32), ("ffn_begin", C.c_uint32),
                ("gate_up_row_bytes", C.c_uint64), ("gate_up_byte_offset", C.c_uint64),
                ("gate_up_bytes", C.c_uint64), ("down_row_bytes_full", C.c_uint64),
                ("down_row_bytes_local", C.c_uint64), ("down_row_byte_offset", C.c_uint64),
                ("down_bytes", C.c_uint64)]


def shard_plan(scheme: int, d_model: int, d_ffn: int, world: int, rank: int) -> Shard:
    s = Shard()
    check(lib.rlxq_tp_shard_plan(int(scheme), d_model, d_ffn, world, rank, C.byref(s)))
    return s


def shard_weights(scheme: int, gate: np.ndarray, up: np.ndarray, down: np.ndarray, d_model: int, d_ffn: int,
                  world: int, rank: int) -> tuple[np.ndarray, np.ndarray, Shard]:
    """(gate_up_r, down_r, plan): the rank's gate rows followed by its up rows, and its k-slice of
    every row of down, as packed block bytes."""
    p = shard_plan(scheme, d_model, d_ffn, world, rank)
    a, b = p.gate_up_byte_offset, p.gate_up_byte_offset + p.gate_up_bytes
    gate_up = np.concatenate([gate[a:b], up[a:b]])
    down_r = np.empty(p.down_bytes, np.uint8)
    down = np.ascontiguousarray(down)
    check(lib.rlxq_tp_slice_k_host(int(scheme), down.ctypes.data, d_model, d_ffn, p.ffn_begin, p.ffn_local,
                                   down_r.ctypes.data))
    return gate_up, down_r, p


def ffn_workspace_bytes(scheme: int, m: int, d_model: int, ffn_local: int, x_dtype: int) -> int:
    out = C.c_size_t()
    check(lib.rlxq_tp_ffn_workspace_bytes(int(scheme), int(scheme), m, d_model, ffn_local, x_dtype, C.byref(out)))
    return out.value


class PeerAllReduce:
    """Sum all-reduce of small f32 tensors over NVLink peer memory (rlxq_tp_allreduce_sum): every rank
    allocates a buffer, the ranks exchange CUDA IPC handles through the process group and map each
    other's buffers.  `available` is False when the mapping could not be set up (the caller then keeps
    using the process group's all-reduce)."""

    MAX_ELEMS = 1 << 16            # 256 KiB of f32: the decode sizes; larger tensors go through the library

    def __init__(self, rank: int, world: int, group=None, max_elems: int = MAX_ELEMS):
        import torch
        import torch.distributed as dist
        self.rank, self.world, self.max_elems = rank, world, max_elems
        self.available = False
        self._own = None
        self._peers = {}
        if world < 2 or world > 8:
            return
        ok, handle = 1, bytes(64)
        try:
            own = C.c_void_p()
            check(lib.rlxq_tp_comm_alloc(max_elems, C.byref(own)))
            self._own = own.value
            hb = (C.c_uint8 * 64)()
            check(lib.rlxq_tp_ipc_export(self._own, hb))
            handle = bytes(hb)
        except Exception:
            ok = 0
        gathered = [None] * world
        dist.all_gather_object(gathered, (ok, handle), group=group)
        if all(g[0] for g in gathered):
            try:
                for r, (_, h) in enumerate(gathered):
                    if r == rank:
                        continue
                    p = C.c_void_p()
                    check(lib.rlxq_tp_ipc_open((C.c_uint8 * 64).from_buffer_copy(h), C.byref(p)))
                    self._peers[r] = p.value
            except Exception:
                ok = 0
        else:
            ok = 0
        flags = [None] * world
        dist.all_gather_object(flags, ok, group=group)       # all ranks use it, or none does
        self.available = all(flags)
        if self.available:
            ptrs = [self._own if r == rank else self._peers[r] for r in range(world)]
            self._bufs = (C.c_void_p * world)(*ptrs)
        torch.cuda.synchronize()
        if self.available:
            # One trial against the process group's all-reduce before anything relies on the mapping: a rank
            # that sees a timeout or a different sum votes it down and every rank falls back together.
            good = 1
            try:
                t = torch.arange(1024, dtype=torch.float32, device="cuda") * float(rank + 1)
                want = t.clone()
                dist.all_reduce(want, group=group)
                for _ in range(2):                      # both data slots
                    got = t.clone()
                    self(got)
                    torch.cuda.synchronize()
                    err = C.c_int(0)
                    if lib.rlxq_device_status(C.byref(err)) != 0 or not torch.equal(got, want):
                        good = 0
            except Exception:
                good = 0
            votes = [None] * world
            dist.all_gather_object(votes, good, group=group)
            if not all(votes):
                self.available = False

    def __call__(self, t) -> None:
        """In place: t <- sum over ranks of t, rank order, identical bits on every rank."""
        import torch
        assert self.available and t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
        with torch.cuda.device(t.device):
            check(lib.rlxq_tp_allreduce_sum(torch.cuda.current_stream().cuda_stream, self.rank, self.world, self._bufs,
                                            self.max_elems, t.data_ptr(), t.data_ptr(), t.numel()))

    def fits(self, t) -> bool:
        return self.available and t.numel() <= self.max_elems and t.numel() % 4 == 0

    def close(self) -> None:
        for p in self._peers.values():
            lib.rlxq_tp_ipc_close(p)
        self._peers = {}
        if self._own:
            lib.rlxq_tp_comm_free(self._own)
            self._own = None
        self.available = False


class TensorParallelGroup:
    """The whole layer driven from this process: rlxq_tp_create / rlxq_tp_ffn_load / rlxq_tp_ffn_run / rlxq_tp_destroy.
    Host buffers in, host buffers out; the library owns streams, shards, scratch and communicators."""

    def __init__(self, devices=None, ndev: int | None = None):
        devs = list(devices) if devices is not None else list(range(ndev or 1))
        arr = (C.c_int * len(devs))(*devs)
        h = C.c_void_p()
        check(lib.rlxq_tp_create(len(devs), arr, C.byref(h)))
        self._h = h.value
        self.world = int(lib.rlxq_tp_world(self._h))
        self.d_model = self.d_ffn = 0

    def load(self, scheme: int, gate: np.ndarray, up: np.ndarray, down: np.ndarray, d_model: int, d_ffn: int) -> None:
        g, u, d = (np.ascontiguousarray(a, np.uint8) for a in (gate, up, down))
        check(lib.rlxq_tp_ffn_load(self._h, int(scheme), g.ctypes.data, u.ctypes.data, d.ctypes.data, d_model, d_ffn))
        self.d_model, self.d_ffn = d_model, d_ffn

    def run(self, x: np.ndarray, bf16: bool = False) -> np.ndarray:
        """x: [m, d_model] float32, or uint16 bf16 bit patterns with bf16=True; returns [m, d_model] float32."""
        x = np.ascontiguousarray(x, np.uint16 if bf16 else np.float32)
        m = x.shape[0]
        y = np.empty((m, self.d_model), np.float32)
        check(lib.rlxq_tp_ffn_run(self._h, x.ctypes.data, 1 if bf16 else 0, m, y.ctypes.data))
        return y

    def status(self) -> None:
        code = C.c_int(0)
        check(lib.rlxq_tp_status(self._h, C.byref(code)))

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.rlxq_tp_destroy(h)

    __del__ = close


class TensorParallelFFN:
    def __init__(self, scheme: int, d_model: int, d_ffn: int, rank: int = 0, world: int = 1, device=None,
                 group=None):
        import torch
        self.torch = torch
        self.scheme, self.d_model, self.d_ffn = int(scheme), d_model, d_ffn
        self.rank, self.world, self.group = rank, world, group
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.plan = shard_plan(scheme, d_model, d_ffn, world, rank)
        self.gate_up = self.down = None
        self._ws = {}
        self.peer_reduce = None         # set by enable_peer_allreduce()

    def enable_peer_allreduce(self) -> bool:
        """Use the one-shot NVLink all-reduce for partials of up to 64 K values (decode); a collective over
        the group, so every rank must call it.  Returns whether it is in use."""
        if self.world > 1 and self.peer_reduce is None:
            self.peer_reduce = PeerAllReduce(self.rank, self.world, self.group)
        return bool(self.peer_reduce and self.peer_reduce.available)

    def load(self, gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> None:
        """Full packed weights in host memory -> this rank's shards on its GPU (one upload each)."""
        gu, dn, _ = shard_weights(self.scheme, gate, up, down, self.d_model, self.d_ffn, self.world, self.rank)
        self.gate_up = self.torch.from_numpy(gu).to(self.device)
        self.down = self.torch.from_numpy(dn).to(self.device)

    def load_shards(self, gate_up: np.ndarray, down: np.ndarray) -> None:
        self.gate_up = self.torch.from_numpy(gate_up).to(self.device)
        self.down = self.torch.from_numpy(down).to(self.device)

    def _workspace(self, m: int, x_dtype: int):
        key = (m, x_dtype)
        if key not in self._ws:
            need = ffn_workspace_bytes(self.scheme, m, self.d_model, self.plan.ffn_local, x_dtype)
            self._ws[key] = self.torch.empty(need + 256, dtype=self.torch.uint8, device=self.device)
        return self._ws[key]

    def partial(self, x, out=None):
        """This rank's f32 partial [m, d_model] (no communication)."""
        torch = self.torch
        assert x.is_cuda and x.dim() == 2 and x.shape[1] == self.d_model and x.is_contiguous()
        m = x.shape[0]
        dt = 0 if x.dtype == torch.float32 else 1
        if out is None:
            out = torch.empty((m, self.d_model), dtype=torch.float32, device=x.device)
        ws = self._workspace(m, dt)
        base = (ws.data_ptr() + 255) // 256 * 256
        with torch.cuda.device(x.device):
            check(lib.rlxq_tp_ffn_partial(torch.cuda.current_stream().cuda_stream, self.scheme, self.scheme,
                                          x.data_ptr(), dt, self.gate_up.data_ptr(), self.down.data_ptr(),
                                          out.data_ptr(), m, self.d_model, self.plan.ffn_local, base,
                                          ws.numel() - (base - ws.data_ptr())))
        return out

    def forward(self, x, out=None):
        torch = self.torch
        m = x.shape[0]
        pr = self.peer_reduce
        if self.world > 1 and pr is not None and pr.available and m * self.d_model <= pr.max_elems and (m * self.d_model) % 4 == 0:
            # rlxq_tp_ffn_step: the partial and the peer-memory all-reduce behind one call (option tp_fused = 1: the down
            # projection pushes its tiles to the peers and finishes the sum itself)
            assert x.is_cuda and x.dim() == 2 and x.shape[1] == self.d_model and x.is_contiguous()
            dt = 0 if x.dtype == torch.float32 else 1
            if out is None:
                out = torch.empty((m, self.d_model), dtype=torch.float32, device=x.device)
            ws = self._workspace(m, dt)
            base = (ws.data_ptr() + 255) // 256 * 256
            with torch.cuda.device(x.device):
                check(lib.rlxq_tp_ffn_step(torch.cuda.current_stream().cuda_stream, self.scheme, self.scheme,
                                           x.data_ptr(), dt, self.gate_up.data_ptr(), self.down.data_ptr(),
                                           out.data_ptr(), m, self.d_model, self.plan.ffn_local, base,
                                           ws.numel() - (base - ws.data_ptr()), self.rank, self.world, pr._bufs,
                                           pr.max_elems))
            return out
        y = self.partial(x, out)
        if self.world > 1:
            if pr is not None and pr.fits(y):
                pr(y)
            else:
                import torch.distributed as dist
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
