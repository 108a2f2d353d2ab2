"""Python face of the rlxq library.

Two layers, both thin wrappers over the C ABI:

* `dequant_f32` / `matmul` — the device-pointer entry points (`rlxq_dequant_f32`, `rlxq_matmul`)
  applied to torch CUDA tensors.  torch only owns the memory and the stream.
* `Graph`, `Session`, `CompiledGraph`, `Device`, `DType`, `QuantScheme` — the reference's
  user-facing contract for this path (rlx-runtime/tests/dequant_matmul_gguf.rs:212-227):
  build a graph with `input`, `param` and `dequant_matmul_packed`, `Session(Device.Cuda).compile`,
  `set_param_typed(name, bytes, DType.U8)`, `run([("x", x)])`.  Host arrays in, host arrays out.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Sequence

import numpy as np

from ._lib import RlxqError, check, lib


class QuantScheme(enum.IntEnum):
    """The GGUF schemes of rlx_ir::quant::QuantScheme (is_gguf), with the ids of include/rlxq.h
    (0..5 are the reference's own, rlx-cuda/src/gguf_host.rs:24-34)."""
    GgufQ4K = 0
    GgufQ5K = 1
    GgufQ6K = 2
    GgufQ8K = 3
    GgufQ2K = 4
    GgufQ3K = 5
    GgufQ4_0 = 6
    GgufQ8_0 = 7
    # container types the reference decodes at load time only (no QuantScheme of its own names them)
    GgufQ4_1 = 8
    GgufQ5_0 = 9
    GgufQ5_1 = 10

    def gguf_block_size(self) -> int:
        return scheme_geometry(self)[0]

    def gguf_block_bytes(self) -> int:
        return scheme_geometry(self)[1]


class DType(enum.IntEnum):
    F32 = 0
    BF16 = 1
    U8 = 100   # host-side tag for packed weights; never an activation dtype


class Device(enum.Enum):
    Cuda = "cuda"


def scheme_geometry(scheme: int) -> tuple[int, int]:
    e, b = C.c_uint32(), C.c_uint32()
    check(lib.rlxq_scheme_geometry(int(scheme), C.byref(e), C.byref(b)))
    return e.value, b.value


def packed_bytes(scheme: int, k: int, n: int) -> int:
    out = C.c_uint64()
    check(lib.rlxq_packed_bytes(int(scheme), k, n, C.byref(out)))
    return out.value


def workspace_bytes(scheme: int, m: int, k: int, n: int, x_dtype: int = 0, y_dtype: int = 0) -> int:
    out = C.c_size_t()
    check(lib.rlxq_workspace_bytes(int(scheme), m, k, n, int(x_dtype), int(y_dtype), C.byref(out)))
    return out.value


def set_option(key: str, value: int) -> None:
    check(lib.rlxq_set_option(key.encode(), int(value)))


def get_option(key: str) -> int:
    v = C.c_int64()
    check(lib.rlxq_get_option(key.encode(), C.byref(v)))
    return v.value


def launch_count() -> int:
    return int(lib.rlxq_launch_count())


def device_status() -> None:
    """Synchronise and raise if a kernel gave up on a bounded wait."""
    code = C.c_int()
    check(lib.rlxq_device_status(C.byref(code)))


# ------------------------------------------------------------------ device-pointer layer
def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("rlx_b200 needs a CUDA device; there is no CPU path")
    return torch


def _stream_ptr(torch) -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t, torch) -> int:
    if t.dtype == torch.float32:
        return int(DType.F32)
    if t.dtype == torch.bfloat16:
        return int(DType.BF16)
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


def dequant_f32(w_blocks, scheme: int, n_elems: int, out=None):
    """rlxq_dequant_f32 on a torch uint8 CUDA tensor of raw blocks."""
    torch = _torch()
    assert w_blocks.is_cuda and w_blocks.dtype == torch.uint8 and w_blocks.is_contiguous()
    if out is None:
        out = torch.empty(n_elems, dtype=torch.float32, device=w_blocks.device)
    with torch.cuda.device(w_blocks.device):
        check(lib.rlxq_dequant_f32(_stream_ptr(torch), int(scheme), w_blocks.data_ptr(), n_elems,
                                   out.data_ptr()))
    return out


def matmul(x, w_blocks, scheme: int, n: int, out=None, out_dtype=None, workspace=None):
    """rlxq_matmul: y[m,n] = x[m,k] . W^T for torch CUDA tensors (x f32 or bf16)."""
    torch = _torch()
    assert x.is_cuda and x.dim() == 2 and x.is_contiguous()
    assert w_blocks.is_cuda and w_blocks.dtype == torch.uint8 and w_blocks.is_contiguous()
    m, k = x.shape
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or torch.float32, device=x.device)
    need = workspace_bytes(scheme, m, k, n, _dt(x, torch), _dt(out, torch))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.rlxq_matmul(_stream_ptr(torch), int(scheme), x.data_ptr(), _dt(x, torch),
                              w_blocks.data_ptr(), out.data_ptr(), _dt(out, torch), m, k, n,
                              workspace.data_ptr() if need else None, need))
    return out


class ChainLayer(C.Structure):
    """rlxq_chain_layer: one layer of rlxq_matmul_chain."""
    _fields_ = [("w_blocks", C.c_void_p), ("k", C.c_uint32), ("n", C.c_uint32), ("swiglu", C.c_uint32)]


def matmul_chain(x, layers, scheme: int, out=None, out_dtype=None, workspace=None):
    """rlxq_matmul_chain: `layers` is a list of (w_blocks, n) or (w_blocks, n, swiglu) in order; layer i takes the
    previous layer's output (or, with swiglu, the product up * silu(gate) of its [gate | up] halves).  CUDA tensors."""
    torch = _torch()
    assert x.is_cuda and x.dim() == 2 and x.is_contiguous()
    m, width = x.shape
    arr = (ChainLayer * len(layers))()
    for i, ly in enumerate(layers):
        w, n = ly[0], int(ly[1])
        sw = int(bool(ly[2])) if len(ly) > 2 else 0
        assert w.is_cuda and w.dtype == torch.uint8 and w.is_contiguous()
        k = width // 2 if sw else width
        arr[i] = ChainLayer(w.data_ptr(), k, n, sw)
        width = n
    if out is None:
        out = torch.empty((m, width), dtype=out_dtype or torch.float32, device=x.device)
    need = C.c_size_t()
    check(lib.rlxq_chain_workspace_bytes(int(scheme), C.cast(arr, C.c_void_p), len(layers), m, _dt(x, torch), C.byref(need)))
    if workspace is None or workspace.numel() < need.value:
        workspace = torch.empty(max(need.value, 256), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.rlxq_matmul_chain(_stream_ptr(torch), int(scheme), C.cast(arr, C.c_void_p), len(layers), x.data_ptr(),
                                    _dt(x, torch), out.data_ptr(), _dt(out, torch), m, workspace.data_ptr(), workspace.numel()))
    return out


def chain_workspace_bytes(scheme: int, layers, m: int, x_dtype: int = 0) -> int:
    """layers: list of (k, n, swiglu)."""
    arr = (ChainLayer * len(layers))()
    for i, (k, n, sw) in enumerate(layers):
        arr[i] = ChainLayer(None, k, n, int(bool(sw)))
    need = C.c_size_t()
    check(lib.rlxq_chain_workspace_bytes(int(scheme), C.cast(arr, C.c_void_p), len(layers), m, int(x_dtype), C.byref(need)))
    return need.value


# ------------------------------------------------------------------ MoE expert stacks
def grouped_matmul(x, w_blocks, expert_idx, scheme: int, n: int, num_experts: int, out=None, out_dtype=None,
                   workspace=None):
    """Op::DequantGroupedMatMul: y[i] = x[i] . W_e^T with e = expert_idx[i] (f32-encoded, as the reference's
    graph input); w_blocks holds num_experts packed [n, k] slabs back to back.  CUDA tensors in and out."""
    torch = _torch()
    assert x.is_cuda and x.dim() == 2 and x.is_contiguous()
    assert w_blocks.is_cuda and w_blocks.dtype == torch.uint8 and w_blocks.is_contiguous()
    assert expert_idx.is_cuda and expert_idx.dtype == torch.float32 and expert_idx.is_contiguous()
    m, k = x.shape
    assert expert_idx.numel() == m
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or torch.float32, device=x.device)
    need = C.c_size_t()
    check(lib.rlxq_grouped_workspace_bytes(int(scheme), m, k, n, num_experts, C.byref(need)))
    if workspace is None or workspace.numel() < need.value:
        workspace = torch.empty(max(need.value, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.rlxq_grouped_matmul(_stream_ptr(torch), int(scheme), x.data_ptr(), _dt(x, torch), w_blocks.data_ptr(),
                                      expert_idx.data_ptr(), out.data_ptr(), _dt(out, torch), m, k, n, num_experts,
                                      workspace.data_ptr(), need.value))
    return out


# ------------------------------------------------------------------ tied LM head
LM_MAX_CAP = 64


def lm_head_workspace_bytes(scheme: int, n_embd: int, n_vocab: int, x_dtype: int = 0, cap: int = 1) -> int:
    out = C.c_size_t()
    check(lib.rlxq_lm_head_workspace_bytes(int(scheme), n_embd, n_vocab, x_dtype, cap, C.byref(out)))
    return out.value


def gguf_tied_lm_topk(hidden, w_bytes, n_embd: int, n_vocab: int, scheme: int, cap: int, exact: bool = True,
                      workspace=None):
    """rlx_cpu::lm_head::gguf_tied_lm_topk (rlx-cpu/src/lm_head.rs:172-199) on the GPU: the `cap` best
    (token id, logit) pairs, best first.  hidden: CUDA tensor [n_embd], f32 or bf16; w_bytes: CUDA uint8
    tensor holding the packed embedding [n_vocab, n_embd].  Returns two CUDA tensors: int32 token ids (-1 where
    fewer than cap rows could be chosen) and f32 logits."""
    torch = _torch()
    assert hidden.is_cuda and hidden.is_contiguous() and hidden.numel() == n_embd
    assert w_bytes.is_cuda and w_bytes.dtype == torch.uint8 and w_bytes.is_contiguous()
    cap = max(1, min(cap, n_vocab))          # the reference clamps the same way
    need = lm_head_workspace_bytes(scheme, n_embd, n_vocab, _dt(hidden, torch), cap)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=hidden.device)
    idx = torch.empty(cap, dtype=torch.int32, device=hidden.device)
    val = torch.empty(cap, dtype=torch.float32, device=hidden.device)
    with torch.cuda.device(hidden.device):
        check(lib.rlxq_lm_head_topk(_stream_ptr(torch), int(scheme), hidden.data_ptr(), _dt(hidden, torch),
                                    w_bytes.data_ptr(), n_embd, n_vocab, cap, 1 if exact else 0,
                                    workspace.data_ptr(), need, idx.data_ptr(), val.data_ptr()))
    return idx, val


def gguf_tied_lm_argmax(hidden, w_bytes, n_embd: int, n_vocab: int, scheme: int, exact: bool = True, workspace=None):
    """rlx_cpu::lm_head::gguf_tied_lm_argmax (rlx-cpu/src/lm_head.rs:223-251) on the GPU: (token id, logit)
    as two one-element CUDA tensors; nothing is copied to the host."""
    torch = _torch()
    assert hidden.is_cuda and hidden.is_contiguous() and hidden.numel() == n_embd
    assert w_bytes.is_cuda and w_bytes.dtype == torch.uint8 and w_bytes.is_contiguous()
    need = lm_head_workspace_bytes(scheme, n_embd, n_vocab, _dt(hidden, torch), 1)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=hidden.device)
    idx = torch.empty(1, dtype=torch.int32, device=hidden.device)
    val = torch.empty(1, dtype=torch.float32, device=hidden.device)
    with torch.cuda.device(hidden.device):
        check(lib.rlxq_lm_head_argmax(_stream_ptr(torch), int(scheme), hidden.data_ptr(), _dt(hidden, torch),
                                      w_bytes.data_ptr(), n_embd, n_vocab, 1 if exact else 0,
                                      workspace.data_ptr(), need, idx.data_ptr(), val.data_ptr()))
    return idx, val


# ------------------------------------------------------------------ Graph / Session mirror
class Graph:
    """rlx_ir::Graph restricted to this path's ops."""

    def __init__(self, name: str):
        self._h = lib.rlxq_graph_new(name.encode())
        if not self._h:
            raise MemoryError("rlxq_graph_new")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.rlxq_graph_free(h)

    def input(self, name: str, shape: Sequence[int], dtype: DType = DType.F32) -> int:
        m, k = shape
        return check(lib.rlxq_graph_input(self._h, name.encode(), m, k, int(dtype)))

    def param(self, name: str, shape: Sequence[int], dtype: DType = DType.U8) -> int:
        if dtype != DType.U8 or len(shape) != 1:
            raise ValueError("packed weights are declared as Shape([bytes], U8)")
        return check(lib.rlxq_graph_param_u8(self._h, name.encode(), shape[0]))

    def dequant_matmul_packed(self, x: int, w_packed: int, scheme: QuantScheme, n: int,
                              out_dtype: DType = DType.F32) -> int:
        return check(lib.rlxq_graph_dequant_matmul(self._h, x, w_packed, int(scheme), n, int(out_dtype)))

    def swiglu_mul(self, gate: int, up: int) -> int:
        return check(lib.rlxq_graph_swiglu_mul(self._h, gate, up))

    def dequant_grouped_matmul_packed(self, x: int, w_packed: int, expert_idx: int, scheme: QuantScheme, n: int,
                                      num_experts: int) -> int:
        """add_node(Op::DequantGroupedMatMul{scheme}, [x, w_packed, expert_idx], Shape([m, n], F32))."""
        return check(lib.rlxq_graph_dequant_grouped_matmul(self._h, x, w_packed, expert_idx, int(scheme), n, num_experts))

    def set_outputs(self, nodes: Sequence[int]) -> None:
        if len(nodes) != 1:
            raise ValueError("one output node")
        check(lib.rlxq_graph_set_output(self._h, nodes[0]))


class CompiledGraph:
    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.rlxq_compiled_free(h)

    def set_param_typed(self, name: str, data, dtype: DType = DType.U8) -> None:
        if dtype != DType.U8:
            raise ValueError("packed weights are uploaded as DType.U8 bytes")
        a = np.ascontiguousarray(np.frombuffer(data, np.uint8) if not isinstance(data, np.ndarray) else data)
        assert a.dtype == np.uint8
        check(lib.rlxq_compiled_set_param_typed(self._h, name.encode(), a.ctypes.data, a.nbytes))

    def run(self, inputs: Sequence[tuple[str, np.ndarray]], out_shape: tuple[int, int]) -> np.ndarray:
        """run(&[("x", &[f32])]) -> f32 output [m, n]."""
        n = len(inputs)
        names = (C.c_char_p * n)(*[nm.encode() for nm, _ in inputs])
        arrs = [np.ascontiguousarray(a, np.float32) for _, a in inputs]
        ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
        elems = (C.c_uint64 * n)(*[a.size for a in arrs])
        out = np.empty(out_shape, np.float32)
        check(lib.rlxq_compiled_run(self._h, n, names, ptrs, elems, out.ctypes.data, out.size))
        return out

    def run_typed(self, inputs: Sequence[tuple[str, np.ndarray, DType]], out_shape: tuple[int, int],
                  out_dtype: DType) -> np.ndarray:
        """Typed I/O: bf16 tensors travel as uint16 arrays of bit patterns."""
        n = len(inputs)
        names = (C.c_char_p * n)(*[nm.encode() for nm, _, _ in inputs])
        arrs = [np.ascontiguousarray(a) for _, a, _ in inputs]
        ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
        nbytes = (C.c_uint64 * n)(*[a.nbytes for a in arrs])
        dts = (C.c_uint32 * n)(*[int(d) for _, _, d in inputs])
        out = np.empty(out_shape, np.float32 if out_dtype == DType.F32 else np.uint16)
        check(lib.rlxq_compiled_run_typed(self._h, n, names, ptrs, nbytes, dts, out.ctypes.data,
                                          out.nbytes, int(out_dtype)))
        return out

    def run_raw(self, names, ptrs, nbytes, dtypes, out_ptr: int, out_bytes: int, out_dtype: int) -> None:
        """Pointer-level run_typed for callers that manage their own (pinned) host buffers."""
        n = len(names)
        check(lib.rlxq_compiled_run_typed(
            self._h, n, (C.c_char_p * n)(*[s.encode() for s in names]), (C.c_void_p * n)(*ptrs),
            (C.c_uint64 * n)(*nbytes), (C.c_uint32 * n)(*dtypes), out_ptr, out_bytes, out_dtype))

    def bind_raw(self, names, ptrs, nbytes, dtypes, out_ptr: int, out_bytes: int, out_dtype: int):
        """run_raw with the argument arrays built once: returns a callable for a decode loop that runs
        the same host buffers every step."""
        n = len(names)
        args = (self._h, n, (C.c_char_p * n)(*[s.encode() for s in names]), (C.c_void_p * n)(*ptrs),
                (C.c_uint64 * n)(*nbytes), (C.c_uint32 * n)(*dtypes), out_ptr, out_bytes, out_dtype)
        fn = lib.rlxq_compiled_run_typed

        def step(_keep=self) -> None:
            rc = fn(*args)
            if rc:
                check(rc)
        return step

    @property
    def arena_bytes(self) -> int:
        return int(lib.rlxq_compiled_arena_bytes(self._h))

    def fused_ffn_count(self) -> int:
        """SwiGLU FFN groups the compiler fused (stacked gate / up matmul + down projection with the product inside)."""
        return int(lib.rlxq_compiled_fused_ffn_count(self._h))

    def clear_scratch(self) -> None:
        """Zeroes the kernels' scratch region; the step to take after device_status() raised a timeout."""
        check(lib.rlxq_compiled_clear_scratch(self._h))


class Session:
    """Session::new(Device::Cuda) — rlx-runtime/src/session.rs:42-87."""

    def __init__(self, device: Device = Device.Cuda, index: int = 0, exec_mode: str = "graph"):
        if device != Device.Cuda:
            raise ValueError("only Device.Cuda exists here")
        self.index = index
        self.exec_mode = {"stream": 0, "graph": 1}[exec_mode]

    def compile(self, graph: Graph) -> CompiledGraph:
        h = C.c_void_p()
        check(lib.rlxq_session_compile(graph._h, self.index, self.exec_mode, C.byref(h)))
        return CompiledGraph(h.value)


__all__ = ["QuantScheme", "DType", "Device", "Graph", "Session", "CompiledGraph", "RlxqError",
           "dequant_f32", "matmul", "scheme_geometry", "packed_bytes", "workspace_bytes",
           "set_option", "get_option", "launch_count", "device_status",
           "matmul_chain", "chain_workspace_bytes", "ChainLayer",
           "grouped_matmul", "gguf_tied_lm_argmax", "gguf_tied_lm_topk", "lm_head_workspace_bytes", "LM_MAX_CAP"]
