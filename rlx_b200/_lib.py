"""ctypes binding of librlxq.so, the C-ABI library (include/rlxq.h, rlxq_session.h, rlxq_tp.h, rlxq_lm.h, rlxq_moe.h, rlxq_gguf.h).

The library is the product: if it is missing or does not load, importing this module raises.
There is no Python or CPU fallback for any compute entry point.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librlxq.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m rlx_b200.build` (needs nvcc). "
        "rlx_b200 has no fallback path.")

lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)

u32, u64, i64, vp, cp = C.c_uint32, C.c_uint64, C.c_int64, C.c_void_p, C.c_char_p

_SIGS = {
    "rlxq_version": (C.c_int, []),
    "rlxq_status_string": (cp, [C.c_int]),
    "rlxq_last_error": (cp, []),
    "rlxq_scheme_geometry": (C.c_int, [u32, C.POINTER(u32), C.POINTER(u32)]),
    "rlxq_packed_bytes": (C.c_int, [u32, u64, u64, C.POINTER(u64)]),
    "rlxq_workspace_bytes": (C.c_int, [u32, u32, u32, u32, u32, u32, C.POINTER(C.c_size_t)]),
    "rlxq_dequant_f32": (C.c_int, [vp, u32, vp, u64, vp]),
    "rlxq_matmul": (C.c_int, [vp, u32, vp, u32, vp, vp, u32, u32, u32, u32, vp, C.c_size_t]),
    "rlxq_matmul_static_scratch": (C.c_int, [vp, u32, vp, u32, vp, vp, u32, u32, u32, u32]),
    "rlxq_chain_workspace_bytes": (C.c_int, [u32, vp, u32, u32, u32, C.POINTER(C.c_size_t)]),
    "rlxq_matmul_chain": (C.c_int, [vp, u32, vp, u32, vp, u32, vp, u32, u32, vp, C.c_size_t]),
    "rlxq_init_device": (C.c_int, []),
    "rlxq_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "rlxq_launch_count": (u64, []),
    "rlxq_set_option": (C.c_int, [cp, i64]),
    "rlxq_get_option": (C.c_int, [cp, C.POINTER(i64)]),
    "rlxq_tp_shard_plan": (C.c_int, [u32, u32, u32, u32, u32, vp]),
    "rlxq_tp_slice_k_host": (C.c_int, [u32, vp, u32, u32, u32, u32, vp]),
    "rlxq_tp_ffn_workspace_bytes": (C.c_int, [u32, u32, u32, u32, u32, u32, C.POINTER(C.c_size_t)]),
    "rlxq_tp_ffn_partial": (C.c_int, [vp, u32, u32, vp, u32, vp, vp, vp, u32, u32, u32, vp, C.c_size_t]),
    "rlxq_tp_comm_bytes": (C.c_int, [u32, C.POINTER(C.c_size_t)]),
    "rlxq_tp_comm_alloc": (C.c_int, [u32, C.POINTER(vp)]),
    "rlxq_tp_comm_free": (C.c_int, [vp]),
    "rlxq_tp_ipc_export": (C.c_int, [vp, vp]),
    "rlxq_tp_ipc_open": (C.c_int, [vp, C.POINTER(vp)]),
    "rlxq_tp_ipc_close": (C.c_int, [vp]),
    "rlxq_tp_allreduce_sum": (C.c_int, [vp, u32, u32, C.POINTER(vp), u32, vp, vp, u32]),
    "rlxq_tp_ffn_step": (C.c_int, [vp, u32, u32, vp, u32, vp, vp, vp, u32, u32, u32, vp, C.c_size_t, u32, u32, C.POINTER(vp), u32]),
    "rlxq_tp_create": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(vp)]),
    "rlxq_tp_world": (C.c_int, [vp]),
    "rlxq_tp_ffn_load": (C.c_int, [vp, u32, vp, vp, vp, u32, u32]),
    "rlxq_tp_ffn_run": (C.c_int, [vp, vp, u32, u32, vp]),
    "rlxq_tp_status": (C.c_int, [vp, C.POINTER(C.c_int)]),
    "rlxq_tp_destroy": (C.c_int, [vp]),
    "rlxq_lm_head_workspace_bytes": (C.c_int, [u32, u32, u32, u32, u32, C.POINTER(C.c_size_t)]),
    "rlxq_lm_head_topk": (C.c_int, [vp, u32, vp, u32, vp, u32, u32, u32, u32, vp, C.c_size_t, vp, vp]),
    "rlxq_lm_head_argmax": (C.c_int, [vp, u32, vp, u32, vp, u32, u32, u32, vp, C.c_size_t, vp, vp]),
    "rlxq_grouped_workspace_bytes": (C.c_int, [u32, u32, u32, u32, u32, C.POINTER(C.c_size_t)]),
    "rlxq_grouped_matmul": (C.c_int, [vp, u32, vp, u32, vp, vp, vp, u32, u32, u32, u32, u32, vp, C.c_size_t]),
    "rlxq_gguf_open": (C.c_int, [cp, C.POINTER(vp)]),
    "rlxq_gguf_close": (None, [vp]),
    "rlxq_gguf_version": (u32, [vp]),
    "rlxq_gguf_alignment": (u64, [vp]),
    "rlxq_gguf_tensor_count": (u64, [vp]),
    "rlxq_gguf_data_start": (u64, [vp]),
    "rlxq_gguf_tensor_name": (C.c_int, [vp, u64, C.POINTER(cp)]),
    "rlxq_gguf_find": (C.c_int, [vp, cp, vp]),
    "rlxq_gguf_meta_u64": (C.c_int, [vp, cp, C.POINTER(u64)]),
    "rlxq_gguf_meta_str": (C.c_int, [vp, cp, C.POINTER(cp)]),
    "rlxq_gguf_read_tensor": (C.c_int, [vp, cp, vp, u64]),
    "rlxq_gguf_upload_tensor": (C.c_int, [vp, cp, vp, u64, vp]),
    "rlxq_graph_new": (vp, [cp]),
    "rlxq_graph_free": (None, [vp]),
    "rlxq_graph_input": (C.c_int, [vp, cp, u32, u32, u32]),
    "rlxq_graph_param_u8": (C.c_int, [vp, cp, u64]),
    "rlxq_graph_dequant_matmul": (C.c_int, [vp, C.c_int, C.c_int, u32, u32, u32]),
    "rlxq_graph_swiglu_mul": (C.c_int, [vp, C.c_int, C.c_int]),
    "rlxq_graph_dequant_grouped_matmul": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, u32, u32, u32]),
    "rlxq_graph_set_output": (C.c_int, [vp, C.c_int]),
    "rlxq_session_compile": (C.c_int, [vp, C.c_int, C.c_int, C.POINTER(vp)]),
    "rlxq_compiled_free": (None, [vp]),
    "rlxq_compiled_set_param_typed": (C.c_int, [vp, cp, vp, u64]),
    "rlxq_compiled_run": (C.c_int, [vp, u32, C.POINTER(cp), C.POINTER(vp), C.POINTER(u64), vp, u64]),
    "rlxq_compiled_run_typed": (C.c_int, [vp, u32, C.POINTER(cp), C.POINTER(vp), C.POINTER(u64),
                                          C.POINTER(u32), vp, u64, u32]),
    "rlxq_compiled_arena_bytes": (u64, [vp]),
    "rlxq_compiled_clear_scratch": (C.c_int, [vp]),
    "rlxq_compiled_fused_ffn_count": (u32, [vp]),
}


def _bind() -> None:
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)      # AttributeError here means the header and the library disagree
        fn.restype = res
        fn.argtypes = args


_bind()


class RlxqError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        text = lib.rlxq_status_string(status).decode()
        detail = lib.rlxq_last_error().decode()
        super().__init__(f"rlxq status {status} ({text}): {detail}")


def check(status: int) -> int:
    if status < 0:
        raise RlxqError(status)
    return status
