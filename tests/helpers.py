"""Shared helpers for the GPU parity tests: seeded inputs, oracle outputs, the tolerance."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

SCHEMES = dict(O.SCHEMES)

# The path's matmul tolerance: |y - y_ref| <= 1e-3 * ||x_row||_2 * ||w_row||_2 per element,
# y_ref from the f32 oracle on the same (bf16-widened where applicable) inputs.
MATMUL_TOL = 1e-3


def make_case(scheme: int, m: int, k: int, n: int, seed: int, x_bf16: bool = False):
    w = O.fill_weights(scheme, seed, k, n)
    x = O.fill_normal(seed + 1000, m * k).reshape(m, k)
    if x_bf16:
        xb = O.f32_to_bf16_bits(x)
        x = O.bf16_bits_to_f32(xb).reshape(m, k)
    return w, x


def reference(scheme: int, w: np.ndarray, x: np.ndarray, n: int, serial: bool = False) -> np.ndarray:
    m, k = x.shape
    if serial:
        return O.matmul_bt(x, w, m, k, n, scheme)
    return O.matmul_bt_mt(x, w, m, k, n, scheme)


def bound(scheme: int, w: np.ndarray, x: np.ndarray, n: int) -> np.ndarray:
    """[m, n] array of ||x_row|| * ||w_row||."""
    m, k = x.shape
    wn = O.row_norms(scheme, w, k, n)
    xn = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))
    return xn[:, None] * wn[None, :]


def assert_within_tolerance(y: np.ndarray, y_ref: np.ndarray, bnd: np.ndarray, tol: float = MATMUL_TOL,
                            what: str = "") -> float:
    err = np.abs(y.astype(np.float64) - y_ref.astype(np.float64))
    ratio = err / np.maximum(bnd, 1e-30)
    worst = float(ratio.max()) if ratio.size else 0.0
    assert np.isfinite(y).all(), f"{what}: non-finite output"
    assert worst <= tol, f"{what}: max |y-y_ref|/(|x||w|) = {worst:.3e} > {tol:.1e}"
    return worst


def copy_to_device(dst_ptr: int, host: np.ndarray) -> None:
    """cudaMemcpy of a numpy array to a raw device address (for buffers the library allocated itself)."""
    import ctypes as C
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    rt.cudaMemcpy.restype = C.c_int
    host = np.ascontiguousarray(host)
    rc = rt.cudaMemcpy(dst_ptr, host.ctypes.data, host.nbytes, 1)
    assert rc == 0, f"cudaMemcpy failed with {rc}"
