"""ctypes access to the CPU checkers under oracle/ (test infrastructure only).

`oracle()` loads oracle/libknj_oracle.so (the C restatement), building it with
`make` when missing. `ref()` loads oracle/_ref/libknj_ref.so (the reference's
own sources compiled where they lie) or returns None when it was never built
and the reference tree is not present.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from functools import lru_cache

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")


def reference_root() -> str | None:
    """Root of the reference project's source tree: $KNJ_REFERENCE_ROOT, else a directory named `reference` beside
    this repository; None when neither holds the loader sources."""
    for cand in (os.environ.get("KNJ_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "loader")):
            return cand
    return None

u8p = C.POINTER(C.c_uint8)
i8p = C.POINTER(C.c_int8)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)
i32p = C.POINTER(C.c_int32)
u32p = C.POINTER(C.c_uint32)
u16p = C.POINTER(C.c_uint16)


def ptr(a: np.ndarray, typ):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(typ)


@lru_cache(maxsize=None)
def oracle() -> C.CDLL:
    so = os.path.join(ORACLE_DIR, "libknj_oracle.so")
    src = os.path.join(ORACLE_DIR, "knj_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR], stdout=subprocess.DEVNULL)
    lib = C.CDLL(so)
    lib.knj_or_fp16_to_fp32.restype = C.c_float
    lib.knj_or_fp16_to_fp32.argtypes = [C.c_uint16]
    lib.knj_or_q4k_weight.restype = C.c_float
    lib.knj_or_q4k_weight.argtypes = [u8p, C.c_int]
    lib.knj_or_q6k_weight.restype = C.c_float
    lib.knj_or_q6k_weight.argtypes = [u8p, C.c_int]
    lib.knj_or_q4k_span16.argtypes = [u8p, C.c_int, f32p]
    lib.knj_or_dequant_q4k.argtypes = [u8p, f32p, C.c_uint64]
    lib.knj_or_dequant_q6k.argtypes = [u8p, f32p, C.c_uint64]
    lib.knj_or_dot_q4k.restype = C.c_float
    lib.knj_or_dot_q4k.argtypes = [u8p, f32p, C.c_uint64]
    lib.knj_or_matmul_q4k.argtypes = [u8p, C.c_int, C.c_int, f32p, C.c_int, C.c_int, f32p, C.c_int]
    lib.knj_or_matmul_plain.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, f32p, C.c_int, C.c_int, f32p, C.c_int]
    lib.knj_or_rmsnorm_rows.argtypes = [f32p, C.c_int, C.c_int, f32p, C.c_float, f32p]
    lib.knj_or_silu_mul.argtypes = [f32p, f32p, C.c_uint64]
    lib.knj_or_route.argtypes = [C.c_void_p, C.c_int, f32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p, i32p, f32p]
    lib.knj_or_moe.argtypes = [C.c_void_p, C.c_int, u8p, u8p, u8p, f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_int, f32p, i32p, f32p]
    lib.knj_or_build_plan.restype = C.c_int
    lib.knj_or_build_plan.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p, i32p, i32p, i32p, i32p]
    lib.knj_or_gemm_w4_reference.argtypes = [u8p, i8p, f32p, C.c_int, C.c_int, C.c_int]
    lib.knj_or_gemm_w4_i8_mirror.argtypes = [u8p, i8p, f32p, C.c_int, C.c_int, C.c_int]
    lib.knj_or_deinterleave_activations.argtypes = [i8p, u32p, C.c_int, C.c_int]
    lib.knj_or_build_asum.argtypes = [i8p, i32p, C.c_int, C.c_int]
    lib.knj_or_w4_kat_problem.argtypes = [C.c_uint32, C.c_int, C.c_int, C.c_int, u8p, i8p]
    lib.knj_or_compare.argtypes = [f32p, f32p, C.c_int64, f64p]
    lib.knj_or_num_threads.restype = C.c_int
    lib.knj_or_set_threads.argtypes = [C.c_int]
    return lib


@lru_cache(maxsize=None)
def ref():
    so = os.path.join(ORACLE_DIR, "_ref", "libknj_ref.so")
    if not os.path.exists(so):
        root = reference_root()
        if root is None:
            return None
        subprocess.check_call(["make", "-C", ORACLE_DIR, "ref", "REF=" + root], stdout=subprocess.DEVNULL)
    lib = C.CDLL(so)
    lib.ref_fp16_to_fp32.restype = C.c_float
    lib.ref_fp16_to_fp32.argtypes = [C.c_uint16]
    lib.ref_half_bits_to_float.restype = C.c_float
    lib.ref_half_bits_to_float.argtypes = [C.c_uint16]
    lib.ref_host_oracle_h2f.restype = C.c_float
    lib.ref_host_oracle_h2f.argtypes = [C.c_uint16]
    lib.ref_dequant_row_q4k.argtypes = [u8p, f32p, C.c_uint64]
    lib.ref_dequant_row_q6k.argtypes = [u8p, f32p, C.c_uint64]
    lib.ref_dequant_dot_q4k.restype = C.c_float
    lib.ref_dequant_dot_q4k.argtypes = [u8p, f32p, C.c_uint64]
    lib.ref_q4k_weight.restype = C.c_float
    lib.ref_q4k_weight.argtypes = [u8p, C.c_int]
    lib.ref_q6k_weight.restype = C.c_float
    lib.ref_q6k_weight.argtypes = [u8p, C.c_int]
    lib.ref_q4k_span16.argtypes = [u8p, C.c_int, f32p]
    lib.ref_gemm_w4_reference.argtypes = [u8p, i8p, f32p, C.c_int, C.c_int, C.c_int]
    lib.ref_deinterleave_activations.argtypes = [i8p, u32p, C.c_int, C.c_int]
    lib.ref_compare.argtypes = [f32p, f32p, C.c_int, C.c_int, f64p]
    lib.ref_matmul_q4k.argtypes = [u8p, C.c_int, C.c_int, f32p, C.c_int, C.c_int, f32p, C.c_int, C.c_int]
    lib.ref_moe.argtypes = [u16p, u8p, u8p, u8p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p,
                            i32p, f32p, C.c_int]
    lib.ref_hardware_threads.restype = C.c_int
    return lib


# --- numpy-level conveniences over the restatement --------------------------

def dequant_q4k(blocks: np.ndarray) -> np.ndarray:
    """uint8 [..., 144] -> f32 [..., 256] through the restated row decoder."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    n = b.size // 144 * 256
    out = np.empty(n, dtype=np.float32)
    oracle().knj_or_dequant_q4k(ptr(b, u8p), ptr(out, f32p), n)
    return out.reshape(b.shape[:-1] + (256,))


def matmul_q4k(W: np.ndarray, x: np.ndarray) -> np.ndarray:
    """W uint8 [n_out][n_in/256][144], x f32 [m][n_in] -> f32 [m][n_out]."""
    W = np.ascontiguousarray(W, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n_out, nb = W.shape[0], W.shape[1]
    m, n_in = x.shape
    assert nb * 256 == n_in
    y = np.empty((m, n_out), dtype=np.float32)
    oracle().knj_or_matmul_q4k(ptr(W, u8p), n_in, n_out, ptr(x, f32p), m, n_in, ptr(y, f32p), n_out)
    return y


def moe(Wr_bits: np.ndarray, bank: dict, hx: np.ndarray, top_k: int = 8):
    """Restated Model::moe. Returns (out [m][H], chosen [m][K], weight [m][K])."""
    hx = np.ascontiguousarray(hx, dtype=np.float32)
    m, H = hx.shape
    E, F = bank["gate"].shape[0], bank["gate"].shape[1]
    out = np.empty((m, H), dtype=np.float32)
    chosen = np.empty((m, top_k), dtype=np.int32)
    weight = np.empty((m, top_k), dtype=np.float32)
    wr = np.ascontiguousarray(Wr_bits, dtype=np.uint16)
    oracle().knj_or_moe(wr.ctypes.data_as(C.c_void_p), 1, ptr(bank["gate"], u8p), ptr(bank["up"], u8p),
                        ptr(bank["down"], u8p), ptr(hx, f32p), m, H, E, top_k, F, ptr(out, f32p),
                        ptr(chosen, i32p), ptr(weight, f32p))
    return out, chosen, weight


def route(Wr, wr_type: int, hx: np.ndarray, E: int, top_k: int = 8):
    hx = np.ascontiguousarray(hx, dtype=np.float32)
    m, H = hx.shape
    logits = np.empty((m, E), dtype=np.float32)
    chosen = np.empty((m, top_k), dtype=np.int32)
    weight = np.empty((m, top_k), dtype=np.float32)
    Wr = np.ascontiguousarray(Wr)
    oracle().knj_or_route(Wr.ctypes.data_as(C.c_void_p), wr_type, ptr(hx, f32p), m, H, E, top_k,
                          ptr(logits, f32p), ptr(chosen, i32p), ptr(weight, f32p))
    return logits, chosen, weight


def silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """silu(g) * u with the CPU path's own expf (element-wise, f32)."""
    a = np.ascontiguousarray(g, dtype=np.float32).copy()
    u = np.ascontiguousarray(u, dtype=np.float32)
    oracle().knj_or_silu_mul(ptr(a, f32p), ptr(u, f32p), a.size)
    return a


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    oracle().knj_or_rmsnorm_rows(ptr(x, f32p), x.shape[0], x.shape[1], ptr(w, f32p), eps, ptr(out, f32p))
    return out


def compare(got: np.ndarray, want: np.ndarray) -> dict:
    g = np.ascontiguousarray(got, dtype=np.float32).ravel()
    w = np.ascontiguousarray(want, dtype=np.float32).ravel()
    assert g.size == w.size
    out = np.zeros(6, dtype=np.float64)
    oracle().knj_or_compare(ptr(g, f32p), ptr(w, f32p), g.size, ptr(out, f64p))
    return {"rel_rmse": out[0], "max_abs": out[1], "out_rms": out[2], "max_idx": int(out[3]),
            "nonzero": int(out[4]), "total": int(out[5])}
