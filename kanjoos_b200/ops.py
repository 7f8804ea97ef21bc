"""Thin typed wrappers over the C-ABI for torch CUDA tensors (torch supplies
device memory and streams only; every computation is a kernel of
libknj_device.so). Names follow the C entry points."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import DT_BF16, DT_F16, DT_F32, check, lib

_DT = {torch.float32: DT_F32, torch.bfloat16: DT_BF16, torch.float16: DT_F16}


def _p(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, dtype=None):
    if not t.is_cuda:
        raise ValueError("tensor must live on a CUDA device")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"expected {dtype}, got {t.dtype}")
    return t


def device_caps(idx: int = 0) -> _lib.DeviceCapsC:
    caps = _lib.DeviceCapsC()
    check(lib().knj_dev_caps(idx, C.byref(caps)))
    return caps


def control(seed: int, n_threads: int = 64, n_blocks: int = 1) -> torch.Tensor:
    out = torch.full((2,), 0xABABABAB - (1 << 32), dtype=torch.int32, device="cuda")
    check(lib().knj_control_launch(_p(out), seed, n_threads, n_blocks, _stream()))
    return out


def probe_caps(inp: torch.Tensor | None = None) -> torch.Tensor:
    cap = torch.zeros(8, dtype=torch.int32, device="cuda")
    check(lib().knj_probe_caps_launch(_p(cap), _p(inp), _stream()))
    return cap


def build_asum(act: torch.Tensor, M: int, K: int, n_threads: int = 64, n_blocks: int | None = None) -> torch.Tensor:
    _need(act, torch.int32)
    asum = torch.full((M, K // 128), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    if n_blocks is None:
        n_blocks = max(1, (M * (K // 128) + n_threads - 1) // n_threads)
    check(lib().knj_build_asum_launch(_p(act), _p(asum), M, K, n_threads, n_blocks, _stream()))
    return asum


def gemm_w4_i8(Bq: torch.Tensor, act: torch.Tensor, asum: torch.Tensor, M: int, N: int, K: int, n_threads: int = 64,
               n_blocks: int | None = None) -> torch.Tensor:
    _need(Bq, torch.uint8), _need(act, torch.int32), _need(asum, torch.int32)
    Cm = torch.full((M, N), -12345.0, dtype=torch.float32, device="cuda")
    if n_blocks is None:
        n_blocks = max(1, (M * N + n_threads - 1) // n_threads)
    check(lib().knj_gemm_w4_i8_launch(_p(Bq), _p(act), _p(asum), _p(Cm), M, N, K, n_threads, n_blocks, _stream()))
    return Cm


def dot_helpers(a: torch.Tensor, b: torch.Tensor, acc: torch.Tensor):
    """int32 [n] x 3 -> (dot4_i8, dot8_i4, dot2_i16) computed by include/knj_dot.h on the device."""
    _need(a, torch.int32), _need(b, torch.int32), _need(acc, torch.int32)
    outs = [torch.full_like(a, 0x5A5A5A5A) for _ in range(3)]
    check(lib().knj_dot_helpers_launch(_p(a), _p(b), _p(acc), _p(outs[0]), _p(outs[1]), _p(outs[2]), a.numel(), _stream()))
    return outs


def q4k_dequant(blocks: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 144] -> f32 [..., 256]."""
    _need(blocks, torch.uint8)
    assert blocks.shape[-1] == 144
    nb = blocks.numel() // 144
    out = torch.full(blocks.shape[:-1] + (256,), -12345.0, dtype=torch.float32, device="cuda")
    check(lib().knj_q4k_dequant_launch(_p(blocks), _p(out), nb, _stream()))
    return out


def q6k_dequant(blocks: torch.Tensor) -> torch.Tensor:
    _need(blocks, torch.uint8)
    assert blocks.shape[-1] == 210
    nb = blocks.numel() // 210
    out = torch.full(blocks.shape[:-1] + (256,), -12345.0, dtype=torch.float32, device="cuda")
    check(lib().knj_q6k_dequant_launch(_p(blocks), _p(out), nb, _stream()))
    return out


def rmsnorm(x: torch.Tensor, w_bf16: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x), _need(w_bf16, torch.bfloat16)
    T, H = x.shape
    out = torch.empty((T, H), dtype=torch.float32, device="cuda")
    check(lib().knj_rmsnorm_launch(_p(x), _DT[x.dtype], H, _p(w_bf16), eps, T, H, _p(out), _stream()))
    return out


def router_topk(x: torch.Tensor, Wr: torch.Tensor, k: int, bias: torch.Tensor | None = None):
    """x [T][H] (f32/bf16), Wr bf16 [E][H] -> (logits [T][E], pair_exp [T*k], pair_w [T*k])."""
    _need(x), _need(Wr, torch.bfloat16)
    T, H = x.shape
    E = Wr.shape[0]
    logits = torch.empty((T, E), dtype=torch.float32, device="cuda")
    pair_exp = torch.full((T * k,), -1, dtype=torch.int32, device="cuda")
    pair_w = torch.full((T * k,), -12345.0, dtype=torch.float32, device="cuda")
    check(lib().knj_router_topk_launch(_p(x), _DT[x.dtype], H, _p(Wr), _p(bias), T, H, E, k, _p(logits), _p(pair_exp),
                                       _p(pair_w), _stream()))
    return logits, pair_exp, pair_w


def moe_permute(pair_exp: torch.Tensor, E: int, idx_stride: int):
    _need(pair_exp, torch.int32)
    P = pair_exp.numel()
    pair_idx = torch.empty((E, idx_stride), dtype=torch.int32, device="cuda")
    pair_cnt = torch.empty((E,), dtype=torch.int32, device="cuda")
    exp_list = torch.empty((E,), dtype=torch.int32, device="cuda")
    n_active = torch.empty((4,), dtype=torch.int32, device="cuda")
    if P >= 8192 and E <= 256:
        nbytes = int(lib().knj_moe_permute_scratch_bytes(P, E))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        check(lib().knj_moe_permute_ws_launch(_p(pair_exp), P, E, idx_stride, _p(pair_idx), _p(pair_cnt), _p(exp_list),
                                              _p(n_active), _p(scratch), nbytes, _stream()))
    else:
        check(lib().knj_moe_permute_launch(_p(pair_exp), P, E, idx_stride, _p(pair_idx), _p(pair_cnt), _p(exp_list),
                                           _p(n_active), _stream()))
    return pair_idx, pair_cnt, exp_list, n_active


def q4k_gateup(x, Wg, Wu, pair_idx, pair_cnt, exp_list, n_active, P: int, top_k: int, want=("G", "U", "A"),
               pair_tok=None):
    """x [T][K] activation rows (f32/bf16/f16) -> dict of f32 [P][N] outputs (G, U, A = silu(G)*U)."""
    _need(x)
    E, N, nsb, _ = Wg.shape
    K = nsb * 256
    outs = {n: (torch.full((P, N), -12345.0, dtype=torch.float32, device="cuda") if n in want else None)
            for n in ("G", "U", "A")}
    check(lib().knj_q4k_gateup_launch(_p(x), _DT[x.dtype], x.shape[1], _p(Wg), _p(Wu), _p(pair_idx), _p(pair_cnt),
                                      _p(pair_tok), _p(exp_list), _p(n_active), _p(outs["G"]), _p(outs["U"]),
                                      _p(outs["A"]), N, K, nsb * 144, pair_idx.shape[1], E, top_k, None, _stream()))
    return outs


def q4k_proj(a, W, pair_idx, pair_cnt, exp_list, n_active, P: int, pair_row=None):
    """a [rows][K] activation rows (one per pair unless pair_row maps them) -> Y f32 [P][N]."""
    _need(a)
    E, N, nsb, _ = W.shape
    K = nsb * 256
    Y = torch.full((P, N), -12345.0, dtype=torch.float32, device="cuda")
    check(lib().knj_q4k_proj_launch(_p(a), _DT[a.dtype], a.shape[1], _p(W), _p(pair_idx), _p(pair_cnt), _p(pair_row),
                                    _p(exp_list), _p(n_active), _p(Y), N, K, nsb * 144, pair_idx.shape[1], E, None,
                                    _stream()))
    return Y


def q6k_proj(A: torch.Tensor, W6: torch.Tensor, pair_idx, pair_cnt, exp_list, n_active, P: int) -> torch.Tensor:
    """A f32 [P][K], W6 uint8 [E][N][K/256][210] -> Y f32 [P][N] (rows of pairs of inactive experts stay poisoned)."""
    _need(A, torch.float32), _need(W6, torch.uint8)
    E, N, nblk, _ = W6.shape
    Y = torch.full((P, N), -12345.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib().knj_q6k_proj_launch(_p(A), _p(W6), _p(pair_idx), _p(pair_cnt), _p(exp_list), _p(n_active), _p(Y), N,
                                    nblk * 256, pair_idx.shape[1], E, _p(status), _stream()))
    if int(status.item()):
        raise RuntimeError("knj_q6k_proj_launch: a bounded wait for a weight block gave up")
    return Y


def fuse_gateup_silu(G: torch.Tensor, U: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    _need(G, torch.float32), _need(U, torch.float32)
    A = torch.empty(G.shape, dtype=dtype, device="cuda")
    check(lib().knj_fuse_gateup_silu_launch(_p(G), _p(U), _p(A), _DT[dtype], G.numel(), _stream()))
    return A


def moe_combine(Y, pair_exp, pair_w, T: int, k: int, resid=None, out_dtype=torch.float32, pair_row=None):
    H = Y.shape[1]
    out = torch.empty((T, H), dtype=out_dtype, device="cuda")
    check(lib().knj_moe_combine_launch(_p(Y), _p(pair_row), _p(pair_exp), _p(pair_w), _p(resid),
                                       _DT[resid.dtype] if resid is not None else 0, H, _p(out), _DT[out_dtype], H, T, H,
                                       k, _stream()))
    return out


def q4k_matmul(W: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """W uint8 [n_out][n_in/256][144], x [m][n_in] -> f32 [m][n_out] (Model::matmul)."""
    _need(W, torch.uint8), _need(x)
    n_out, nsb, _ = W.shape
    m, n_in = x.shape
    assert nsb * 256 == n_in
    y = torch.full((m, n_out), -12345.0, dtype=torch.float32, device="cuda")
    nbytes = lib().knj_q4k_matmul_workspace_bytes(m, n_in)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    check(lib().knj_q4k_matmul_launch(_p(W), n_in, n_out, _p(x), _DT[x.dtype], n_in, m, _p(y), n_out, _p(ws), nbytes,
                                      _stream()))
    return y


def to_f16(x: torch.Tensor) -> torch.Tensor:
    _need(x)
    rows, K = x.shape
    out = torch.empty((rows, K), dtype=torch.float16, device="cuda")
    check(lib().knj_to_f16_launch(_p(x), _DT[x.dtype], K, rows, K, _p(out), _stream()))
    return out


def q4k_gateup_tc(xh, Wg, Wu, pair_idx, pair_cnt, P: int, top_k: int, pair_tok=None, poison: bool = True):
    """Tensor-core grouped gate+up: returns (A fp16 [P][N] scaled by 2^-6, status int32[1]).
    poison=True pre-fills A with NaN so that tests can see unwritten rows."""
    _need(xh, torch.float16)
    E, N, nsb, _ = Wg.shape
    A = (torch.full((P, N), float("nan"), dtype=torch.float16, device="cuda") if poison
         else torch.empty((P, N), dtype=torch.float16, device="cuda"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib().knj_q4k_gateup_tc_launch(_p(xh), _p(Wg), _p(Wu), _p(pair_idx), _p(pair_cnt), _p(pair_tok), _p(A), N,
                                         nsb * 256, nsb * 144, pair_idx.shape[1], E, top_k, P, _p(status), _stream()))
    return A, status


def q6k_down_tc(ah, W6, pair_idx, pair_cnt, P: int, pair_row=None):
    """Grouped down GEMM over Q6_K weights [E][N][K/256][210] (K <= 1024): fp16 activations as the gate+up GEMM
    writes them -> Y f32 [P][N]."""
    _need(ah, torch.float16), _need(W6, torch.uint8)
    E, N, nsb, _ = W6.shape
    Y = torch.full((P, N), -12345.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib().knj_q6k_down_tc_launch(_p(ah), _p(W6), _p(pair_idx), _p(pair_cnt), _p(pair_row), _p(Y), N, nsb * 256,
                                       pair_idx.shape[1], E, P, _p(status), _stream()))
    return Y, status


def q4k_down_tc(ah, Wd, pair_idx, pair_cnt, P: int, pair_row=None, poison: bool = True):
    _need(ah, torch.float16)
    E, N, nsb, _ = Wd.shape
    Y = (torch.full((P, N), -12345.0, dtype=torch.float32, device="cuda") if poison
         else torch.empty((P, N), dtype=torch.float32, device="cuda"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib().knj_q4k_down_tc_launch(_p(ah), _p(Wd), _p(pair_idx), _p(pair_cnt), _p(pair_row), _p(Y), N, nsb * 256,
                                       nsb * 144, pair_idx.shape[1], E, P, _p(status), _stream()))
    return Y, status
