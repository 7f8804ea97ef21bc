"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations (Qwen3-30B-A3B MoE geometry, GGUF Q4_K experts).

No checkpoint is available offline, so every tensor is drawn from a documented
generator. Tensors for parity tests are generated on the CPU with numpy's Philox
stream (one independent stream per tensor, keyed by config / tensor / layer /
expert) so the CPU checker and the GPU kernels see identical bytes.

Q4_K superblock layout (144 bytes, 256 weights; reference
kernels/knj_q4k.h:66-76): fp16 d, fp16 dmin, 12 bytes of packed 6-bit
scales/mins, 128 bytes of 4-bit codes.
"""
from __future__ import annotations

import numpy as np

QK_K = 256
Q4K_BYTES = 144

# Qwen3-30B-A3B MoE geometry (reference models/qwen3-30b-a3b/config.json).
HIDDEN = 2048
FFN = 768
N_EXPERTS = 128
TOP_K = 8
N_LAYERS = 48
RMS_EPS = 1e-6

_TENSOR_IDS = {"gate": 1, "up": 2, "down": 3, "router": 4, "x": 5, "norm": 6, "perm": 7}


def stream(config: int, tensor: str, layer: int = 0, expert: int = 0) -> np.random.Generator:
    """Independent Philox stream for one tensor."""
    ss = np.random.SeedSequence([0x4B4E4A, int(config), _TENSOR_IDS[tensor], int(layer), int(expert)])
    return np.random.Generator(np.random.Philox(ss))


def q4k_rows(rng: np.random.Generator, rows: int, n_in: int) -> np.ndarray:
    """Q4_K matrix of `rows` output rows over `n_in` inputs -> uint8 [rows, n_in/256, 144].

    Code bytes and the 12 scale bytes are uniform random bytes (so nibbles are
    uniform in 0..15 and the 6-bit scales/mins uniform in 0..63); d and dmin are
    fp16(|N(0,1)| * 0.01).
    """
    assert n_in % QK_K == 0
    nb = n_in // QK_K
    blk = rng.integers(0, 256, size=(rows, nb, Q4K_BYTES), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal(size=(rows, nb, 2))) * 0.01).astype(np.float16)
    blk[:, :, 0:4] = dd.view(np.uint8).reshape(rows, nb, 4)
    return blk


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    w = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    w = w + 0x7FFF + ((w >> 16) & 1)
    return (w >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """f32 array rounded through bf16 (values exactly representable in bf16)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(a))


def router_weight(config: int, layer: int = 0, n_experts: int = N_EXPERTS, hidden: int = HIDDEN,
                  zipf_s: float | None = None) -> tuple[np.ndarray, np.ndarray | None]:
    """Router W_r as bf16 bits [E][H] ~ N(0, 0.02).

    With `zipf_s`, also returns a per-expert f32 logit bias log p_e with
    p_e proportional to rank^-s over a seeded permutation of the experts, which makes
    expert popularity follow Zipf(s). Returns (bits, bias-or-None).
    """
    rng = stream(config, "router", layer)
    w = (rng.standard_normal(size=(n_experts, hidden)) * 0.02).astype(np.float32)
    bias = None
    if zipf_s is not None:
        perm = stream(config, "perm", layer).permutation(n_experts)
        p = np.arange(1, n_experts + 1, dtype=np.float64) ** (-zipf_s)
        p /= p.sum()
        bias = np.empty(n_experts, dtype=np.float32)
        bias[perm] = np.log(p).astype(np.float32)
    return f32_to_bf16_bits(w), bias


def hidden_rows(config: int, n_tokens: int, hidden: int = HIDDEN, layer: int = 0) -> np.ndarray:
    """Activations ~ N(0,1), rounded to bf16, returned as f32 [T][H]."""
    rng = stream(config, "x", layer)
    return bf16_round(rng.standard_normal(size=(n_tokens, hidden)).astype(np.float32))


def norm_weight(config: int, layer: int, hidden: int = HIDDEN) -> np.ndarray:
    """RMSNorm weight 1 + N(0, 0.02) as bf16 bits [H]."""
    rng = stream(config, "norm", layer)
    return f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal(size=hidden)).astype(np.float32))


def expert_bank(config: int, layer: int = 0, n_experts: int = N_EXPERTS, hidden: int = HIDDEN,
                ffn: int = FFN) -> dict[str, np.ndarray]:
    """gate/up [E][F][H/256][144] and down [E][H][F/256][144] Q4_K bytes."""
    out = {}
    for name, rows, n_in in (("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)):
        rng = stream(config, name, layer)
        out[name] = q4k_rows(rng, n_experts * rows, n_in).reshape(n_experts, rows, n_in // QK_K, Q4K_BYTES)
    return out
