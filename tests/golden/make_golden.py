"""Generates the golden vectors in this folder from the REFERENCE's own CPU
sources (oracle/_ref/libknj_ref.so, built by `make -C oracle ref`) and from
gguf-py. Run in a container where the reference tree is mounted:

    python tests/golden/make_golden.py        (golden.npz and golden_q6k.npz)
    python tests/golden/make_golden.py q6k    (golden_q6k.npz only)

The inputs are regenerated from seeds by kanjoos_b200.synth; each fixture stores
a sha256 of the input bytes so a drift in the generator is caught, plus the
reference outputs (full where small, sha256 + samples where large).
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle_lib as ol  # noqa: E402
from kanjoos_b200 import synth  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def crafted_blocks() -> np.ndarray:
    """Random blocks plus the corner cases the reference's validators craft
    (tools/dequant_validate.py: random, all-0x00, all-0xFF) and fp16 corner
    scales (subnormal, zero, largest finite)."""
    rng = np.random.Generator(np.random.Philox(20261125))
    blocks = rng.integers(0, 256, size=(12, 144), dtype=np.uint8)
    blocks[8, :] = 0x00
    blocks[9, :] = 0xFF
    blocks[9, 0:4] = np.array([0.5, 0.25], dtype=np.float16).view(np.uint8)  # 0xFFFF halves are NaN
    blocks[10, 0:4] = np.array([0x0001, 0x03FF], dtype=np.uint16).view(np.uint8)  # subnormal d, dmin
    blocks[11, 0:4] = np.array([0x7BFF, 0x0000], dtype=np.uint16).view(np.uint8)  # max finite d, zero dmin
    for i in range(8):
        blocks[i, 0:4] = (np.abs(rng.standard_normal(2)) * 0.01).astype(np.float16).view(np.uint8)
    return blocks


def crafted_q6k_blocks() -> np.ndarray:
    """Q6_K superblocks (210 bytes: ql[128], qh[64], int8 scales[16], fp16 d): random ones plus all-0x00,
    all-0xFF codes, extreme int8 scales (-128 / 127) and fp16 corner values of d."""
    rng = np.random.Generator(np.random.Philox(20261126))
    blocks = rng.integers(0, 256, size=(12, 210), dtype=np.uint8)
    for i in range(12):
        blocks[i, 208:210] = (np.abs(rng.standard_normal(1)) * 0.01).astype(np.float16).view(np.uint8)
    blocks[6, :208] = 0x00
    blocks[7, :208] = 0xFF
    blocks[8, 192:208] = np.array([-128, 127] * 8, dtype=np.int8).view(np.uint8)
    blocks[9, 208:210] = np.array([0x0001], dtype=np.uint16).view(np.uint8)   # subnormal d
    blocks[10, 208:210] = np.array([0x7BFF], dtype=np.uint16).view(np.uint8)  # largest finite d
    blocks[11, 208:210] = np.array([0x8000], dtype=np.uint16).view(np.uint8)  # -0
    return blocks


def q6k_golden() -> None:
    """Q6_K decode of the reference (src/loader/dequant.cpp:164-191 through dequant_row_f32, and the per-element
    twin kernels/knj_q4k.h knj_q6k_weight), cross-checked against gguf-py."""
    r = ol.ref()
    assert r is not None, "reference library not built: make -C oracle ref"
    import gguf
    from gguf import quants
    blocks = crafted_q6k_blocks()
    deq = np.empty((blocks.shape[0], 256), dtype=np.float32)
    r.ref_dequant_row_q6k(ol.ptr(blocks, ol.u8p), ol.ptr(deq, ol.f32p), deq.size)
    per_elem = np.array([[r.ref_q6k_weight(ol.ptr(blocks[b], ol.u8p), i) for i in range(256)]
                         for b in range(blocks.shape[0])], dtype=np.float32)
    assert np.array_equal(deq.view(np.uint32), per_elem.view(np.uint32)), "the reference's two Q6_K decoders disagree"
    gg = quants.dequantize(blocks, gguf.GGMLQuantizationType.Q6_K).astype(np.float32)
    assert np.array_equal(deq.view(np.uint32), gg.view(np.uint32)), "gguf-py disagrees"
    path = os.path.join(HERE, "golden_q6k.npz")
    np.savez_compressed(path, q6k_blocks=blocks, q6k_blocks_f32=deq)
    print("wrote", path, os.path.getsize(path), "bytes")


def main() -> None:
    r = ol.ref()
    assert r is not None, "reference library not built: make -C oracle ref"
    import gguf
    from gguf import quants

    # 1. fp16 -> f32 over every bit pattern (three reference twins agree).
    tab = np.array([r.ref_fp16_to_fp32(h) for h in range(65536)], dtype=np.float32)
    tab2 = np.array([r.ref_half_bits_to_float(h) for h in range(65536)], dtype=np.float32)
    tab3 = np.array([r.ref_host_oracle_h2f(h) for h in range(65536)], dtype=np.float32)
    fin = ~np.isnan(tab)
    assert np.array_equal(tab[fin], tab2[fin]) and np.array_equal(tab[fin], tab3[fin])
    finite_bits = tab.view(np.uint32).copy()
    finite_bits[~fin] = 0x7FC00000  # NaN payloads do not survive a C float return; canonicalise

    # 2. crafted Q4_K blocks, full outputs.
    blocks = crafted_blocks()
    deq = np.empty((blocks.shape[0], 256), dtype=np.float32)
    r.ref_dequant_row_q4k(ol.ptr(blocks, ol.u8p), ol.ptr(deq, ol.f32p), deq.size)
    per_elem = np.array([[r.ref_q4k_weight(ol.ptr(blocks[b], ol.u8p), i) for i in range(256)]
                         for b in range(blocks.shape[0])], dtype=np.float32)
    assert np.array_equal(deq.view(np.uint32), per_elem.view(np.uint32))
    gg = quants.dequantize(blocks, gguf.GGMLQuantizationType.Q4_K).astype(np.float32)
    assert np.array_equal(deq.view(np.uint32), gg.view(np.uint32)), "gguf-py disagrees"

    # 3. config 1: [768 x 2048] Q4_K GEMV.
    W = synth.q4k_rows(synth.stream(1, "gate"), synth.FFN, synth.HIDDEN)
    x = synth.stream(1, "x").standard_normal(synth.HIDDEN).astype(np.float32)
    full = np.empty(W.shape[0] * synth.HIDDEN, dtype=np.float32)
    r.ref_dequant_row_q4k(ol.ptr(W, ol.u8p), ol.ptr(full, ol.f32p), full.size)
    gg1 = quants.dequantize(W.reshape(W.shape[0], -1), gguf.GGMLQuantizationType.Q4_K).astype(np.float32)
    assert np.array_equal(full.view(np.uint32), gg1.ravel().view(np.uint32))
    y = np.array([r.ref_dequant_dot_q4k(ol.ptr(W[j], ol.u8p), ol.ptr(x, ol.f32p), synth.HIDDEN)
                  for j in range(W.shape[0])], dtype=np.float32)

    # 4. small MoE layer through reference decoders (E=16, H=512, F=256, top-4, 5 and 1 rows).
    bank_s = synth.expert_bank(102, n_experts=16, hidden=512, ffn=256)
    wr_s, _ = synth.router_weight(102, n_experts=16, hidden=512)
    small = {}
    for m in (1, 5):
        hx = synth.hidden_rows(102, m, 512, layer=m)
        out = np.empty((m, 512), np.float32)
        ch = np.empty((m, 4), np.int32)
        wt = np.empty((m, 4), np.float32)
        r.ref_moe(ol.ptr(wr_s, ol.u16p), ol.ptr(bank_s["gate"], ol.u8p), ol.ptr(bank_s["up"], ol.u8p),
                  ol.ptr(bank_s["down"], ol.u8p), ol.ptr(hx, ol.f32p), m, 512, 16, 4, 256,
                  ol.ptr(out, ol.f32p), ol.ptr(ch, ol.i32p), ol.ptr(wt, ol.f32p), 2)
        small[f"moe_small_m{m}_out"] = out
        small[f"moe_small_m{m}_chosen"] = ch
        small[f"moe_small_m{m}_weight"] = wt

    # 5. config 2: full-size layer, batch 1 and batch 8.
    bank = synth.expert_bank(2)
    wr, _ = synth.router_weight(2)
    cfg2 = {}
    for m in (1, 8):
        hx = synth.hidden_rows(2, m, layer=m)
        out = np.empty((m, synth.HIDDEN), np.float32)
        ch = np.empty((m, 8), np.int32)
        wt = np.empty((m, 8), np.float32)
        r.ref_moe(ol.ptr(wr, ol.u16p), ol.ptr(bank["gate"], ol.u8p), ol.ptr(bank["up"], ol.u8p),
                  ol.ptr(bank["down"], ol.u8p), ol.ptr(hx, ol.f32p), m, synth.HIDDEN, synth.N_EXPERTS, 8,
                  synth.FFN, ol.ptr(out, ol.f32p), ol.ptr(ch, ol.i32p), ol.ptr(wt, ol.f32p),
                  r.ref_hardware_threads())
        cfg2[f"cfg2_m{m}_out"] = out
        cfg2[f"cfg2_m{m}_chosen"] = ch
        cfg2[f"cfg2_m{m}_weight"] = wt

    # 6. W4-g128 known-answer problem of the reference's device test.
    M, N, K = 32, 768, 2048
    Bq = np.zeros(N * (K // 128) * 68, np.uint8)
    A = np.zeros(M * K, np.int8)
    ol.oracle().knj_or_w4_kat_problem(0x5EED1234, M, N, K, ol.ptr(Bq, ol.u8p), ol.ptr(A, ol.i8p))
    Cw = np.empty((M, N), np.float32)
    r.ref_gemm_w4_reference(ol.ptr(Bq, ol.u8p), ol.ptr(A, ol.i8p), ol.ptr(Cw, ol.f32p), M, N, K)
    act = np.empty(M * (K // 8) * 2, np.uint32)
    r.ref_deinterleave_activations(ol.ptr(A, ol.i8p), ol.ptr(act, ol.u32p), M, K)

    np.savez_compressed(
        os.path.join(HERE, "golden.npz"),
        fp16_table_sha=np.array(sha(finite_bits)),
        q4k_blocks=blocks, q4k_blocks_f32=deq,
        cfg1_w_sha=np.array(sha(W)), cfg1_x_sha=np.array(sha(x)),
        cfg1_dequant_sha=np.array(sha(full)), cfg1_dequant_head=full[:512].copy(), cfg1_y=y,
        moe_small_in_sha=np.array(sha(bank_s["gate"]) + sha(bank_s["up"]) + sha(bank_s["down"]) + sha(wr_s)),
        cfg2_in_sha=np.array(sha(bank["gate"]) + sha(bank["up"]) + sha(bank["down"]) + sha(wr)),
        w4_bq_sha=np.array(sha(Bq)), w4_act_sha=np.array(sha(A)), w4_deint_sha=np.array(sha(act)),
        w4_c=Cw,
        **small, **cfg2,
    )
    print("wrote", os.path.join(HERE, "golden.npz"), os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "q6k":
        q6k_golden()      # only the Q6_K fixture
    else:
        main()
        q6k_golden()
