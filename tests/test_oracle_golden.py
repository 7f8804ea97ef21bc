"""The CPU restatement (oracle/knj_oracle.c) against the golden vectors that
the reference's own compiled CPU sources produced, and -- where the compiled
reference is present -- against it directly."""
import hashlib

import numpy as np
import pytest

import oracle_lib as ol
from kanjoos_b200 import synth


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_fp16_table(golden):
    o = ol.oracle()
    tab = np.array([o.knj_or_fp16_to_fp32(h) for h in range(65536)], dtype=np.float32)
    b = tab.view(np.uint32).copy()
    b[np.isnan(tab)] = 0x7FC00000
    assert sha(b) == str(golden["fp16_table_sha"])


def test_crafted_blocks_bit_exact(golden):
    blocks = golden["q4k_blocks"]
    want = golden["q4k_blocks_f32"]
    got = ol.dequant_q4k(blocks)
    assert np.array_equal(bits(got), bits(want))
    o = ol.oracle()
    # per-element and 16-span decoders agree with the row decoder
    for b in range(blocks.shape[0]):
        blk = np.ascontiguousarray(blocks[b])
        pe = np.array([o.knj_or_q4k_weight(ol.ptr(blk, ol.u8p), r) for r in range(256)], np.float32)
        assert np.array_equal(bits(pe), bits(want[b]))
        span = np.empty(16, np.float32)
        for r0 in range(0, 256, 16):
            o.knj_or_q4k_span16(ol.ptr(blk, ol.u8p), r0, ol.ptr(span, ol.f32p))
            assert np.array_equal(bits(span), bits(want[b, r0:r0 + 16]))


def test_q6k_crafted_blocks_bit_exact():
    """The Q6_K restatement (row decoder and per-element form) against the reference's decode of crafted blocks:
    random, all-0x00, all-0xFF, extreme int8 scales, fp16 corner values of d (tests/golden/golden_q6k.npz)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_q6k.npz"))
    blocks, want = g["q6k_blocks"], g["q6k_blocks_f32"]
    o = ol.oracle()
    got = np.empty_like(want)
    o.knj_or_dequant_q6k(ol.ptr(np.ascontiguousarray(blocks), ol.u8p), ol.ptr(got, ol.f32p), got.size)
    assert np.array_equal(bits(got), bits(want))
    for b in range(blocks.shape[0]):
        blk = np.ascontiguousarray(blocks[b])
        pe = np.array([o.knj_or_q6k_weight(ol.ptr(blk, ol.u8p), r) for r in range(256)], np.float32)
        assert np.array_equal(bits(pe), bits(want[b]))
    r = ol.ref()
    if r is not None:  # and directly against the compiled reference where it is present
        again = np.empty_like(want)
        r.ref_dequant_row_q6k(ol.ptr(np.ascontiguousarray(blocks), ol.u8p), ol.ptr(again, ol.f32p), again.size)
        assert np.array_equal(bits(again), bits(want))


def test_cfg1_dequant_and_gemv(golden):
    W = synth.q4k_rows(synth.stream(1, "gate"), synth.FFN, synth.HIDDEN)
    x = synth.stream(1, "x").standard_normal(synth.HIDDEN).astype(np.float32)
    assert sha(W) == str(golden["cfg1_w_sha"]) and sha(x) == str(golden["cfg1_x_sha"])
    full = ol.dequant_q4k(W).ravel()
    assert sha(full) == str(golden["cfg1_dequant_sha"])
    assert np.array_equal(bits(full[:512]), bits(golden["cfg1_dequant_head"]))
    y = ol.matmul_q4k(W, x[None])[0]
    assert np.array_equal(bits(y), bits(golden["cfg1_y"]))  # same f32 operation order -> bit equal


@pytest.mark.parametrize("m", [1, 5])
def test_moe_small(golden, m):
    bank = synth.expert_bank(102, n_experts=16, hidden=512, ffn=256)
    wr, _ = synth.router_weight(102, n_experts=16, hidden=512)
    assert sha(bank["gate"]) + sha(bank["up"]) + sha(bank["down"]) + sha(wr) == str(golden["moe_small_in_sha"])
    hx = synth.hidden_rows(102, m, 512, layer=m)
    out, ch, wt = ol.moe(wr, bank, hx, 4)
    assert np.array_equal(ch, golden[f"moe_small_m{m}_chosen"])
    assert np.array_equal(bits(wt), bits(golden[f"moe_small_m{m}_weight"]))
    assert np.array_equal(bits(out), bits(golden[f"moe_small_m{m}_out"]))


@pytest.mark.parametrize("m", [1, 8])
def test_cfg2_layer(golden, m):
    bank = synth.expert_bank(2)
    wr, _ = synth.router_weight(2)
    assert sha(bank["gate"]) + sha(bank["up"]) + sha(bank["down"]) + sha(wr) == str(golden["cfg2_in_sha"])
    hx = synth.hidden_rows(2, m, layer=m)
    out, ch, wt = ol.moe(wr, bank, hx)
    assert np.array_equal(ch, golden[f"cfg2_m{m}_chosen"])
    assert np.array_equal(bits(wt), bits(golden[f"cfg2_m{m}_weight"]))
    assert np.array_equal(bits(out), bits(golden[f"cfg2_m{m}_out"]))


def test_w4_known_answer(golden):
    o = ol.oracle()
    M, N, K = 32, 768, 2048
    Bq = np.zeros(N * (K // 128) * 68, np.uint8)
    A = np.zeros(M * K, np.int8)
    o.knj_or_w4_kat_problem(0x5EED1234, M, N, K, ol.ptr(Bq, ol.u8p), ol.ptr(A, ol.i8p))
    assert sha(Bq) == str(golden["w4_bq_sha"]) and sha(A) == str(golden["w4_act_sha"])
    act = np.empty(M * (K // 8) * 2, np.uint32)
    o.knj_or_deinterleave_activations(ol.ptr(A, ol.i8p), ol.ptr(act, ol.u32p), M, K)
    assert sha(act) == str(golden["w4_deint_sha"])
    C = np.empty((M, N), np.float32)
    o.knj_or_gemm_w4_reference(ol.ptr(Bq, ol.u8p), ol.ptr(A, ol.i8p), ol.ptr(C, ol.f32p), M, N, K)
    assert np.array_equal(bits(C), bits(golden["w4_c"]))
    # the integer device formula agrees with the double reference to the reference's 2e-3 bound
    Cm = np.empty((M, N), np.float32)
    o.knj_or_gemm_w4_i8_mirror(ol.ptr(Bq, ol.u8p), ol.ptr(A, ol.i8p), ol.ptr(Cm, ol.f32p), M, N, K)
    st = ol.compare(Cm, C)
    assert st["rel_rmse"] <= 2e-3 and st["nonzero"] == st["total"]
    asum = np.empty(M * (K // 128), np.int32)
    o.knj_or_build_asum(ol.ptr(A, ol.i8p), ol.ptr(asum, ol.i32p), M, K)
    assert np.array_equal(asum.reshape(M, K // 128), A.reshape(M, K // 128, 128).astype(np.int32).sum(-1))


def test_against_compiled_reference_when_present():
    r = ol.ref()
    if r is None:
        pytest.skip("compiled reference not present on this machine")
    rng = np.random.Generator(np.random.Philox(7))
    W = synth.q4k_rows(rng, 64, 1024)
    x = rng.standard_normal((3, 1024)).astype(np.float32)
    want = np.empty((3, 64), np.float32)
    r.ref_matmul_q4k(ol.ptr(W, ol.u8p), 1024, 64, ol.ptr(x, ol.f32p), 3, 1024, ol.ptr(want, ol.f32p), 64, 2)
    assert np.array_equal(bits(ol.matmul_q4k(W, x)), bits(want))
    want1 = np.empty((1, 64), np.float32)
    r.ref_matmul_q4k(ol.ptr(W, ol.u8p), 1024, 64, ol.ptr(x, ol.f32p), 1, 1024, ol.ptr(want1, ol.f32p), 64, 1)
    assert np.array_equal(bits(ol.matmul_q4k(W, x[:1])), bits(want1))


def test_compare_metric_matches_reference_definition():
    rng = np.random.default_rng(3)
    want = rng.standard_normal(1000).astype(np.float32)
    want[::7] = 0.0
    got = want + rng.standard_normal(1000).astype(np.float32) * 1e-3
    st = ol.compare(got, want)
    nz = want != 0
    rr = np.sqrt(((got[nz].astype(np.float64) - want[nz]) ** 2).sum() / (want[nz].astype(np.float64) ** 2).sum())
    assert abs(st["rel_rmse"] - rr) < 1e-12
    assert st["max_idx"] == int(np.argmax(np.abs(got.astype(np.float64) - want)))
    assert st["nonzero"] == int((got != 0).sum()) and st["total"] == 1000
