"""The tcgen05 grouped GEMMs alone (gate+up with SiLU*up epilogue, down)
against the CPU restatement, on ragged per-expert buckets: empty experts, a
1-token bucket, buckets that are not multiples of 16, and one above 256 tokens
(two buckets). Tolerance: rel-RMSE <= 1e-3 over every output (the budget of the
tensor-core path); fp16 operands land near 3e-4."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import dev, report
from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 1e-3


def ragged_problem(E, F, H, counts, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    T = int(sum(counts))  # one pair per token here (top_k = 1)
    pe = np.concatenate([np.full(c, e, np.int32) for e, c in enumerate(counts)])
    pe = pe[rng.permutation(T)]
    Wg = synth.q4k_rows(rng, E * F, H).reshape(E, F, H // 256, 144)
    Wu = synth.q4k_rows(rng, E * F, H).reshape(E, F, H // 256, 144)
    Wd = synth.q4k_rows(rng, E * H, F).reshape(E, H, F // 256, 144)
    x = synth.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    return pe, Wg, Wu, Wd, x


@pytest.mark.parametrize("E,F,H,counts,single_sm", [
    (4, 256, 256, [5, 0, 1, 40], 0),
    (3, 256, 512, [16, 300, 0], 0),
    (2, 768, 2048, [33, 7], 0),
    (3, 256, 512, [16, 300, 0], 1),   # the same buckets on single SMs (tcgen05 cta_group::1)
    (2, 256, 768, [130, 9], 0),       # 768 = 3 x 256 rows of the down matrix: odd tile count, single-SM form
    (2, 256, 256, [256, 255], 0),     # a full bucket and one token short of it, CTA pairs
])
def test_grouped_gemms(E, F, H, counts, single_sm):
    from kanjoos_b200 import ops, _lib
    _lib.lib().knj_q4k_tc_single_sm(single_sm)
    try:
        _grouped_gemms(ops, E, F, H, counts)
    finally:
        _lib.lib().knj_q4k_tc_single_sm(0)


def _grouped_gemms(ops, E, F, H, counts):
    pe, Wg, Wu, Wd, x = ragged_problem(E, F, H, counts, [E, F, H])
    T = len(pe)
    pair_idx, pair_cnt, _, _ = ops.moe_permute(dev(pe), E, T)
    xh = ops.to_f16(dev(x))
    A, st = ops.q4k_gateup_tc(xh, dev(Wg), dev(Wu), pair_idx, pair_cnt, T, 1)
    torch.cuda.synchronize()
    assert int(st.item()) == 0, "a bounded wait inside the kernel gave up"
    A_host = A.float().cpu().numpy() * 64.0
    want_a = np.zeros((T, F), np.float32)
    for e in range(E):
        rows = np.nonzero(pe == e)[0]
        if len(rows) == 0:
            continue
        g = ol.matmul_q4k(Wg[e], x[rows])
        u = ol.matmul_q4k(Wu[e], x[rows])
        want_a[rows] = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
    assert not np.isnan(A_host).any(), "unwritten activation outputs"
    stt = report(A_host, want_a, f"tc gate+up E={E} F={F} H={H} counts={counts}")
    assert stt["rel_rmse"] <= TOL

    # down on the device's own fp16 activations (so this step is judged alone)
    Y, st = ops.q4k_down_tc(A, dev(Wd), pair_idx, pair_cnt, T)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want_y = np.zeros((T, H), np.float32)
    for e in range(E):
        rows = np.nonzero(pe == e)[0]
        if len(rows):
            want_y[rows] = ol.matmul_q4k(Wd[e], np.ascontiguousarray(A_host[rows]))
    sty = report(Y.cpu().numpy(), want_y, "tc down")
    assert sty["unwritten"] == 0 and sty["rel_rmse"] <= TOL


@pytest.mark.parametrize("E,F,H,counts,single_sm", [
    (3, 256, 512, [16, 300, 0], 0),    # CTA pairs, a ragged and a two-bucket expert, an empty one
    (2, 768, 2048, [33, 7], 0),        # the full-size down shape: three superblocks per row
    (2, 512, 384, [130, 9], 0),        # 384 = 3 x 128 rows: odd tile count, single-SM form
    (2, 1024, 256, [256, 255], 1),     # four superblocks per row (the staging's limit), single SMs forced
])
def test_q6k_down_gemm(E, F, H, counts, single_sm):
    """The grouped down GEMM over Q6_K weights (whole-tile staging, per-slab decode) against the CPU decoder and
    a double-precision product, on fp16 activations scaled as the gate+up GEMM writes them."""
    from kanjoos_b200 import ops, _lib
    rng = np.random.Generator(np.random.Philox([E, F, H, 6]))
    T = int(sum(counts))
    pe = np.concatenate([np.full(c, e, np.int32) for e, c in enumerate(counts)])
    pe = pe[rng.permutation(T)]
    nsb = F // 256
    W6 = rng.integers(0, 256, size=(E, H, nsb, 210), dtype=np.uint8)
    W6[..., 208:210] = (np.abs(rng.standard_normal((E, H, nsb, 1))) * 0.01).astype(np.float16).view(np.uint8)
    Wd = np.empty((E * H * nsb, 256), np.float32)
    ol.oracle().knj_or_dequant_q6k(ol.ptr(W6, ol.u8p), ol.ptr(Wd, ol.f32p), Wd.size)
    Wd = Wd.reshape(E, H, F)
    a = (rng.standard_normal((T, F)) * 3.0).astype(np.float32)
    ah = torch.from_numpy((a / 64.0).astype(np.float16)).cuda()      # the 2^-6 prescale of the stored activations
    a_seen = ah.float().cpu().numpy() * 64.0
    pair_idx, pair_cnt, _, _ = ops.moe_permute(dev(pe), E, T)
    _lib.lib().knj_q4k_tc_single_sm(single_sm)
    try:
        Y, st = ops.q6k_down_tc(ah, dev(W6), pair_idx, pair_cnt, T)
        torch.cuda.synchronize()
    finally:
        _lib.lib().knj_q4k_tc_single_sm(0)
    assert int(st.item()) == 0, "a bounded wait inside the kernel gave up"
    want = np.zeros((T, H), np.float32)
    for e in range(E):
        rows = np.nonzero(pe == e)[0]
        if len(rows):
            want[rows] = (a_seen[rows].astype(np.float64) @ Wd[e].astype(np.float64).T).astype(np.float32)
    sty = report(Y.cpu().numpy(), want, f"tc down, Q6_K, E={E} F={F} H={H} counts={counts}")
    assert sty["unwritten"] == 0 and sty["rel_rmse"] <= TOL
