"""RMSNorm, router top-k and the permutation tables against the CPU path."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import bf16_dev, dev, report, routing_sets_match
from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H", [(1, 2048), (7, 2048), (3, 768)])
def test_rmsnorm(T, H):
    from kanjoos_b200 import ops
    x = synth.hidden_rows(40, T, H)
    wb = synth.norm_weight(40, 0, H)
    want = ol.rmsnorm(x, synth.bf16_bits_to_f32(wb), synth.RMS_EPS)
    got = ops.rmsnorm(dev(x), bf16_dev(wb), synth.RMS_EPS).cpu().numpy()
    # the CPU path sums x^2 sequentially in f32 (error ~ sqrt(H) ulp); the budget is the f32-accumulate one
    assert report(got, want, f"rmsnorm f32 {T}x{H}")["rel_rmse"] <= 1e-5
    got = ops.rmsnorm(dev(x).to(torch.bfloat16), bf16_dev(wb), synth.RMS_EPS).cpu().numpy()
    assert report(got, want, f"rmsnorm bf16-in {T}x{H}")["rel_rmse"] <= 1e-5


@pytest.mark.parametrize("T,E,k,zipf", [(1, 128, 8, None), (64, 128, 8, None), (300, 128, 8, 1.1), (9, 16, 4, None),
                                        (5, 8, 8, None), (33, 40, 3, None)])
def test_router_topk(T, E, k, zipf):
    from kanjoos_b200 import ops
    wr, bias = synth.router_weight(50 + E, n_experts=E, zipf_s=zipf)
    x = synth.hidden_rows(50, T)
    logits, pe, pw = ops.router_topk(dev(x), bf16_dev(wr), k, None if bias is None else dev(bias))
    lg_cpu, ch_cpu, wt_cpu = ol.route(wr, 1, x, E, k)
    if bias is not None:
        # the CPU path has no bias input: fold it in by re-running its selection on biased logits
        lg_cpu = lg_cpu + bias[None]
        ch_cpu = np.argsort(-lg_cpu, axis=1, kind="stable")[:, :k].astype(np.int32)
        pr = np.exp(lg_cpu - lg_cpu.max(1, keepdims=True))
        pr /= pr.sum(1, keepdims=True)
        sel = np.take_along_axis(pr, ch_cpu, 1)
        wt_cpu = (sel / sel.sum(1, keepdims=True)).astype(np.float32)
    assert report(logits.cpu().numpy(), lg_cpu, "router logits")["rel_rmse"] <= 1e-5
    ch_gpu = pe.cpu().numpy().reshape(T, k)
    checked, skipped = routing_sets_match(ch_gpu, lg_cpu, ch_cpu, k)
    assert checked >= T - max(1, T // 20), f"too many near-ties skipped: {skipped}"
    same = (ch_gpu == ch_cpu).all(1)
    assert np.abs(pw.cpu().numpy().reshape(T, k)[same] - wt_cpu[same]).max() <= 2e-6
    assert np.allclose(pw.cpu().numpy().reshape(T, k).sum(1), 1.0, atol=1e-6)
    # slot order: descending probability
    lgp = np.take_along_axis(lg_cpu, ch_gpu, 1)
    assert (np.diff(lgp, axis=1) <= 1e-5).all()


def test_router_tie_break_lowest_id():
    from kanjoos_b200 import ops
    E, H, k = 32, 256, 4
    wr = np.zeros((E, H), np.float32)  # all logits equal -> the k lowest ids win, in order
    x = np.ones((2, H), np.float32)
    _, pe, pw = ops.router_topk(dev(x), bf16_dev(synth.f32_to_bf16_bits(wr)), k)
    assert pe.cpu().tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
    assert np.allclose(pw.cpu().numpy(), 0.25)


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (64, 128, 8), (777, 128, 8), (5, 4, 2), (4099, 128, 8), (16384, 16, 2),
                                   (1100, 64, 8)])  # the last three take the counting-sort form (P >= 8192), one ragged
def test_permute_tables(T, E, k):
    from kanjoos_b200 import ops
    rng = np.random.default_rng(T)
    pe = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32).ravel()
    if T == 64:
        pe[:] = np.tile(np.arange(k), T)  # every token to the same k experts: others get 0 tokens
    if T == 16384:
        pe[::7] = -1  # pairs of experts that live elsewhere (expert-parallel plans) are skipped
    pair_idx, pair_cnt, exp_list, n_active = [t.cpu().numpy() for t in ops.moe_permute(dev(pe), E, T)]
    for e in range(E):
        want = np.nonzero(pe == e)[0]
        assert pair_cnt[e] == len(want)
        assert np.array_equal(pair_idx[e, :len(want)], want)
        assert (pair_idx[e, len(want):] == -1).all()
    hist = np.bincount(pe[pe >= 0], minlength=E)
    act = np.nonzero(hist)[0]
    assert n_active[0] == len(act) and np.array_equal(exp_list[:len(act)], act)
    assert n_active[1] == hist.max()
