"""The MoE-FFN layer through the C-ABI against the CPU path (restated
Model::moe) and the golden vectors of the compiled reference.
Tolerances: rel-RMSE <= 1e-5 over every output for the f32-accurate (decode)
path; <= 1e-3 for the bf16 tensor-core (prefill) path."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from gpu_util import SENTINEL, bf16_dev, dev, report, routing_sets_match
from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu

TOL_DECODE = 1e-5
TOL_PREFILL = 1e-3


def make_layer(bank, wr, top_k, max_tokens, bias=None, norm=None, residual=False):
    from kanjoos_b200.moe import ExpertBank, MoeFfnLayer
    eb = ExpertBank.from_numpy(bank, wr, bias, norm)
    return MoeFfnLayer(eb, top_k=top_k, max_tokens=max_tokens, residual=residual, use_norm=norm is not None)


@pytest.fixture(scope="module")
def cfg2():
    bank = synth.expert_bank(2)
    wr, _ = synth.router_weight(2)
    return bank, wr


@pytest.mark.parametrize("m", [1, 5])
def test_small_layer_vs_golden(golden, m):
    bank = synth.expert_bank(102, n_experts=16, hidden=512, ffn=256)
    wr, _ = synth.router_weight(102, n_experts=16, hidden=512)
    hx = synth.hidden_rows(102, m, 512, layer=m)
    layer = make_layer(bank, wr, 4, 8)
    out, pe, pw = layer.decode(dev(hx), return_routing=True)
    assert np.array_equal(pe.cpu().numpy().reshape(m, 4), golden[f"moe_small_m{m}_chosen"])
    st = report(out.cpu().numpy(), golden[f"moe_small_m{m}_out"], f"small layer m={m}")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE


@pytest.mark.parametrize("m", [1, 8])
def test_cfg2_decode_vs_golden(golden, cfg2, m):
    """Config 2: the Qwen3-30B-A3B-shaped layer, decode batch 1 (and 8), bf16 hidden rows."""
    bank, wr = cfg2
    hx = synth.hidden_rows(2, m, layer=m)
    layer = make_layer(bank, wr, 8, 8)
    x = dev(hx).to(torch.bfloat16)  # exactly representable: generated through bf16
    out, pe, pw = layer.decode(x, return_routing=True)
    assert np.array_equal(np.sort(pe.cpu().numpy().reshape(m, 8), 1), np.sort(golden[f"cfg2_m{m}_chosen"], 1))
    st = report(out.cpu().numpy(), golden[f"cfg2_m{m}_out"], f"cfg2 decode B={m}")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE


def test_cfg2_decode_batch64(cfg2):
    bank, wr = cfg2
    hx = synth.hidden_rows(2, 64, layer=64)
    want, ch, wt = ol.moe(wr, bank, hx)
    layer = make_layer(bank, wr, 8, 64)
    out, pe, _ = layer.decode(dev(hx), return_routing=True)
    lg, _, _ = ol.route(wr, 1, hx, 128, 8)
    routing_sets_match(pe.cpu().numpy().reshape(64, 8), lg, ch, 8)
    st = report(out.cpu().numpy(), want, "cfg2 decode B=64")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE


def test_all_tokens_to_one_expert_and_empty_experts():
    """A bias that forces every token onto the same top-k: k experts get all the
    tokens, the rest get none."""
    bank = synth.expert_bank(103, n_experts=8, hidden=256, ffn=256)
    wr, _ = synth.router_weight(103, n_experts=8, hidden=256)
    bias = np.full(8, -60.0, np.float32)  # exp(-60) vanishes in f32 softmax; chosen logits keep full precision
    bias[[2, 5]] = 0.0
    hx = synth.hidden_rows(103, 37, 256)
    layer = make_layer(bank, wr, 2, 40, bias=bias)
    out, pe, pw = layer.decode(dev(hx), return_routing=True)
    assert set(pe.cpu().tolist()) == {2, 5}
    # CPU path with the same forced routing: bias folded into an f32 router of one extra input
    wr_f = np.concatenate([synth.bf16_bits_to_f32(wr), bias[:, None]], 1).astype(np.float32)
    hx1 = np.concatenate([hx, np.ones((37, 1), np.float32)], 1)
    _, ch, wt = ol.route(wr_f, 0, hx1, 8, 2)
    want = np.zeros_like(hx)
    for e in (2, 5):
        rows = np.nonzero((ch == e).any(1))[0]
        g = ol.matmul_q4k(bank["gate"][e], hx[rows])
        u = ol.matmul_q4k(bank["up"][e], hx[rows])
        a = (g / (1.0 + np.exp(-g))) * u
        y = ol.matmul_q4k(bank["down"][e], a.astype(np.float32))
        w = np.array([wt[r][list(ch[r]).index(e)] for r in rows], np.float32)
        want[rows] += w[:, None] * y
    st = report(out.cpu().numpy(), want, "forced routing, 37 tokens -> 2 experts")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE


def test_norm_residual_and_bf16_out():
    """RMSNorm ahead of the router, residual add after, bf16 residual stream:
    one layer of the resident stack (config 4's layer step)."""
    bank = synth.expert_bank(104, n_experts=16, hidden=512, ffn=256)
    wr, _ = synth.router_weight(104, n_experts=16, hidden=512)
    nb = synth.norm_weight(104, 0, 512)
    hx = synth.hidden_rows(104, 6, 512)
    xn = ol.rmsnorm(hx, synth.bf16_bits_to_f32(nb), synth.RMS_EPS)
    moe_out, _, _ = ol.moe(wr, bank, xn, 4)
    want = hx + moe_out
    layer = make_layer(bank, wr, 4, 8, norm=nb, residual=True)
    out32 = layer.decode(dev(hx).to(torch.bfloat16), out_dtype=torch.float32)
    assert report(out32.cpu().numpy(), want, "norm+moe+residual f32 out")["rel_rmse"] <= TOL_DECODE
    out16 = layer.decode(dev(hx).to(torch.bfloat16), out_dtype=torch.bfloat16)
    assert report(out16.float().cpu().numpy(), synth.bf16_round(want), "bf16 out")["rel_rmse"] <= 3e-3


def test_zero_tokens_is_a_no_op(cfg2):
    bank, wr = cfg2
    layer = make_layer(bank, wr, 8, 8)
    out = layer.decode(torch.empty((0, synth.HIDDEN), dtype=torch.float32, device="cuda"))
    assert out.shape == (0, synth.HIDDEN)


def test_stack_of_layers_and_graph_replay():
    """Three layers of the resident decode loop (RMSNorm -> MoE -> residual, bf16
    stream) against the CPU path layer by layer; a CUDA-graph replay gives the
    same bits as eager launches."""
    from kanjoos_b200.moe import ExpertBank, MoeStack
    L, E, H, F, k, B = 3, 16, 512, 256, 4, 3
    banks, cpu = [], []
    for l in range(L):
        bank = synth.expert_bank(105, l, n_experts=E, hidden=H, ffn=F)
        wr, _ = synth.router_weight(105, l, n_experts=E, hidden=H)
        nb = synth.norm_weight(105, l, H)
        banks.append(ExpertBank.from_numpy(bank, wr, None, nb))
        cpu.append((bank, wr, nb))
    stack = MoeStack(banks, top_k=k, max_tokens=4)
    x0 = synth.hidden_rows(105, B, H) * 200.0  # residual of the size the layers produce
    x0 = synth.bf16_round(x0)
    x = dev(x0).to(torch.bfloat16)
    got = stack.step(x).float().cpu().numpy()
    cur = x0
    for bank, wr, nb in cpu:
        xn = ol.rmsnorm(cur, synth.bf16_bits_to_f32(nb), synth.RMS_EPS)
        mo, _, _ = ol.moe(wr, bank, xn, k)
        cur = synth.bf16_round(cur + mo)
    st = report(got, cur, "3-layer stack, bf16 stream")
    assert st["rel_rmse"] <= 1e-2  # bf16 stream: one rounding flip per layer is 4e-3 of an element
    g, out = stack.capture(x)
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), got)


def test_prefill_t512_zipf(cfg2):
    """Config 3: T=512, router biased so expert popularity follows Zipf(1.1)."""
    bank, _ = cfg2
    wr, bias = synth.router_weight(3, zipf_s=1.1)
    hx = synth.hidden_rows(3, 512)
    layer = make_layer(bank, wr, 8, 512, bias=bias)
    out, pe, pw = layer.prefill(dev(hx).to(torch.bfloat16), return_routing=True)
    ch = pe.cpu().numpy().reshape(512, 8)
    cnt = np.bincount(ch.ravel(), minlength=128)
    print("zipf bucket sizes: max", cnt.max(), "min", cnt.min(), "empty", int((cnt == 0).sum()))
    # CPU path on the device's routing decision (the CPU router has no bias input)
    wts = pw.cpu().numpy().reshape(512, 8)
    want = np.zeros_like(hx)
    for e in np.nonzero(cnt)[0]:
        rows, slots = np.nonzero(ch == e)
        g = ol.matmul_q4k(bank["gate"][e], hx[rows])
        u = ol.matmul_q4k(bank["up"][e], hx[rows])
        a = ((g / (1.0 + np.exp(-g))) * u).astype(np.float32)
        y = ol.matmul_q4k(bank["down"][e], a)
        want[rows] += wts[rows, slots][:, None] * y
    st = report(out.cpu().numpy(), want, "cfg3 prefill T=512 Zipf(1.1)")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_PREFILL


def test_decode_b64_zipf_unbalanced_experts(cfg2):
    """Batch 64 with a Zipf(1.1) router: a few experts hold far more tokens than one pass of the projection
    kernels takes, the case in which their work is split by token pass. Combine order on the CPU side is
    ascending expert id, as in the CPU path."""
    bank, _ = cfg2
    wr, bias = synth.router_weight(3, zipf_s=1.1)
    hx = synth.hidden_rows(3, 64, layer=64)
    layer = make_layer(bank, wr, 8, 64, bias=bias)
    out, pe, pw = layer.decode(dev(hx), return_routing=True)
    ch = pe.cpu().numpy().reshape(64, 8)
    cnt = np.bincount(ch.ravel(), minlength=128)
    print("zipf bucket sizes at batch 64: max", cnt.max(), "experts above 8 tokens", int((cnt > 8).sum()))
    assert cnt.max() > 8
    wts = pw.cpu().numpy().reshape(64, 8)
    want = np.zeros_like(hx)
    for e in np.nonzero(cnt)[0]:
        rows, slots = np.nonzero(ch == e)
        g = ol.matmul_q4k(bank["gate"][e], hx[rows])
        u = ol.matmul_q4k(bank["up"][e], hx[rows])
        a = ((g / (1.0 + np.exp(-g))) * u).astype(np.float32)
        y = ol.matmul_q4k(bank["down"][e], a)
        want[rows] += wts[rows, slots][:, None] * y
    st = report(out.cpu().numpy(), want, "decode batch 64 Zipf(1.1)")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE


def test_mixed_format_layer_q6k_down():
    """A layer whose down matrices are Q6_K (as half of them are in Q4_K_M files): decode launch against the CPU
    pieces -- router, Q4_K gate/up and SiLU*up from the restatement, Q6_K decode + double-precision product for
    down, weighted sum in ascending expert order."""
    E, H, F, k, T = 8, 512, 256, 2, 6
    bank = synth.expert_bank(105, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(105, n_experts=E, hidden=H)
    rng = np.random.Generator(np.random.Philox(105))
    nblk = F // 256
    W6 = rng.integers(0, 256, size=(E, H, nblk, 210), dtype=np.uint8)
    W6[..., 208:210] = (np.abs(rng.standard_normal((E, H, nblk, 1))) * 0.01).astype(np.float16).view(np.uint8)
    Wd = np.empty((E * H * nblk, 256), np.float32)
    ol.oracle().knj_or_dequant_q6k(ol.ptr(W6, ol.u8p), ol.ptr(Wd, ol.f32p), Wd.size)
    Wd = Wd.reshape(E, H, F)
    hx = synth.hidden_rows(105, T, H)
    _, ch, wt = ol.route(wr, 1, hx, E, k)
    want = np.zeros_like(hx)
    for t in range(T):
        for s_ in sorted(range(k), key=lambda s_: ch[t][s_]):
            e = int(ch[t][s_])
            g = ol.matmul_q4k(bank["gate"][e], hx[t:t + 1])
            u = ol.matmul_q4k(bank["up"][e], hx[t:t + 1])
            a = ol.silu_mul(g, u)[0]
            y = (Wd[e].astype(np.float64) @ a.astype(np.float64)).astype(np.float32)
            want[t] = want[t] + np.float32(wt[t][s_]) * y
    mixed = dict(bank, down=W6)
    layer = make_layer(mixed, wr, k, T)
    out = layer.decode(dev(hx))
    st = report(out.cpu().numpy(), want, "mixed-format layer (Q6_K down), decode launch")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_DECODE
    # the prefill launch takes the Q6_K down matrices through the tensor-core grouped GEMM
    pre = layer.prefill(dev(hx))
    st = report(pre.cpu().numpy(), want, "mixed-format layer (Q6_K down), prefill launch")
    assert st["unwritten"] == 0 and st["rel_rmse"] <= TOL_PREFILL


def _sample_want(bank, hx, ch, wts, sample):
    """CPU path on the device's routing decision for the sampled tokens (a token's output depends on its own
    row only), experts in ascending order as the CPU path sums them."""
    want = np.zeros((len(sample), hx.shape[1]), np.float32)
    chs, ws = ch[sample], wts[sample]
    for e in np.unique(chs):
        rows, slots = np.nonzero(chs == e)
        xs = hx[sample[rows]]
        g = ol.matmul_q4k(bank["gate"][e], xs)
        u = ol.matmul_q4k(bank["up"][e], xs)
        y = ol.matmul_q4k(bank["down"][e], ol.silu_mul(g, u))
        want[rows] += ws[rows, slots][:, None] * y
    return want


@pytest.fixture(scope="module")
def cfg5():
    return synth.expert_bank(5)


@pytest.mark.parametrize("T,routing", [(4096, "uniform"), (4096, "zipf"), (16384, "uniform"), (16384, "zipf")])
def test_config5_prefill_sampled_tokens(cfg5, T, routing):
    """Config 5 on one GPU at the benchmark's sizes (every expert holds several full 256-token buckets): 256
    seeded tokens of the layer's output against the CPU path, both combine forms; routing sets against the CPU
    router for the unbiased case."""
    bank = cfg5
    wr, bias = synth.router_weight(5, zipf_s=1.1 if routing == "zipf" else None)
    hx = synth.bf16_round(synth.hidden_rows(5, T))
    layer = make_layer(bank, wr, 8, T, bias=bias)
    x = dev(hx).to(torch.bfloat16)
    out, pe, pw = layer.prefill(x, return_routing=True, fused_combine=True)
    ch, wts = pe.cpu().numpy().reshape(T, 8), pw.cpu().numpy().reshape(T, 8)
    cnt = np.bincount(ch.ravel(), minlength=128)
    print(f"T={T} {routing}: bucket sizes max {cnt.max()} min {cnt.min()}")
    sample = np.sort(np.random.Generator(np.random.Philox([T, len(routing)])).choice(T, 256, replace=False))
    want = _sample_want(bank, hx, ch, wts, sample)
    got = out.cpu().numpy()
    st = report(got[sample], want, f"cfg5 prefill T={T} {routing}, fused combine, 256 sampled tokens")
    assert (got == SENTINEL).sum() == 0 and st["rel_rmse"] <= TOL_PREFILL
    ordered = layer.prefill(x).cpu().numpy()
    st = report(ordered[sample], want, f"cfg5 prefill T={T} {routing}, ordered combine")
    assert st["rel_rmse"] <= TOL_PREFILL
    # the two combine forms differ by the order of eight f32 additions per output only
    assert report(got, ordered, "fused vs ordered combine, all tokens")["rel_rmse"] <= 1e-6
    if routing == "uniform":
        logits, ch_cpu, _ = ol.route(wr, 1, hx[sample], 128, 8)
        checked, skipped = routing_sets_match(ch[sample], logits, ch_cpu, 8)
        assert checked >= 200


def test_prefill_combine_forms_with_residual_and_bf16_output(cfg2):
    """The fused epilogue starts the token's sum from the residual row and ends in a bf16 store; the ordered form
    is bit-reproducible from run to run."""
    bank, wr = cfg2
    hx = synth.bf16_round(synth.hidden_rows(2, 300, layer=7))
    layer = make_layer(bank, wr, 8, 300, residual=True)
    x = dev(hx).to(torch.bfloat16)
    fused = layer.prefill(x, out_dtype=torch.bfloat16, fused_combine=True).float().cpu().numpy()
    o1 = layer.prefill(x, out_dtype=torch.bfloat16).float().cpu().numpy()
    o2 = layer.prefill(x, out_dtype=torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(o1, o2)
    assert np.mean(fused != o1) < 0.01 and report(fused, o1, "fused vs ordered, bf16 out + residual")["rel_rmse"] <= 5e-3
    want, _, _ = ol.moe(wr, bank, hx)
    assert report(o1, synth.bf16_round(hx + want), "ordered, residual, bf16 out vs CPU path")["rel_rmse"] <= 5e-3
