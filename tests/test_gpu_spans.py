"""The device-span ring behind a host profiler: eager layer launches are bracketed per stage, offsets come from
one epoch on the stream, a full ring counts what it drops, captured launches record nothing."""
import numpy as np
import pytest
import torch

from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu


def _layer(T):
    from kanjoos_b200.moe import ExpertBank, MoeFfnLayer
    bank = synth.expert_bank(601, n_experts=8, hidden=512, ffn=256)
    wr, _ = synth.router_weight(601, n_experts=8, hidden=512)
    eb = ExpertBank.from_numpy(bank, wr)
    x = torch.from_numpy(synth.hidden_rows(601, T, 512)).cuda()
    return MoeFfnLayer(eb, top_k=2, max_tokens=T, use_norm=False), x


def test_prefill_stages_are_recorded_in_order():
    from kanjoos_b200.profiling import DeviceSpans
    layer, x = _layer(64)
    layer.prefill(x)  # warm-up outside the recording
    with DeviceSpans(capacity=64) as spans:
        with spans.span("step"):
            layer.prefill(x)
        with spans.span("step"):
            layer.prefill(x)
    names = [r[0] for r in spans.rows]
    stages = ["moe-router", "moe-gather", "moe-gate", "moe-down", "moe-scatter"]
    assert names == ["step"] + stages + ["step"] + stages and spans.dropped == 0
    for (_, a, b) in spans.rows:
        assert 0 <= a <= b
    inner = [r for r in spans.rows if r[0] != "step"]
    assert all(inner[i][2] <= inner[i + 1][1] + 1000 for i in range(len(inner) - 1))  # stages follow one another
    tab = spans.table()
    assert tab["step"][0] == 2 and tab["moe-gate"][0] == 2
    outer = sum(b - a for n, a, b in spans.rows if n == "step")
    assert abs(sum(t for _, t in tab.values()) - outer) <= 0.01 * outer + 2000  # self times add up to the steps


def test_decode_stages_and_full_ring():
    from kanjoos_b200.profiling import DeviceSpans
    layer, x = _layer(4)
    layer.decode(x)
    with DeviceSpans(capacity=64) as spans:
        layer.decode(x)
    assert [r[0] for r in spans.rows] == ["moe-router", "moe-gate", "moe-down"]
    with DeviceSpans(capacity=2) as small:
        layer.decode(x)
        layer.decode(x)
    assert len(small.rows) == 2 and small.dropped == 4


def test_captured_launches_record_nothing():
    from kanjoos_b200.profiling import DeviceSpans
    layer, x = _layer(4)
    out = torch.empty_like(x)
    layer.decode(x, out=out)
    torch.cuda.synchronize()
    with DeviceSpans(capacity=16) as spans:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            layer.decode(x, out=out)
        g.replay()
        torch.cuda.synchronize()
    assert spans.rows == [] and spans.dropped == 0


def test_reference_profiler_fed_from_the_span_ring():
    """The reference's own Profiler (its profiler.cpp, compiled where it lies into oracle/_ref/knj_ref_profiler_check
    together with oracle/ref_profiler_check.cpp) receives the spans of three eager layer launches through
    knj_spans_flush -> Profiler::device_span and reports them: Device domain, all spans counted, none dropped,
    rows named as the CPU path's stages. The binary is built where the reference tree exists (make -C oracle ref)
    and travels prebuilt; it is test infrastructure."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "knj_ref_profiler_check")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/knj_ref_profiler_check was not built (no reference tree on the build machine)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout
