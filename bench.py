#!/usr/bin/env python
"""Benchmark of the Q4_K MoE-FFN path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--tokens T] [--routing uniform|zipf] [--no-decode]

Workload (all N): the expert-parallel MoE layer of the benchmark configs --
Qwen3-30B-A3B geometry (hidden 2048, ffn 768, 128 experts, top-8), T tokens per
step (default 4096, bf16 ~ N(0,1)), random-init Q4_K experts split evenly over
the N GPUs, token dispatch/combine by all-to-all when N > 1. One step = one pass
of the layer over the T tokens; value = tokens/s of the whole job. Total work is
fixed as N grows ("strong" scaling). Successive steps rotate over several
distinct weight banks so the weights a step reads never sit in L2 from the step
before. At N = 1 the line also carries the decode numbers (48-layer resident
stack, batch 1/8/64) with their HBM roofline, and a CPU baseline.

--impl reference times the reference's own CPU code for the same layer
(oracle/_ref when present, else the C restatement) on the host cores, on a
bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, F, E, TOPK, LAYERS = 2048, 768, 128, 8, 48
EXPERT_BYTES = 3 * F * (H // 256) * 144  # 2,654,208
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """SM clock and throttle reasons sampled every few milliseconds while the timed regions run
    (NVML reads only; nvidia-smi polling as the fallback)."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.sm, self.mx, self.reasons = index, [], None, set()
        self.proc, self.th, self.stop_flag, self.nvml = None, None, threading.Event(), None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and all(v.strip().isdigit() for v in vis.split(",")) else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.th = threading.Thread(target=self._poll_nvml, daemon=True)
            self.th.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read_smi, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _poll_nvml(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for bit, name in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.003)

    def _read_smi(self):
        for line in self.proc.stdout:
            r = [c.strip() for c in line.split(",")]
            if len(r) < 6:
                continue
            try:
                self.sm.append(float(r[0]))
                self.mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)

    def stop(self):
        if self.nvml is None and not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"], "samples": 0}
        self.stop_flag.set()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.th:
            self.th.join(timeout=3)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.mx, "reasons": sorted(self.reasons),
                "samples": len(sm), "source": "nvml" if self.nvml else "nvidia-smi"}


# --------------------------------------------------------------------------- reference arm

def cpu_layer_tokens_per_s(sample_tokens: int, steps: int, warmup: int, routing: str):
    """The reference's CPU MoE layer on a bounded sample of the workload."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    from kanjoos_b200 import synth
    bank = synth.expert_bank(5)
    wr, bias = synth.router_weight(5, zipf_s=1.1 if routing == "zipf" else None)
    hx = synth.hidden_rows(5, sample_tokens)
    r = ol.ref()
    out = np.empty((sample_tokens, H), np.float32)
    if r is not None:
        kind, cores = "reference", r.ref_hardware_threads()

        def run():
            r.ref_moe(ol.ptr(wr, ol.u16p), ol.ptr(bank["gate"], ol.u8p), ol.ptr(bank["up"], ol.u8p),
                      ol.ptr(bank["down"], ol.u8p), ol.ptr(hx, ol.f32p), sample_tokens, H, E, TOPK, F,
                      ol.ptr(out, ol.f32p), None, None, cores)
    else:
        kind, cores = "port", ol.oracle().knj_or_num_threads()

        def run():
            ol.moe(wr, bank, hx, TOPK)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    return {"value": sample_tokens / dt, "unit": "tokens/s", "cores": int(cores), "kind": kind,
            "sample": f"{sample_tokens} tokens of the layer per step (uniform router; the CPU path has no bias input), "
                      f"{steps} steps, wall clock"}, dt


def run_reference(args):
    """The reference arm: the reference's own CPU layer on the host cores. One of its steps is a bounded SAMPLE
    of the workload's step (cpu_sample tokens of the T), and the line says so: `steps` / `warmup` are the steps
    actually run, `ms_per_step` is the time of one sample step, and `config` carries both token counts."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, min(args.steps, 5)), min(args.warmup, 1)
    cb, dt = cpu_layer_tokens_per_s(args.cpu_sample, steps, warm, args.routing)
    cfg = workload_config(args, args.gpus)
    cfg["sample_tokens_per_step"] = args.cpu_sample
    cfg["sample_note"] = (f"each timed step runs {args.cpu_sample} of the workload's {args.tokens} tokens on the host "
                          "(per-token cost of the CPU path does not depend on T); value = sample tokens / sample time")
    line = {"impl": "reference", "metric": "moe_ffn_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "steps_requested": args.steps,
            "ms_per_step": dt * 1e3, "ms_per_full_step_extrapolated": dt * 1e3 * args.tokens / args.cpu_sample,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(args, world):
    q6 = getattr(args, "down_format", "q4k") == "q6k"
    return {"workload": f"ep_moe_layer_T{args.tokens}_{args.routing}" + ("_q6k_down" if q6 else ""), "hidden": H, "ffn": F,
            "experts": E, "top_k": TOPK, "tokens_per_step": args.tokens, "experts_per_gpu": E // world,
            "weight_format": "GGUF Q4_K gate/up, Q6_K down" if q6 else "GGUF Q4_K",
            "l2_policy": "inputs larger than L2: steps rotate over distinct weight banks",
            "parallelism": f"ep{world}"}


# --------------------------------------------------------------------------- GPU arm

def decode_section(torch, steps, warmup, pk, layers=LAYERS, batches=(1, 8, 64), inputs=("chained", "fresh"), down="q4k"):
    """Resident stack (48 layers by default): tokens/s and HBM roofline of the decode path, one cooperative launch
    per step (knj_moe_stack_*). Two inputs per batch: `chained` feeds each layer the previous layer's output (the
    decode loop as it runs; with random-init weights the residual stream concentrates the routing on a third of
    the experts after a few layers) and `fresh` gives every layer its own N(0,1) rows (the expert spread of a
    trained router: ~126 of 128 experts at batch 64). Algorithmic bytes use the distinct experts actually routed."""
    from kanjoos_b200.moe import ExpertBank, FusedMoeStack
    banks = [ExpertBank.random(seed=1000 + l) for l in range(layers)]
    # down == "mixed": every second layer's down matrices are Q6_K, as Q4_K_M files hold them; "q6k": every layer's
    q6_layers = [l for l in range(layers) if down == "q6k" or (down == "mixed" and l % 2 == 1)]
    q6_down_bytes = H * (F // 256) * 210
    for l in q6_layers:
        g6 = torch.Generator(device="cuda")
        g6.manual_seed(9000 + l)
        w6 = torch.randint(0, 256, (E, H, F // 256, 210), dtype=torch.uint8, device="cuda", generator=g6)
        d6 = (torch.randn((E, H, F // 256, 1), device="cuda", generator=g6).abs() * 0.002).to(torch.float16)
        w6[..., 208:210] = d6.view(torch.uint8).reshape(E, H, F // 256, 2)
        banks[l].down = w6
    expert_bytes = [EXPERT_BYTES - F * (H // 256) * 144 + q6_down_bytes if l in q6_layers else EXPERT_BYTES for l in range(layers)]
    out = {"layers": layers, "down_format": down, "q6k_down_layers": len(q6_layers),
           "resident_weight_gib": round(E * sum(expert_bytes) / 2**30, 2), "batches": {}}
    for B in batches:
        g = torch.Generator(device="cuda")
        g.manual_seed(B)
        x = torch.randn((B, H), device="cuda", generator=g).to(torch.bfloat16)
        for mode in inputs:
            if mode == "fresh" and B == 1:
                continue  # one token routes to eight experts whatever its row is
            ins = ([torch.randn((B, H), device="cuda", generator=g).to(torch.bfloat16) for _ in range(layers)]
                   if mode == "fresh" else None)
            stack = FusedMoeStack(banks, top_k=TOPK, n_tokens=B, taps=True, layer_inputs=ins)
            for _ in range(max(3, warmup)):
                stack.step(x)
            stack.status()
            per_layer = [int(torch.unique(t[0]).numel()) for t in stack.taps]
            distinct = sum(per_layer)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            reps = max(steps, int(0.3 / max(1e-4, layers * 150e-6)))  # at least ~0.3 s of timed launches
            ev[0].record()
            for _ in range(reps):
                stack.step()
            ev[1].record()
            torch.cuda.synchronize()
            stack.status()
            ms = ev[0].elapsed_time(ev[1]) / reps
            alg = sum(d * eb for d, eb in zip(per_layer, expert_bytes)) + layers * (E * H * 2 + H * 2 + B * H * 2 * 2)
            key = str(B) if mode == "chained" else f"{B}_fresh"
            out["batches"][key] = {"tokens_per_s": B / (ms * 1e-3), "ms_per_step": ms, "timed_steps": reps,
                                   "path": "one cooperative launch per step (knj_moe_stack_decode_launch)",
                                   "inputs": mode, "distinct_experts_per_layer": distinct / layers,
                                   "algorithmic_bytes": alg, "hbm_gbs": alg / (ms * 1e-3) / 1e9,
                                   "frac_of_" + pk["_source"]: alg / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
            stack.close()
            del stack
    del banks
    torch.cuda.empty_cache()
    return out


def check_parity(torch, args, world, rank, e_loc, n_banks, banks, router, bias, x, step, out):
    """Relative RMSE of the layer's output rows against an independent computation (never timed)."""
    import numpy as np
    from kanjoos_b200 import ops
    from kanjoos_b200.moe import ExpertBank, MoeFfnLayer
    got_all = out.float().cpu().numpy()   # the step over bank 0 that every rank has just run
    if world == 1:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as ol
        n = 64
        bk = banks[0]
        bank = {k: getattr(bk, k).cpu().numpy() for k in ("gate", "up", "down")}
        _, pe, pw = ops.router_topk(x[:n].contiguous(), router, TOPK, bias)
        ch, wts = pe.cpu().numpy().reshape(n, TOPK), pw.cpu().numpy().reshape(n, TOPK)
        hx = x[:n].float().cpu().numpy()
        want = np.zeros((n, H), np.float32)
        for e in np.unique(ch):
            rows, slots = np.nonzero(ch == e)
            g = ol.matmul_q4k(bank["gate"][e], hx[rows])
            u = ol.matmul_q4k(bank["up"][e], hx[rows])
            a = ol.silu_mul(g, u)
            if bank["down"].shape[-1] == 210:   # Q6_K: the CPU decoder and a double-precision product
                w6 = np.ascontiguousarray(bank["down"][e])
                wd = np.empty((w6.shape[0] * w6.shape[1], 256), np.float32)
                ol.oracle().knj_or_dequant_q6k(ol.ptr(w6, ol.u8p), ol.ptr(wd, ol.f32p), wd.size)
                y = (a.astype(np.float64) @ wd.reshape(w6.shape[0], -1).astype(np.float64).T).astype(np.float32)
            else:
                y = ol.matmul_q4k(bank["down"][e], a)
            want[rows] += wts[rows, slots][:, None] * y
        ref_kind = "CPU path (oracle) on the device's routing decision"
    else:
        n = min(256, x.shape[0])
        parts = [ExpertBank.random(n_experts=e_loc, seed=100 + 1000 * r, with_norm=False) for r in range(world)]
        full = ExpertBank(gate=torch.cat([b.gate for b in parts]), up=torch.cat([b.up for b in parts]),
                          down=torch.cat([b.down for b in parts]), router=router, router_bias=bias)
        layer = MoeFfnLayer(full, top_k=TOPK, max_tokens=n, use_norm=False)
        want = layer.prefill(x[:n].contiguous()).cpu().numpy()
        del parts, full, layer
        ref_kind = "single-GPU layer over all experts (ordered combine)"
    got = got_all[:n]
    d = (got.astype(np.float64) - want.astype(np.float64))
    rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
    return {"rel_rmse": float(np.sqrt((d ** 2).mean()) / max(rms, 1e-30)), "max_abs": float(np.abs(d).max()),
            "n_tokens": int(n), "against": ref_kind, "note": "the timed workload with f32 output rows"}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.down_format == "q6k" and world > 1:
        raise SystemExit("--down-format q6k is a single-GPU measurement (the expert-parallel layer holds Q4_K banks)")
    from kanjoos_b200 import _lib, ops
    from kanjoos_b200.ep import CudaCompute, EpMoeLayer
    from kanjoos_b200.moe import ExpertBank, MoeFfnLayer
    _lib.check(_lib.lib().knj_dev_open(local))
    pk = peaks()
    if args.section == "decode":
        # decode-only run (used for profiling captures): one line about the resident stack
        dec = decode_section(torch, args.steps, args.warmup, pk, args.decode_layers,
                             tuple(int(b) for b in args.decode_batches.split(",")), tuple(args.decode_inputs.split(",")),
                             args.decode_down)
        print(json.dumps({"metric": "moe_ffn_decode", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                          "data": "synthetic", "decode": dec}))
        return

    T = args.tokens
    assert T % world == 0 and E % world == 0
    T_loc, e_loc = T // world, E // world
    bank_bytes = e_loc * EXPERT_BYTES
    n_banks = max(2, math.ceil(400e6 / bank_bytes))
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    router = (torch.randn((E, H), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    bias = None
    if args.routing == "zipf":
        p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.1
        perm = torch.randperm(E, generator=torch.Generator().manual_seed(3))
        b = torch.empty(E, dtype=torch.float32)
        b[perm] = torch.log(p / p.sum()).float()
        bias = b.cuda()
    banks = []
    for i in range(n_banks):
        bk = ExpertBank.random(n_experts=e_loc, seed=100 + 17 * i + 1000 * rank, with_norm=False)
        bk.router, bk.router_bias = router, bias
        if args.down_format == "q6k":
            g6 = torch.Generator(device="cuda")
            g6.manual_seed(7000 + i)
            w6 = torch.randint(0, 256, (e_loc, H, F // 256, 210), dtype=torch.uint8, device="cuda", generator=g6)
            d6 = (torch.randn((e_loc, H, F // 256, 1), device="cuda", generator=g6).abs() * 0.002).to(torch.float16)
            w6[..., 208:210] = d6.view(torch.uint8).reshape(e_loc, H, F // 256, 2)
            bk.down = w6
        banks.append(bk)
    gx = torch.Generator(device="cuda")
    gx.manual_seed(11 + rank)
    x = torch.randn((T_loc, H), device="cuda", generator=gx).to(torch.bfloat16)
    out = torch.empty((T_loc, H), dtype=torch.bfloat16, device="cuda")

    if world == 1:
        layers = [MoeFfnLayer(bk, top_k=TOPK, max_tokens=T_loc, use_norm=False) for bk in banks[:1]]
        ws = layers[0].workspace
        layers += [MoeFfnLayer(bk, top_k=TOPK, max_tokens=T_loc, use_norm=False, workspace=ws) for bk in banks[1:]]

        def step(i, xin=x, dst=out):
            layers[i % n_banks].prefill(xin, out=dst)
    else:
        cp = CudaCompute(router, TOPK, bias)
        eps = [EpMoeLayer(bk, E, cp, None, TOPK, exchange=args.exchange) for bk in banks]

        def step(i, xin=x, dst=out):
            eps[i % n_banks].forward(xin, out=dst)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    W = max(3, args.warmup)
    for i in range(W):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # a first pass of K steps sizes the timed region: the K-step loop is repeated until it lasts half a second
    barrier()
    e0.record()
    for i in range(args.steps):
        step(W + i)
    e1.record()
    barrier()
    probe = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(probe, op=dist.ReduceOp.MAX)
    repeats = max(1, int(math.ceil(500.0 / max(float(probe.item()), 1e-3))))
    barrier()
    e0.record()
    for r in range(repeats):
        for i in range(args.steps):
            step(W + i)
    e1.record()
    barrier()
    ms_step = e0.elapsed_time(e1) / (args.steps * repeats)

    # end to end: pinned host rows in, bf16 result rows out, every step's copies inside the timed region.
    # Three streams and two device buffers per direction: the copy-in of step i+1 and the copy-out of
    # step i-1 overlap the compute of step i (PCIe is full duplex); nothing is cached across steps.
    hx = torch.empty((T_loc, H), dtype=torch.bfloat16).pin_memory()
    hx.copy_(x.cpu())
    hout = [torch.empty((T_loc, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    xin = [torch.empty_like(x) for _ in range(2)]
    dout = [torch.empty_like(out) for _ in range(2)]
    s_c = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_run(n, first):
        ev_in = [None, None]     # copy-in of the step that last used buffer b
        ev_comp = [None, None]   # compute of that step
        ev_out = [None, None]    # copy-out of that step
        for k in range(n):
            b = k & 1
            with torch.cuda.stream(s_in):
                if ev_comp[b] is not None:
                    s_in.wait_event(ev_comp[b])      # the step two back has read xin[b]
                xin[b].copy_(hx, non_blocking=True)
                ev_in[b] = torch.cuda.Event()
                ev_in[b].record(s_in)
            s_c.wait_event(ev_in[b])
            if ev_out[b] is not None:
                s_c.wait_event(ev_out[b])            # dout[b] has been copied out
            step(first + k, xin[b], dout[b])
            ev_comp[b] = torch.cuda.Event()
            ev_comp[b].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                hout[b].copy_(dout[b], non_blocking=True)
                ev_out[b] = torch.cuda.Event()
                ev_out[b].record(s_out)
        s_c.wait_stream(s_out)
        s_c.wait_stream(s_in)

    e2e_run(2, 0)
    barrier()
    e0.record()
    e2e_run(args.steps * repeats, W)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / (args.steps * repeats)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_step, ms_e2e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e = t.tolist()

    # dominant kernel alone (rank 0): gate+up grouped product on this rank's rows, CUDA events on its stream
    roof = None
    imbalance = None
    if rank == 0:
        _, pe, _ = ops.router_topk(x, router, TOPK, bias)
        # load imbalance of this rank's tokens: busiest expert / mean and busiest expert owner / mean
        per_e = torch.bincount(pe.long(), minlength=E).double()
        per_r = per_e.view(world, e_loc).sum(1)
        imbalance = {"per_expert": float(per_e.max() / per_e.mean()), "per_rank": float(per_r.max() / per_r.mean())}
        own = (pe // e_loc) == 0 if world > 1 else torch.ones_like(pe, dtype=torch.bool)
        rows = int(own.sum().item()) if world > 1 else T_loc * TOPK
        # plan over this rank's experts only, tokens from the local shard stand in for received rows
        pe_loc = torch.where(own, pe % e_loc, torch.full_like(pe, -1)) if world > 1 else pe
        pair_idx, pair_cnt, exp_list, n_active = ops.moe_permute(pe_loc.contiguous(), e_loc, T_loc * TOPK)
        xh = ops.to_f16(x)
        A = torch.empty((T_loc * TOPK, F), dtype=torch.float16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        import ctypes as C

        def gateup(i):
            bk = banks[i % n_banks]
            _lib.check(_lib.lib().knj_q4k_gateup_tc_launch(
                C.c_void_p(xh.data_ptr()), C.c_void_p(bk.gate.data_ptr()), C.c_void_p(bk.up.data_ptr()),
                C.c_void_p(pair_idx.data_ptr()), C.c_void_p(pair_cnt.data_ptr()), None, C.c_void_p(A.data_ptr()), F, H,
                (H // 256) * 144, pair_idx.shape[1], e_loc, TOPK, T_loc * TOPK, C.c_void_p(status.data_ptr()),
                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        for i in range(3):
            gateup(i)
        torch.cuda.synchronize()
        e0.record()
        for i in range(args.steps):
            gateup(3 + i)
        e1.record()
        torch.cuda.synchronize()
        ms_k = e0.elapsed_time(e1) / args.steps
        # the down GEMM alone, over the rows the gate+up launch has just left in A
        Y = torch.empty((T_loc * TOPK, H), dtype=torch.float32, device="cuda")

        def down(i):
            bk = banks[i % n_banks]
            common = (C.c_void_p(pair_idx.data_ptr()), C.c_void_p(pair_cnt.data_ptr()), None, C.c_void_p(Y.data_ptr()), H, F)
            tail = (pair_idx.shape[1], e_loc, T_loc * TOPK, C.c_void_p(status.data_ptr()),
                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
            if bk.down.shape[-1] == 210:
                _lib.check(_lib.lib().knj_q6k_down_tc_launch(C.c_void_p(A.data_ptr()), C.c_void_p(bk.down.data_ptr()), *common, *tail))
            else:
                _lib.check(_lib.lib().knj_q4k_down_tc_launch(C.c_void_p(A.data_ptr()), C.c_void_p(bk.down.data_ptr()), *common,
                                                             (F // 256) * 144, *tail))
        for i in range(3):
            down(i)
        torch.cuda.synchronize()
        e0.record()
        for i in range(args.steps):
            down(3 + i)
        e1.record()
        torch.cuda.synchronize()
        ms_d = e0.elapsed_time(e1) / args.steps
        del Y
        flops = rows * 2 * 2 * H * F
        t_tensor = flops / (pk["bf16_tflops"] * 1e12)
        assert int(status.item()) == 0, "a bounded wait inside the grouped GEMM gave up"
        # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum of this kernel) as ncu counted them on
        # this workload in a one-pass capture of the same command: at T=16384 532.3 + 184.3 MB, at T=4096
        # 261.5 + 38.7 MB (uniform router, N=1); other sizes have no capture
        w_bytes = int((pair_cnt > 0).sum().item()) * 2 * F * (H // 256) * 144
        measured = {(16384, "uniform"): 716.6e6, (4096, "uniform"): 300.2e6}
        traffic = measured.get((T, args.routing)) if world == 1 else None
        traffic_note = ("ncu one-pass DRAM counters of this kernel on this workload; algorithmic bytes (weights once + fp16 rows "
                        "in + fp16 rows out) = %.1f MB" % ((w_bytes + rows // TOPK * H * 2 + rows * F * 2) / 1e6)) if traffic else None
        roof = {"kernel": "q4k_grouped_tc_kernel<2,true,2> (gate+up, tcgen05 cta_group::2)", "bound": "tensor", "achieved": flops / (ms_k * 1e-3) / 1e12,
                "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": flops / (ms_k * 1e-3) / 1e12 / pk["bf16_tflops"],
                "peak_source": pk["_source"], "traffic": traffic, "traffic_note": traffic_note, "ms_per_launch": ms_k,
                "algorithmic_flops_per_launch": flops,
                "weight_bytes_per_launch": int((pair_cnt > 0).sum().item()) * 2 * F * (H // 256) * 144,
                "t_tensor_ms": t_tensor * 1e3,
                "down": {"kernel": ("q4k_grouped_tc_kernel<1,false,2,1> (Q6_K down)" if args.down_format == "q6k"
                                    else "q4k_grouped_tc_kernel<2,false,2> (Q4_K down)"),
                         "ms_per_launch": ms_d, "achieved": rows * 2 * H * F / (ms_d * 1e-3) / 1e12, "unit": "TFLOP/s",
                         "frac": rows * 2 * H * F / (ms_d * 1e-3) / 1e12 / pk["bf16_tflops"]}}

    # parity, outside the timed regions: the first rows of rank 0's shard against the CPU path (N = 1: 64 tokens on
    # the device's routing decision) or against the single-GPU layer over the same experts (N > 1: 256 tokens)
    parity = None
    out32 = torch.empty((T_loc, H), dtype=torch.float32, device="cuda")
    step(0, x, out32)   # bank 0 with f32 output rows, every rank takes part
    barrier()
    if rank == 0:
        parity = check_parity(torch, args, world, rank, e_loc, n_banks, banks, router, bias, x, step, out32)
        if parity["rel_rmse"] > 1e-3:
            raise SystemExit(f"parity check failed: {parity}")

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    cb = None
    dec = None
    if world == 1:
        if args.cpu_sample > 0 and args.down_format == "q4k":   # the CPU arm is the Q4_K layer
            cb, _ = cpu_layer_tokens_per_s(args.cpu_sample, 3, 1, "uniform")
        if not args.no_decode and args.down_format == "q4k":
            del banks, layers
            torch.cuda.empty_cache()
            dec = decode_section(torch, max(5, args.steps), args.warmup, pk)

    # kernels of this library per layer step: router logits + top-k, permutation (count, scan, scatter for
    # P >= 8192, else one kernel) + active list, to_f16, gate+up, down, then combine (N = 1) or the exchange kernels
    n_perm = 4 if T * TOPK >= 8192 else 2
    if world == 1:
        launches = 2 + n_perm + 1 + 2 + 1
    elif args.exchange == "peer":
        # rows to fp16, router (2), table stores, arrival, wait, local expert ids, plan, gate+up, down, partial sums to
        # the owners, arrival, wait, rank reduce (the rows themselves travel as copy-engine copies, not kernels)
        launches = 1 + 2 + 1 + 1 + 1 + 1 + n_perm + 2 + 1 + 1 + 1 + 1
    elif args.exchange == "gather":
        launches = 2 + 1 + n_perm + 2 + 2
    else:
        launches = 2 + n_perm + 2 + 2 + 1 + 2 + 1  # pack (2), plan (2)
    line = {"metric": "moe_ffn_tokens_per_s", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "timed_repeats": repeats, "timed_steps": args.steps * repeats, "warmup": W,
            "ms_per_step": ms_step, "parity": parity, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16 operands (Q4_K unpacked), f32 accumulate", "data": "synthetic",
            "config": dict(workload_config(args, world), routing_imbalance=imbalance), "clocks": clocks,
            "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T_loc * H * 2 * world,
                    "d2h_bytes_per_step": T_loc * H * 2 * world, "ms_per_step": ms_e2e},
            "gpu_launches": launches * args.steps * repeats, "roofline": roof, "cpu_baseline": cb, "decode": dec,
            "flops_per_step": T * TOPK * 3 * 2 * H * F + 2 * T * H * E}
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--routing", default="uniform", choices=["uniform", "zipf"])
    ap.add_argument("--cpu-sample", type=int, default=1024, dest="cpu_sample")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--down-format", default="q4k", choices=["q4k", "q6k"], dest="down_format",
                    help="q6k: the layer's down matrices are Q6_K, as in the mixed-format layers of Q4_K_M files (N = 1, "
                         "prefill section only)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "gather", "dispatch"], help="expert-parallel exchange (N > 1)")
    ap.add_argument("--section", default="all", choices=["all", "decode"])
    ap.add_argument("--decode-layers", type=int, default=LAYERS, dest="decode_layers")
    ap.add_argument("--decode-batches", default="1,8,64", dest="decode_batches")
    ap.add_argument("--decode-down", default="q4k", choices=["q4k", "q6k", "mixed"], dest="decode_down",
                    help="--section decode: down matrices of the resident stack; mixed = Q6_K in every second layer, as "
                         "Q4_K_M files hold them")
    ap.add_argument("--decode-inputs", default="chained,fresh", dest="decode_inputs",
                    help="per-layer inputs of the decode section: chained (each layer feeds the next), fresh, or both")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
