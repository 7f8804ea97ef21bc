"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle_lib as ol

SENTINEL = -12345.0  # the reference's poison value (tools/bench/q4k_moe_ffn.hip:96)


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_dev(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.detach().cpu().numpy()


def report(got, want, what=""):
    """The reference's metric: rel-RMSE over all outputs, max-abs, unwritten count."""
    g = np.ascontiguousarray(got, dtype=np.float32)
    st = ol.compare(g, want)
    st["unwritten"] = int((g == SENTINEL).sum())
    print(f"[parity] {what}: rel_rmse={st['rel_rmse']:.3e} max_abs={st['max_abs']:.3e} out_rms={st['out_rms']:.3e} "
          f"worst_idx={st['max_idx']} unwritten={st['unwritten']} total={st['total']}")
    return st


def routing_sets_match(chosen_gpu: np.ndarray, logits_cpu: np.ndarray, chosen_cpu: np.ndarray, k: int, tol=1e-5):
    """Top-k sets must be identical wherever the k-th / (k+1)-th logit gap is
    larger than accumulation-order noise; returns (n_checked, n_skipped)."""
    checked = skipped = 0
    for t in range(chosen_cpu.shape[0]):
        srt = np.sort(logits_cpu[t])[::-1]
        gap = srt[k - 1] - srt[k] if logits_cpu.shape[1] > k else np.inf
        if gap <= tol * max(1.0, np.abs(srt).max()):
            skipped += 1
            continue
        assert set(chosen_gpu[t].tolist()) == set(chosen_cpu[t].tolist()), f"token {t}: routed sets differ"
        checked += 1
    return checked, skipped
