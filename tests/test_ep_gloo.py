"""Host logic of the expert-parallel layer on CPU ranks (gloo, world_size 2 and
1): split sizes, dispatch/combine all-to-all, the receiving rank's local plan and
the inverse permutation. The arithmetic is supplied by a stand-in built on the
CPU restatement of the reference, so the sharded result must equal the
single-process Model::moe result bit for bit (same per-expert row order, same
ascending-expert combine)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from kanjoos_b200 import ep, synth

E, H, F, K, T = 8, 256, 256, 2, 12
CFG = 301


class OracleCompute:
    """LocalCompute stand-in on CPU tensors, arithmetic from oracle/."""

    def __init__(self, wr_bits, top_k):
        self.wr, self.top_k = wr_bits, top_k

    def route(self, x):
        _, ch, wt = ol.route(self.wr, 1, x.numpy(), self.wr.shape[0], self.top_k)
        return torch.from_numpy(ch.ravel().copy()), torch.from_numpy(wt.ravel().copy())

    def permute(self, pair_exp, n_exp, stride):
        pe = pair_exp.numpy()
        idx = np.full((n_exp, stride * self.top_k), -1, np.int32)
        cnt = np.zeros(n_exp, np.int32)
        for p, e in enumerate(pe):
            idx[e, cnt[e]] = p
            cnt[e] += 1
        return torch.from_numpy(idx), torch.from_numpy(cnt), None, None

    def pack(self, x, pair_idx, pair_cnt, n_exp, P):
        order = np.concatenate([pair_idx[e, :int(pair_cnt[e])].numpy() for e in range(n_exp)]).astype(np.int64)
        send = x[torch.from_numpy(order // self.top_k)].contiguous()
        pair_row = np.empty(P, np.int32)
        pair_row[order] = np.arange(P, dtype=np.int32)
        return send, torch.from_numpy(pair_row)

    def local_plan(self, recv_counts, stride):
        return ep.plan_from_counts(recv_counts)

    def expert_ffn(self, rows, bank, plan, n_rows, max_tokens):
        Y = np.zeros((n_rows, rows.shape[1]), np.float32)
        xr = rows.numpy()
        for e, ids in enumerate(plan):
            if not ids:
                continue
            g = ol.matmul_q4k(bank["gate"][e], xr[ids])
            u = ol.matmul_q4k(bank["up"][e], xr[ids])
            a = ol.silu_mul(g, u)
            Y[ids] = ol.matmul_q4k(bank["down"][e], a)
        return torch.from_numpy(Y)

    def combine(self, Yback, pair_row, pair_exp, pair_w, T_loc, out_dtype):
        out = np.zeros((T_loc, Yback.shape[1]), np.float32)
        pe, pw, pr, Y = pair_exp.numpy(), pair_w.numpy(), pair_row.numpy(), Yback.numpy()
        for t in range(T_loc):
            slots = sorted(range(self.top_k), key=lambda s: pe[t * self.top_k + s])
            for s in slots:
                p = t * self.top_k + s
                out[t] = out[t] + np.float32(pw[p]) * Y[pr[p]]
        return torch.from_numpy(out)


def problem():
    bank = synth.expert_bank(CFG, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(CFG, n_experts=E, hidden=H)
    hx = synth.hidden_rows(CFG, T, H)
    return bank, wr, hx


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bank, wr, hx = problem()
        e_loc, t_loc = E // world, T // world
        local = {k: np.ascontiguousarray(v[rank * e_loc:(rank + 1) * e_loc]) for k, v in bank.items()}
        layer = ep.EpMoeLayer(local, E, OracleCompute(wr, K), None, K)
        x = torch.from_numpy(hx[rank * t_loc:(rank + 1) * t_loc].copy())
        out = layer.forward(x)
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.numpy())
        np.save(os.path.join(out_dir, f"rows{rank}.npy"), np.array([layer.last_stats["rows_received"]]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_equals_single_process(tmp_path, world):
    bank, wr, hx = problem()
    want, chosen, _ = ol.moe(wr, bank, hx, K)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # every routed pair reached the rank that owns its expert
    rows = [int(np.load(tmp_path / f"rows{r}.npy")[0]) for r in range(world)]
    owner_rows = np.bincount(chosen.ravel() // (E // world), minlength=world)
    assert rows == owner_rows.tolist() and sum(rows) == T * K


def test_world_one_takes_the_same_path(tmp_path):
    bank, wr, hx = problem()
    want, _, _ = ol.moe(wr, bank, hx, K)
    layer = ep.EpMoeLayer(bank, E, OracleCompute(wr, K), None, K)
    got = layer.forward(torch.from_numpy(hx.copy())).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_split_sizes_and_plan():
    counts = torch.tensor([[1, 0, 2, 3], [0, 4, 1, 0]], dtype=torch.int32)  # [src rank][global expert], 2 ranks x 2 local
    send, recv, rc = ep.split_sizes(counts, 0, 2, 2)
    assert send == [1, 5] and recv == [1, 4] and rc.tolist() == [[1, 0], [0, 4]]
    send, recv, rc = ep.split_sizes(counts, 1, 2, 2)
    assert send == [4, 1] and recv == [5, 1] and rc.tolist() == [[2, 3], [1, 0]]
    assert ep.plan_from_counts(rc) == [[0, 1, 5], [2, 3, 4]]
