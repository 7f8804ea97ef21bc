"""Host logic of the expert-parallel layer on CPU ranks (gloo, world_size 1, 2
and 4), both exchanges. The arithmetic is supplied by a stand-in built on the CPU
restatement of the reference.
"dispatch": split sizes, per-pair all-to-all, the receiving rank's local plan and
the inverse permutation; the sharded result must equal the single-process
Model::moe result bit for bit (same per-expert row order, same ascending-expert
combine).
"gather": all-gather of rows and routing tables, the plan restricted to the
rank's experts, per-token partial sums, equal-split all-to-all and the
rank-ordered sum; bit-equal at world 1, and equal up to the regrouping of the f32
additions (<= 1e-6 relative RMSE) at world 2 and 4."""
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


def _gather_methods():
    """The gather-exchange half of the stand-in (added to OracleCompute below)."""

    def plan_for_experts(self, pair_exp_all, exp_lo, e_loc, stride):
        pe = pair_exp_all.numpy()
        return [[int(p) for p in np.nonzero(pe == exp_lo + e)[0]] for e in range(e_loc)]

    def expert_ffn_tokens(self, x_all, bank, plan, P, hint):
        xr = x_all.numpy()
        Y = np.full((P, xr.shape[1]), np.nan, np.float32)  # rows of foreign pairs must never be read
        for e, pairs in enumerate(plan):
            if not pairs:
                continue
            rows = xr[[p // self.top_k for p in pairs]]
            g = ol.matmul_q4k(bank["gate"][e], rows)
            u = ol.matmul_q4k(bank["up"][e], rows)
            Y[pairs] = ol.matmul_q4k(bank["down"][e], ol.silu_mul(g, u))
        return torch.from_numpy(Y)

    def combine_partial(self, Y, pair_exp_all, pair_w_all, T_all, exp_lo, exp_hi):
        pe, pw, Yn = pair_exp_all.numpy(), pair_w_all.numpy(), Y.numpy()
        out = np.zeros((T_all, Yn.shape[1]), np.float32)
        for t in range(T_all):
            slots = [s for s in range(self.top_k) if exp_lo <= pe[t * self.top_k + s] < exp_hi]
            for s in sorted(slots, key=lambda s: pe[t * self.top_k + s]):
                p = t * self.top_k + s
                out[t] = out[t] + np.float32(pw[p]) * Yn[p]
        return torch.from_numpy(out)

    def reduce_parts(self, parts, out_dtype):
        acc = parts[0].numpy().copy()
        for r in range(1, parts.shape[0]):
            acc = acc + parts[r].numpy()
        return torch.from_numpy(acc)

    return plan_for_experts, expert_ffn_tokens, combine_partial, reduce_parts


(OracleCompute.plan_for_experts, OracleCompute.expert_ffn_tokens, OracleCompute.combine_partial,
 OracleCompute.reduce_parts) = _gather_methods()


def problem():
    bank = synth.expert_bank(CFG, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(CFG, n_experts=E, hidden=H)
    hx = synth.hidden_rows(CFG, T, H)
    return bank, wr, hx


def _rank_main(rank, world, port, out_dir, exchange="dispatch"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bank, wr, hx = problem()
        e_loc, t_loc = E // world, T // world
        local = {k: np.ascontiguousarray(v[rank * e_loc:(rank + 1) * e_loc]) for k, v in bank.items()}
        layer = ep.EpMoeLayer(local, E, OracleCompute(wr, K), None, K, exchange=exchange)
        x = torch.from_numpy(hx[rank * t_loc:(rank + 1) * t_loc].copy())
        out = layer.forward(x)
        np.save(os.path.join(out_dir, f"out{rank}.npy"), out.numpy())
        np.save(os.path.join(out_dir, f"rows{rank}.npy"), np.array([layer.last_stats.get("rows_received", -1)]))
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
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), "dispatch"), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # every routed pair reached the rank that owns its expert
    rows = [int(np.load(tmp_path / f"rows{r}.npy")[0]) for r in range(world)]
    owner_rows = np.bincount(chosen.ravel() // (E // world), minlength=world)
    assert rows == owner_rows.tolist() and sum(rows) == T * K


@pytest.mark.parametrize("world", [2, 4])
def test_gather_exchange_matches_single_process(tmp_path, world):
    bank, wr, hx = problem()
    want, _, _ = ol.moe(wr, bank, hx, K)
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), "gather"), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    st = ol.compare(np.ascontiguousarray(got, dtype=np.float32), want)
    assert st["rel_rmse"] <= 1e-6, st  # same products, additions regrouped per rank


@pytest.mark.parametrize("exchange", ["dispatch", "gather"])
def test_world_one_takes_the_same_path(tmp_path, exchange):
    bank, wr, hx = problem()
    want, _, _ = ol.moe(wr, bank, hx, K)
    layer = ep.EpMoeLayer(bank, E, OracleCompute(wr, K), None, K, exchange=exchange)
    got = layer.forward(torch.from_numpy(hx.copy())).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_split_sizes_and_plan():
    counts = torch.tensor([[1, 0, 2, 3], [0, 4, 1, 0]], dtype=torch.int32)  # [src rank][global expert], 2 ranks x 2 local
    send, recv, rc = ep.split_sizes(counts, 0, 2, 2)
    assert send == [1, 5] and recv == [1, 4] and rc.tolist() == [[1, 0], [0, 4]]
    send, recv, rc = ep.split_sizes(counts, 1, 2, 2)
    assert send == [4, 1] and recv == [5, 1] and rc.tolist() == [[2, 3], [1, 0]]
    assert ep.plan_from_counts(rc) == [[0, 1, 5], [2, 3, 4]]
