"""Expert-parallel MoE-FFN layer: experts split contiguously over the ranks of
a torch.distributed group (owner(e) = e // (E / world)), tokens data-parallel.

Per step and rank: route the local tokens -> pack hidden rows in (destination,
expert, pair) order -> all-to-all #1 (dispatch, bf16 rows) -> grouped expert FFN
on the received rows -> all-to-all #2 (combine, f32 rows back to their source)
-> ordered weighted sum. torch.distributed carries the exchange (NCCL on GPUs,
gloo in the CPU tests); every kernel is a C-ABI call of libknj_device.so.

With world == 1 the same kernels run with pack and exchange elided (rows are
gathered straight from the token buffer through the pair->token map).

The arithmetic is delegated to a `LocalCompute` object so the host logic
(counts, splits, plan, inverse permutation) can be exercised on CPU ranks with
a stand-in compute in the tests.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import synth


def split_sizes(counts_all: torch.Tensor, rank: int, world: int, e_loc: int):
    """counts_all int [world][E]: pairs each rank routes to each global expert.
    Returns (send_splits, recv_splits, recv_counts [world][e_loc]) for `rank`."""
    per_dest = counts_all.view(world, world, e_loc).sum(-1)  # [src][dst]
    send = per_dest[rank].tolist()
    recv = per_dest[:, rank].tolist()
    recv_counts = counts_all[:, rank * e_loc:(rank + 1) * e_loc].contiguous()
    return send, recv, recv_counts


def plan_from_counts(recv_counts: torch.Tensor):
    """Host restatement of knj_ep_plan: rows from source r arrive contiguously,
    experts ascending. Returns per local expert the list of received-row ids."""
    world, e_loc = recv_counts.shape
    rows = [[] for _ in range(e_loc)]
    base = 0
    for r in range(world):
        for e in range(e_loc):
            c = int(recv_counts[r, e])
            rows[e].extend(range(base, base + c))
            base += c
    return rows


class CudaCompute:
    """The kernels of libknj_device.so behind the LocalCompute interface."""

    def __init__(self, router: torch.Tensor, top_k: int, router_bias: torch.Tensor | None = None):
        from . import ops  # deferred: needs the CUDA library
        self.ops, self.router, self.top_k, self.bias = ops, router, top_k, router_bias

    def route(self, x):
        _, pe, pw = self.ops.router_topk(x, self.router, self.top_k, self.bias)
        return pe, pw

    def permute(self, pair_exp, E, stride):
        return self.ops.moe_permute(pair_exp, E, stride)

    def pack(self, x, pair_idx, pair_cnt, E, P):
        from ._lib import check, lib
        row_bytes = x.shape[1] * x.element_size()
        send = torch.empty((P, x.shape[1]), dtype=x.dtype, device=x.device)
        off = torch.empty(E + 1, dtype=torch.int32, device=x.device)
        pair_row = torch.empty(P, dtype=torch.int32, device=x.device)
        check(lib().knj_ep_pack_launch(C.c_void_p(x.data_ptr()), row_bytes, self.top_k, C.c_void_p(pair_idx.data_ptr()),
                                       pair_idx.shape[1], C.c_void_p(pair_cnt.data_ptr()), E, C.c_void_p(off.data_ptr()),
                                       C.c_void_p(send.data_ptr()), C.c_void_p(pair_row.data_ptr()),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return send, pair_row

    def local_plan(self, recv_counts, stride):
        from ._lib import check, lib
        world, e_loc = recv_counts.shape
        dev = recv_counts.device
        pair_idx = torch.empty((e_loc, stride), dtype=torch.int32, device=dev)
        pair_cnt = torch.empty(e_loc, dtype=torch.int32, device=dev)
        exp_list = torch.empty(e_loc, dtype=torch.int32, device=dev)
        n_active = torch.empty(4, dtype=torch.int32, device=dev)
        check(lib().knj_ep_plan_launch(C.c_void_p(recv_counts.data_ptr()), world, e_loc, stride,
                                       C.c_void_p(pair_idx.data_ptr()), C.c_void_p(pair_cnt.data_ptr()),
                                       C.c_void_p(exp_list.data_ptr()), C.c_void_p(n_active.data_ptr()),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return pair_idx, pair_cnt, exp_list, n_active

    def expert_ffn(self, rows, bank, plan, n_rows, max_tokens):
        """rows [R][H] -> Y f32 [R][H]; row i of `rows` is pair i of the local plan."""
        pair_idx, pair_cnt, exp_list, n_active = plan
        ops = self.ops
        xp = ops.act_prep(rows)
        A = ops.q4k_gateup(xp, bank.gate, bank.up, pair_idx, pair_cnt, exp_list, n_active, n_rows, 1, max_tokens,
                           want=("A",))["A"]
        ap = ops.act_prep(A)
        return ops.q4k_proj(ap, bank.down, pair_idx, pair_cnt, exp_list, n_active, n_rows, max_tokens)

    def combine(self, Yback, pair_row, pair_exp, pair_w, T, out_dtype):
        return self.ops.moe_combine(Yback, pair_exp, pair_w, T, self.top_k, out_dtype=out_dtype, pair_row=pair_row)


class EpMoeLayer:
    """One expert-parallel MoE-FFN layer on this rank.

    bank: the LOCAL experts (E/world of them, ids rank*E/world ...); the router
    weight inside `compute` covers all E experts and is replicated.
    """

    def __init__(self, bank, n_experts: int, compute, group=None, top_k: int = synth.TOP_K):
        self.bank, self.E, self.compute, self.group, self.top_k = bank, n_experts, compute, group, top_k
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert n_experts % self.world == 0
        self.e_loc = n_experts // self.world
        self.last_stats = {}

    def forward(self, x: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
        T, H = x.shape
        P = T * self.top_k
        cp = self.compute
        pair_exp, pair_w = cp.route(x)
        pair_idx, pair_cnt, _, _ = cp.permute(pair_exp, self.E, max(T, 1))
        if self.world == 1:
            counts_all = pair_cnt.view(1, self.E)
            recv_counts = counts_all
            send_rows, pair_row = cp.pack(x, pair_idx, pair_cnt, self.E, P)
            recv_rows = send_rows
            n_recv = P
        else:
            counts_all = torch.empty((self.world, self.E), dtype=torch.int32, device=x.device)
            dist.all_gather_into_tensor(counts_all.view(-1), pair_cnt, group=self.group)
            send_rows, pair_row = cp.pack(x, pair_idx, pair_cnt, self.E, P)
            send, recv, recv_counts = split_sizes(counts_all.cpu(), self.rank, self.world, self.e_loc)
            recv_counts = recv_counts.to(x.device)
            n_recv = sum(recv)
            recv_rows = torch.empty((n_recv, H), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(recv_rows, send_rows, recv, send, group=self.group)
        plan = cp.local_plan(recv_counts, max(n_recv, 1))
        self.last_stats = {"rows_received": int(n_recv)}
        Y = cp.expert_ffn(recv_rows, self.bank, plan, n_recv, n_recv)
        if self.world == 1:
            Yback = Y
        else:
            Yback = torch.empty((P, H), dtype=torch.float32, device=x.device)
            dist.all_to_all_single(Yback, Y, send, recv, group=self.group)
        return cp.combine(Yback, pair_row, pair_exp, pair_w, T, out_dtype)
