"""Expert-parallel MoE-FFN layer: experts split contiguously over the ranks of
a torch.distributed group (owner(e) = e // (E / world)), tokens data-parallel.

Two exchanges are implemented behind `EpMoeLayer(exchange=...)`:

"gather" (default when every rank holds the same number of tokens): all-gather
the token rows and the routing tables (pair_exp, pair_w) -> every rank runs the
grouped expert FFN for the pairs of ITS experts, reading token rows through the
pair -> token map (no per-pair copies of rows) -> per-token partial sums over the
rank's experts -> equal-split all-to-all of the partial rows -> sum over ranks
in ascending rank order. Per rank and step (N-1)/N * T * (row + 8 k bytes) come
in and (N-1)/N * T * 4 H bytes go out, independent of k; all sizes are static, so
the step needs no host synchronisation.

"peer": the gather exchange carried by this library's own kernels over NVLink
peer mappings (torch symmetric memory gives every rank pointers to every other
rank's exchange buffers). Steps whose buckets are large enough for the
tensor-core GEMMs run as ONE C-ABI call on the library's layer object
(knj_ep_forward_launch): rows and routing tables are stored into the peers'
buffers while the router runs, flag barriers in peer memory order the ranks,
partial rows are stored straight into the token owner's buffer and only for
tokens that have an expert on the sending rank; no allocation and no
collective in the step. Smaller steps pull the rows with plain loads, run the
f32-accurate kernels, and use two small all-reduces as barriers. CUDA only.

"dispatch": route -> pack hidden rows in (destination, expert, pair) order ->
all-to-all #1 (one row per routed pair) -> grouped expert FFN on the received
rows -> all-to-all #2 (one f32 row per pair back) -> ordered weighted sum. Moves
k rows per token each way and needs the split sizes on the host; kept for ranks
with unequal token counts and as the bit-exact restatement of the single-device
order (its result equals the single-process result bit for bit).

torch.distributed carries the exchange (NCCL on GPUs, gloo in the CPU tests);
every kernel is a C-ABI call of libknj_device.so. With world == 1 the same
kernels run with the exchange elided.

The arithmetic is delegated to a `LocalCompute` object so the host logic
(counts, splits, plans, inverse permutation, partial sums) can be exercised on
CPU ranks with a stand-in compute in the tests.
"""
from __future__ import annotations

import ctypes as C
import os

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

    def __init__(self, router: torch.Tensor, top_k: int, router_bias: torch.Tensor | None = None,
                 tc_rows_per_expert: int = 16):
        from . import ops  # deferred: needs the CUDA library
        self.ops, self.router, self.top_k, self.bias = ops, router, top_k, router_bias
        # received rows per local expert from which the tensor-core grouped GEMMs take over
        # (below it the f32-accurate GEMV-class kernels run)
        self.tc_rows_per_expert = tc_rows_per_expert

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
        if n_rows >= self.tc_rows_per_expert * pair_cnt.shape[0]:
            xh = ops.to_f16(rows)
            A, st = ops.q4k_gateup_tc(xh, bank.gate, bank.up, pair_idx, pair_cnt, n_rows, 1, poison=False)
            Y, st2 = ops.q4k_down_tc(A, bank.down, pair_idx, pair_cnt, n_rows, poison=False)
            self.last_status = (st, st2)  # device flags: non-zero if a bounded wait inside the kernels gave up
            return Y
        A = ops.q4k_gateup(rows, bank.gate, bank.up, pair_idx, pair_cnt, exp_list, n_active, n_rows, 1,
                           want=("A",))["A"]
        return ops.q4k_proj(A, bank.down, pair_idx, pair_cnt, exp_list, n_active, n_rows)

    def combine(self, Yback, pair_row, pair_exp, pair_w, T, out_dtype):
        return self.ops.moe_combine(Yback, pair_exp, pair_w, T, self.top_k, out_dtype=out_dtype, pair_row=pair_row)

    # ---- gather exchange
    def plan_for_experts(self, pair_exp_all, exp_lo, e_loc, stride):
        """Plan over the global pair list restricted to experts [exp_lo, exp_lo + e_loc): pair ids stay global."""
        local_ids = pair_exp_all - exp_lo  # ids outside [0, e_loc) match no expert of the plan
        return self.ops.moe_permute(local_ids, e_loc, stride)

    def rows_for_gather(self, x, n_local_pairs_hint, e_loc):
        if x.dtype == torch.bfloat16 and n_local_pairs_hint >= self.tc_rows_per_expert * e_loc:
            return self.ops.to_f16(x)
        return x

    def expert_ffn_tokens(self, x_all, bank, plan, P, n_local_pairs_hint):
        """x_all [T][H] -> Y f32 [P][H], rows = global pair ids (rows of other ranks' pairs stay unwritten)."""
        pair_idx, pair_cnt, exp_list, n_active = plan
        ops, k = self.ops, self.top_k
        if n_local_pairs_hint >= self.tc_rows_per_expert * pair_cnt.shape[0]:
            xh = x_all if x_all.dtype == torch.float16 else ops.to_f16(x_all)
            A, st = ops.q4k_gateup_tc(xh, bank.gate, bank.up, pair_idx, pair_cnt, P, k, poison=False)
            Y, st2 = ops.q4k_down_tc(A, bank.down, pair_idx, pair_cnt, P, poison=False)
            self.last_status = (st, st2)
            return Y
        A = ops.q4k_gateup(x_all, bank.gate, bank.up, pair_idx, pair_cnt, exp_list, n_active, P, k, want=("A",))["A"]
        return ops.q4k_proj(A, bank.down, pair_idx, pair_cnt, exp_list, n_active, P)  # rows of foreign pairs stay unwritten

    def combine_partial(self, Y, pair_exp_all, pair_w_all, T, exp_lo, exp_hi):
        from ._lib import check, lib
        H = Y.shape[1]
        out = torch.empty((T, H), dtype=torch.float32, device=Y.device)
        check(lib().knj_ep_combine_partial_launch(C.c_void_p(Y.data_ptr()), C.c_void_p(pair_exp_all.data_ptr()),
                                                  C.c_void_p(pair_w_all.data_ptr()), T, H, self.top_k, exp_lo, exp_hi,
                                                  C.c_void_p(out.data_ptr()),
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def peer_gather(self, ptr_table, world, bytes_per_rank, dst):
        from ._lib import check, lib
        check(lib().knj_ep_peer_gather_launch(C.c_void_p(ptr_table.data_ptr()), world, bytes_per_rank,
                                              C.c_void_p(dst.data_ptr()),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def combine_partial_peer(self, Y, pair_exp_all, pair_w_all, T, exp_lo, exp_hi, parts_ptrs, rank, T_loc):
        from ._lib import check, lib
        check(lib().knj_ep_combine_partial_peer_launch(C.c_void_p(Y.data_ptr()), C.c_void_p(pair_exp_all.data_ptr()),
                                                       C.c_void_p(pair_w_all.data_ptr()), T, Y.shape[1], self.top_k,
                                                       exp_lo, exp_hi, C.c_void_p(parts_ptrs.data_ptr()), rank, T_loc,
                                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def reduce_sel(self, parts, pair_exp_local, k, e_loc, out_dtype):
        from ._lib import check, lib
        world, T_loc, H = parts.shape
        out = torch.empty((T_loc, H), dtype=out_dtype, device=parts.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}[out_dtype]
        check(lib().knj_ep_reduce_sel_launch(C.c_void_p(parts.data_ptr()), world, T_loc, H,
                                             C.c_void_p(pair_exp_local.data_ptr()), k, e_loc, None, 0,
                                             C.c_void_p(out.data_ptr()), dt,
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def reduce_parts(self, parts, out_dtype):
        """parts f32 [world][T_loc][H] -> [T_loc][H], ranks summed in ascending order."""
        from ._lib import check, lib
        world, T_loc, H = parts.shape
        out = torch.empty((T_loc, H), dtype=out_dtype, device=parts.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}[out_dtype]
        check(lib().knj_ep_reduce_launch(C.c_void_p(parts.data_ptr()), world, T_loc * H, T_loc, H, None, 0,
                                         C.c_void_p(out.data_ptr()), dt,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out


class PeerBuffers:
    """Exchange buffers of one rank that every rank of the group maps into its own address space
    (torch symmetric memory), plus device tables of the ranks' pointers for the peer kernels."""

    def __init__(self, group, world, rank, T_loc, H, k, row_dtype, device):
        import torch.distributed._symmetric_memory as symm
        g = group if group is not None else dist.group.WORLD
        self.group = group
        self.xpub = symm.empty((T_loc, H), dtype=row_dtype, device=device)
        self.pepub = symm.empty((T_loc * k,), dtype=torch.int32, device=device)
        self.pwpub = symm.empty((T_loc * k,), dtype=torch.float32, device=device)
        self.parts = symm.empty((world, T_loc, H), dtype=torch.float32, device=device)
        self._handles = [symm.rendezvous(t, g) for t in (self.xpub, self.pepub, self.pwpub, self.parts)]

        def table(h):
            return torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=device)
        self.x_ptrs, self.pe_ptrs, self.pw_ptrs, self.parts_ptrs = (table(h) for h in self._handles)
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def barrier(self):
        """Stream-ordered barrier over the group: everything the ranks enqueued before it (their stores into
        peers' buffers included) has completed when work enqueued after it starts."""
        dist.all_reduce(self._token, group=self.group)


class EpPeerContext:
    """The rank's expert-parallel layer object of the C-ABI (knj_ep_create): symmetric-memory exchange buffers
    whose per-rank addresses are handed to the library once; a step is one knj_ep_forward_launch, which
    allocates nothing and calls no collective."""

    def __init__(self, group, world, rank, T_loc, H, F, E, k, device, n_chunks=1):
        import torch.distributed._symmetric_memory as symm
        from ._lib import EP_FLAG_WORDS
        g = group if group is not None else dist.group.WORLD
        T = T_loc * world
        self.x_all = symm.empty((T, H), dtype=torch.float16, device=device)
        self.pe_all = symm.empty((T * k,), dtype=torch.int32, device=device)
        self.pw_all = symm.empty((T * k,), dtype=torch.float32, device=device)
        self.parts = symm.empty((world, T_loc, H), dtype=torch.float32, device=device)
        self.flags = symm.empty((EP_FLAG_WORDS,), dtype=torch.int32, device=device)
        self.flags.zero_()
        bufs = (self.x_all, self.pe_all, self.pw_all, self.parts, self.flags)
        self._handles = [symm.rendezvous(t, g) for t in bufs]
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every rank's flag words are zero before anyone's first step
        self._bind(world, rank, T_loc, H, F, E, k, [[int(p) for p in h.buffer_ptrs] for h in self._handles], n_chunks)

    def _bind(self, world, rank, T_loc, H, F, E, k, ptrs, n_chunks=1):
        """ptrs: five lists (rows, expert ids, weights, partial sums, flags) of `world` device addresses."""
        from ._lib import EpDescC, check, lib
        self._tables = [C.cast((C.c_void_p * world)(*p), C.POINTER(C.c_void_p)) for p in ptrs]
        d = EpDescC(world, rank, T_loc, H, F, E, k, n_chunks, *self._tables)
        self._ctx = C.c_void_p()
        check(lib().knj_ep_create(C.byref(d), C.byref(self._ctx)))
        self.shape = (T_loc, H)
        if os.environ.get("KNJ_EP_TRANSPORT"):  # measurement override: two letters, c(opy) or s(tores), rows then partials
            t = os.environ["KNJ_EP_TRANSPORT"]  # third letter h: partial rows as fp16
            self.set_transport(t[0] == "s", t[1] == "s", t[2:3] == "h")

    @classmethod
    def from_pointers(cls, world, rank, T_loc, H, F, E, k, ptrs, keep=None, n_chunks=1):
        """A layer object over exchange buffers the caller mapped itself (any peer mapping; the tests emulate two
        ranks inside one process this way). `keep` holds whatever owns the memory."""
        self = cls.__new__(cls)
        self._keep = keep
        self._bind(world, rank, T_loc, H, F, E, k, ptrs, n_chunks)
        return self

    def forward(self, x, router, bias, bank, residual, out_dtype):
        assert tuple(x.shape) == self.shape and x.stride(1) == 1
        out = torch.empty(self.shape, dtype=out_dtype, device=x.device)
        return self.forward_into(x, router, bias, bank, residual, out)

    def forward_into(self, x, router, bias, bank, residual, out):
        from ._lib import DT_BF16, DT_F16, DT_F32, check, lib
        dt = {torch.float32: DT_F32, torch.bfloat16: DT_BF16, torch.float16: DT_F16}
        check(lib().knj_ep_forward_launch(self._ctx, C.c_void_p(x.data_ptr()), dt[x.dtype], x.stride(0),
                                          C.c_void_p(router.data_ptr()),
                                          C.c_void_p(bias.data_ptr() if bias is not None else None),
                                          C.c_void_p(bank.gate.data_ptr()), C.c_void_p(bank.up.data_ptr()),
                                          C.c_void_p(bank.down.data_ptr()), int(bool(residual)),
                                          C.c_void_p(out.data_ptr()), dt[out.dtype],
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    def barrier(self):
        from ._lib import check, lib
        check(lib().knj_ep_barrier_launch(self._ctx, C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def set_wait(self, cycles: int):
        from ._lib import check, lib
        check(lib().knj_ep_set_wait(self._ctx, int(cycles)))

    def set_transport(self, sm_rows: bool, sm_partials: bool, f16_partials: bool = False):
        """How rows / partial sums reach the peers: stores of the library's kernels (True) or block copies by the
        copy engines (False); f16_partials: the stored partial rows travel as fp16 under a per-row scale."""
        from ._lib import check, lib
        check(lib().knj_ep_set_transport(self._ctx, (1 if sm_rows else 0) | (2 if sm_partials else 0) | (4 if f16_partials else 0)))

    def status(self):
        """Synchronises; raises KnjError (KNJ_E_TIMEOUT) if a bounded device-side wait gave up in the last step."""
        from ._lib import check, lib
        check(lib().knj_ep_status(self._ctx, C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def close(self):
        from ._lib import lib
        if self._ctx:
            lib().knj_ep_destroy(self._ctx)
            self._ctx = C.c_void_p()


_PEER_BUFFERS = {}


def peer_buffers(group, world, rank, T_loc, H, k, row_dtype, device) -> PeerBuffers:
    """One set per (group, shape): allocation is a collective, so every rank asks in the same order."""
    key = (id(group), world, T_loc, H, k, row_dtype, str(device))
    if key not in _PEER_BUFFERS:
        _PEER_BUFFERS[key] = PeerBuffers(group, world, rank, T_loc, H, k, row_dtype, device)
    return _PEER_BUFFERS[key]


_EP_CONTEXTS = {}


def ep_chunks(T_loc: int, k: int, world: int, e_loc: int) -> int:
    """Chunks of a step. One: on 2 and 4 B200s two chunks were slower than one at the benchmark's size (the two
    half-size GEMM launches lose more than the overlapped transfers save); more can be asked for explicitly."""
    return 1


def ep_context(group, world, rank, T_loc, H, F, E, k, device, n_chunks=None) -> EpPeerContext:
    """One layer object per (group, shape), shared by the layers of a stack (the weights are per-call arguments):
    creation is a collective, so every rank asks in the same order."""
    if n_chunks is None:
        n_chunks = int(os.environ.get("KNJ_EP_CHUNKS", "0")) or ep_chunks(T_loc, k, world, E // world)
    key = (id(group), world, T_loc, H, F, E, k, str(device), n_chunks)
    if key not in _EP_CONTEXTS:
        _EP_CONTEXTS[key] = EpPeerContext(group, world, rank, T_loc, H, F, E, k, device, n_chunks)
    return _EP_CONTEXTS[key]


class EpMoeLayer:
    """One expert-parallel MoE-FFN layer on this rank.

    bank: the LOCAL experts (E/world of them, ids rank*E/world ...); the router
    weight inside `compute` covers all E experts and is replicated.
    exchange: "gather" or "dispatch" (see the module text). "gather" needs the
    same token count on every rank.
    """

    def __init__(self, bank, n_experts: int, compute, group=None, top_k: int = synth.TOP_K, exchange: str = "gather"):
        assert exchange in ("gather", "dispatch", "peer")
        self.bank, self.E, self.compute, self.group, self.top_k = bank, n_experts, compute, group, top_k
        self.exchange = exchange
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert n_experts % self.world == 0
        self.e_loc = n_experts // self.world
        self.last_stats = {}

    def forward(self, x: torch.Tensor, out_dtype=torch.float32, out: torch.Tensor | None = None) -> torch.Tensor:
        """out: optional dense result rows [T_loc][H] to write into (its dtype then is the output's)."""
        if out is not None:
            out_dtype = out.dtype
        if self.exchange == "dispatch":
            res = self._forward_dispatch(x, out_dtype)
        elif (self.exchange == "peer" and self.world > 1 and x.is_cuda and (x.shape[0] * self.top_k) % 4 == 0
                and self._peer_ready(x)):
            if self._layer_object(x):
                return self._forward_layer_object(x, out_dtype, out)
            res = self._forward_peer(x, out_dtype)
        else:
            res = self._forward_gather(x, out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def _layer_object(self, x: torch.Tensor) -> bool:
        """Buckets large enough for the tensor-core GEMMs take the library's layer object (knj_ep_*): one call per
        step, no allocation, no collective. Smaller steps keep the f32-accurate kernels behind `_forward_peer`."""
        cp = self.compute
        return (hasattr(cp, "router") and x.shape[1] % 256 == 0 and
                x.shape[0] * self.top_k >= getattr(cp, "tc_rows_per_expert", 1 << 30) * self.e_loc)

    def _forward_layer_object(self, x, out_dtype, out):
        T_loc, H = x.shape
        cp = self.compute
        ctx = ep_context(self.group, self.world, self.rank, T_loc, H, self.bank.ffn, self.E, self.top_k, x.device)
        self.last_stats = {"tokens_gathered": int(T_loc * self.world), "layer_object": True}
        self.context = ctx
        if out is None:
            return ctx.forward(x, cp.router, cp.bias, self.bank, False, out_dtype)
        return ctx.forward_into(x, cp.router, cp.bias, self.bank, False, out)

    def _peer_ready(self, x: torch.Tensor) -> bool:
        """The peer mappings are set up once per shape, and the ranks agree on the outcome: if any rank cannot
        map its peers' buffers (no peer access, symmetric memory unavailable), all of them use the collectives."""
        T_loc, H = x.shape
        cp = self.compute
        tc = (x.dtype == torch.bfloat16 and
              T_loc * self.top_k >= getattr(cp, "tc_rows_per_expert", 1 << 30) * self.e_loc)
        keys = [(T_loc, H, self.top_k, torch.float16 if tc else x.dtype)]  # the dtype rows_for_gather will return
        verdict = self.__dict__.setdefault("_peer_verdict", {})
        if keys[0] in verdict:
            return verdict[keys[0]]
        ok = 1
        try:
            if self._layer_object(x):
                ep_context(self.group, self.world, self.rank, T_loc, H, self.bank.ffn, self.E, self.top_k, x.device)
            else:
                for (_, _, _, d) in keys:
                    peer_buffers(self.group, self.world, self.rank, T_loc, H, self.top_k, d, x.device)
        except Exception as ex:  # noqa: BLE001 - any failure means "use the collectives"
            self.last_stats["peer_setup_error"] = repr(ex)
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=x.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        verdict[keys[0]] = bool(int(flag.item()))
        return verdict[keys[0]]

    def _forward_peer(self, x: torch.Tensor, out_dtype) -> torch.Tensor:
        """The gather exchange with this library's own kernels moving the rows over NVLink peer mappings:
        publish (fp16 rows, routing tables) -> barrier -> pull every rank's rows into local memory -> expert
        GEMMs -> partial sums stored straight into the token owners' buffers -> barrier -> rank-ordered sum."""
        T_loc, H = x.shape
        world, k, cp = self.world, self.top_k, self.compute
        T = T_loc * world
        pair_exp, pair_w = cp.route(x)
        xg = cp.rows_for_gather(x, (T * k) // world, self.e_loc)
        pb = peer_buffers(self.group, world, self.rank, T_loc, H, k, xg.dtype, x.device)
        pb.xpub.copy_(xg)
        pb.pepub.copy_(pair_exp)
        pb.pwpub.copy_(pair_w)
        pb.barrier()
        x_all = torch.empty((T, H), dtype=xg.dtype, device=x.device)
        pe_all = torch.empty(T * k, dtype=torch.int32, device=x.device)
        pw_all = torch.empty(T * k, dtype=torch.float32, device=x.device)
        cp.peer_gather(pb.x_ptrs, world, T_loc * H * xg.element_size(), x_all)
        cp.peer_gather(pb.pe_ptrs, world, T_loc * k * 4, pe_all)
        cp.peer_gather(pb.pw_ptrs, world, T_loc * k * 4, pw_all)
        lo = self.rank * self.e_loc
        plan = cp.plan_for_experts(pe_all, lo, self.e_loc, max(T, 1))
        self.last_stats = {"tokens_gathered": int(T)}
        Y = cp.expert_ffn_tokens(x_all, self.bank, plan, T * k, (T * k) // world)
        cp.combine_partial_peer(Y, pe_all, pw_all, T, lo, lo + self.e_loc, pb.parts_ptrs, self.rank, T_loc)
        pb.barrier()
        return cp.reduce_sel(pb.parts, pair_exp, k, self.e_loc, out_dtype)

    def _forward_gather(self, x: torch.Tensor, out_dtype) -> torch.Tensor:
        T_loc, H = x.shape
        world, k, cp = self.world, self.top_k, self.compute
        T = T_loc * world
        pair_exp, pair_w = cp.route(x)
        # 16-bit rows that the tensor-core GEMMs would convert to fp16 anyway are converted before they travel:
        # every rank converts its own rows once instead of all rows of all ranks (bf16 -> fp16 is exact in range)
        if world > 1 and hasattr(cp, "rows_for_gather"):
            x = cp.rows_for_gather(x, (T * k) // world, self.e_loc)
        if world == 1:
            x_all, pe_all, pw_all = x, pair_exp, pair_w
        else:
            x_all = torch.empty((T, H), dtype=x.dtype, device=x.device)
            pe_all = torch.empty(T * k, dtype=pair_exp.dtype, device=x.device)
            pw_all = torch.empty(T * k, dtype=pair_w.dtype, device=x.device)
            dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
            dist.all_gather_into_tensor(pe_all, pair_exp, group=self.group)
            dist.all_gather_into_tensor(pw_all, pair_w, group=self.group)
        lo = self.rank * self.e_loc
        plan = cp.plan_for_experts(pe_all, lo, self.e_loc, max(T, 1))
        self.last_stats = {"tokens_gathered": int(T)}
        Y = cp.expert_ffn_tokens(x_all, self.bank, plan, T * k, (T * k) // world)
        part = cp.combine_partial(Y, pe_all, pw_all, T, lo, lo + self.e_loc)
        if world == 1:
            parts = part.view(1, T, H)
        else:
            parts = torch.empty((world, T_loc, H), dtype=torch.float32, device=x.device)
            dist.all_to_all_single(parts.view(T, H), part, group=self.group)  # block j of `part` -> rank j
        return cp.reduce_parts(parts, out_dtype)

    def _forward_dispatch(self, x: torch.Tensor, out_dtype) -> torch.Tensor:
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
