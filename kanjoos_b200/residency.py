"""The layer with its experts streamed through a few device slots instead of
held resident: the mode the reference's residency tiers exist for
(src/residency/residency.h; device models tools/bench/q4k_stream_ffn.hip:219-674,
bit-for-bit check records/2026-10-07_gfx1201_expert_streaming.txt:57-95).

On a B200 every expert fits in HBM, so this is off the timed path; it shows that
the CUDA slot pool, copy engine and pinned arena (include/knj_residency.h) carry
the same kernels to the same bits. Per step: route on the device, read the routed
expert ids, bring the missing experts' matrices from pinned host memory into
slots (demand class), make the compute stream wait for those copies, run the
decode-class kernels over SLOT ids, combine in EXPERT-id order.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import ops
from ._lib import lib


class SlotPool:
    """n_slots device slots of slot_bytes each plus the copy engine that fills them (one matrix per slot)."""

    def __init__(self, n_slots: int, slot_bytes: int, engine):
        self.L, self.engine, self.n_slots, self.slot_bytes = lib(), engine, n_slots, slot_bytes
        self.h = self.L.knj_res_slots_create(n_slots, slot_bytes)
        first = self.L.knj_res_slot_acquire(self.h, 0, 0, slot_bytes)
        self.base = self.L.knj_res_slot_ptr(self.h, first)  # slot 0: the pool is one allocation
        assert first == 0 and self.base
        self.L.knj_res_slot_release(self.h, first)

    def close(self):
        if self.h:
            self.L.knj_res_slots_destroy(self.h)
            self.h = None


class StreamedMoeLayer:
    """Decode-class MoE-FFN layer over host-resident experts and `n_slots` device slots per matrix kind."""

    def __init__(self, bank_np: dict, router_bits: np.ndarray, top_k: int, n_slots: int, layer_id: int = 0):
        self.L = lib()
        self.k, self.layer_id, self.n_slots = top_k, layer_id, n_slots
        self.E = bank_np["gate"].shape[0]
        assert n_slots >= top_k, "a token's experts must fit the slots together"
        self.arena = self.L.knj_res_arena_create()
        self.engine = self.L.knj_res_engine_create(None)
        self.router = torch.from_numpy(router_bits.view(np.int16).copy()).view(torch.bfloat16).cuda()
        self.host, self.pools, self.shape = {}, {}, {}
        for kind in ("gate", "up", "down"):
            w = np.ascontiguousarray(bank_np[kind])
            per = w[0].nbytes
            buf = self.L.knj_res_arena_alloc(self.arena, w.nbytes)
            assert buf, "pinned staging allocation failed"
            C.memmove(buf, w.ctypes.data, w.nbytes)
            self.host[kind] = (buf, per)
            self.pools[kind] = SlotPool(n_slots, per, self.engine)
            self.shape[kind] = w.shape[1:]
        self.slot_of = {}          # expert id -> slot index (the same in the three pools)
        self.last_use = {}
        self.clock = 0
        self.loads = self.evictions = 0

    def close(self):
        torch.cuda.synchronize()
        for p in self.pools.values():
            p.close()
        self.L.knj_res_engine_destroy(self.engine)
        for buf, _ in self.host.values():
            self.L.knj_res_arena_free(self.arena, buf)
        self.L.knj_res_arena_destroy(self.arena)

    def _slot_tensor(self, kind):
        p = self.pools[kind]
        n = p.n_slots * p.slot_bytes

        class _Holder:  # a CUDA tensor view over the pool, no copy
            __cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (p.base, False), "version": 2}
        return torch.as_tensor(_Holder(), device="cuda").view((p.n_slots,) + tuple(self.shape[kind]))

    def _ensure(self, experts, stream):
        """Make every expert in `experts` slot-resident; evict least-recently-used experts that are not needed."""
        n_slots = self.pools["gate"].n_slots
        if len(experts) > n_slots:
            raise ValueError(f"a step routes to {len(experts)} distinct experts but the pools hold {n_slots} slots: "
                             "split the step or give the layer more slots")
        need = [e for e in experts if e not in self.slot_of]
        # victims for ALL three pools leave before any slot is acquired, so the pools stay in lockstep
        n_evict = max(0, len(self.slot_of) + len(need) - n_slots)
        victims = sorted((x for x in self.slot_of if x not in experts), key=lambda x: self.last_use[x])[:n_evict]
        for victim in victims:
            for kd in ("gate", "up", "down"):
                pv = self.pools[kd]
                self.L.knj_res_slot_release(pv.h, self.slot_of[victim])
                while not self.L.knj_res_slot_released(pv.h, self.slot_of[victim]):
                    pass  # its loads finished long ago; release completes at once
            del self.slot_of[victim]
            self.evictions += 1
        waits = []
        for e in need:
            slots = {}
            for kind in ("gate", "up", "down"):
                p = self.pools[kind]
                h = self.L.knj_res_slot_acquire(p.h, self.layer_id, e, p.slot_bytes)
                assert h >= 0, "a slot was freed for every expert that has to come in"
                slots[kind] = h
            assert len(set(slots.values())) == 1, "the three pools evolve in lockstep"
            for kind, h in slots.items():
                p = self.pools[kind]
                buf, per = self.host[kind]
                tid = self.L.knj_res_submit_h2d(self.engine, self.L.knj_res_slot_ptr(p.h, h), buf + e * per, per, 0)
                assert tid
                self.L.knj_res_slot_watch(p.h, h, self.engine, tid)
                waits.append(tid)
            self.slot_of[e] = slots["gate"]
            self.loads += 1
        for tid in waits:  # the kernels that follow on `stream` see complete copies
            assert self.L.knj_res_wait_on_stream(self.engine, tid, C.c_void_p(stream.cuda_stream)) == 0
        self.clock += 1
        for e in experts:
            self.last_use[e] = self.clock

    def forward(self, x: torch.Tensor, resident_bank=None) -> torch.Tensor:
        """x [T][H] -> f32 [T][H]. With `resident_bank` (gate, up, down CUDA tensors over all experts) the same
        kernels run without streaming: the comparison arm of the bit-identity test."""
        T = x.shape[0]
        P, k = T * self.k, self.k
        _, pe, pw = ops.router_topk(x, self.router, k)
        st = torch.cuda.current_stream()
        if resident_bank is None:
            experts = sorted(set(pe.cpu().tolist()))
            # the previous step's kernels may still read slots that are about to be evicted
            st.synchronize()
            self._ensure(experts, st)
            table = torch.full((self.E,), -1, dtype=torch.int32)
            for e, s in self.slot_of.items():
                table[e] = s
            ids = table.cuda()[pe.long()].contiguous()
            n_units = self.n_slots
            gate, up, down = (self._slot_tensor(kd) for kd in ("gate", "up", "down"))
        else:
            ids, n_units = pe, self.E
            gate, up, down = resident_bank
        pair_idx, pair_cnt, exp_list, n_active = ops.moe_permute(ids, n_units, T)
        A = ops.q4k_gateup(x, gate, up, pair_idx, pair_cnt, exp_list, n_active, P, k, want=("A",))["A"]
        Y = ops.q4k_proj(A, down, pair_idx, pair_cnt, exp_list, n_active, P)
        return ops.moe_combine(Y, pe, pw, T, k)
