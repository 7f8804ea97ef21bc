"""CUDA back ends of the residency gates (slot pool, copy engine, pinned arena) and the streamed layer: with fewer
slots than experts, over several steps that force evictions and reloads, the streamed layer's output equals the
resident layer's bit for bit (the I1 check of records/2026-10-07_gfx1201_expert_streaming.txt:57-95)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu


def test_slot_pool_and_copy_engine(tmp_path):
    from kanjoos_b200._lib import lib
    L = lib()
    arena, eng = L.knj_res_arena_create(), L.knj_res_engine_create(None)
    slots = L.knj_res_slots_create(2, 4096)
    host = L.knj_res_arena_alloc(arena, 4096)
    back = L.knj_res_arena_alloc(arena, 4096)
    src = np.arange(4096, dtype=np.uint8)
    C.memmove(host, src.ctypes.data, 4096)
    a = L.knj_res_slot_acquire(slots, 0, 7, 4096)
    b = L.knj_res_slot_acquire(slots, 0, 8, 100)
    assert a >= 0 and b >= 0 and a != b
    assert L.knj_res_slot_acquire(slots, 0, 9, 4096) == -1          # no room: the caller must not block
    assert L.knj_res_slot_acquire(slots, 0, 9, 8192) == -1          # larger than a slot
    assert L.knj_res_slot_bytes(slots, b) == 100
    t1 = L.knj_res_submit_h2d(eng, L.knj_res_slot_ptr(slots, a), host, 4096, 0)
    L.knj_res_slot_watch(slots, a, eng, t1)
    t2 = L.knj_res_submit_d2h(eng, back, L.knj_res_slot_ptr(slots, a), 4096, 0)   # same stream: ordered after t1
    while L.knj_res_poll(eng, t2) == 0:
        pass
    assert L.knj_res_poll(eng, t1) == 1 and L.knj_res_poll(eng, t2) == 1 and L.knj_res_slot_load_fired(slots, a) == 1
    got = np.frombuffer((C.c_uint8 * 4096).from_address(back), dtype=np.uint8)
    assert np.array_equal(got, src)                                  # a reload reproduces the same bytes
    L.knj_res_slot_pin(slots, a)
    L.knj_res_slot_release(slots, a)                                 # pinned: stays
    assert L.knj_res_slot_released(slots, a) == 0
    L.knj_res_slot_unpin(slots, a)
    L.knj_res_slot_release(slots, a)
    assert L.knj_res_slot_released(slots, a) == 1 and L.knj_res_slot_acquire(slots, 1, 1, 64) == a
    assert L.knj_res_cancel(eng, t1) == 0 and L.knj_res_poll(eng, 12345) == 2
    # file tier: write a block, read it back through the worker thread
    path = tmp_path / "backing.bin"
    path.write_bytes(bytes(8192))
    feng = L.knj_res_engine_create(str(path).encode())
    w = L.knj_res_submit_nvme_write(feng, host, 4096, 4096, 1)
    while L.knj_res_poll(feng, w) == 0:
        pass
    C.memset(back, 0, 4096)
    r = L.knj_res_submit_nvme_read(feng, back, 4096, 4096, 0)
    while L.knj_res_poll(feng, r) == 0:
        pass
    assert L.knj_res_poll(feng, w) == 1 and L.knj_res_poll(feng, r) == 1
    assert np.array_equal(np.frombuffer((C.c_uint8 * 4096).from_address(back), dtype=np.uint8), src)
    assert L.knj_res_submit_nvme_read(eng, back, 0, 16, 0) == 0      # no backing file: refused
    L.knj_res_engine_destroy(feng)
    L.knj_res_slots_destroy(slots)
    L.knj_res_engine_destroy(eng)
    L.knj_res_arena_free(arena, host)
    L.knj_res_arena_free(arena, back)
    L.knj_res_arena_destroy(arena)
    assert os.path.getsize(path) == 8192


def test_streamed_equals_resident_bit_for_bit():
    from kanjoos_b200.residency import StreamedMoeLayer
    E, H, F, k = 16, 512, 256, 2
    bank = synth.expert_bank(701, n_experts=E, hidden=H, ffn=F)
    wr, _ = synth.router_weight(701, n_experts=E, hidden=H)
    layer = StreamedMoeLayer(bank, wr, top_k=k, n_slots=6)
    resident = tuple(torch.from_numpy(bank[kd]).cuda() for kd in ("gate", "up", "down"))
    try:
        for step in range(6):
            x = torch.from_numpy(synth.hidden_rows(701 + step, 3, H)).cuda()   # 3 tokens x top-2 <= 6 slots
            want = layer.forward(x, resident_bank=resident)
            got = layer.forward(x)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int32), want.view(torch.int32)), f"step {step}: streamed != resident"
        assert layer.loads > 6 and layer.evictions > 0      # the slots were recycled along the way
        # a step that routes to more distinct experts than there are slots is refused up front, and the pools stay
        # usable afterwards
        many = torch.from_numpy(synth.hidden_rows(799, 12, H)).cuda()
        with pytest.raises(ValueError):
            layer.forward(many)
        x = torch.from_numpy(synth.hidden_rows(701, 3, H)).cuda()
        assert torch.equal(layer.forward(x).view(torch.int32), layer.forward(x, resident_bank=resident).view(torch.int32))
    finally:
        layer.close()


def test_reference_residency_manager_over_the_cuda_gates():
    """The reference's own ResidencyManager (its residency.cpp, compiled where it lies into
    oracle/_ref/knj_ref_residency_check together with oracle/ref_residency_check.cpp) constructed over this
    library's slot pool, copy engine and pinned arena, driven through demand, pool-full fallback, eviction,
    pinning, reload and prefetch with real asynchronous copies. The binary is built where the reference tree
    exists (make -C oracle ref); it is test infrastructure and travels prebuilt."""
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "knj_ref_residency_check")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/knj_ref_residency_check was not built (no reference tree on the build machine)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout
