"""Device layer + the control / capability kernels, through the C-ABI, in the
order the reference's device driver runs them (tests/test_gemm_w4.hip:122-183:
arch guard -> control kernel -> capability probe)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from kanjoos_b200 import _lib
    lib = _lib.lib()
    _lib.check(lib.knj_dev_open(0))
    return lib


def test_arch_guard_exit_codes(L, monkeypatch):
    monkeypatch.delenv("KNJ_BUILD_ARCH", raising=False)
    assert L.knj_arch_check() == 7
    monkeypatch.setenv("KNJ_BUILD_ARCH", "gfx1201")
    assert L.knj_arch_check() == 6
    monkeypatch.setenv("KNJ_BUILD_ARCH", "sm_100")
    assert L.knj_arch_check() == 0


def test_device_caps(L):
    from kanjoos_b200 import ops
    caps = ops.device_caps(0)
    assert caps.arch == b"sm_100" and caps.cc_major == 10
    assert caps.sms >= 100 and caps.wave_size == 32 and caps.has_mma == 1
    assert caps.vram_total > 100 * 2**30 and caps.smem_per_block_optin >= 200 * 1024


def test_control_kernel(L):
    from kanjoos_b200 import ops
    out = ops.control(0x1234, 64, 1).cpu().numpy().view(np.uint32)
    assert out[0] == 0x1235 and out[1] == 1
    out = ops.control(0xFFFFFFFF, 128, 7).cpu().numpy().view(np.uint32)
    assert out[0] == 0 and out[1] == 7


def test_probe_caps(L):
    from kanjoos_b200 import ops
    inp = torch.tensor([424242], dtype=torch.int32, device="cuda")
    cap = ops.probe_caps(inp).cpu().numpy().view(np.uint32)
    assert cap[2] == 1, "probe kernel never dispatched"
    assert cap[0] == 1, "dp4a identity failed"
    assert cap[1] == 1 and cap[4] == 0x4000, f"packed fp16 fma gave 0x{cap[4]:04x}, want 0x4000"
    assert cap[3] == 424242
    assert cap[5] == 1, "fp16 tensor-core MMA over subnormal-encoded 4-bit integers is not exact"
    assert cap[6] == 1, "bulk async copy + mbarrier did not complete"
    cap0 = ops.probe_caps(None).cpu().numpy().view(np.uint32)
    assert cap0[3] == 0 and cap0[2] == 1


def test_runtime_layer_roundtrip(L):
    from kanjoos_b200._lib import check
    p = C.c_void_p()
    h = C.c_void_p()
    n = 1 << 20
    check(L.knj_malloc(C.byref(p), n))
    check(L.knj_host_malloc(C.byref(h), n))
    src = (np.arange(n) % 251).astype(np.uint8)
    C.memmove(h, src.ctypes.data, n)
    s = C.c_void_p()
    e0, e1 = C.c_void_p(), C.c_void_p()
    check(L.knj_stream_create(C.byref(s)))
    check(L.knj_event_create(C.byref(e0), 1))
    check(L.knj_event_create(C.byref(e1), 1))
    check(L.knj_event_record(e0, s))
    check(L.knj_memcpy_h2d_async(p, h, n, s))
    back = np.zeros(n, np.uint8)
    check(L.knj_event_record(e1, s))
    check(L.knj_stream_sync(s))
    check(L.knj_memcpy_d2h(back.ctypes.data, p, n))
    assert np.array_equal(back, src)
    ms = C.c_float(-1)
    check(L.knj_event_elapsed_ms(C.byref(ms), e0, e1))
    assert ms.value >= 0
    assert L.knj_event_query(e1) == 0 and L.knj_stream_query(s) == 0
    fr, tot = C.c_size_t(), C.c_size_t()
    check(L.knj_mem_info(C.byref(fr), C.byref(tot)))
    assert 0 < fr.value <= tot.value
    for ev in (e0, e1):
        check(L.knj_event_destroy(ev))
    check(L.knj_stream_destroy(s))
    check(L.knj_host_free(h))
    check(L.knj_free(p))


def test_graph_capture_replays_control(L):
    from kanjoos_b200._lib import check
    s = C.c_void_p()
    check(L.knj_stream_create(C.byref(s)))
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    check(L.knj_graph_begin(s))
    check(L.knj_control_launch(C.c_void_p(out.data_ptr()), 41, 64, 3, s))
    g = C.c_void_p()
    check(L.knj_graph_end(s, C.byref(g)))
    assert out.cpu().tolist() == [0, 0]  # capture did not run it
    check(L.knj_graph_launch(g, s))
    check(L.knj_stream_sync(s))
    assert out.cpu().tolist() == [42, 3]
    check(L.knj_graph_destroy(g))
    check(L.knj_stream_destroy(s))


def test_backend_create_is_arch_guarded(L, monkeypatch):
    monkeypatch.delenv("KNJ_BUILD_ARCH", raising=False)
    assert not L.knj_backend_create()
    assert b"KNJ_BUILD_ARCH is not set" in L.knj_backend_last_refusal()
    monkeypatch.setenv("KNJ_BUILD_ARCH", "sm_100")
    b = L.knj_backend_create()
    assert b and L.knj_backend_last_refusal() == b""
    assert L.knj_backend_arch(b) == b"sm_100"
    assert L.knj_backend_launch(b, 0, None, None) == 1 and L.knj_backend_launch(b, 1, None, None) == 1
    L.knj_backend_destroy(b)


def test_dot_helpers_on_the_device_match_their_definition():
    """knj_dot4_i32_i8 / knj_dot8_i32_i4 / knj_dot2_i32_i16 executed in a kernel against the plain-integer
    definition (kernels/knj_dot.h:117-174), incl. the sign corners of every field width."""
    from kanjoos_b200 import ops
    rng = np.random.Generator(np.random.Philox(77))
    n = 4096
    a = rng.integers(-2**31, 2**31, size=n, dtype=np.int64).astype(np.int32)
    b = rng.integers(-2**31, 2**31, size=n, dtype=np.int64).astype(np.int32)
    acc = rng.integers(-2**20, 2**20, size=n, dtype=np.int64).astype(np.int32)
    corners = np.array([0, -1, 0x7fffffff, -2**31, 0x88888888 - 2**32, 0x77777777, 0x80808080 - 2**32, 0x7f7f7f7f,
                        0x80008000 - 2**32, 0x7fff7fff], dtype=np.int64).astype(np.int32)
    a[:corners.size] = corners
    b[:corners.size] = corners[::-1]

    def fields(x, bits):
        u = x.astype(np.int64) & 0xffffffff
        out = []
        for i in range(32 // bits):
            f = (u >> (bits * i)) & ((1 << bits) - 1)
            out.append(np.where(f >= (1 << (bits - 1)), f - (1 << bits), f))
        return out
    want = {}
    for bits in (8, 4, 16):
        s = acc.astype(np.int64)
        for fa, fb in zip(fields(a, bits), fields(b, bits)):
            s = s + fa * fb
        want[bits] = ((s + 2**31) % 2**32 - 2**31).astype(np.int32)
    d4, d8, d2 = (t.cpu().numpy() for t in ops.dot_helpers(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(),
                                                          torch.from_numpy(acc).cuda()))
    assert np.array_equal(d4, want[8]) and np.array_equal(d8, want[4]) and np.array_equal(d2, want[16])


def test_fuse_gateup_silu_kernel():
    """knj_fuse_gateup_silu_launch (tools/bench/q4k_stream_ffn.hip:1021-1031) against the CPU path's silu * up."""
    import oracle_lib as ol
    from kanjoos_b200 import ops
    rng = np.random.Generator(np.random.Philox(78))
    g = (rng.standard_normal((37, 768)) * 4).astype(np.float32)
    u = rng.standard_normal((37, 768)).astype(np.float32)
    g[0, :4] = [0.0, -100.0, 100.0, -1e-8]
    want = ol.silu_mul(g, u)
    got = ops.fuse_gateup_silu(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda()).cpu().numpy()
    assert ol.compare(got, want)["rel_rmse"] <= 1e-6
    got16 = ops.fuse_gateup_silu(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda(), dtype=torch.bfloat16).float().cpu().numpy()
    assert ol.compare(got16, want)["rel_rmse"] <= 5e-3
