"""CPU-only checks of the boundary: the shared library loads and exports every
symbol include/knj_device.h and include/knj_residency.h declare, argument validation refuses bad calls
before any device work, and the host-side device layer (arch guard, capability
table, cap line, Backend gating) behaves like the reference's
tests/unit/test_c2_device.cpp expects of its own."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from kanjoos_b200 import _lib, build
    build.build()
    return _lib.lib()


def declared_symbols():
    text = "".join(open(os.path.join(ROOT, "include", h)).read() for h in ("knj_device.h", "knj_residency.h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(knj_[a-z0-9_]+)\s*\(", text))
    names -= {"knj_q4k_down_launch"}  # a #define alias of knj_q4k_proj_launch
    return sorted(names)


def test_every_declared_symbol_is_exported_and_bound(L):
    from kanjoos_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 50
    handle = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/ but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"


def test_status_codes_without_a_device(L):
    n = C.c_int(-1)
    rc = L.knj_dev_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a GPU is present; the no-device path is not reachable")
    assert rc == -2 and n.value == 0 and b"CUDA error" in L.knj_last_error_string()


def test_arch_guard_unset_refuses_before_touching_a_device(L, monkeypatch):
    monkeypatch.delenv("KNJ_BUILD_ARCH", raising=False)
    assert L.knj_arch_check() == 7
    monkeypatch.setenv("KNJ_BUILD_ARCH", "gfx1031")
    assert L.knj_arch_check() == 6


def test_null_and_geometry_refusals(L):
    assert L.knj_control_launch(None, 1, 64, 1, None) == -1
    assert L.knj_gemm_w4_i8_launch(None, None, None, None, 1, 1, 128, 64, 1, None) == -1
    assert L.knj_q4k_dequant_launch(None, None, 1, None) == -1
    assert L.knj_q4k_dequant_launch(None, None, 0, None) == 0
    assert L.knj_router_topk_launch(None, 0, 0, None, None, 1, 256, 8, 2, None, None, None, None) == -1
    assert L.knj_moe_ffn_decode_launch(None, None) == -1
    from kanjoos_b200._lib import MoeFfnArgs
    a = MoeFfnArgs()
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == 0  # zero tokens: nothing to do, nothing to validate
    a.n_tokens = 1
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == -1
    assert b"null tensor pointer" in L.knj_last_error_string()
    one = C.c_void_p(4096)  # never dereferenced: validation fails first
    a.x = a.w_router = a.w_gate = a.w_up = a.w_down = a.out = 4096
    a.n_tokens, a.hidden, a.ffn, a.n_experts, a.top_k = 1, 2000, 768, 128, 8
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == -1 and b"multiples of 256" in L.knj_last_error_string()
    a.hidden = 2048
    a.top_k = 9
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == -1 and b"top_k" in L.knj_last_error_string()
    a.top_k = 8
    a.ldx = a.ldo = 2048
    a.w_gate = 4100  # misaligned base
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == -1 and b"16-byte aligned" in L.knj_last_error_string()
    a.w_gate = 4096
    assert L.knj_moe_ffn_decode_launch(C.byref(a), None) == -4 and b"workspace" in L.knj_last_error_string()
    del one


def test_workspace_sizes(L):
    assert L.knj_q4k_matmul_workspace_bytes(1, 2048) == 512   # identity pair list + the one-expert plan
    assert L.knj_q4k_matmul_workspace_bytes(0, 2048) == 0
    small = L.knj_moe_ffn_workspace_bytes(1, 2048, 768, 128, 8, 0)
    big = L.knj_moe_ffn_workspace_bytes(64, 2048, 768, 128, 8, 0)
    assert 0 < small < big and big % 256 == 0
    assert L.knj_moe_ffn_workspace_bytes(0, 2048, 768, 128, 8, 0) == 256


# ---- the device layer's host logic (mirrors tests/unit/test_c2_device.cpp) ----

CAPS = dict(Dot4I32I8=0, Dot8I32I4=1, PkFmaF16=2, WmmaF16=3, Fp8=4, Sdot4Builtin=5, Dp4a=6, TcGen05=7, Tmem=8,
            TmaBulk=9)


def test_check_arch_verdicts(L):
    reason = C.c_char_p()
    assert L.knj_check_arch_c(None, b"sm_100", C.byref(reason)) == 1 and b"KNJ_BUILD_ARCH is not set" in reason.value
    assert L.knj_check_arch_c(b"", b"sm_100", C.byref(reason)) == 1 and b"not set" in reason.value
    assert L.knj_check_arch_c(b"gfx1201", b"sm_100", C.byref(reason)) == 1 and b"arch mismatch" in reason.value
    assert L.knj_check_arch_c(b"sm_100", b"", C.byref(reason)) == 1
    assert L.knj_check_arch_c(b"sm_100", b"sm_100", C.byref(reason)) == 0 and reason.value == b""


def test_capability_table(L):
    av = lambda arch, cap: L.knj_cap_available_c(arch, CAPS[cap])
    for cap in ("Dot4I32I8", "Dot8I32I4", "PkFmaF16"):
        assert av(b"sm_100", cap) and av(b"gfx1201", cap) and av(b"gfx1031", cap)
    assert av(b"sm_100", "WmmaF16") and av(b"gfx1201", "WmmaF16") and not av(b"gfx1031", "WmmaF16")
    assert av(b"sm_100", "Fp8") and not av(b"gfx1031", "Fp8")
    assert not av(b"sm_100", "Sdot4Builtin") and av(b"gfx1031", "Sdot4Builtin") and not av(b"gfx1201", "Sdot4Builtin")
    for cap in ("Dp4a", "TcGen05", "Tmem", "TmaBulk"):
        assert av(b"sm_100", cap) and not av(b"gfx1201", cap)
    for cap in CAPS:
        assert not av(b"", cap) and not av(None, cap) and not av(b"sm_90", cap)
    labels = [L.knj_cap_label_c(i) for i in range(10)]
    assert labels[:6] == [b"dot4_i32_i8", b"dot8_i32_i4", b"pk_fma_f16", b"wmma_f16", b"fp8", b"sdot4"]
    assert L.knj_cap_label_c(99) == b"unknown"


def test_cap_line_fields_and_order(L):
    buf = C.create_string_buffer(256)
    L.knj_cap_line(b"sm_100", 1, 1, 0, 1, buf, 256)
    line = buf.value.decode()
    assert line == "capabilities  wmma=on  fp8=on  dot=intrinsic(dp4a)  smi=lane-split  v_pk_fma_f16=yes"
    L.knj_cap_line(b"sm_100", 0, 0, 0, 0, buf, 256)
    assert buf.value.decode() == "capabilities  wmma=off  fp8=off  dot=intrinsic(dp4a)  smi=lane-split  v_pk_fma_f16=no"
    # a record carrying the reference's arch strings prints the reference's spellings
    L.knj_cap_line(b"gfx1031", 0, 0, 1, 1, buf, 256)
    assert "dot=builtin(sdot4)" in buf.value.decode()
    L.knj_cap_line(b"gfx1201", 1, 1, 0, 1, buf, 256)
    assert "dot=asm(v_dot4_i32_i8)" in buf.value.decode()
    pos = [buf.value.decode().index(k) for k in ("wmma=", "fp8=", "dot=", "smi=", "v_pk_fma_f16=")]
    assert pos == sorted(pos)


def test_backend_gating_with_injected_caps(L, monkeypatch):
    monkeypatch.delenv("KNJ_BUILD_ARCH", raising=False)
    assert not L.knj_backend_create()
    assert b"KNJ_BUILD_ARCH is not set" in L.knj_backend_last_refusal()
    monkeypatch.setenv("KNJ_BUILD_ARCH", "gfx1201")
    assert not L.knj_backend_create() and b"arch mismatch" in L.knj_backend_last_refusal()

    full = L.knj_backend_from_caps(b"sm_100", 1, 1, 0, 1)
    assert L.knj_backend_last_refusal() == b""
    for cap in ("Dot4I32I8", "PkFmaF16", "WmmaF16", "Fp8", "Dp4a", "TcGen05", "Tmem", "TmaBulk"):
        assert L.knj_backend_would_instantiate(full, CAPS[cap])
    assert not L.knj_backend_would_instantiate(full, CAPS["Sdot4Builtin"])
    # empty plan: the launches answer the gate and run nothing
    assert L.knj_backend_launch(full, 0, None, None) == 1
    assert L.knj_backend_launch(full, 1, None, None) == 1
    assert L.knj_backend_launch(full, 2, None, None) == 1
    L.knj_backend_destroy(full)

    # a device that nominally is sm_100 but whose probe found no matrix unit / fp8
    stripped = L.knj_backend_from_caps(b"sm_100", 0, 0, 0, 1)
    assert not L.knj_backend_would_instantiate(stripped, CAPS["WmmaF16"])
    assert not L.knj_backend_would_instantiate(stripped, CAPS["TcGen05"])
    assert not L.knj_backend_would_instantiate(stripped, CAPS["Fp8"])
    assert L.knj_backend_would_instantiate(stripped, CAPS["Dot4I32I8"])
    assert L.knj_backend_launch(stripped, 0, None, None) == 0  # tensor-core path refused
    assert L.knj_backend_launch(stripped, 1, None, None) == 1  # warp-level path allowed
    L.knj_backend_destroy(stripped)

    refused = L.knj_backend_from_caps(b"", 1, 1, 0, 0)
    assert not L.knj_backend_would_instantiate(refused, CAPS["Dot4I32I8"])
    assert L.knj_backend_launch(refused, 1, None, None) == 0 and L.knj_backend_launch(refused, 2, None, None) == 0
    L.knj_backend_destroy(refused)

    ref_arch = L.knj_backend_from_caps(b"gfx1031", 0, 0, 1, 1)
    assert L.knj_backend_would_instantiate(ref_arch, CAPS["Sdot4Builtin"])
    assert not L.knj_backend_would_instantiate(ref_arch, CAPS["WmmaF16"])
    L.knj_backend_destroy(ref_arch)


def test_helper_headers_compile_as_c_and_agree_with_the_oracle(tmp_path):
    """include/knj_q4k.h, knj_pack.h, knj_dot.h are usable from plain C on the host."""
    import subprocess
    import numpy as np
    import oracle_lib as ol
    src = tmp_path / "t.c"
    src.write_text(r'''
#include "knj_q4k.h"
#include "knj_pack.h"
#include "knj_dot.h"
float t_weight(const uint8_t* b, int r) { return knj_q4k_weight(b, r); }
float t_weight6(const uint8_t* b, int r) { return knj_q6k_weight(b, r); }
void t_span(const uint8_t* b, int r0, float* o) { knj_q4k_span16(b, r0, o); }
void t_span6(const uint8_t* b, int r0, float* o) { knj_q6k_span16(b, r0, o); }
float t_h2f(uint16_t h) { return knj_half_bits_to_float(h); }
int t_dot4(int a, int b, int c) { return knj_dot4_i32_i8(a, b, c); }
int t_dot8(int a, int b, int c) { return knj_dot8_i32_i4(a, b, c); }
int t_dot2(int a, int b, int c) { return knj_dot2_i32_i16(a, b, c); }
void t_unpack(uint32_t p, int* lo, int* hi) { knj_unpack8_u4(p, lo, hi); }
int t_stride(void) { return KNJ_GROUP_STRIDE_BYTES(4, KNJ_GROUP_EXPERT); }
''')
    so = tmp_path / "t.so"
    subprocess.check_call(["gcc", "-std=gnu11", "-O1", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"),
                           str(src), "-o", str(so)])
    t = C.CDLL(str(so))
    t.t_weight.restype = t.t_weight6.restype = t.t_h2f.restype = C.c_float
    t.t_h2f.argtypes = [C.c_uint16]
    o = ol.oracle()
    rng = np.random.default_rng(1)
    blk = rng.integers(0, 256, 144, dtype=np.uint8)
    blk[0:4] = np.array([0.0123, 0.0045], np.float16).view(np.uint8)
    bp = blk.ctypes.data_as(ol.u8p)
    span = np.empty(16, np.float32)
    for r in range(256):
        assert t.t_weight(bp, r) == o.knj_or_q4k_weight(bp, r)
    for r0 in range(0, 256, 16):
        t.t_span(bp, r0, span.ctypes.data_as(ol.f32p))
        assert all(span[i] == o.knj_or_q4k_weight(bp, r0 + i) for i in range(16))
    b6 = rng.integers(0, 256, 210, dtype=np.uint8)
    b6[208:210] = np.array([0.031], np.float16).view(np.uint8)
    b6p = b6.ctypes.data_as(ol.u8p)
    for r in range(256):
        assert t.t_weight6(b6p, r) == o.knj_or_q6k_weight(b6p, r)
    for r0 in range(0, 256, 16):
        t.t_span6(b6p, r0, span.ctypes.data_as(ol.f32p))
        assert all(span[i] == o.knj_or_q6k_weight(b6p, r0 + i) for i in range(16))
    for h in (0, 1, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x7C00, 0x8001, 0xFBFF):
        assert t.t_h2f(h) == o.knj_or_fp16_to_fp32(h)
    assert t.t_dot4(0x01010101, 0x01010101, 0) == 4
    assert t.t_dot4(C.c_int(0xFF02FE03 - (1 << 32)).value, 0x01020304, 10) == 10 + 3 * 4 + (-2) * 3 + 2 * 2 + (-1) * 1
    assert t.t_dot8(0x11111111, 0x11111111, 0) == 8
    assert t.t_dot8(C.c_int(0xF0000000 - (1 << 32)).value, 0x70000000, 5) == 5 + (-1) * 7
    assert t.t_dot2(0x00020003, C.c_int(0xFFFF0004 - (1 << 32)).value, 1) == 1 + 3 * 4 + 2 * (-1)
    lo, hi = C.c_int(), C.c_int()
    t.t_unpack(0xA1B2C3D4, C.byref(lo), C.byref(hi))
    assert lo.value == 0x01020304 and hi.value == 0x0A0B0C0D
    assert t.t_stride() == 68


def test_residency_objects_without_a_device(L, tmp_path):
    """The gates refuse cleanly where there is no device: no slot, no device copy; the file tier still works."""
    n = C.c_int(-1)
    if L.knj_dev_count(C.byref(n)) == 0 and n.value > 0:
        pytest.skip("a GPU is present")
    slots = L.knj_res_slots_create(2, 1024)
    assert L.knj_res_slot_acquire(slots, 0, 0, 16) == -1 and L.knj_res_slot_ptr(slots, 0) is None
    L.knj_res_slots_destroy(slots)
    path = tmp_path / "tier.bin"
    path.write_bytes(bytes(range(256)) * 4)
    eng = L.knj_res_engine_create(str(path).encode())
    buf = C.create_string_buffer(256)
    assert L.knj_res_submit_h2d(eng, buf, buf, 16, 0) == 0
    t = L.knj_res_submit_nvme_read(eng, buf, 256, 256, 1)
    assert t != 0
    while L.knj_res_poll(eng, t) == 0:
        pass
    assert L.knj_res_poll(eng, t) == 1 and buf.raw == bytes(range(256))
    bad = L.knj_res_submit_nvme_read(eng, buf, 1 << 20, 256, 0)   # past the end of the file: fails, does not hang
    while L.knj_res_poll(eng, bad) == 0:
        pass
    assert L.knj_res_poll(eng, bad) == 2
    L.knj_res_engine_destroy(eng)


def test_stack_create_refuses_bad_arguments(L):
    from kanjoos_b200._lib import MoeFfnArgs
    h = C.c_void_p()
    assert L.knj_moe_stack_create(None, 1, C.byref(h)) == -1 and not h.value
    a = (MoeFfnArgs * 1)()
    a[0].n_tokens, a[0].hidden, a[0].ffn, a[0].n_experts, a[0].top_k = 65, 2048, 768, 128, 8
    assert L.knj_moe_stack_create(a, 1, C.byref(h)) == -1 and b"n_tokens" in L.knj_last_error_string()
    a[0].n_tokens, a[0].hidden = 1, 4096
    assert L.knj_moe_stack_create(a, 1, C.byref(h)) == -1 and b"hidden" in L.knj_last_error_string()
    a[0].hidden = 2048
    assert L.knj_moe_stack_create(a, 1, C.byref(h)) == -1 and b"null tensor" in L.knj_last_error_string()
    assert L.knj_moe_stack_decode_launch(None, None) == -1
    L.knj_moe_stack_destroy(None)


def _run_ref_binary(name):
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", name)
    if not os.path.exists(exe):
        pytest.skip(f"oracle/_ref/{name} was not built (no reference tree on the build machine)")
    env = {k: v for k, v in os.environ.items() if k != "KNJ_BUILD_ARCH"}
    return subprocess.run([exe], capture_output=True, text=True, timeout=120, env=env).stdout


def test_reference_device_unit_test_passes_on_its_own_headers():
    """Baseline: the reference's tests/unit/test_c2_device.cpp, compiled unmodified against the reference's own
    src/device headers and backend.cpp with its gfx1201 build definitions: 91 assertions, none failing."""
    out = _run_ref_binary("knj_ref_c2_test")
    assert "tests passed: 91" in out and "tests failed: 0" in out, out[-2000:]


def test_reference_device_unit_test_compiled_unmodified_against_this_library():
    """The same source file, unmodified, compiled against include/device_caps.h + include/backend.h and linked
    with libknj_device.so: arch guard, capability table, labels, cap line, host probe, Backend::create /
    from_caps / would_instantiate / the four launches and the doctor header all answer as the reference's own
    implementation does. One assertion of 91 differs, and must: the dot-product label of a device without the
    sdot4 builtin names the instruction this hardware has (dp4a) instead of the gfx one."""
    out = _run_ref_binary("knj_ref_c2_on_this_library")
    assert "tests passed: 90" in out and "tests failed: 1" in out, out[-2000:]
    fails = [ln for ln in out.splitlines() if "FAIL" in ln and "RESULT" not in ln]
    assert len(fails) == 1 and "dot label mismatch" in fails[0], fails
    assert 'expected: "asm(v_dot4_i32_i8)", got: "intrinsic(dp4a)"' in out
