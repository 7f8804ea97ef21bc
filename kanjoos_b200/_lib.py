"""ctypes binding of libknj_device.so (the C-ABI in include/knj_device.h).

The library is the product; there is no fallback. Importing this module when
the shared object is missing raises, and every call that returns a negative
status raises KnjError with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# KNJ_DEVICE_LIB points at another build of the same library (e.g. a measurement build); default: the in-tree one
LIB_PATH = os.environ.get("KNJ_DEVICE_LIB") or os.path.join(PKG, "libknj_device.so")

DT_F32, DT_BF16, DT_F16 = 0, 1, 2
EP_FLAG_WORDS, EP_MAX_CHUNKS = 4096, 8  # KNJ_EP_FLAG_WORDS, KNJ_EP_MAX_CHUNKS


class KnjError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libknj_device status {code}: {msg}")
        self.code = code


class DeviceCapsC(C.Structure):
    _fields_ = [("arch", C.c_char * 16), ("name", C.c_char * 64), ("has_mma", C.c_int32), ("has_fp8", C.c_int32),
                ("has_dot_builtin", C.c_int32), ("wave_size", C.c_int32), ("vram_total", C.c_uint64),
                ("vram_usable", C.c_uint64), ("rebar_full_aperture", C.c_int32), ("sms", C.c_uint32),
                ("clock_khz", C.c_uint32), ("max_streams", C.c_uint32), ("num_queue_groups", C.c_uint32),
                ("smem_per_block_optin", C.c_uint32), ("l2_bytes", C.c_uint32), ("cc_major", C.c_int32),
                ("cc_minor", C.c_int32)]


class MoeFfnArgs(C.Structure):
    _fields_ = [("n_tokens", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("n_experts", C.c_int32),
                ("top_k", C.c_int32), ("x_dtype", C.c_int32), ("x", C.c_void_p), ("ldx", C.c_int64),
                ("w_router", C.c_void_p), ("router_bias", C.c_void_p), ("w_gate", C.c_void_p), ("w_up", C.c_void_p),
                ("w_down", C.c_void_p), ("norm_w", C.c_void_p), ("rms_eps", C.c_float), ("residual", C.c_int32),
                ("out", C.c_void_p), ("out_dtype", C.c_int32), ("ldo", C.c_int64), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("tap_pair_exp", C.c_void_p), ("tap_pair_w", C.c_void_p),
                ("down_format", C.c_int32), ("fused_combine", C.c_int32)]



class EpDescC(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("n_tokens_local", C.c_int32), ("hidden", C.c_int32),
                ("ffn", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32), ("n_chunks", C.c_int32),
                ("xall_ptrs", C.POINTER(C.c_void_p)), ("pe_ptrs", C.POINTER(C.c_void_p)),
                ("pw_ptrs", C.POINTER(C.c_void_p)), ("parts_ptrs", C.POINTER(C.c_void_p)),
                ("flag_ptrs", C.POINTER(C.c_void_p))]

_vp, _i, _i64, _u32, _u64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_uint32, C.c_uint64, C.c_size_t, C.c_float

# name -> (restype, argtypes); every symbol include/knj_device.h declares
SIGNATURES = {
    "knj_last_error_string": (C.c_char_p, []),
    "knj_dev_count": (_i, [C.POINTER(_i)]),
    "knj_dev_open": (_i, [_i]),
    "knj_dev_current": (_i, [C.POINTER(_i)]),
    "knj_dev_caps": (_i, [_i, C.POINTER(DeviceCapsC)]),
    "knj_dev_sync": (_i, []),
    "knj_mem_info": (_i, [C.POINTER(_sz), C.POINTER(_sz)]),
    "knj_arch_check": (_i, []),
    "knj_malloc": (_i, [C.POINTER(_vp), _sz]),
    "knj_free": (_i, [_vp]),
    "knj_host_malloc": (_i, [C.POINTER(_vp), _sz]),
    "knj_host_free": (_i, [_vp]),
    "knj_memset": (_i, [_vp, _i, _sz, _vp]),
    "knj_memcpy_h2d": (_i, [_vp, _vp, _sz]),
    "knj_memcpy_d2h": (_i, [_vp, _vp, _sz]),
    "knj_memcpy_d2d": (_i, [_vp, _vp, _sz]),
    "knj_memcpy_h2d_async": (_i, [_vp, _vp, _sz, _vp]),
    "knj_memcpy_d2h_async": (_i, [_vp, _vp, _sz, _vp]),
    "knj_memcpy_d2d_async": (_i, [_vp, _vp, _sz, _vp]),
    "knj_stream_create": (_i, [C.POINTER(_vp)]),
    "knj_stream_destroy": (_i, [_vp]),
    "knj_stream_sync": (_i, [_vp]),
    "knj_stream_query": (_i, [_vp]),
    "knj_stream_wait_event": (_i, [_vp, _vp]),
    "knj_event_create": (_i, [C.POINTER(_vp), _i]),
    "knj_event_destroy": (_i, [_vp]),
    "knj_event_record": (_i, [_vp, _vp]),
    "knj_event_query": (_i, [_vp]),
    "knj_event_sync": (_i, [_vp]),
    "knj_event_elapsed_ms": (_i, [C.POINTER(_f), _vp, _vp]),
    "knj_graph_begin": (_i, [_vp]),
    "knj_graph_end": (_i, [_vp, C.POINTER(_vp)]),
    "knj_graph_launch": (_i, [_vp, _vp]),
    "knj_graph_destroy": (_i, [_vp]),
    "knj_control_launch": (_i, [_vp, _u32, _u32, _u32, _vp]),
    "knj_probe_caps_launch": (_i, [_vp, _vp, _vp]),
    "knj_build_asum_launch": (_i, [_vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "knj_gemm_w4_i8_launch": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp]),
    "knj_dot_helpers_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "knj_q4k_dequant_launch": (_i, [_vp, _vp, _u64, _vp]),
    "knj_q6k_dequant_launch": (_i, [_vp, _vp, _u64, _vp]),
    "knj_q6k_proj_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i, _vp, _vp]),
    "knj_rmsnorm_launch": (_i, [_vp, _i, _i64, _vp, _f, _i, _i, _vp, _vp]),
    "knj_router_topk_launch": (_i, [_vp, _i, _i64, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "knj_moe_permute_launch": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "knj_moe_permute_scratch_bytes": (_sz, [_i, _i]),
    "knj_moe_permute_ws_launch": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "knj_moe_front_launch": (_i, [_vp, _i, _i64, _vp, _f, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp,
                                  _vp, _vp, _vp, _vp]),
    "knj_active_list_launch": (_i, [_vp, _i, _vp, _vp, _vp]),
    "knj_moe_stack_create": (_i, [_vp, _i, C.POINTER(_vp)]),
    "knj_moe_stack_decode_launch": (_i, [_vp, _vp]),
    "knj_moe_stack_status": (_i, [_vp, _vp]),
    "knj_moe_stack_set_wait": (_i, [_vp, C.c_longlong, _i]),
    "knj_moe_stack_destroy": (None, [_vp]),
    "knj_res_arena_create": (_vp, []),
    "knj_res_arena_alloc": (_vp, [_vp, _u64]),
    "knj_res_arena_free": (None, [_vp, _vp]),
    "knj_res_arena_destroy": (None, [_vp]),
    "knj_res_slots_create": (_vp, [_i, _u64]),
    "knj_res_slot_acquire": (_i, [_vp, _u32, _u32, _u64]),
    "knj_res_slot_release": (None, [_vp, _i]),
    "knj_res_slot_released": (_i, [_vp, _i]),
    "knj_res_slot_pin": (None, [_vp, _i]),
    "knj_res_slot_unpin": (None, [_vp, _i]),
    "knj_res_slot_load_fired": (_i, [_vp, _i]),
    "knj_res_slot_ptr": (_vp, [_vp, _i]),
    "knj_res_slot_bytes": (_u64, [_vp, _i]),
    "knj_res_slot_watch": (None, [_vp, _i, _vp, _u64]),
    "knj_res_slots_destroy": (None, [_vp]),
    "knj_res_engine_create": (_vp, [C.c_char_p]),
    "knj_res_submit_nvme_read": (_u64, [_vp, _vp, _u64, _u64, _i]),
    "knj_res_submit_nvme_write": (_u64, [_vp, _vp, _u64, _u64, _i]),
    "knj_res_submit_h2d": (_u64, [_vp, _vp, _vp, _u64, _i]),
    "knj_res_submit_d2h": (_u64, [_vp, _vp, _vp, _u64, _i]),
    "knj_res_poll": (_i, [_vp, _u64]),
    "knj_res_cancel": (_i, [_vp, _u64]),
    "knj_res_wait_on_stream": (_i, [_vp, _u64, _vp]),
    "knj_res_engine_destroy": (None, [_vp]),
    "knj_spans_enable": (_i, [_i]),
    "knj_spans_disable": (_i, []),
    "knj_spans_active": (_i, []),
    "knj_spans_epoch": (_i, [_vp]),
    "knj_span_begin": (_i, [C.c_char_p, _vp]),
    "knj_span_end": (_i, [_i, _vp]),
    "knj_spans_dropped": (_u64, []),
    "knj_spans_flush": (_i, [_vp, _vp]),
    "knj_ep_pack_launch": (_i, [_vp, _i, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "knj_ep_plan_launch": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "knj_ep_combine_partial_launch": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "knj_ep_reduce_launch": (_i, [_vp, _i, _i64, _i, _i, _vp, _i, _vp, _i, _vp]),
    "knj_ep_peer_gather_launch": (_i, [_vp, _i, _i64, _vp, _vp]),
    "knj_ep_combine_partial_peer_launch": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _vp]),
    "knj_ep_reduce_sel_launch": (_i, [_vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _vp, _i, _vp]),
    "knj_ep_create": (_i, [C.POINTER(EpDescC), C.POINTER(_vp)]),
    "knj_ep_forward_launch": (_i, [_vp, _vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "knj_ep_barrier_launch": (_i, [_vp, _vp]),
    "knj_ep_set_wait": (_i, [_vp, C.c_longlong]),
    "knj_ep_set_transport": (_i, [_vp, _i]),
    "knj_ep_status": (_i, [_vp, _vp]),
    "knj_ep_destroy": (None, [_vp]),
    "knj_moe_combine_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _vp, _i, _i64, _i, _i, _i, _vp]),
    "knj_q4k_gateup_launch": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64,
                                   _i, _i, _vp, _vp]),
    "knj_q4k_proj_launch": (_i, [_vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _vp, _vp]),
    "knj_decode_wait_limit": (None, [C.c_longlong]),
    "knj_q4k_tc_single_sm": (None, [_i]),
    "knj_launch_overlap": (None, [_i]),
    "knj_to_f16_launch": (_i, [_vp, _i, _i64, _i, _i, _vp, _vp]),
    "knj_q4k_gateup_tc_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _i, _i, _vp, _vp]),
    "knj_q4k_down_tc_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _i, _vp, _vp]),
    "knj_q6k_down_tc_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i, _i, _vp, _vp]),
    "knj_q4k_down_combine_tc_launch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i64, _i, _i, _vp, _vp]),
    "knj_moe_acc_init_launch": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp]),
    "knj_moe_acc_finish_launch": (_i, [_vp, _vp, _i, _i64, _i, _i, _vp]),
    "knj_fuse_gateup_silu_launch": (_i, [_vp, _vp, _vp, _i, _i64, _vp]),
    "knj_q4k_matmul_workspace_bytes": (_sz, [_i, _i]),
    "knj_q4k_matmul_launch": (_i, [_vp, _i, _i, _vp, _i, _i64, _i, _vp, _i64, _vp, _sz, _vp]),
    "knj_q4k_matmul_noalloc_max_scratch": (_sz, []),
    "knj_q4k_matmul_noalloc_launch": (_i, [_vp, _i, _i, _vp, _i, _i64, _i, _vp, _i64, _vp]),
    "knj_moe_ffn_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "knj_moe_ffn_decode_launch": (_i, [C.POINTER(MoeFfnArgs), _vp]),
    "knj_moe_ffn_prefill_launch": (_i, [C.POINTER(MoeFfnArgs), _vp]),
    "knj_moe_ffn_status": (_i, [C.POINTER(MoeFfnArgs), _i, _vp]),
    # flat C cover of the C++ Backend (include/backend.h)
    "knj_backend_create": (_vp, []),
    "knj_backend_from_caps": (_vp, [C.c_char_p, _i, _i, _i, _i]),
    "knj_backend_destroy": (None, [_vp]),
    "knj_backend_last_refusal": (C.c_char_p, []),
    "knj_backend_last_launch_status": (_i, []),
    "knj_backend_would_instantiate": (_i, [_vp, _i]),
    "knj_backend_arch": (C.c_char_p, [_vp]),
    "knj_backend_launch": (_i, [_vp, _i, C.POINTER(MoeFfnArgs), _vp]),
    "knj_cap_line": (_i, [C.c_char_p, _i, _i, _i, _i, C.c_char_p, _sz]),
    "knj_cap_available_c": (_i, [C.c_char_p, _i]),
    "knj_cap_label_c": (C.c_char_p, [_i]),
    "knj_check_arch_c": (_i, [C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library with typed signatures. Raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m kanjoos_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise KnjError(rc, lib().knj_last_error_string().decode(errors="replace"))
    return rc
