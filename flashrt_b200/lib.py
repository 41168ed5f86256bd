"""ctypes binding of libfrx.so, the C ABI declared in include/frx.h.

There is no fallback: if the library has not been built, importing this module raises, and every
call that fails raises FrxError with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfrx.so")

OK, ERR_ARG, ERR_SHAPE, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE = range(6)


class FrxError(RuntimeError):
    """A libfrx call returned a non-zero status (the reference throws std::runtime_error there)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libfrx error {code}: {message}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python -m flashrt_b200.build` (needs nvcc); "
                      "there is no CPU fallback")

lib = C.CDLL(LIB_PATH)

_vp, _sz, _i, _i64 = C.c_void_p, C.c_size_t, C.c_int, C.c_int64

# name -> (restype, argtypes); every symbol include/frx.h declares
SIGNATURES = {
    "frx_version": (_i, []),
    "frx_last_error": (C.c_char_p, []),
    "frx_profile_begin": (_i, []),
    "frx_profile_end": (_i, [_vp, _vp, _i]),
    "frx_profile_class_name": (C.c_char_p, [_i]),
    "frx_q2_mat_bytes": (_sz, [_i, _i]),
    "frx_q2_expert_bytes": (_sz, [_i, _i]),
    "frx_q2_expert_stride": (_sz, [_i, _i]),
    "frx_q2_repack": (_i, [_vp, _i, _i, _vp, _vp]),
    "frx_q2_tile_experts": (_i, [_vp, _sz, _vp, _sz, _i, _i, _i, _vp]),
    "frx_q2_untile_experts": (_i, [_vp, _sz, _vp, _sz, _i, _i, _i, _vp]),
    "frx_q2_dequant_expert": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp]),
    "frx_arena_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i]),
    "frx_arena_destroy": (_i, [_vp]),
    "frx_arena_base": (_vp, [_vp]),
    "frx_arena_blob": (_vp, [_vp, _i, _i]),
    "frx_arena_stride": (_sz, [_vp]),
    "frx_arena_total_bytes": (_sz, [_vp]),
    "frx_arena_load_planar": (_i, [_vp, _i, _i, _i, _vp, _sz, _vp]),
    "frx_route_topk": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "frx_quantize_q8": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "frx_moe_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "frx_moe_decode_workspace_offset": (_sz, [_i, _i, _i, _i, C.c_char_p]),
    "frx_moe_decode": (_i, [_vp, _sz, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "frx_moe_decode_static": (_i, [_vp, _sz, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "frx_moe_decode_ep": (_i, [_vp, _sz, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "frx_moe_layer_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "frx_moe_layer": (_i, [_vp, _sz, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "frx_gguf_open": (_i, [_vp, C.c_char_p]),
    "frx_gguf_close": (_i, [_vp]),
    "frx_gguf_tensor_count": (_i, [_vp]),
    "frx_gguf_tensor_name": (C.c_char_p, [_vp, _i]),
    "frx_gguf_get_int": (C.c_int64, [_vp, C.c_char_p, C.c_int64]),
    "frx_gguf_tensor": (_i, [_vp, C.c_char_p, _vp, _vp, _vp, _vp, _vp]),
    "frx_arena_load_gguf": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "frx_router_logits": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "frx_moe_layer_ep": (_i, [_vp, _sz, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "frx_ep_buffer_bytes": (_sz, [_i, _i]),
    "frx_ep_flags_offset": (_sz, [_i, _i]),
    "frx_ep_buffer_create": (_i, [_vp, _i, _i]),
    "frx_ep_buffer_destroy": (_i, [_vp]),
    "frx_ipc_export": (_i, [_vp, _vp]),
    "frx_ipc_open": (_i, [_vp, _vp]),
    "frx_ipc_close": (_i, [_vp]),
    "frx_ep_debug_stamps": (_i, [_vp, _i, _i, _vp]),
    "frx_debug_set_consumer_warps": (_i, [_i]),
    "frx_debug_set_gate_up_chunks": (_i, [_i]),
    "frx_debug_set_narrow_items": (_i, [_i]),
    "frx_debug_set_four_group_tasks": (_i, [_i]),
    "frx_debug_set_small_launch_limits": (_i, [_i, _i]),
    "frx_debug_set_fused_ffn": (_i, [_i]),
    "frx_debug_set_fold_quant": (_i, [_i]),
    "frx_debug_set_evict_first": (_i, [_i]),
    "frx_debug_set_down_task_weight": (_i, [_i]),
    "frx_debug_set_down_item_weight": (_i, [_i]),
    "frx_debug_set_stream_stamps": (_i, [_vp]),
    "frx_debug_set_ffn_buffers": (_i, [_i, _i]),
    "frx_debug_set_wait_limit_ns": (_i, [C.c_ulonglong]),
    "frx_moe_decode_static_status": (_i, [_vp]),
    "frx_moe_layer_ep_allreduce": (_i, [_vp, _sz, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "frx_moe_layer_ep_allreduce_dealt": (_i, [_vp, _sz, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "frx_moe_layer_host_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "frx_moe_layer_host": (_i, [_vp, _sz, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_moe_layers_host_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "frx_moe_layers_host": (_i, [_vp, _sz, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_workspace_status": (_i, [_vp, _vp]),
    "frx_moe_hits_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "frx_moe_hits": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp, _sz, _vp, _vp, _i]),
    "frx_moe_combine": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "frx_moe_prefill_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "frx_moe_prefill": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_moe_prefill_umma": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_moe_prefill_stream": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_moe_prefill_ex": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp, _i, _i]),
    "frx_moe_prefill_umma_ex": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp, _i, _i]),
    "frx_moe_prefill_stream_ex": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp, _i, _i]),
    "frx_chain_rmsnorm_unit": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "frx_moe_prefill_q8_ep": (_i, [_vp, _sz, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp, _i]),
    "frx_moe_prefill_stream_q8_ep": (_i, [_vp, _sz, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _sz, _vp]),
    "frx_moe_combine_partial": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "frx_gemv_q8_1_bytes": (_sz, [_i64, _i]),
    "frx_gemv_row_bytes": (_i64, [C.c_uint32, _i64]),
    "frx_gemv_quantize_q8_1": (_i, [_vp, _i64, _i, _vp, _vp]),
    "frx_gemv_swiglu_q8_1": (_i, [_vp, _vp, _i64, _i, _vp, _vp]),
    "frx_gemv_matvec_q": (_i, [C.c_uint32, _vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "frx_gemv_matvec": (_i, [C.c_uint32, _vp, _vp, _vp, _i64, _i64, _i, _vp, _vp]),
    "frx_gemv_moe_q2_0": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _i, _vp]),
    "frx_gemv_moe_q": (_i, [C.c_uint32, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _i, _vp]),
    "frx_gemm_workspace_bytes": (_sz, [_i64, _i64]),
    "frx_gemm_moe_prepare": (_i, [_vp, C.c_uint32, _i, _vp, _i, _vp, _i64, _i, _i64, _vp, _sz, _vp]),
    "frx_gemm_moe_run": (_i, [_vp, _vp, _i64, _vp, _i64, _vp]),
    "frx_gemm_moe": (_i, [C.c_uint32, _vp, _i64, _i, _vp, _i, _vp, _i64, _i, _vp, _i64, _i64, _vp, _sz, _vp]),
    "frx_convert_q8_0_to_q2_0": (_i, [_vp, _vp, _sz, _vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)   # AttributeError here means the header and the library disagree
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.frx_last_error().decode(errors="replace")


def check(rc: int) -> None:
    if rc != OK:
        raise FrxError(rc, last_error())
