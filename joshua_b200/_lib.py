"""Loads `libjoshua_b200.so` (built in-tree by `joshua_b200.build`) through ctypes.

There is no fallback: if the library is missing or cannot be loaded, importing
any compute entry point raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libjoshua_b200.so"

OK, E_INVALID, E_TYPE, E_CUDA, E_NOMEM, E_EXPERT_RANGE, E_TOO_LARGE, E_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7


class JoshuaB200Error(RuntimeError):
    """A C-ABI call returned a negative status; `.code` holds it."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


_lib = None

u64, i32, u32, vp, f32 = ctypes.c_uint64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_float
pp = ctypes.POINTER(ctypes.c_void_p)

_SIGNATURES = {
    "jq_last_error": (ctypes.c_char_p, []),
    "jq_block_size": (i32, [u32, ctypes.POINTER(u64), ctypes.POINTER(u64)]),
    "jq_init": (i32, [i32, pp]),
    "jq_free": (None, [vp]),
    "jq_device_status": (i32, [vp]),
    "jq_weight_upload": (i32, [vp, u32, vp, u64, pp]),
    "jq_weight_from_device": (i32, [vp, u32, vp, u64, pp]),
    "jq_weight_slice": (i32, [vp, u64, u64, pp]),
    "jq_weight_free": (None, [vp]),
    "jq_weight_type": (u32, [vp]),
    "jq_weight_storage_size": (u64, [vp]),
    "jq_weight_block_elems": (u64, [vp]),
    "jq_weight_device_ptr": (vp, [vp]),
    "jq_matmul_t": (i32, [vp, u64, u64, u64, vp, u64, vp, u64]),
    "jq_matmul_t_f16": (i32, [vp, u64, u64, u64, vp, u64, vp, u64]),
    "jq_matmul_t_dev": (i32, [vp, u64, u64, u64, vp, vp, vp]),
    "jq_matmul_t_dev_noalloc": (i32, [vp, u64, u64, u64, vp, vp, vp]),
    "jq_dequantize": (i32, [vp, vp, u64, i32]),
    "jq_dequantize_dev": (i32, [vp, vp, u64, i32, vp]),
    "jq_embedding": (i32, [vp, vp, u64, u64, u64, vp]),
    "jq_weight_from_float": (i32, [vp, vp, u64]),
    "jq_matmul_swiglu_dev": (i32, [vp, vp, u64, u64, u64, vp, vp, ctypes.c_float, vp]),
    "jq_embedding_dev": (i32, [vp, vp, u64, u64, u64, vp, vp, vp]),
    "jq_rmsnorm_dev": (i32, [vp, vp, vp, ctypes.c_float, u64, u64, vp, vp, vp]),
    "jq_rope_append_dev": (i32, [vp, vp, u32, u32, u32, u32, u32, ctypes.c_float, vp, vp, vp, vp, vp]),
    "jq_attention_scratch_bytes": (u64, [u32, u32, u32, u32]),
    "jq_attention_decode_dev": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, vp, vp, vp, vp]),
    "jq_add_dev": (i32, [vp, vp, u64, vp, vp]),
    "jq_argmax_scratch_bytes": (u64, [u64]),
    "jq_argmax_dev": (i32, [vp, u64, u64, vp, vp, vp, vp]),
    "jq_attention_fused_qknorm_dev": (i32, [vp, vp, u32, u32, u32, u32, u32, f32, vp, vp, f32, vp, vp, vp, vp, vp, vp]),
    "jq_rope_append_prefill_dev": (i32, [vp, vp, u32, u32, u32, u32, u32, f32, vp, vp, f32, vp, vp, vp, vp, vp]),
    "jq_attention_prefill_dev": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, vp, vp, vp]),
    "jq_swiglu_dev": (i32, [vp, vp, u64, f32, vp, vp]),
    "jq_rmsnorm_strided_dev": (i32, [vp, u64, vp, f32, u64, u64, vp, vp]),
    "jq_mla_assemble_dev": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, vp, f32, vp, vp, vp, vp]),
    "jq_attention_decode_qkv_dev": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, vp, vp, vp, vp]),
    "jq_sample_greedy_dev": (i32, [vp, u64, u64, f32, vp, vp, vp, vp, vp, vp]),
    "jq_moe_create": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, pp]),
    "jq_moe_free": (None, [vp]),
    "jq_moe_forward": (i32, [vp, vp, u64, vp, vp]),
    "jq_moe_reserve": (i32, [vp, u64, u64]),
    "jq_moe_forward_dev": (i32, [vp, vp, u64, vp, vp, vp]),
    "jq_moe_route_dev": (i32, [vp, vp, u64, vp, vp, vp, vp]),
    "jq_moe_experts_dev": (i32, [vp, vp, u64, vp, vp, vp]),
    "jq_moe_experts_replay_dev": (i32, [vp, vp, vp]),
    "jq_moe_route_norm_dev": (i32, [vp, vp, u64, vp, f32, vp, vp, vp, vp]),
    "jq_moe_status": (i32, [vp]),
    "jq_moe_last_routing": (i32, [vp, u64, vp, vp]),
    "jq_ep_create": (i32, [vp, u32, u32, u32, u32, u32, u32, ctypes.POINTER(vp)]),
    "jq_ep_free": (None, [vp]),
    "jq_ep_export": (i32, [vp, vp]),
    "jq_ep_connect": (i32, [vp, vp]),
    "jq_ep_connect_loopback": (i32, [vp]),
    "jq_ep_set_poll_limit": (i32, [vp, u32]),
    "jq_ep_rows_served": (i32, [vp, ctypes.POINTER(u32)]),
    "jq_ep_forward_dev": (i32, [vp, vp, vp, vp, u64, vp, vp, vp]),
    "jq_ep_forward_norm_dev": (i32, [vp, vp, vp, vp, u64, vp, f32, vp, vp, vp, vp]),
    "jq_moe_forward_add_dev": (i32, [vp, vp, u64, vp, vp, vp, vp]),
    "jq_moe_forward_norm_add_dev": (i32, [vp, vp, u64, vp, vp, f32, vp, vp, vp]),
    "jq_matmul_swiglu_norm_dev": (i32, [vp, vp, u64, u64, u64, vp, vp, f32, vp, f32, vp]),
    "jq_matmul_norm_dev": (i32, [vp, u64, u64, u64, vp, vp, f32, vp, vp, vp]),
    "jq_attention_fused_scratch_bytes": (u64, [u32, u32, u32, u32, u32]),
    "jq_attention_fused_dev": (i32, [vp, vp, u32, u32, u32, u32, u32, f32, vp, vp, vp, vp, vp, vp]),
}


_PROFILING_SIGNATURES = {
    "jq_debug_moe_trace": (i32, [vp]),
    "jq_debug_gemm_trace": (i32, [vp]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build the CUDA library first (python -m joshua_b200.build); "
                "joshua_b200 has no CPU fallback"
            )
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        for name, (res, args) in _PROFILING_SIGNATURES.items():  # present in profiling builds only
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.restype = res
                fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise JoshuaB200Error(rc, lib().jq_last_error().decode())
