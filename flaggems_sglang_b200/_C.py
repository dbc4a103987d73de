"""ctypes binding of libfmoe_b200.so (the C ABI declared in include/fmoe_b200.h).

There is no CPU implementation behind these ops: a missing library or a call
without a CUDA device raises instead of falling back.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p

import torch  # noqa: F401  (loads the CUDA runtime the library links against)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfmoe_b200.so")

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_TIMEOUT = 0, 1, 2, 3, 4
F32, BF16, E4M3 = 0, 1, 2
VARIANT_AUTO, VARIANT_SIMT, VARIANT_STREAM, VARIANT_TCGEN05 = 0, 1, 2, 3
W_K_MAJOR, W_N_MAJOR = 0, 1
SCALE_BLOCK128, SCALE_CHANNEL = 0, 1
VARIANTS = {"auto": 0, "simt": 1, "stream": 2, "tcgen05": 3}
ACTIVATIONS = {"silu": 0, "gelu": 1, "swiglu_oai": 2}
VARIANT_NAMES = {v: k for k, v in VARIANTS.items()}

DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float8_e4m3fn: E4M3}


class FmoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"fmoe_b200 error {code}: {msg}")
        self.code = code


class _SizedStructure(Structure):
    """ctypes mirror of an argument struct that begins with `struct_size`: filled in on construction."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.struct_size = ctypes.sizeof(type(self))


class GemmArgs(_SizedStructure):
    """Mirror of struct fmoe_gemm_args."""

    _fields_ = [
        ("struct_size", c_uint32), ("w_layout", c_int32),
        ("dtype", c_int32), ("out_dtype", c_int32), ("variant", c_int32), ("num_experts", c_int32),
        ("top_k", c_int32), ("block_size", c_int32), ("a_gather", c_int32), ("activation", c_int32),
        ("numel", c_int64), ("n", c_int64), ("k", c_int64), ("a_rows", c_int64),
        ("sorted_cap", c_int64), ("max_blocks", c_int64),
        ("a", c_void_p), ("a_scale", c_void_p), ("w", c_void_p), ("w_scale", c_void_p),
        ("sorted_token_ids", c_void_p), ("expert_ids", c_void_p), ("num_tokens_post_padded", c_void_p),
        ("row_scale", c_void_p), ("out", c_void_p), ("out_scale", c_void_p),
        ("bias", c_void_p), ("act_alpha", c_float), ("act_limit", c_float), ("out_rows", c_void_p),
        ("split_ws", c_void_p), ("split_ws_bytes", c_int64), ("scale_mode", c_int32), ("a_scale_gather", c_int32),
    ]


class FusedArgs(_SizedStructure):
    """Mirror of struct fmoe_fused_args."""

    _fields_ = [
        ("struct_size", c_uint32), ("w_layout", c_int32),
        ("dtype", c_int32), ("variant", c_int32), ("num_experts", c_int32), ("top_k", c_int32),
        ("apply_router_weight_on_input", c_int32), ("no_combine", c_int32), ("zero_dropped", c_int32),
        ("activation", c_int32),
        ("T", c_int64), ("H", c_int64), ("I", c_int64),
        ("routed_scaling_factor", c_float), ("scale_mode", c_int32),
        ("hidden", c_void_p), ("w1", c_void_p), ("w2", c_void_p), ("w1_scale", c_void_p), ("w2_scale", c_void_p),
        ("topk_weights", c_void_p), ("topk_ids", c_void_p), ("out", c_void_p), ("workspace", c_void_p),
        ("workspace_bytes", c_int64), ("b1", c_void_p), ("b2", c_void_p), ("act_alpha", c_float),
        ("act_limit", c_float), ("out_rows", c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/fmoe_b200.h declares
SIGNATURES = {
    "fmoe_version": (c_int, []),
    "fmoe_gemm_split_workspace_bytes": (c_int64, []),
    "fmoe_debug_tail_plan": (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    "fmoe_last_error": (c_char_p, []),
    "fmoe_sm_count": (c_int, []),
    "fmoe_topk_softmax": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fmoe_topk_grouped": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_void_p, c_void_p, c_void_p]),
    "fmoe_moe_align_block_size": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                          c_void_p, c_void_p]),
    "fmoe_moe_align_workspace_bytes": (c_int64, [c_int64, c_int]),
    "fmoe_moe_align_block_size_ws": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                             c_void_p, c_void_p, c_int64, c_void_p]),
    "fmoe_quant_fp8_group128": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p,
                                        c_void_p, c_void_p, c_void_p]),
    "fmoe_quant_fp8_per_token": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p,
                                         c_void_p, c_void_p, c_void_p]),
    "fmoe_gather_rows": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p, c_void_p,
                                 c_void_p]),
    "fmoe_gemm1_silu": (c_int, [POINTER(GemmArgs), c_void_p]),
    "fmoe_gemm2": (c_int, [POINTER(GemmArgs), c_void_p]),
    "fmoe_moe_sum": (c_int, [c_void_p, c_int, c_int64, c_int, c_int64, c_float, c_void_p, c_void_p]),
    "fmoe_moe_sum_add": (c_int, [c_void_p, c_int, c_int64, c_int, c_int64, c_float, c_void_p, c_void_p, c_void_p]),
    "fmoe_pick_variant": (c_int, [c_int, c_int64, c_int, c_int64, c_int64, c_int, POINTER(c_int), POINTER(c_int)]),
    "fmoe_fused_experts_workspace_bytes": (c_int64, [POINTER(FusedArgs)]),
    "fmoe_fused_experts": (c_int, [POINTER(FusedArgs), c_void_p]),
    "fmoe_static_scratch_bytes": (c_int64, []),
    "fmoe_fused_experts_static": (c_int, [POINTER(FusedArgs), c_void_p]),
    "fmoe_ep_buffer_create": (c_int, [c_int64, POINTER(c_void_p), c_void_p]),
    "fmoe_ep_buffer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "fmoe_ep_buffer_close": (c_int, [c_void_p]),
    "fmoe_ep_buffer_destroy": (c_int, [c_void_p]),
    "fmoe_ep_expert_counts": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "fmoe_ep_dispatch_sorted": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "fmoe_ep_recv_tables": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_void_p, c_int64, c_void_p,
                                    c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "fmoe_ep_scatter_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "fmoe_selftest_bounded_wait": (c_int, [c_int64, c_void_p]),
    "fmoe_debug_tcgen05_wait_profile": (c_int, [c_void_p, c_int]),
    "fmoe_debug_stage_events": (c_int, [c_void_p, c_int]),
    "fmoe_debug_wait_profile": (c_int, [c_int, c_void_p, c_int]),
    "fmoe_check_device_status": (c_int, [c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises ImportError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m flaggems_sglang_b200.build` "
                "(there is no CPU fallback for these ops)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise FmoeError(rc, lib().fmoe_last_error().decode("utf-8", "replace"))


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "flaggems_sglang_b200 ops run on CUDA (sm_100a) tensors only; there is no CPU path "
                f"(got a tensor on {t.device})"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise RuntimeError("no tensor given")
    return dev


def check_device_status(device=None) -> None:
    """Synchronises the current stream and raises if a bounded wait inside a tcgen05 kernel gave up."""
    check(lib().fmoe_check_device_status(stream_ptr(device)))
