"""ctypes view of ``libb200mk.so`` (declarations in ``include/b200_megakernel.h``).

There is no fallback: if the library is absent and cannot be built, importing
callers get a ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache

from . import build as _build

MK_ABI_VERSION = 1
MK_ERR_BAD_ARGUMENT = 10001
MK_ERR_UNSUPPORTED = 10002
MK_ERR_RESIDENCY = 10003
MK_ERR_DEVICE_WAIT = 10004

MK_STEP_EMBED = 1
MK_STEP_RESET_BARRIERS = 2
MK_STEP_WRITE_TOKEN = 4
MK_STEP_TIMINGS = 8

MK_TP_HANDLE_BYTES = 64
MK_OPT_WAIT_BUDGET_CYCLES = 0
MK_OPT_EARLY_POLL_SHIFT = 1
MK_OPT_MAX_INFLIGHT_TILES = 2
MK_OPT_DOWN_FOLD_LAST = 3
MK_OPT_DOWN_FOLD_LOCAL = 4
MK_OPT_COOPERATIVE_LAUNCH = 5

MK_WEIGHTS_BF16 = 0
MK_WEIGHTS_NVFP4 = 1

EXPORTED_SYMBOLS = [
    "mk_last_error", "mk_create", "mk_set_schedule", "mk_step", "mk_query", "mk_status",
    "mk_set_wait_budget", "mk_status_detail", "mk_destroy", "mk_nvfp4_quantize", "mk_gemv", "mk_abi_sizeof", "mk_set_option",
    "mk_gemv_static", "mk_tp_init", "mk_tp_connect", "mk_gemv_workspace_bytes",
    "mk_linear_batched", "mk_linear_batched_splits",
    "mk_nvfp4_native_scale_bytes", "mk_nvfp4_quantize_native", "mk_linear_batched_nvfp4",
    "mk_batched_create", "mk_step_batched", "mk_batched_status", "mk_batched_destroy",
    "mk_batched_set_activation_scale",
    "mk_fp4_chain_prepare", "mk_fp4_chain_run", "mk_fp4_chain_status", "mk_fp4_chain_destroy",
    "mk_prefill_batched", "mk_batched_set_overlap", "mk_throughput_bind", "mk_throughput_set_schedule", "mk_step_throughput",
]


class MkNvfp4Matrix(C.Structure):
    _fields_ = [("packed", C.c_void_p), ("scales", C.c_void_p), ("tensor_scale", C.c_float)]


class MkModelDesc(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("weight_format", C.c_int32),
        ("hidden_size", C.c_int32), ("num_layers", C.c_int32), ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("intermediate_size", C.c_int32),
        ("vocab_size", C.c_int32), ("attn_scale", C.c_float), ("rms_norm_eps", C.c_float),
        ("qkv_w", C.c_void_p), ("o_w", C.c_void_p), ("up_w", C.c_void_p), ("gate_w", C.c_void_p),
        ("down_w", C.c_void_p), ("lm_head_w", C.c_void_p),
        ("attn_norm_w", C.c_void_p), ("mlp_norm_w", C.c_void_p), ("lm_head_norm_w", C.c_void_p),
        ("embed_w", C.c_void_p),
        ("qkv_q", C.POINTER(MkNvfp4Matrix)), ("o_q", C.POINTER(MkNvfp4Matrix)), ("up_q", C.POINTER(MkNvfp4Matrix)),
        ("gate_q", C.POINTER(MkNvfp4Matrix)), ("down_q", C.POINTER(MkNvfp4Matrix)),
        ("lm_head_q", C.POINTER(MkNvfp4Matrix)),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("kv_batch", C.c_int32), ("kv_max_len", C.c_int32),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("rope_positions", C.c_int32),
        ("hidden_states", C.c_void_p), ("q_post_rope", C.c_void_p), ("attn_out", C.c_void_p),
        ("attn_lse_intermediates", C.c_void_p), ("attn_out_intermediates", C.c_void_p),
        ("max_partials", C.c_int32), ("silu_out", C.c_void_p), ("logits", C.c_void_p),
        ("barriers", C.c_void_p), ("barrier_rows", C.c_int32), ("barrier_cols", C.c_int32),
        ("skip_attn_reduction", C.c_int32),
    ]


class MkFp4ChainOperand(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("x_packed", C.c_void_p), ("x_scales_native", C.c_void_p), ("output", C.c_void_p),
        ("w_packed", C.c_void_p), ("w_scales_native", C.c_void_p), ("m", C.c_int32), ("k", C.c_int32),
        ("input_tensor_scale", C.c_float), ("alpha", C.c_float),
    ]


class MkThroughputBuffers(C.Structure):
    _fields_ = [
        ("rms_rope_intermediates", C.c_void_p), ("rms_gate_intermediates", C.c_void_p),
        ("rms_lm_head_intermediates", C.c_void_p), ("post_ln_rope_q", C.c_void_p), ("attn_out", C.c_void_p),
        ("silu_out", C.c_void_p), ("barriers", C.c_void_p), ("barrier_cols", C.c_int32), ("batch_size", C.c_int32),
    ]


class MkLaunchInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "cooperative_launch", "physical_sms", "resident_worker_capacity", "active_workers", "threads_per_cta",
        "consumer_warps", "registers_per_thread", "local_bytes_per_thread", "static_smem_bytes",
        "dynamic_smem_bytes", "stage_count", "stage_bytes", "resident_ctas_per_sm", "queue_len",
    )] + [("scratch_bytes", C.c_int64), ("down_fold_mode", C.c_int32), ("reserved", C.c_int32)]


class MkStatus(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("code", "worker", "opcode", "slot", "detail", "expected")]


class MegakernelError(RuntimeError):
    """A non-zero return code from the library, with its error text."""

    def __init__(self, code: int, text: str):
        super().__init__(f"[{code}] {text}")
        self.code = code


@lru_cache(maxsize=1)
def load() -> C.CDLL:
    try:
        path = _build.build_library()
    except Exception as exc:  # no silent fallback
        if not _build.LIBRARY.exists():
            raise RuntimeError(
                f"libb200mk.so is missing and could not be built ({exc}); "
                "run `python -m thor_megakernels_b200.build`"
            ) from exc
        path = _build.LIBRARY  # stale but present (e.g. no nvcc on this box)
    lib = C.CDLL(str(path))
    vp, i32, u32, f32 = C.c_void_p, C.c_int32, C.c_uint32, C.c_float
    lib.mk_last_error.restype = C.c_char_p
    lib.mk_last_error.argtypes = []
    lib.mk_create.argtypes = [C.POINTER(MkModelDesc), C.POINTER(vp)]
    lib.mk_set_schedule.argtypes = [vp, vp, vp, i32, i32]
    lib.mk_step.argtypes = [vp, i32, u32, vp, vp, vp]
    lib.mk_query.argtypes = [vp, C.POINTER(MkLaunchInfo)]
    lib.mk_status.argtypes = [vp, C.POINTER(MkStatus), vp]
    lib.mk_set_wait_budget.argtypes = [vp, C.c_int64]
    lib.mk_destroy.argtypes = [vp]
    lib.mk_destroy.restype = None
    lib.mk_nvfp4_quantize.argtypes = [vp, vp, vp, vp, i32, i32, f32, vp]
    lib.mk_gemv.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, i32, i32, vp, C.c_int64, vp]
    lib.mk_gemv_static.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, i32, i32, vp]
    lib.mk_gemv_workspace_bytes.argtypes = [i32, i32]
    lib.mk_linear_batched.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    lib.mk_linear_batched_splits.argtypes = [i32, i32, i32]
    lib.mk_nvfp4_native_scale_bytes.argtypes = [i32, i32]
    lib.mk_nvfp4_native_scale_bytes.restype = C.c_int64
    lib.mk_nvfp4_quantize_native.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    lib.mk_linear_batched_nvfp4.argtypes = [vp, vp, f32, vp, vp, f32, vp, vp, i32, i32, i32, i32, vp, vp]
    lib.mk_batched_create.argtypes = [C.POINTER(MkModelDesc), i32, C.POINTER(vp)]
    lib.mk_step_batched.argtypes = [vp, vp, vp, i32, vp, vp]
    lib.mk_batched_status.argtypes = [vp, vp]
    lib.mk_batched_set_activation_scale.argtypes = [vp, f32]
    lib.mk_batched_destroy.argtypes = [vp]
    lib.mk_batched_destroy.restype = None
    lib.mk_fp4_chain_prepare.argtypes = [C.POINTER(MkFp4ChainOperand), i32, i32, i32, C.POINTER(vp)]
    lib.mk_fp4_chain_run.argtypes = [vp, vp]
    lib.mk_fp4_chain_status.argtypes = [vp, vp]
    lib.mk_fp4_chain_destroy.argtypes = [vp]
    lib.mk_fp4_chain_destroy.restype = None
    lib.mk_batched_set_overlap.argtypes = [i32]
    lib.mk_status_detail.argtypes = [vp, vp, i32, C.POINTER(C.c_int32)]
    lib.mk_prefill_batched.argtypes = [vp, vp, i32, i32, i32, vp, vp]
    lib.mk_throughput_bind.argtypes = [vp, C.POINTER(MkThroughputBuffers)]
    lib.mk_throughput_set_schedule.argtypes = [vp, vp, i32, i32]
    lib.mk_step_throughput.argtypes = [vp, i32, vp]
    lib.mk_tp_init.argtypes = [vp, i32, i32, i32, vp]
    lib.mk_tp_connect.argtypes = [vp, vp, i32]
    lib.mk_abi_sizeof.argtypes = [i32]
    lib.mk_set_option.argtypes = [vp, i32, C.c_int64]
    for name in EXPORTED_SYMBOLS:
        if name not in ("mk_last_error", "mk_destroy", "mk_gemv_workspace_bytes", "mk_batched_destroy", "mk_fp4_chain_destroy",
                        "mk_nvfp4_native_scale_bytes"):
            getattr(lib, name).restype = C.c_int
    lib.mk_gemv_workspace_bytes.restype = C.c_int64
    return lib


def check(code: int):
    if code != 0:
        raise MegakernelError(code, load().mk_last_error().decode())
