"""ctypes binding of libmoe_b200.so (declared in include/moe_b200.h).

There is no CPU fallback: importing this module without the built shared library raises, and
every compute call fails with MoEError when no sm_100 device is present.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmoe_b200.so"

# status codes
OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_STATE, ERR_TIMEOUT, ERR_NCCL = 0, -1, -2, -3, -4, -5, -6
# enums
GATE_TOPK, GATE_SWITCH, GATE_SHARED_TOPK = 0, 1, 2
ACT_SILU, ACT_GELU_TANH, ACT_RELU, ACT_IDENTITY = 0, 1, 2, 3
DTYPE_F32, DTYPE_BF16 = 0, 1
SHARED_NONE, SHARED_GATING, SHARED_LAYER_BLEND = 0, 1, 2
LAYOUT_IN_CONTIG, LAYOUT_OUT_CONTIG = 0, 1
EXPERT_GATED, EXPERT_STANDARD = 0, 1

EXPORTS = [
    "moe_layer_create", "moe_layer_set_expert", "moe_layer_set_expert_standard", "moe_layer_set_router", "moe_layer_set_router_noise", "moe_layer_weights_image_bytes", "moe_layer_export_weights", "moe_layer_import_weights", "moe_layer_set_aux_free", "moe_layer_aux_free_state", "moe_layer_set_router_noise_network", "moe_layer_dims",
    "moe_layer_forward", "moe_layer_forward_host", "moe_compute_gates", "moe_compute_gates_jitter", "moe_compute_loss",
    "moe_layer_set_profiling", "moe_layer_stage_ms", "moe_layer_tile_rows", "moe_layer_gemm_kernel", "moe_layer_launch_count", "moe_layer_router_rechecks",
    "moe_layer_graph_replays",
    "moe_layer_device_status", "moe_selftest_bounded_wait", "moe_ep_unique_id", "moe_ep_init", "moe_ep_set_timeout_ms",
    "moe_ep_layout", "moe_layer_destroy",
    "moe_last_error", "moe_version", "moe_route_static", "moe_route_static_scratch_bytes",
    "moe_route_static_error",
]

# Return types that are not `int` (every other export returns a status code).  One table, applied
# after the argument types, so that no later loop can overwrite a 64-bit or pointer return type.
RESTYPES = {
    "moe_layer_weights_image_bytes": C.c_int64,
    "moe_layer_launch_count": C.c_int64,
    "moe_ep_layout": C.c_int64,
    "moe_route_static_scratch_bytes": C.c_int64,
    "moe_route_static_error": C.c_char_p,
    "moe_last_error": C.c_char_p,
    "moe_version": C.c_char_p,
}


class MoEError(RuntimeError):
    """Raised for any non-zero status of the C ABI (the reference raises error()/ArgumentError)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[moe_b200 {code}] {message}")
        self.code = code


class MoeConfig(C.Structure):
    _fields_ = [
        ("num_experts", C.c_int32), ("num_shared", C.c_int32), ("top_k", C.c_int32),
        ("input_dim", C.c_int32), ("hidden_dim", C.c_int32), ("output_dim", C.c_int32),
        ("gate_kind", C.c_int32), ("activation", C.c_int32), ("compute_dtype", C.c_int32),
        ("shared_mode", C.c_int32), ("balance_alpha", C.c_float), ("z_loss_weight", C.c_float),
        ("index_base", C.c_int32), ("bias_gates_only", C.c_int32),
        ("capacity_factor", C.c_float), ("drop_tokens", C.c_int32), ("expert_kind", C.c_int32),
    ]


class ForwardOutputs(C.Structure):
    _fields_ = [
        ("loss", C.c_void_p), ("indices", C.c_void_p), ("gates", C.c_void_p), ("probs", C.c_void_p),
        ("logits", C.c_void_p), ("tokens_per_expert", C.c_void_p), ("routing_entropy", C.c_void_p),
    ]


def _load():
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m mixtureofexperts_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
    lib.moe_layer_create.argtypes = [C.POINTER(MoeConfig), i32, C.POINTER(vp)]
    lib.moe_layer_set_expert.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32]
    lib.moe_layer_set_expert_standard.argtypes = [vp, i32, vp, vp, vp, vp, i32, i32, i32]
    lib.moe_layer_set_router_noise_network.argtypes = [vp, vp, i32, i32]
    lib.moe_layer_set_aux_free.argtypes = [vp, i32, C.c_float, C.c_float, i32, vp, i64]
    lib.moe_layer_aux_free_state.argtypes = [vp, vp, vp, vp]
    lib.moe_layer_weights_image_bytes.argtypes = [vp]
    lib.moe_layer_export_weights.argtypes = [vp, vp, i64]
    lib.moe_layer_import_weights.argtypes = [vp, vp, i64]
    lib.moe_layer_set_router.argtypes = [vp, vp, vp, i32, i32]
    lib.moe_layer_set_router_noise.argtypes = [vp, vp, f32]
    lib.moe_layer_dims.argtypes = [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.moe_layer_forward.argtypes = [vp, vp, i32, i64, i32, vp, C.POINTER(ForwardOutputs), vp]
    lib.moe_layer_forward_host.argtypes = [vp, vp, i32, i64, i32, vp, C.POINTER(ForwardOutputs)]
    lib.moe_compute_gates.argtypes = [i32, i32, i32, i32, i32, vp, i64, vp, vp, vp, vp]
    lib.moe_compute_gates_jitter.argtypes = [i32, i32, i32, i32, i32, vp, vp, C.c_float, i64, vp, vp, vp, vp]
    lib.moe_compute_loss.argtypes = [f32, f32, i32, i32, i32, vp, vp, vp, i32, i64, vp, vp]
    lib.moe_layer_set_profiling.argtypes = [vp, i32]
    lib.moe_layer_stage_ms.argtypes = [vp, i32, C.POINTER(C.c_float)]
    lib.moe_layer_tile_rows.argtypes = [vp, i64]
    lib.moe_layer_gemm_kernel.argtypes = [vp, i64]
    lib.moe_layer_launch_count.argtypes = [vp]
    lib.moe_layer_router_rechecks.argtypes = [vp, C.POINTER(C.c_int64)]
    lib.moe_layer_graph_replays.argtypes = [vp, C.POINTER(C.c_int64)]
    lib.moe_layer_device_status.argtypes = [vp, C.POINTER(C.c_int32)]
    lib.moe_ep_unique_id.argtypes = [vp]
    lib.moe_ep_init.argtypes = [vp, vp, i32, i32]
    lib.moe_ep_set_timeout_ms.argtypes = [vp, i32]
    lib.moe_selftest_bounded_wait.argtypes = [i32, i32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.moe_ep_layout.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    lib.moe_layer_destroy.argtypes = [vp]
    lib.moe_route_static.argtypes = [i32, i32, i32, i32, i32, vp, i32, i64, i32, vp, vp, f32, f32, i32, vp, vp, vp, vp, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        fn.restype = RESTYPES.get(name, C.c_int)
    return lib


lib = _load()


def check(code: int) -> None:
    if code != OK:
        raise MoEError(code, lib.moe_last_error().decode("utf-8", "replace"))


def version() -> str:
    return lib.moe_version().decode()
