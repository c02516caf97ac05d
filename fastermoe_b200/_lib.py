"""ctypes binding of libfmoe_b200.so (declared in include/fmoe_b200.h).

The library is the product: there is no fallback.  Importing this module
without the built library raises, and every call converts a negative status
into ``RuntimeError`` carrying the library's error text.
"""
import ctypes
import os
from ctypes import c_int32, c_int64, c_size_t, c_void_p, c_char_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfmoe_b200.so")

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
GEMM_FORMS = {"auto": 0, "pair": 1, "tc1": 2, "simt": 3}
MAX_EXPERTS = 4096


class PeerSeg(ctypes.Structure):
    _fields_ = [("dst_rank", c_int32), ("reserved", c_int32), ("src_row", c_int64), ("dst_row", c_int64),
                ("rows", c_int64)]


class Move(ctypes.Structure):
    """Mirror of fmoe_move_t."""
    _fields_ = [("peer", c_int32), ("is_send", c_int32), ("src_row", c_int64), ("dst_row", c_int64),
                ("rows", c_int64), ("local", c_int32), ("step", c_int32)]


class Arrival(ctypes.Structure):
    """Mirror of fmoe_arrival_t."""
    _fields_ = [("comm", c_void_p), ("plan", c_void_p), ("out", c_void_p), ("in_rows", c_int64), ("out_rows", c_int64),
                ("row_bytes", c_int64), ("n_expert", c_int32), ("overlap_sms", c_int32), ("gather", c_int32),
                ("use", c_int32), ("src", c_void_p), ("row_of", c_void_p), ("scale", c_void_p), ("src_rows", c_int64),
                ("row_div", c_int32), ("dtype", c_int32)]


class FusedGeometry(ctypes.Structure):
    """Mirror of fmoe_fused_geometry_t."""
    _fields_ = [("n_steps", c_int32), ("gran", c_int32), ("global_rows", c_int64), ("shadow_rows", c_int64)]


class MlpParams(ctypes.Structure):
    """Mirror of fmoe_mlp_params_t."""
    _fields_ = [(n, c_void_p) for n in ("w1", "w2", "b1", "b2", "gw1", "gw2", "gb1", "gb2")]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m fastermoe_b200.build` "
            "(there is no CPU or PyTorch fallback for the CUDA operators)")
    # NCCL is bound lazily with dlopen(RTLD_NOLOAD) inside the library; importing
    # torch first makes sure the copy it ships is the one found.
    return ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)


lib = _load()

P = c_void_p
I32, I64 = c_int32, c_int64
PEER_UNAVAILABLE = 1      # FMOE_PEER_UNAVAILABLE

_SIGS = {
    "fmoe_last_error_string": (c_char_p, []),
    "fmoe_version": (c_int32, []),
    "fmoe_built_for_sm": (c_int32, []),
    "fmoe_device_status": (I32, [POINTER(c_int32)]),
    "fmoe_gemm_set_form": (I32, [I32]),
    "fmoe_gemm_set_sm_limit": (I32, [I32]),
    "fmoe_routing_scratch_bytes": (c_size_t, [I64, I32]),
    "fmoe_expert_count": (I32, [P, P, I64, I32, P]),
    "fmoe_assign_pos": (I32, [P, P, P, I64, I32, P, P]),
    "fmoe_count_and_pos": (I32, [P, I64, I32, P, P, P, P, P, P]),
    "fmoe_static_scratch_capacity": (c_size_t, []),
    "fmoe_count_and_pos_static": (I32, [P, I64, I32, P, P, P, P, P]),
    "fmoe_limit_by_capacity": (I32, [P, P, P, I32, I32, P]),
    "fmoe_prune_gate_by_capacity": (I32, [P, P, P, I64, I32, P, P]),
    "fmoe_local_scatter": (I32, [P, P, P, I64, I64, I64, I32, P]),
    "fmoe_local_gather": (I32, [P, P, P, I64, I64, I64, P, P]),
    "fmoe_local_gather_inv": (I32, [P, P, P, I64, I64, P]),
    "fmoe_local_gather_sum": (I32, [P, P, P, I64, I32, I64, I32, P]),
    "fmoe_local_gather_add_scratch_bytes": (c_size_t, [I64]),
    "fmoe_local_gather_add": (I32, [P, P, P, I64, I64, I64, I32, P, P]),
    "fmoe_combine_forward": (I32, [P, P, P, P, I64, I32, I64, I32, P]),
    "fmoe_combine_backward": (I32, [P, P, P, P, P, P, I64, I32, I64, I32, P]),
    "fmoe_linear_scratch_bytes": (c_size_t, [I64, I64, I64, I32, I32]),
    "fmoe_linear_forward": (I32, [P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, P]),
    "fmoe_linear_backward": (I32, [P, P, P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, I32, P, P]),
    "fmoe_linear_backward_colsum": (I32, [P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, I32, P, P]),
    "fmoe_comm_unique_id": (I32, [P]),
    "fmoe_comm_init": (I32, [P, I32, I32, I32, POINTER(c_void_p)]),
    "fmoe_comm_destroy": (I32, [P]),
    "fmoe_comm_rank": (I32, [P, POINTER(c_int32), POINTER(c_int32)]),
    "fmoe_expert_exchange": (I32, [P, P, P, P, P, I32, I32, P]),
    "fmoe_plan_global_scatter": (I32, [P, P, P, I32, I32, I32, P, I32, POINTER(c_int32), POINTER(c_int64)]),
    "fmoe_global_scatter": (I32, [P, P, P, P, P, P, I64, I64, I64, I32, I32, P, P]),
    "fmoe_global_gather": (I32, [P, P, P, P, P, P, I64, I64, I64, I32, I32, P, P]),
    "fmoe_gate_topk": (I32, [P, I64, I32, I32, I32, P, P, P]),
    "fmoe_gate_topk_backward": (I32, [P, P, I64, I32, I32, I32, P, P]),
    "fmoe_peer_plan": (I32, [P, P, I32, I32, I32, I32, P, POINTER(c_int32), P, POINTER(c_int32), I32, POINTER(c_int64)]),
    "fmoe_peer_enable": (I32, [P, I64, I64, P]),
    "fmoe_peer_pool_bytes": (I64, [P]),
    "fmoe_pool_alloc": (P, [c_size_t, I32, P]),
    "fmoe_pool_free": (None, [P, c_size_t, I32, P]),
    "fmoe_peer_wait_probe": (I32, [P, I32, I32, P]),
    "fmoe_peer_set_timeout_ms": (I32, [P, I32]),
    "fmoe_peer_plan_bytes": (c_size_t, [I32, I32]),
    "fmoe_peer_plan_offsets_at": (I64, [I32, I32]),
    "fmoe_peer_plan_table_at": (I64, [I32, I32]),
    "fmoe_peer_plan_exchange": (I32, [P, P, P, I64, P, I32, P]),
    "fmoe_peer_plan_from_table": (I32, [P, P, P, I32, I32, I32, P, P]),
    "fmoe_peer_plan_read": (I32, [P, I32, I32, I32, P, I32, POINTER(c_int32), POINTER(c_int64), POINTER(c_int64), POINTER(c_int32)]),
    "fmoe_peer_scatter_planned": (I32, [P, P, P, P, I64, I64, I64, I32, P]),
    "fmoe_peer_gather_planned": (I32, [P, P, P, P, I64, I64, I64, I32, P]),
    "fmoe_peer_scatter_planned_async": (I32, [P, P, P, P, I64, I64, I64, I32, I32, P, P]),
    "fmoe_peer_arrival_finish": (I32, [P, P]),
    "fmoe_peer_gather_planned_async": (I32, [P, P, P, P, I64, I64, I64, I32, I32, I32, P, P]),
    "fmoe_peer_scatter_planned_rows": (I32, [P, P, I64, P, I32, P, I32, P, P, I64, I64, I64, I32, P]),
    "fmoe_abi_sizeof": (ctypes.c_size_t, [ctypes.c_char_p]),
    "fmoe_peer_scatter_fused_begin": (I32, [P, P, I64, P, I32, P, I32, P, P, I64, I64, I64, I32, P, P]),
    "fmoe_peer_gather_fused_begin": (I32, [P, P, P, I64, I64, I32, P, P]),
    "fmoe_linear_forward_overlapped": (I32, [P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, P, P, P]),
    "fmoe_linear_backward_overlapped": (I32, [P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, I32, P, P, P, P]),
    "fmoe_device_status_clear": (I32, []),
    "fmoe_peer_slot_bytes": (I64, [P]),
    "fmoe_peer_global_scatter": (I32, [P, P, P, P, P, I64, I64, I64, I32, I32, P]),
    "fmoe_peer_global_gather": (I32, [P, P, P, P, P, I64, I64, I64, I32, I32, P]),
    "fmoe_exchange_cache_info": (I32, [P, P, P, I32, I32, P]),
    "fmoe_model_broadcast": (I32, [P, P, I64, I32, P]),
    "fmoe_gradient_reduce": (I32, [P, P, I64, I32, I32, P]),
    "fmoe_generate_cached_count": (I32, [P, P, P, P, I32, I32, I32, P]),
    "fmoe_fused_compute_ptrs": (I32, [P, P, P, I32, I32, I32, P, P, P]),
    "fmoe_fused_geometry": (I32, [P, P, P, I32, I32, I32, I32, P]),
    "fmoe_fused_forward": (I32, [P, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, I32, I32, P, P, P]),
    "fmoe_fused_backward": (I32, [P, P, P, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I32, I32, I32, I32, I32, P, P, P]),
}

EXPORTS = tuple(_SIGS)

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error():
    s = lib.fmoe_last_error_string()
    return s.decode("utf-8", "replace") if s else ""


def check(status, what):
    """Raise RuntimeError for a non-zero status returned by the library."""
    if status != 0:
        raise RuntimeError(f"{what} failed (status {status}): {last_error()}")
