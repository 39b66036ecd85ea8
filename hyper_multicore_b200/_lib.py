"""ctypes binding of libhmc_b200.so (the C ABI declared in include/hmc_b200.h).

The library is the only compute path of this package: there is no CPU or PyTorch fallback.
Loading fails loudly when the shared library has not been built.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_float, c_int32, c_int64, c_uint64, c_void_p
from pathlib import Path

import torch

_PACKAGE = Path(__file__).resolve().parent
LIBRARY_PATH = _PACKAGE / "libhmc_b200.so"

HMC_GEMM_RAGGED_M = 0
HMC_GEMM_RAGGED_K = 1
HMC_MAJOR_K = 0
HMC_MAJOR_MN = 1
HMC_EPI_STORE_BF16 = 0
HMC_EPI_STORE_F32 = 1
HMC_EPI_SWIGLU = 2
HMC_EPI_SWIGLU_GRAD = 3
HMC_EPI_SWIGLU_MXQ = 4
HMC_EPI_SWIGLU_GRAD_MXQ = 5
HMC_STATUS_WORDS = 8
HMC_CTRL_SOURCE = 1296
HMC_CTRL_COUNTS = 1552
HMC_CLAMP_NONE, HMC_CLAMP_BEFORE_SILU, HMC_CLAMP_AFTER_SILU = 0, 1, 2
HMC_PROFILE_KINDS = ("grouped_gemm", "mx_gemm", "mx_quant", "ep", "route")
HMC_MOE_LAYOUT = {"EIO": 0, "EOI": 1}
HMC_MOE_DISPATCH = {"push": 0, "pull": 1}

STATUS_NAMES = {
    0: "ok",
    1: "pipeline wait timed out",
    2: "rows of an expert never arrived",
    3: "a peer never published ready",
    4: "an index was out of range",
}


class HmcError(RuntimeError):
    """A check inside the native library failed."""


class GemmCombine(ctypes.Structure):
    """Mirror of ``hmc_gemm_combine``."""

    _fields_ = [
        ("segment_start", c_void_p), ("combine_target_off", c_void_p),
        ("peer_buffers", c_void_p), ("peer_ctrl", c_void_p),
        ("ep", c_int64), ("local_experts", c_int64), ("target_rows_limit", c_int64),
    ]


class GroupedGemmArgs(ctypes.Structure):
    """Mirror of ``hmc_grouped_gemm_args``."""

    _fields_ = [
        ("mode", c_int32),
        ("a_major", c_int32),
        ("b_major", c_int32),
        ("epilogue", c_int32),
        ("groups", c_int32),
        ("max_ctas", c_int32),
        ("tile_mode", c_int32),
        ("swiglu_clamp", c_int32),
        ("rows", c_int64),
        ("m", c_int64),
        ("n", c_int64),
        ("k", c_int64),
        ("a", c_void_p),
        ("b", c_void_p),
        ("c", c_void_p),
        ("aux", c_void_p),
        ("group_ends", c_void_p),
        ("ready_counters", c_void_p),
        ("ready_budget_ns", c_uint64),
        ("status", c_void_p),
        ("swiglu_limit", c_float),
        ("reserved", c_int32),
        ("row_probs", c_void_p),
        ("row_dot", c_void_p),
        ("combine", c_void_p),
        ("pipe_budget_ns", c_uint64),
        ("dispatch", c_void_p),
        ("skip_flag", c_void_p),
    ]


class GateRouteArgs(ctypes.Structure):
    """Mirror of ``hmc_gate_route_args``."""

    _fields_ = [
        ("logits", c_void_p), ("text_bias", c_void_p), ("vision_bias", c_void_p), ("image_mask", c_void_p),
        ("use_vision_bias", c_int32), ("experts", c_int32), ("top_k", c_int32), ("scoring", c_int32),
        ("tokens", c_int64), ("scale", c_float),
        ("weights", c_void_p), ("indices", c_void_p), ("route_scores", c_void_p), ("selected", c_void_p),
        ("denominator", c_void_p), ("n_group", c_int32), ("topk_group", c_int32),
    ]


class GateRouteGradArgs(ctypes.Structure):
    """Mirror of ``hmc_gate_route_grad_args``."""

    _fields_ = [
        ("logits", c_void_p), ("route_scores", c_void_p), ("selected", c_void_p), ("denominator", c_void_p),
        ("indices", c_void_p), ("grad_weights", c_void_p),
        ("experts", c_int32), ("top_k", c_int32), ("scoring", c_int32), ("reserved", c_int32),
        ("tokens", c_int64), ("scale", c_float),
        ("grad_logits", c_void_p), ("status", c_void_p),
    ]


class MegaMhcArgs(ctypes.Structure):
    """Mirror of ``hmc_mega_mhc_args``."""

    _fields_ = [
        ("tokens", c_int64), ("hidden", c_int64),
        ("previous_output", c_void_p), ("residual", c_void_p), ("previous_pre_mix", c_void_p),
        ("previous_post_mix", c_void_p), ("previous_residual_mix", c_void_p), ("phi", c_void_p),
        ("alpha", c_void_p), ("bias", c_void_p), ("norm_weight", c_void_p),
        ("new_residual", c_void_p), ("next_pre_mix", c_void_p), ("next_post_mix", c_void_p),
        ("next_residual_mix", c_void_p), ("block_input", c_void_p),
        ("hc_before_norm", c_void_p), ("inv_rms", c_void_p), ("sum_out", c_void_p), ("norm_out", c_void_p),
        ("mixed_input", c_void_p), ("rms_rstd", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("hc_eps", c_float), ("norm_eps", c_float), ("num_iters", c_int32), ("need_backward", c_int32),
        ("status", c_void_p),
    ]


class MegaMhcGradArgs(ctypes.Structure):
    """Mirror of ``hmc_mega_mhc_grad_args``."""

    _fields_ = [
        ("tokens", c_int64), ("hidden", c_int64),
        ("grad_new_residual", c_void_p), ("grad_next_pre_mix", c_void_p), ("grad_next_post_mix", c_void_p),
        ("grad_next_residual_mix", c_void_p), ("grad_block_input", c_void_p),
        ("new_residual", c_void_p), ("hc_before_norm", c_void_p), ("inv_rms", c_void_p),
        ("mixed_input", c_void_p), ("rms_rstd", c_void_p),
        ("previous_output", c_void_p), ("residual", c_void_p), ("previous_pre_mix", c_void_p),
        ("previous_post_mix", c_void_p), ("previous_residual_mix", c_void_p), ("phi", c_void_p),
        ("alpha", c_void_p), ("bias", c_void_p), ("norm_weight", c_void_p),
        ("grad_residual", c_void_p), ("grad_phi", c_void_p), ("grad_alpha", c_void_p), ("grad_bias", c_void_p),
        ("grad_previous_output", c_void_p), ("grad_previous_pre_mix", c_void_p),
        ("grad_previous_post_mix", c_void_p), ("grad_previous_residual_mix", c_void_p),
        ("grad_norm_weight", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("hc_eps", c_float), ("num_iters", c_int32),
        ("status", c_void_p),
    ]


class EpDispatchArgs(ctypes.Structure):
    """Mirror of ``hmc_ep_dispatch_args``."""

    _fields_ = [
        ("tokens", c_void_p), ("source_of_row", c_void_p), ("expert_of_row", c_void_p),
        ("dispatch_src_off", c_void_p), ("dispatch_target_off", c_void_p),
        ("rows", c_int64), ("top_k", c_int64), ("hidden", c_int64), ("ep", c_int64), ("local_experts", c_int64),
        ("capacity_rows", c_int64),
        ("peer_buffers", c_void_p), ("peer_ctrl", c_void_p), ("local_ctrl", c_void_p),
        ("generation", c_int32), ("max_ctas", c_int32), ("budget_ns", c_uint64), ("status", c_void_p),
        ("row_values", c_void_p), ("value_index", c_void_p), ("value_plane_offset", c_int64),
        ("rank", c_int64), ("send_order_start", c_void_p), ("skip_flag", c_void_p),
    ]


class EpCombineArgs(ctypes.Structure):
    """Mirror of ``hmc_ep_combine_args``."""

    _fields_ = [
        ("results", c_void_p), ("segment_start", c_void_p), ("combine_target_off", c_void_p),
        ("rows", c_int64), ("hidden", c_int64), ("ep", c_int64), ("local_experts", c_int64),
        ("target_rows_limit", c_int64),
        ("peer_buffers", c_void_p), ("peer_ctrl", c_void_p), ("local_ctrl", c_void_p),
        ("generation", c_int32), ("max_ctas", c_int32), ("budget_ns", c_uint64), ("status", c_void_p),
        ("result_values", c_void_p), ("value_plane_offset", c_int64),
    ]


class EpExchangeArgs(ctypes.Structure):
    """Mirror of ``hmc_ep_exchange_args``."""

    _fields_ = [
        ("counts", c_void_p), ("header", c_int32 * 4), ("peer_tables", c_void_p), ("peer_ctrl", c_void_p),
        ("local_ctrl", c_void_p), ("ep", c_int64), ("rank", c_int64), ("experts", c_int64),
        ("exchange", c_int32), ("reserved", c_int32), ("budget_ns", c_uint64), ("status", c_void_p),
    ]


class EpPullArgs(ctypes.Structure):
    """Mirror of ``hmc_ep_pull_args``."""

    _fields_ = [
        ("peer_sources", c_void_p), ("source_row_off", c_void_p), ("segment_start", c_void_p),
        ("out", c_void_p), ("out_values", c_void_p),
        ("rows", c_int64), ("hidden", c_int64), ("ep", c_int64), ("local_experts", c_int64),
        ("source_rows_limit", c_int64), ("value_plane_offset", c_int64),
        ("local_ctrl", c_void_p), ("generation", c_int32), ("max_ctas", c_int32), ("budget_ns", c_uint64),
        ("status", c_void_p),
    ]


class MxGemmArgs(ctypes.Structure):
    """Mirror of ``hmc_mx_gemm_args``."""

    _fields_ = [
        ("mode", c_int32), ("b_major", c_int32), ("epilogue", c_int32), ("groups", c_int32),
        ("max_ctas", c_int32), ("tile_mode", c_int32),
        ("rows", c_int64), ("pad_blocks", c_int64), ("m", c_int64), ("n", c_int64), ("k", c_int64),
        ("a", c_void_p), ("a_scale", c_void_p), ("b", c_void_p), ("b_scale", c_void_p), ("c", c_void_p),
        ("group_ends", c_void_p), ("status", c_void_p), ("combine", c_void_p),
        ("act_row_data", c_void_p), ("act_row_scale", c_void_p), ("act_col_data", c_void_p), ("act_col_scale", c_void_p),
        ("aux", c_void_p), ("skip_flag", c_void_p),
    ]


class MxQuantArgs(ctypes.Structure):
    """Mirror of ``hmc_mx_quant_args``."""

    _fields_ = [
        ("kind", c_int32), ("groups", c_int32),
        ("rows", c_int64), ("pad_blocks", c_int64), ("width", c_int64),
        ("src", c_void_p), ("aux", c_void_p), ("group_ends", c_void_p),
        ("row_data", c_void_p), ("row_scale", c_void_p), ("col_data", c_void_p), ("col_scale", c_void_p),
        ("dense", c_void_p), ("skip_flag", c_void_p),
    ]


class MoeTransport(ctypes.Structure):
    """Mirror of ``hmc_moe_transport``."""

    _fields_ = [
        ("ep", c_int64), ("rank", c_int64), ("peer_dispatch", c_void_p), ("peer_combine", c_void_p),
        ("peer_ctrl", c_void_p), ("dispatch_rows_limit", c_int64), ("combine_rows_limit", c_int64),
        ("dispatch_plane_offset", c_int64), ("combine_plane_offset", c_int64), ("generation", c_int32),
        ("dispatch_mode", c_int32), ("wait_budget_ns", c_uint64), ("copy_stream", c_void_p),
    ]


class MegaMoeArgs(ctypes.Structure):
    """Mirror of ``hmc_mega_moe_args``."""

    _fields_ = [
        ("dispatch_target", c_void_p), ("dispatch_target_off", c_void_p), ("dispatch_src", c_void_p),
        ("dispatch_src_off", c_void_p), ("dispatch_size", c_void_p), ("up_proj_weight", c_void_p),
        ("up_proj_glist", c_void_p), ("up_proj_y", c_void_p), ("swiglu_out", c_void_p),
        ("down_proj_weight", c_void_p), ("down_proj_glist", c_void_p), ("down_proj_y", c_void_p),
        ("combine_target", c_void_p), ("combine_target_off", c_void_p), ("combine_src_off", c_void_p),
        ("combine_size", c_void_p), ("all_event_counters", c_void_p), ("diagnostic_buffer", c_void_p),
        ("rank_id", c_int64), ("ep", c_int64), ("expert_num", c_int64), ("hidden_size", c_int64),
        ("seq_size", c_int64), ("intermediate_size", c_int64), ("top_k", c_int64), ("routed_rows", c_int64),
        ("received_rows", c_int64), ("weight_layout", c_int32), ("swiglu_clamp", c_int32),
        ("swiglu_limit", c_float), ("fuse_dispatch", c_int32), ("probs_before_fc2", c_int32), ("reserved", c_int32),
        ("dispatch_src_index", c_void_p),
        ("expert_of_row", c_void_p), ("recv_segment_start", c_void_p), ("send_order_start", c_void_p), ("route_probs", c_void_p),
        ("row_probs", c_void_p), ("transport", c_void_p), ("saved_dispatch", c_void_p),
        ("saved_combine", c_void_p), ("saved_row_probs", c_void_p), ("mapping", c_void_p),
        ("topk_probs", c_void_p), ("output", c_void_p), ("skip_flag", c_void_p),
    ]


class MegaMoeGradArgs(ctypes.Structure):
    """Mirror of ``hmc_mega_moe_grad_args``."""

    _fields_ = [
        ("dispatch_target", c_void_p), ("dispatch_target_off", c_void_p), ("dy", c_void_p),
        ("dispatch_src_off", c_void_p), ("dispatch_size", c_void_p), ("hidden", c_void_p), ("hidden_dw", c_void_p),
        ("w2", c_void_p), ("act_grad_y", c_void_p), ("gate", c_void_p), ("grad_gate", c_void_p), ("w1", c_void_p),
        ("gate_dx", c_void_p), ("grad_x", c_void_p), ("combine_target_off", c_void_p),
        ("combine_src_off", c_void_p), ("combine_size", c_void_p), ("permute_out", c_void_p),
        ("gate_dw", c_void_p), ("group_list", c_void_p), ("all_event_counters", c_void_p),
        ("diagnostic_buffer", c_void_p), ("rank_id", c_int64), ("ep", c_int64), ("expert_num", c_int64),
        ("hidden_size", c_int64), ("seq_size", c_int64), ("intermediate_size", c_int64), ("top_k", c_int64),
        ("routed_rows", c_int64), ("received_rows", c_int64), ("weight_layout", c_int32),
        ("swiglu_clamp", c_int32), ("swiglu_limit", c_float), ("fuse_dispatch", c_int32),
        ("weight_grad_f32", c_int32), ("probs_before_fc2", c_int32), ("dispatch_src_index", c_void_p),
        ("expert_of_row", c_void_p), ("recv_segment_start", c_void_p), ("send_order_start", c_void_p), ("row_probs", c_void_p),
        ("row_dot", c_void_p), ("transport", c_void_p), ("grad_output", c_void_p), ("saved_combine", c_void_p),
        ("mapping", c_void_p), ("topk_probs", c_void_p), ("grad_probs", c_void_p), ("grad_hidden", c_void_p),
    ]


class MegaMoeMxfp8Args(ctypes.Structure):
    """Mirror of ``hmc_mega_moe_mxfp8_args``."""

    _fields_ = [
        ("dispatch_buffer", c_void_p), ("dispatch_target_off", c_void_p), ("source_buffer", c_void_p),
        ("dispatch_src_off", c_void_p), ("dispatch_size", c_void_p), ("w1_col_data", c_void_p),
        ("group_list", c_void_p), ("up", c_void_p), ("a_row", c_void_p), ("w2_col_data", c_void_p),
        ("group_list2", c_void_p), ("down", c_void_p), ("routed_buffer", c_void_p),
        ("combine_target_off", c_void_p), ("combine_src_off", c_void_p), ("combine_size", c_void_p),
        ("x_row", c_void_p), ("x_scale", c_void_p), ("x_col", c_void_p), ("x_col_scale", c_void_p),
        ("a_scale", c_void_p), ("a_col", c_void_p), ("a_col_scale", c_void_p), ("w1_col_scale", c_void_p),
        ("w2_col_scale", c_void_p), ("all_event_counters", c_void_p), ("diagnostic_buffer", c_void_p),
        ("rank_id", c_int64), ("ep", c_int64), ("expert_num", c_int64), ("hidden_size", c_int64),
        ("seq_size", c_int64), ("intermediate_size", c_int64), ("top_k", c_int64), ("routed_rows", c_int64),
        ("received_rows", c_int64), ("pad_blocks", c_int64), ("dispatch_src_index", c_void_p),
        ("expert_of_row", c_void_p), ("recv_segment_start", c_void_p), ("transport", c_void_p),
        ("saved_combine", c_void_p), ("mapping", c_void_p), ("topk_probs", c_void_p), ("output", c_void_p),
        ("skip_flag", c_void_p),
    ]


class MegaMoeMxfp8GradArgs(ctypes.Structure):
    """Mirror of ``hmc_mega_moe_mxfp8_grad_args``."""

    _fields_ = [
        ("dispatch", c_void_p), ("dispatch_target_off", c_void_p), ("source", c_void_p),
        ("dispatch_src_off", c_void_p), ("dispatch_size", c_void_p), ("a_col", c_void_p), ("dw2", c_void_p),
        ("w2_row_data", c_void_p), ("da", c_void_p), ("up", c_void_p), ("du_row", c_void_p),
        ("w1_row_data", c_void_p), ("dx", c_void_p), ("routed_buffer", c_void_p), ("combine_target_off", c_void_p),
        ("combine_src_off", c_void_p), ("combine_size", c_void_p), ("x_col", c_void_p), ("dw1", c_void_p),
        ("group_list", c_void_p), ("dy_row", c_void_p), ("dy_scale", c_void_p), ("dy_col", c_void_p),
        ("dy_col_scale", c_void_p), ("a_col_scale", c_void_p), ("w2_row_scale", c_void_p), ("du_scale", c_void_p),
        ("du_col", c_void_p), ("du_col_scale", c_void_p), ("w1_row_scale", c_void_p), ("x_col_scale", c_void_p),
        ("all_event_counters", c_void_p), ("diagnostic_buffer", c_void_p), ("rank_id", c_int64), ("ep", c_int64),
        ("expert_num", c_int64), ("hidden_size", c_int64), ("seq_size", c_int64), ("intermediate_size", c_int64),
        ("top_k", c_int64), ("routed_rows", c_int64), ("received_rows", c_int64), ("pad_blocks", c_int64),
        ("weight_grad_f32", c_int32), ("reserved", c_int32), ("recv_segment_start", c_void_p),
        ("expert_of_row", c_void_p), ("transport", c_void_p), ("grad_output", c_void_p),
        ("saved_combine", c_void_p), ("mapping", c_void_p), ("topk_probs", c_void_p), ("grad_probs", c_void_p),
        ("grad_hidden", c_void_p), ("skip_flag", c_void_p),
    ]

HMC_MAX_EP = 16
HMC_CTRL_ARRIVAL = 0
HMC_CTRL_COMBINE = 1024
HMC_CTRL_READY = 1040
HMC_CTRL_READY_STRIDE = 16
HMC_CTRL_WORDS = 2048
HMC_SCORE = {"sqrtsoftplus": 0, "softmax": 1, "sigmoid": 2}

_LIB: ctypes.CDLL | None = None

# name -> (restype, argtypes); every symbol include/hmc_b200.h declares.
_P = c_void_p
_I = c_int32
_L = c_int64
_F = c_float
_D = c_double
SIGNATURES: dict[str, tuple] = {
    "hmc_last_error": (c_char_p, []),
    "hmc_abi_version": (_I, []),
    "hmc_mega_moe_transport_version": (_I, []),
    "hmc_worker_queue_layout_version": (_I, []),
    "hmc_launch_count": (_L, []),
    "hmc_profile_enable": (_I, [_I]),
    "hmc_profile_enable_kinds": (_I, [ctypes.c_uint32]),
    "hmc_profile_collect": (_I, [ctypes.POINTER(c_double), ctypes.POINTER(c_int64), _I]),
    "hmc_profile_dump": (_I, [ctypes.POINTER(c_int32), ctypes.POINTER(c_double), ctypes.POINTER(c_double), _I]),
    "hmc_grouped_gemm": (_I, [ctypes.POINTER(GroupedGemmArgs), _P]),
    "hmc_grouped_gemm_combine_units": (_L, [_L]),
    "hmc_mx_gemm": (_I, [ctypes.POINTER(MxGemmArgs), _P]),
    "hmc_mx_gemm_combine_units": (_L, [_L]),
    "hmc_mx_quant": (_I, [ctypes.POINTER(MxQuantArgs), _P]),
    "hmc_mx_quant_weight": (_I, [_P, _L, _L, _L, _P, _P, _P, _P, _P]),
    "hmc_mx_pack_weight_scale": (_I, [_P, _I, _L, _L, _L, _P, _P]),
    "hmc_gate_project_promoted_workspace_bytes": (_L, [_L, _L]),
    "hmc_gate_project_promoted": (_I, [_P, _P, _I, _L, _L, _L, _P, _P, _L, _P, _P]),
    "hmc_gate_route": (_I, [ctypes.POINTER(GateRouteArgs), _P]),
    "hmc_gate_project_route_supported": (_I, [_L, _I]),
    "hmc_gate_project_route": (_I, [_P, _P, _I, _L, _P, _P, _L, ctypes.POINTER(GateRouteArgs), _P, _P]),
    "hmc_gate_route_grad": (_I, [ctypes.POINTER(GateRouteGradArgs), _P]),
    "hmc_gate_project": (_I, [_P, _I, _P, _I, _L, _L, _L, _P, _P]),
    "hmc_gate_project_workspace_bytes": (_L, [_L, _L, _L]),
    "hmc_gate_project_tc": (_I, [_P, _P, _I, _L, _L, _L, _P, _P, _L, _P]),
    "hmc_moe_sort_workspace_bytes": (_L, [_L, _L]),
    "hmc_moe_histogram": (_I, [_P, _I, _L, _L, _P, _P, _P]),
    "hmc_moe_sort_routes": (_I, [_P, _I, _L, _L, _P, _L, _P, _P, _P, _P, _P, _P, _P]),
    "hmc_moe_sort_routes_static": (_I, [_P, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P]),
    "hmc_moe_gather_rows": (_I, [_P, _P, _L, _L, _L, _P, _P]),
    "hmc_moe_permute_from_mapping": (_I, [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P]),
    "hmc_moe_unpermute": (_I, [_P, _P, _P, _L, _L, _L, _L, _P, _P, _P]),
    "hmc_moe_unpermute_grad": (_I, [_P, _P, _P, _P, _L, _L, _L, _P, _P, _P, _P]),
    "hmc_moe_token_permute_grad": (_I, [_P, _P, _L, _L, _L, _P, _P, _P]),
    "hmc_zero_empty_expert_grad": (_I, [_P, _L, _P, _L, _P, _L, _P]),
    "hmc_route_offsets": (_I, [_P, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "hmc_symm_alloc": (_I, [_L, ctypes.POINTER(c_void_p)]),
    "hmc_symm_free": (_I, [_P]),
    "hmc_ipc_get_handle": (_I, [_P, _P]),
    "hmc_ipc_open_handle": (_I, [_P, ctypes.POINTER(c_void_p)]),
    "hmc_ipc_close_handle": (_I, [_P]),
    "hmc_ep_publish_ready": (_I, [_P, _L, _L, _I, _P]),
    "hmc_store_words": (_I, [_P, _P, _L, _P]),
    "hmc_store_words_pair": (_I, [_P, _P, _L, _P, _L, _P]),
    "hmc_ep_publish_source": (_I, [_P, _L, _L, _I, _P]),
    "hmc_ep_exchange_table_bytes": (_L, [_L, _L]),
    "hmc_ep_exchange_counts": (_I, [ctypes.POINTER(EpExchangeArgs), _P]),
    "hmc_ep_pull": (_I, [ctypes.POINTER(EpPullArgs), _P]),
    "hmc_ep_dispatch": (_I, [ctypes.POINTER(EpDispatchArgs), _P]),
    "hmc_ep_combine": (_I, [ctypes.POINTER(EpCombineArgs), _P]),
    "hmc_ep_wait": (_I, [_P, _I, c_uint64, _P, _P]),
    "hmc_ep_wait_unless": (_I, [_P, _I, c_uint64, _P, _P, _P]),
    "hmc_route_guard": (_I, [_P, _L, _L, _L, _L, _P, _P, _P, _P]),
    "hmc_ep_wait_groups_unless": (_I, [_P, _P, _L, ctypes.c_uint64, _P, _P, _P]),
    "hmc_ep_wait_groups": (_I, [_P, _P, _L, c_uint64, _P, _P]),
    "hmc_mega_mhc_workspace_bytes": (_L, [_L, _L]),
    "hmc_mega_mhc_grad_workspace_bytes": (_L, [_L, _L]),
    "hmc_mega_mhc": (_I, [ctypes.POINTER(MegaMhcArgs), _P]),
    "hmc_mega_mhc_grad": (_I, [ctypes.POINTER(MegaMhcGradArgs), _P]),
    "hmc_mega_moe": (_I, [ctypes.POINTER(MegaMoeArgs), _P]),
    "hmc_mega_moe_grad": (_I, [ctypes.POINTER(MegaMoeGradArgs), _P]),
    "hmc_mega_moe_mxfp8": (_I, [ctypes.POINTER(MegaMoeMxfp8Args), _P]),
    "hmc_mega_moe_mxfp8_grad": (_I, [ctypes.POINTER(MegaMoeMxfp8GradArgs), _P]),
    "hmc_mega_moe_mxfp8_abi_version": (_I, []),
}


def load() -> ctypes.CDLL:
    """Load the native library once; raise if it is missing (no fallback exists)."""
    global _LIB  # pylint: disable=global-statement
    if _LIB is not None:
        return _LIB
    if not LIBRARY_PATH.exists():
        raise HmcError(
            f"{LIBRARY_PATH} is missing: build it with `python -m hyper_multicore_b200.csrc.build` "
            "(this package has no CPU or PyTorch fallback path)."
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib


def check(code: int) -> None:
    """Turn a negative return code into HmcError carrying the library's message."""
    if code != 0:
        message = load().hmc_last_error().decode("utf-8", "replace")
        raise HmcError(f"hmc error {code}: {message}")


def ptr(tensor: torch.Tensor | None) -> int | None:
    """Device address of a tensor, or NULL."""
    return None if tensor is None else tensor.data_ptr()


def stream_ptr(device: torch.device | None = None) -> int:
    """cudaStream_t of torch's current stream on ``device``."""
    return torch.cuda.current_stream(device).cuda_stream


def new_status(device: torch.device) -> torch.Tensor:
    """Zeroed device status words for kernels with bounded waits."""
    return torch.zeros(HMC_STATUS_WORDS, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor, what: str) -> None:
    """Synchronising check of device status words (used by tests and debug paths)."""
    words = status.tolist()
    if words[0] != 0:
        raise HmcError(f"{what}: device status {words[0]} ({STATUS_NAMES.get(words[0], '?')}), detail {words[1:4]}")


def launch_count() -> int:
    """Kernels this library has launched in this process (counted where they are launched, in C)."""
    return int(load().hmc_launch_count())


class profile:  # pylint: disable=invalid-name
    """Context manager: device time and call counts per kind of entry point while it is active.

    ``with profile() as p: ...`` then ``p.ms["grouped_gemm"]``, ``p.calls["grouped_gemm"]`` (synchronises at exit).
    """

    def __enter__(self):
        self.ms, self.calls = {}, {}
        check(load().hmc_profile_enable(1))
        return self

    def __exit__(self, *exc):
        lib = load()
        lib.hmc_profile_enable(0)
        kinds = len(HMC_PROFILE_KINDS)
        ms = (c_double * kinds)()
        calls = (c_int64 * kinds)()
        check(lib.hmc_profile_collect(ms, calls, kinds))
        self.ms = dict(zip(HMC_PROFILE_KINDS, ms))
        self.calls = dict(zip(HMC_PROFILE_KINDS, calls))
        return False
