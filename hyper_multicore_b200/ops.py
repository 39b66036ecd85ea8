"""Operator-level wrappers with the names, argument order and allocation rules of the reference's
``hyper_multicore/torch/ops.py`` (the drop-in boundary of the module layer).

Each function validates like the reference's C++ binding did (contiguity, dtype, device, extents),
allocates exactly the outputs the reference wrapper allocated, and launches through the C ABI.
``runtime_config``, ``all_event_counters`` and ``diagnostic_buffer`` are accepted and ignored:
tiles are scheduled on the device, so there is no serialised host schedule to pass.
"""

from __future__ import annotations

import math

import torch

from . import kernels

_MHC_STREAMS = 4


def _check(condition: bool, message: str) -> None:
    """TORCH_CHECK equivalent: the reference's bindings raise RuntimeError."""
    if not condition:
        raise RuntimeError(message)


def _check_cuda_contiguous(name: str, tensor: torch.Tensor, dtype=None) -> None:
    _check(isinstance(tensor, torch.Tensor), f"{name} must be a Tensor")
    _check(tensor.is_cuda, f"{name} must be a CUDA tensor")
    _check(tensor.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _check(tensor.dtype == dtype, f"{name} must have dtype {dtype}, got {tensor.dtype}")


def mega_moe_transport_version() -> int:
    """reference: torch/csrc/registration.cpp:21."""
    from . import _lib

    return _lib.load().hmc_mega_moe_transport_version()


def worker_queue_layout_version() -> int:
    """reference: torch/csrc/registration.cpp:22."""
    from . import _lib

    return _lib.load().hmc_worker_queue_layout_version()


# --------------------------------------------------------------------------------------- MegaGate
def _mega_gate_route(logits, text_bias, vision_bias, image_mask, runtime_config=None, diagnostic_buffer=None, *,
                     top_k: int, routed_scaling_factor: float, use_vision_bias: bool, scoring_func: str = "sqrtsoftplus",
                     diagnostics=None):
    """reference: torch/ops.py:954-1012, checks torch/csrc/mega_gate.cpp:40-61.

    Returns (weights [T,K] f32, indices [T,K] i64, route_scores [T,E] f32, selected [T,K] f32,
    denominator [T,1] f32). ``scoring_func`` extends the native op to softmax and sigmoid.
    """
    del runtime_config, diagnostic_buffer, diagnostics
    _check_cuda_contiguous("logits", logits, torch.float32)
    _check(logits.ndim == 2 and logits.shape[0] > 0, "logits must be a non-empty [tokens, experts] tensor")
    tokens, experts = logits.shape
    for name, bias in (("text_bias", text_bias), ("vision_bias", vision_bias)):
        _check_cuda_contiguous(name, bias, torch.float32)
        _check(tuple(bias.shape) == (experts,) and bias.device == logits.device, f"{name} must be [experts] on the logits device")
    _check(1 <= top_k <= experts, "top_k must be in [1, expert_count]")
    _check(math.isfinite(routed_scaling_factor), "routed_scaling_factor must be finite")
    _check(not logits.requires_grad, "mega_gate_route does not record autograd; use MegaGate")
    if use_vision_bias:
        _check_cuda_contiguous("image_mask", image_mask, torch.bool)
        _check(image_mask.numel() == tokens, "image_mask must have one entry per token")
    from .modules.mega_gate import route

    return route(logits, text_bias, vision_bias, image_mask if use_vision_bias else None, bool(use_vision_bias),
                 int(top_k), float(routed_scaling_factor), scoring_func)


def _mega_gate_route_grad(logits, route_scores, selected_scores, normalization_denominator, expert_indices,
                          grad_routing_weights, runtime_config=None, diagnostic_buffer=None, *, top_k: int,
                          routed_scaling_factor: float, scoring_func: str = "sqrtsoftplus") -> torch.Tensor:
    """reference: torch/ops.py:1015-1044, checks torch/csrc/mega_gate.cpp:132-176."""
    del runtime_config, diagnostic_buffer
    tokens, experts = logits.shape
    _check_cuda_contiguous("logits", logits, torch.float32)
    _check_cuda_contiguous("route_scores", route_scores, torch.float32)
    _check_cuda_contiguous("selected_scores", selected_scores, torch.float32)
    _check_cuda_contiguous("normalization_denominator", normalization_denominator, torch.float32)
    _check_cuda_contiguous("expert_indices", expert_indices, torch.int64)
    _check_cuda_contiguous("grad_routing_weights", grad_routing_weights, torch.float32)
    _check(tuple(route_scores.shape) == (tokens, experts), "route_scores must match logits")
    _check(tuple(selected_scores.shape) == (tokens, top_k) and tuple(expert_indices.shape) == (tokens, top_k)
           and tuple(grad_routing_weights.shape) == (tokens, top_k), "top-k tensors must be [tokens, top_k]")
    _check(normalization_denominator.numel() == tokens, "normalization_denominator must be [tokens, 1]")
    grad_logits = torch.empty_like(logits)
    kernels.gate_route_grad_out(logits, route_scores, selected_scores, normalization_denominator, expert_indices,
                                grad_routing_weights, int(top_k), float(routed_scaling_factor), scoring_func, grad_logits)
    return grad_logits


# ------------------------------------------------------------------------------ MoE row helpers
def moe_token_permute_out(tokens, indices, output, mapping) -> None:
    """reference: torch/ops.py:493-509, checks torch/csrc/moe_token_permute_out.cpp:25-48.

    ``output[mapping[t * K + k]] = tokens[t]`` with rows expert-major, stable by flat index.
    """
    _check_cuda_contiguous("tokens", tokens)
    _check_cuda_contiguous("indices", indices)
    _check_cuda_contiguous("output", output, tokens.dtype)
    _check_cuda_contiguous("mapping", mapping, torch.int32)
    _check(tokens.ndim == 2 and indices.ndim == 2 and indices.shape[0] == tokens.shape[0], "indices must be [tokens, top_k]")
    _check(indices.dtype in (torch.int32, torch.int64), "indices must be INT32 or INT64")
    rows = indices.numel()
    _check(tuple(output.shape) == (rows, tokens.shape[1]) and mapping.numel() == rows,
           "output must be [tokens * top_k, hidden] and mapping [tokens * top_k]")
    _check(output.data_ptr() != tokens.data_ptr(), "output must not overlap tokens")
    experts = int(indices.max().item()) + 1 if rows else 1
    result, sources, _, _, _ = kernels.moe_sort_routes(indices, experts)
    mapping.copy_(result)
    if rows:
        kernels.moe_gather_rows(tokens, sources, indices.shape[1], output)


def moe_token_permute_from_mapping_out(tokens, mapping, probabilities, output, output_probabilities) -> None:
    """reference: torch/ops.py:512-528 (utilities.asc:162-209): bit-preserving expansion through an existing map."""
    _check_cuda_contiguous("tokens", tokens)
    _check_cuda_contiguous("mapping", mapping, torch.int32)
    _check_cuda_contiguous("probabilities", probabilities, torch.float32)
    _check_cuda_contiguous("output", output, tokens.dtype)
    _check_cuda_contiguous("output_probabilities", output_probabilities, torch.float32)
    top_k = mapping.numel() // max(tokens.shape[0], 1)
    _check(mapping.numel() == tokens.shape[0] * top_k and probabilities.numel() == mapping.numel(),
           "mapping and probabilities must hold tokens * top_k entries")
    _check(output.shape[0] == mapping.numel() and output_probabilities.numel() == mapping.numel(),
           "outputs must have tokens * top_k rows")
    kernels.moe_permute_from_mapping(tokens, mapping, probabilities, top_k, output, output_probabilities)


def mega_moe_unpermute_grad_out(permuted_tokens, grad_output, sorted_indices, probs, grad_permuted, grad_probs) -> None:
    """reference: torch/ops.py:531-551 (torch/csrc/mega_moe_unpermute.cpp:56-65)."""
    for name, tensor in (("permuted_tokens", permuted_tokens), ("grad_output", grad_output), ("grad_permuted", grad_permuted)):
        _check_cuda_contiguous(name, tensor, torch.bfloat16)
    _check_cuda_contiguous("sorted_indices", sorted_indices, torch.int32)
    _check_cuda_contiguous("probs", probs, torch.float32)
    _check_cuda_contiguous("grad_probs", grad_probs, torch.float32)
    top_k = probs.shape[-1]
    _check(sorted_indices.numel() == grad_output.shape[0] * top_k, "sorted_indices must hold tokens * top_k entries")
    kernels.moe_unpermute_grad(permuted_tokens, grad_output, sorted_indices, probs, top_k, grad_permuted, grad_probs)


def moe_token_permute_grad(grad_permuted_tokens, sorted_indices, num_tokens: int, top_k: int) -> torch.Tensor:
    """reference: torch/ops.py:931-951 (torch/csrc/moe_token_permute_grad.cpp:29-38). Returns owned [T, H]."""
    _check_cuda_contiguous("grad_permuted_tokens", grad_permuted_tokens, torch.bfloat16)
    _check_cuda_contiguous("sorted_indices", sorted_indices, torch.int32)
    _check(sorted_indices.numel() == num_tokens * top_k, "sorted_indices must hold num_tokens * top_k entries")
    out = torch.empty((num_tokens, grad_permuted_tokens.shape[1]), dtype=grad_permuted_tokens.dtype,
                      device=grad_permuted_tokens.device)
    kernels.moe_token_permute_grad(grad_permuted_tokens, sorted_indices, num_tokens, top_k, out)
    return out


def zero_empty_expert_gradients(first, second, cumulative_groups) -> None:
    """reference: torch/ops.py:1047-1057 (torch/csrc/mega_moe_utilities.cpp:64-92)."""
    _check_cuda_contiguous("first", first)
    _check_cuda_contiguous("second", second)
    _check_cuda_contiguous("cumulative_groups", cumulative_groups, torch.int64)
    _check(first.shape[0] == cumulative_groups.numel() == second.shape[0], "one gradient slice per local expert")
    kernels.zero_empty_expert_grad(first, second, cumulative_groups)


def route_offsets(counts, rank: int, ub_bytes: int = 0, hidden_size: int = 1) -> dict:
    """reference: torch/ops.py:1060-1064 (utilities.asc:89-151). Returns the named row-unit descriptors
    (the reference packs them into two flat tensors); ``hidden_size`` > 1 adds element-unit copies."""
    del ub_bytes
    _check_cuda_contiguous("counts", counts, torch.int32)
    _check(counts.ndim == 2 and counts.shape[1] % counts.shape[0] == 0, "counts must be [ep, experts]")
    rows = kernels.route_offsets(counts, int(rank))
    if hidden_size != 1:
        for name in ("dispatch_src_off", "dispatch_target_off", "dispatch_size", "combine_src_off",
                     "combine_target_off", "combine_size"):
            rows[name + "_elements"] = rows[name] * hidden_size
    return rows


# ------------------------------------------------------------------------------------------- mHC
def _allocate_hyper_mega_mhc_forward_cache(residual: torch.Tensor, num_iters: int):
    """The six backward intermediates in the reference's order (torch/ops.py:230-268)."""
    batch, sequence, streams, hidden = residual.shape
    mix = streams * streams + 2 * streams
    f32 = dict(dtype=torch.float32, device=residual.device)
    return (torch.empty((batch, sequence, mix), **f32), torch.empty((batch, sequence, 1), **f32),
            torch.empty((2 * num_iters, batch, sequence, streams), **f32),
            torch.empty((2 * num_iters, batch, sequence, streams, streams), **f32),
            torch.empty((batch, sequence, hidden), dtype=residual.dtype, device=residual.device),
            torch.empty((batch, sequence, 1), **f32))


def hyper_mega_mhc(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
                   bias, norm_weight, runtime_config=None, all_event_counters=None, diagnostic_buffer=None, *,
                   hc_eps: float = 1e-6, norm_eps: float = 1e-6, num_iters: int = 20, need_backward: bool,
                   diagnostics=None):
    """reference: torch/ops.py:270-369. BSND inputs; returns the five outputs followed by the six caches."""
    del runtime_config, all_event_counters, diagnostic_buffer, diagnostics
    if residual.ndim != 4:
        raise ValueError(f"residual must be BSND [B, S, 4, H], got {tuple(residual.shape)}.")
    batch, sequence, streams, hidden = residual.shape
    _check(streams == _MHC_STREAMS, "residual must have four streams")
    f32 = dict(dtype=torch.float32, device=residual.device)
    new_residual = torch.empty_like(residual)
    next_pre = torch.empty((batch, sequence, streams), **f32)
    next_post = torch.empty_like(next_pre)
    next_mix = torch.empty((batch, sequence, streams * streams), **f32)
    block_input = torch.empty((batch, sequence, hidden), dtype=residual.dtype, device=residual.device)
    cache = _allocate_hyper_mega_mhc_forward_cache(residual, num_iters)
    inputs = [t.contiguous() for t in (previous_output, residual, previous_pre_mix, previous_post_mix,
                                       previous_residual_mix, phi, alpha, bias, norm_weight)]
    kernels.mega_mhc_out(*inputs, new_residual, next_pre, next_post, next_mix, block_input, *cache, hc_eps=hc_eps,
                         norm_eps=norm_eps, num_iters=num_iters, need_backward=need_backward)
    return (new_residual, next_pre, next_post, next_mix.reshape(batch, sequence, streams, streams), block_input, *cache)


def hyper_mega_mhc_grad(grad_hin_placeholder, grad_h_post, grad_h_res, x, phi, alpha, bias, previous_pre,
                        hc_before_norm, inv_rms, sum_out, norm_out, grad_current_pre, mixed_input, rms_rstd,
                        norm_weight, direct_grad_x, previous_residual, previous_output, previous_post,
                        previous_residual_mix, runtime_config=None, all_event_counters=None, diagnostic_buffer=None, *,
                        hc_eps: float = 1e-6, grad_block_input=None, diagnostics=None):
    """reference: torch/ops.py:397-490, argument order of the native backward ABI.

    ``x`` is the forward new_residual, ``direct_grad_x`` its direct gradient, ``grad_current_pre /
    grad_h_post / grad_h_res`` the gradients of the predicted mappings. The gradient of block_input,
    which the reference folds into ``grad_hin_placeholder``, may also be given as ``grad_block_input``.
    Returns (grad_residual, grad_phi, grad_alpha, grad_bias, grad_previous_output, grad_previous_pre,
    grad_previous_post, grad_previous_residual_mix, grad_norm_weight fp32).
    """
    del runtime_config, all_event_counters, diagnostic_buffer, diagnostics, sum_out, norm_out
    block_grad = grad_block_input if grad_block_input is not None else grad_hin_placeholder
    hidden = previous_residual.shape[-1]
    tokens = previous_residual.numel() // (_MHC_STREAMS * hidden)
    f32 = dict(dtype=torch.float32, device=previous_residual.device)
    result = dict(
        grad_residual=torch.empty_like(previous_residual), grad_phi=torch.empty_like(phi),
        grad_alpha=torch.empty_like(alpha), grad_bias=torch.empty_like(bias),
        grad_previous_output=torch.empty_like(previous_output), grad_previous_pre_mix=torch.empty_like(previous_pre),
        grad_previous_post_mix=torch.empty_like(previous_post),
        grad_previous_residual_mix=torch.empty_like(previous_residual_mix),
        grad_norm_weight=torch.empty(norm_weight.shape, **f32))
    tensors = dict(
        grad_new_residual=direct_grad_x.contiguous(), grad_next_pre_mix=grad_current_pre.contiguous(),
        grad_next_post_mix=grad_h_post.contiguous(), grad_next_residual_mix=grad_h_res.reshape(tokens, 16).contiguous(),
        grad_block_input=block_grad.contiguous(), new_residual=x.contiguous(), hc_before_norm=hc_before_norm,
        inv_rms=inv_rms, mixed_input=mixed_input, rms_rstd=rms_rstd, previous_output=previous_output.contiguous(),
        residual=previous_residual.contiguous(), previous_pre_mix=previous_pre.contiguous(),
        previous_post_mix=previous_post.contiguous(), previous_residual_mix=previous_residual_mix.contiguous(),
        phi=phi, alpha=alpha, bias=bias, norm_weight=norm_weight, **result)
    kernels.mega_mhc_grad_out(tensors, hc_eps=hc_eps, num_iters=20)
    return tuple(result.values())
