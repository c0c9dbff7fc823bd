"""Public operator surface of the B200 MegaMoE expert backend.

Same names, signatures and semantics as the reference's ``vllm_sm107_megamoe/api.py`` (:39-266, which itself follows
DeepGEMM's MegaMoE API), so that a layer written against that module -- the ``DeepGemmMegaMoEExperts`` subclass reaches
it through ``_import_backend()`` -- can switch backend without other changes.  Every function hands off to
``vllm_plugin_b200.backend`` through function-local imports: importing this module imports neither torch nor CUDA.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple, Union


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                                 intermediate_hidden: int, num_shared_experts: int = 0,
                                 use_fp8_dispatch: Union[bool, None] = None, mma_type: str = "fp8xfp4",
                                 activation: str = "swiglu"):
    """Allocate (collectively) the workspace of the layer; returns a ``SymmBuffer``.  ``num_max_tokens_per_rank`` is
    aligned up to 1920; the aligned value is ``SymmBuffer.num_max_tokens_per_rank``."""
    from .backend.frontend import require_sm100
    from .backend.workspace import get_symm_buffer_for_mega_moe as _impl

    require_sm100()
    return _impl(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                 num_shared_experts, use_fp8_dispatch, mma_type, activation)


def transform_weights_for_mega_moe(l1_weights, l2_weights, activation: str = "swiglu"):
    """Rearrange ``(weights, scale factors)`` pairs into the layout the kernels read (pure torch, any device)."""
    from .backend.weights import transform_weights_for_mega_moe as _impl

    return _impl(l1_weights, l2_weights, activation)


def fp8_fp4_mega_moe(y, l1_weights: Tuple[Any, Any], l2_weights: Tuple[Any, Any], sym_buffer,
                     shared_l1_weights: Optional[Tuple[Any, Any]] = None,
                     shared_l2_weights: Optional[Tuple[Any, Any]] = None, cumulative_local_expert_recv_stats=None,
                     recipe: Tuple[int, int, int] = (1, 1, 32), activation: str = "swiglu",
                     activation_clamp: Optional[float] = None, fast_math: bool = True, activation_alpha: float = 1.0,
                     activation_beta: float = 0.0, *, residual=None):
    """Fused MegaMoE for one rank.  The BLOCK_M variant is selected from ``y.size(0)`` of this call.  ``residual``
    (keyword only, an addition to the reference's signature): BF16 ``(M, H)`` added to the output in the combine pass."""
    from .backend.frontend import fp8_fp4_mega_moe as _impl

    return _impl(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights,
                 cumulative_local_expert_recv_stats, recipe, activation, activation_clamp, fast_math, activation_alpha,
                 activation_beta, residual=residual)


def get_block_m_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_tokens: int,
                             num_topk: int, mma_type: str = "fp8xfp4") -> int:
    """BLOCK_M used for ``num_tokens`` tokens on the calling rank (a forced value, ``set_kernel_options(block_m=...)``, wins)."""
    from .backend.frontend import get_block_m_for_mega_moe as _impl

    return _impl(num_ranks, num_experts, num_max_tokens_per_rank, num_tokens, num_topk, mma_type)


def get_token_alignment_for_mega_moe() -> int:
    """Alignment (1920 = lcm of the candidate BLOCK_M) applied to ``num_max_tokens_per_rank``."""
    from .backend.heuristics import get_token_alignment_for_mega_moe as _impl

    return _impl()


def get_unsupported_reason_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                        hidden: int, intermediate_hidden: int, num_shared_experts: int = 0,
                                        mma_type: str = "fp8xfp4", activation: str = "swiglu", *,
                                        fast_math: bool = True, localized_shared_weights: bool = False,
                                        allow_unvalidated: bool = False) -> Optional[str]:
    """``None`` when this backend can serve the geometry, else a short reason.  Total: never raises."""
    from .backend.heuristics import get_mega_moe_unsupported_reason as _impl

    return _impl(num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                 num_shared_experts, mma_type, activation, fast_math=fast_math,
                 localized_shared_weights=localized_shared_weights, allow_unvalidated=allow_unvalidated)


def stage_inputs_for_mega_moe(sym_buffer, hidden_states, topk_ids, topk_weights, *, is_padding=None,
                              block_m: Optional[int] = None) -> int:
    """Quantise and stage one call's inputs into ``sym_buffer`` (one CUDA launch); returns the BLOCK_M used."""
    from .backend.staging import stage_inputs as _impl

    return _impl(sym_buffer, hidden_states, topk_ids, topk_weights, is_padding=is_padding, block_m=block_m)


def route_and_stage_inputs_for_mega_moe(sym_buffer, hidden_states, router_logits, *, replica_map=None, is_padding=None,
                                        block_m: Optional[int] = None) -> int:
    """Router (top-k by logit, softmax over the selected, optional logical -> physical replica choice) fused in front of
    the input staging: one CUDA launch; returns the BLOCK_M used.  Not part of the reference's surface: there the
    serving engine routes before it calls the layer."""
    from .backend.staging import route_and_stage_inputs as _impl

    return _impl(sym_buffer, hidden_states, router_logits, replica_map=replica_map, is_padding=is_padding, block_m=block_m)


def prepare_megamoe_nvfp4_inputs(hidden_states, global_scale: float, out=None):
    """NVFP4 (E2M1 + E4M3 scale per 16 + per-tensor scale) staging of BF16 hidden states; returns ``(packed, scales)``."""
    from .backend.staging import prepare_megamoe_nvfp4_inputs as _impl

    return _impl(hidden_states, global_scale, out)


def precompile_mega_moe_variants(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                 hidden: int, intermediate_hidden: int, num_shared_experts: int = 0, *,
                                 activation_clamp: Optional[float] = None, activation_alpha: float = 1.0,
                                 activation_beta: float = 0.0, fast_math: bool = True, per_die: bool = False,
                                 localized_weights: bool = False, localized_shared_weights: bool = False
                                 ) -> Tuple[int, ...]:
    """Prepare every BLOCK_M variant the geometry can select, before CUDA-graph capture; returns the variants."""
    from .backend.frontend import precompile_mega_moe_variants as _impl

    return _impl(num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                 num_shared_experts, activation_clamp=activation_clamp, activation_alpha=activation_alpha,
                 activation_beta=activation_beta, fast_math=fast_math, per_die=per_die,
                 localized_weights=localized_weights, localized_shared_weights=localized_shared_weights)


def read_status(sym_buffer) -> None:
    """Synchronise and raise if a device-side wait expired (``RuntimeError``) or an expert id was out of range
    (``AssertionError``) in any call on ``sym_buffer`` since the last read; clears the condition."""
    from .backend.frontend import read_status as _impl

    return _impl(sym_buffer)


def set_kernel_options(**kwargs):
    from .backend.frontend import set_kernel_options as _impl

    return _impl(**kwargs)


def get_kernel_options():
    from .backend.frontend import get_kernel_options as _impl

    return _impl()


def is_localization_available() -> bool:
    from .backend.locality import is_localization_available as _impl

    return _impl()


def get_balanced_sm_locality_domains():
    from .backend.locality import get_balanced_sm_locality_domains as _impl

    return _impl()


def localize(t, dim: int = -2):
    from .backend.locality import localize as _impl

    return _impl(t, dim)


def localize_mega_moe_weights(l1_weights, l2_weights):
    """Two-slice form of the routed weight tensors of ``(weights, sf)`` pairs; scale factors are left as they are."""
    from .backend.locality import localize as _impl

    return (_impl(l1_weights[0]), l1_weights[1]), (_impl(l2_weights[0]), l2_weights[1])


def __getattr__(name: str):
    if name == "SymmBuffer":
        from .backend.workspace import SymmBuffer

        return SymmBuffer
    raise AttributeError(name)


__all__ = [
    "get_symm_buffer_for_mega_moe", "transform_weights_for_mega_moe", "fp8_fp4_mega_moe", "get_block_m_for_mega_moe",
    "get_token_alignment_for_mega_moe", "get_unsupported_reason_for_mega_moe", "stage_inputs_for_mega_moe",
    "route_and_stage_inputs_for_mega_moe", "prepare_megamoe_nvfp4_inputs",
    "precompile_mega_moe_variants", "set_kernel_options", "get_kernel_options", "is_localization_available",
    "get_balanced_sm_locality_domains", "localize", "localize_mega_moe_weights", "read_status", "SymmBuffer",
]
