"""Input staging of the MegaMoE layer: BF16 hidden states -> MXFP8 (E4M3 + packed UE8M0 scales) plus the routing repack,
written straight into the views of the workspace by ONE launch of the CUDA quantiser (``mmoe_stage_inputs``).

Mirrors ``backend/staging.py`` of the reference (``prepare_megamoe_inputs`` :152-196, ``stage_inputs`` :254-283) with the
same argument meaning and the same errors (``ValueError`` for malformed inputs, :221-234).  The reference's fast path is
a Triton kernel and its fallback a torch implementation; here the CUDA kernel is the only path.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _native
from .heuristics import align


def get_shared_sf_rows(num_tokens: int, block_m: int, device=None) -> torch.Tensor:
    """Destination row of every token in the BLOCK_M-dependent shared-expert scale layout."""
    t = torch.arange(num_tokens, dtype=torch.int64, device=device)
    m = t % block_m
    return (t // block_m) * align(block_m, 128) + (m // 128) * 128 + (m % 32) * 4 + (m % 128) // 32


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def stage_inputs(sym_buffer, hidden_states: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, *,
                 is_padding: Optional[torch.Tensor] = None, block_m: Optional[int] = None) -> int:
    """Stage one call's inputs into ``sym_buffer`` and return the BLOCK_M used for the shared-expert scale layout
    (that of THIS call's token count unless given)."""
    num_tokens, hidden_size = hidden_states.shape
    assert num_tokens <= sym_buffer.num_max_tokens_per_rank, "num_tokens must be <= num_max_tokens_per_rank"
    if block_m is None:
        from .frontend import get_block_m_for_mega_moe
        block_m = get_block_m_for_mega_moe(sym_buffer.num_ranks, sym_buffer.num_experts,
                                           sym_buffer.num_max_tokens_per_rank, num_tokens, sym_buffer.num_topk,
                                           sym_buffer.mma_type)
    if num_tokens == 0:
        return block_m
    if hidden_size % 128 != 0 or hidden_size != sym_buffer.hidden:
        raise ValueError("MegaMoE input staging requires hidden_size to be a multiple of 128 and to match the buffer.")
    if topk_weights.shape != topk_ids.shape:
        raise ValueError("MegaMoE input staging requires topk_weights and topk_ids to have the same shape.")
    if topk_ids.shape != (num_tokens, sym_buffer.num_topk):
        raise ValueError("MegaMoE input staging requires topk_ids of shape (num_tokens, num_topk).")
    if block_m <= 0:
        raise ValueError("MegaMoE shared_block_m must be positive.")
    if hidden_states.dtype != torch.bfloat16:
        raise ValueError("MegaMoE input staging requires BF16 hidden states.")
    if not hidden_states.is_cuda:
        raise RuntimeError("MegaMoE input staging runs on the GPU only (there is no CPU path).")
    hidden_states = hidden_states.contiguous()
    ids = topk_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    w = topk_weights.to(torch.float32).contiguous()
    pad_ptr = None
    if is_padding is not None:
        pad = is_padding[:num_tokens].to(torch.uint8).contiguous()
        pad_ptr = pad.data_ptr()
    lib = _native.load()
    _native.check(lib.mmoe_stage_inputs(
        ctypes.byref(sym_buffer.geo), sym_buffer.base_ptr, hidden_states.data_ptr(), ids.data_ptr(),
        1 if ids.dtype == torch.int64 else 0, w.data_ptr(), pad_ptr, num_tokens,
        block_m if sym_buffer.num_shared_experts > 0 else 0, _stream_ptr(hidden_states.device)))
    return block_m


def route_and_stage_inputs(sym_buffer, hidden_states: torch.Tensor, router_logits: torch.Tensor, *,
                           replica_map: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                           is_padding: Optional[torch.Tensor] = None, block_m: Optional[int] = None) -> int:
    """Router + staging in ONE launch: per token the ``num_topk`` largest ``router_logits`` (ties: the lower expert id),
    weights = softmax over the selected logits, optional logical -> physical replica choice, then everything
    :func:`stage_inputs` does.  ``replica_map = (count int32 [L], slots int32 [L, C])``: logical expert ``l`` selected at
    ``(token, slot)`` goes to ``slots[l, (token + slot) % count[l]]``.  Returns the BLOCK_M used."""
    num_tokens, hidden_size = hidden_states.shape
    assert num_tokens <= sym_buffer.num_max_tokens_per_rank, "num_tokens must be <= num_max_tokens_per_rank"
    if block_m is None:
        from .frontend import get_block_m_for_mega_moe
        block_m = get_block_m_for_mega_moe(sym_buffer.num_ranks, sym_buffer.num_experts,
                                           sym_buffer.num_max_tokens_per_rank, num_tokens, sym_buffer.num_topk,
                                           sym_buffer.mma_type)
    if num_tokens == 0:
        return block_m
    if hidden_size != sym_buffer.hidden or hidden_states.dtype != torch.bfloat16 or not hidden_states.is_cuda:
        raise ValueError("MegaMoE input staging requires BF16 CUDA hidden states that match the buffer.")
    if router_logits.dim() != 2 or router_logits.shape[0] != num_tokens or router_logits.dtype != torch.float32:
        raise ValueError("MegaMoE routing requires float32 router_logits of shape (num_tokens, num_logical_experts).")
    hidden_states = hidden_states.contiguous()
    logits = router_logits.contiguous()
    count_ptr = slots_ptr = None
    copies = 0
    if replica_map is not None:
        count, slots = replica_map
        if count.dtype != torch.int32 or slots.dtype != torch.int32 or slots.dim() != 2 or slots.shape[0] != logits.shape[1]:
            raise ValueError("replica_map must be (count int32 [L], slots int32 [L, C]).")
        count, slots = count.contiguous(), slots.contiguous()
        count_ptr, slots_ptr, copies = count.data_ptr(), slots.data_ptr(), slots.shape[1]
    pad_ptr = None
    if is_padding is not None:
        pad = is_padding[:num_tokens].to(torch.uint8).contiguous()
        pad_ptr = pad.data_ptr()
    lib = _native.load()
    _native.check(lib.mmoe_route_stage_inputs(
        ctypes.byref(sym_buffer.geo), sym_buffer.base_ptr, hidden_states.data_ptr(), logits.data_ptr(), logits.shape[1],
        count_ptr, slots_ptr, copies, pad_ptr, num_tokens, block_m if sym_buffer.num_shared_experts > 0 else 0,
        _stream_ptr(hidden_states.device)))
    return block_m


def prepare_megamoe_nvfp4_inputs(hidden_states: torch.Tensor, global_scale: float,
                                 out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """NVFP4 staging of BF16 hidden states (the name the serving engine's hook imports beside the MXFP8 call): returns
    ``(packed E2M1 uint8 [M, H/2], E4M3 scale bytes uint8 [M, H/16])``; ``global_scale`` is the per-tensor FP32 scale of
    the two-level recipe (typically ``448 * 6 / amax`` of a calibration pass)."""
    if hidden_states.dtype != torch.bfloat16 or not hidden_states.is_cuda or hidden_states.dim() != 2:
        raise ValueError("NVFP4 staging requires 2-D BF16 CUDA hidden states.")
    m, h = hidden_states.shape
    if h % 16 != 0:
        raise ValueError("NVFP4 staging requires hidden_size to be a multiple of 16.")
    hidden_states = hidden_states.contiguous()
    if out is None:
        out = (torch.empty((m, h // 2), dtype=torch.uint8, device=hidden_states.device),
               torch.empty((m, h // 16), dtype=torch.uint8, device=hidden_states.device))
    q, sf = out
    assert q.is_contiguous() and sf.is_contiguous() and q.shape == (m, h // 2) and sf.shape == (m, h // 16)
    _native.check(_native.load().mmoe_stage_inputs_nvfp4(hidden_states.data_ptr(), float(global_scale), q.data_ptr(),
                                                         sf.data_ptr(), m, h, _stream_ptr(hidden_states.device)))
    return q, sf


def prepare_megamoe_inputs(hidden_states, topk_weights, topk_ids, sym_buffer, is_padding=None, shared_block_m=None) -> None:
    """Argument order of the serving engine's staging call; the output views are those of ``sym_buffer``."""
    stage_inputs(sym_buffer, hidden_states, topk_ids, topk_weights, is_padding=is_padding, block_m=shared_block_m)
