"""Minimal stand-in of the serving engine's native ``DeepGemmMegaMoEExperts`` layer, for tests and examples on machines
whose vLLM does not ship that layer.

It implements only the surface the plugin subclass relies on (constructor keywords, the parameter set and its kernel
layout, ``_load_weight`` / ``weight_loader`` for ``w1`` / ``w3`` / ``w2`` checkpoint shards, ``_map_global_expert_id``,
``get_symm_buffer``, ``get_block_m``, ``forward``, ``set_eplb_state``), written from how the reference plugin and its
tests use that layer (``vllm_sm107_megamoe/experts.py:99-295``, ``tests/eplb_harness.py:102-185``,
``patches/vllm-megamoe-plugin.patch``).  Parameters are kept in the kernel layout: W13 rows and scales gate/up
interleaved by 8, scales as UE8M0 bytes per 32 K elements; the packed int32 scale words the kernels take are derived
from them after loading.  With a vLLM that has the real layer, ``register()`` builds the subclass on the real base.
"""

from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any, Dict, List, Optional

import torch
from torch import nn

MEGA_MOE_MXFP4 = "mxfp4"


@dataclass(frozen=True)
class MegaMoEActivation:
    name: str = "swiglu"
    clamp: Optional[float] = 10.0
    alpha: float = 1.0
    beta: float = 0.0


_EP_GROUP: Any = SimpleNamespace(world_size=1, rank_in_group=0, device_group=None, cpu_group=None)


def set_ep_group(group: Any) -> None:
    """Install the expert-parallel group object (``world_size``, ``rank_in_group``, ``device_group``, ``cpu_group``)."""
    global _EP_GROUP
    _EP_GROUP = group


def get_ep_group() -> Any:
    return _EP_GROUP


def interleave_rows(t: torch.Tensor, gran: int = 8) -> torch.Tensor:
    """``[gate | up]`` rows (dim 0) -> ``[g0..7, u0..7, g8..15, ...]``."""
    half = t.shape[0] // 2
    gate = t[:half].reshape(half // gran, gran, *t.shape[1:])
    up = t[half:].reshape(half // gran, gran, *t.shape[1:])
    return torch.stack([gate, up], dim=1).reshape(t.shape)


class DeepGemmMegaMoEExperts(nn.Module):
    """Routed experts (and optionally one shared expert) as one MegaMoE call."""

    def __init__(self, vllm_config: Any, *, prefix: str, num_experts: int, num_local_experts: int,
                 experts_start_idx: int, top_k: int, hidden_size: int, intermediate_size: int,
                 weight_format: str = MEGA_MOE_MXFP4, activation: MegaMoEActivation = MegaMoEActivation(),
                 num_logical_experts: Optional[int] = None, shared_experts: Any = None, device: Any = "cpu"):
        super().__init__()
        self.prefix = prefix
        self.num_experts = num_experts
        self.num_logical_experts = num_logical_experts if num_logical_experts is not None else num_experts
        self.num_local_experts = num_local_experts
        self.experts_start_idx = experts_start_idx
        self.experts_end_idx = experts_start_idx + num_local_experts
        self.top_k = top_k
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.weight_format = weight_format
        self.activation = activation
        self.fast_math = True
        self.max_num_tokens = vllm_config.scheduler_config.max_num_batched_tokens
        self.num_shared_experts = 1 if shared_experts is not None else 0
        self._shared_source = shared_experts
        self._kernel_kwargs: Dict[str, Any] = dict(activation_clamp=activation.clamp, activation_alpha=activation.alpha,
                                                   activation_beta=activation.beta)
        self.eplb_state = SimpleNamespace(logical_to_physical_map=None, expert_load_view=None)
        self._device = torch.device(device)
        self._kernel_weights = None
        self._create_weights()

    # ------------------------------------------------------------------------------------------------ parameters
    def _create_weights(self) -> None:
        e, h, i, dev = self.num_local_experts, self.hidden_size, self.intermediate_size, self._device

        def param(shape, dtype):
            return nn.Parameter(torch.zeros(shape, dtype=dtype, device=dev), requires_grad=False)

        self.w13_weight = param((e, 2 * i, h // 2), torch.uint8)
        self.w13_weight_scale = param((e, 2 * i, h // 32), torch.uint8)
        self.w2_weight = param((e, h, i // 2), torch.uint8)
        self.w2_weight_scale = param((e, h, i // 32), torch.uint8)
        if self.num_shared_experts:
            self.shared_w13_weight = param((2 * i, h), torch.uint8)
            self.shared_w13_weight_scale = param((2 * i, h // 32), torch.uint8)
            self.shared_w2_weight = param((h, i), torch.uint8)
            self.shared_w2_weight_scale = param((h, i // 32), torch.uint8)
            if self._shared_source is not None:
                self.load_shared_expert_weight(self._shared_source)

    def load_shared_expert_weight(self, mlp: Any) -> None:
        gate_up, down = mlp.gate_up_proj, mlp.down_proj
        self.shared_w13_weight.data.copy_(interleave_rows(gate_up.weight.view(torch.uint8)))
        self.shared_w13_weight_scale.data.copy_(interleave_rows(gate_up.weight_scale.view(torch.uint8)))
        self.shared_w2_weight.data.copy_(down.weight.view(torch.uint8))
        self.shared_w2_weight_scale.data.copy_(down.weight_scale.view(torch.uint8))
        self._kernel_weights = None

    def _map_global_expert_id(self, expert_id: int) -> List[int]:
        """Local slots that hold logical expert ``expert_id`` under the initial placement (physical ``p`` holds logical
        ``p % num_logical_experts``)."""
        return [p - self.experts_start_idx for p in range(self.experts_start_idx, self.experts_end_idx)
                if p % self.num_logical_experts == expert_id]

    def _load_weight(self, dst: torch.Tensor, loaded: torch.Tensor, shard_id: str, is_scale: bool) -> None:
        """Write one checkpoint shard into ``dst`` = one expert's ``(N, K')`` slice in kernel layout: ``w1`` is the gate
        half, ``w3`` the up half of the 8-row interleave; ``w2`` is stored as is."""
        src = loaded.view(torch.uint8)
        if shard_id == "w2":
            dst.copy_(src)
            return
        s = 0 if shard_id == "w1" else 1
        view = dst.view(-1, 2, 8, dst.shape[-1])            # (groups, gate/up, 8 rows, K')
        view[:, s].copy_(src.view(-1, 8, src.shape[-1]))

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, weight_name: str, shard_id: str,
                      expert_id: int, return_success: bool = False):
        local_ids = self._map_global_expert_id(expert_id)
        prefix = "w2_" if shard_id == "w2" else "w13_"
        if not local_ids or prefix not in weight_name:
            return False if return_success else None
        for local_id in local_ids:
            self._load_weight(param.data[local_id], loaded_weight, shard_id, weight_name.endswith("scale"))
        self._kernel_weights = None
        return True if return_success else None

    # ------------------------------------------------------------------------------------------------ EPLB
    def set_eplb_state(self, moe_layer_idx: int, expert_load_view: torch.Tensor, logical_to_physical_map: torch.Tensor,
                       logical_replica_count: torch.Tensor) -> None:
        self.eplb_state = SimpleNamespace(expert_load_view=expert_load_view[moe_layer_idx],
                                          logical_to_physical_map=logical_to_physical_map[moe_layer_idx],
                                          logical_replica_count=logical_replica_count[moe_layer_idx])

    def update_expert_map(self) -> None:
        self._kernel_weights = None

    def get_expert_weights(self) -> List[torch.Tensor]:
        return [p.data.view(self.num_local_experts, -1) for n, p in self.named_parameters(recurse=False)
                if not n.startswith("shared_")]

    # ------------------------------------------------------------------------------------------------ forward
    @staticmethod
    def _import_backend():
        raise NotImplementedError("the stand-in base has no backend of its own")

    def get_symm_buffer(self):
        backend = self._import_backend()
        key = (self.num_experts, self.max_num_tokens, self.top_k, self.hidden_size, self.intermediate_size,
               self.num_shared_experts)
        cache = self.__class__.__dict__.get("_buffer_cache")
        if cache is None:
            cache = {}
            setattr(self.__class__, "_buffer_cache", cache)
        if key not in cache:
            group = get_ep_group().device_group
            if group is None:
                from .backend.workspace import SingleRankGroup
                group = SingleRankGroup()
            cache[key] = backend.get_symm_buffer_for_mega_moe(group, self.num_experts, self.max_num_tokens, self.top_k,
                                                              self.hidden_size, self.intermediate_size,
                                                              self.num_shared_experts)
        return cache[key]

    def get_block_m(self, num_tokens: int) -> int:
        backend = self._import_backend()
        return backend.get_block_m_for_mega_moe(get_ep_group().world_size, self.num_experts, self.max_num_tokens,
                                                num_tokens, self.top_k)

    def kernel_weights(self):
        """``(weights, packed scale words)`` pairs over the live parameters.  The packed FP4 / FP8 bytes are the
        parameters themselves (no copy); only the scale bytes are packed into the int32 words the kernels read."""
        if self._kernel_weights is None:
            from .backend.weights import sf_to_required_layout, transpose_sf_for_utccp
            e, h, i = self.num_local_experts, self.hidden_size, self.intermediate_size
            w13, w2 = self.w13_weight.data, self.w2_weight.data
            w13 = w13.view(torch.int8)
            w2 = w2.view(torch.int8)
            s13 = transpose_sf_for_utccp(sf_to_required_layout(self.w13_weight_scale.data, 2 * i, h, e))
            s2 = transpose_sf_for_utccp(sf_to_required_layout(self.w2_weight_scale.data, h, i, e))
            sl1 = sl2 = None
            if self.num_shared_experts:
                sl1 = (self.shared_w13_weight.data.view(torch.float8_e4m3fn),
                       transpose_sf_for_utccp(sf_to_required_layout(self.shared_w13_weight_scale.data, 2 * i, h)))
                sl2 = (self.shared_w2_weight.data.view(torch.float8_e4m3fn),
                       transpose_sf_for_utccp(sf_to_required_layout(self.shared_w2_weight_scale.data, h, i)))
            self._kernel_weights = ((w13, s13), (w2, s2), sl1, sl2)
        return self._kernel_weights

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                is_padding: Optional[torch.Tensor] = None) -> torch.Tensor:
        backend = self._import_backend()
        buf = self.get_symm_buffer()
        m = hidden_states.shape[0]
        block_m = self.get_block_m(m)
        backend.stage_inputs_for_mega_moe(buf, hidden_states, topk_ids, topk_weights, is_padding=is_padding,
                                          block_m=block_m)
        l1, l2, sl1, sl2 = self.kernel_weights()
        y = torch.empty((m, self.hidden_size), dtype=torch.bfloat16, device=hidden_states.device)
        backend.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2,
                                 cumulative_local_expert_recv_stats=self.eplb_state.expert_load_view,
                                 fast_math=self.fast_math, **self._kernel_kwargs)
        return y
