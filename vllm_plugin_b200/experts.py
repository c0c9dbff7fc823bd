"""The ``DeepGemmMegaMoEExperts`` subclass that routes the serving engine's MegaMoE layer to the B200 backend.

Same overrides as the reference's ``SM107MegaMoEExperts`` (``vllm_sm107_megamoe/experts.py:81-298``): the EPLB
communicator gate, the admission call before weights are created, two-slice ("localized") routed weights created once
so that reloads and load-balancer row moves keep every address, logical -> physical slot mapping for reloads after a
rebalance, preparation of every BLOCK_M variant plus a CPU barrier before CUDA-graph capture, and the
``(num_local_experts, -1)`` in-place views the load balancer moves rows through.

The class is built by :func:`make_experts_class` on whatever base is available: the real layer when the installed vLLM
ships it, otherwise the stand-in of ``_standin.py`` (tests).
"""

from __future__ import annotations

from typing import Any, ClassVar, Dict, Optional, Set, Tuple

import torch
from torch import nn

LOCALIZED_WEIGHTS = ("w13_weight", "w2_weight")

SUPPORTED_EPLB_COMMUNICATORS = frozenset({"symm_mem", "torch_gloo", "torch_nccl", "pynccl"})
# NCCL transfers on the asynchronous load-balancer stream would share the GPU with the persistent expert kernels (one
# CTA per SM, all shared memory): keep them synchronous, as the reference does.
_SYNC_ONLY_EPLB_COMMUNICATORS = frozenset({"torch_nccl", "pynccl"})
_UNSUPPORTED_EPLB_COMMUNICATORS = {
    "nixl": "it registers the live expert weights for RDMA reads by peers, which the two-slice weight tensors of this "
            "backend have not been checked with",
    "torch_xccl": "it is the XPU backend",
}


def _check_eplb(parallel_config: Any) -> None:
    """Refuse load-balancer setups this backend cannot serve (same decisions as ``experts.py:49-78`` of the reference)."""
    if getattr(parallel_config, "enable_elastic_ep", False):
        raise NotImplementedError("B200 MegaMoE does not support elastic EP: the workspace and the prepared kernel "
                                  "variants are built for a fixed EP size and physical expert count")
    eplb_config = parallel_config.eplb_config
    communicator = eplb_config.communicator
    if communicator in SUPPORTED_EPLB_COMMUNICATORS:
        if communicator in _SYNC_ONLY_EPLB_COMMUNICATORS and getattr(eplb_config, "use_async", False):
            raise NotImplementedError(
                f"B200 MegaMoE cannot use EPLB communicator {communicator!r} with use_async=true: its NCCL kernels "
                "would run next to the persistent expert kernels. Set --eplb-config.communicator=symm_mem.")
        return
    reason = _UNSUPPORTED_EPLB_COMMUNICATORS.get(communicator, "it has not been checked with two-slice routed weights")
    raise NotImplementedError(f"B200 MegaMoE cannot use EPLB communicator {communicator!r}: {reason}. "
                              "Set --eplb-config.communicator=symm_mem, or torch_gloo.")


def make_experts_class(base: type, get_ep_group=None, mxfp4_format: Any = None) -> type:
    """Build the plugin layer class on ``base`` (the engine's ``DeepGemmMegaMoEExperts`` or the stand-in)."""
    if get_ep_group is None:
        try:
            from vllm.distributed import get_ep_group as _g
            get_ep_group = _g
        except Exception:  # noqa: BLE001
            from ._standin import get_ep_group as _g
            get_ep_group = _g

    class B200MegaMoEExperts(base):  # type: ignore[misc, valid-type]
        """MXFP4 routed experts with one fused MXFP8 shared expert on B200."""

        _prepared_variants: ClassVar[Set[Tuple]] = set()
        _ep_group_getter = staticmethod(get_ep_group)

        def __init__(self, vllm_config: Any, **kwargs: Any):
            parallel_config = vllm_config.parallel_config
            if getattr(parallel_config, "enable_eplb", False):
                _check_eplb(parallel_config)
            if mxfp4_format is not None and kwargs.get("weight_format", mxfp4_format) != mxfp4_format:
                raise NotImplementedError("B200 MegaMoE requires MXFP4 weights")
            if kwargs["activation"].name != "swiglu":
                raise NotImplementedError("B200 MegaMoE requires SwiGLU")
            backend = self._import_backend()
            if not backend.is_localization_available():
                raise NotImplementedError("B200 MegaMoE requires a CUDA device of compute capability 10.0")
            super().__init__(vllm_config, **kwargs)

        @staticmethod
        def _import_backend():
            from . import api as backend

            return backend

        def _create_weights(self) -> None:
            backend = self._import_backend()
            reason = backend.get_unsupported_reason_for_mega_moe(
                self._ep_group_getter().world_size, self.num_experts, self.max_num_tokens, self.top_k, self.hidden_size,
                self.intermediate_size, self.num_shared_experts, fast_math=self.fast_math)
            if reason is not None:
                raise NotImplementedError(f"B200 MegaMoE: {reason}")
            super()._create_weights()
            for name in LOCALIZED_WEIGHTS:
                param = getattr(self, name)
                param.data = backend.localize(param.data)

        def _map_global_expert_id(self, expert_id: int):
            """Local slots of logical expert ``expert_id``: the initial placement before the load balancer is set up,
            its current replica map afterwards (a reload then writes every replica)."""
            mapping = self.eplb_state.logical_to_physical_map
            if mapping is None:
                return super()._map_global_expert_id(expert_id)
            return [p - self.experts_start_idx for p in mapping[expert_id].tolist()
                    if self.experts_start_idx <= p < self.experts_end_idx]

        def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, weight_name: str, shard_id: str,
                          expert_id: int, return_success: bool = False) -> Optional[bool]:
            if param is not self.w13_weight and param is not self.w2_weight:
                return super().weight_loader(param, loaded_weight, weight_name, shard_id, expert_id, return_success)
            local_ids = self._map_global_expert_id(expert_id)
            param_prefix = "w2_" if shard_id == "w2" else "w13_"
            if not local_ids or param_prefix not in weight_name:
                return False if return_success else None
            for local_id in local_ids:
                dst = param.data[:, local_id]               # (2, N/2, K'): the expert's two slices
                logical = dst.flatten(0, 1).clone()         # (N, K') in the base layer's layout
                self._load_weight(logical, loaded_weight, shard_id, False)
                dst.copy_(logical.view_as(dst))             # in place: addresses, graphs and bound launches survive
            if hasattr(self, "_kernel_weights"):
                self._kernel_weights = None
            return True if return_success else None

        def get_symm_buffer(self):
            buffer = getattr(self, "_runtime_buffer", None)
            if buffer is not None:
                return buffer
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm up B200 MegaMoE before CUDA-graph capture")
            buffer = super().get_symm_buffer()
            group = self._ep_group_getter()
            key = (id(getattr(group, "device_group", None)), torch.cuda.current_device() if torch.cuda.is_available() else -1,
                   self.num_experts, buffer.num_max_tokens_per_rank, self.top_k, self.hidden_size,
                   self.intermediate_size, self.num_shared_experts, self.activation, self.fast_math)
            if key not in self._prepared_variants:
                backend = self._import_backend()
                backend.get_balanced_sm_locality_domains()
                backend.precompile_mega_moe_variants(
                    group.world_size, self.num_experts, buffer.num_max_tokens_per_rank, self.top_k, self.hidden_size,
                    self.intermediate_size, self.num_shared_experts, **self._kernel_kwargs, fast_math=self.fast_math,
                    per_die=True, localized_weights=True)
                cpu_group = getattr(group, "cpu_group", None)
                if cpu_group is not None and group.world_size > 1:
                    torch.distributed.barrier(group=cpu_group)   # every rank is ready before any capture starts
                self._prepared_variants.add(key)
            self._runtime_buffer = buffer
            return buffer

        def get_expert_weights(self):
            """Routed parameters as ``(num_local_experts, -1)`` views for the load balancer, which moves an expert by
            copying whole rows in place.  A two-slice weight gives one view per slice; both halves of an expert move
            together because the same row moves are applied to every view."""
            views = []
            for name, param in self.named_parameters(recurse=False):
                if name.startswith("shared_"):
                    continue
                tensor = param.data
                if name in LOCALIZED_WEIGHTS:
                    if tensor.dim() != 4 or tensor.shape[1] != self.num_local_experts:
                        raise AssertionError(f"B200 MegaMoE EPLB {name}: expected two-slice (2, {self.num_local_experts}, "
                                             f"N/2, K/2), got shape={tuple(tensor.shape)}")
                    parts = tensor.unbind(0)
                else:
                    parts = (tensor,)
                for idx, part in enumerate(parts):
                    view = self._eplb_view(name, part)
                    offset = idx * tensor.stride(0) * tensor.element_size() if len(parts) > 1 else 0
                    if view.data_ptr() != tensor.data_ptr() + offset or view.numel() != part.numel() or not view.is_contiguous():
                        raise AssertionError(f"B200 MegaMoE EPLB {name}: the view of part {idx} does not cover its memory in place")
                    views.append(view)
            return views

        def _eplb_view(self, name: str, t: torch.Tensor) -> torch.Tensor:
            e = self.num_local_experts
            if t.shape[0] == e:
                if t.is_contiguous():
                    return t.view(e, -1)
                if t.dim() == 3 and t.stride(1) == 1 and t.stride(2) == t.shape[1]:
                    back = t.transpose(1, 2)        # MN-major scales: shape (E, M, N), memory (E, N, M)
                    if back.is_contiguous():
                        return back.view(e, -1)
            raise AssertionError(f"B200 MegaMoE EPLB {name}: expected contiguous memory with {e} local experts on dim 0, "
                                 f"got shape={tuple(t.shape)} stride={tuple(t.stride())} dtype={t.dtype}")

        def kernel_weights(self):
            """Stand-in base only: the kernels take the two-slice tensors as they are."""
            if getattr(self, "_kernel_weights", None) is None:
                w13, w2 = self.w13_weight.data, self.w2_weight.data
                try:
                    self.w13_weight.data = w13.movedim(0, 1).flatten(1, 2)   # temporary logical view for the base helper
                    self.w2_weight.data = w2.movedim(0, 1).flatten(1, 2)
                    (_, s13), (_, s2), sl1, sl2 = super().kernel_weights()
                finally:
                    self.w13_weight.data, self.w2_weight.data = w13, w2
                self._kernel_weights = ((w13.view(torch.int8), s13), (w2.view(torch.int8), s2), sl1, sl2)
            return self._kernel_weights

    B200MegaMoEExperts.weight_loader.supports_moe_loading = True  # type: ignore[attr-defined]
    B200MegaMoEExperts.__qualname__ = "B200MegaMoEExperts"
    return B200MegaMoEExperts


def standin_experts_class() -> type:
    """The plugin class on the stand-in base (tests, examples without the engine's layer)."""
    from . import _standin

    return make_experts_class(_standin.DeepGemmMegaMoEExperts, _standin.get_ep_group, _standin.MEGA_MOE_MXFP4)
