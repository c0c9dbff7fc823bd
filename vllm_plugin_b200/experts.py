"""The serving engine's MegaMoE layer on the B200 backend.

What the engine's hook asks of a plugin layer (``patches/vllm-megamoe-plugin.patch`` of the reference, and the class it
ships, ``vllm_sm107_megamoe/experts.py:81-298``): a subclass of ``DeepGemmMegaMoEExperts`` that names its backend module
(``_import_backend``), answers the admission question before any weight exists, keeps the routed weights in the
two-slice form at addresses that never change (reloads and load-balancer row moves write in place), resolves a logical
expert to its local physical slots after a rebalance, prepares every BLOCK_M variant before CUDA-graph capture, and
hands the load balancer ``(num_local_experts, -1)`` views that alias the parameters.

This module is organised around three small pieces the class composes: a table of load-balancer transports with what
each may be used for, a helper that treats one expert of a two-slice tensor as its logical ``(N, K')`` matrix, and a
ledger of geometries that have been warmed up in this process.  The class itself is produced by
:func:`make_experts_class` on whatever base is available: the engine's layer when the installed engine ships it,
otherwise the stand-in of ``_standin.py`` (tests).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Iterator, List, Optional, Set, Tuple

import torch
from torch import nn

#: routed parameters kept in the two-slice form ``(2, E_l, N/2, K')``
TWO_SLICE_PARAMETERS = ("w13_weight", "w2_weight")


# ---------------------------------------------------------------------------------------------------------------------
# load-balancer transports
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class _Transport:
    usable: bool
    background_moves: bool      # may move rows on the load balancer's own stream while layers run
    objection: str = ""


# The expert kernels are persistent (one CTA per SM holding all shared memory), so a transport whose row moves are NCCL
# kernels must not run beside them: those stay synchronous, as in the reference (``experts.py:29-78``).
_TRANSPORTS: Dict[str, _Transport] = {
    "symm_mem": _Transport(True, True),
    "torch_gloo": _Transport(True, True),
    "torch_nccl": _Transport(True, False, "its NCCL kernels would run next to the persistent expert kernels"),
    "pynccl": _Transport(True, False, "its NCCL kernels would run next to the persistent expert kernels"),
    "nixl": _Transport(False, False, "it registers the live expert weights for RDMA reads by peers, which the two-slice "
                                     "weight tensors of this backend have not been checked with"),
    "torch_xccl": _Transport(False, False, "it is the XPU backend"),
}
_ADVICE = "Set --eplb-config.communicator=symm_mem, or torch_gloo."


def _check_eplb(parallel_config: Any) -> None:
    """Raise ``NotImplementedError`` for a load-balancer setup this backend cannot serve."""
    if getattr(parallel_config, "enable_elastic_ep", False):
        raise NotImplementedError("B200 MegaMoE does not support elastic EP: the workspace and the prepared kernel "
                                  "variants are built for a fixed EP size and physical expert count")
    config = parallel_config.eplb_config
    name = config.communicator
    transport = _TRANSPORTS.get(name, _Transport(False, False, "it has not been checked with two-slice routed weights"))
    if not transport.usable:
        raise NotImplementedError(f"B200 MegaMoE cannot use EPLB communicator {name!r}: {transport.objection}. {_ADVICE}")
    if getattr(config, "use_async", False) and not transport.background_moves:
        raise NotImplementedError(f"B200 MegaMoE cannot use EPLB communicator {name!r} with use_async=true: "
                                  f"{transport.objection}. {_ADVICE}")


# ---------------------------------------------------------------------------------------------------------------------
# one expert of a two-slice tensor as its logical matrix
# ---------------------------------------------------------------------------------------------------------------------
class _ExpertRows:
    """Slot ``slot`` of a ``(2, E_l, N/2, K')`` tensor: slice 0 holds the first half of the expert's rows, slice 1 the
    second.  ``gather`` returns a private ``(N, K')`` copy in the base layer's layout, ``scatter`` writes one back into
    the same storage (addresses, captured graphs and cached launches survive)."""

    def __init__(self, tensor: torch.Tensor, slot: int):
        self.halves = (tensor[0, slot], tensor[1, slot])

    def gather(self) -> torch.Tensor:
        return torch.cat(self.halves, dim=0)

    def scatter(self, rows: torch.Tensor) -> None:
        first, second = rows.split(self.halves[0].shape[0], dim=0)
        self.halves[0].copy_(first)
        self.halves[1].copy_(second)


def _rows_as_matrix(name: str, block: torch.Tensor, num_local: int) -> torch.Tensor:
    """``(num_local, -1)`` view of a per-expert tensor over exactly its own memory: plain contiguous tensors, and the
    MN-major scale tensors whose memory order is ``(expert, column, row)``."""
    if block.shape[0] == num_local:
        if block.is_contiguous():
            return block.view(num_local, -1)
        if block.dim() == 3:
            swapped = block.permute(0, 2, 1)
            if swapped.is_contiguous():
                return swapped.view(num_local, -1)
    raise AssertionError(f"B200 MegaMoE EPLB {name}: expected contiguous memory with {num_local} local experts on dim 0, "
                         f"got shape={tuple(block.shape)} stride={tuple(block.stride())} dtype={block.dtype}")


def _expert_major_blocks(name: str, tensor: torch.Tensor, num_local: int) -> Iterator[Tuple[int, torch.Tensor]]:
    """(byte offset inside the parameter, per-expert block) pairs: one per slice for a two-slice parameter."""
    if name not in TWO_SLICE_PARAMETERS:
        yield 0, tensor
        return
    if tensor.dim() != 4 or tensor.shape[0] != 2 or tensor.shape[1] != num_local:
        raise AssertionError(f"B200 MegaMoE EPLB {name}: expected two-slice (2, {num_local}, N/2, K/2), "
                             f"got shape={tuple(tensor.shape)}")
    for s in range(2):
        yield s * tensor.stride(0) * tensor.element_size(), tensor[s]


# ---------------------------------------------------------------------------------------------------------------------
# the layer class
# ---------------------------------------------------------------------------------------------------------------------
def make_experts_class(base: type, get_ep_group=None, mxfp4_format: Any = None) -> type:
    """Build the plugin layer class on ``base`` (the engine's ``DeepGemmMegaMoEExperts`` or the stand-in)."""
    if get_ep_group is None:
        try:
            from vllm.distributed import get_ep_group as engine_group
            get_ep_group = engine_group
        except Exception:  # noqa: BLE001
            from ._standin import get_ep_group as standin_group
            get_ep_group = standin_group

    class B200MegaMoEExperts(base):  # type: ignore[misc, valid-type]
        """MXFP4 routed experts with one fused MXFP8 shared expert on B200."""

        _warmed_up: ClassVar[Set[Tuple]] = set()        # geometries whose kernel variants are ready in this process
        _ep_group_getter = staticmethod(get_ep_group)

        # -------------------------------------------------------------------------------------------- construction
        def __init__(self, vllm_config: Any, **kwargs: Any):
            self._refuse_unservable(vllm_config.parallel_config, kwargs)
            super().__init__(vllm_config, **kwargs)

        @classmethod
        def _refuse_unservable(cls, parallel_config: Any, kwargs: Dict[str, Any]) -> None:
            if getattr(parallel_config, "enable_eplb", False):
                _check_eplb(parallel_config)
            if mxfp4_format is not None and kwargs.get("weight_format", mxfp4_format) != mxfp4_format:
                raise NotImplementedError("B200 MegaMoE requires MXFP4 weights")
            if kwargs["activation"].name != "swiglu":
                raise NotImplementedError("B200 MegaMoE requires SwiGLU")
            if not cls._import_backend().is_localization_available():
                raise NotImplementedError("B200 MegaMoE requires a CUDA device of compute capability 10.0")

        @staticmethod
        def _import_backend():
            from . import api

            return api

        def _create_weights(self) -> None:
            api = self._import_backend()
            verdict = api.get_unsupported_reason_for_mega_moe(
                self._ep_group_getter().world_size, self.num_experts, self.max_num_tokens, self.top_k, self.hidden_size,
                self.intermediate_size, self.num_shared_experts, fast_math=self.fast_math)
            if verdict is not None:
                raise NotImplementedError(f"B200 MegaMoE: {verdict}")
            super()._create_weights()
            # once, here: from now on the routed weights live at these addresses in the two-slice form
            for name in TWO_SLICE_PARAMETERS:
                parameter = getattr(self, name)
                parameter.data = api.localize(parameter.data)

        # -------------------------------------------------------------------------------------------- checkpoint loading
        def _map_global_expert_id(self, expert_id: int) -> List[int]:
            """Local slots of logical expert ``expert_id``: the initial placement until the load balancer publishes its
            replica map, that map afterwards (a reload after a rebalance then writes every replica)."""
            replica_map = self.eplb_state.logical_to_physical_map
            if replica_map is None:
                return super()._map_global_expert_id(expert_id)
            lo, hi = self.experts_start_idx, self.experts_end_idx
            return [slot - lo for slot in replica_map[expert_id].tolist() if lo <= slot < hi]

        def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, weight_name: str, shard_id: str,
                          expert_id: int, return_success: bool = False) -> Optional[bool]:
            if not any(param is getattr(self, name) for name in TWO_SLICE_PARAMETERS):
                return super().weight_loader(param, loaded_weight, weight_name, shard_id, expert_id, return_success)
            family = "w2_" if shard_id == "w2" else "w13_"
            slots = self._map_global_expert_id(expert_id) if family in weight_name else []
            for slot in slots:
                rows = _ExpertRows(param.data, slot)
                logical = rows.gather()
                self._load_weight(logical, loaded_weight, shard_id, False)     # the base layer's own shard placement
                rows.scatter(logical)
            if slots and hasattr(self, "_kernel_weights"):
                self._kernel_weights = None
            if not return_success:
                return None
            return bool(slots)

        # -------------------------------------------------------------------------------------------- warm-up
        def get_symm_buffer(self):
            cached = getattr(self, "_runtime_buffer", None)
            if cached is not None:
                return cached
            on_gpu = torch.cuda.is_available()
            if on_gpu and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm up B200 MegaMoE before CUDA-graph capture")
            buffer = super().get_symm_buffer()
            self._warm_up(buffer, torch.cuda.current_device() if on_gpu else -1)
            self._runtime_buffer = buffer
            return buffer

        def _warm_up(self, buffer: Any, device_index: int) -> None:
            """Prepare every BLOCK_M variant of this geometry once per process and device, then meet the other ranks at a
            host barrier so that no rank starts capturing while another still prepares."""
            group = self._ep_group_getter()
            ledger_key = (id(getattr(group, "device_group", None)), device_index, self.num_experts,
                          buffer.num_max_tokens_per_rank, self.top_k, self.hidden_size, self.intermediate_size,
                          self.num_shared_experts, self.activation, self.fast_math)
            if ledger_key in self._warmed_up:
                return
            api = self._import_backend()
            api.get_balanced_sm_locality_domains()
            api.precompile_mega_moe_variants(
                group.world_size, self.num_experts, buffer.num_max_tokens_per_rank, self.top_k, self.hidden_size,
                self.intermediate_size, self.num_shared_experts, **self._kernel_kwargs, fast_math=self.fast_math,
                per_die=True, localized_weights=True)
            host_group = getattr(group, "cpu_group", None)
            if host_group is not None and group.world_size > 1:
                torch.distributed.barrier(group=host_group)
            self._warmed_up.add(ledger_key)

        # -------------------------------------------------------------------------------------------- load balancer
        def get_expert_weights(self) -> List[torch.Tensor]:
            """Routed parameters as ``(num_local_experts, -1)`` views for the load balancer, which moves an expert by
            copying whole rows in place.  A two-slice weight gives one view per slice; both halves of an expert move
            together because the same row moves are applied to every view."""
            views: List[torch.Tensor] = []
            count = self.num_local_experts
            for name, parameter in self.named_parameters(recurse=False):
                if name.startswith("shared_"):
                    continue
                whole = parameter.data
                for offset, block in _expert_major_blocks(name, whole, count):
                    view = _rows_as_matrix(name, block, count)
                    in_place = (view.data_ptr() == whole.data_ptr() + offset and view.numel() == block.numel()
                                and view.is_contiguous())
                    if not in_place:
                        raise AssertionError(f"B200 MegaMoE EPLB {name}: the view at byte offset {offset} does not cover "
                                             "its memory in place")
                    views.append(view)
            return views

        # -------------------------------------------------------------------------------------------- stand-in base only
        def kernel_weights(self):
            """The stand-in base packs scale words from logical ``(E_l, N, K')`` parameters; show it that view for the
            duration of the call and hand the kernels the two-slice tensors themselves."""
            if getattr(self, "_kernel_weights", None) is None:
                held = {name: getattr(self, name).data for name in TWO_SLICE_PARAMETERS}
                try:
                    for name, tensor in held.items():
                        getattr(self, name).data = tensor.movedim(0, 1).flatten(1, 2)
                    (_, s13), (_, s2), shared_l1, shared_l2 = super().kernel_weights()
                finally:
                    for name, tensor in held.items():
                        getattr(self, name).data = tensor
                self._kernel_weights = ((held["w13_weight"].view(torch.int8), s13), (held["w2_weight"].view(torch.int8), s2),
                                        shared_l1, shared_l2)
            return self._kernel_weights

    B200MegaMoEExperts.weight_loader.supports_moe_loading = True  # type: ignore[attr-defined]
    B200MegaMoEExperts.__qualname__ = "B200MegaMoEExperts"
    return B200MegaMoEExperts


def standin_experts_class() -> type:
    """The plugin class on the stand-in base (tests, examples without the engine's layer)."""
    from . import _standin

    return make_experts_class(_standin.DeepGemmMegaMoEExperts, _standin.get_ep_group, _standin.MEGA_MOE_MXFP4)
