"""Shared helpers of the test-suite: seeded layer instances in both the oracle's and the kernels' formats."""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import List, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import mmoe_oracle as O  # noqa: E402


@dataclass
class Layer:
    hidden: int
    inter: int
    num_experts: int
    num_topk: int
    experts: List[O.ExpertWeights]
    shared: Optional[O.ExpertWeights]


def make_layer(hidden: int, inter: int, num_experts: int, num_topk: int, shared: bool, seed: int = 0) -> Layer:
    return Layer(hidden, inter, num_experts, num_topk, O.make_experts(num_experts, hidden, inter, seed),
                 O.make_shared_expert(hidden, inter, seed + 1000) if shared else None)


def kernel_weights(layer: Layer, device, lo: int = 0, hi: Optional[int] = None, localized: bool = False):
    """Weights of local experts [lo, hi) in the format ``fp8_fp4_mega_moe`` takes (after the backend's transform)."""
    from vllm_plugin_b200 import api

    hi = layer.num_experts if hi is None else hi
    ex = layer.experts[lo:hi]
    h, i = layer.hidden, layer.inter
    w13 = torch.stack([e.w13 for e in ex])
    w2 = torch.stack([e.w2 for e in ex])
    from vllm_plugin_b200.backend.weights import sf_to_required_layout
    s13 = sf_to_required_layout(torch.stack([e.w13_sf for e in ex]), 2 * i, h, len(ex))
    s2 = sf_to_required_layout(torch.stack([e.w2_sf for e in ex]), h, i, len(ex))
    l1, l2 = api.transform_weights_for_mega_moe((w13, s13), (w2, s2))
    l1 = (l1[0].to(device), _to_device_keep_strides(l1[1], device))
    l2 = (l2[0].to(device), _to_device_keep_strides(l2[1], device))
    if localized:
        l1, l2 = api.localize_mega_moe_weights(l1, l2)
    sl1 = sl2 = None
    if layer.shared is not None:
        s = layer.shared
        ss13 = sf_to_required_layout(s.w13_sf, 2 * i, h)
        ss2 = sf_to_required_layout(s.w2_sf, h, i)
        t1, t2 = api.transform_weights_for_mega_moe((s.w13, ss13), (s.w2, ss2))
        sl1 = (t1[0].to(device), _to_device_keep_strides(t1[1], device))
        sl2 = (t2[0].to(device), _to_device_keep_strides(t2[1], device))
    return l1, l2, sl1, sl2


def _to_device_keep_strides(t: torch.Tensor, device) -> torch.Tensor:
    out = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=device)
    out.copy_(t)
    return out


def run_layer(layer: Layer, hidden, ids, w, *, t_max: int = 1920, clamp=10.0, fast_math=True, engine=0, pad=None,
              localized=False, stats=None, buf=None, weights=None, orientation=0):
    """Stage + forward on cuda:0 at EP1; returns ``(y, buf)``."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup

    dev = torch.device("cuda", 0)
    if buf is None:
        buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), layer.num_experts, t_max, layer.num_topk, layer.hidden,
                                               layer.inter, 1 if layer.shared is not None else 0)
    if weights is None:
        weights = kernel_weights(layer, dev, localized=localized)
    l1, l2, sl1, sl2 = weights
    api.set_kernel_options(engine=engine, orientation=orientation)
    try:
        m = hidden.shape[0]
        y = torch.empty((m, layer.hidden), dtype=torch.bfloat16, device=dev)
        api.stage_inputs_for_mega_moe(buf, hidden.to(dev), ids.to(dev), w.to(dev),
                                      is_padding=None if pad is None else pad.to(dev))
        api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp,
                             fast_math=fast_math)
        from vllm_plugin_b200.backend.frontend import read_status
        read_status(buf)
    finally:
        api.set_kernel_options(engine=0, orientation=0)
    return y, buf


def oracle_layer(layer: Layer, hidden, ids, w, clamp=10.0, pad=None):
    return O.moe_layer([hidden], [ids], [w], layer.experts, layer.shared, clamp,
                       None if pad is None else [pad])[0]
