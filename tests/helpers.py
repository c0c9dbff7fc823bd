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
    from vllm_plugin_b200.backend.frontend import _use_scalar_validation_kernels
    api.set_kernel_options(orientation=orientation)
    _use_scalar_validation_kernels(engine == 1)
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
        api.set_kernel_options(orientation=0)
        _use_scalar_validation_kernels(False)
    return y, buf


def oracle_layer(layer: Layer, hidden, ids, w, clamp=10.0, pad=None):
    return O.moe_layer([hidden], [ids], [w], layer.experts, layer.shared, clamp,
                       None if pad is None else [pad])[0]


def synthetic_expert(syn, e: int) -> O.ExpertWeights:
    """Physical expert ``e`` of a :class:`vllm_plugin_b200.testing.SyntheticLayer` in the oracle's (untransformed) format."""
    w13, s13, w2, s2 = syn.raw
    return O.ExpertWeights(w13[e].cpu(), s13[e].cpu(), w2[e].cpu(), s2[e].cpu())


def synthetic_shared(syn) -> Optional[O.ExpertWeights]:
    if syn.shared_raw is None:
        return None
    q13, e13, q2, e2 = syn.shared_raw
    return O.ExpertWeights(q13.cpu(), e13.cpu(), q2.cpu(), e2.cpu(), fp8=True)


def oracle_token_sample(hidden, ids, w, sample, expert_of, shared: Optional[O.ExpertWeights], clamp=10.0):
    """Oracle output of the tokens ``sample`` (indices) of one call, dequantising ONE expert at a time (``expert_of(e)``
    returns its :class:`ExpertWeights`), so that a call over hundreds of resident experts can be checked: only the
    experts the sampled tokens hit are touched.  A token's output does not depend on the rest of the call."""
    sample = torch.as_tensor(sample, dtype=torch.long)
    hid = hidden.cpu()[sample]
    q, sf, ids_s, w_s, _ = O.stage_inputs(hid, ids.cpu()[sample], w.cpu()[sample], None)
    n, k = ids_s.shape
    slot_out = torch.zeros((k, n, hid.shape[1]), dtype=torch.bfloat16)
    sf_bytes = O.unpack_sf_words(sf)
    for e in torch.unique(ids_s[ids_s >= 0]).tolist():
        tok, slot = torch.nonzero(ids_s == e, as_tuple=True)
        w13, w2 = expert_of(e).dequant()
        slot_out[slot, tok] = O.expert_forward(q[tok], sf_bytes[tok], w_s[tok, slot], w13, w2, clamp)
    sh = None
    if shared is not None:
        s13, s2 = shared.dequant()
        sh = O.expert_forward(q, sf_bytes, torch.ones(n, dtype=torch.float32), s13, s2, clamp)
    return O.combine(slot_out, ids_s, sh)


def strict_metrics(y, ref) -> dict:
    """rel-L2, the strict max_abs and the number of elements above 2e-2 (the tolerance tests additionally allow one BF16
    ulp of the reference where that ulp exceeds 2e-2)."""
    a, b = y.float().cpu(), ref.float().cpu()
    d = (a - b).abs()
    return {"rel_l2": float((a - b).norm() / b.norm().clamp(min=1e-30)), "max_abs_strict": float(d.max()) if d.numel() else 0.0,
            "n_over_2e-2": int((d > 2e-2).sum()), "n": int(d.numel()), "max_abs_ref": float(b.abs().max()) if b.numel() else 0.0}


def log_parity(name: str, metrics: dict) -> None:
    """Append the metrics of a parity case to the file named by MMOE_PARITY_LOG (when set), for the measurement notes."""
    path = os.environ.get("MMOE_PARITY_LOG")
    if path:
        import json
        with open(path, "a") as f:
            f.write(json.dumps({"case": name, **metrics}) + "\n")
