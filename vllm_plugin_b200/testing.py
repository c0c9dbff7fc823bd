"""Seeded synthetic layer instances for benchmarks and tests, generated on any torch device (the GPU for the full-size
configurations: 384 experts are 7.2 GB of packed weights).

Shapes, sizes and value distributions follow the reference's own GPU harness (``tests/eplb_gpu_harness.py:189-207,
229-244,357-372``: Gaussian activations, Zipf routing over a fixed shuffle, UE8M0 scales, E4M3 shared weights) and the
benchmark configurations: routed weights ``N(0, 0.02)`` quantised to MXFP4 (one UE8M0 scale per 32 elements,
``2^ceil(log2(amax / 6))``, round to nearest even on the E2M1 grid, low nibble = even K), the shared expert ``N(0, 0.02)``
quantised to E4M3 with one power-of-two scale per 128x128 block expanded to per-32 UE8M0 scales.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .backend.weights import sf_to_required_layout, transform_weights_for_mega_moe


def _ceil_pow2_exponent(x: torch.Tensor) -> torch.Tensor:
    """Biased exponent byte of the smallest power of two >= x (x > 0), clamped to [1, 254]."""
    bits = x.float().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).int()
    return exp.clamp(1, 254)


def quantize_mxfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """float ``[..., K]`` -> (packed E2M1 int8 ``[..., K/2]``, UE8M0 exponent bytes uint8 ``[..., K/32]``)."""
    *lead, k = w.shape
    g = w.float().reshape(*lead, k // 32, 32)
    amax = g.abs().amax(dim=-1).clamp(min=2.0 ** -100)
    exp = _ceil_pow2_exponent(amax / 6.0)
    sf = (exp << 23).view(torch.float32)
    v = (g / sf.unsqueeze(-1)).clamp(-6.0, 6.0)
    a = v.abs()
    q = torch.where(a < 2.0, torch.round(a * 2) / 2, torch.where(a < 4.0, torch.round(a), torch.round(a / 2) * 2))
    code = torch.where(q < 2.0, (q * 2).to(torch.int32), torch.where(q < 4.0, (q + 2).to(torch.int32), (q / 2 + 4).to(torch.int32)))
    code = code | (((v < 0) & (q > 0)).to(torch.int32) << 3)
    code = code.reshape(*lead, k // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8).view(torch.int8)
    return packed, exp.to(torch.uint8)


def quantize_fp8_block128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """float ``[N, K]`` -> (E4M3 ``[N, K]``, UE8M0 bytes ``[N, K/32]``) with one power-of-two scale per 128x128 block."""
    n, k = w.shape
    blk = w.float().view(n // 128, 128, k // 128, 128)
    amax = blk.abs().amax(dim=(1, 3)).clamp(min=1e-4)
    exp = _ceil_pow2_exponent(amax / 448.0)
    sf = (exp << 23).view(torch.float32)
    q = (blk / sf[:, None, :, None]).to(torch.float8_e4m3fn).view(n, k)
    return q, exp.to(torch.uint8).repeat_interleave(128, dim=0).repeat_interleave(4, dim=1)


def routed_expert_raw(hidden: int, inter: int, seed: int, index: int, device, std: float = 0.02):
    """Physical routed expert ``index`` of the synthetic layer ``seed`` in checkpoint order: ``(w13 [2I, H/2] packed E2M1,
    s13 [2I, H/32] UE8M0 bytes, w2 [H, I/2], s2 [H, I/32])``.  A function of ``(seed, index)`` alone, so any rank of an
    expert-parallel run can reproduce any expert."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed * 100003 + index)
    w13, s13 = quantize_mxfp4(torch.randn((2 * inter, hidden), generator=g, device=dev) * std)
    w2, s2 = quantize_mxfp4(torch.randn((hidden, inter), generator=g, device=dev) * std)
    return w13, s13, w2, s2


def shared_expert_raw(hidden: int, inter: int, seed: int, device, std: float = 0.02):
    """The synthetic layer's shared expert: ``(w13 [2I, H] E4M3, s13 [2I, H/32], w2 [H, I], s2 [H, I/32])``."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed * 100003 + 99991)
    a = torch.randn((2 * inter, hidden), generator=g, device=dev) * std
    b = torch.randn((hidden, inter), generator=g, device=dev) * std
    return quantize_fp8_block128(a) + quantize_fp8_block128(b)


class SyntheticLayer:
    """Weights of ``num_local`` routed experts (+ optional shared expert) in the kernels' format, built expert by expert
    on ``device`` so that peak memory stays one expert of FP32 above the packed result."""

    def __init__(self, hidden: int, inter: int, num_local: int, shared: bool, device, seed: int = 0, std: float = 0.02,
                 first_expert: int = 0, localized: bool = False):
        self.hidden, self.inter, self.num_local = hidden, inter, num_local
        dev = torch.device(device)
        w13 = torch.empty((num_local, 2 * inter, hidden // 2), dtype=torch.int8, device=dev)
        w2 = torch.empty((num_local, hidden, inter // 2), dtype=torch.int8, device=dev)
        s13 = torch.empty((num_local, 2 * inter, hidden // 32), dtype=torch.uint8, device=dev)
        s2 = torch.empty((num_local, hidden, inter // 32), dtype=torch.uint8, device=dev)
        for e in range(num_local):
            w13[e], s13[e], w2[e], s2[e] = routed_expert_raw(hidden, inter, seed, first_expert + e, dev, std)
        self.raw = (w13, s13, w2, s2)
        l13 = sf_to_required_layout(s13, 2 * inter, hidden, num_local)
        l2 = sf_to_required_layout(s2, hidden, inter, num_local)
        self.l1, self.l2 = transform_weights_for_mega_moe((w13, l13), (w2, l2))
        if localized:
            from .backend.locality import localize
            self.l1 = (localize(self.l1[0]), self.l1[1])
            self.l2 = (localize(self.l2[0]), self.l2[1])
        self.shared_l1 = self.shared_l2 = None
        self.shared_raw = None
        if shared:
            q13, e13, q2, e2 = self.shared_raw = shared_expert_raw(hidden, inter, seed, dev, std)
            self.shared_l1, self.shared_l2 = transform_weights_for_mega_moe(
                (q13, sf_to_required_layout(e13, 2 * inter, hidden)), (q2, sf_to_required_layout(e2, hidden, inter)))

    def weight_bytes(self) -> int:
        w13, s13, w2, s2 = self.raw
        return sum(t.numel() * t.element_size() for t in (w13, s13, w2, s2))


def make_routing(num_tokens: int, num_experts: int, num_topk: int, seed: int, device="cpu", zipf_s: float = 0.0,
                 mask_frac: float = 0.0, hot: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gate logits ``N(0,1)`` (+ log-popularity bias: Zipf over a seeded shuffle, ``hot`` experts at 4x the mean), top-k by
    score, weights = softmax over the selected scores; ``mask_frac`` of the routes set to -1."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn((num_tokens, num_experts), generator=g)
    if zipf_s > 0.0:
        perm = torch.randperm(num_experts, generator=g)
        pop = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float32) ** zipf_s
        bias = torch.empty(num_experts)
        bias[perm] = torch.log(pop / pop.mean())
        logits = logits + bias
    if hot:
        logits[:, torch.randperm(num_experts, generator=g)[:hot]] += math.log(4.0)
    score, idx = torch.topk(logits, num_topk, dim=1)
    w = torch.softmax(score, dim=1).float()
    idx = idx.to(torch.int64)
    if mask_frac > 0.0:
        m = torch.rand(idx.shape, generator=g) < mask_frac
        idx = torch.where(m, torch.full_like(idx, -1), idx)
    return idx.to(device), w.to(device)


def make_hidden(num_tokens: int, hidden: int, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn((num_tokens, hidden), generator=g).to(torch.bfloat16).to(device)


def layer_work(num_valid_routes: int, num_tokens: int, distinct_experts: int, hidden: int, inter: int,
               shared: bool) -> Tuple[int, int]:
    """Algorithmic ``(flops, bytes)`` of one call: 6*H*I flop per (token, expert) pair; bytes = packed weights and scales
    of every expert hit (+ the shared expert) + BF16 activations in and out."""
    flop_pair = 6 * hidden * inter
    w_routed = 3 * inter * hidden // 2 + 3 * inter * hidden // 32
    w_shared = 3 * inter * hidden + 3 * inter * hidden // 32
    flops = (num_valid_routes + (num_tokens if shared else 0)) * flop_pair
    nbytes = distinct_experts * w_routed + (w_shared if shared else 0) + num_tokens * hidden * 4
    return flops, nbytes
