"""Weight layout of the B200 MegaMoE kernels (``transform_weights_for_mega_moe``).

Input contract = the reference's (``backend/weights.py:5-13``): L1 weights ``(E_l, 2I, H/2)`` int8, two E2M1 values per
byte with the low nibble holding the even K index, rows ``[gate | up]``; L2 weights ``(E_l, H, I/2)``; scale factors
int32 ``(E_l, N, ceil(K/128))`` with four UE8M0 bytes per word (byte ``b`` of word ``w`` = K group ``4w + b``) stored
MN-major (``stride(-2) == 1``), which is what :func:`sf_to_required_layout` produces from per-32 scales
(``backend/weights.py:37-80``).

Output = bit-identical to the reference's transform (``backend/weights.py:83-145``), which is also the layout the
serving engine's native layer keeps its parameters in, so parameters loaded by that layer can be handed to the kernels
unchanged: L1 weights and scales get the gate/up 8-row interleave (``[g0..7, u0..7, g8..15, u8..15, ...]``), then L1 and
L2 scales get the 4x32 transpose inside every 128-row block (stored position ``4c + a`` holds row ``32a + c``), which
makes each (128 rows, 128 K) block of scales one contiguous 512-byte chunk in the order ``tcgen05.cp`` copies into
tensor memory.  The sm_100a kernels undo the interleave for free: a 5-D TMA box lands the 128 gate rows and the 128 up
rows of a channel tile in two separate shared-memory tiles.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

_SUPPORTED_ACTIVATIONS = ("swiglu",)


def _align(x: int, a: int) -> int:
    return -(-x // a) * a


def sf_to_required_layout(sf: torch.Tensor, mn: int, k: int, num_groups: Optional[int] = None) -> torch.Tensor:
    """Per-32-K UE8M0 scales (float32 powers of two or uint8 exponent bytes, ``([G,] mn, ceil(k/32))``) -> int32
    ``([G,] mn, ceil(k/128))``, MN-major (strides ``(ceil(k/128) * align(mn, 4), 1, align(mn, 4))``)."""
    assert sf.dim() == (3 if num_groups is not None else 2), "expected ([G,] mn, k/32) scales"
    squeeze = num_groups is None
    if squeeze:
        sf = sf.unsqueeze(0)
    g, n, k32 = sf.shape
    assert n == mn and k32 == -(-k // 32), f"scale shape {tuple(sf.shape)} does not match mn={mn}, k={k}"
    if num_groups is not None:
        assert g == num_groups
    if sf.dtype == torch.uint8:
        bytes_ = sf
    else:
        assert sf.dtype == torch.float32, "scales must be float32 (UE8M0 values) or uint8 (E8M0 bytes)"
        bits = sf.view(torch.int32)
        assert (bits >= 0).all() and (bits & 0x7FFFFF == 0).all(), "float32 scales must be non-negative powers of two"
        bytes_ = (bits >> 23).to(torch.uint8)
    k128 = -(-k32 // 4)
    if k32 % 4:
        bytes_ = torch.nn.functional.pad(bytes_, (0, k128 * 4 - k32), value=127)
    packed = bytes_.contiguous().view(torch.int32)
    n4 = _align(mn, 4)
    out = torch.empty_strided((g, mn, k128), (k128 * n4, 1, n4), dtype=torch.int32, device=sf.device)
    out.copy_(packed)
    return out.squeeze(0) if squeeze else out


def transpose_sf_for_utccp(sf: torch.Tensor) -> torch.Tensor:
    """4x32 transpose of int32 scale words ``([G,] MN, K/128)`` inside every 128-row block; keeps the input strides."""
    assert sf.dtype == torch.int32 and sf.dim() in (2, 3)
    squeeze = sf.dim() == 2
    if squeeze:
        sf = sf.unsqueeze(0)
    g, mn, kw = sf.shape
    assert mn % 128 == 0, "scale rows must be a multiple of 128"
    res = sf.reshape(g, -1, 4, 32, kw).transpose(2, 3).reshape(g, mn, kw)
    out = torch.empty_like(sf).copy_(res)
    return out.squeeze(0) if squeeze else out


def interleave_weights(t: torch.Tensor, gran: int = 8) -> torch.Tensor:
    """``[gate | up]`` rows -> ``[gate 0..7, up 0..7, gate 8..15, up 8..15, ...]`` along dim 1 (dim 0 for 2-D inputs)."""
    assert t.dim() in (2, 3)
    squeeze = t.dim() == 2
    if squeeze:
        t = t.unsqueeze(0)
    g, n, *rest = t.shape
    half = n // 2
    assert half % gran == 0
    gate = t[:, :half].reshape(g, half // gran, gran, *rest)
    up = t[:, half:].reshape(g, half // gran, gran, *rest)
    out = torch.empty_like(t).copy_(torch.stack([gate, up], dim=2).reshape(g, n, *rest))
    return out.squeeze(0) if squeeze else out


def transform_weights_for_mega_moe(l1_weights: Tuple[torch.Tensor, torch.Tensor],
                                   l2_weights: Tuple[torch.Tensor, torch.Tensor], activation: str = "swiglu"
                                   ) -> Tuple[Tuple[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]:
    """``(weights, sf)`` pairs in, ``(weights, sf)`` pairs out; shared-expert pairs (2-D tensors) go through the same
    function."""
    assert activation in _SUPPORTED_ACTIVATIONS, f"Activation must be one of {_SUPPORTED_ACTIVATIONS}, got `{activation}`"
    if not isinstance(l1_weights, tuple) or not isinstance(l2_weights, tuple):
        raise NotImplementedError("only (weights, scale factors) pairs are supported (MXFP4 / MXFP8 weights)")
    for w, sf in (l1_weights, l2_weights):
        assert sf.dtype == torch.int32, "scale factors must be packed int32 words"
        assert sf.stride(-2) == 1, "scale factors must be MN-major (stride(-2) == 1)"
        assert w.shape[-2] == sf.shape[-2], "weights and scale factors disagree on the row count"
    if l1_weights[0].is_cuda and _native_transform_applies(l1_weights) and _native_transform_applies(l2_weights):
        # device tensors: two HBM-bound CUDA kernels per pair (bit-identical to the indexing ops below)
        return ((_native_transform(l1_weights, True)), (l2_weights[0], _native_transform(l2_weights, False)[1]))
    l1 = (interleave_weights(l1_weights[0]), transpose_sf_for_utccp(interleave_weights(l1_weights[1])))
    l2 = (l2_weights[0], transpose_sf_for_utccp(l2_weights[1]))
    return l1, l2


def _native_transform_applies(pair: Tuple[torch.Tensor, torch.Tensor]) -> bool:
    w, sf = pair
    rows = w.shape[-2]
    dense = sf.stride(-1) == rows and (sf.dim() == 2 or sf.stride(0) == rows * sf.shape[-1])
    return (w.is_cuda and sf.is_cuda and w.is_contiguous() and w.element_size() == 1 and rows % 128 == 0
            and w.shape[-1] % 16 == 0 and dense and w.data_ptr() % 16 == 0 and sf.data_ptr() % 16 == 0)


def _native_transform(pair: Tuple[torch.Tensor, torch.Tensor], interleave: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    from . import _native
    w, sf = pair
    groups = w.shape[0] if w.dim() == 3 else 1
    rows, row_bytes, k_words = w.shape[-2], w.shape[-1], sf.shape[-1]
    w_out = torch.empty_like(w) if interleave else w
    sf_out = torch.empty_like(sf)                      # keeps the MN-major strides
    assert sf_out.stride() == sf.stride()
    stream = torch.cuda.current_stream(w.device).cuda_stream
    with torch.cuda.device(w.device):
        _native.check(_native.load().mmoe_transform_weights(
            w.data_ptr() if interleave else None, w_out.data_ptr() if interleave else None, sf.data_ptr(),
            sf_out.data_ptr(), groups, rows, row_bytes, k_words, 1 if interleave else 0, stream))
    return w_out, sf_out
