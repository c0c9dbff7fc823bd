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


def _exponent_bytes(sf: torch.Tensor) -> torch.Tensor:
    """UE8M0 exponent byte of every scale: uint8 input as is, float32 powers of two by their exponent field."""
    if sf.dtype == torch.uint8:
        return sf
    if sf.dtype != torch.float32:
        raise AssertionError("scales must be float32 (UE8M0 values) or uint8 (E8M0 bytes)")
    raw = sf.contiguous().view(torch.int32)
    if bool((raw < 0).any()) or bool((raw & 0x7FFFFF).ne(0).any()):
        raise AssertionError("float32 scales must be non-negative powers of two")
    return (raw >> 23).to(torch.uint8)


def sf_to_required_layout(sf: torch.Tensor, mn: int, k: int, num_groups: Optional[int] = None) -> torch.Tensor:
    """Per-32-K UE8M0 scales (float32 powers of two or uint8 exponent bytes, ``([G,] mn, ceil(k/32))``) -> int32
    ``([G,] mn, ceil(k/128))`` with byte ``b`` of word ``w`` = K group ``4w + b``, stored MN-major: the rows of one word
    column are contiguous (strides ``(words * align(mn, 4), 1, align(mn, 4))``).  Missing K groups of the last word hold
    exponent 127 (scale 1.0)."""
    grouped = num_groups is not None
    if sf.dim() != (3 if grouped else 2):
        raise AssertionError("expected ([G,] mn, k/32) scales")
    exps = _exponent_bytes(sf if grouped else sf[None])
    groups, rows, per32 = exps.shape
    if rows != mn or per32 != (k + 31) // 32 or (grouped and groups != num_groups):
        raise AssertionError(f"scale shape {tuple(sf.shape)} does not match mn={mn}, k={k}")
    words = (per32 + 3) // 4
    # assemble each word from its four bytes with shifts (byte 0 in the low bits)
    lanes = torch.full((groups, rows, words * 4), 127, dtype=torch.int32, device=sf.device)
    lanes[..., :per32] = exps.to(torch.int32)
    lanes = lanes.view(groups, rows, words, 4)
    word = lanes[..., 0] | (lanes[..., 1] << 8) | (lanes[..., 2] << 16) | (lanes[..., 3] << 24)
    pitch = (mn + 3) // 4 * 4
    out = torch.empty_strided((groups, mn, words), (words * pitch, 1, pitch), dtype=torch.int32, device=sf.device)
    out.copy_(word)
    return out if grouped else out[0]


def _permute_rows(t: torch.Tensor, source_row: torch.Tensor) -> torch.Tensor:
    """``out[..., r, :] = t[..., source_row[r], :]`` along dim -2, in a tensor with the strides of ``t``."""
    out = torch.empty_like(t)                   # preserve_format keeps dense non-contiguous (MN-major) strides
    out.copy_(t.index_select(t.dim() - 2, source_row.to(t.device)))
    return out


def _utccp_source_rows(rows: int) -> torch.Tensor:
    """Stored position ``128 b + 4 c + a`` holds row ``128 b + 32 a + c``: the order in which ``tcgen05.cp`` (32 lanes x
    four 32-bit columns, replicated to the four lane quadrants) wants the scales of a 128-row block."""
    if rows % 128:
        raise AssertionError("scale rows must be a multiple of 128")
    p = torch.arange(rows)
    within = p % 128
    return p - within + 32 * (within % 4) + within // 4


def _gate_up_source_rows(rows: int, gran: int) -> torch.Tensor:
    """Stored row ``2 gran g + j`` holds gate row ``gran g + j`` for ``j < gran`` and up row ``gran g + j - gran`` after."""
    half = rows // 2
    if rows % 2 or half % gran:
        raise AssertionError(f"{rows} rows cannot be interleaved in groups of {gran}")
    p = torch.arange(rows)
    group, j = p // (2 * gran), p % (2 * gran)
    return torch.where(j < gran, group * gran + j, half + group * gran + j - gran)


def transpose_sf_for_utccp(sf: torch.Tensor) -> torch.Tensor:
    """4x32 transpose of int32 scale words ``([G,] MN, K/128)`` inside every 128-row block; keeps the input strides."""
    if sf.dtype != torch.int32 or sf.dim() not in (2, 3):
        raise AssertionError("expected int32 scale words ([G,] MN, K/128)")
    return _permute_rows(sf, _utccp_source_rows(sf.shape[-2]))


def interleave_weights(t: torch.Tensor, gran: int = 8) -> torch.Tensor:
    """``[gate | up]`` rows -> ``[gate 0..7, up 0..7, gate 8..15, up 8..15, ...]`` along dim -2."""
    if t.dim() not in (2, 3):
        raise AssertionError("expected ([G,] rows, columns)")
    return _permute_rows(t, _gate_up_source_rows(t.shape[-2], gran))


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
