"""Routed-weight "localisation" on B200.

The reference targets a two-die GPU with two memory locality domains and moves the two row halves of every routed
weight matrix into die-local memory: ``(*B, N, K) -> (2, *B, N/2, K)`` with the two slices padded apart to the 2 MiB
allocation granularity (``backend/locality.py:573-587``).  B200 exposes a single locality domain to CUDA, so nothing is
moved; the *shape contract* is kept (the layer class, checkpoint reload and the load-balancer views index the slices),
on ordinary device memory, and the kernels read the two-slice form through a 3-D tensor map.
"""

from __future__ import annotations

from typing import List

import torch

ALLOC_GRANULARITY = 2 << 20  # slices start on 2 MiB boundaries, as with the reference's driver allocations


def is_localization_available() -> bool:
    """True on a CUDA device of compute capability 10.0 (the two-slice form is then plain device memory)."""
    try:
        return torch.cuda.is_available() and tuple(torch.cuda.get_device_capability()) == (10, 0)
    except Exception:  # noqa: BLE001
        return False


def get_balanced_sm_locality_domains() -> List[int]:
    """SM -> locality domain map.  One domain on B200: every SM maps to domain 0."""
    n = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return [0] * n


def slice_stride_bytes(t: torch.Tensor, dim: int = -2) -> int:
    dim = dim % t.dim()
    half_shape = list(t.shape)
    half_shape[dim] //= 2
    nbytes = t.element_size()
    for s in half_shape:
        nbytes *= s
    return -(-nbytes // ALLOC_GRANULARITY) * ALLOC_GRANULARITY


def localize(t: torch.Tensor, dim: int = -2) -> torch.Tensor:
    """``(*B, N, K) -> (2, *B, N/2, K)``: slice ``s`` holds rows ``[s*N/2, (s+1)*N/2)`` along ``dim``; the slices are
    contiguous and ``slice_stride_bytes`` apart.  Works on any device (tests run it on the host)."""
    dim = dim % t.dim()
    n = t.shape[dim]
    assert n % 2 == 0, "the split dimension must be even"
    stride_b = slice_stride_bytes(t, dim)
    assert stride_b % t.element_size() == 0
    store = torch.empty(2 * stride_b, dtype=torch.uint8, device=t.device)
    half_shape = list(t.shape)
    half_shape[dim] = n // 2
    numel = 1
    for s in half_shape:
        numel *= s
    stride_e = stride_b // t.element_size()
    flat = store.view(t.dtype)
    contiguous_strides = []
    acc = 1
    for s in reversed(half_shape):
        contiguous_strides.append(acc)
        acc *= s
    contiguous_strides.reverse()
    out = torch.as_strided(flat, [2] + half_shape, [stride_e] + contiguous_strides)
    halves = t.split(n // 2, dim=dim)
    out[0].copy_(halves[0])
    out[1].copy_(halves[1])
    return out


def is_canonical_localized(t: torch.Tensor) -> bool:
    """Two contiguous slices a whole number of allocation granules apart."""
    if t.dim() < 3 or t.shape[0] != 2:
        return False
    return t[0].is_contiguous() and t[1].is_contiguous() and (t.stride(0) * t.element_size()) % ALLOC_GRANULARITY == 0


def delocalize(t: torch.Tensor, dim: int = -2) -> torch.Tensor:
    """Inverse of :func:`localize` (a copy): ``(2, *B, N/2, K) -> (*B, N, K)``."""
    dim = dim % (t.dim() - 1)
    return torch.cat([t[0], t[1]], dim=dim)
