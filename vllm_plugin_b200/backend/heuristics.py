"""Host-side decisions of the MegaMoE expert backend: BLOCK_M selection, the set of BLOCK_M variants a geometry can
reach, and the admission gate.  Pure Python (no torch, no CUDA) so that the plugin can answer "can you serve this
geometry?" on any host.

Mirrors the reference's ``backend/heuristics.py``:

* :func:`get_block_m_for_mega_moe`   -- ``heuristics.py:123-197`` (float32 arithmetic, part of the staging contract)
* :func:`get_block_m_variants`       -- ``heuristics.py:217-228``
* :data:`VALIDATED_GEOMETRIES`, :data:`VALIDATED_EP_GEOMETRIES`, :data:`MIN_VALIDATED_EXPERTS_PER_RANK`
                                      -- ``heuristics.py:1354-1391`` (the geometry tables, kept as data)
* :func:`get_mega_moe_unsupported_reason` -- ``heuristics.py:1408-1503`` (total: never raises)

The reference additionally derives an SM107 shared-memory / ring configuration per variant; the B200 kernels size their
own pipelines (see ``csrc/``), so the structural part of the gate here is the set of shape rules those kernels need.
"""

from __future__ import annotations

import struct
from functools import lru_cache
from typing import Dict, Optional, Tuple

CANDIDATE_BLOCK_MS: Tuple[int, ...] = (8, 16, 32, 64, 96, 128, 192, 240)
VALID_BLOCK_MS: Tuple[int, ...] = (16, 32, 64, 128, 192, 240)  # what the selection can return
TOKEN_ALIGNMENT = 1920  # lcm of the candidates: the per-rank token capacity is rounded up to it
MAX_RANKS = 32
MAX_SHARED_EXPERTS = 1
GROUP_K = 32            # one UE8M0 scale per 32 K elements
TILE_K = 128            # K elements per pipeline stage (four scale groups = one packed int32 word)
TILE_ROWS = 128         # weight rows per tensor-core tile


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def align(a: int, b: int) -> int:
    return cdiv(a, b) * b


def _f32(x: float) -> float:
    """Round to the nearest float32 (the selection below is specified in float32 arithmetic)."""
    return struct.unpack("<f", struct.pack("<f", x))[0]


def get_token_alignment_for_mega_moe() -> int:
    return TOKEN_ALIGNMENT


def _parse_mma_type(mma_type: str) -> None:
    if mma_type not in ("fp8xfp4", "fp8xfp8", "bf16xbf16"):
        raise AssertionError(f"unsupported mma_type {mma_type!r}")


@lru_cache(maxsize=None)
def _block_m(num_ranks: int, num_experts: int, num_topk: int, num_tokens: int) -> int:
    # expected tokens per expert, each operation rounded to float32, left to right
    e = _f32(_f32(_f32(float(num_tokens)) * num_ranks) * num_topk)
    e = _f32(e / num_experts)
    covered = _f32(e + _f32(e ** 0.5))  # one standard deviation of head-room
    if e <= 10:
        return 16
    if e <= 24:
        return 32
    q = _f32(covered / 240)
    num_blocks = int(q) + (q > int(q))
    if num_blocks == 1 and covered > 192 and (num_experts // num_ranks) < 14:
        num_blocks = 2  # few experts per rank: prefer two medium blocks to one nearly full large block
    for cand in (64, 128, 192, 240):
        if _f32(float(num_blocks * cand)) >= covered:
            return cand
    return 240


def get_block_m_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_tokens: int,
                             num_topk: int, mma_type: str = "fp8xfp4") -> int:
    """BLOCK_M used for a call with ``num_tokens`` tokens on the calling rank (``num_max_tokens_per_rank`` is ignored,
    as in the reference)."""
    if num_tokens < 0:
        raise AssertionError("num_tokens must be >= 0")
    if num_ranks <= 0 or num_experts <= 0:
        raise AssertionError("num_ranks and num_experts must be positive")
    _parse_mma_type(mma_type)
    return _block_m(int(num_ranks), int(num_experts), int(num_topk), int(num_tokens))


@lru_cache(maxsize=None)
def get_block_m_variants(num_ranks: int, num_experts: int, num_topk: int, max_tokens: int) -> Tuple[int, ...]:
    """Sorted distinct BLOCK_M values reachable for ``M in [0, max_tokens]``: the variants to prepare before CUDA-graph
    capture.  The selection is not monotonic in M, so every M is evaluated."""
    seen = {_block_m(num_ranks, num_experts, num_topk, m) for m in range(0, max(1, max_tokens) + 1)}
    return tuple(sorted(seen))


# ---------------------------------------------------------------------------------------------------------------------
# Admission gate
# ---------------------------------------------------------------------------------------------------------------------
#: ``(hidden, intermediate, top-k) -> (admitted num_experts values, note)``; admitted at any EP size that leaves at
#: least :data:`MIN_VALIDATED_EXPERTS_PER_RANK` experts per rank.
VALIDATED_GEOMETRIES: Dict[Tuple[int, int, int], Tuple[Tuple[int, ...], str]] = {
    (5120, 2304, 6): ((32, 96, 192, 384), "target model: 384 routed experts, top-6; 192 / 96 / 32 are test sizes"),
    (5120, 2304, 3): ((128,), "draft model: 128 routed experts, top-3"),
}
MIN_VALIDATED_EXPERTS_PER_RANK = 12
#: ``(hidden, intermediate, top-k) -> ((num_experts, num_ranks) pairs, note)``: admitted exactly as listed.
VALIDATED_EP_GEOMETRIES: Dict[Tuple[int, int, int], Tuple[Tuple[Tuple[int, int], ...], str]] = {
    (5120, 2304, 6): (((388, 4), (392, 8), (400, 8), (400, 16), (416, 32)),
                      "target model with redundant (load-balancing) physical experts"),
    (5120, 2304, 3): (((128, 16), (128, 32), (132, 4), (136, 8), (144, 8), (144, 16), (160, 32)),
                      "draft model at large EP and with redundant physical experts"),
}


def get_validated_geometries():
    return dict(VALIDATED_GEOMETRIES)


def get_validated_ep_geometries():
    return dict(VALIDATED_EP_GEOMETRIES)


# ---- the gate as a list of rules, each returning a reason or None; the first reason wins ---------------------------------
class _Ask:
    """One admission question with every size coerced to ``int`` (a non-integer size is itself a reason to refuse)."""

    __slots__ = ("ranks", "experts", "tokens", "topk", "hidden", "inter", "shared", "mma", "act", "sms", "fast", "die_shared",
                 "any_geometry")

    def __init__(self, ranks, experts, tokens, topk, hidden, inter, shared, mma, act, sms, fast, die_shared, any_geometry):
        sizes = dict(num_ranks=ranks, num_experts=experts, num_max_tokens_per_rank=tokens, num_topk=topk, hidden=hidden,
                     intermediate_hidden=inter, num_shared_experts=shared)
        for name, value in sizes.items():
            if isinstance(value, bool) or not isinstance(value, int):
                raise TypeError(f"{name}={value!r} is not an integer")
        self.ranks, self.experts, self.tokens, self.topk = ranks, experts, tokens, topk
        self.hidden, self.inter, self.shared = hidden, inter, shared
        self.mma, self.act, self.sms, self.fast = mma, act, sms, fast
        self.die_shared, self.any_geometry = die_shared, any_geometry

    @property
    def shape_key(self) -> Tuple[int, int, int]:
        return (self.hidden, self.inter, self.topk)

    def describe(self) -> str:
        return (f"geometry (hidden={self.hidden}, intermediate_hidden={self.inter}, num_experts={self.experts}, "
                f"top-k={self.topk})")


def _rule_options(q: _Ask) -> Optional[str]:
    if q.mma != "fp8xfp4":
        return f"mma_type={q.mma!r} is not supported (only 'fp8xfp4')"
    if q.act != "swiglu":
        return f"activation={q.act!r} is not supported (only 'swiglu')"
    if q.fast not in (True, False, 0, 1):
        return f"fast_math={q.fast!r} is not supported"
    if q.die_shared:
        return "die-local shared-expert weights are not supported (B200 exposes one memory locality domain)"
    if q.sms is not None and q.sms < 1:
        return f"num_sms={q.sms} must be positive"
    return None


def _rule_ranges(q: _Ask) -> Optional[str]:
    if not 0 <= q.shared <= MAX_SHARED_EXPERTS:
        return f"num_shared_experts={q.shared} is outside the supported range [0, {MAX_SHARED_EXPERTS}]"
    if not 1 <= q.ranks <= MAX_RANKS:
        return f"num_ranks={q.ranks} is outside the supported range [1, {MAX_RANKS}]"
    positive = (("num_experts", q.experts), ("num_topk", q.topk), ("hidden", q.hidden), ("intermediate_hidden", q.inter),
                ("num_max_tokens_per_rank", q.tokens))
    bad = [f"{name}={value}" for name, value in positive if value < 1]
    return f"{bad[0]} must be positive" if bad else None


def _listed(q: _Ask) -> Tuple[bool, bool]:
    """(the (experts, ranks) pair is listed exactly, the expert count is listed for this shape)."""
    exact = (q.experts, q.ranks) in VALIDATED_EP_GEOMETRIES.get(q.shape_key, ((), ""))[0]
    general = q.experts in VALIDATED_GEOMETRIES.get(q.shape_key, ((), ""))[0]
    return exact, general


def _tables_as_text() -> str:
    general = "; ".join(f"hidden={h}, intermediate_hidden={i}, top-k={k}, num_experts in {list(es)}"
                        for (h, i, k), (es, _) in VALIDATED_GEOMETRIES.items())
    exact = "; ".join(f"hidden={h}, intermediate_hidden={i}, top-k={k}, (num_experts, EP size) in {list(ps)}"
                      for (h, i, k), (ps, _) in VALIDATED_EP_GEOMETRIES.items())
    return f"validated: {general}; exact pairs: {exact}"


def _rule_validated(q: _Ask) -> Optional[str]:
    """The geometry list is the reference plugin's (geometries its authors ran on their GPUs); on B200 this backend has
    run the listed shapes at EP 1, 2, 4 and 8.  ``allow_unvalidated`` skips the list, never the kernel limits."""
    if q.any_geometry:
        return None
    exact, general = _listed(q)
    if exact:
        return None
    if not general:
        return f"{q.describe()} has not been validated on GPUs with {q.ranks} ranks ({_tables_as_text()})"
    per_rank, rest = divmod(q.experts, q.ranks)
    if rest == 0 and per_rank < MIN_VALIDATED_EXPERTS_PER_RANK:
        return (f"{q.describe()} has not been validated on GPUs with {per_rank} experts per rank "
                f"(the smallest experts-per-rank that has run is {MIN_VALIDATED_EXPERTS_PER_RANK})")
    return None


#: limits the C library enforces on a geometry (``check_geometry`` behind ``mmoe_layout``); kept equal by a test
MAX_EXPERTS = 2048
MAX_EXPERTS_PER_RANK = 512
MAX_TOPK = 31


def _rule_kernel_limits(q: _Ask) -> Optional[str]:
    if q.experts % q.ranks:
        return f"num_experts={q.experts} is not divisible by num_ranks={q.ranks}"
    if q.experts > MAX_EXPERTS or q.experts // q.ranks > MAX_EXPERTS_PER_RANK:
        return f"num_experts={q.experts} exceeds {MAX_EXPERTS} (or {MAX_EXPERTS_PER_RANK} per rank)"
    if q.topk > MAX_TOPK:
        return f"num_topk={q.topk} exceeds the combine slot mask ({MAX_TOPK})"
    if q.hidden % 256:
        return f"hidden={q.hidden} must be a multiple of 256 (two {TILE_ROWS}-row weight tiles per task, combine vector width)"
    if q.inter % TILE_K:
        return f"intermediate_hidden={q.inter} must be a multiple of {TILE_K}"
    rows = align(q.tokens, TOKEN_ALIGNMENT) * q.ranks * min(q.topk, q.experts // q.ranks)
    if rows >= 2 ** 31:
        return "token pool exceeds 32-bit row indices"
    return None


_RULES = (_rule_options, _rule_ranges, _rule_validated, _rule_kernel_limits)


def get_mega_moe_unsupported_reason(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                    hidden: int, intermediate_hidden: int, num_shared_experts: int = 0,
                                    mma_type: str = "fp8xfp4", activation: str = "swiglu", *,
                                    num_sms: Optional[int] = None, fast_math: bool = True,
                                    localized_shared_weights: bool = False,
                                    allow_unvalidated: bool = False) -> Optional[str]:
    """``None`` when this backend can serve the geometry, else a short reason.  Total: returns a reason (never raises)
    for every input, including non-positive or non-integer sizes, so a caller can fall through to another backend."""
    try:
        ask = _Ask(num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                   num_shared_experts, mma_type, activation, num_sms, fast_math, localized_shared_weights,
                   allow_unvalidated)
        for rule in _RULES:
            reason = rule(ask)
            if reason is not None:
                return reason
        return None
    except Exception as exc:  # noqa: BLE001 - nothing may escape the predicate
        return f"geometry cannot be derived ({type(exc).__name__}: {exc})"
