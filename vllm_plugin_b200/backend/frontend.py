"""``fp8_fp4_mega_moe`` and its companions: host-side checks, BLOCK_M selection, variant preparation and the launch
sequence of one forward call.  Mirrors ``backend/frontend.py`` of the reference (``KernelOptions`` :72-116,
``get_block_m_for_mega_moe`` :157-171, ``check_mega_moe_arguments`` :437-623, ``fp8_fp4_mega_moe`` :627-848,
``precompile_mega_moe_variants`` :851-897) on top of the C ABI of ``libmmoe_b200.so``.

At EP = 1 one call is: route ordering -> pool placement -> grouped GEMM1 (+SwiGLU/requant) -> grouped GEMM2 -> combine.
At EP > 1 the default transport is the device-side exchange over NVLink peer memory (``mmoe_forward_ep``: counts and rows
pushed into the peers' symmetric workspaces, GEMM2 writing its rows straight back to the rank they came from); the
host-driven alternative issues the same three exchanges as ``torch.distributed`` all-to-allv calls on the caller's group.

Like the reference (``frontend.py:650-754``) a call with the tensors of the previous call skips the argument checks: the
record of the last validated call is kept on the buffer, and a call whose weight tensors are the same objects at the same
addresses goes straight to the launch.
"""

from __future__ import annotations

import ctypes
import dataclasses
import math
from typing import Any, Dict, Optional, Tuple

import torch

from . import _native
from . import heuristics as _h


@dataclasses.dataclass(frozen=True)
class KernelOptions:
    """Process-wide launch options (the reference keeps every tuning knob an explicit field, never an environment
    variable: ``backend/frontend.py:72-116``)."""

    block_m: int = 0          # > 0 forces the BLOCK_M variant
    timeout_ms: int = 2000    # bound of every device-side wait
    ep_transport: str = "peer"  # EP > 1: "peer" = device-side exchange over NVLink peer memory (graph-capturable),
                                # "nccl" = host-driven all-to-allv (also used when symmetric memory is unavailable)
    fuse_return: bool = True    # "peer" transport: GEMM2's epilogue stores its rows straight into the source rank's
                                # buffer over NVLink, and the dispatch overlaps the shared expert's GEMMs on a second
                                # stream; False = one stream, separate copy kernel after GEMM2 (same result)
    status_poll_interval: int = 32   # eager calls between two non-blocking reads of the device status words (a bounded
                                     # wait that expired, an expert id out of range); 0 = never, 1 = every call
    orientation: int = 0        # grouped-GEMM kernel family: 0 = chosen per call from the expected rows per expert,
                                # 1 = weights-as-A (small token counts) always, 2 = tokens-as-A wherever the geometry
                                # allows, 3 = tokens-as-A on CTA pairs; every rank of a group must use the same value


_kernel_options = KernelOptions()
_engine = _native.ENGINE_TENSOR_CORE     # the test-suite may switch to the scalar validation kernels, see below
_prepared: Dict[Tuple, Tuple[int, ...]] = {}


def set_kernel_options(**kwargs: Any) -> KernelOptions:
    global _kernel_options
    _kernel_options = dataclasses.replace(_kernel_options, **kwargs)
    if _kernel_options.block_m and _kernel_options.block_m not in _h.VALID_BLOCK_MS:
        raise AssertionError(f"block_m={_kernel_options.block_m} is not one of {_h.VALID_BLOCK_MS}")
    if "orientation" in kwargs:
        _native.check(_native.load().mmoe_set_tuning(0, int(_kernel_options.orientation)))
    return _kernel_options


def get_kernel_options() -> KernelOptions:
    return _kernel_options


def _use_scalar_validation_kernels(on: bool) -> None:
    """Test hook, not an option of the product: run the grouped GEMMs of subsequent calls with the library's scalar
    validation kernels (plain FP32 dot products over the same plan, pool and epilogues) instead of the tensor-core ones."""
    global _engine
    _engine = _native.ENGINE_SCALAR_VALIDATION if on else _native.ENGINE_TENSOR_CORE


def require_sm100() -> None:
    """The kernels are compiled for sm_100a only (the reference gates on its own architecture the same way,
    ``backend/frontend.py:261-270``)."""
    if not torch.cuda.is_available():
        raise RuntimeError("The B200 MegaMoE backend needs a CUDA device of compute capability 10.0; none is visible.")
    cc = tuple(torch.cuda.get_device_capability())
    if cc != (10, 0):
        raise RuntimeError(f"The B200 MegaMoE backend needs compute capability 10.0 (sm_100a), got {cc[0]}.{cc[1]}.")


def get_block_m_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_tokens: int,
                             num_topk: int, mma_type: str = "fp8xfp4") -> int:
    if _kernel_options.block_m > 0:
        return _kernel_options.block_m
    return _h.get_block_m_for_mega_moe(num_ranks, num_experts, num_max_tokens_per_rank, num_tokens, num_topk, mma_type)


def precompile_mega_moe_variants(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                 hidden: int, intermediate_hidden: int, num_shared_experts: int = 0, *,
                                 activation_clamp: Optional[float] = None, activation_alpha: float = 1.0,
                                 activation_beta: float = 0.0, fast_math: bool = True, per_die: bool = False,
                                 localized_weights: bool = False, localized_shared_weights: bool = False
                                 ) -> Tuple[int, ...]:
    """Make every BLOCK_M variant the geometry can reach launchable (kernel images loaded, shared-memory limits raised,
    tensor-map encoder resolved) and return them.  Must run outside CUDA-graph capture; calls after the first are free."""
    require_sm100()
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("MegaMoE variants must be prepared before CUDA-graph capture")
    if activation_alpha != 1.0 or activation_beta != 0.0:
        raise NotImplementedError("activation_alpha / activation_beta other than (1, 0) are not supported")
    if localized_shared_weights:
        raise NotImplementedError("localized shared-expert weights are not supported")
    t = _h.align(num_max_tokens_per_rank, _h.TOKEN_ALIGNMENT)
    key = (torch.cuda.current_device(), num_ranks, num_experts, t, num_topk, hidden, intermediate_hidden, num_shared_experts)
    if key in _prepared:
        return _prepared[key]
    geo = _native.MmoeGeometry(num_ranks, 0, num_experts, num_topk, hidden, intermediate_hidden, num_shared_experts, t)
    out = (ctypes.c_int32 * 8)()
    n = ctypes.c_int32(0)
    _native.check(_native.load().mmoe_prepare(ctypes.byref(geo), out, 8, ctypes.byref(n),
                                              torch.cuda.current_stream().cuda_stream))
    variants = tuple(int(out[i]) for i in range(n.value))
    assert variants == _h.get_block_m_variants(num_ranks, num_experts, num_topk, t), "host and library disagree on the variants"
    _prepared[key] = variants
    return variants


def built_block_ms(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                   intermediate_hidden: int, num_shared_experts: int = 0) -> Tuple[int, ...]:
    t = _h.align(num_max_tokens_per_rank, _h.TOKEN_ALIGNMENT)
    key = (torch.cuda.current_device(), num_ranks, num_experts, t, num_topk, hidden, intermediate_hidden, num_shared_experts)
    return _prepared.get(key, ())


# ---------------------------------------------------------------------------------------------------------------------
# argument checks (the reference's host asserts raise AssertionError)
# ---------------------------------------------------------------------------------------------------------------------
def _split_weights(w: torch.Tensor, what: str, e_l: int, n: int, k_packed: int) -> Tuple[torch.Tensor, int]:
    """Accept the plain ``(E_l, N, K/2)`` tensor or the two-slice ``(2, E_l, N/2, K/2)`` one; return (tensor, slice stride)."""
    assert w.dtype in (torch.int8, torch.uint8), f"{what} must be packed FP4 in int8"
    if w.dim() == 3:
        assert tuple(w.shape) == (e_l, n, k_packed) and w.is_contiguous(), f"{what}: expected contiguous {(e_l, n, k_packed)}, got {tuple(w.shape)}"
        return w, 0
    assert w.dim() == 4 and tuple(w.shape) == (2, e_l, n // 2, k_packed), f"{what}: expected {(2, e_l, n // 2, k_packed)}, got {tuple(w.shape)}"
    assert w[0].is_contiguous() and w[1].is_contiguous(), f"{what}: each slice must be contiguous"
    return w, w.stride(0) * w.element_size()


def _check_sf(sf: torch.Tensor, what: str, lead: Tuple[int, ...], n: int, k: int) -> None:
    assert sf.dtype == torch.int32, f"{what} must be int32 (four UE8M0 bytes per word)"
    assert tuple(sf.shape) == lead + (n, k // 128), f"{what}: expected {lead + (n, k // 128)}, got {tuple(sf.shape)}"
    assert sf.stride(-2) == 1 and sf.stride(-1) == n, f"{what} must be dense MN-major (stride(-2) == 1, stride(-1) == rows)"
    if lead:
        assert sf.stride(0) == n * (k // 128), f"{what}: experts must be contiguous"


def check_mega_moe_arguments(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights, stats, recipe,
                             activation, activation_clamp, fast_math, activation_alpha, activation_beta):
    assert tuple(recipe) == (1, 1, 32), f"unsupported recipe {recipe}"
    assert activation == "swiglu", f"unsupported activation {activation!r}"
    if activation_alpha != 1.0 or activation_beta != 0.0:
        raise NotImplementedError("activation_alpha / activation_beta other than (1, 0) are not supported")
    h, inter = sym_buffer.hidden, sym_buffer.intermediate_hidden
    r = sym_buffer.num_ranks
    assert r <= _h.MAX_RANKS
    e_l = sym_buffer.num_experts // r
    m = y.size(0)
    assert y.dim() == 2 and y.size(1) == h and y.dtype == torch.bfloat16 and y.is_contiguous(), "y must be contiguous BF16 (M, H)"
    assert y.is_cuda and y.data_ptr() % 16 == 0, "y must be a 16-byte aligned CUDA tensor"
    assert m <= sym_buffer.num_max_tokens_per_rank, "num_tokens must be <= num_max_tokens_per_rank"
    w13, s13 = _split_weights(l1_weights[0], "l1 weights", e_l, 2 * inter, h // 2)
    w2, s2 = _split_weights(l2_weights[0], "l2 weights", e_l, h, inter // 2)
    _check_sf(l1_weights[1], "l1 scale factors", (e_l,), 2 * inter, h)
    _check_sf(l2_weights[1], "l2 scale factors", (e_l,), h, inter)
    n_shared = sym_buffer.num_shared_experts
    assert n_shared <= _h.MAX_SHARED_EXPERTS
    assert (shared_l1_weights is None) == (shared_l2_weights is None)
    assert (shared_l1_weights is not None) == (n_shared > 0), "shared expert weights must be given iff the buffer has a shared expert"
    if shared_l1_weights is not None:
        sw13, ssf13 = shared_l1_weights
        sw2, ssf2 = shared_l2_weights
        assert sw13.dtype == torch.float8_e4m3fn and tuple(sw13.shape) == (2 * inter * n_shared, h) and sw13.is_contiguous()
        assert sw2.dtype == torch.float8_e4m3fn and tuple(sw2.shape) == (h, inter * n_shared) and sw2.is_contiguous()
        _check_sf(ssf13, "shared l1 scale factors", (), 2 * inter, h)
        _check_sf(ssf2, "shared l2 scale factors", (), h, inter)
    if stats is not None:
        assert stats.dtype == torch.int32 and stats.numel() == e_l and stats.is_contiguous() and stats.is_cuda
    if activation_clamp is not None:
        assert activation_clamp > 0, "activation_clamp must be positive"
    assert isinstance(fast_math, (bool, int))
    return s13, s2


def _weights_struct(l1, l2, sl1, sl2, s13: int, s2: int) -> _native.MmoeWeights:
    w = _native.MmoeWeights()
    w.w13, w.w13_sf = l1[0].data_ptr(), l1[1].data_ptr()
    w.w2, w.w2_sf = l2[0].data_ptr(), l2[1].data_ptr()
    if sl1 is not None:
        w.shared_w13, w.shared_w13_sf = sl1[0].data_ptr(), sl1[1].data_ptr()
        w.shared_w2, w.shared_w2_sf = sl2[0].data_ptr(), sl2[1].data_ptr()
    w.w13_slice_stride, w.w2_slice_stride = s13, s2
    return w


# ---------------------------------------------------------------------------------------------------------------------
# EP > 1 exchanges (NCCL all-to-allv through torch.distributed); device-agnostic so that the host logic is testable
# with gloo ranks on CPU tensors
# ---------------------------------------------------------------------------------------------------------------------
def exchange_counts(group, send_count: torch.Tensor, recv_count: torch.Tensor) -> Tuple[list, list]:
    """``send_count`` int32 ``[E]`` (routes of this rank per destination physical expert) -> ``recv_count`` int32
    ``[R, E_l]`` (per source rank and local expert).  Returns the per-peer row counts ``(send_splits, recv_splits)``."""
    import torch.distributed as dist
    r = group.size()
    dist.all_to_all_single(recv_count.view(-1), send_count.view(-1), group=group)
    send_splits = send_count.view(r, -1).sum(dim=1).tolist()
    recv_splits = recv_count.view(r, -1).sum(dim=1).tolist()
    return send_splits, recv_splits


def exchange_rows(group, dst: torch.Tensor, src: torch.Tensor, dst_splits, src_splits) -> None:
    """All-to-allv of whole rows: peer ``p`` gets ``src_splits[p]`` consecutive rows of ``src`` and contributes
    ``dst_splits[p]`` consecutive rows of ``dst`` (source ranks ascending)."""
    import torch.distributed as dist
    n_src, n_dst = sum(src_splits), sum(dst_splits)
    s = src[:n_src]
    d = dst[:n_dst]
    if s.dtype == torch.float8_e4m3fn:
        s, d = s.view(torch.uint8), d.view(torch.uint8)
    dist.all_to_all_single(d, s, list(dst_splits), list(src_splits), group=group)


class _CallRecord:
    """What the last validated call on a buffer established: the tensor objects it checked (kept alive, so that their
    identities cannot be reused), the structures built from them, and the status poll state."""

    __slots__ = ("tensors", "addresses", "weights", "stats", "options_key", "options", "peers", "variants_ready")

    def matches(self, tensors) -> bool:
        kept = self.tensors
        for a, b, addr in zip(tensors, kept, self.addresses):
            if a is not b or (a is not None and a.data_ptr() != addr):
                return False
        return True


class _StatusPoll:
    """Non-blocking watch on the device status words of one buffer: every ``interval`` eager calls the words are copied
    to pinned host memory behind the call; a later call that finds the copy complete inspects it."""

    def __init__(self, sym_buffer):
        self.host = torch.zeros(8, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.calls = 0

    def before_call(self, sym_buffer) -> None:
        if self.pending and self.event.query():
            self.pending = False
            words = self.host.tolist()
            if words[0] != 0 or words[4] != 0:
                sym_buffer.status.zero_()                      # re-arm: the next healthy call reports healthy
                if words[0] != 0:
                    raise RuntimeError(f"a device-side wait of an earlier MegaMoE call expired (kernel {words[1]}, role "
                                       f"{words[2]}, block {words[3]}): its output is not valid")
                raise AssertionError(f"{words[4]} expert ids of an earlier MegaMoE call were >= num_experts")

    def after_call(self, sym_buffer, interval: int) -> None:
        self.calls += 1
        if interval > 0 and not self.pending and self.calls % interval == 0:
            self.host.copy_(sym_buffer.status, non_blocking=True)
            self.event.record()
            self.pending = True


def _validate(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights, stats, recipe, activation,
              activation_clamp, fast_math, activation_alpha, activation_beta, tensors) -> _CallRecord:
    require_sm100()
    s13, s2 = check_mega_moe_arguments(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights,
                                       stats, recipe, activation, activation_clamp, fast_math, activation_alpha,
                                       activation_beta)
    rec = _CallRecord()
    rec.tensors = tensors
    rec.addresses = tuple(t.data_ptr() if t is not None else 0 for t in tensors)
    rec.weights = _weights_struct(l1_weights, l2_weights, shared_l1_weights, shared_l2_weights, s13, s2)
    rec.options_key = None
    rec.options = None
    rec.peers = None
    if sym_buffer.peer_ptrs is not None:
        rec.peers = (ctypes.c_void_p * sym_buffer.num_ranks)(*sym_buffer.peer_ptrs)
    rec.variants_ready = False
    return rec


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer, shared_l1_weights=None, shared_l2_weights=None,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                     recipe: Tuple[int, int, int] = (1, 1, 32), activation: str = "swiglu",
                     activation_clamp: Optional[float] = None, fast_math: bool = True, activation_alpha: float = 1.0,
                     activation_beta: float = 0.0, *, residual: Optional[torch.Tensor] = None) -> None:
    """One MegaMoE layer call for this rank: reads the staged inputs of ``sym_buffer`` (first ``y.size(0)`` tokens),
    writes ``y``.  Launches on the current stream and never synchronises (the host-driven NCCL transport aside).

    ``residual`` (not in the reference's signature; keyword only): BF16 ``(M, H)`` added to the layer output inside the
    combine pass, ``y = bf16(bf16(layer output) + residual)`` -- bit for bit what the engine's separate addition after the
    layer leaves; it may be ``y`` itself."""
    stats = cumulative_local_expert_recv_stats
    tensors = (l1_weights[0], l1_weights[1], l2_weights[0], l2_weights[1],
               shared_l1_weights[0] if shared_l1_weights is not None else None,
               shared_l1_weights[1] if shared_l1_weights is not None else None,
               shared_l2_weights[0] if shared_l2_weights is not None else None,
               shared_l2_weights[1] if shared_l2_weights is not None else None, stats)
    rec = getattr(sym_buffer, "_call_record", None)
    m = y.size(0)
    if (rec is None or not rec.matches(tensors) or tuple(recipe) != (1, 1, 32) or activation != "swiglu"
            or activation_alpha != 1.0 or activation_beta != 0.0):
        rec = _validate(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights, shared_l2_weights, stats, recipe,
                        activation, activation_clamp, fast_math, activation_alpha, activation_beta, tensors)
        sym_buffer._call_record = rec
    else:
        # the record vouches for everything but the output tensor and the clamp
        assert y.dim() == 2 and y.size(1) == sym_buffer.hidden and y.dtype == torch.bfloat16 and y.is_contiguous(), \
            "y must be contiguous BF16 (M, H)"
        assert y.is_cuda and y.data_ptr() % 16 == 0, "y must be a 16-byte aligned CUDA tensor"
        assert m <= sym_buffer.num_max_tokens_per_rank, "num_tokens must be <= num_max_tokens_per_rank"
        assert activation_clamp is None or activation_clamp > 0, "activation_clamp must be positive"
    if residual is not None:
        assert residual.shape == y.shape and residual.dtype == torch.bfloat16 and residual.is_contiguous(), \
            "residual must be contiguous BF16 (M, H)"
        assert residual.device == y.device and residual.data_ptr() % 16 == 0, "residual must be a 16-byte aligned tensor on y's device"
    ko = _kernel_options
    key = (activation_clamp, bool(fast_math), _engine, ko.timeout_ms)
    if rec.options_key != key:
        rec.options = _native.MmoeOptions(float(activation_clamp) if activation_clamp is not None else math.inf,
                                          1 if fast_math else 0, _engine, ko.timeout_ms)
        rec.options_key = key
    capturing = torch.cuda.is_current_stream_capturing()
    if not rec.variants_ready and _engine == _native.ENGINE_TENSOR_CORE and not capturing:
        precompile_mega_moe_variants(sym_buffer.num_ranks, sym_buffer.num_experts, sym_buffer.num_max_tokens_per_rank,
                                     sym_buffer.num_topk, sym_buffer.hidden, sym_buffer.intermediate_hidden,
                                     sym_buffer.num_shared_experts)
        rec.variants_ready = True
    poll = None
    if ko.status_poll_interval > 0 and not capturing:
        poll = getattr(sym_buffer, "_status_poll", None)
        if poll is None:
            poll = sym_buffer._status_poll = _StatusPoll(sym_buffer)
        poll.before_call(sym_buffer)
    lib = _native.load()
    bm = get_block_m_for_mega_moe(sym_buffer.num_ranks, sym_buffer.num_experts, sym_buffer.num_max_tokens_per_rank, m,
                                  sym_buffer.num_topk, sym_buffer.mma_type)
    rec.options.residual = residual.data_ptr() if residual is not None and m > 0 else None
    res_ptr = rec.options.residual
    w, opts = ctypes.byref(rec.weights), ctypes.byref(rec.options)
    stats_ptr = stats.data_ptr() if stats is not None else None
    stream = torch.cuda.current_stream(y.device).cuda_stream
    ws = sym_buffer.base_ptr
    g = ctypes.byref(sym_buffer.geo)
    if sym_buffer.num_ranks == 1:
        _native.check(lib.mmoe_forward(g, ws, w, opts, y.data_ptr(), m, bm, stats_ptr, stream))
    elif rec.peers is not None and ko.ep_transport == "peer":
        # device-side exchange: no host round trip, capturable in a CUDA graph
        peers = rec.peers
        if ko.fuse_return:
            _native.check(lib.mmoe_forward_ep(g, ws, peers, w, opts, y.data_ptr(), m, bm, stats_ptr, stream))
        else:
            _native.check(lib.mmoe_dispatch_count(g, ws, m, stream))
            _native.check(lib.mmoe_ep_dispatch(g, ws, peers, m, opts, stream))
            _native.check(lib.mmoe_dispatch_place(g, ws, m, bm, stats_ptr, stream))
            _native.check(lib.mmoe_experts(g, ws, w, opts, m, bm, stream))
            _native.check(lib.mmoe_ep_return(g, ws, peers, opts, stream))
            _native.check(lib.mmoe_combine_residual(g, ws, y.data_ptr(), res_ptr, m, stream))
    else:
        group = sym_buffer.group
        _native.check(lib.mmoe_dispatch_count(g, ws, m, stream))
        _native.check(lib.mmoe_dispatch_pack(g, ws, m, stream))
        send_splits, recv_splits = exchange_counts(group, sym_buffer.send_count, sym_buffer.recv_count)
        exchange_rows(group, sym_buffer.recv_x, sym_buffer.send_x, recv_splits, send_splits)
        exchange_rows(group, sym_buffer.recv_sf, sym_buffer.send_sf, recv_splits, send_splits)
        exchange_rows(group, sym_buffer.recv_w, sym_buffer.send_w, recv_splits, send_splits)
        _native.check(lib.mmoe_dispatch_place(g, ws, m, bm, stats_ptr, stream))
        _native.check(lib.mmoe_experts(g, ws, w, opts, m, bm, stream))
        exchange_rows(group, sym_buffer.ret_recv, sym_buffer.ret, send_splits, recv_splits)
        _native.check(lib.mmoe_combine_residual(g, ws, y.data_ptr(), res_ptr, m, stream))
    if poll is not None:
        poll.after_call(sym_buffer, ko.status_poll_interval)


def read_status(sym_buffer) -> None:
    """Synchronise, read the device status words of the buffer and clear them; raises ``RuntimeError`` if a bounded
    device-side wait expired in any call since the last read (the output of that call is not valid) and
    ``AssertionError`` if the dispatch saw expert ids >= ``num_experts`` (they were treated as masked).  After the read
    the buffer reports healthy again.  Eager calls also watch the words without blocking, see
    ``KernelOptions.status_poll_interval``."""
    words = (ctypes.c_int32 * 8)()
    stream = torch.cuda.current_stream(sym_buffer.device).cuda_stream
    _native.check(_native.load().mmoe_read_status(ctypes.byref(sym_buffer.geo), sym_buffer.base_ptr, words, stream))
