"""The per-rank workspace of the MegaMoE layer (``SymmBuffer``) and its typed views.

Mirrors ``backend/workspace.py`` of the reference: the attributes a serving engine writes or reads are the same
(``x``, ``x_sf``, ``topk_idx``, ``topk_weights``, ``shared_l1_acts_sf`` and the *aligned* ``num_max_tokens_per_rank``,
``workspace.py:72-76``), the token capacity is rounded up to 1920 (``workspace.py:92-95``), the buffer is zeroed and the
group synchronised once at creation (``workspace.py:129-131``).  The regions behind the engine-facing views belong to
the B200 kernels and are laid out by the C library (``mmoe_layout``).  At EP > 1 the buffer is a symmetric allocation
(``torch.distributed._symmetric_memory``, as in the reference, ``workspace.py:125-128``): every rank holds every peer's
base pointer and the exchange kernels store counts and rows straight into the peers' ``recv_*`` / ``ret_recv`` regions
over NVLink (plain peer stores: no multicast object is bound to the allocation).  When symmetric memory cannot be set up
on ANY rank, every rank falls back together to ordinary device memory and the host-driven NCCL all-to-allv.
"""

from __future__ import annotations

import warnings
from typing import Optional, Union

import torch

from . import _native
from .heuristics import TOKEN_ALIGNMENT, align

_SUPPORTED_ACTIVATIONS = ("swiglu",)


def everyone_succeeded(group, ok: bool, device) -> bool:
    """True only if ``ok`` is true on every rank of ``group`` (a MIN all-reduce of one flag): the choice between the
    peer-memory exchange and the NCCL one must come out the same on all ranks.  A group that cannot reduce (a test
    double) keeps this rank's own outcome."""
    try:
        import torch.distributed as dist

        if isinstance(group, dist.ProcessGroup):
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            return bool(flag.item())
    except Exception:  # noqa: BLE001
        pass
    return ok


class SymmBuffer:
    """Workspace of one (group, geometry).  Created through :func:`get_symm_buffer_for_mega_moe`."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, num_shared_experts: int = 0, mma_type: str = "fp8xfp4",
                 activation: str = "swiglu", device: Optional[torch.device] = None):
        assert activation in _SUPPORTED_ACTIVATIONS, f"Activation must be one of {_SUPPORTED_ACTIVATIONS}, got `{activation}`"
        assert mma_type == "fp8xfp4", f"unsupported mma_type {mma_type!r}"
        self.group = group
        self.num_experts = num_experts
        self.num_max_tokens_per_rank = align(num_max_tokens_per_rank, TOKEN_ALIGNMENT)
        self.num_topk = num_topk
        self.hidden = hidden
        self.intermediate_hidden = intermediate_hidden
        self.num_shared_experts = num_shared_experts
        self.mma_type = mma_type
        self.activation = activation
        self.geo = _native.MmoeGeometry(group.size(), group.rank(), num_experts, num_topk, hidden, intermediate_hidden,
                                        num_shared_experts, self.num_max_tokens_per_rank)
        self.layout = _native.layout_of(self.geo)
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.peer_ptrs = None          # EP > 1: every rank's buffer mapped into this process (symmetric allocation)
        self.handle = None
        if group.size() > 1 and device.type == "cuda":
            self._allocate_symmetric(group, device)
        if getattr(self, "buffer", None) is None:
            self.buffer = torch.empty(self.layout.total_bytes, dtype=torch.int8, device=device)
        assert self.buffer.data_ptr() % 1024 == 0
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        if group.size() > 1:
            work = group.barrier()
            if hasattr(work, "wait"):
                work.wait()
        torch.cuda.synchronize(device)
        self._build_views()

    def _allocate_symmetric(self, group, device) -> None:
        """Symmetric allocation + rendezvous; the outcome is agreed on by the whole group, so that no rank runs the peer
        transport while another runs the NCCL one."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer stores only
        problem = None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            self.buffer = symm_mem.empty(self.layout.total_bytes, dtype=torch.int8, device=device)
            self.handle = symm_mem.rendezvous(self.buffer, group)
            self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
            assert self.peer_ptrs[group.rank()] == self.buffer.data_ptr()
        except Exception as exc:  # noqa: BLE001 - no symmetric memory: the host-driven NCCL exchange still works
            problem = f"{type(exc).__name__}: {exc}"
        everyone_ok = everyone_succeeded(group, problem is None, device)
        if not everyone_ok:
            warnings.warn(f"symmetric memory is unavailable ({problem or 'on another rank'}); using the NCCL exchange")
            self.peer_ptrs = None
            self.handle = None
            self.buffer = None

    # ---------------------------------------------------------------------------------------------------- views
    def _view(self, offset: int, shape, dtype, strides=None) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        flat = self.buffer[offset:offset + nbytes].view(dtype)
        return flat.view(*shape) if strides is None else torch.as_strided(flat, shape, strides)

    def _build_views(self) -> None:
        lay, t, h, k = self.layout, self.num_max_tokens_per_rank, self.hidden, self.num_topk
        inter = self.intermediate_hidden
        self.x = self._view(lay.x, (t, h), torch.float8_e4m3fn)
        self.x_sf = self._view(lay.x_sf, (t, h // 128), torch.int32)
        self.topk_idx = self._view(lay.topk_idx, (t, k), torch.int64)
        self.topk_weights = self._view(lay.topk_weights, (t, k), torch.float32)
        self.shared_l1_acts = self.x
        self.shared_l1_acts_sf = None
        self.shared_l2_acts = None
        self.shared_l2_acts_sf = None
        if self.num_shared_experts > 0:
            rows = lay.shared_sf_rows
            self.shared_l1_acts_sf = self._view(lay.shared_x_sf, (rows, h // 128), torch.int32, (1, rows))
            self.shared_l2_acts = self._view(lay.shared_act_x, (t, inter), torch.float8_e4m3fn)
            self.shared_l2_acts_sf = self._view(lay.shared_act_sf, (rows, inter // 128), torch.int32, (1, rows))
        e, r = self.num_experts, self.num_ranks
        self.send_count = self._view(lay.send_count, (e,), torch.int32)
        self.send_offset = self._view(lay.send_offset, (e + 1,), torch.int32)
        self.route_pos = self._view(lay.route_pos, (t, k), torch.int32)
        self.sorted_route = self._view(lay.sorted_route, (t * k,), torch.int32)
        self.recv_count = self._view(lay.recv_count, (r, e // r), torch.int32)
        self.l1_acts = self._view(lay.pool_x, (lay.pool_rows, h), torch.float8_e4m3fn)
        self.l1_acts_sf = self._view(lay.pool_sf, (lay.pool_sf_rows, h // 128), torch.int32, (1, lay.pool_sf_rows))
        self.l1_topk_weights = self._view(lay.pool_w, (lay.pool_rows,), torch.float32)
        self.pool_dst = self._view(lay.pool_dst, (lay.pool_rows,), torch.int32)
        self.l2_acts = self._view(lay.act_x, (lay.pool_rows, inter), torch.float8_e4m3fn)
        self.l2_acts_sf = self._view(lay.act_sf, (lay.pool_sf_rows, inter // 128), torch.int32, (1, lay.pool_sf_rows))
        self.ret = self._view(lay.ret, (r * lay.max_routes, h), torch.bfloat16)
        self.status = self._view(lay.status, (8,), torch.int32)
        self.plan_words = self._view(lay.plan, (16,), torch.int32)
        if r > 1:
            m = lay.max_routes
            self.send_x = self._view(lay.send_x, (m, h), torch.float8_e4m3fn)
            self.send_sf = self._view(lay.send_sf, (m, h // 128), torch.int32)
            self.send_w = self._view(lay.send_w, (m,), torch.float32)
            self.recv_x = self._view(lay.recv_x, (r * m, h), torch.float8_e4m3fn)
            self.recv_sf = self._view(lay.recv_sf, (r * m, h // 128), torch.int32)
            self.recv_w = self._view(lay.recv_w, (r * m,), torch.float32)
            self.ret_recv = self._view(lay.ret_recv, (m, h), torch.bfloat16)

    # ---------------------------------------------------------------------------------------------------- plan readers
    def plan_tables(self):
        """Host copies of the dispatch plan of the last call: ``(header dict, expert_total, expert_block_off)``."""
        e_l, r = self.num_experts // self.num_ranks, self.num_ranks
        words = 16 + e_l + 2 * (e_l + 1)
        raw = self._view(self.layout.plan, (words,), torch.int32).cpu()
        hdr = dict(num_routed_tiles=int(raw[0]), num_shared_tiles=int(raw[1]), num_pool_blocks=int(raw[2]),
                   total_recv=int(raw[3]), block_m=int(raw[4]), num_tokens=int(raw[5]))
        total = raw[16:16 + e_l].clone()
        block_off = raw[16 + e_l:16 + e_l + e_l + 1].clone()
        return hdr, total, block_off

    @property
    def rank(self) -> int:
        return self.group.rank()

    @property
    def num_ranks(self) -> int:
        return self.group.size()

    @property
    def base_ptr(self) -> int:
        return self.buffer.data_ptr()

    def destroy(self) -> None:
        if getattr(self, "buffer", None) is not None:
            torch.cuda.synchronize(self.device)
        self.buffer = None
        self.group = None
        for name in ("x", "x_sf", "topk_idx", "topk_weights", "shared_l1_acts", "shared_l1_acts_sf", "shared_l2_acts",
                     "shared_l2_acts_sf", "l1_acts", "l1_acts_sf", "l2_acts", "l2_acts_sf"):
            setattr(self, name, None)


class SingleRankGroup:
    """Stand-in process group for EP = 1 callers that have no ``torch.distributed`` group."""

    def size(self) -> int:
        return 1

    def rank(self) -> int:
        return 0

    def barrier(self) -> None:
        return None


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                                 intermediate_hidden: int, num_shared_experts: int = 0,
                                 use_fp8_dispatch: Union[bool, None] = None, mma_type: str = "fp8xfp4",
                                 activation: str = "swiglu") -> SymmBuffer:
    if use_fp8_dispatch is not None:
        assert use_fp8_dispatch == (mma_type.split("x")[0] == "fp8")
        warnings.warn("`use_fp8_dispatch` will be deprecated in the future, please use `mma_type`", DeprecationWarning,
                      stacklevel=3)
    return SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                      num_shared_experts, mma_type=mma_type, activation=activation)
