"""`mmoe_route_order_noalloc`: the route-ordering step for callers that cannot let the library allocate device memory
(a serving process whose own pool already owns all free HBM, or a decode loop that cannot take the device-wide
synchronisation an allocation implies).  Its scratch is a fixed array inside the library image, so the test checks that
two calls in a row -- the second one smaller, so stale cells of the first are still in the array -- give exactly what
the workspace-based entry point `mmoe_dispatch_count` gives on the same routing.  Collected last on purpose: a run that
stops at the first failure has then already run every other test."""

import ctypes

import pytest
import torch

import helpers as H
from helpers import O

pytestmark = pytest.mark.gpu


def _reference_order(buf, ids):
    """Route ordering through the existing, workspace-based entry point."""
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    m, k = ids.shape
    buf.topk_idx[:m].copy_(ids)
    _native.check(lib.mmoe_dispatch_count(ctypes.byref(buf.geo), buf.base_ptr, m, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    e = buf.num_experts
    return (buf.send_count.clone(), buf.send_offset.clone(), buf.route_pos[:m].reshape(-1).clone(),
            buf.sorted_route[: int(buf.send_offset[e])].clone())


def _noalloc_order(ids, e):
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    m, k = ids.shape
    dev = ids.device
    send_count = torch.full((e,), -7, dtype=torch.int32, device=dev)
    send_offset = torch.full((e + 1,), -7, dtype=torch.int32, device=dev)
    route_pos = torch.full((m * k,), -7, dtype=torch.int32, device=dev)
    sorted_route = torch.full((m * k,), -7, dtype=torch.int32, device=dev)
    _native.check(lib.mmoe_route_order_noalloc(ids.data_ptr(), m, k, e, send_count.data_ptr(), send_offset.data_ptr(),
                                               route_pos.data_ptr(), sorted_route.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return send_count, send_offset, route_pos, sorted_route[: int(send_offset[e])]


def test_noalloc_route_order_matches_workspace_entry_point_twice():
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    e, k = 384, 6
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), e, 3840, k, 512, 256, 0)
    cases = [O.make_routing(3000, e, k, seed=5, zipf_s=1.2, mask_frac=0.05, hot=2)[0],
             O.make_routing(37, e, k, seed=6, mask_frac=0.3)[0]]          # second call: smaller, stale scratch behind it
    for ids in cases:
        ids = ids.cuda().contiguous()
        want = _reference_order(buf, ids)
        got = _noalloc_order(ids, e)
        for a, b, name in zip(got, want, ("send_count", "send_offset", "route_pos", "sorted_route")):
            assert torch.equal(a, b), name                                # integer work: bit-exact
        plan = O.dispatch_plan([ids.cpu()], e, 0, 16)
        assert torch.equal(got[0].cpu().long(), plan.recv_total)          # and equal to the oracle's per-expert counts


def test_noalloc_route_order_rejects_sizes_beyond_the_built_in_scratch():
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    z = torch.zeros(8, dtype=torch.int64, device="cuda")
    out = torch.zeros(1024, dtype=torch.int32, device="cuda")
    args = (out.data_ptr(), out.data_ptr(), out.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    for m, k, e in ((4097, 1, 8), (1, 1, 513), (1, 32, 8)):
        with pytest.raises(AssertionError):
            _native.check(lib.mmoe_route_order_noalloc(z.data_ptr(), m, k, e, *args))
