"""Failure detection without faulting a GPU: a bounded device-side wait that nobody satisfies must run out, leave a
status record the host can read, and leave the context usable.  Here a two-rank geometry is driven by ONE process: the
"peer" workspace is a second local buffer, so the peer's arrival flag is never written."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class _LoneRankOfTwo:
    def size(self):
        return 2

    def rank(self):
        return 0

    def barrier(self):
        return None


def test_peer_wait_times_out_and_reports_status():
    from vllm_plugin_b200.backend import _native
    from vllm_plugin_b200.backend.workspace import SymmBuffer
    lib = _native.load()
    mine = SymmBuffer(_LoneRankOfTwo(), 16, 1920, 4, 512, 256, 1)          # plain device memory: no rendezvous happens
    other = torch.zeros(mine.layout.total_bytes, dtype=torch.int8, device="cuda")
    ids = torch.randint(0, 16, (8, 4), dtype=torch.int64, device="cuda")
    mine.topk_idx[:8].copy_(ids)
    stream = torch.cuda.current_stream().cuda_stream
    geo = ctypes.byref(mine.geo)
    _native.check(lib.mmoe_dispatch_count(geo, mine.base_ptr, 8, stream))
    peers = (ctypes.c_void_p * 2)(mine.base_ptr, other.data_ptr())
    opts = _native.MmoeOptions(10.0, 1, 0, 300, 0)                         # 300 ms budget for every device-side wait
    _native.check(lib.mmoe_ep_dispatch(geo, mine.base_ptr, peers, 8, ctypes.byref(opts), stream))
    words = (ctypes.c_int32 * 8)()
    code = lib.mmoe_read_status(geo, mine.base_ptr, words, stream)
    assert code == _native.MMOE_ERR_DEVICE_TIMEOUT
    assert words[0] == 1 and words[1] in (10, 11) and words[2] == 1       # barrier kernel, missing rank = 1
    with pytest.raises(RuntimeError, match="device-side wait expired"):
        _native.check(code)
    # the context is still healthy: an ordinary single-rank call right after works
    import helpers as H
    from helpers import O
    layer = H.make_layer(512, 256, 8, 2, True, seed=1)
    hid = O.make_hidden(5, 512, 1)
    rid, w = O.make_routing(5, 8, 2, 2)
    y, _ = H.run_layer(layer, hid, rid, w)
    assert O.parity_metrics(y.cpu(), H.oracle_layer(layer, hid, rid, w))["rel_l2"] <= 1e-3
    # reading the status cleared it: the buffer that timed out reports healthy again
    assert lib.mmoe_read_status(geo, mine.base_ptr, words, stream) == _native.MMOE_OK and words[0] == 0


def test_eager_calls_notice_a_bad_status_without_blocking():
    """The production path never calls ``read_status``: eager calls copy the status words to pinned memory behind the
    launch (here after every call) and a later call raises.  The condition used is an expert id >= num_experts, which the
    dispatch counts and treats as masked; after the report the buffer is healthy again."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    import helpers as H
    from helpers import O
    layer = H.make_layer(512, 256, 8, 2, True, seed=3)
    l1, l2, sl1, sl2 = H.kernel_weights(layer, "cuda")
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), 8, 1920, 2, 512, 256, 1)
    hid = O.make_hidden(6, 512, 1).cuda()
    ids, w = O.make_routing(6, 8, 2, 2)
    bad = ids.clone()
    bad[0, 0] = 99
    y = torch.empty((6, 512), dtype=torch.bfloat16, device="cuda")
    api.set_kernel_options(status_poll_interval=1)
    try:
        def call(which):
            api.stage_inputs_for_mega_moe(buf, hid, which.cuda(), w.cuda())
            api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, activation_clamp=10.0)
        call(bad)
        torch.cuda.synchronize()
        with pytest.raises(AssertionError, match="expert ids"):
            for _ in range(3):                 # the copy was queued behind the first call; one of the next calls sees it
                call(ids)
                torch.cuda.synchronize()
        for _ in range(3):                     # re-armed: healthy calls stay quiet
            call(ids)
            torch.cuda.synchronize()
        api.read_status(buf)
    finally:
        api.set_kernel_options(status_poll_interval=32)
    ref = H.oracle_layer(layer, hid.cpu(), ids, w)
    assert O.parity_metrics(y.cpu(), ref)["rel_l2"] <= 1e-3


def test_host_side_argument_errors_map_to_the_reference_exception_classes():
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    import helpers as H
    layer = H.make_layer(512, 256, 8, 2, True, seed=2)
    l1, l2, sl1, sl2 = H.kernel_weights(layer, "cuda")
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), 8, 1920, 2, 512, 256, 1)
    y = torch.empty((4, 512), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):
        api.fp8_fp4_mega_moe(y, l1, l2, buf, None, None)                  # buffer has a shared expert, none given
    with pytest.raises(AssertionError):
        api.fp8_fp4_mega_moe(y.float(), l1, l2, buf, sl1, sl2)            # y must be BF16
    with pytest.raises(AssertionError):
        api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, recipe=(1, 1, 128))
    with pytest.raises(NotImplementedError):
        api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, activation_alpha=1.702)
    with pytest.raises(AssertionError):
        api.fp8_fp4_mega_moe(y, (l1[0], l1[1].contiguous()), l2, buf, sl1, sl2)   # scales must be MN-major
