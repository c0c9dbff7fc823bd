"""Oracle parity at the benchmark's own sizes (H=5120, I=2304): every BLOCK_M variant and both grouped-GEMM kernel
families with 40-stage K loops, and the headline geometry with all 384 experts resident.  The oracle dequantises one
expert at a time and evaluates a seeded sample of tokens (a token's output does not depend on the rest of the call);
per-expert receive counts and pool-block offsets of the WHOLE call are compared bit for bit."""

import pytest
import torch

import helpers as H
from helpers import O
from test_gpu_layer import assert_parity

pytestmark = pytest.mark.gpu

HID, INTER = 5120, 2304


def _run(syn, buf, hid, ids, w, stats=None):
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.frontend import read_status
    y = torch.empty((hid.shape[0], HID), dtype=torch.bfloat16, device="cuda")
    api.stage_inputs_for_mega_moe(buf, hid, ids, w)
    api.fp8_fp4_mega_moe(y, syn.l1, syn.l2, buf, syn.shared_l1, syn.shared_l2, cumulative_local_expert_recv_stats=stats,
                         activation_clamp=10.0)
    read_status(buf)
    return y


def _check_counts(buf, ids, num_experts):
    hdr, total, block_off = buf.plan_tables()
    plan = O.dispatch_plan([ids.cpu()], num_experts, 0, hdr["block_m"])
    assert torch.equal(buf.send_count.cpu().long(), plan.recv_total), "per-expert receive counts"
    assert torch.equal(total.long(), plan.recv_total), "per-expert totals of the plan"
    assert torch.equal(block_off.long(), plan.pool_block_offset), "pool block offsets"
    return hdr["block_m"]


@pytest.fixture(scope="module")
def layer16():
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    from vllm_plugin_b200.testing import SyntheticLayer
    syn = SyntheticLayer(HID, INTER, 16, True, "cuda", seed=5)
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), 16, 1920, 6, HID, INTER, 1)
    return syn, buf


@pytest.mark.parametrize("bm,orientation", [(64, 1), (128, 1), (192, 1), (240, 1), (64, 2), (128, 2), (192, 2), (240, 2), (192, 3)])
def test_every_block_m_at_full_hidden_and_intermediate(layer16, bm, orientation):
    """16 resident experts, 640 tokens, top-6: Zipf(1.2) popularity, two experts at 4x the mean load, 5 % of the routes
    masked -- experts from a handful to several hundred rows, so every tile size of the variant occurs (80- and 112-row
    tiles of the weights-as-A kernels, 128-row tiles and the 64-row token box of the tokens-as-A kernels)."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.testing import make_hidden, make_routing
    syn, buf = layer16
    m = 640
    hid = make_hidden(m, HID, 11, "cuda")
    ids, w = make_routing(m, 16, 6, 12, "cuda", zipf_s=1.2, mask_frac=0.05, hot=2)
    api.set_kernel_options(block_m=bm, orientation=orientation)
    try:
        y = _run(syn, buf, hid, ids, w)
    finally:
        api.set_kernel_options(block_m=0, orientation=0)
    assert _check_counts(buf, ids, 16) == bm
    sample = torch.randperm(m, generator=torch.Generator().manual_seed(bm))[:48]
    ref = H.oracle_token_sample(hid, ids, w, sample, lambda e: H.synthetic_expert(syn, e), H.synthetic_shared(syn))
    H.log_parity(f"full H/I E=16 M=640 block_m={bm} orientation={orientation}", H.strict_metrics(y[sample.cuda()], ref))
    assert_parity(y[sample.cuda()], ref, f"block_m {bm} orientation {orientation}")


@pytest.fixture(scope="module")
def layer384():
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    from vllm_plugin_b200.testing import SyntheticLayer
    syn = SyntheticLayer(HID, INTER, 384, True, "cuda", seed=1)
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), 384, 3840, 6, HID, INTER, 1)
    return syn, buf


@pytest.mark.parametrize("m", [64, 1024, 3840])
def test_headline_geometry_against_the_oracle(layer384, m):
    """E=384 resident experts, top-6, one shared expert (the benchmark's headline geometry) at a decode, a mid and the
    headline token count: 64 sampled tokens against the oracle (about 240 experts dequantised one at a time), receive
    counts, totals, pool offsets and the cumulative statistics of the whole call bit-exact."""
    from vllm_plugin_b200.testing import make_hidden, make_routing
    syn, buf = layer384
    hid = make_hidden(m, HID, 21, "cuda")
    ids, w = make_routing(m, 384, 6, 22, "cuda")
    stats = torch.full((384,), 3, dtype=torch.int32, device="cuda")
    y = _run(syn, buf, hid, ids, w, stats)
    bm = _check_counts(buf, ids, 384)
    assert bm == O.get_block_m(1, 384, m, 6)
    assert torch.equal(stats.cpu().long() - 3, torch.bincount(ids.cpu().flatten(), minlength=384))
    sample = torch.randperm(m, generator=torch.Generator().manual_seed(m))[:64]
    ref = H.oracle_token_sample(hid, ids, w, sample, lambda e: H.synthetic_expert(syn, e), H.synthetic_shared(syn))
    H.log_parity(f"E=384 M={m} block_m={bm}", H.strict_metrics(y[sample.cuda()], ref))
    assert_parity(y[sample.cuda()], ref, f"E=384 M={m}")


@pytest.mark.parametrize("m,bm", [(1, 16), (8, 16), (21, 16), (100, 16), (30, 32), (128, 32)])
def test_small_call_path_equals_the_general_sequence(layer16, m, bm):
    """Calls of at most 128 tokens order the routes and build the plan in one block (which, up to 128 routes, also
    places the rows) and launch their kernels as a programmatic chain.  Every intermediate and the output must equal,
    bit for bit, what the general sequence leaves: three ordering passes, plan, placement, GEMMs, combine."""
    import ctypes
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import _native
    from vllm_plugin_b200.backend.frontend import _weights_struct, check_mega_moe_arguments, read_status
    from vllm_plugin_b200.testing import make_hidden, make_routing
    syn, buf = layer16
    hid = make_hidden(m, HID, 31 + m, "cuda")
    ids, w = make_routing(m, 16, 6, 32 + m, "cuda", zipf_s=1.2, mask_frac=0.05)
    api.set_kernel_options(block_m=bm, orientation=1)
    try:
        y_one = _run(syn, buf, hid, ids, w)
        pool_one = buf.l1_acts.view(torch.uint8).clone()
        act_one = buf.l2_acts.view(torch.uint8).clone()
        ret_one = buf.ret.view(torch.int16).clone()
        y = torch.empty_like(y_one)
        s13, s2 = check_mega_moe_arguments(y, syn.l1, syn.l2, buf, syn.shared_l1, syn.shared_l2, None, (1, 1, 32),
                                           "swiglu", 10.0, True, 1.0, 0.0)
        ws = _weights_struct(syn.l1, syn.l2, syn.shared_l1, syn.shared_l2, s13, s2)
        lib = _native.load()
        geo, base = ctypes.byref(buf.geo), buf.base_ptr
        sp = torch.cuda.current_stream().cuda_stream
        api.stage_inputs_for_mega_moe(buf, hid, ids, w, block_m=bm)
        _native.check(lib.mmoe_dispatch_count(geo, base, m, sp))
        _native.check(lib.mmoe_dispatch_place(geo, base, m, bm, None, sp))
        for mask in (1, 2):
            opts = _native.MmoeOptions(10.0, 1, 0, 2000, mask)
            _native.check(lib.mmoe_experts(geo, base, ctypes.byref(ws), ctypes.byref(opts), m, bm, sp))
        _native.check(lib.mmoe_combine(geo, base, y.data_ptr(), m, sp))
        read_status(buf)
    finally:
        api.set_kernel_options(block_m=0, orientation=0)
    # rows of the pool that hold no route are never written by either sequence: compare the regions whole
    assert torch.equal(buf.l1_acts.view(torch.uint8), pool_one), "placed rows"
    assert torch.equal(buf.l2_acts.view(torch.uint8), act_one), "SwiGLU output of the routed experts"
    assert torch.equal(buf.ret.view(torch.int16), ret_one), "expert output rows"
    assert torch.equal(y, y_one)
