"""GPU parity of the integer / byte work: the input quantiser against the reference's golden vectors (bit-exact), the
dispatch counts, pool-block offsets and per-expert route multisets against the oracle (bit-exact), and the cumulative
receive statistics.  Everything goes through the C ABI (ctypes) of libmmoe_b200.so."""

import os

import numpy as np
import pytest
import torch

import helpers as H
from helpers import O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(H.ROOT, "tests", "golden")


def _buffer(num_experts, k, hidden, inter, shared=1, t=1920):
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    return api.get_symm_buffer_for_mega_moe(SingleRankGroup(), num_experts, t, k, hidden, inter, shared)


@pytest.mark.parametrize("bm", [16, 32, 64, 128, 192, 240])
def test_staging_matches_reference_golden(bm):
    from vllm_plugin_b200 import api
    g = np.load(os.path.join(GOLD, "staging.npz"))
    x = torch.from_numpy(g["x_bits"]).view(torch.bfloat16)
    ids = torch.from_numpy(g["ids"])
    w = torch.from_numpy(g["w"])
    pad = torch.from_numpy(g["pad"])
    m, h = x.shape
    buf = _buffer(32, ids.shape[1], h, 256)
    got_bm = api.stage_inputs_for_mega_moe(buf, x.cuda(), ids.to(torch.int32).cuda(), w.cuda(), is_padding=pad.cuda(), block_m=bm)
    assert got_bm == bm
    torch.cuda.synchronize()
    assert np.array_equal(buf.x[:m].cpu().view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(buf.x_sf[:m].cpu().numpy(), g["sf"])
    assert np.array_equal(buf.topk_idx[:m].cpu().numpy(), g["ids_out"])
    assert np.array_equal(buf.topk_weights[:m].cpu().numpy(), g["w_out"])
    gold_sh = g[f"shared_sf_{bm}"]
    assert np.array_equal(buf.shared_l1_acts_sf[: gold_sh.shape[0]].cpu().numpy(), gold_sh)
    assert int(buf.shared_l1_acts_sf[gold_sh.shape[0]:].abs().sum()) == 0       # rows of other tokens stay untouched


@pytest.mark.parametrize("m", [1, 7, 64, 1000, 1920])
def test_staging_matches_oracle_random(m):
    from vllm_plugin_b200 import api
    h, k = 1024, 6
    g = torch.Generator().manual_seed(m)
    x = (torch.randn((m, h), generator=g) * torch.exp(torch.randn((m, 1), generator=g) * 3)).to(torch.bfloat16)
    ids, w = O.make_routing(m, 32, k, m)
    buf = _buffer(32, k, h, 256)
    bm = api.stage_inputs_for_mega_moe(buf, x.cuda(), ids.cuda(), w.cuda())
    assert bm == O.get_block_m(1, 32, m, k)
    q, sf, io, wo, sh = O.stage_inputs(x, ids, w, None, buf.layout.shared_sf_rows, bm)
    assert torch.equal(buf.x[:m].cpu().view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(buf.x_sf[:m].cpu(), sf)
    assert torch.equal(buf.shared_l1_acts_sf.cpu(), sh)
    assert torch.equal(buf.topk_idx[:m].cpu(), io) and torch.equal(buf.topk_weights[:m].cpu(), wo)


def test_staging_rejects_malformed_inputs():
    from vllm_plugin_b200 import api
    buf = _buffer(32, 6, 512, 256)
    x = torch.zeros((4, 512), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((4, 6), dtype=torch.int64, device="cuda")
    w = torch.zeros((4, 6), device="cuda")
    with pytest.raises(ValueError):
        api.stage_inputs_for_mega_moe(buf, x[:, :384], ids, w)
    with pytest.raises(ValueError):
        api.stage_inputs_for_mega_moe(buf, x, ids, w[:, :5])
    with pytest.raises(AssertionError):
        api.stage_inputs_for_mega_moe(buf, torch.zeros((1921, 512), dtype=torch.bfloat16, device="cuda"),
                                      torch.zeros((1921, 6), dtype=torch.int64, device="cuda"), torch.zeros((1921, 6), device="cuda"))
    assert api.stage_inputs_for_mega_moe(buf, x[:0], ids[:0], w[:0]) == 16       # empty call: nothing launched


def _dispatch(buf, ids, w, block_m, stats=None):
    import ctypes
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    m, k = ids.shape
    buf.topk_idx[:m].copy_(ids)
    buf.topk_weights[:m].copy_(w)
    stream = torch.cuda.current_stream().cuda_stream
    _native.check(lib.mmoe_dispatch_count(ctypes.byref(buf.geo), buf.base_ptr, m, stream))
    _native.check(lib.mmoe_dispatch_place(ctypes.byref(buf.geo), buf.base_ptr, m, block_m,
                                          None if stats is None else stats.data_ptr(), stream))
    torch.cuda.synchronize()


@pytest.mark.parametrize("m,e,k,bm,kw", [
    (1, 32, 6, 16, {}), (33, 8, 2, 16, {}), (200, 32, 6, 32, dict(zipf_s=1.2, mask_frac=0.05, hot=2)),
    (640, 16, 4, 128, dict(zipf_s=1.2)), (700, 8, 2, 240, {}), (1920, 384, 6, 32, dict(mask_frac=0.05)),
    (5, 32, 6, 64, dict(mask_frac=1.0)),
])
def test_dispatch_counts_offsets_and_multisets(m, e, k, bm, kw):
    ids, w = O.make_routing(m, e, k, seed=m + e, **kw)
    buf = _buffer(e, k, 512, 256)
    stats = torch.full((e,), 7, dtype=torch.int32, device="cuda")
    _dispatch(buf, ids.cuda(), w.cuda(), bm, stats)
    plan = O.dispatch_plan([ids], e, 0, bm)
    hdr, total, block_off = buf.plan_tables()
    assert torch.equal(buf.send_count.cpu().long(), plan.recv_total)                  # per-expert counts
    assert torch.equal(buf.recv_count.cpu().long(), plan.recv_count)                  # per-(source, expert) counts
    assert torch.equal(total.long(), plan.recv_total)
    assert torch.equal(block_off.long(), plan.pool_block_offset)                      # BLOCK_M-aligned expert offsets
    assert hdr["total_recv"] == int(plan.recv_total.sum()) and hdr["num_pool_blocks"] == int(plan.pool_block_offset[-1])
    assert torch.equal(stats.cpu().long(), plan.recv_total + 7)                       # cumulative statistics
    # pool layout: rows of expert e start at block_off[e]*bm; their (token, slot) multiset equals the oracle's and,
    # beyond the reference's contract, the order is the fixed (source, token, slot) order
    pos = buf.route_pos[:m].cpu()
    dst = buf.pool_dst.cpu()
    pw = buf.l1_topk_weights.cpu()
    inv = {int(p): (t, s) for t in range(m) for s in range(k) if (p := int(pos[t, s])) >= 0}
    assert len(inv) == int(plan.recv_total.sum())
    for ex in range(e):
        base = int(block_off[ex]) * bm
        got = [inv[int(dst[base + j])] for j in range(int(plan.recv_total[ex]))]
        assert got == [(t, s) for (_, t, s) in plan.routes[ex]]
        for j, (t, s) in enumerate(got):
            assert float(pw[base + j]) == float(w[t, s])
    masked = ids < 0
    assert bool((pos[masked] == -1).all())


def test_dispatch_rejects_out_of_range_expert():
    from vllm_plugin_b200.backend.frontend import read_status
    ids = torch.tensor([[0, 9]], dtype=torch.int64)
    buf = _buffer(8, 2, 512, 256)
    _dispatch(buf, ids.cuda(), torch.ones((1, 2)).cuda(), 16)
    with pytest.raises(AssertionError):
        read_status(buf)


@pytest.mark.parametrize("m,logical,k,replicas", [(1, 384, 6, 0), (37, 384, 6, 8), (500, 128, 3, 16), (260, 64, 8, 0)])
def test_router_fused_in_front_of_the_quantiser(m, logical, k, replicas):
    """Top-k by logit (indices bit-exact against torch.topk; Gaussian logits have no ties), softmax over the selected
    logits (within float32 rounding), the replica choice (token + slot) % copies, and a staged result identical to
    staging the same ids and weights through the ordinary entry point."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    physical = logical + replicas
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), physical, 1920, k, 512, 256, 1)
    g = torch.Generator().manual_seed(m)
    logits = torch.randn((m, logical), generator=g)
    hid = O.make_hidden(m, 512, 3).cuda()
    replica_map = None
    ids_ref = torch.topk(logits, k, dim=1).indices
    w_ref = torch.softmax(torch.topk(logits, k, dim=1).values, dim=1)
    if replicas:
        count = torch.ones(logical, dtype=torch.int32)
        slots = torch.arange(logical, dtype=torch.int32).view(-1, 1).repeat(1, 2)
        hot = torch.randperm(logical, generator=g)[:replicas]
        count[hot] = 2
        slots[hot, 1] = torch.arange(logical, physical, dtype=torch.int32)
        replica_map = (count.cuda(), slots.cuda())
        tok = torch.arange(m).view(-1, 1)
        slot = torch.arange(k).view(1, -1)
        pick = (tok + slot) % count[ids_ref].long()
        ids_ref = slots[ids_ref, pick].long()
    pad = torch.zeros(m, dtype=torch.bool)
    if m > 3:
        pad[2] = True
    bm = api.route_and_stage_inputs_for_mega_moe(buf, hid, logits.cuda(), replica_map=replica_map, is_padding=pad.cuda())
    torch.cuda.synchronize()
    got_ids, got_w = buf.topk_idx[:m].cpu(), buf.topk_weights[:m].cpu()
    want_ids = torch.where(pad.view(-1, 1), torch.full_like(ids_ref, -1), ids_ref)
    assert torch.equal(got_ids, want_ids)
    assert torch.allclose(got_w[~pad], w_ref[~pad], rtol=2e-6, atol=1e-7) and float(got_w[pad].abs().sum()) == 0.0
    staged = (buf.x[:m].view(torch.uint8).clone(), buf.x_sf[:m].clone(), buf.shared_l1_acts_sf.clone())
    assert api.stage_inputs_for_mega_moe(buf, hid, got_ids.cuda(), got_w.cuda(), is_padding=pad.cuda()) == bm
    torch.cuda.synchronize()
    assert torch.equal(buf.x[:m].view(torch.uint8), staged[0]) and torch.equal(buf.x_sf[:m], staged[1])
    assert torch.equal(buf.shared_l1_acts_sf, staged[2])
    assert torch.equal(buf.topk_idx[:m].cpu(), want_ids) and torch.equal(buf.topk_weights[:m].cpu(), got_w)


@pytest.mark.parametrize("m,h,scale", [(1, 512, 1.0), (77, 5120, 448.0 * 6.0 / 5.0), (300, 1024, 37.5)])
def test_nvfp4_staging_matches_the_oracle(m, h, scale):
    """Packed E2M1 bytes and E4M3 block scales bit-exact against the oracle's two-level NVFP4 quantiser, including
    all-zero blocks, values that saturate the E2M1 grid and exact ties."""
    from vllm_plugin_b200 import api
    x = O.make_hidden(m, h, 5).float()
    x[0, :16] = 0.0                                                   # a zero block: scale 0, values 0
    if m > 1:
        x[1, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 4) * (6.0 / scale)   # ties on the grid
        x[1, 32:48] = 1e4                                             # saturates the block scale
    x = x.to(torch.bfloat16)
    q, sf = api.prepare_megamoe_nvfp4_inputs(x.cuda(), scale)
    torch.cuda.synchronize()
    q_ref, sf_ref = O.quantize_nvfp4(x, scale)
    assert torch.equal(sf.cpu(), sf_ref)
    assert torch.equal(q.cpu(), q_ref)
