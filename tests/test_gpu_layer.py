"""GPU parity of the whole layer against the CPU oracle on identical seeded inputs, through the package's public API
(which calls the C ABI).  Tolerance of the BF16 output: relative L2 <= 1e-3 and max_abs <= 2e-2; one BF16 ulp of the
reference is larger than 2e-2 wherever |y| >= 4, and a one-ulp disagreement is inherent to the FP32 summation order, so
the element-wise bound is max(2e-2, one BF16 ulp of the reference value)."""

import pytest
import torch

import helpers as H
from helpers import O

pytestmark = pytest.mark.gpu

REL_L2 = 1e-3
MAX_ABS = 2e-2


def assert_parity(y, ref, what=""):
    a, b = y.float().cpu(), ref.float()
    assert torch.isfinite(a).all(), what
    rel = float((a - b).norm() / b.norm().clamp(min=1e-30))
    ulp = torch.pow(2.0, torch.floor(torch.log2(b.abs().clamp(min=2.0 ** -126))) - 7)
    bound = torch.clamp(ulp, min=MAX_ABS)
    worst = float(((a - b).abs() - bound).max())
    assert rel <= REL_L2, f"{what}: rel_l2 {rel}"
    assert worst <= 0, f"{what}: an element exceeds max(2e-2, 1 ulp) by {worst}"


SMALL = dict(hidden=512, inter=256, num_experts=8, num_topk=2)


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("m", [1, 5, 33, 130])
@pytest.mark.parametrize("shared", [True, False])
def test_small_layer_matches_oracle(engine, m, shared):
    layer = H.make_layer(shared=shared, seed=m, **SMALL)
    hid = O.make_hidden(m, layer.hidden, 1)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 2, mask_frac=0.1 if m > 1 else 0.0)
    y, buf = H.run_layer(layer, hid, ids, w, engine=engine)
    assert_parity(y, H.oracle_layer(layer, hid, ids, w), f"engine {engine} m {m}")
    # the dispatch tables of the call (M <= 128 takes the fused single-launch route/plan kernel) against the oracle
    hdr, total, block_off = buf.plan_tables()
    plan = O.dispatch_plan([ids], layer.num_experts, 0, hdr["block_m"])
    assert torch.equal(buf.send_count.cpu().long(), plan.recv_total) and torch.equal(total.long(), plan.recv_total)
    assert torch.equal(block_off.long(), plan.pool_block_offset)
    pos = buf.route_pos[:m].cpu()
    dst = buf.pool_dst.cpu()
    inv = {int(pos[t, s]): (t, s) for t in range(m) for s in range(layer.num_topk) if int(pos[t, s]) >= 0}
    for ex in range(layer.num_experts):
        base = int(block_off[ex]) * hdr["block_m"]
        assert [inv[int(dst[base + j])] for j in range(int(total[ex]))] == [(t, s) for (_, t, s) in plan.routes[ex]]


@pytest.mark.parametrize("bm", [16, 32, 64, 128, 192, 240])
def test_every_block_m_variant(bm):
    """Forced BLOCK_M with ~150 tokens per expert (Zipf: some experts far more): several pool blocks per expert,
    partially filled last blocks, and experts whose rows are cut into two or more equal tensor-core tiles that do not
    follow the block boundaries."""
    from vllm_plugin_b200 import api
    layer = H.make_layer(shared=True, seed=3, **SMALL)
    m = 600
    hid = O.make_hidden(m, layer.hidden, 4)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 5, zipf_s=1.2)
    api.set_kernel_options(block_m=bm)
    try:
        y, buf = H.run_layer(layer, hid, ids, w)
        assert buf.plan_tables()[0]["block_m"] == bm
    finally:
        api.set_kernel_options(block_m=0)
    assert_parity(y, H.oracle_layer(layer, hid, ids, w), f"block_m {bm}")


@pytest.mark.parametrize("geom", [dict(hidden=512, inter=256, num_experts=8, num_topk=2),
                                  dict(hidden=1024, inter=384, num_experts=4, num_topk=2)])
@pytest.mark.parametrize("orientation", [2, 3])
@pytest.mark.parametrize("bm", [16, 64, 128, 192, 240])
def test_tokens_as_a_kernels_every_block_m(geom, bm, orientation):
    """The tokens-as-A kernel family forced on (it is otherwise chosen from the expected rows per expert): tiles of up
    to 128 rows under every BLOCK_M pool layout, weight blocks of 192 stored rows with the short last block of a half
    (64 or 128 rows, loaded through the shifted box), scale chunks starting at row 0 and 64 of a 128-row chunk, the
    shared expert's tiles, masked routes and experts without tokens.  Orientation 3 runs them on CTA pairs (two tiles of
    an expert per task, an empty second tile where an expert has an odd number; BLOCK_M < 128 falls back to single
    CTAs).  Against the oracle, and against the weights-as-A kernels on the same inputs."""
    from vllm_plugin_b200 import api
    layer = H.make_layer(shared=True, seed=21, **geom)
    m = 600
    hid = O.make_hidden(m, layer.hidden, 4)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 5, zipf_s=1.2, mask_frac=0.05)
    ids[ids == 1] = -1                                      # an expert that receives nothing
    api.set_kernel_options(block_m=bm)
    try:
        y_tm, buf = H.run_layer(layer, hid, ids, w, orientation=orientation)
        assert buf.plan_tables()[0]["block_m"] == bm
        y_sa, _ = H.run_layer(layer, hid, ids, w, orientation=1)
    finally:
        api.set_kernel_options(block_m=0)
    ref = H.oracle_layer(layer, hid, ids, w)
    assert_parity(y_tm, ref, f"tokens-as-A block_m {bm}")
    assert_parity(y_sa, ref, f"weights-as-A block_m {bm}")
    diff = (y_tm.float() - y_sa.float()).abs().max().item()
    assert diff <= 2e-2, f"the two kernel families differ by {diff}"


@pytest.mark.parametrize("orientation", [2, 3])
@pytest.mark.parametrize("m", [1, 40, 129, 700])
def test_tokens_as_a_kernels_token_counts_and_options(m, orientation):
    """Forced tokens-as-A kernels over small and ragged token counts (tiles of 1..128 rows, the 64-row token box), with
    the two-slice weight form, without clamp, and with the IEEE sigmoid."""
    layer = H.make_layer(shared=True, seed=23, hidden=1024, inter=512, num_experts=4, num_topk=2)
    hid = (O.make_hidden(m, layer.hidden, 1).float() * 3).to(torch.bfloat16)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 2, mask_frac=0.1 if m > 1 else 0.0)
    for clamp, fast, localized in ((10.0, True, False), (None, False, True)):
        y, _ = H.run_layer(layer, hid, ids, w, clamp=clamp, fast_math=fast, localized=localized, orientation=orientation)
        assert_parity(y, H.oracle_layer(layer, hid, ids, w, clamp=clamp), f"m {m} clamp {clamp} fast {fast}")


def test_options_fast_math_clamp_and_localized_weights():
    layer = H.make_layer(shared=True, seed=9, **SMALL)
    hid = (O.make_hidden(40, layer.hidden, 1).float() * 6).to(torch.bfloat16)       # large activations: the clamp bites
    ids, w = O.make_routing(40, layer.num_experts, layer.num_topk, 2)
    for clamp in (10.0, 0.5, None):
        ref = H.oracle_layer(layer, hid, ids, w, clamp=clamp)
        for fast in (True, False):
            y, _ = H.run_layer(layer, hid, ids, w, clamp=clamp, fast_math=fast)
            assert_parity(y, ref, f"clamp {clamp} fast_math {fast}")
    y0, _ = H.run_layer(layer, hid, ids, w)
    y1, _ = H.run_layer(layer, hid, ids, w, localized=True)                         # two-slice routed weights
    assert torch.equal(y0, y1)


def test_masked_tokens_padding_and_empty_call():
    layer = H.make_layer(shared=False, seed=11, **SMALL)
    m = 20
    hid = O.make_hidden(m, layer.hidden, 1)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 2)
    pad = torch.zeros(m, dtype=torch.bool)
    pad[[0, 7, 19]] = True
    y, _ = H.run_layer(layer, hid, ids, w, pad=pad)
    ref = H.oracle_layer(layer, hid, ids, w, pad=pad)
    assert_parity(y, ref, "padding")
    assert float(y[pad.cuda()].float().abs().max()) == 0.0          # no valid slot and no shared expert: exact zeros
    y_empty, _ = H.run_layer(layer, hid[:0], ids[:0], w[:0])
    assert y_empty.shape == (0, layer.hidden)


@pytest.mark.parametrize("m", [1, 40, 300])
def test_residual_added_in_the_combine_pass(m):
    """``residual=`` gives bit for bit what a separate BF16 addition after the layer gives, also in place (residual is y),
    at decode and prefill sizes (chained small-call path and the two-stream path)."""
    from vllm_plugin_b200 import api
    layer = H.make_layer(shared=True, seed=12, **SMALL)
    hid = O.make_hidden(m, layer.hidden, 5)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 6, mask_frac=0.1)
    y, buf = H.run_layer(layer, hid, ids, w)
    dev = y.device
    res = (torch.randn(m, layer.hidden, generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16).to(dev)
    want = y + res                                           # the engine's own addition
    l1, l2, sl1, sl2 = H.kernel_weights(layer, dev)
    out = torch.empty_like(y)
    api.stage_inputs_for_mega_moe(buf, hid.to(dev), ids.to(dev), w.to(dev))
    api.fp8_fp4_mega_moe(out, l1, l2, buf, sl1, sl2, activation_clamp=10.0, residual=res)
    assert torch.equal(out, want)
    inplace = res.clone()
    api.fp8_fp4_mega_moe(inplace, l1, l2, buf, sl1, sl2, activation_clamp=10.0, residual=inplace)
    assert torch.equal(inplace, want)
    api.fp8_fp4_mega_moe(out, l1, l2, buf, sl1, sl2, activation_clamp=10.0)        # and none again: the plain output
    assert torch.equal(out, y)
    with pytest.raises(AssertionError):
        api.fp8_fp4_mega_moe(out, l1, l2, buf, sl1, sl2, activation_clamp=10.0, residual=res.float())


def test_outputs_do_not_depend_on_batch_composition():
    """Size-independent property: a token's output is bit-identical whatever other tokens share the call (columns of the
    tensor-core tiles are independent and the K order is fixed)."""
    layer = H.make_layer(shared=True, seed=13, **SMALL)
    m = 300
    hid = O.make_hidden(m, layer.hidden, 1)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 2)
    y, _ = H.run_layer(layer, hid, ids, w)
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(0))
    y_perm, _ = H.run_layer(layer, hid[perm], ids[perm], w[perm])
    assert torch.equal(y_perm.cpu(), y.cpu()[perm])
    y_head, _ = H.run_layer(layer, hid[:17], ids[:17], w[:17])
    assert torch.equal(y_head.cpu(), y.cpu()[:17])


def test_reference_cpu_configuration():
    """The CPU-runnable configuration of the benchmark: H=5120, I=2304, E=32, top-6, one shared expert, M=128, seed 0."""
    layer = H.make_layer(5120, 2304, 32, 6, True, seed=0)
    hid = O.make_hidden(128, 5120, 0)
    ids, w = O.make_routing(128, 32, 6, 0)
    y, buf = H.run_layer(layer, hid, ids, w)
    assert buf.plan_tables()[0]["block_m"] == 32
    ref = H.oracle_layer(layer, hid, ids, w)
    H.log_parity("config 0: E=32 M=128", H.strict_metrics(y, ref))
    assert_parity(y, ref, "config 0")


def test_full_size_engines_agree_and_permutation_invariance():
    """E=384 resident experts (7.2 GB of packed weights generated on the GPU), M=256 decode-side point: the tensor-core
    kernels against the scalar validation kernels on the same pool, per-expert counts against the routing, and the
    batch-composition property at full size."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    from vllm_plugin_b200.backend.frontend import _use_scalar_validation_kernels
    from vllm_plugin_b200.testing import SyntheticLayer, make_hidden, make_routing
    e, k, h, i, m = 384, 6, 5120, 2304, 256
    syn = SyntheticLayer(h, i, e, True, "cuda", seed=1)
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), e, 3840, k, h, i, 1)
    hid = make_hidden(m, h, 1, "cuda")
    ids, w = make_routing(m, e, k, 2, "cuda")
    stats = torch.zeros(e, dtype=torch.int32, device="cuda")

    def run(hh, ii, ww, engine, st=None):
        y = torch.empty((hh.shape[0], h), dtype=torch.bfloat16, device="cuda")
        _use_scalar_validation_kernels(engine == 1)
        try:
            api.stage_inputs_for_mega_moe(buf, hh, ii, ww)
            api.fp8_fp4_mega_moe(y, syn.l1, syn.l2, buf, syn.shared_l1, syn.shared_l2,
                                 cumulative_local_expert_recv_stats=st, activation_clamp=10.0)
        finally:
            _use_scalar_validation_kernels(False)
        from vllm_plugin_b200.backend.frontend import read_status
        read_status(buf)
        return y

    y_tc = run(hid, ids, w, 0, stats)
    y_sc = run(hid, ids, w, 1)
    assert torch.equal(stats.cpu().long(), torch.bincount(ids.cpu().flatten(), minlength=e))
    assert_parity(y_tc, y_sc.cpu(), "tensor-core vs scalar engine, E=384")
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(1)).cuda()
    assert torch.equal(run(hid[perm], ids[perm], w[perm], 0), y_tc[perm])


def test_layer_class_loads_a_checkpoint_and_runs(monkeypatch):
    """The plugin layer class end to end: checkpoint shards (w1 / w3 / w2 + scales) through ``weight_loader`` into the
    two-slice parameters, ``forward`` through the real backend, reload in place, output against the oracle."""
    from types import SimpleNamespace
    from vllm_plugin_b200 import _standin, api
    from vllm_plugin_b200.experts import make_experts_class

    layer_def = H.make_layer(shared=True, seed=21, **SMALL)
    h, i, e, k = layer_def.hidden, layer_def.inter, layer_def.num_experts, layer_def.num_topk
    backend = SimpleNamespace(**{name: getattr(api, name) for name in api.__all__ if name != "SymmBuffer"})
    backend.get_unsupported_reason_for_mega_moe = (
        lambda *a, **kw: api.get_unsupported_reason_for_mega_moe(*a, **{**kw, "allow_unvalidated": True}))
    cls = make_experts_class(_standin.DeepGemmMegaMoEExperts, _standin.get_ep_group, _standin.MEGA_MOE_MXFP4)
    monkeypatch.setattr(cls, "_import_backend", staticmethod(lambda: backend))
    cfg = SimpleNamespace(parallel_config=SimpleNamespace(enable_eplb=False),
                          scheduler_config=SimpleNamespace(max_num_batched_tokens=256))
    sh = layer_def.shared
    shared_mlp = SimpleNamespace(
        gate_up_proj=SimpleNamespace(weight=sh.w13.cuda(), weight_scale=sh.w13_sf.cuda()),
        down_proj=SimpleNamespace(weight=sh.w2.cuda(), weight_scale=sh.w2_sf.cuda()))
    mod = cls(cfg, prefix="model.layers.0.experts", num_experts=e, num_local_experts=e, experts_start_idx=0, top_k=k,
              hidden_size=h, intermediate_size=i, weight_format=_standin.MEGA_MOE_MXFP4,
              activation=_standin.MegaMoEActivation(clamp=10.0), shared_experts=shared_mlp, device="cuda")
    ptrs = [p.data_ptr() for p in mod.parameters()]

    def load(experts):
        for ex, ew in enumerate(experts):
            for shard, w, s in (("w1", ew.w13[:i], ew.w13_sf[:i]), ("w3", ew.w13[i:], ew.w13_sf[i:]), ("w2", ew.w2, ew.w2_sf)):
                prefix = "w2" if shard == "w2" else "w13"
                assert mod.weight_loader(getattr(mod, f"{prefix}_weight"), w.cuda(), f"experts.{prefix}_weight", shard, ex, True)
                assert mod.weight_loader(getattr(mod, f"{prefix}_weight_scale"), s.cuda(), f"experts.{prefix}_weight_scale", shard, ex, True)

    load(layer_def.experts)
    m = 50
    hid = O.make_hidden(m, h, 1)
    ids, w = O.make_routing(m, e, k, 2)
    y = mod(hid.cuda(), w.cuda(), ids.cuda())
    assert_parity(y, H.oracle_layer(layer_def, hid, ids, w), "layer class")
    # reload other weights into the same parameters: addresses unchanged, outputs follow the new weights
    layer2 = H.make_layer(shared=True, seed=22, **SMALL)
    layer2.shared = layer_def.shared
    load(layer2.experts)
    assert [p.data_ptr() for p in mod.parameters()] == ptrs
    y2 = mod(hid.cuda(), w.cuda(), ids.cuda())
    assert_parity(y2, H.oracle_layer(layer2, hid, ids, w), "layer class after reload")


def test_cuda_graph_replay_of_every_variant():
    """Every BLOCK_M variant is prepared before capture; a captured call replays bit-identically and follows new inputs
    staged into the same buffers."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    layer = H.make_layer(shared=True, seed=31, **SMALL)
    dev = torch.device("cuda", 0)
    l1, l2, sl1, sl2 = H.kernel_weights(layer, dev)
    buf = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), layer.num_experts, 1920, layer.num_topk, layer.hidden, layer.inter, 1)
    variants = api.precompile_mega_moe_variants(1, layer.num_experts, 1920, layer.num_topk, layer.hidden, layer.inter, 1)
    assert variants == (16, 32, 64, 128, 192, 240)
    for m in (1, 40, 130, 700, 1900):
        hid_a, hid_b = O.make_hidden(m, layer.hidden, m), O.make_hidden(m, layer.hidden, m + 1)
        ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, m)
        x = hid_a.cuda()
        ids_d, w_d = ids.cuda(), w.cuda()
        y = torch.empty((m, layer.hidden), dtype=torch.bfloat16, device=dev)

        def call():
            api.stage_inputs_for_mega_moe(buf, x, ids_d, w_d)
            api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, activation_clamp=10.0)

        call()
        eager = y.clone()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call()
        y.zero_()
        g.replay()
        assert torch.equal(y, eager), m
        x.copy_(hid_b.cuda())
        g.replay()
        assert_parity(y, H.oracle_layer(layer, hid_b, ids, w), f"graph replay m={m}")


@pytest.mark.parametrize("m,bm", [(7, 16), (130, 32), (300, 128), (300, 192)])
def test_shared_expert_ahead_of_the_routed_plan(m, bm):
    """The split the expert-parallel forward uses, on one GPU: shared expert planned and run first (both GEMMs), routed
    experts afterwards, leaves bit for bit what one launch over the whole plan leaves."""
    import ctypes
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import _native
    from vllm_plugin_b200.backend.frontend import _weights_struct, check_mega_moe_arguments, read_status
    layer = H.make_layer(shared=True, seed=21, **SMALL)
    hid = O.make_hidden(m, layer.hidden, 3)
    ids, w = O.make_routing(m, layer.num_experts, layer.num_topk, 4, zipf_s=1.2, mask_frac=0.05)
    api.set_kernel_options(block_m=bm)
    try:
        y_whole, buf = H.run_layer(layer, hid, ids, w)
    finally:
        api.set_kernel_options(block_m=0)
    dev = torch.device("cuda", 0)
    l1, l2, sl1, sl2 = H.kernel_weights(layer, dev)
    y = torch.empty_like(y_whole)
    s13, s2 = check_mega_moe_arguments(y, l1, l2, buf, sl1, sl2, None, (1, 1, 32), "swiglu", 10.0, True, 1.0, 0.0)
    ws = _weights_struct(l1, l2, sl1, sl2, s13, s2)
    lib = _native.load()
    geo, base = ctypes.byref(buf.geo), buf.base_ptr
    opts = _native.MmoeOptions(10.0, 1, 0, 2000, 0)
    sp = torch.cuda.current_stream(dev).cuda_stream
    api.stage_inputs_for_mega_moe(buf, hid.to(dev), ids.to(dev), w.to(dev), block_m=bm)
    _native.check(lib.mmoe_plan_shared(geo, base, m, bm, sp))
    _native.check(lib.mmoe_experts_select(geo, base, ctypes.byref(ws), ctypes.byref(opts), m, bm, 2, sp))
    _native.check(lib.mmoe_dispatch_count(geo, base, m, sp))
    _native.check(lib.mmoe_dispatch_place(geo, base, m, bm, None, sp))
    _native.check(lib.mmoe_experts_select(geo, base, ctypes.byref(ws), ctypes.byref(opts), m, bm, 1, sp))
    _native.check(lib.mmoe_combine(geo, base, y.data_ptr(), m, sp))
    read_status(buf)
    assert torch.equal(y, y_whole)
