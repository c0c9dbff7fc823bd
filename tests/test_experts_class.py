"""The layer class on CPU: shard loading into the two-slice routed weights, reload in place, load-balancer views,
logical -> physical mapping after a rebalance, communicator gate.  Modelled on the reference's tests/test_experts.py
and tests/test_eplb.py; the engine's base layer is replaced by the stand-in of vllm_plugin_b200/_standin.py and the
backend's device probe by a fake (as the reference's tests do), so nothing here touches a GPU."""

from types import SimpleNamespace

import pytest
import torch

from vllm_plugin_b200 import _standin, api
from vllm_plugin_b200.experts import _check_eplb, make_experts_class

HIDDEN, INTER = 256, 256


def fake_backend():
    return SimpleNamespace(
        is_localization_available=lambda: True,
        get_unsupported_reason_for_mega_moe=lambda *a, **k: None,
        localize=api.localize,
    )


def make_config(enable_eplb=False, communicator=None, elastic_ep=False, use_async=False):
    return SimpleNamespace(
        parallel_config=SimpleNamespace(enable_eplb=enable_eplb, enable_elastic_ep=elastic_ep,
                                        eplb_config=SimpleNamespace(communicator=communicator, use_async=use_async)),
        scheduler_config=SimpleNamespace(max_num_batched_tokens=4),
    )


@pytest.fixture()
def plugin_cls(monkeypatch):
    cls = make_experts_class(_standin.DeepGemmMegaMoEExperts, lambda: SimpleNamespace(world_size=1),
                             _standin.MEGA_MOE_MXFP4)
    backend = fake_backend()
    monkeypatch.setattr(cls, "_import_backend", staticmethod(lambda: backend))
    return cls


def kwargs(num_experts=2, num_local=2, start=0, num_logical=None):
    return dict(num_experts=num_experts, num_local_experts=num_local, experts_start_idx=start, top_k=1,
                hidden_size=HIDDEN, intermediate_size=INTER, weight_format=_standin.MEGA_MOE_MXFP4,
                activation=_standin.MegaMoEActivation(), num_logical_experts=num_logical)


def checkpoint(seed, num_logical):
    g = torch.Generator().manual_seed(seed)
    shards = []
    for expert in range(num_logical):
        for shard in ("w1", "w2", "w3"):
            rows, cols = (HIDDEN, INTER) if shard == "w2" else (INTER, HIDDEN)
            prefix = "w2" if shard == "w2" else "w13"
            for suffix, width in (("weight", cols // 2), ("weight_scale", cols // 32)):
                value = torch.randint(0, 256, (rows, width), generator=g, dtype=torch.uint8)
                shards.append((expert, shard, f"{prefix}_{suffix}", value))
    return shards


def test_reload_preserves_parameters_and_matches_base_bytes(plugin_cls):
    native = _standin.DeepGemmMegaMoEExperts(make_config(), prefix="model.layers.0.experts", **kwargs())
    actual = plugin_cls(make_config(), prefix="model.layers.1.experts", **kwargs())
    assert tuple(actual.w13_weight.shape) == (2, 2, INTER, HIDDEN // 2)      # (slices, E_l, N/2, K/2)
    parameters = list(actual.parameters())
    pointers = [p.data_ptr() for p in parameters]
    for seed in (0, 1):
        g = torch.Generator().manual_seed(seed)
        shards = checkpoint(seed, 2)
        for index in torch.randperm(len(shards), generator=g).tolist():
            expert, shard, name, value = shards[index]
            for layer in (native, actual):
                assert layer.weight_loader(getattr(layer, name), value, f"experts.{name}", shard, expert, return_success=True)
        for name, expected in native.named_parameters():
            value = getattr(actual, name)
            if value.dim() == 4:
                value = value.movedim(0, 1).flatten(1, 2)
            assert torch.equal(value, expected), name
        assert all(a is b for a, b in zip(parameters, actual.parameters()))
        assert [p.data_ptr() for p in actual.parameters()] == pointers


def test_base_layout_is_the_kernel_layout():
    """A ``w1``/``w3`` pair lands as the gate/up 8-row interleave, i.e. exactly what transform_weights_for_mega_moe
    produces from ``[gate | up]`` rows."""
    layer = _standin.DeepGemmMegaMoEExperts(make_config(), prefix="x", **kwargs(1, 1))
    g = torch.Generator().manual_seed(3)
    w1 = torch.randint(0, 256, (INTER, HIDDEN // 2), generator=g, dtype=torch.uint8)
    w3 = torch.randint(0, 256, (INTER, HIDDEN // 2), generator=g, dtype=torch.uint8)
    layer.weight_loader(layer.w13_weight, w1, "experts.w13_weight", "w1", 0)
    layer.weight_loader(layer.w13_weight, w3, "experts.w13_weight", "w3", 0)
    from vllm_plugin_b200.backend.weights import interleave_weights
    assert torch.equal(layer.w13_weight.data[0], interleave_weights(torch.cat([w1, w3])))


def test_eplb_views_alias_parameters_in_place(plugin_cls):
    layer = plugin_cls(make_config(), prefix="x", **kwargs(4, 4))
    views = layer.get_expert_weights()
    assert len(views) == 6                                  # two slices for each of w13 / w2, plus the two scale tensors
    assert all(v.shape[0] == 4 and v.is_contiguous() for v in views)
    for v in views:
        v[1].fill_(0x5A)                                    # what the load balancer does: whole-row writes
    assert bool((layer.w13_weight.data[:, 1] == 0x5A).all()) and bool((layer.w13_weight.data[:, 0] == 0).all())
    assert bool((layer.w2_weight.data[:, 1] == 0x5A).all()) and bool((layer.w13_weight_scale.data[1] == 0x5A).all())
    w = layer.w13_weight.data
    assert views[0].data_ptr() == w.data_ptr() and views[1].data_ptr() == w.data_ptr() + w.stride(0)


def test_reload_after_rebalance_follows_the_replica_map(plugin_cls):
    # 3 logical experts on 4 physical slots: logical 0 has a replica in slot 3
    layer = plugin_cls(make_config(), prefix="x", **kwargs(4, 4, 0, 3))
    assert layer._map_global_expert_id(0) == [0, 3] and layer._map_global_expert_id(1) == [1]
    mapping = torch.tensor([[[2, -1], [0, 3], [1, -1]]])    # after a rebalance: logical 1 lives in slots 0 and 3
    layer.set_eplb_state(0, torch.zeros((1, 4), dtype=torch.int32), mapping, torch.tensor([[1, 2, 1]]))
    assert layer._map_global_expert_id(1) == [0, 3] and layer._map_global_expert_id(0) == [2]
    g = torch.Generator().manual_seed(0)
    value = torch.randint(0, 256, (HIDDEN, INTER // 2), generator=g, dtype=torch.uint8)
    assert layer.weight_loader(layer.w2_weight, value, "experts.w2_weight", "w2", 1, return_success=True)
    flat = layer.w2_weight.data.movedim(0, 1).flatten(1, 2)
    assert torch.equal(flat[0], value) and torch.equal(flat[3], value)
    assert int(flat[1].sum()) == 0 and int(flat[2].sum()) == 0


def test_admission_runs_before_weights_are_created(monkeypatch):
    cls = make_experts_class(_standin.DeepGemmMegaMoEExperts, lambda: SimpleNamespace(world_size=1), _standin.MEGA_MOE_MXFP4)
    backend = SimpleNamespace(is_localization_available=lambda: True, localize=api.localize,
                              get_unsupported_reason_for_mega_moe=api.get_unsupported_reason_for_mega_moe)
    monkeypatch.setattr(cls, "_import_backend", staticmethod(lambda: backend))
    with pytest.raises(NotImplementedError, match="has not been validated"):
        cls(make_config(), prefix="x", **kwargs(2, 2))      # (256, 256, top-1) is not a validated geometry
    no_gpu = SimpleNamespace(is_localization_available=lambda: False)
    monkeypatch.setattr(cls, "_import_backend", staticmethod(lambda: no_gpu))
    with pytest.raises(NotImplementedError, match="compute capability 10.0"):
        cls(make_config(), prefix="x", **kwargs(2, 2))


@pytest.mark.parametrize("communicator,use_async,ok", [
    ("symm_mem", True, True), ("torch_gloo", True, True), ("torch_nccl", False, True), ("pynccl", False, True),
    ("torch_nccl", True, False), ("pynccl", True, False), ("nixl", False, False), ("torch_xccl", False, False),
    ("something_else", False, False),
])
def test_eplb_communicator_gate(communicator, use_async, ok):
    cfg = make_config(True, communicator, use_async=use_async).parallel_config
    if ok:
        _check_eplb(cfg)
    else:
        with pytest.raises(NotImplementedError):
            _check_eplb(cfg)
    with pytest.raises(NotImplementedError, match="elastic EP"):
        _check_eplb(make_config(True, "symm_mem", elastic_ep=True).parallel_config)


def test_register_is_a_no_op_without_opt_in(monkeypatch):
    import vllm_plugin_b200
    monkeypatch.delenv("VLLM_PLUGINS", raising=False)
    assert vllm_plugin_b200.register() is None
    monkeypatch.setenv("VLLM_PLUGINS", "some_other_plugin")
    assert vllm_plugin_b200.register() is None
