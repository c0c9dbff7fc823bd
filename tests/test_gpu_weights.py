"""Load-time weight transform on the GPU (``mmoe_transform_weights``): bit-identical to the indexing-op form and to the
golden vectors generated from the reference's own transform."""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _mn_major(t: torch.Tensor) -> torch.Tensor:
    g, mn, kw = t.shape
    out = torch.empty_strided((g, mn, kw), (kw * mn, 1, mn), dtype=t.dtype, device=t.device)
    out.copy_(t)
    return out


def _torch_form(l1, l2):
    from vllm_plugin_b200.backend import weights as W
    return ((W.interleave_weights(l1[0]), W.transpose_sf_for_utccp(W.interleave_weights(l1[1]))),
            (l2[0], W.transpose_sf_for_utccp(l2[1])))


@pytest.mark.parametrize("e,inter,hidden", [(3, 256, 512), (2, 2304, 5120), (1, 128, 256)])
def test_native_transform_equals_indexing_ops(e, inter, hidden):
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import weights as W
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device="cpu").manual_seed(e * 1000 + inter)
    w13 = torch.randint(-128, 128, (e, 2 * inter, hidden // 2), dtype=torch.int8, generator=gen).to(dev)
    w2 = torch.randint(-128, 128, (e, hidden, inter // 2), dtype=torch.int8, generator=gen).to(dev)
    s13 = _mn_major(torch.randint(-2**31, 2**31 - 1, (e, 2 * inter, hidden // 128), dtype=torch.int32, generator=gen).to(dev))
    s2 = _mn_major(torch.randint(-2**31, 2**31 - 1, (e, hidden, -(-inter // 128)), dtype=torch.int32, generator=gen).to(dev))
    assert W._native_transform_applies((w13, s13)) and W._native_transform_applies((w2, s2))
    (a1, a1s), (a2, a2s) = api.transform_weights_for_mega_moe((w13, s13), (w2, s2))
    (b1, b1s), (b2, b2s) = _torch_form((w13, s13), (w2, s2))
    assert torch.equal(a1, b1) and torch.equal(a1s, b1s) and a1s.stride() == b1s.stride()
    assert a2.data_ptr() == w2.data_ptr() and torch.equal(a2s, b2s) and a2s.stride() == b2s.stride()
    # the 2-D (shared expert) form
    (c1, c1s), (c2, c2s) = api.transform_weights_for_mega_moe((w13[0], s13[0]), (w2[0], s2[0]))
    assert torch.equal(c1, b1[0]) and torch.equal(c1s, b1s[0]) and torch.equal(c2s, b2s[0])


def test_native_transform_matches_reference_golden_vectors():
    from vllm_plugin_b200 import api
    g = np.load(os.path.join(GOLD, "weights.npz"))
    dev = torch.device("cuda", 0)
    w13, w2 = torch.from_numpy(g["w13"]).to(dev), torch.from_numpy(g["w2"]).to(dev)
    l13 = _mn_major(torch.from_numpy(g["l13"]).to(dev))
    l2 = _mn_major(torch.from_numpy(g["l2"]).to(dev))
    assert list(l13.stride()) == [int(x) for x in g["l13_strides"]]
    (t13, t13sf), (t2, t2sf) = api.transform_weights_for_mega_moe((w13, l13), (w2, l2))
    assert torch.equal(t13.cpu(), torch.from_numpy(g["t13"]))
    assert torch.equal(t13sf.cpu(), torch.from_numpy(g["t13sf"]))
    assert torch.equal(t2sf.cpu(), torch.from_numpy(g["t2sf"]))
