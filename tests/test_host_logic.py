"""Host logic of the package (BLOCK_M, variants, admission gate, weight layouts, C-ABI export) against the reference's
golden outputs.  No GPU: nothing here launches a kernel."""

import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

from helpers import ROOT

GOLD = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def host_logic():
    with open(os.path.join(GOLD, "host_logic.json")) as f:
        return json.load(f)


def test_block_m_python_and_c(host_logic):
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    ms = host_logic["ms"]
    for key, expect in host_logic["block_m"].items():
        r, e, k = map(int, key.split(","))
        assert [api.get_block_m_for_mega_moe(r, e, 0, m, k) for m in ms] == expect, key
        assert [lib.mmoe_block_m(r, e, m, k) for m in ms] == expect, key


def test_block_m_variants(host_logic):
    from vllm_plugin_b200.backend import heuristics as H
    for key, expect in host_logic["variants"].items():
        r, e, k, t = map(int, key.split(","))
        assert list(H.get_block_m_variants(r, e, k, t)) == expect, key


def test_token_alignment_and_tables(host_logic):
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import heuristics as H
    assert api.get_token_alignment_for_mega_moe() == host_logic["token_alignment"] == 1920
    assert {",".join(map(str, k)): list(v[0]) for k, v in H.VALIDATED_GEOMETRIES.items()} == host_logic["validated_geometries"]
    assert {",".join(map(str, k)): [list(p) for p in v[0]] for k, v in H.VALIDATED_EP_GEOMETRIES.items()} == host_logic["validated_ep_geometries"]
    assert H.MIN_VALIDATED_EXPERTS_PER_RANK == host_logic["min_experts_per_rank"]


def test_admission_gate_matches_reference(host_logic):
    from vllm_plugin_b200 import api
    for case in host_logic["admission"]:
        reason = api.get_unsupported_reason_for_mega_moe(*case["args"], **case["kwargs"])
        assert (reason is None) == case["admitted"], (case, reason)
        if case["unvalidated"]:
            assert "has not been validated" in reason


def test_admission_gate_is_total():
    from vllm_plugin_b200 import api
    for bad in [(None, 384, 2560, 6, 5120, 2304), ("x", 1, 1, 1, 1, 1), (1, 384, 2560, 6, 5120.5, 2304), (1, [], 1, 1, 1, 1)]:
        reason = api.get_unsupported_reason_for_mega_moe(*bad)
        assert isinstance(reason, str) and reason


def test_weight_transform_against_reference_layouts():
    from vllm_plugin_b200.backend import weights as W
    g = np.load(os.path.join(GOLD, "weights.npz"))
    sf13 = torch.from_numpy(g["sf13"])
    e_l, n13, k32 = sf13.shape
    l13 = W.sf_to_required_layout(sf13, n13, k32 * 32, e_l)
    assert list(l13.stride()) == list(g["l13_strides"])
    assert np.array_equal(l13.contiguous().numpy(), g["l13"])
    w13 = torch.from_numpy(g["w13"])
    w2 = torch.from_numpy(g["w2"])
    sf2 = torch.from_numpy(g["sf2"])
    l2 = W.sf_to_required_layout(sf2, sf2.shape[1], sf2.shape[2] * 32, e_l)
    (t13, t13sf), (t2, t2sf) = W.transform_weights_for_mega_moe((w13, l13), (w2, l2))
    # bit-identical to the reference's transform: gate/up 8-row interleave + 4x32 scale transpose
    assert np.array_equal(t13.numpy(), g["t13"]) and np.array_equal(t2.numpy(), g["t2"])
    assert np.array_equal(t13sf.contiguous().numpy(), g["t13sf"]) and list(t13sf.stride()) == list(g["t13sf_strides"])
    assert np.array_equal(t2sf.contiguous().numpy(), g["t2sf"])
    assert t13sf.stride() == l13.stride()
    with pytest.raises(AssertionError):
        W.transform_weights_for_mega_moe((w13, l13), (w2, l2), activation="silu")


def test_localize_shape_and_round_trip():
    from vllm_plugin_b200.backend import locality as L
    t = torch.arange(3 * 8 * 6, dtype=torch.int8).view(3, 8, 6)
    loc = L.localize(t)
    assert tuple(loc.shape) == (2, 3, 4, 6)
    assert (loc.stride(0) * loc.element_size()) % (2 << 20) == 0
    assert L.is_canonical_localized(loc)
    assert torch.equal(loc.movedim(0, 1).flatten(1, 2), t)             # how the reference's tests undo the split
    assert torch.equal(L.delocalize(loc), t)


def test_library_exports_every_declared_symbol():
    from vllm_plugin_b200.backend import _native
    header = open(os.path.join(ROOT, "include", "mmoe.h")).read()
    declared = set(re.findall(r"\b(mmoe_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_native.EXPORTED_SYMBOLS)
    lib = ctypes.CDLL(_native.library_path())
    for name in declared:
        assert hasattr(lib, name), name
    assert _native.load().mmoe_abi_version() == 3


def test_layout_is_consistent():
    from vllm_plugin_b200.backend import _native
    geo = _native.MmoeGeometry(8, 3, 392, 6, 5120, 2304, 1, 3840)
    lay = _native.layout_of(geo)
    offs = [(n, getattr(lay, n)) for n in _native._LAYOUT_FIELDS[1:32] if n not in ("shared_sf_rows",)]
    vals = [v for _, v in offs]
    assert vals == sorted(vals) and all(v % 1024 == 0 for v in vals)
    assert lay.total_bytes > vals[-1]
    assert lay.shared_sf_rows == -(-3840 // 8) * 128
    assert lay.max_routes == 3840 * 6
    with pytest.raises(AssertionError):
        _native.layout_of(_native.MmoeGeometry(8, 3, 390, 6, 5120, 2304, 1, 3840))
    with pytest.raises(AssertionError):
        _native.layout_of(_native.MmoeGeometry(1, 0, 384, 6, 5120, 2304, 1, 2560))   # capacity must be aligned to 1920
    with pytest.raises(NotImplementedError):
        _native.layout_of(_native.MmoeGeometry(1, 0, 384, 6, 5120, 2304, 2, 3840))


def test_entry_points_reject_bad_arguments_before_touching_the_device():
    """Argument errors come back as status codes from the C ABI (mapped to the reference's exception classes) without
    any CUDA call, so they can be checked on a machine without a GPU."""
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    buf = (ctypes.c_int32 * 64)()
    p = ctypes.addressof(buf)
    with pytest.raises(AssertionError, match="multiple of 128"):
        _native.check(lib.mmoe_transform_weights(p, p + 64, p, p + 128, 1, 100, 64, 1, 1, None))
    with pytest.raises(AssertionError, match="distinct"):
        _native.check(lib.mmoe_transform_weights(None, None, p, p, 1, 128, 64, 1, 0, None))
    geo1 = _native.MmoeGeometry(1, 0, 384, 6, 5120, 2304, 1, 3840)
    opts = _native.MmoeOptions(10.0, 1, 0, 2000, 0)
    w = _native.MmoeWeights()
    peers = (ctypes.c_void_p * 1)(p)
    with pytest.raises(AssertionError, match="num_ranks > 1"):
        _native.check(lib.mmoe_forward_ep(ctypes.byref(geo1), p, peers, ctypes.byref(w), ctypes.byref(opts), p, 1, 16, None, None))
    with pytest.raises(AssertionError, match="num_ranks > 1"):
        _native.check(lib.mmoe_experts_ep_return(ctypes.byref(geo1), p, peers, ctypes.byref(w), ctypes.byref(opts), 1, 16, None))
    geo2 = _native.MmoeGeometry(2, 0, 384, 6, 5120, 2304, 1, 3840)
    peers2 = (ctypes.c_void_p * 2)(p, None)
    with pytest.raises(AssertionError, match="NULL"):
        _native.check(lib.mmoe_forward_ep(ctypes.byref(geo2), p, peers2, ctypes.byref(w), ctypes.byref(opts), p, 1, 16, None, None))


def test_import_is_light():
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); import vllm_plugin_b200, vllm_plugin_b200.api as a; "
            "vllm_plugin_b200.register(); a.get_unsupported_reason_for_mega_moe(1, 384, 2560, 6, 5120, 2304, 1); a.get_token_alignment_for_mega_moe(); "
            "bad = [m for m in ('torch', 'vllm', 'triton') if m in sys.modules]; assert not bad, bad" % ROOT)
    env = {k: v for k, v in os.environ.items() if k != "VLLM_PLUGINS"}
    subprocess.run([sys.executable, "-c", code], check=True, env=env)


def test_admission_gate_and_library_agree_on_the_kernel_limits():
    """Whatever the Python gate admits with ``allow_unvalidated=True`` the C library must lay out, and what the library
    refuses the gate must refuse (the gate may be stricter only where the engine-facing contract is: none here)."""
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import _native
    lib = _native.load()
    cases = []
    for ranks in (1, 2, 3, 8, 32, 33):
        for experts in (8, 48, 384, 392, 2048, 2056, 16416):
            for topk in (1, 6, 31, 32):
                for hidden, inter in ((5120, 2304), (512, 256), (384, 128), (256, 192), (1024, 64)):
                    cases.append((ranks, experts, 1920, topk, hidden, inter, 1))
    agree = 0
    for ranks, experts, tokens, topk, hidden, inter, shared in cases:
        reason = api.get_unsupported_reason_for_mega_moe(ranks, experts, tokens, topk, hidden, inter, shared,
                                                         allow_unvalidated=True)
        geo = _native.MmoeGeometry(ranks, 0, experts, topk, hidden, inter, shared, 1920)
        lay = _native.MmoeLayout()
        code = lib.mmoe_layout(ctypes.byref(geo), ctypes.byref(lay))
        assert (reason is None) == (code == _native.MMOE_OK), (ranks, experts, topk, hidden, inter, reason, code)
        agree += 1
    assert agree == len(cases)
