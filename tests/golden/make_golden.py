"""Generate the golden fixtures in this folder by running the reference's own importable Python on seeded inputs.

Run from the repository root, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference cannot travel to the GPU machines, so its outputs are committed here as small ``.npz`` / ``.json`` files
and the tests compare the oracle, the host logic and the CUDA kernels against them.  Nothing here is read at run time
except the generated files.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from vllm_sm107_megamoe.backend import heuristics as H
    from vllm_sm107_megamoe.backend import staging as S
    from vllm_sm107_megamoe.backend import weights as W

    # ---- 1. BLOCK_M selection and variant sets (backend/heuristics.py:123-228) ------------------------------------
    geos = [(1, 32, 6), (1, 96, 6), (1, 192, 6), (1, 384, 6), (2, 384, 6), (4, 384, 6), (8, 384, 6), (16, 384, 6),
            (32, 384, 6), (4, 388, 6), (8, 392, 6), (8, 400, 6), (16, 400, 6), (32, 416, 6), (1, 128, 3), (4, 128, 3),
            (8, 128, 3), (16, 128, 3), (32, 128, 3), (4, 132, 3), (8, 136, 3), (8, 144, 3), (16, 144, 3), (32, 160, 3),
            (1, 8, 2), (2, 16, 4)]
    ms = sorted(set(list(range(0, 66)) + [96, 100, 127, 128, 129, 192, 255, 256, 257, 384, 500, 512, 640, 768, 1000,
                                           1024, 1500, 1920, 2048, 2530, 2560, 3000, 3072, 3840, 4096, 5120, 5376,
                                           5760, 8190, 8192]))
    block_m = {}
    for (r, e, k) in geos:
        block_m[f"{r},{e},{k}"] = [H.get_block_m_for_mega_moe(r, e, 0, m, k) for m in ms]
    variants = {}
    for (r, e, k) in geos:
        for t in (1920, 3840, 5760):
            variants[f"{r},{e},{k},{t}"] = list(H.get_block_m_variants(r, e, k, t))

    # ---- 2. admission gate (backend/heuristics.py:1354-1503), at the build's SM count -----------------------------
    admission = []
    cases = []
    for (hid, inter, k), (es, _) in H.VALIDATED_GEOMETRIES.items():
        for e in es:
            for r in (1, 2, 4, 8, 16, 32):
                cases.append((r, e, 2560, k, hid, inter, 1))
    for (hid, inter, k), (pairs, _) in H.VALIDATED_EP_GEOMETRIES.items():
        for (e, r) in pairs:
            cases.append((r, e, 2560, k, hid, inter, 1))
            cases.append((r * 2, e, 2560, k, hid, inter, 1))
    cases += [(4, 400, 2560, 6, 5120, 2304, 1), (1, 64, 2560, 6, 5120, 2304, 1), (1, 384, 2560, 8, 5120, 2304, 1),
              (1, 384, 2560, 6, 4096, 2304, 1), (1, 384, 2560, 6, 5120, 2048, 1), (1, 384, 2560, 6, 5120, 2304, 2),
              (33, 384, 2560, 6, 5120, 2304, 1), (0, 384, 2560, 6, 5120, 2304, 1), (1, 384, 0, 6, 5120, 2304, 1),
              (1, 384, 320, 6, 5120, 2304, 0), (8, 128, 5120, 3, 5120, 2304, 1)]
    for c in cases:
        r, e, t, k, hid, inter, s = c
        for kw in ({}, {"allow_unvalidated": True}):
            reason = H.get_mega_moe_unsupported_reason(r, e, t, k, hid, inter, s, num_sms=148, **kw)
            admission.append({"args": list(c), "kwargs": kw, "admitted": reason is None,
                              "unvalidated": bool(reason and "has not been validated" in reason)})
    for extra in ({"mma_type": "bf16xbf16"}, {"activation": "silu"}, {"localized_shared_weights": True}):
        reason = H.get_mega_moe_unsupported_reason(1, 384, 2560, 6, 5120, 2304, 1, num_sms=148, **extra)
        admission.append({"args": [1, 384, 2560, 6, 5120, 2304, 1], "kwargs": extra, "admitted": reason is None,
                          "unvalidated": False})
    meta = {
        "ms": ms, "block_m": block_m, "variants": variants, "admission": admission,
        "validated_geometries": {",".join(map(str, k)): list(v[0]) for k, v in H.VALIDATED_GEOMETRIES.items()},
        "validated_ep_geometries": {",".join(map(str, k)): [list(p) for p in v[0]] for k, v in H.VALIDATED_EP_GEOMETRIES.items()},
        "min_experts_per_rank": H.MIN_VALIDATED_EXPERTS_PER_RANK,
        "token_alignment": H.get_token_alignment_for_mega_moe(),
    }
    with open(os.path.join(HERE, "host_logic.json"), "w") as f:
        json.dump(meta, f, separators=(",", ":"))

    # ---- 3. input staging (backend/staging.py:51-82, 85-95, 199-251) ---------------------------------------------
    g = torch.Generator().manual_seed(0)
    m, h, k = 37, 512, 6
    x = torch.randn((m, h), generator=g)
    x[3] *= 1e-6          # below the 1e-4 amax clamp
    x[5] *= 300.0         # large magnitudes
    x[7, :64] = 0.0       # an all-zero group
    x[8, 5] = -0.0
    x[9] *= 1e3
    x[11, ::2] = 448.0
    x[12] = torch.rand((h,), generator=g) * 2.0 ** -130   # float32 denormal range before the BF16 cast
    x = x.to(torch.bfloat16)
    ids = torch.randint(0, 32, (m, k), generator=g, dtype=torch.int64)
    w = torch.rand((m, k), generator=g)
    pad = torch.zeros(m, dtype=torch.bool)
    pad[[2, 30]] = True
    stage = {}
    q, sf = S.per_token_cast_to_fp8(x)
    stage["x_bits"] = x.view(torch.int16).numpy()
    stage["ids"] = ids.numpy()
    stage["w"] = w.numpy()
    stage["pad"] = pad.numpy()
    stage["q"] = q.view(torch.uint8).numpy()
    stage["sf"] = sf.numpy()
    for bm in (16, 32, 64, 128, 192, 240):
        t_aligned = 1920
        n_s = -(-t_aligned // 8) * 128
        xo = torch.zeros((t_aligned, h), dtype=torch.float8_e4m3fn)
        sfo = torch.zeros((t_aligned, h // 128), dtype=torch.int32)
        io = torch.zeros((t_aligned, k), dtype=torch.int64)
        wo = torch.zeros((t_aligned, k), dtype=torch.float32)
        sh = torch.empty_strided((n_s, h // 128), (1, n_s), dtype=torch.int32).zero_()
        S.prepare_megamoe_inputs_torch(x, w, ids.to(torch.int32), xo, sfo, io, wo, pad, sh, bm)
        assert torch.equal(xo[:m].view(torch.uint8), q.view(torch.uint8)) and torch.equal(sfo[:m], sf)
        rows = S.get_shared_sf_rows(m, bm)
        stage[f"shared_rows_{bm}"] = rows.numpy()
        stage[f"shared_sf_{bm}"] = sh[: int(rows.max()) + 1].contiguous().numpy()
        stage["ids_out"] = io[:m].numpy()
        stage["w_out"] = wo[:m].numpy()
    np.savez_compressed(os.path.join(HERE, "staging.npz"), **stage)

    # ---- 4. weight scale-factor layouts (backend/weights.py:37-145) -----------------------------------------------
    g = torch.Generator().manual_seed(1)
    e_l, n13, hk, n2, ik = 3, 256, 512, 384, 256
    sf13 = torch.randint(110, 130, (e_l, n13, hk // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    sf2 = torch.randint(110, 130, (e_l, n2, ik // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    w13 = torch.randint(-128, 128, (e_l, n13, hk // 2), generator=g, dtype=torch.int32).to(torch.int8)
    w2 = torch.randint(-128, 128, (e_l, n2, ik // 2), generator=g, dtype=torch.int32).to(torch.int8)
    l13 = W.sf_to_required_layout(sf13, n13, hk, e_l)
    l2 = W.sf_to_required_layout(sf2, n2, ik, e_l)
    (t13, t13sf), (t2, t2sf) = W.transform_weights_for_mega_moe((w13, l13), (w2, l2))
    np.savez_compressed(
        os.path.join(HERE, "weights.npz"),
        sf13=sf13.numpy(), sf2=sf2.numpy(), w13=w13.numpy(), w2=w2.numpy(),
        l13=l13.contiguous().numpy(), l13_strides=np.array(l13.stride()), l2=l2.contiguous().numpy(),
        t13=t13.numpy(), t13sf=t13sf.contiguous().numpy(), t13sf_strides=np.array(t13sf.stride()),
        t2=t2.numpy(), t2sf=t2sf.contiguous().numpy(),
        utccp13=W.transpose_sf_for_utccp(l13).contiguous().numpy(),
    )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
