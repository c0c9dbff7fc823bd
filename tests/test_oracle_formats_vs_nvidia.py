"""The oracle's number formats against NVIDIA's own host-side definitions (cuda_fp4.h / cuda_fp8.h), which the oracle's
author did not write: E2M1 and E4M3 decode tables, the nibble order of a packed FP4 byte, and the round-to-nearest-even
encoders.  ``oracle/nv_formats.cpp`` prints the tables; it is compiled here with nvcc for the host (no GPU involved)."""

import math
import os
import shutil
import struct
import subprocess

import pytest
import torch

from oracle import mmoe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def nvidia_tables():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed")
    out_dir = os.path.join(ROOT, "oracle", "_build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "nv_formats")
    src = os.path.join(ROOT, "oracle", "nv_formats.cpp")
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        subprocess.run([nvcc, "-Wno-deprecated-gpu-targets", "-o", exe, src], check=True, capture_output=True)
    text = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    tables = {"fp4": [], "fp8": [], "q4": [], "q8": []}
    for line in text.splitlines():
        kind, *rest = line.split()
        tables[kind].append(rest)
    return tables


def test_e2m1_decode_and_nibble_order(nvidia_tables):
    want = torch.tensor([[float(lo), float(hi)] for _, lo, hi in nvidia_tables["fp4"]])
    got = O.e2m1_unpack(torch.arange(256, dtype=torch.uint8).view(256, 1))          # [256, 2]: (low nibble, high nibble)
    assert want.shape == (256, 2)
    assert torch.equal(got, want)
    assert torch.equal(torch.signbit(got), torch.signbit(want))                      # -0 of codes 8 and 0x80


def test_e4m3_decode(nvidia_tables):
    rows = nvidia_tables["fp8"]
    want = torch.tensor([float("nan") if v == "nan" else float(v) for _, v in rows])
    got = O.e4m3_to_f32(torch.arange(256, dtype=torch.uint8))
    nan = torch.isnan(want)
    assert nan.sum() == 2 and torch.equal(torch.isnan(got), nan)                     # 0x7F and 0xFF
    assert torch.equal(got[~nan], want[~nan])


def _floats(rows):
    return torch.tensor([struct.unpack("<f", bytes.fromhex(h)[::-1])[0] for h, _ in rows], dtype=torch.float32)


def test_e4m3_encode_round_to_nearest_even_saturating(nvidia_tables):
    rows = nvidia_tables["q8"]
    x = _floats(rows)
    want = torch.tensor([int(c) for _, c in rows], dtype=torch.uint8)
    # the oracle's quantisers clamp to the finite range before they cast (quantize_mxfp8, swiglu_requant, quantize_nvfp4)
    got = x.clamp(-O.FP8_MAX, O.FP8_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(got, want)


def test_e2m1_encode_round_to_nearest_even(nvidia_tables):
    rows = [(h, c) for h, c in nvidia_tables["q4"]]
    x = _floats(rows)
    want = torch.tensor([int(c) for _, c in rows], dtype=torch.uint8)
    keep = x.abs() <= 6.0                                          # inside a block whose scale is exactly 1
    x, want = x[keep], want[keep]
    n = x.numel() // 15 * 15
    # blocks of 16: fifteen probes and one 6.0, so that amax * global_scale / 6 == 1 and the probes are quantised as they are
    block = torch.cat([x[:n].view(-1, 15), torch.full((n // 15, 1), 6.0)], dim=1)
    packed, sf = O.quantize_nvfp4(block, 1.0)
    assert torch.equal(sf, torch.full_like(sf, 0x38))              # E4M3 1.0
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).view(-1, 16)[:, :15].reshape(-1)
    assert torch.equal(codes, want[:n])
    assert n > 1500 and math.isclose(float(x.abs().max()), 6.0)
