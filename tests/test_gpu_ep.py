"""Expert parallelism on real GPUs: one process per GPU over NCCL (NVLS off), each rank checked against the oracle.
Skipped on machines with fewer GPUs than ranks."""

import pytest
import torch

from ep_harness import layer_body, run_ranks

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


SMALL = dict(hidden=512, inter=256, num_experts=16, num_topk=4, shared=True)


def test_redundant_physical_experts_under_cuda_graph():
    """Load-balancer geometry: 12 logical + 4 redundant physical experts over 2 ranks, decode-sized calls replayed from
    a CUDA graph."""
    _need(2)
    run_ranks(2, "nccl", layer_body, SMALL, (16, 64), 5, dict(zipf_s=1.2), 1920, "peer", True, 4, timeout=240)


@pytest.mark.parametrize("world,tokens,kw,transport,graph", [
    (2, (70, 33), dict(zipf_s=1.2, mask_frac=0.05, hot=2), "peer", False),
    (2, (70, 33), dict(zipf_s=1.2, mask_frac=0.05, hot=2), "peer-unfused", False),
    (2, (70, 33), dict(zipf_s=1.2, mask_frac=0.05, hot=2), "nccl", False),
    (2, (1, 0), {}, "peer", False),
    (2, (40, 130), dict(zipf_s=1.2, mask_frac=0.05), "peer", True),
    (4, (130, 64, 7, 300), dict(zipf_s=1.2, mask_frac=0.05), "peer", False),
])
def test_layer_matches_oracle_at_ep(world, tokens, kw, transport, graph):
    """Per-rank output against the oracle, receive counts / block offsets / statistics bit-exact; with the device-side
    peer exchange (write-back fused into GEMM2, checked bit-identical to the separate copy kernel; also replayed from a
    CUDA graph) and with the host-driven NCCL exchange."""
    _need(world)
    run_ranks(world, "nccl", layer_body, SMALL, tokens, 3, kw, 1920, transport, graph, timeout=240)
