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


@pytest.mark.parametrize("world,tokens,kw", [
    (2, (70, 33), dict(zipf_s=1.2, mask_frac=0.05, hot=2)),
    (2, (1, 0), {}),
    (4, (130, 64, 7, 300), dict(zipf_s=1.2, mask_frac=0.05)),
])
def test_layer_matches_oracle_at_ep(world, tokens, kw):
    _need(world)
    run_ranks(world, "nccl", layer_body, SMALL, tokens, 3, kw, 1920, timeout=600)
