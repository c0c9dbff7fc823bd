"""Expert-parallel host logic with world_size 2 and 3 on CPU (gloo ranks): count exchange, row exchange order, return
path.  No GPU and no CUDA library call: the exchanges are device-agnostic torch.distributed code."""

import pytest

from ep_harness import agreement_body, exchange_body, run_ranks


@pytest.mark.parametrize("world,num_experts,k,tokens", [(2, 16, 4, (37, 5)), (2, 8, 2, (0, 9)), (3, 12, 3, (11, 20, 1))])
def test_exchanges_with_gloo_ranks(world, num_experts, k, tokens):
    run_ranks(world, "gloo", exchange_body, num_experts, k, tokens, 7, timeout=180)


@pytest.mark.parametrize("world,failing_rank", [(2, 1), (3, 0), (2, -1)])
def test_transport_choice_is_agreed_on_by_the_whole_group(world, failing_rank):
    run_ranks(world, "gloo", agreement_body, failing_rank, timeout=120)
