"""Multi-rank harness shared by the CPU (gloo) and GPU (NCCL) expert-parallel tests: one process per rank, spawned with
torch.multiprocessing, rendezvous on 127.0.0.1."""

from __future__ import annotations

import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, backend, port, fn, args, errors):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    # every rank also evaluates the CPU oracle: without a share of the cores per rank the ranks' thread pools
    # oversubscribe the host (eight ranks took more than five minutes for seconds of work)
    torch.set_num_threads(max(1, (os.cpu_count() or world) // world))
    try:
        from datetime import timedelta
        limit = timedelta(seconds=90)          # a rank that failed must not keep the others waiting for long
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=limit)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=limit)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(world: int, backend: str, fn, *args, timeout: float = 600.0) -> None:
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, backend, port, fn, args, errors)) for r in range(world)]
    import time
    for p in procs:
        p.start()
    msgs = []
    deadline = time.time() + timeout
    while time.time() < deadline and any(p.is_alive() for p in procs):
        while not errors.empty():
            msgs.append("rank %d:\n%s" % errors.get())
        if msgs or any(p.exitcode not in (None, 0) for p in procs):
            break                     # one rank failed: do not wait for the others' collective timeouts
        time.sleep(0.2)
    # After a failure the other ranks leave by themselves: their device-side waits are bounded (seconds) and their next
    # collective ends with the process group's timeout.  Give them that long; a rank is killed only as the last resort
    # (it holds a symmetric workspace, so a clean exit is preferred).
    grace = time.time() + (110.0 if msgs or any(p.exitcode not in (None, 0) for p in procs) else 0.0)
    while time.time() < grace and any(p.is_alive() for p in procs):
        time.sleep(0.5)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()                      # the exact processes started above
    for p in procs:
        p.join(10)
    while not errors.empty():
        msgs.append("rank %d:\n%s" % errors.get())
    assert not msgs, "\n".join(msgs)
    assert not hung, "ranks did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


# ---------------------------------------------------------------------------------------------------------------------
# rank bodies (module level so that spawn can pickle them)
# ---------------------------------------------------------------------------------------------------------------------
def agreement_body(rank, world, failing_rank):
    """The outcome of the symmetric allocation is agreed on by the whole group: one failing rank turns the peer-memory
    transport off everywhere; without a failure everyone keeps it."""
    from vllm_plugin_b200.backend.workspace import everyone_succeeded

    group = dist.group.WORLD
    cpu = torch.device("cpu")
    assert everyone_succeeded(group, rank != failing_rank, cpu) is (failing_rank < 0)
    assert everyone_succeeded(group, True, cpu) is True


def exchange_body(rank, world, num_experts, k, tokens_per_rank, seed):
    """Host logic of the EP exchanges on CPU tensors: what each rank receives and in which order, and that the return
    exchange puts every row back where its route expects it."""
    from oracle import mmoe_oracle as O
    from vllm_plugin_b200.backend import frontend as F

    group = dist.group.WORLD
    e_l = num_experts // world
    ids_all = [O.make_routing(tokens_per_rank[r], num_experts, k, seed + r, zipf_s=1.2, mask_frac=0.1)[0] for r in range(world)]
    ids = ids_all[rank]
    m = ids.shape[0]
    # what mmoe_dispatch_count / mmoe_dispatch_pack produce: routes sorted by (expert, token, slot)
    flat = ids.reshape(-1)
    routes = sorted((int(flat[i]), i) for i in range(flat.numel()) if int(flat[i]) >= 0)
    send_count = torch.bincount(torch.tensor([e for e, _ in routes], dtype=torch.int64), minlength=num_experts).to(torch.int32)
    recv_count = torch.zeros((world, e_l), dtype=torch.int32)
    send_splits, recv_splits = F.exchange_counts(group, send_count, recv_count)
    plan = O.dispatch_plan(ids_all, num_experts, rank, 16)
    assert torch.equal(recv_count.long(), plan.recv_count)                      # bit-exact receive counts
    assert send_splits == [int(send_count[r * e_l:(r + 1) * e_l].sum()) for r in range(world)]
    # rows carry (source rank, route id) so that the order can be checked after the exchange
    send_rows = torch.tensor([[rank, i] for _, i in routes], dtype=torch.int32).reshape(-1, 2)
    recv_rows = torch.full((int(sum(recv_splits)) + 3, 2), -1, dtype=torch.int32)
    F.exchange_rows(group, recv_rows, send_rows, recv_splits, send_splits)
    lo = rank * e_l
    want = []
    for src in range(world):                                                     # receive order: source, expert, token, slot
        f = ids_all[src].reshape(-1)
        want += [[src, i] for e, i in sorted((int(f[i]), i) for i in range(f.numel()) if lo <= int(f[i]) < lo + e_l)]
    assert recv_rows[: len(want)].tolist() == want
    assert bool((recv_rows[len(want):] == -1).all())
    # per-expert pool = concatenation over sources, which is the oracle's (source, token, slot) order
    k_ = ids.shape[1]
    for ex in range(e_l):
        got = [(s, i // k_, i % k_) for s, i in want if int(ids_all[s].reshape(-1)[i]) == lo + ex]
        assert sorted(got) == plan.routes[ex] and got == plan.routes[ex]
    # return path: every rank sends back what it received; rows come home in the sender's own send order
    back = torch.full((len(routes) + 2, 2), -1, dtype=torch.int32)
    F.exchange_rows(group, back, recv_rows, send_splits, recv_splits)
    assert torch.equal(back[: len(routes)], send_rows)


def layer_body(rank, world, geometry, tokens_per_rank, seed, routing_kw, t_max, transport="peer", graph=False, replicas=0):
    """Whole layer at EP = world on GPUs: per-rank output against the oracle, receive counts and statistics bit-exact."""
    import helpers as H
    from oracle import mmoe_oracle as O
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.frontend import read_status

    dev = torch.device("cuda", rank)
    layer = H.make_layer(seed=seed, **geometry)
    e, k = layer.num_experts, layer.num_topk
    if replicas:
        # load-balancer placement: the last `replicas` physical experts are copies of the hottest logical experts; the
        # router's logical ids are mapped to a physical replica by (token + slot) % copies, as the engine does before
        # the layer is called
        logical = e - replicas
        for j in range(replicas):
            layer.experts[logical + j] = layer.experts[j]
    e_l = e // world
    hid = [O.make_hidden(tokens_per_rank[r], layer.hidden, seed + 10 + r) for r in range(world)]
    routing = [O.make_routing(tokens_per_rank[r], e, k, seed + 20 + r, **routing_kw) for r in range(world)]
    ids = [r_[0] for r_ in routing]
    w = [r_[1] for r_ in routing]
    if replicas:
        logical = e - replicas
        for r in range(world):
            lid = ids[r] % logical
            lid = torch.where(ids[r] < 0, ids[r], lid)
            tok = torch.arange(lid.shape[0]).view(-1, 1)
            slot = torch.arange(k).view(1, -1)
            use_copy = (lid >= 0) & (lid < replicas) & (((tok + slot) % 2) == 1)
            ids[r] = torch.where(use_copy, lid + logical, lid)
    buf = api.get_symm_buffer_for_mega_moe(dist.group.WORLD, e, t_max, k, layer.hidden, layer.inter,
                                           1 if layer.shared is not None else 0)
    l1, l2, sl1, sl2 = H.kernel_weights(layer, dev, rank * e_l, (rank + 1) * e_l)
    stats = torch.zeros(e_l, dtype=torch.int32, device=dev)
    m = tokens_per_rank[rank]
    y = torch.empty((m, layer.hidden), dtype=torch.bfloat16, device=dev)
    fused = transport != "peer-unfused"
    if transport == "peer-unfused":
        transport = "peer"
    api.set_kernel_options(ep_transport=transport, fuse_return=fused)
    if transport == "peer":
        assert buf.peer_ptrs is not None, "symmetric memory was expected to be available"
    hid_d, ids_d, w_d = hid[rank].to(dev), ids[rank].to(dev), w[rank].to(dev)

    def call():
        api.stage_inputs_for_mega_moe(buf, hid_d, ids_d, w_d)
        api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0)

    call()
    if graph:                                                                    # second call as a CUDA-graph replay
        api.precompile_mega_moe_variants(world, e, t_max, k, layer.hidden, layer.inter, 1 if layer.shared is not None else 0)
        torch.cuda.synchronize()
        dist.barrier()
        snapshot = stats.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call()
        stats.copy_(snapshot)          # the capture itself does not run the kernels; keep "one call so far"
        y.zero_()
        g.replay()
    else:
        call()                                                                   # second call: cumulative statistics
    read_status(buf)
    if transport == "peer" and fused and not graph:
        # the write-back fused into GEMM2 and the separate copy kernel must leave identical rows
        y_fused = y.clone()
        snapshot = stats.clone()
        api.set_kernel_options(fuse_return=False)
        call()
        api.set_kernel_options(fuse_return=True)
        read_status(buf)
        stats.copy_(snapshot)
        assert torch.equal(y, y_fused), "fused and unfused write-back differ"
    bm = api.get_block_m_for_mega_moe(world, e, t_max, m, k)
    plan = O.dispatch_plan(ids, e, rank, bm)
    assert torch.equal(buf.recv_count.cpu().long(), plan.recv_count)
    hdr, total, block_off = buf.plan_tables()
    assert torch.equal(total.long(), plan.recv_total) and torch.equal(block_off.long(), plan.pool_block_offset)
    assert torch.equal(stats.cpu().long(), 2 * plan.recv_total)
    ref = O.moe_layer(hid, ids, w, layer.experts, layer.shared, 10.0, only_ranks=[rank])[rank]
    met = O.parity_metrics(y.cpu(), ref)
    assert met["rel_l2"] <= 1e-3, met
    a, b = y.float().cpu(), ref.float()
    if a.numel():
        ulp = torch.pow(2.0, torch.floor(torch.log2(b.abs().clamp(min=2.0 ** -126))) - 7)
        assert float(((a - b).abs() - torch.clamp(ulp, min=2e-2)).max()) <= 0, met


def eplb_body(rank, world, token_counts, seed):
    """Load-balancer geometry of the benchmark's configuration 4 at reduced H / I: 384 logical experts + 8 redundant
    copies of the 8 hottest ones (from a seeded Zipf(1.2) histogram) = 392 physical experts, top-6, one shared expert.
    Every token count is captured as a CUDA graph and replayed; then the weights are reloaded IN PLACE under a reshuffled
    physical -> logical map (addresses unchanged, as the layer class reloads), the routing is re-mapped, and the same
    graphs are replayed again.  A token's output does not depend on the placement, so the second replay must equal the
    first bit for bit, and both must match the oracle (cf. tests/eplb_gpu_harness.py:396-562 of the reference)."""
    import helpers as H
    from oracle import mmoe_oracle as O
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend.frontend import read_status

    dev = torch.device("cuda", rank)
    hidden, inter, k, logical_n, redundant = 512, 256, 6, 384, 8
    physical_n = logical_n + redundant
    e_l = physical_n // world
    logical = O.make_experts(logical_n, hidden, inter, seed)
    shared = O.make_shared_expert(hidden, inter, seed + 1000)
    g = torch.Generator().manual_seed(seed + 1)
    pop = 1.0 / torch.arange(1, logical_n + 1, dtype=torch.float32) ** 1.2
    hist = torch.zeros(logical_n)
    hist[torch.randperm(logical_n, generator=g)] = pop
    hottest = torch.topk(hist, redundant).indices.tolist()
    placements = [list(range(logical_n)) + hottest]                         # physical slot -> logical expert
    shuffle = torch.randperm(physical_n, generator=g).tolist()
    placements.append([placements[0][p] for p in shuffle])                  # after the rebalance

    def physical_ids(logical_ids, placement):
        """Replica choice the engine makes before the layer: copy (token + slot) % copies, slots ascending."""
        slots = {}
        for p, l in enumerate(placement):
            slots.setdefault(l, []).append(p)
        out = logical_ids.clone()
        for t in range(logical_ids.shape[0]):
            for s in range(k):
                l = int(logical_ids[t, s])
                if l >= 0:
                    copies = slots[l]
                    out[t, s] = copies[(t + s) % len(copies)]
        return out

    def rank_weights(placement):
        layer = H.Layer(hidden, inter, physical_n, k, [logical[l] for l in placement], shared)
        return layer, H.kernel_weights(layer, dev, rank * e_l, (rank + 1) * e_l)

    layer0, (l1, l2, sl1, sl2) = rank_weights(placements[0])
    buf = api.get_symm_buffer_for_mega_moe(dist.group.WORLD, physical_n, 1920, k, hidden, inter, 1)
    assert world == 1 or buf.peer_ptrs is not None, "symmetric memory was expected to be available"
    api.set_kernel_options(ep_transport="peer", fuse_return=True)
    variants = api.precompile_mega_moe_variants(world, physical_n, 1920, k, hidden, inter, 1)
    assert set(api.get_block_m_for_mega_moe(world, physical_n, 1920, m, k) for m in token_counts) <= set(variants)
    stats = torch.zeros(e_l, dtype=torch.int32, device=dev)

    cases = []
    for j, m in enumerate(token_counts):
        hid = [O.make_hidden(m, hidden, seed + 100 * j + r) for r in range(world)]
        routed = [O.make_routing(m, logical_n, k, seed + 100 * j + 50 + r, zipf_s=1.2, mask_frac=0.05) for r in range(world)]
        cases.append((m, hid, [r_[0] for r_ in routed], [r_[1] for r_ in routed]))

    graphs = []
    for m, hid, lids, w in cases:
        ids_d = physical_ids(lids[rank], placements[0]).to(dev)             # updated in place before the second replay
        hid_d, w_d = hid[rank].to(dev), w[rank].to(dev)
        y = torch.empty((m, hidden), dtype=torch.bfloat16, device=dev)

        def call(hid_d=hid_d, ids_d=ids_d, w_d=w_d, y=y):
            api.stage_inputs_for_mega_moe(buf, hid_d, ids_d, w_d)
            api.fp8_fp4_mega_moe(y, l1, l2, buf, sl1, sl2, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0)

        call()                                                               # warm-up outside capture
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
        graphs.append((graph, ids_d, y, (hid_d, w_d)))       # the graph reads these buffers at every replay: keep them

    def replay_all(placement):
        outs = []
        for (graph, ids_d, y, _inputs), (m, hid, lids, w) in zip(graphs, cases):
            ids_d.copy_(physical_ids(lids[rank], placement))
            y.zero_()
            stats.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            graph.replay()
            read_status(buf)
            phys = [physical_ids(lids[r], placement) for r in range(world)]
            bm = api.get_block_m_for_mega_moe(world, physical_n, 1920, m, k)
            plan = O.dispatch_plan(phys, physical_n, rank, bm)
            assert torch.equal(buf.recv_count.cpu().long(), plan.recv_count), f"receive counts, M={m}"
            assert torch.equal(stats.cpu().long(), plan.recv_total), f"statistics, M={m}"
            layer = H.Layer(hidden, inter, physical_n, k, [logical[l] for l in placement], shared)
            ref = O.moe_layer(hid, phys, w, layer.experts, shared, 10.0, only_ranks=[rank])[rank]
            met = O.parity_metrics(y.cpu(), ref)
            assert met["rel_l2"] <= 1e-3, (m, met)
            outs.append(y.clone())
        return outs

    first = replay_all(placements[0])
    # reload in place under the reshuffled map: same tensors, same addresses, new rows
    _, (n1, n2, _, _) = rank_weights(placements[1])
    before = (l1[0].data_ptr(), l1[1].data_ptr(), l2[0].data_ptr(), l2[1].data_ptr())
    for dst, src in ((l1[0], n1[0]), (l1[1], n1[1]), (l2[0], n2[0]), (l2[1], n2[1])):
        dst.copy_(src)
    assert before == (l1[0].data_ptr(), l1[1].data_ptr(), l2[0].data_ptr(), l2[1].data_ptr())
    torch.cuda.synchronize()
    dist.barrier()
    second = replay_all(placements[1])
    for a, b, (m, *_rest) in zip(first, second, cases):
        assert torch.equal(a, b), f"output changed with the placement at M={m}"
