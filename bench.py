"""Benchmark of the MegaMoE expert layer (routed MXFP8 x MXFP4 experts + one fused FP8 shared expert).

    python bench.py --gpus N --steps K --warmup W              # this backend (CUDA, sm_100a)
    python bench.py --impl reference --gpus N --steps K --warmup W   # the reference arithmetic on the host cores

One step = one pass of the hot path over one batch of synthetic input: input staging (BF16 -> MXFP8) + the layer call.
Workload at N = 1: H=5120, I=2304, E=384 physical experts, top-6, one shared expert, all experts resident, M=3840
tokens; at N > 1 the experts are sharded E/N per rank (expert parallelism) and every rank brings M=3840 tokens of its
own (weak scaling).  Inputs are seeded synthetic tensors with the shapes and distributions of the reference's harness.
Every step streams far more distinct weight bytes than the 126 MB L2 holds, so no cache flush is needed between steps;
the decode points of the sweep rotate through several routings for the same reason.

After the timed regions every rank checks what it computed: per-expert receive counts and the cumulative statistics
against a bincount of all ranks' routing (bit-exact), and a seeded sample of its output tokens against the CPU oracle
(the checker; never inside a timed region).

Prints ONE JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, K = 5120, 2304, 384, 6
M_HEADLINE = 3840
SWEEP = (1, 8, 64, 256, 1024, 2048, 3840)
# DRAM read + write of the grouped-GEMM1 launches over what they must move (weights and weight scales of the experts
# hit, FP8 token rows and scales in, FP8 activations and scales out), from ncu captures of small cases: weights-as-A
# kernels at E=64 / M=640 (867.5 MB measured / 860.8 MB), tokens-as-A kernels at E=8 / M=640 (157.5 / 158.9 MB, the
# last activation rows still in L2 when the kernel ends).  Both parts grow in proportion to the experts and tokens.
NCU_TRAFFIC_RATIO_GEMM1 = {"weights-as-A": 1.008, "tokens-as-A": 0.991}
# tensor pipe rate of `tcgen05.mma.kind::mxf8f6f4.block_scale` measured with back-to-back instructions (M=128, N>=160):
# 8190 MAC per clock and SM, i.e. the nominal 8192
TENSOR_MAC_PER_CLK_SM = 8192
NUM_SMS = 148
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
CONFIG0 = dict(experts=32, tokens=128)       # the benchmark's CPU-runnable configuration


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons of one GPU every few milliseconds through NVML while a
    timed region runs (read-only queries)."""

    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mask = [], 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - no NVML: the clocks entry reports no samples
            self._nvml = None

    def _loop(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                self.mask |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
            except Exception:  # noqa: BLE001
                break
            time.sleep(0.002)

    def start(self):
        if self._nvml is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        reasons = [name for name, bit in self.REASONS if self.mask & bit]
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


# ---------------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle (a restatement of the reference's arithmetic; the reference ships no CPU
# forward of the layer) on the host cores, on a bounded sample of the workload
# ---------------------------------------------------------------------------------------------------------------------
def config0_workload() -> str:
    return (f"config 0 of the benchmark (the CPU-runnable case): MegaMoE layer H={H} I={I} E={CONFIG0['experts']} top-{K} "
            f"1 shared expert, EP1, M={CONFIG0['tokens']}")


def cpu_reference(steps: int, warmup: int, want_output: bool = False):
    """Times the oracle on config 0 (E=32 resident experts, M=128): the headline geometry's 384 experts would need 54 GB
    as FP32.  Returns (tokens/s, seconds per pass, cores, sample description[, inputs and output for a same-config check])."""
    from oracle import mmoe_oracle as O
    cores = os.cpu_count() or 1
    try:
        os.sched_setaffinity(0, range(cores))       # the CPU arm uses every host core, whatever the GPU arm was bound to
    except OSError:
        pass
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    e_sample, m_sample = CONFIG0["experts"], CONFIG0["tokens"]
    experts = O.make_experts(e_sample, H, I, seed=0)
    shared = O.make_shared_expert(H, I, seed=1000)
    deq = [ew.dequant() for ew in experts]          # dequantisation happens once, outside the timed region
    sdeq = shared.dequant()
    hid = O.make_hidden(m_sample, H, 0)
    ids, w = O.make_routing(m_sample, e_sample, K, 0)
    times = []
    y = None
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        y = O.moe_layer([hid], [ids], [w], experts, shared, 10.0, dequantized=deq, shared_dequantized=sdeq)[0]
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    sample = (f"config 0: M={m_sample} tokens, top-{K}, {e_sample} resident experts (FP32-dequantised weights of the headline's "
              f"{E} experts would need 54 GB), one shared expert; quantise+dispatch+GEMM1+SwiGLU/requant+GEMM2+combine, "
              f"weight dequantisation excluded; median of {len(times)} passes")
    if want_output:
        return m_sample / t, t, cores, sample, (experts, shared, hid, ids, w, y)
    return m_sample / t, t, cores, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 8))
    value, t, cores, sample = cpu_reference(steps, min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 2), "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (dequantised MXFP8 x MXFP4)", "data": "synthetic",
        "config": {"workload": config0_workload(),
                   "same_config_as_gpu_arm": False,
                   "gpu_arm_same_config_point": "sweep.config0 of the GPU arm's line (N=1) runs exactly this workload",
                   "impl_note": "CPU restatement of the reference arithmetic (the reference ships no CPU forward and its "
                                "GPU kernel runs on compute capability 10.7 only); the headline workload (E=384) does not "
                                "fit host memory as FP32, so this arm times the benchmark's CPU-runnable configuration"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# this backend
# ---------------------------------------------------------------------------------------------------------------------
def bind_to_gpu_cores(local_rank: int) -> None:
    """Run this process on the CPU cores NVML reports as local to its GPU (best effort; a serving engine does the same
    so that pinned staging buffers and the copy engines share a NUMA node)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = int(visible.split(",")[local_rank]) if visible and visible.split(",")[local_rank].isdigit() else local_rank
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cores = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        cores &= set(os.sched_getaffinity(0))
        if cores:
            os.sched_setaffinity(0, cores)
    except Exception:
        pass


def graph_latency(layer_call, sets, out, dev, reps):
    """p50 / p90 latency (us) of one layer call replayed from CUDA graphs, one graph per input set, rotating."""
    stream = torch.cuda.current_stream(dev)
    graphs = []
    side = torch.cuda.Stream(dev)
    for hs, is_, ws in sets:
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            for _ in range(2):
                layer_call(hs, is_, ws, out)
        stream.wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            layer_call(hs, is_, ws, out)
        graphs.append(g)
    for j in range(3):
        graphs[j % len(graphs)].replay()
    es = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for j in range(reps):
        es[j][0].record(stream)
        graphs[j % len(graphs)].replay()
        es[j][1].record(stream)
    torch.cuda.synchronize(dev)
    lat = sorted(a.elapsed_time(b) * 1e3 for a, b in es)
    del graphs
    return lat[len(lat) // 2], lat[int(len(lat) * 0.9)]


def run_ours(args):
    import ctypes

    from vllm_plugin_b200 import api
    from vllm_plugin_b200.backend import _native
    from vllm_plugin_b200.backend.frontend import read_status
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    from vllm_plugin_b200.testing import SyntheticLayer, layer_work, make_hidden, make_routing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    group = SingleRankGroup()
    if world > 1:
        # the exchange uses plain peer stores: no NVLink multicast object is bound to the symmetric workspace
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    e_local = E // world
    t_cap = 3840
    sampler = ClockSampler(local_rank)      # NVML is initialised before anything is timed
    bind_to_gpu_cores(local_rank)           # pinned host buffers are first touched on the GPU's own NUMA node

    syn = SyntheticLayer(H, I, e_local, True, dev, seed=0, first_expert=rank * e_local)
    buf = api.get_symm_buffer_for_mega_moe(group, E, t_cap, K, H, I, 1)
    api.precompile_mega_moe_variants(world, E, t_cap, K, H, I, 1, activation_clamp=10.0)
    api.set_kernel_options(ep_transport="nccl" if args.ep_transport == "nccl" else "peer",
                           fuse_return=args.ep_transport == "peer", orientation=args.orientation)
    lib = _native.load()
    stats = torch.zeros(e_local, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev)
    peak_hbm, peak_kind = measured_peaks()

    def inputs(m, seed):
        hid = make_hidden(m, H, seed + 17 * rank, dev)
        ids, w = make_routing(m, E, K, seed + 31 * rank, dev)
        return hid, ids, w

    def layer_call(hid, ids, w, y):
        api.stage_inputs_for_mega_moe(buf, hid, ids, w)
        api.fp8_fp4_mega_moe(y, syn.l1, syn.l2, buf, syn.shared_l1, syn.shared_l2,
                             cumulative_local_expert_recv_stats=stats, activation_clamp=10.0, fast_math=True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def reduce_ranks(value: float, op: str = "max") -> float:
        if dist is None:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN}[op])
        return float(t.item())

    # ---- headline: K timed steps at M = 3840 per rank, inputs resident in HBM ----------------------------------
    m = M_HEADLINE
    hid, ids, w = inputs(m, 1)
    y = torch.empty((m, H), dtype=torch.bfloat16, device=dev)
    for _ in range(max(args.warmup, 3)):
        layer_call(hid, ids, w, y)
    barrier()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        layer_call(hid, ids, w, y)
    ev1.record(stream)
    barrier()
    step_ms = reduce_ranks(ev0.elapsed_time(ev1) / args.steps)
    value = world * m / (step_ms * 1e-3)
    # EP1: quantiser, 3 route-ordering passes, plan, place, shared-expert plan, 2 shared-expert GEMMs (running beside
    # the ordering / placement on a second stream), 2 routed GEMMs, combine = 12 (6 at M <= 128: one fused ordering/plan
    # launch and one launch per GEMM).  The peer exchange adds publish, push, 2 flag waits and a flag kernel (17);
    # its unfused form has one launch per GEMM and a return copy (14); NCCL: the pack kernel, one launch per GEMM (10)
    launches_per_step = (12 if m > 128 else (6 if m * K > 128 else 5)) if world == 1 else {"nccl": 10, "peer-unfused": 14, "peer": 17}[args.ep_transport]

    # ---- eager host cost of one call (staging + layer), microseconds of CPU time per call with nothing to wait for
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(10):
        layer_call(hid, ids, w, y)
    host_us = (time.perf_counter() - t0) / 10 * 1e6
    barrier()

    # ---- end to end through the public API with host buffers (pinned): every step copies its inputs host -> device and
    # its result device -> host inside the timed region.  The copies of step i+1 / i-1 run on two copy streams (one per
    # direction) while step i computes (two input and two output buffers), as a serving engine pipelines them.
    hid_h, ids_h, w_h = hid.cpu().pin_memory(), ids.cpu().pin_memory(), w.cpu().pin_memory()
    y_h = [torch.empty((m, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ins = [(torch.empty_like(hid), torch.empty_like(ids), torch.empty_like(w)) for _ in range(2)]
    outs = [torch.empty((m, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    copy_stream = torch.cuda.Stream(dev)       # host -> device
    back_stream = torch.cuda.Stream(dev)       # device -> host: its own stream, the link is full duplex
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]

    def h2d(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(in_free[slot])
            ins[slot][0].copy_(hid_h, non_blocking=True)
            ins[slot][1].copy_(ids_h, non_blocking=True)
            ins[slot][2].copy_(w_h, non_blocking=True)
            in_ready[slot].record(copy_stream)

    def e2e_run(steps, compute=True):
        for ev in in_free + out_free:
            ev.record(stream)
        h2d(0)
        for i in range(steps):
            slot = i & 1
            if i + 1 < steps:
                h2d(slot ^ 1)
            stream.wait_event(in_ready[slot])
            stream.wait_event(out_free[slot])
            if compute:
                layer_call(*ins[slot], outs[slot])
            in_free[slot].record(stream)
            out_ready[slot].record(stream)
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(out_ready[slot])
                y_h[slot].copy_(outs[slot], non_blocking=True)
                out_free[slot].record(back_stream)
        stream.wait_stream(copy_stream)
        stream.wait_stream(back_stream)

    def timed_e2e(compute):
        e2e_run(3, compute)
        barrier()
        ev0.record(stream)
        e2e_run(args.steps, compute)
        ev1.record(stream)
        barrier()
        return reduce_ranks(ev0.elapsed_time(ev1) / args.steps)

    e2e_ms = timed_e2e(True)
    clocks = sampler.stop() if rank == 0 else None
    copy_only_ms = timed_e2e(False)           # the same copies with no kernel between them: what the host link alone costs
    h2d_bytes = hid_h.numel() * 2 + ids_h.numel() * 8 + w_h.numel() * 4
    d2h_bytes = y_h[0].numel() * 2

    # ---- the phases of one call timed back to back on one stream through the C ABI (the product call overlaps the
    # exchange / ordering with the shared expert on a second stream; these are the costs of the parts).  Every rank runs
    # the same sequence, the exchange kernels wait for their peers.
    geo = ctypes.byref(buf.geo)
    wst = _weights_struct(syn)
    bm = api.get_block_m_for_mega_moe(world, E, t_cap, m, K)
    opts1 = _native.MmoeOptions(10.0, 1, 0, 2000, 1)
    opts2 = _native.MmoeOptions(10.0, 1, 0, 2000, 2)
    sp = stream.cuda_stream
    ws = buf.base_ptr
    peers = (ctypes.c_void_p * world)(*buf.peer_ptrs) if world > 1 and buf.peer_ptrs is not None else None
    # past 128 tokens the product call runs the shared expert as launches of its own (tiles planned from the token
    # count alone) and the routed experts as one launch per GEMM; the phases are timed in that structure
    split = m > 128
    opts0 = _native.MmoeOptions(10.0, 1, 0, 2000, 0)
    names = ["stage", "order", "exchange", "place", "shared", "gemm1", "gemm2", "return", "combine"]
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
    acc = {n: [] for n in names}
    can_time_phases = world == 1 or peers is not None
    for it in range((3 + min(args.steps, 10)) if can_time_phases else 0):
        evs[0].record(stream)
        api.stage_inputs_for_mega_moe(buf, hid, ids, w)
        evs[1].record(stream)
        _native.check(lib.mmoe_dispatch_count(geo, ws, m, sp))
        evs[2].record(stream)
        if world > 1:
            _native.check(lib.mmoe_ep_dispatch(geo, ws, peers, m, ctypes.byref(opts1), sp))
        evs[3].record(stream)
        _native.check(lib.mmoe_dispatch_place(geo, ws, m, bm, None, sp))
        evs[4].record(stream)
        if split:
            _native.check(lib.mmoe_plan_shared(geo, ws, m, bm, sp))
            _native.check(lib.mmoe_experts_select(geo, ws, ctypes.byref(wst), ctypes.byref(opts0), m, bm, 2, sp))
        evs[5].record(stream)
        if split:
            _native.check(lib.mmoe_experts_select(geo, ws, ctypes.byref(wst), ctypes.byref(opts1), m, bm, 1, sp))
        else:
            _native.check(lib.mmoe_experts(geo, ws, ctypes.byref(wst), ctypes.byref(opts1), m, bm, sp))
        evs[6].record(stream)
        if split:
            _native.check(lib.mmoe_experts_select(geo, ws, ctypes.byref(wst), ctypes.byref(opts2), m, bm, 1, sp))
        else:
            _native.check(lib.mmoe_experts(geo, ws, ctypes.byref(wst), ctypes.byref(opts2), m, bm, sp))
        evs[7].record(stream)
        if world > 1:
            _native.check(lib.mmoe_ep_return(geo, ws, peers, ctypes.byref(opts1), sp))
        evs[8].record(stream)
        _native.check(lib.mmoe_combine(geo, ws, y.data_ptr(), m, sp))
        evs[9].record(stream)
        torch.cuda.synchronize(dev)
        if it >= 3:
            for j, n in enumerate(names):
                acc[n].append(evs[j].elapsed_time(evs[j + 1]))
    barrier()
    phases = {n + "_ms": reduce_ranks(statistics.mean(v)) for n, v in acc.items() if v} if can_time_phases else {}

    # ---- algorithmic work of this rank's share of the step
    all_ids = ids
    if dist is not None:
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        all_ids = torch.cat(gathered)
    mine = all_ids[(all_ids >= rank * e_local) & (all_ids < (rank + 1) * e_local)]
    routes_here = int(mine.numel())
    distinct_here = int(torch.unique(mine).numel())
    flops_here, bytes_here = layer_work(routes_here, m, distinct_here, H, I, True)
    flops_mean = reduce_ranks(float(flops_here), "sum") / world
    bytes_mean = reduce_ranks(float(bytes_here), "sum") / world
    distinct_mean = reduce_ranks(float(distinct_here), "sum") / world
    pairs_mean = reduce_ranks(float(routes_here + m), "sum") / world       # (token, expert) pairs incl. the shared expert
    expected_rows = m * world * K / E
    family = {0: "tokens-as-A" if (bm >= 64 and expected_rows >= 80) else "weights-as-A", 1: "weights-as-A",
              2: "tokens-as-A", 3: "tokens-as-A"}[args.orientation]
    kernel_name = ("tm_kernel<1> (grouped GEMM1 + SwiGLU/requant, tokens-as-A)" if family == "tokens-as-A"
                   else "umma_kernel<1> (grouped GEMM1 + SwiGLU/requant, weights-as-A)")
    kernel_name += ", the launch over the routed experts' tiles" if m > 128 else ", one launch over routed and shared tiles"
    sm_mhz = float((clocks or {}).get("sm_mhz") or 0.0)
    sm_mhz = reduce_ranks(sm_mhz, "max") or 1965.0                               # rank 0 samples its GPU
    tensor_peak = 2 * TENSOR_MAC_PER_CLK_SM * NUM_SMS * sm_mhz * 1e6 / 1e12      # TFLOP/s at the sampled SM clock
    tensor_peak_max = 2 * TENSOR_MAC_PER_CLK_SM * NUM_SMS * 1965.0 * 1e6 / 1e12
    roofline = None
    kernels = dict(phases)
    if "gemm1_ms" in phases:
        g1_ms, g2_ms = phases["gemm1_ms"], phases["gemm2_ms"]
        # rows and weights of the timed launches: the routed experts alone when the shared expert has its own launches
        shared_rows = 0 if split else m
        rows = pairs_mean - m + shared_rows
        pairs_mean = rows
        g1_flops, g2_flops = rows * 4 * I * H, rows * 2 * I * H
        w13_bytes = distinct_mean * (I * H + 2 * I * H // 32) + (0 if split else 2 * I * H + 2 * I * H // 32)
        w2_bytes = distinct_mean * (H * I // 2 + H * I // 32) + (0 if split else H * I + H * I // 32)
        g1_tflops, g1_gbs = g1_flops / (g1_ms * 1e-3) / 1e12, w13_bytes / (g1_ms * 1e-3) / 1e9
        tensor_bound = g1_flops / (tensor_peak * 1e12) > w13_bytes / (peak_hbm * 1e9)
        token_side_bytes = pairs_mean * (H + H // 32 + I + I // 32)     # FP8 rows + scales in, activations + scales out
        common = {"kernel": kernel_name, "traffic": (w13_bytes + token_side_bytes) * NCU_TRAFFIC_RATIO_GEMM1[family],
                  "traffic_source": "DRAM read+write over (weight bytes + token rows in + activations out) from the ncu capture "
                                    "of a small case of this kernel, scaled by the experts hit and the rows processed",
                  "token_side_bytes_per_launch": token_side_bytes,
                  "algorithmic_bytes_per_launch": w13_bytes, "algorithmic_flops_per_launch": g1_flops, "ms_per_launch": g1_ms}
        if tensor_bound:
            roofline = {"bound": "tensor", "achieved": g1_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                        "frac": g1_tflops / tensor_peak,
                        "peak_kind": "of measured: 8192 MAC/clk/SM (back-to-back tcgen05.mma kind::mxf8f6f4.block_scale "
                                     f"micro-benchmark) x 148 SMs at the SM clock sampled during the run ({sm_mhz:.0f} MHz)",
                        "peak_at_max_clock": tensor_peak_max, "frac_of_peak_at_max_clock": g1_tflops / tensor_peak_max,
                        **common}
        else:
            roofline = {"bound": "hbm", "achieved": g1_gbs, "peak": peak_hbm, "unit": "GB/s", "frac": g1_gbs / peak_hbm,
                        "peak_kind": f"of {peak_kind}", **common}
        kernels.update({
            "gemm1_tflops": g1_tflops, "gemm2_tflops": g2_flops / (g2_ms * 1e-3) / 1e12,
            "gemm1_gbs": g1_gbs, "gemm2_gbs": w2_bytes / (g2_ms * 1e-3) / 1e9,
            "gemm1_tensor_frac": g1_tflops / tensor_peak, "gemm2_tensor_frac": g2_flops / (g2_ms * 1e-3) / 1e12 / tensor_peak})
    kernels.update({
        "kernel_family": family,
        "phase_note": "phases timed back to back on one stream in the product call's launch structure (past 128 tokens: "
                      "shared_ms = the shared expert's two GEMM launches, gemm1_ms / gemm2_ms = the routed experts' "
                      "launches); the product call overlaps ordering / exchange with the shared expert",
        "layer_tflops_per_gpu": flops_mean / (step_ms * 1e-3) / 1e12,
        "layer_tensor_frac": flops_mean / (step_ms * 1e-3) / 1e12 / tensor_peak,
        "layer_algorithmic_gbs_per_gpu": bytes_mean / (step_ms * 1e-3) / 1e9,
        "layer_hbm_frac": bytes_mean / (step_ms * 1e-3) / 1e9 / peak_hbm,
        "tensor_peak_tflops_at_sampled_clock": tensor_peak})
    line_extra = {"kernels": kernels}

    # ---- self-check of what was just timed (the oracle is the checker here, outside every timed region) ------------
    line_extra["parity"] = self_check(syn, buf, hid, ids, w, y, all_ids, rank, world, e_local, dev, reduce_ranks)

    if world == 1:
        # ---- token sweep (latency per call; decode points rotate through 8 routings so weights come from HBM) ----
        sweep = {}
        for ms in SWEEP if not args.no_sweep else ():
            # each point is captured once as a CUDA graph per input set and replayed (the reference publishes CUDA-graph
            # latencies); the sets rotate so that consecutive replays hit different experts and weights come from HBM
            sets = [inputs(ms, 100 + j) for j in range(8 if ms <= 256 else 2)]
            ys = torch.empty((ms, H), dtype=torch.bfloat16, device=dev)
            p50, p90 = graph_latency(layer_call, sets, ys, dev, 24 if ms <= 256 else 8)
            uniq = statistics.mean(int(torch.unique(s[1]).numel()) for s in sets)
            fl, nb = layer_work(ms * K, ms, int(round(uniq)), H, I, True)
            sweep[str(ms)] = {"p50_us": p50, "p90_us": p90, "tokens_per_s": ms / (p50 * 1e-6),
                              "gbs": nb / (p50 * 1e-6) / 1e9, "hbm_frac": nb / (p50 * 1e-6) / 1e9 / peak_hbm,
                              "tflops": fl / (p50 * 1e-6) / 1e12, "experts_hit": uniq, "cuda_graph": True}
        line_extra["sweep"] = sweep
        if "64" in sweep:
            line_extra["p50_us_at_M64"] = sweep["64"]["p50_us"]

        # ---- load-time weight transform (checkpoint row order -> kernel layout) of all routed W13: read once, written once
        if not args.no_sweep:
            pair = (syn.l1[0], syn.l1[1])
            api.transform_weights_for_mega_moe(pair, (syn.l2[0], syn.l2[1]))     # warm-up
            tt = []
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                out = api.transform_weights_for_mega_moe(pair, (syn.l2[0], syn.l2[1]))
                e1.record(stream)
                torch.cuda.synchronize(dev)
                tt.append(e0.elapsed_time(e1))
                del out
            moved = 2 * (syn.l1[0].numel() + syn.l1[1].numel() * 4 + syn.l2[1].numel() * 4)
            t_ms = statistics.median(tt)
            line_extra["weight_transform"] = {"ms": t_ms, "bytes_read_plus_written": moved, "gbs": moved / (t_ms * 1e-3) / 1e9,
                                              "hbm_frac": moved / (t_ms * 1e-3) / 1e9 / peak_hbm}

    read_status(buf)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp8 x mxfp4 (e4m3 x e2m1, ue8m0 scales per 32), fp32 accumulate, bf16 out", "data": "synthetic",
            "config": {"workload": f"MegaMoE layer H={H} I={I} E={E} top-{K} 1 shared expert, EP{world}, M={m}/rank",
                       "parallelism": f"ep{world}", "ep_transport": args.ep_transport if world > 1 else None, "l2": "inputs larger than L2 (each step streams the packed weights of every expert hit)"},
            "e2e": {"value": world * m / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "ms_per_step": e2e_ms, "copy_only_ms": copy_only_ms,
                    "copy_only_h2d_gbs_per_rank": h2d_bytes / (copy_only_ms * 1e-3) / 1e9,
                    "copy_only_d2h_gbs_per_rank": d2h_bytes / (copy_only_ms * 1e-3) / 1e9},
            "host_us_per_call": host_us,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if roofline is not None:
            line["roofline"] = roofline
        line.update(line_extra)
        if world == 1 and not args.no_cpu_baseline:
            pair_pt, cpu = config0_pair(api, dev, peak_hbm)
            line["cpu_baseline"] = cpu
            line.setdefault("sweep", {})["config0"] = pair_pt
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def self_check(syn, buf, hid, ids, w, y, all_ids, rank, world, e_local, dev, reduce_ranks):
    """One more (untimed) call, then: receive counts of this rank's experts and the cumulative statistics against a
    bincount of ALL ranks' routing (bit-exact), and 8 sampled output tokens of this rank against the CPU oracle, which
    dequantises one expert at a time (any rank can regenerate any expert of the synthetic layer from its seed)."""
    from oracle import mmoe_oracle as O
    from vllm_plugin_b200 import api
    from vllm_plugin_b200.testing import routed_expert_raw

    stats = torch.zeros(e_local, dtype=torch.int32, device=dev)
    api.stage_inputs_for_mega_moe(buf, hid, ids, w)
    api.fp8_fp4_mega_moe(y, syn.l1, syn.l2, buf, syn.shared_l1, syn.shared_l2, cumulative_local_expert_recv_stats=stats,
                         activation_clamp=10.0, fast_math=True)
    torch.cuda.synchronize(dev)
    want = torch.bincount(all_ids[all_ids >= 0].flatten().cpu(), minlength=e_local * world)[rank * e_local:(rank + 1) * e_local]
    _, total, _ = buf.plan_tables()
    counts_exact = bool(torch.equal(stats.cpu().long(), want)) and bool(torch.equal(total.long(), want))
    m = hid.shape[0]
    sample = torch.randperm(m, generator=torch.Generator().manual_seed(7 + rank))[:8]
    hid_s, ids_s, w_s = hid[sample.to(dev)].cpu(), ids[sample.to(dev)].cpu(), w[sample.to(dev)].cpu()
    q, sf, ids_q, w_q, _ = O.stage_inputs(hid_s, ids_s, w_s, None)
    sfb = O.unpack_sf_words(sf)
    n = ids_q.shape[0]
    slot_out = torch.zeros((ids_q.shape[1], n, hid.shape[1]), dtype=torch.bfloat16)
    for e in torch.unique(ids_q[ids_q >= 0]).tolist():
        raw = [t.cpu() for t in routed_expert_raw(syn.hidden, syn.inter, 0, e, dev)]
        w13, w2 = O.ExpertWeights(*raw).dequant()
        tok, slot = torch.nonzero(ids_q == e, as_tuple=True)
        slot_out[slot, tok] = O.expert_forward(q[tok], sfb[tok], w_q[tok, slot], w13, w2, 10.0)
    s13, s2 = O.ExpertWeights(*[t.cpu() for t in syn.shared_raw], fp8=True).dequant()
    sh = O.expert_forward(q, sfb, torch.ones(n), s13, s2, 10.0)
    ref = O.combine(slot_out, ids_q, sh).float()
    got = y[sample.to(dev)].float().cpu()
    d = (got - ref).abs()
    ulp = torch.pow(2.0, torch.floor(torch.log2(ref.abs().clamp(min=2.0 ** -126))) - 7)
    within = bool(((d - torch.clamp(ulp, min=2e-2)) <= 0).all())
    rel = float((got - ref).norm() / ref.norm().clamp(min=1e-30))
    return {
        "checked": "8 sampled tokens per rank against the CPU oracle; receive counts and statistics of every local expert "
                   "against a bincount of all ranks' routing",
        "rel_l2": reduce_ranks(rel, "max"), "max_abs_strict": reduce_ranks(float(d.max()), "max"),
        "n_over_2e-2": int(reduce_ranks(float((d > 2e-2).sum()), "sum")), "n_elements": int(reduce_ranks(float(d.numel()), "sum")),
        "within_max_2e-2_or_1ulp": bool(reduce_ranks(1.0 if within else 0.0, "min") > 0.5),
        "counts_exact": bool(reduce_ranks(1.0 if counts_exact else 0.0, "min") > 0.5),
        "ok": bool(reduce_ranks(1.0 if (within and rel <= 1e-3 and counts_exact) else 0.0, "min") > 0.5)}


def config0_pair(api, dev, peak_hbm):
    """The same workload on both arms: config 0 (E=32, M=128) on the host cores through the oracle and on the GPU through
    the public API with the oracle's own weights; the GPU output is compared with the oracle's over all 128 tokens."""
    from vllm_plugin_b200.backend.weights import sf_to_required_layout
    from vllm_plugin_b200.backend.workspace import SingleRankGroup
    from vllm_plugin_b200.testing import layer_work

    v, t, cores, sample, (experts, shared, hid, ids, w, y_ref) = cpu_reference(3, 1, want_output=True)
    e0, m0 = CONFIG0["experts"], CONFIG0["tokens"]
    w13 = torch.stack([e.w13 for e in experts]).to(dev)
    w2 = torch.stack([e.w2 for e in experts]).to(dev)
    s13 = sf_to_required_layout(torch.stack([e.w13_sf for e in experts]).to(dev), 2 * I, H, e0)
    s2 = sf_to_required_layout(torch.stack([e.w2_sf for e in experts]).to(dev), H, I, e0)
    l1, l2 = api.transform_weights_for_mega_moe((w13, s13), (w2, s2))
    sl1, sl2 = api.transform_weights_for_mega_moe(
        (shared.w13.to(dev), sf_to_required_layout(shared.w13_sf.to(dev), 2 * I, H)),
        (shared.w2.to(dev), sf_to_required_layout(shared.w2_sf.to(dev), H, I)))
    buf0 = api.get_symm_buffer_for_mega_moe(SingleRankGroup(), e0, 1920, K, H, I, 1)
    hid_d, ids_d, w_d = hid.to(dev), ids.to(dev), w.to(dev)
    y0 = torch.empty((m0, H), dtype=torch.bfloat16, device=dev)

    def call(h_, i_, w_, out):
        api.stage_inputs_for_mega_moe(buf0, h_, i_, w_)
        api.fp8_fp4_mega_moe(out, l1, l2, buf0, sl1, sl2, activation_clamp=10.0, fast_math=True)

    # 0.6 GB of weights against a 126 MB L2: flush it before every replay with a 256 MB write, whose time is subtracted
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.int32, device=dev)

    def call_flushed(h_, i_, w_, out):
        flush.zero_()
        call(h_, i_, w_, out)

    p50_with_flush, _ = graph_latency(call_flushed, [(hid_d, ids_d, w_d)], y0, dev, 12)
    stream = torch.cuda.current_stream(dev)
    ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(6):
        ea.record(stream)
        flush.zero_()
        eb.record(stream)
        torch.cuda.synchronize(dev)
        ts.append(ea.elapsed_time(eb) * 1e3)
    p50 = p50_with_flush - statistics.median(ts)
    call(hid_d, ids_d, w_d, y0)
    torch.cuda.synchronize(dev)
    got, ref = y0.float().cpu(), y_ref.float()
    d = (got - ref).abs()
    fl, nb = layer_work(int((ids >= 0).sum()), m0, int(torch.unique(ids[ids >= 0]).numel()), H, I, True)
    point = {"workload": config0_workload(), "p50_us": p50, "tokens_per_s": m0 / (p50 * 1e-6), "cuda_graph": True,
             "l2": "flushed with a 256 MB write before every replay (its time subtracted)",
             "gbs": nb / (p50 * 1e-6) / 1e9, "hbm_frac": nb / (p50 * 1e-6) / 1e9 / peak_hbm, "tflops": fl / (p50 * 1e-6) / 1e12,
             "cpu_tokens_per_s_same_config": v, "gpu_over_cpu_same_config": (m0 / (p50 * 1e-6)) / v,
             "parity_vs_oracle_all_tokens": {"rel_l2": float((got - ref).norm() / ref.norm()), "max_abs_strict": float(d.max()),
                                             "n_over_2e-2": int((d > 2e-2).sum()), "n_elements": int(d.numel())}}
    cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    return point, cpu


def _weights_struct(syn):
    from vllm_plugin_b200.backend import _native
    w = _native.MmoeWeights()
    w.w13, w.w13_sf = syn.l1[0].data_ptr(), syn.l1[1].data_ptr()
    w.w2, w.w2_sf = syn.l2[0].data_ptr(), syn.l2[1].data_ptr()
    w.shared_w13, w.shared_w13_sf = syn.shared_l1[0].data_ptr(), syn.shared_l1[1].data_ptr()
    w.shared_w2, w.shared_w2_sf = syn.shared_l2[0].data_ptr(), syn.shared_l2[1].data_ptr()
    return w


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--experts", type=int, default=E, help="physical experts (smaller values give a small profiling case)")
    ap.add_argument("--tokens", type=int, default=M_HEADLINE, help="tokens per rank of the timed step")
    ap.add_argument("--ep-transport", default="peer", choices=("peer", "peer-unfused", "nccl"),
                    help="N > 1: device-side NVLink exchange with the write-back fused into GEMM2 (default), the same "
                         "with a separate copy kernel, or the host-driven NCCL all-to-allv")
    ap.add_argument("--orientation", type=int, default=0, choices=(0, 1, 2, 3),
                    help="grouped-GEMM kernel family: 0 chosen per call, 1 weights-as-A, 2 tokens-as-A, 3 tokens-as-A on CTA pairs")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    globals()["E"] = args.experts
    globals()["M_HEADLINE"] = args.tokens
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
