"""Benchmark of the MoE layer: forward + backward tokens/s on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c4layer|c5] [--impl reference]

Prints ONE JSON line (rank 0).  ``value`` is whole-job tokens/s with inputs resident in HBM;
``e2e`` is the same metric through the public layer with HOST buffers (pinned inputs copied in,
outputs copied back, inside the timed region); ``roofline`` describes the dominant kernel (the
tcgen05 grouped GEMM) against the measured bf16 peak; ``cpu_baseline`` is the CPU oracle timed on
this host on a bounded token sample.  ``--impl reference`` times that CPU implementation alone.

Workloads are the synthetic shapes of the upstream project's MoE layer study: c2 = 16384 tokens,
d 1024, 8 experts top-2, hidden 2816; c3 = 32768 tokens, d 2048, 64 experts top-6, hidden 1408,
skewed routing (per-expert router bias N(0, 0.5), realised as a constant-one input column);
c4layer = one layer of the 12-layer decoder (65536 tokens, d 1024, 16 experts top-2, hidden 2048);
c5 = c3's layer on 64 tokens (decode latency, forward only).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c2": dict(tokens=16384, d=1024, E=8, k=2, h=2816, router_std=0.01, bias_std=0.0),
    "c3": dict(tokens=32768, d=2048, E=64, k=6, h=1408, router_std=0.02, bias_std=0.5),
    "c4layer": dict(tokens=65536, d=1024, E=16, k=2, h=2048, router_std=0.02, bias_std=0.0),
    # c3 cut to a quarter of the tokens and experts (same rows per expert, same tile shapes): small enough for a profiler capture
    "c3s": dict(tokens=8192, d=2048, E=16, k=6, h=1408, router_std=0.02, bias_std=0.5),
    "c5": dict(tokens=64, d=2048, E=64, k=6, h=1408, router_std=0.02, bias_std=0.5),
}
# DRAM bytes (read + written) of the five expert tensor-core launches of one step, from profiler captures of the
# same command (profiles/grouped_gemm_c2_ncu_full.md, profiles/grouped_gemm_c3s_ncu_full.md); c3 is too large to
# capture and has exactly four times c3s's experts and tokens at the same rows per expert: 4 x the c3s figure
GEMM_DRAM_BYTES_PER_STEP = {"c2": 3.74e9, "c3s": 4.70e9, "c3": 4 * 4.70e9}
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            peaks = json.load(handle)
        return dict(hbm_gbs=float(peaks["hbm_gbs"]), bf16_tflops=float(peaks["bf16_tflops"]),
                    bf16_tflops_sustained=float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
                    source="measured")
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


def layer_flops(w, tokens=None):
    """Algorithmic FLOPs of one forward + backward: expert GEMMs 18*A*d*h, router 6*T*d*E."""
    T = w["tokens"] if tokens is None else tokens
    return 18.0 * T * w["k"] * w["d"] * w["h"], 6.0 * T * w["d"] * w["E"]


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        # samples under load: the upper half (the sampler also sees the idle edges of the region)
        busy = clocks[len(clocks) // 2:] if clocks else []
        median = busy[len(busy) // 2] if busy else None
        return dict(sm_mhz=median, sm_max_mhz=max_clock, samples=len(clocks), reasons=sorted(reasons))


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (a numpy float64 restatement of the upstream pure-Python CPU path)
# ------------------------------------------------------------------------------------------------
def cpu_sample_inputs(w, sample_tokens, seed=0):
    import numpy as np

    rng = np.random.default_rng(seed)
    d, E, h = w["d"], w["E"], w["h"]
    x = rng.standard_normal((sample_tokens, d))
    router = rng.standard_normal((E, d)) * w["router_std"]
    if w["bias_std"]:
        x[:, d - 1] = 1.0
        router[:, d - 1] = rng.standard_normal(E) * w["bias_std"]
    # one weight block shared by all experts: values do not change the cost, and 64 distinct
    # float64 expert matrices would need several GB and tens of seconds just to draw
    gate = [rng.standard_normal((h, d)) / np.sqrt(d)] * E
    up = [rng.standard_normal((h, d)) / np.sqrt(d)] * E
    down = [rng.standard_normal((d, h)) / np.sqrt(h)] * E
    grad = rng.standard_normal((sample_tokens, d))
    return x, router, gate, up, down, grad


def cpu_step(w, inputs):
    from oracle import moe_oracle as oracle

    x, router, gate, up, down, grad = inputs
    y, aux, ctx = oracle.moe_forward(x, router, gate, up, down, w["k"])
    oracle.moe_backward(ctx, grad, 0.01)
    return y


def pure_python_rate():
    """Multiply-accumulates per second of the scalar triple loop the upstream CPU path runs
    (measured on a small product; the upstream layer is that loop almost entirely)."""
    from array import array
    from oracle import moe_pure

    n = 48
    a = array("d", [0.5] * (n * n))
    start = time.perf_counter()
    moe_pure.gemm(a, a, n, n, n, transpose_right=True)
    return n ** 3 / (time.perf_counter() - start)


def time_cpu(w, steps, warmup, sample_tokens):
    inputs = cpu_sample_inputs(w, sample_tokens)
    for _ in range(warmup):
        cpu_step(w, inputs)
    start = time.perf_counter()
    for _ in range(steps):
        cpu_step(w, inputs)
    seconds = (time.perf_counter() - start) / steps
    return sample_tokens / seconds, seconds


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_sample_tokens(w):
    # about 1e11 algorithmic FLOP per step: a second or two of multi-threaded float64 BLAS
    flops_per_token = sum(layer_flops(w, 1))
    return int(max(16, min(w["tokens"], 1.0e11 // flops_per_token)))


def run_reference(args, w, rank):
    if rank != 0:
        return
    sample = cpu_sample_tokens(w)
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    value, seconds = time_cpu(w, steps, warmup, sample)
    cores = host_cores()
    line = dict(
        impl="reference", metric="moe_layer_fwd_bwd_tokens_per_s", value=value, unit="tokens/s",
        n_gpus=args.gpus, steps=steps, warmup=warmup, ms_per_step=seconds * 1e3, higher_is_better=True,
        scaling="strong", vs_baseline=None, dtype="f64", data="synthetic",
        config=workload_config(args.workload, w, args.gpus),
        cpu_baseline=dict(value=value, unit="tokens/s", cores=cores, kind="port",
                          sample=f"{sample} of {w['tokens']} tokens per step, full d/E/k/h, numpy float64 "
                                 f"restatement of the upstream pure-Python CPU path, BLAS on {cores} threads"),
        e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def workload_config(name, w, gpus):
    return dict(workload=f"{name}: MoE layer fwd+bwd, tokens {w['tokens']}, d_model {w['d']}, experts {w['E']}, "
                         f"top_k {w['k']}, d_expert {w['h']}", tokens=w["tokens"], d_model=w["d"], n_experts=w["E"],
                top_k=w["k"], d_expert=w["h"], parallelism=f"ep{gpus}" if gpus > 1 else "single",
                l2="inputs larger than L2 (weights and activations are re-streamed every step)")


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_layer(w, torch, device, seed=0):
    import numpy as np

    from qutai_b200 import lib
    from qutai_b200.layers import SparseMoE

    class Cfg:
        d_model, n_experts, top_k, d_expert, n_layers = w["d"], w["E"], w["k"], w["h"], 1

    layer = SparseMoE(Cfg, device="cuda", dtype="float32", seed=seed)
    d, E, h = w["d"], w["E"], w["h"]
    fill = lambda storage, std, key: lib.call("qmoe_normal_fill", storage.ptr, lib.QMOE_F32, storage.size, 0.0, std, key, 0)
    fill(layer._gate, d ** -0.5, 101)
    fill(layer._up, d ** -0.5, 102)
    fill(layer._down, h ** -0.5, 103)
    rng = np.random.default_rng(seed)
    router = (rng.standard_normal((E, d)) * w["router_std"]).astype(np.float32)
    if w["bias_std"]:
        router[:, d - 1] = (rng.standard_normal(E) * w["bias_std"]).astype(np.float32)
    layer.router.weight.storage.upload_bytes(router.tobytes())
    return layer


def build_ep_layer(w, rank, world, seed=0, transport="p2p", gather=None):
    import numpy as np

    from qutai_b200 import lib
    from qutai_b200.expert_parallel import ExpertParallelMoE

    class Cfg:
        d_model, n_experts, top_k, d_expert, n_layers = w["d"], w["E"], w["k"], w["h"], 1

    layer = ExpertParallelMoE(Cfg, rank=rank, world=world, seed=seed, transport=transport, gather=gather)
    d, E, h = w["d"], w["E"], w["h"]
    fill = lambda storage, std, key: lib.call("qmoe_normal_fill", storage.ptr, lib.QMOE_F32, storage.size, 0.0, std, key, 0)
    fill(layer._gate, d ** -0.5, 101 + 10 * rank)
    fill(layer._up, d ** -0.5, 102 + 10 * rank)
    fill(layer._down, h ** -0.5, 103 + 10 * rank)
    rng = np.random.default_rng(seed)   # the replicated router: same draws on every rank
    router = (rng.standard_normal((E, d)) * w["router_std"]).astype(np.float32)
    if w["bias_std"]:
        router[:, d - 1] = (rng.standard_normal(E) * w["bias_std"]).astype(np.float32)
    layer.router.weight.storage.upload_bytes(router.tobytes())
    layer.router_host = router
    return layer


def balanced_placement(counts, world):
    """Static load-aware expert placement: longest-processing-time greedy.  Returns ``order`` with
    ``order[new_index] = old_index`` such that rank p owns new indices [p*L, (p+1)*L) and the rows
    per rank are as even as the per-expert loads allow."""
    E = len(counts)
    L = E // world
    loads, members = [0] * world, [[] for _ in range(world)]
    for e in sorted(range(E), key=lambda i: (-counts[i], i)):
        p = min((r for r in range(world) if len(members[r]) < L), key=lambda r: (loads[r], r))
        members[p].append(e)
        loads[p] += counts[e]
    return [e for p in range(world) for e in sorted(members[p])]


def host_inputs(w, torch, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(w["tokens"], w["d"], generator=gen, dtype=torch.float32)
    if w["bias_std"]:
        x[:, w["d"] - 1] = 1.0
    g = torch.randn(w["tokens"], w["d"], generator=gen, dtype=torch.float32)
    return x.to(torch.bfloat16).pin_memory(), g.to(torch.bfloat16).pin_memory()


def run_gpu(args, w, rank, world):
    import torch
    import torch.distributed as dist

    from qutai_b200 import lib
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.workload == "c5" and world == 1:
        # the decode-shaped forward is replayed from a CUDA graph, which needs a stream other than the default one
        torch.cuda.set_stream(torch.cuda.Stream())
    stream = torch.cuda.current_stream().cuda_stream
    if world > 1:
        from qutai_b200.expert_parallel import init_communicator

        dist.init_process_group("nccl", device_id=device)

        def share(payload):
            box = [payload]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        def gather(payload):
            box = [None] * world
            dist.all_gather_object(box, payload)
            return box

        init_communicator(rank, world, share=share)
        layer = build_ep_layer(w, rank, world, transport=args.transport, gather=gather)
    else:
        layer = build_layer(w, torch, device)
    layer.stream = stream
    x_host, g_host = host_inputs(w, torch)
    T_global, d = w["tokens"], w["d"]
    T = T_global // world                      # tokens of this rank (contiguous shard)
    x_host = x_host[rank * T:(rank + 1) * T].clone().pin_memory()
    g_host = g_host[rank * T:(rank + 1) * T].clone().pin_memory()
    x_dev, g_dev = x_host.to(device), g_host.to(device)
    aux_grad = torch.full((1,), 0.01, dtype=torch.float32, device=device)
    y_host = torch.empty_like(x_host).pin_memory()
    dx_host = torch.empty_like(x_host).pin_memory()
    wrap = lambda t, dtype: DeviceStorage.wrap(t.data_ptr(), t.numel(), dtype, owner=t)
    xs, gs = Tensor(wrap(x_dev, "bfloat16"), (T, d)), Tensor(wrap(g_dev, "bfloat16"), (T, d))
    ga = wrap(aux_grad, "float32") if world == 1 else 0.01
    forward_only = args.workload == "c5"
    if forward_only and hasattr(layer, "refresh_operands"):
        layer.refresh_operands = False   # decode: the weights are fixed, their bf16 copies are built once
    placement = "contiguous"
    if world > 1 and args.placement == "balanced":
        # Experts are placed on ranks by measured load (one profiling forward), not by index.  With
        # synthetic iid expert weights this is a relabelling of the experts, i.e. of the router rows.
        layer(xs)
        order = balanced_placement(layer.last_counts, world)
        layer.router.weight.storage.upload_bytes(layer.router_host[order].copy().tobytes())
        placement = "balanced (LPT greedy on the counts of a profiling forward)"

    parameters = layer.parameters()

    graphs, graph_mode = {}, {"on": True}

    def forward(x):
        """The layer's forward; for the decode shape on one GPU, a replay of its recorded graph (one per input buffer)."""
        if not (graph_mode["on"] and forward_only and world == 1 and stream):
            return layer(x)
        key = x.storage.ptr
        if key not in graphs:
            graphs[key] = layer.capture_forward(x)
        return graphs[key].replay()

    def step():
        for parameter in parameters:  # what optimizer.zero_grad() does before every training step
            parameter.grad = None
        y, aux = forward(xs)
        dx = None if forward_only else layer.backward(gs, ga)
        return y, aux, dx

    # End-to-end arm: every step's inputs come from pinned host memory and every step's outputs (y, dx,
    # aux) go back to pinned host memory.  The copies run on their own streams, double-buffered, so the
    # H2D of step i+1 and the D2H of step i-1 overlap the compute of step i — the way a host that feeds
    # the layer from its own buffers would drive it.
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    x_buf = [x_dev, torch.empty_like(x_dev)]
    g_buf = [g_dev, torch.empty_like(g_dev)]
    xs_buf = [Tensor(wrap(t, "bfloat16"), (T, d)) for t in x_buf]
    gs_buf = [Tensor(wrap(t, "bfloat16"), (T, d)) for t in g_buf]
    aux_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    e2e_state = dict(i=0, ready=[None, None], free=[None, None], pending=[])

    def issue_h2d(b):
        with torch.cuda.stream(copy_in):
            if e2e_state["free"][b] is not None:
                copy_in.wait_event(e2e_state["free"][b])      # the step that last read this buffer is done
            x_buf[b].copy_(x_host, non_blocking=True)
            if not forward_only:
                g_buf[b].copy_(g_host, non_blocking=True)
            event = torch.cuda.Event()
            event.record(copy_in)
            e2e_state["ready"][b] = event

    def step_e2e():
        i = e2e_state["i"]
        b = i % 2
        if e2e_state["ready"][b] is None:
            issue_h2d(b)
        issue_h2d(1 - b)                                       # next step's inputs travel during this step
        main.wait_event(e2e_state["ready"][b])
        e2e_state["ready"][b] = None
        if graphs and e2e_state.get("copied") is not None:
            main.wait_event(e2e_state["copied"])   # a replay writes the same output buffer: the last copy-out has left it
        for parameter in parameters:
            parameter.grad = None
        y, aux = forward(xs_buf[b])
        dx = None if forward_only else layer.backward(gs_buf[b], ga)
        done = torch.cuda.Event()
        done.record(main)
        e2e_state["free"][b] = done
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            s_out = copy_out.cuda_stream
            lib.call("qmoe_memcpy_d2h", y_host.data_ptr(), y.storage.ptr, y.storage.nbytes, s_out)
            if dx is not None:
                lib.call("qmoe_memcpy_d2h", dx_host.data_ptr(), dx.storage.ptr, dx.storage.nbytes, s_out)
            lib.call("qmoe_memcpy_d2h", aux_host.data_ptr(), aux.storage.ptr, 4, s_out)
            copied = torch.cuda.Event()
            copied.record(copy_out)
            e2e_state["copied"] = copied
        # outputs stay alive until their copy has finished (two steps later at most)
        e2e_state["pending"] = [item for item in e2e_state["pending"] if not item[0].query()] + [(copied, y, dx)]
        main.wait_event(copied) if i + 1 == e2e_state.get("last", -1) else None
        e2e_state["i"] = i + 1

    def timed(fn, steps):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        if world > 1:  # the job is as slow as its slowest rank
            worst = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(worst.item())
        return ms

    sampler = ClockSampler(local)   # samples clocks from the warm-up through the last timed pass: all of it is this step under load
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if args.trace:  # kernel timeline of two steps (diagnosis only; nothing measured under it is reported)
        from torch.profiler import ProfilerActivity, profile

        traced = step_e2e if os.environ.get("QUTAI_BENCH_TRACE_E2E") else step   # which arm's timeline to look at
        for _ in range(4):
            traced()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                traced()
            torch.cuda.synchronize()
        if rank == 0:
            prof.export_chrome_trace(args.trace)
    counts = layer.last_counts
    launches_before = lib.load().qmoe_launch_count()
    ms = timed(step, args.steps)
    launches = (lib.load().qmoe_launch_count() - launches_before) // args.steps
    for _ in range(max(4, args.warmup)):  # until the output buffers of the steps in flight all come from the cache
        step_e2e()
    torch.cuda.synchronize()
    e2e_state["last"] = e2e_state["i"] + args.steps           # the last timed step waits for its own copy-out
    ms_e2e = timed(step_e2e, args.steps)
    e2e_state["pending"].clear()

    # the floor of the end-to-end arm: the same host<->device copies on the same streams with no compute between
    def copies_only():
        with torch.cuda.stream(copy_in):
            x_buf[1].copy_(x_host, non_blocking=True)
            if not forward_only:
                g_buf[1].copy_(g_host, non_blocking=True)
        with torch.cuda.stream(copy_out):
            lib.call("qmoe_memcpy_d2h", y_host.data_ptr(), x_buf[0].data_ptr(), x_buf[0].numel() * 2, copy_out.cuda_stream)
            if not forward_only:
                lib.call("qmoe_memcpy_d2h", dx_host.data_ptr(), g_buf[0].data_ptr(), g_buf[0].numel() * 2, copy_out.cuda_stream)

    def timed_copies(steps):
        torch.cuda.synchronize()
        begin = time.perf_counter()
        for _ in range(steps):
            copies_only()
        torch.cuda.synchronize()
        return (time.perf_counter() - begin) * 1e3 / steps

    timed_copies(2)
    ms_copies = timed_copies(max(3, args.steps // 2))
    if world > 1:
        worst = torch.tensor([ms_copies], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        ms_copies = float(worst.item())
    # per-kernel-class device time, measured in a separate pass so the events do not sit inside the headline timing
    graph_mode["on"] = False   # the recorded graph holds no timing events: this pass runs launch by launch
    lib.timing(True)
    for _ in range(args.steps):
        step()
    classes = lib.timing_read()
    lib.timing(False)
    graph_mode["on"] = True
    clocks = sampler.stop()
    status = lib.device_status(stream)

    peaks = load_peaks()
    gemm_flops, router_flops = layer_flops(w)
    if world > 1:  # this rank's share: the rows its experts received, its own tokens for the router
        L = w["E"] // world
        gemm_flops = 18.0 * sum(counts[rank * L:(rank + 1) * L]) * w["d"] * w["h"]
        router_flops /= world
    if forward_only:
        gemm_flops, router_flops = gemm_flops / 3, router_flops / 3
    gemm_ms = (classes["expert_gemm"][0] + classes["wgrad_gemm"][0]) / args.steps
    gemm_launches = (classes["expert_gemm"][1] + classes["wgrad_gemm"][1]) // args.steps
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    peak = peaks["bf16_tflops_sustained"]
    active = sum(1 for c in (counts if world == 1 else counts[rank * (w["E"] // world):(rank + 1) * (w["E"] // world)]) if c)
    weight_bytes = active * 3 * w["d"] * w["h"] * 2     # bf16 weights of the experts that received tokens, read once
    A, h, E, k = T * w["k"], w["h"], w["E"], w["k"]
    hbm_bytes = dict(permute=T * d * 2 + A * d * 2 + A * 4, combine=A * d * 2 + 3 * A * 4 + T * d * 2,
                     combine_backward=T * d * 2 + 2 * A * d * 2 + A * 4, unpermute=A * d * 2 + T * d * 2 + A * 4,
                     route=2 * T * E * 4 + 2 * A * 4)
    hbm = {}
    for name, nbytes in hbm_bytes.items():
        t = classes[name][0] / args.steps
        if t > 0:
            gbs = nbytes / (t * 1e-3) / 1e9
            hbm[name] = dict(ms=round(t, 4), achieved_gbs=round(gbs, 1), frac=round(gbs / peaks["hbm_gbs"], 3))
    tokens_per_s = T_global / (ms * 1e-3)
    bytes_in = x_host.numel() * 2 * (1 if forward_only else 2)
    bytes_out = x_host.numel() * 2 * (1 if forward_only else 2) + 4
    line = dict(
        metric="moe_layer_fwd_bwd_tokens_per_s" if not forward_only else "moe_layer_fwd_tokens_per_s",
        value=tokens_per_s, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
        config=workload_config(args.workload, w, world),
        e2e=dict(value=T_global / (ms_e2e * 1e-3), unit="tokens/s", ms_per_step=ms_e2e, h2d_bytes_per_step=bytes_in,
                 d2h_bytes_per_step=bytes_out, copies_alone_ms_per_step=ms_copies,
                 note="copies_alone = the same pinned-host copies, both directions at once, without the layer: the floor this box's host link sets"),
        gpu_launches=int(launches), clocks=clocks,
        roofline=dict(bound="tensor", kernel="grouped_gemm_kernel (tcgen05)", achieved=achieved, peak=peak,
                      unit="TFLOP/s", frac=achieved / peak, peak_source=peaks["source"] + " (sustained cuBLAS bf16)",
                      traffic=(GEMM_DRAM_BYTES_PER_STEP.get(args.workload) if world == 1 else None),
                      traffic_unit="DRAM bytes per step over the same launches (profiler capture, see profiles/)",
                      launches_per_step=int(gemm_launches), ms_per_step=gemm_ms,
                      algorithmic_flops_per_step=gemm_flops, whole_layer_frac=(gemm_flops + router_flops) / (ms * 1e-3) / 1e12 / peak),
        hbm_kernels=hbm,
        decode_roofline=(dict(bound="hbm", kernel="grouped_gemm_kernel (tcgen05), weight streaming", achieved=weight_bytes / (gemm_ms * 1e-3) / 1e9,
                              peak=peaks["hbm_gbs"], unit="GB/s", frac=weight_bytes / (gemm_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              bytes_per_step=weight_bytes) if forward_only and gemm_ms > 0 else None),
        class_ms_per_step={name: round(v[0] / args.steps, 4) for name, v in classes.items() if v[1]},
        expert_counts=dict(max=max(counts), mean=sum(counts) / len(counts), max_over_mean=max(counts) * len(counts) / max(1, sum(counts))),
        device_status=status,
    )
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = cpu_sample_tokens(w)
        value, seconds = time_cpu(w, 2, 1, sample)
        cores = host_cores()
        line["cpu_baseline"] = dict(
            value=value, unit="tokens/s", cores=cores, kind="port",
            sample=f"{sample} of {T_global} tokens, full d/E/k/h, numpy float64 restatement of the upstream CPU path on "
                   f"{cores} threads, {seconds:.2f} s per forward+backward",
            pure_python_estimate=dict(
                mac_per_s=pure_python_rate(), cores=1,
                note="scalar triple-loop rate of the upstream pure-Python path; tokens/s = rate / (9*k*d*h + 3*d*E) MAC per token"))
        rate = line["cpu_baseline"]["pure_python_estimate"]["mac_per_s"]
        line["cpu_baseline"]["pure_python_estimate"]["tokens_per_s"] = rate / (9.0 * k * d * h + 3.0 * d * E)
    if world == 1 and not forward_only and any(p.grad is not None for p in layer.parameters()):
        # the optimizer step either side of the layer (not part of `value`): AdamW over every parameter that has a
        # gradient, one launch, refreshing the bf16 operand copies in the same pass; HBM-bound at 30 bytes per element
        from qutai_b200.optim import AdamW

        optimizer = AdamW(layer.parameters(), learning_rate=1e-5, shadows=layer.operand_shadows(), stream=stream)
        updated = sum(p.storage.size for p in layer.parameters() if p.grad is not None)
        shadowed = sum(p.storage.size for p in layer.parameters() if p.grad is not None and p in optimizer.shadows)
        optimizer.step()                       # allocates the moments
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(3):
            optimizer.step()
        end.record()
        torch.cuda.synchronize()
        adam_ms = begin.elapsed_time(end) / 3
        adam_bytes = 28 * updated + 2 * shadowed
        line["optimizer_step"] = dict(kernel="adamw_multi_kernel", ms=adam_ms, parameters=updated, launches=1,
                                      bytes=adam_bytes, achieved_gbs=adam_bytes / (adam_ms * 1e-3) / 1e9,
                                      frac=adam_bytes / (adam_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], bound="hbm")
        del optimizer
    if forward_only:
        # decode-shaped workload: per-call latency percentiles over 200 calls, each bracketed by its own events
        marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
        torch.cuda.synchronize()
        for begin, end in marks:
            begin.record()
            step()
            end.record()
        torch.cuda.synchronize()
        lat = sorted(b.elapsed_time(e) for b, e in marks)
        line["latency_ms"] = dict(p50=lat[len(lat) // 2], p99=lat[int(len(lat) * 0.99)], calls=len(lat))
    if world > 1:
        line["config"]["expert_placement"] = placement
        line["config"]["transport"] = args.transport
        line["per_rank_rows"] = [sum(counts[p * (w["E"] // world):(p + 1) * (w["E"] // world)]) for p in range(world)]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        from qutai_b200.expert_parallel import finalize_communicator

        dist.barrier()
        finalize_communicator()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--trace", default="", help="write a chrome trace of two steps (rank 0) to this path")
    parser.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"])
    parser.add_argument("--transport", default="p2p", choices=["p2p", "nccl"],
                        help="expert-parallel exchange: direct peer-memory stores, or NCCL send/receive")
    args = parser.parse_args()
    args.warmup = max(3, args.warmup)
    w = WORKLOADS[args.workload]
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, w, rank)
        return
    run_gpu(args, w, rank, world)


if __name__ == "__main__":
    main()
