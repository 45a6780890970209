"""Benchmark of the MoE layer: forward + backward tokens/s on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c2|c4layer|c5] [--impl reference]

Prints ONE JSON line (rank 0).  ``value`` is whole-job tokens/s with inputs resident in HBM;
``e2e`` is the same metric through the public layer with HOST buffers (pinned inputs copied in,
outputs copied back, inside the timed region); ``roofline`` describes the dominant kernel (the
tcgen05 grouped GEMM) against the measured bf16 peak; ``cpu_baseline`` is the CPU oracle timed on
this host on a bounded token sample; ``ep_check`` compares the values the timed path produces with the
CPU oracle (routing counts bit-exact over all ranks' tokens, sampled outputs and gradients at the bf16
bar) and the process exits non-zero when it fails; ``decode`` is the decode-shaped forward latency (c5);
``block_ffn`` times the layer with the RMS norm before it and the residual add after it fused in;
``lm_head`` and ``attention`` time the language-model head with its loss and causal attention at the shapes of
the 12-block decoder configuration, and ``decoder_step`` a whole training step of that decoder (loss, backward,
AdamW): all experts on the GPU at N = 1, data- and expert-parallel ranks with 4 sequences each at N > 1.
``--impl reference`` times the CPU implementation alone.

Workloads are the synthetic shapes of the upstream project's MoE layer study: c2 = 16384 tokens,
d 1024, 8 experts top-2, hidden 2816; c3 = 32768 tokens, d 2048, 64 experts top-6, hidden 1408,
skewed routing (per-expert router bias N(0, 0.5), realised as a constant-one input column);
c4layer = one layer of the 12-layer decoder (65536 tokens, d 1024, 16 experts top-2, hidden 2048);
c5 = c3's layer on 64 tokens (decode latency, forward only).
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# The CPU oracle (numpy) runs on rank 0 only: it gets all the host's cores, whatever the launcher put into
# OMP_NUM_THREADS (torch.distributed.run sets 1).  Must happen before numpy is first imported.
if int(os.environ.get("RANK", "0")) == 0:
    for _name in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_name] = str(host_cores())

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
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
BF16_TOL = 2e-2          # max |a - b| / max |b| of outputs and gradients, bf16 activations
AUX_GRAD = 0.01          # upstream gradient of the auxiliary loss used by every step
EXPERT_SEED = 100        # expert e's weights are drawn with keys EXPERT_SEED + 3 e (+0 gate, +1 up, +2 down)


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


def load_gemm_traffic(workload):
    """DRAM bytes (read + written) of the expert tensor-core launches of one step, from the profiler summary
    ``profiles/grouped_gemm_dram_bytes.txt`` (lines ``workload  launch  bytes``; the file says which capture
    made it).  c3 is too large to capture and has exactly four times c3s's experts and tokens at the same rows
    per expert, so its traffic is taken as four times c3s's.  None when the file has no line for the workload."""
    path = os.path.join(ROOT, "profiles", "grouped_gemm_dram_bytes.txt")
    per_workload = {}
    try:
        with open(path) as handle:
            for line in handle:
                parts = line.split()
                if len(parts) == 3 and not line.startswith("#"):
                    per_workload.setdefault(parts[0], {})[parts[1]] = float(parts[2])
    except OSError:
        return None
    scale = 1.0
    if workload == "c3" and "c3" not in per_workload:
        workload, scale = "c3s", 4.0
    launches = per_workload.get(workload)
    return scale * sum(launches.values()) if launches else None


def layer_flops(w, tokens=None):
    """Algorithmic FLOPs of one forward + backward: expert GEMMs 18*A*d*h, router 6*T*d*E."""
    T = w["tokens"] if tokens is None else tokens
    return 18.0 * T * w["k"] * w["d"] * w["h"], 6.0 * T * w["d"] * w["E"]


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while the benchmark runs; ``begin()`` /
    ``end()`` bracket the timed region, and only samples taken inside it are summarised."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc, self.t0, self.t1 = index, [], None, None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except Exception:
            self.proc = None

    def begin(self):
        self.t0 = datetime.datetime.now()

    def end(self):
        self.t1 = datetime.datetime.now()

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        parsed, max_clock = [], None
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clock, max_clock, power = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
            except ValueError:
                stamp = None
            parsed.append((stamp, clock, power, [name for name, flag in zip(names, parts[5:9]) if flag.lower().startswith("active")]))
        inside = [p for p in parsed if p[0] is not None and self.t0 is not None and self.t0 <= p[0] <= (self.t1 or p[0])]
        window = "samples inside the timed regions only"
        if not inside:   # no usable time stamps: fall back to every sample of the run (the power filter below still applies)
            inside, window = parsed, "all samples of the run (time stamps unusable)"
        if not inside:
            return dict(sm_mhz=None, sm_max_mhz=max_clock, samples=0, reasons=[])
        samples = [(clock, power) for _, clock, power, _ in inside]
        reasons = {name for item in inside for name in item[3]}
        # under load = the samples whose power draw is within 60 % of the region's maximum (under a power cap the
        # loaded samples are the ones with the LOW clocks; idle edges draw little)
        top = max(power for _, power in samples)
        loaded = sorted(clock for clock, power in samples if power >= 0.6 * top)
        return dict(sm_mhz=loaded[len(loaded) // 2], sm_min_mhz=loaded[0], sm_max_mhz=max_clock, samples=len(samples),
                    samples_under_load=len(loaded), power_w_max=top, reasons=sorted(reasons), window=window)


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
    oracle.moe_backward(ctx, grad, AUX_GRAD)
    return y


def pure_python_layer(max_seconds=6.0):
    """The scalar-loop restatement of the upstream pure-Python layer (the code path ``device="cpu"`` runs
    upstream), forward + backward, timed at the shape of the tiny CPU configuration's MoE layer (d 64, 4 experts
    top-2, hidden 128; that configuration has 128 tokens per layer) on a token sample sized to stay within
    ``max_seconds``.  Returns measured tokens/s on one core and multiply-accumulates per second."""
    import random
    from array import array

    from oracle import moe_pure

    d, E, k, h = 64, 4, 2, 128
    rng = random.Random(0)
    draw = lambda n, std: array("d", (rng.gauss(0.0, std) for _ in range(n)))
    router = draw(E * d, 0.02)
    gate, up, down = [draw(h * d, 0.02) for _ in range(E)], [draw(h * d, 0.02) for _ in range(E)], [draw(d * h, 0.01) for _ in range(E)]
    mac_per_token = 9 * k * d * h + 3 * d * E
    tokens, seconds = 4, 0.0
    while True:
        x, grad = draw(tokens * d, 1.0), draw(tokens * d, 1.0)
        start = time.perf_counter()
        moe_pure.moe_forward_backward(x, router, gate, up, down, tokens, d, h, k, grad, AUX_GRAD)
        seconds = time.perf_counter() - start
        if tokens >= 128 or seconds * 4 > max_seconds:
            break
        tokens = min(128, tokens * 4)
    return dict(tokens_per_s=tokens / seconds, mac_per_s=tokens * mac_per_token / seconds, seconds=seconds, cores=1,
                sample=f"{tokens} of 128 tokens of the tiny CPU configuration's MoE layer (d 64, 4 experts top-2, hidden 128), "
                       "float64 scalar loops, forward + backward")


def time_cpu(w, steps, warmup, sample_tokens):
    inputs = cpu_sample_inputs(w, sample_tokens)
    for _ in range(warmup):
        cpu_step(w, inputs)
    start = time.perf_counter()
    for _ in range(steps):
        cpu_step(w, inputs)
    seconds = (time.perf_counter() - start) / steps
    return sample_tokens / seconds, seconds


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
class Cfg:
    def __init__(self, w):
        self.d_model, self.n_experts, self.top_k, self.d_expert, self.n_layers = w["d"], w["E"], w["k"], w["h"], 1


def router_weights(w, seed=0):
    import numpy as np

    rng = np.random.default_rng(seed)   # the same draws on every rank: the router is replicated
    router = (rng.standard_normal((w["E"], w["d"])) * w["router_std"]).astype(np.float32)
    if w["bias_std"]:
        router[:, w["d"] - 1] = (rng.standard_normal(w["E"]) * w["bias_std"]).astype(np.float32)
    return router


def fill_experts(layer, w, expert_ids):
    """Synthetic expert weights N(0, 1/sqrt(fan_in)), keyed by the model's expert number: the layer computes the
    same function however its experts are spread over ranks."""
    d, h = w["d"], w["h"]
    for expert, e in zip(layer.experts, expert_ids):
        expert.gate.weight.storage.fill_normal(0.0, d ** -0.5, EXPERT_SEED + 3 * e)
        expert.up.weight.storage.fill_normal(0.0, d ** -0.5, EXPERT_SEED + 3 * e + 1)
        expert.down.weight.storage.fill_normal(0.0, h ** -0.5, EXPERT_SEED + 3 * e + 2)


def build_layer(w, seed=0):
    from qutai_b200.layers import SparseMoE

    layer = SparseMoE(Cfg(w), device="cuda", dtype="float32", seed=seed)
    fill_experts(layer, w, range(w["E"]))
    layer.router.weight.storage.upload_bytes(router_weights(w, seed).tobytes())
    return layer


def build_ep_layer(w, rank, world, seed=0, transport="p2p", gather=None, overlap=False):
    from qutai_b200.expert_parallel import ExpertParallelMoE

    layer = ExpertParallelMoE(Cfg(w), rank=rank, world=world, seed=seed, transport=transport, gather=gather, overlap=overlap)
    fill_experts(layer, w, layer.expert_ids)
    layer.router.weight.storage.upload_bytes(router_weights(w, seed).tobytes())
    return layer


def host_inputs(w, torch, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(w["tokens"], w["d"], generator=gen, dtype=torch.float32)
    if w["bias_std"]:
        x[:, w["d"] - 1] = 1.0
    g = torch.randn(w["tokens"], w["d"], generator=gen, dtype=torch.float32)
    return x.to(torch.bfloat16).pin_memory(), g.to(torch.bfloat16).pin_memory()


def percentile(sorted_values, fraction):
    return sorted_values[min(len(sorted_values) - 1, int(len(sorted_values) * fraction))]


def run_gpu(args, w, rank, world):
    import numpy as np
    import torch
    import torch.distributed as dist

    from qutai_b200 import lib
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # a stream of the benchmark's own: the decode-shaped forward is replayed from a CUDA graph, which the default stream cannot record
    torch.cuda.set_stream(torch.cuda.Stream())
    stream = torch.cuda.current_stream().cuda_stream
    gather = None
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
        layer = build_ep_layer(w, rank, world, transport=args.transport, gather=gather, overlap=args.overlap)
    else:
        layer = build_layer(w)
    layer.stream = stream
    x_host, g_host = host_inputs(w, torch)
    T_global, d, E, k, h = w["tokens"], w["d"], w["E"], w["k"], w["h"]
    T = T_global // world                      # tokens of this rank (contiguous shard)
    L = E // world                             # experts of this rank
    x_host = x_host[rank * T:(rank + 1) * T].clone().pin_memory()
    g_host = g_host[rank * T:(rank + 1) * T].clone().pin_memory()
    x_dev, g_dev = x_host.to(device), g_host.to(device)
    aux_grad = torch.full((1,), AUX_GRAD, dtype=torch.float32, device=device)
    y_host = torch.empty_like(x_host).pin_memory()
    dx_host = torch.empty_like(x_host).pin_memory()
    wrap = lambda t, dtype: DeviceStorage.wrap(t.data_ptr(), t.numel(), dtype, owner=t)
    xs, gs = Tensor(wrap(x_dev, "bfloat16"), (T, d)), Tensor(wrap(g_dev, "bfloat16"), (T, d))
    ga = wrap(aux_grad, "float32") if world == 1 else AUX_GRAD
    forward_only = args.workload == "c5"
    parameters = layer.parameters()
    graphs, graph_mode = {}, {"on": True}

    def forward(x):
        """The layer's forward; for the decode shape on one GPU, a replay of its recorded graph (one per input buffer)."""
        if not (graph_mode["on"] and forward_only and world == 1):
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

    def timed(fn, steps):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.begin() if sampler.t0 is None else None
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        sampler.end()
        ms = start.elapsed_time(stop) / steps
        if world > 1:  # the job is as slow as its slowest rank
            worst = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(worst.item())
        return ms

    def preroll(seconds):
        """Back-to-back steps until the GPU has worked for ``seconds``: the timed steps then sit at the operating
        point a long job sees under the power cap, whatever --warmup says."""
        done = 0
        begin = time.perf_counter()
        while seconds > 0:
            for _ in range(10):
                step()
            done += 10
            torch.cuda.synchronize()
            elapsed = torch.tensor([time.perf_counter() - begin], dtype=torch.float64, device=device)
            if world > 1:   # every rank must leave the loop after the same number of steps
                dist.all_reduce(elapsed, op=dist.ReduceOp.MIN)
            if float(elapsed.item()) >= seconds:
                break
        return done

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    contiguous = None
    if world > 1:
        placement_label = "contiguous blocks of E / N experts per rank"
        if args.placement == "balanced":
            # the contiguous placement first (device time only), then the experts move to the load-balanced one
            preroll(args.preroll / 2)
            ms_contiguous = timed(step, args.steps)
            rows = [sum(layer.last_counts[p * L + j] for j in range(L)) for p in range(world)]
            contiguous = dict(ms_per_step=ms_contiguous, value=T_global / (ms_contiguous * 1e-3), unit="tokens/s",
                              per_rank_rows=rows, placement=placement_label)
            sampler.t0 = None   # the clock summary covers the headline placement's timed regions
            layer.rebalance()   # LPT greedy on the counts of the last forward; the weights travel over NCCL
            parameters = layer.parameters()
            placement_label = "balanced: longest-processing-time greedy on measured per-expert counts (ExpertParallelMoE.rebalance)"
            for _ in range(args.warmup):
                step()
    if args.trace:  # kernel timeline of a few steps (diagnosis only; nothing measured under it is reported)
        from torch.profiler import ProfilerActivity, profile

        for _ in range(4):
            step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                step()
            torch.cuda.synchronize()
        if rank == 0:
            prof.export_chrome_trace(args.trace)
    # the same steps timed right after the warm-up, before the GPU has settled against its power cap: what a short
    # run reads (reported beside the steady-state headline, not instead of it)
    ms_short = timed(step, args.steps)
    sampler.t0 = None
    prerolled = preroll(args.preroll)
    logical_counts = layer.last_counts
    physical = getattr(layer, "_logical_of_physical", list(range(E)))
    counts = [logical_counts[e] for e in physical]          # in the layer's internal (rank-major) expert order
    launches_before = lib.load().qmoe_launch_count()
    ms = timed(step, args.steps)
    launches_timed = lib.load().qmoe_launch_count() - launches_before      # this library's kernels inside the timed region (this rank)
    launches = launches_timed // args.steps

    # ---- end-to-end arm: every step's inputs come from pinned host memory and every step's outputs (y, dx, aux)
    # go back to pinned host memory.  The copies run on their own streams, double-buffered, so the H2D of step
    # i+1 and the D2H of step i-1 overlap the compute of step i — the way a host that feeds the layer from its
    # own buffers would drive it.
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
    for _ in range(5):
        step()
    lib.timing(True)
    sampler_end = sampler.t1
    for _ in range(args.steps):
        step()
    classes = lib.timing_read()
    lib.timing(False)
    sampler.t1 = sampler_end
    graph_mode["on"] = True
    clocks = sampler.stop()
    status = lib.device_status(stream)

    peaks = load_peaks()
    gemm_flops, router_flops = layer_flops(w)
    if world > 1:  # this rank's share: the rows its experts received, its own tokens for the router
        gemm_flops = 18.0 * sum(counts[rank * L:(rank + 1) * L]) * d * h
        router_flops /= world
    if forward_only:
        gemm_flops, router_flops = gemm_flops / 3, router_flops / 3
    gemm_ms = (classes["expert_gemm"][0] + classes["wgrad_gemm"][0]) / args.steps
    gemm_launches = (classes["expert_gemm"][1] + classes["wgrad_gemm"][1]) // args.steps
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    peak = peaks["bf16_tflops_sustained"]
    active = sum(1 for c in counts[rank * L:(rank + 1) * L] if c)
    weight_bytes = active * 3 * d * h * 2     # bf16 weights of the experts that received tokens, read once
    A = T * k
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
    mhz = clocks.get("sm_mhz")
    line = dict(
        metric="moe_layer_fwd_bwd_tokens_per_s" if not forward_only else "moe_layer_fwd_tokens_per_s",
        value=tokens_per_s, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
        higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
        config=workload_config(args.workload, w, world),
        e2e=dict(value=T_global / (ms_e2e * 1e-3), unit="tokens/s", ms_per_step=ms_e2e, h2d_bytes_per_step=bytes_in,
                 d2h_bytes_per_step=bytes_out, copies_alone_ms_per_step=ms_copies,
                 note="copies_alone = the same pinned-host copies, both directions at once, without the layer: the floor this box's host link sets"),
        gpu_launches=int(launches_timed), gpu_launches_per_step=int(launches), clocks=clocks,
        steady_state=dict(preroll_steps=prerolled, preroll_seconds=args.preroll, ms_per_step_before_preroll=ms_short,
                          ms_x_mhz=(ms * mhz if mhz else None), gemm_ms_x_mhz=(gemm_ms * mhz if mhz else None),
                          note="back-to-back steps ran for preroll_seconds before the timed ones; ms_x_mhz = ms_per_step x median SM MHz under load, comparable across boxes"),
        roofline=dict(bound="tensor", kernel="grouped_gemm_kernel (tcgen05)", achieved=achieved, peak=peak,
                      unit="TFLOP/s", frac=achieved / peak, peak_source=peaks["source"] + " (sustained cuBLAS bf16)",
                      traffic=(load_gemm_traffic(args.workload) if world == 1 else None),
                      traffic_unit="DRAM bytes per step over the same launches (profiler capture, profiles/grouped_gemm_dram_bytes.txt)",
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
    if world > 1:
        line["expert_parallel"] = dict(placement=placement_label, transport=args.transport,
                                       overlap=("rows of half of every rank's experts travel behind the first product on the other half"
                                                if args.overlap and args.transport == "p2p" else "none"),
                                       per_rank_rows=[sum(counts[p * L:(p + 1) * L]) for p in range(world)],
                                       contiguous=contiguous)

    # ---- value check of the timed path against the CPU oracle (outside every timed region) ----------------
    check = ep_check(layer, w, rank, world, step, x_dev, g_dev, counts, physical, torch, dist, np)
    line["ep_check"] = check

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = cpu_sample_tokens(w)
        value, seconds = time_cpu(w, 2, 1, sample)
        cores = host_cores()
        pure = pure_python_layer()
        pure["scaled_to_this_workload_tokens_per_s"] = pure["mac_per_s"] / (9.0 * k * d * h + 3.0 * d * E)
        line["cpu_baseline"] = dict(
            value=value, unit="tokens/s", cores=cores, kind="port",
            sample=f"{sample} of {T_global} tokens, full d/E/k/h, numpy float64 restatement of the upstream CPU path on "
                   f"{cores} threads, {seconds:.2f} s per forward+backward",
            pure_python=pure)
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
    if world == 1 and not forward_only and not args.no_block:
        line["block_ffn"] = block_ffn(layer, w, xs, gs, ga, x_dev, g_dev, args.steps, ms, torch, np)
    if world == 1 and not forward_only and not args.no_head:
        line["lm_head"] = lm_head(args.steps, peaks, torch, np)
    if world == 1 and not forward_only and not args.no_attention:
        line["attention"] = attention_block(args.steps, peaks, torch, np)
    if not forward_only and not args.no_decoder:
        line["decoder_step"] = decoder_step(torch, np, rank=rank, world=world, dist=dist, gather=gather, device=device,
                                            placement=args.placement)
    if world == 1 and not forward_only and not args.no_library_gemm:
        here = library_gemm_here(torch)
        line["roofline"]["library_gemm_on_this_gpu"] = here
        line["roofline"]["frac_of_library_gemm_on_this_gpu"] = achieved / here["tflops"]
    if forward_only:
        line["latency_ms"] = call_latency(step, torch, dist, world, device)
    elif args.workload == "c3" and not args.no_decode:
        # the decode-shaped configuration (c3's layer on 64 tokens, forward only): per-call latency of 200 calls
        line["decode"] = decode_latency(layer, w, rank, world, torch, dist, device, Tensor, wrap, peaks)
    ok = (bool(check["ok"]) and bool(line.get("block_ffn", {}).get("check", {}).get("ok", True))
          and bool(line.get("lm_head", {}).get("check", {}).get("ok", True))
          and bool(line.get("attention", {}).get("check", {}).get("ok", True))
          and bool(line.get("decoder_step", {}).get("check", {}).get("ok", True)))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        from qutai_b200.expert_parallel import finalize_communicator

        dist.barrier()
        finalize_communicator()
        dist.destroy_process_group()
    if not ok:
        sys.exit(1)


def call_latency(call, torch, dist, world, device, calls=200):
    """p50 / p99 of ``calls`` single calls, each bracketed by its own pair of events (max over ranks per call)."""
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(calls)]
    for _ in range(10):
        call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    for begin, end in marks:
        begin.record()
        call()
        end.record()
    torch.cuda.synchronize()
    times = torch.tensor([b.elapsed_time(e) for b, e in marks], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    lat = sorted(times.tolist())
    return dict(p50=percentile(lat, 0.5), p99=percentile(lat, 0.99), calls=calls)


def decode_latency(layer, w, rank, world, torch, dist, device, Tensor, wrap, peaks):
    """Forward latency of the same layer on 64 tokens (64 sequences x 1 step): a replayed CUDA graph on one GPU,
    the expert-parallel forward (8 tokens per rank at 8 GPUs) on several."""
    tokens_global, d = 64, w["d"]
    tokens = tokens_global // world
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(tokens_global, d, generator=gen, dtype=torch.float32)
    if w["bias_std"]:
        x[:, d - 1] = 1.0
    x_dev = x[rank * tokens:(rank + 1) * tokens].to(torch.bfloat16).to(device)
    xs = Tensor(wrap(x_dev, "bfloat16"), (tokens, d))
    layer.refresh_operands = False           # decode: the weights are fixed, their bf16 copies are built once
    if world == 1:
        graph = layer.capture_forward(xs)
        call, how = graph.replay, "CUDA graph replay of the forward (one launch per call)"
    else:
        call, how = (lambda: layer(xs)), "expert-parallel forward, launched call by call"
    out = call_latency(call, torch, dist, world, device)
    active = sum(1 for c in layer.last_counts if c)
    weight_bytes = active * 3 * d * w["h"] * 2 / world   # bf16 weights of the experts that received tokens, per GPU
    out.update(workload=f"c5: {tokens_global} tokens, d_model {d}, experts {w['E']}, top_k {w['k']}, d_expert {w['h']}, forward only",
               how=how, unit="ms per layer call", tokens_per_s=tokens_global / (out["p50"] * 1e-3),
               weight_bytes_per_gpu=weight_bytes, weight_stream_gbs_at_p50=weight_bytes / (out["p50"] * 1e-3) / 1e9,
               weight_stream_frac_of_hbm_peak=weight_bytes / (out["p50"] * 1e-3) / 1e9 / peaks["hbm_gbs"])
    return out


def block_ffn(layer, w, xs, gs, ga, x_dev, g_dev, steps, layer_ms, torch, np):
    """The step either side of the layer fused into it: ``out = x + MoE(rms_norm(x))`` forward + backward
    (``MoEFeedForward``), timed like the layer alone, and its values checked against the CPU oracle on sampled
    tokens (out and dx of a token depend on that token alone when the auxiliary gradient is left out)."""
    from oracle import moe_oracle as oracle
    from qutai_b200.layers import MoEFeedForward, RMSNorm

    T, d, E, k, h = w["tokens"], w["d"], w["E"], w["k"], w["h"]
    eps = 1e-6
    block = MoEFeedForward(RMSNorm(d, eps, stream=layer.stream), layer)
    norm_weight = (1.0 + 0.1 * np.random.default_rng(3).standard_normal(d)).astype(np.float32)
    block.ffn_norm.weight.storage.upload_bytes(norm_weight.tobytes(), layer.stream)
    parameters = block.parameters()

    def step(grad_aux):
        for parameter in parameters:
            parameter.grad = None
        out, aux = block(xs)
        return out, block.backward(gs, grad_aux)

    layer_parameters = layer.parameters()

    def layer_step():
        for parameter in layer_parameters:
            parameter.grad = None
        layer(xs)
        layer.backward(gs, ga)

    def timed(fn):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / steps

    for _ in range(5):
        step(ga)
    torch.cuda.synchronize()
    # the block and the layer alone in turn, three rounds each: the SM clock drifts under the power cap, so only
    # measurements taken side by side compare
    rounds = [(timed(lambda: step(ga)), timed(layer_step)) for _ in range(3)]
    ms = sorted(r[0] for r in rounds)[1]
    layer_ms = sorted(r[1] for r in rounds)[1]
    out, dx = step(None)
    torch.cuda.synchronize()
    device = x_dev.device
    buf = layer._saved[0]["buf"]

    def as_tensor(storage, shape, dtype):
        from qutai_b200 import lib

        t = torch.empty(shape, dtype=dtype, device=device)
        lib.call("qmoe_memcpy_d2d", t.data_ptr(), storage.ptr, storage.nbytes, layer.stream)
        return t

    sample = torch.from_numpy(np.sort(np.random.default_rng(4321).choice(T, size=min(48, T), replace=False))).to(device)
    scores = as_tensor(buf["scores"], (T, E), torch.float32)[sample]
    out_s, dx_s = as_tensor(out.storage, (T, d), torch.bfloat16)[sample], as_tensor(dx.storage, (T, d), torch.bfloat16)[sample]
    weights = {name: StackedWeights(as_tensor(buf[name], shape, torch.bfloat16))
               for name, shape in (("w_gate", (E, h, d)), ("w_up", (E, h, d)), ("w_down", (E, d, h)))}
    torch.cuda.synchronize()
    x_s = x_dev[sample].float().cpu().numpy().astype(np.float64)
    g_s = g_dev[sample].float().cpu().numpy().astype(np.float64)
    want_out, _, ctx = oracle.block_ffn_forward(x_s, norm_weight, eps, router_weights(w).astype(np.float64), weights["w_gate"],
                                                weights["w_up"], weights["w_down"], k, scores=scores.cpu().numpy().astype(np.float64))
    grads = oracle.block_ffn_backward(ctx, g_s, 0.0)
    out_err = oracle.max_rel_err(out_s.float().cpu().numpy(), want_out)
    dx_err = oracle.max_rel_err(dx_s.float().cpu().numpy(), grads["x"])
    # what the unfused chain moves on top of the layer: the norm kernel reads x and writes an fp32 copy (2 + 4 bytes per
    # element), the residual kernel reads x and the layer's output and writes the sum (2 + 2 + 2); mirrored in the
    # backward.  Fused, one statistics pass and one residual read per direction remain (2 + 2).
    elements = T * d
    return dict(ms_per_step=ms, layer_alone_ms_per_step=layer_ms, added_ms=ms - layer_ms,
                rounds_ms=[(round(a, 4), round(b, 4)) for a, b in rounds],
                what="x + MoE(rms_norm(x)) forward + backward, norm and residual fused into the layer (qmoe_block_forward / _backward)",
                unfused_extra_bytes_per_step=2 * elements * (6 + 6), fused_extra_bytes_per_step=2 * elements * (2 + 2),
                check=dict(ok=bool(out_err <= BF16_TOL and dx_err <= BF16_TOL), out=out_err, dx=dx_err, tolerance=BF16_TOL,
                           sampled_tokens=int(sample.numel())))


def decoder_step(torch, np, steps=3, rank=0, world=1, dist=None, gather=None, device=None, placement="balanced"):
    """One rank's share of the full decoder training step (12 blocks, d_model 1024, 16 heads in 4 key/value groups,
    16 experts top-2 of hidden width 2048, vocabulary 32000; 4 sequences of 2048 tokens, Zipf(1.1) ids): loss,
    backward and the AdamW step of ``qutai_b200.decoder.Decoder``.  One GPU: all experts local.  N GPUs: every rank
    has 4 sequences of its own (weak scaling, the configuration's 32 at N = 8), the 16 experts of every block are
    spread over the ranks, the gradients of the replicated parameters are summed over the ranks inside ``backward``;
    the time is the slowest rank's."""
    import gc

    from qutai_b200.decoder import Config, Decoder
    from qutai_b200.optim import AdamW
    from qutai_b200.storage import empty_cache

    gc.collect()
    empty_cache()
    config = Config(vocab_size=32000, d_model=1024, n_heads=16, n_kv_heads=4, n_layers=12, n_experts=16, top_k=2, d_expert=2048)
    batch, time_ = 4, 2048
    stream = torch.cuda.current_stream().cuda_stream
    model = Decoder(config, seed=7, stream=stream, rank=rank, world=world, parallel=dict(gather=gather) if world > 1 else None)
    rng = np.random.default_rng(31 + rank)
    weights = np.arange(1, config.vocab_size + 1, dtype=np.float64) ** -1.1        # Zipf(1.1) over the vocabulary: P(id) ~ (id + 1)^-1.1
    tokens = rng.choice(config.vocab_size, size=(batch, time_), p=weights / weights.sum()).tolist()
    model.loss(tokens)            # a first forward makes the bf16 operand copies that the optimizer then keeps current
    if world > 1 and placement == "balanced":
        # every block moves its experts to the placement that evens out the rows per rank of this first forward
        # (the blocks' loads differ); the parameters are new objects afterwards, so this comes before the optimizer
        for block in model.blocks:
            block.ffn.rebalance()
        model.loss(tokens)
    optimizer = AdamW(model.parameters(), learning_rate=1e-4, shadows=model.operand_shadows(), stream=stream)

    def step():
        model.zero_grad()
        loss = model.loss(tokens)
        model.backward()
        optimizer.step()
        return loss

    losses = [float(step().storage.tolist(stream)[0]) for _ in range(2)]
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        loss = step()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / steps
    losses.append(float(loss.storage.tolist(stream)[0]))
    parameters = sum(p.storage.size for p in model.parameters())
    same_on_every_rank = True
    if world > 1:
        slowest = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        ms = float(slowest.item())
        seen = [None] * world
        dist.all_gather_object(seen, losses)
        same_on_every_rank = all(other == seen[0] for other in seen)
        local = sum(p.storage.size for block in model.blocks for expert in block.ffn.experts for p in expert.parameters())
        held = torch.tensor([local], dtype=torch.int64, device=device)
        dist.all_reduce(held)     # the model = one copy of the replicated parameters + every rank's experts
        parameters = parameters - local + int(held.item())
    # where the step's device time goes, by kernel class (a pass of its own: the events sit between the launches)
    from qutai_b200 import lib

    lib.timing(True)
    step()
    torch.cuda.synchronize()
    classes = {name: round(value[0], 3) for name, value in lib.timing_read().items() if value[1]}
    lib.timing(False)
    host_begin = time.time()
    step()
    host_ms = (time.time() - host_begin) * 1e3          # the host's share: issuing one step without waiting for it
    torch.cuda.synchronize()
    by_rank = load = None
    if world > 1:   # waiting shows up in different classes on different ranks: keep every rank's view of them
        # rows every rank's experts received in the last step, block by block: the step walks the blocks in lockstep
        # (barriers), so its expert time follows the sum over the blocks of the fullest rank, not the fullest sum
        fullest = mean = 0.0
        worst = []
        for block in model.blocks:
            counts, owner = block.ffn.last_counts, block.ffn.placement
            rows = [sum(c for c, o in zip(counts, owner) if o == r) for r in range(world)]
            fullest += max(rows)
            mean += sum(rows) / world
            worst.append(round(max(rows) * world / max(sum(rows), 1), 2))
        load = dict(fullest_rank_over_mean=round(fullest / mean, 3), per_block=worst)
        seen = [None] * world
        dist.all_gather_object(seen, {name: classes.get(name, 0.0) for name in ("barrier", "all_reduce", "exchange", "expert_gemm", "wgrad_gemm")})
        by_rank = {name: [other[name] for other in seen] for name in seen[0]}
    del model, optimizer
    gc.collect()
    empty_cache()
    return dict(ms_per_step=ms, tokens_per_s=world * batch * time_ / (ms * 1e-3), tokens=world * batch * time_, parameters=parameters,
                config=f"12 blocks, d_model 1024, 16 heads / 4 kv heads, 16 experts top-2 hidden 2048, vocab 32000, {world} x 4 x 2048 tokens, bf16 activations, fp32 parameters",
                what="loss + backward + AdamW of qutai_b200.decoder.Decoder"
                     + (" (all experts local)" if world == 1 else f" on {world} ranks: experts spread over the ranks ({placement} placement per block), replicated gradients summed (NCCL)"),
                class_ms=classes, class_ms_by_rank=by_rank, expert_rows=load, host_issue_ms=host_ms, losses=losses,
                check=dict(ok=bool(np.isfinite(losses).all() and losses[-1] < losses[0] and same_on_every_rank),
                           how="finite, falling over the steps on the same batch, the same value on every rank"))


def attention_block(steps, peaks, torch, np):
    """Causal self-attention with grouped key/value heads (``qutai_b200.attention``) at one rank's share of the full
    decoder step: 4 sequences of 2048 positions, 16 heads of width 64 in 4 key/value groups, bf16; forward + backward,
    timed with events, one (sequence, group) checked against the float64 oracle on the same bf16 values."""
    from oracle import moe_oracle as oracle
    from qutai_b200.attention import attention_backward, attention_forward
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    batch, time_, heads, kv_heads, dim = 4, 2048, 16, 4, 64
    generator = torch.Generator(device="cuda").manual_seed(21)
    make = lambda width, scale: (torch.randn((batch, time_, width), device="cuda", generator=generator) * scale).to(torch.bfloat16)
    q, k, v, grad = make(heads * dim, 0.6), make(kv_heads * dim, 0.6), make(kv_heads * dim, 1.0), make(heads * dim, 1.0)
    wrap = lambda t: Tensor(DeviceStorage.wrap(t.data_ptr(), t.numel(), "bfloat16", owner=t), tuple(t.shape))
    qt, kt, vt, gt = wrap(q), wrap(k), wrap(v), wrap(grad)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        out, lse = attention_forward(qt, kt, vt, heads, kv_heads, stream)
        return out, attention_backward(gt, qt, kt, vt, out, lse, heads, kv_heads, stream)

    for _ in range(3):
        out, grads = step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        out, grads = step()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / steps
    # the products of the causal half: forward 2 (Q K^T, P V), backward 5 (S and dP once per kernel = 4, dQ, dV, dK = 3,
    # of which S and dP are formed in both backward kernels), each 2 * 64 flops per (query, key <= query) pair and head
    pairs = batch * heads * time_ * (time_ + 1) / 2
    flops = (2 + 7) * 2.0 * dim * pairs

    def host(storage, like):
        t = torch.empty_like(like)
        from qutai_b200 import lib

        lib.call("qmoe_memcpy_d2d", t.data_ptr(), storage.ptr, storage.nbytes, stream)
        torch.cuda.synchronize()
        return t.float().cpu().numpy().astype(np.float64)

    group = heads // kv_heads
    b, g = 1, 2
    wide, narrow = slice(g * group * dim, (g + 1) * group * dim), slice(g * dim, (g + 1) * dim)
    f = lambda t, cols: t[b:b + 1, :, cols].float().cpu().numpy().astype(np.float64)
    want_out, lse = oracle.attention_forward(f(q, wide), f(k, narrow), f(v, narrow), group, 1)
    want = oracle.attention_backward(f(grad, wide), f(q, wide), f(k, narrow), f(v, narrow), want_out, lse, group, 1)
    got_out = host(out, q)[b:b + 1, :, wide]
    got = (host(grads[0], q)[b:b + 1, :, wide], host(grads[1], k)[b:b + 1, :, narrow], host(grads[2], v)[b:b + 1, :, narrow])
    errors = dict(out=oracle.max_rel_err(got_out, want_out), dq=oracle.max_rel_err(got[0], want[0]),
                  dk=oracle.max_rel_err(got[1], want[1]), dv=oracle.max_rel_err(got[2], want[2]))
    return dict(ms_per_step=ms, batch=batch, time=time_, heads=heads, kv_heads=kv_heads, dim=dim, dtype="bf16",
                tflops=flops / (ms * 1e-3) / 1e12, frac_of_sustained_peak=flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                launches_per_step=3,
                what="causal attention forward + backward (qmoe_attention_forward / _backward): tcgen05, the scores never leave the chip",
                check=dict(ok=bool(max(errors.values()) <= BF16_TOL), tolerance=BF16_TOL, sampled="sequence 1, key/value group 2", **errors))


def library_gemm_here(torch, seconds=2.0, n=8192):
    """The denominator of the roofline measured again on THIS GPU in THIS run, the way the committed figure was taken
    (a library bf16 product n^3, back to back for ``seconds``, CUDA events): boxes of the pool differ in their power
    cap by a quarter, and every tensor-bound kernel runs against that cap, so a fraction of a figure measured on
    another box mixes the kernel with the box.  Reported beside the official fraction, never instead of it."""
    a = torch.randn((n, n), device="cuda").to(torch.bfloat16)
    b = torch.randn((n, n), device="cuda").to(torch.bfloat16)
    for _ in range(5):
        torch.matmul(a, b)
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    calls, begin, end = 0, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    started = time.time()
    sampler.begin()
    begin.record()
    while time.time() - started < seconds:
        for _ in range(20):
            torch.matmul(a, b)
        calls += 20
        torch.cuda.synchronize()
    end.record()
    torch.cuda.synchronize()
    sampler.end()
    clocks = sampler.stop()
    ms = begin.elapsed_time(end) / calls
    return dict(tflops=2.0 * n ** 3 / (ms * 1e-3) / 1e12, n=n, calls=calls, sm_mhz=clocks.get("sm_mhz"),
                power_w_max=clocks.get("power_w_max"), how="torch.matmul bf16 n^3 back to back for 2 s after the timed steps")


def lm_head(steps, peaks, torch, np):
    """The language-model head with its cross-entropy loss (``qutai_b200.head``) at one rank's share of the full
    decoder step: 4 sequences of 2048 positions, width 1024, vocabulary 32000, bf16; forward (logits once, loss and
    gradient of the logits in one pass) + backward (two products), timed with events, the losses of sampled rows
    checked against float64 arithmetic on the same bf16 values."""
    from oracle import moe_oracle as oracle
    from qutai_b200.head import LMHead
    from qutai_b200.layers import Tensor
    from qutai_b200.storage import DeviceStorage

    batch, time, width, vocab = 4, 2048, 1024, 32000
    generator = torch.Generator(device="cuda").manual_seed(11)
    hidden = torch.randn((batch, time, width), device="cuda", generator=generator).to(torch.bfloat16)
    weight = (torch.randn((vocab, width), device="cuda", generator=generator) * 0.02).to(torch.bfloat16)
    rng = np.random.default_rng(12)
    zipf = np.arange(1, vocab + 1, dtype=np.float64) ** -1.1                       # Zipf(1.1) over the vocabulary
    labels_host = rng.choice(vocab, size=(batch, time), p=zipf / zipf.sum()).astype(np.int64)
    labels = torch.from_numpy(labels_host).cuda()
    wrap = lambda t, dtype: DeviceStorage.wrap(t.data_ptr(), t.numel(), dtype, owner=t)
    h, wt = Tensor(wrap(hidden, "bfloat16"), tuple(hidden.shape)), Tensor(wrap(weight, "bfloat16"), tuple(weight.shape))
    label_storage = wrap(labels, "int64")
    stream = torch.cuda.current_stream().cuda_stream    # the events below are recorded on this stream
    head = LMHead(stream=stream)

    def step():
        loss = head.forward(h, wt, label_storage)
        head.backward()
        return loss

    for _ in range(3):
        loss = step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        loss = step()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / steps
    rows = batch * (time - 1)
    flops = 3 * 2.0 * rows * width * vocab
    # one read and one write of the logits by the loss pass; each product streams them once more
    logits_bytes = rows * vocab * 2
    row_loss = torch.empty(rows, dtype=torch.float32, device="cuda")
    from qutai_b200 import lib

    lib.call("qmoe_memcpy_d2d", row_loss.data_ptr(), head._buffers["row_loss"].ptr, rows * 4, stream)
    torch.cuda.synchronize()
    sample = np.sort(rng.choice(rows, size=32, replace=False))
    inputs = hidden[:, :-1, :].reshape(rows, width)[torch.from_numpy(sample).cuda()].float().cpu().numpy().astype(np.float64)
    z = oracle.round_bf16(inputs @ weight.float().cpu().numpy().astype(np.float64).T)
    peak = z.max(axis=1)
    targets = labels_host[:, 1:].reshape(-1)[sample]
    want = np.log(np.exp(z - peak[:, None]).sum(axis=1)) - (z[np.arange(len(sample)), targets] - peak)
    got = row_loss.cpu().numpy()[sample]
    error = float(np.abs(got - want).max() / max(1.0, float(np.abs(want).max())))
    total = float(row_loss.double().sum().item() / rows)
    value = float(loss.storage.tolist(stream)[0])
    return dict(ms_per_step=ms, rows=rows, width=width, vocab=vocab, dtype="bf16", tflops=flops / (ms * 1e-3) / 1e12,
                frac_of_sustained_peak=flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                logits_bytes=logits_bytes, launches_per_step=9,
                what="LM head + cross-entropy forward + backward (qmoe_head_forward / _backward): 3 tcgen05 products, one pass over the logits",
                loss=value,
                check=dict(ok=bool(error <= BF16_TOL and abs(value - total) <= 1e-3 * abs(total)), row_loss=error,
                           mean_of_rows=total, tolerance=BF16_TOL, sampled_rows=int(len(sample))))


class StackedWeights:
    """Per-expert view of a gathered [experts, rows, columns] bf16 tensor on the device; an expert's block
    crosses to the host only when the oracle asks for it."""

    def __init__(self, tensor):
        self.tensor = tensor

    def __len__(self):
        return self.tensor.shape[0]

    def __getitem__(self, e):
        return self.tensor[e].float().cpu().numpy()


def ep_check(layer, w, rank, world, step, x_dev, g_dev, counts, logical_of_physical, torch, dist, np):
    """One more step, its results compared with the CPU oracle: the per-expert counts over all ranks' tokens
    (bit-exact, from the devices' own fp32 logits) and the auxiliary loss; y and dx of 48 tokens per rank; the
    three weight gradients of one expert of rank 0.  Expert numbers are the layer's internal (rank-major) ones.
    Every rank takes part in the gathers; rank 0 computes and shares the verdict."""
    T_global, d, E, k, h = w["tokens"], w["d"], w["E"], w["k"], w["h"]
    T, L = T_global // world, E // world
    device = x_dev.device
    y, aux, dx = step()
    torch.cuda.synchronize()
    buf = layer._saved[0]["buf"]

    def as_tensor(storage, shape, dtype):
        from qutai_b200 import lib

        out = torch.empty(shape, dtype=dtype, device=device)
        lib.call("qmoe_memcpy_d2d", out.data_ptr(), storage.ptr, storage.nbytes, torch.cuda.current_stream().cuda_stream)
        return out

    def gathered(tensor):
        if world == 1:
            return tensor
        out = torch.empty((world * tensor.shape[0], *tensor.shape[1:]), dtype=tensor.dtype, device=device)
        dist.all_gather_into_tensor(out, tensor.contiguous())
        return out

    rng = np.random.default_rng(1234)
    sample_local = torch.from_numpy(np.sort(rng.choice(T, size=min(48, T), replace=False))).to(device)
    scores = gathered(as_tensor(buf["scores"], (T, E), torch.float32))
    x_all, g_all = gathered(x_dev), gathered(g_dev)
    y_s = gathered(as_tensor(y.storage, (T, d), torch.bfloat16)[sample_local])
    forward_only = dx is None
    dx_s = None if forward_only else gathered(as_tensor(dx.storage, (T, d), torch.bfloat16)[sample_local])
    aux_value = as_tensor(aux.storage, (1,), torch.float32)
    shape = {"w_gate": (L, h, d), "w_up": (L, h, d), "w_down": (L, d, h)}
    weights = {name: StackedWeights(gathered(as_tensor(buf[name], shape[name], torch.bfloat16))) for name in shape}
    torch.cuda.synchronize()
    verdict = None
    if rank == 0:
        from oracle import moe_oracle as oracle

        router = router_weights(w)[logical_of_physical].astype(np.float64)     # rows in the layer's internal order
        scores_host = scores.cpu().numpy().astype(np.float64)
        route = oracle.routing(scores_host, k)
        counts_exact = tuple(counts) == route["counts"] and sum(route["counts"]) == T_global * k
        aux_err = abs(float(aux_value.item()) - route["aux"])
        sample = torch.cat([sample_local + p * T for p in range(world)])
        idx = sample.cpu().numpy()
        xs_host = x_all[sample].float().cpu().numpy().astype(np.float64)
        ys, _, ctx = oracle.moe_forward(xs_host, router, weights["w_gate"], weights["w_up"], weights["w_down"], k,
                                        scores=scores_host[idx])
        y_err = oracle.max_rel_err(y_s.float().cpu().numpy(), ys)
        dx_err = dw_err = None
        if not forward_only:
            gs_host = g_all[sample].float().cpu().numpy().astype(np.float64)
            grads = oracle.moe_backward(ctx, gs_host, 0.0)
            # the auxiliary-loss path needs the utilisation over ALL tokens (src/qutai/backends/cpu_lm.py:262-275)
            probs, util = route["probs"][idx], route["utilization"]
            d_scores_aux = AUX_GRAD * E / T_global * probs * (util[None, :] - (probs @ util)[:, None])
            dx_err = oracle.max_rel_err(dx_s.float().cpu().numpy(), grads["x"] + d_scores_aux @ router)
            # one expert of rank 0 (the one whose row count is the median of the rank's): all its rows, whichever rank sent them
            local = sorted(range(L), key=lambda j: (counts[j], j))
            e = local[len(local) // 2]
            members = torch.from_numpy(route["ids"][e]).to(device)
            gate_w = route["weights"][route["ids"][e], route["slots"][e]]
            xe = x_all[members].float().cpu().numpy().astype(np.float64)
            dy = g_all[members].float().cpu().numpy().astype(np.float64) * gate_w[:, None]
            _, saved = oracle.expert_forward(xe, weights["w_gate"][e], weights["w_up"][e], weights["w_down"][e])
            want = oracle.expert_backward(saved, dy, weights["w_gate"][e], weights["w_up"][e], weights["w_down"][e])[:3]
            expert = layer.experts[e]
            got = [as_tensor(p.grad.storage, shape, torch.float32).cpu().numpy() for p, shape in
                   ((expert.gate.weight, (h, d)), (expert.up.weight, (h, d)), (expert.down.weight, (d, h)))]
            dw_err = max(oracle.max_rel_err(a, b) for a, b in zip(got, want))
        ok = counts_exact and aux_err <= 1e-5 and y_err <= BF16_TOL and (forward_only or (dx_err <= BF16_TOL and dw_err <= BF16_TOL))
        verdict = dict(ok=bool(ok), counts_exact=bool(counts_exact), aux_abs_err=aux_err, y=y_err, dx=dx_err, dw=dw_err,
                       tolerance=BF16_TOL, sampled_tokens=int(idx.size),
                       how="CPU float64 oracle on the devices' own fp32 logits; max |a - b| / max |b|; counts over all ranks' tokens")
    if world > 1:
        box = [verdict]
        dist.broadcast_object_list(box, src=0)
        verdict = box[0]
    return verdict


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-decode", action="store_true", help="leave the decode-shaped latency block out of the c3 line")
    parser.add_argument("--no-library-gemm", action="store_true", help="do not time the library bf16 product on this GPU")
    parser.add_argument("--no-decoder", action="store_true", help="leave the whole-decoder training step out of the line")
    parser.add_argument("--no-attention", action="store_true", help="leave the attention block out of the line")
    parser.add_argument("--no-head", action="store_true", help="leave the language-model head out of the line")
    parser.add_argument("--no-block", action="store_true", help="leave the fused norm + layer + residual block out of the line")
    parser.add_argument("--preroll", type=float, default=2.0,
                        help="seconds of back-to-back steps before the timed ones (the power-capped operating point)")
    parser.add_argument("--trace", default="", help="write a chrome trace of a few steps (rank 0) to this path")
    parser.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                        help="N > 1: 'balanced' times the contiguous placement first and reports it beside the headline")
    parser.add_argument("--overlap", action="store_true",
                        help="N > 1: let half of the experts' rows travel behind the first product on the other half")
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
