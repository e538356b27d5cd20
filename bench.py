#!/usr/bin/env python
"""Benchmark of the MoE block: tokens/s through one Mixtral-8x7B-shaped layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--tokens T]

One "step" is one forward of the block over one batch of synthetic tokens (seeded; weights
N(0, 0.02^2) rounded to bf16, activations N(0, 1), per-expert logit bias N(0, 0.5^2) for load skew).
At N = 1 the default workload is the Mixtral-8x7B layer at 4096 tokens in bf16.  At N > 1 the experts
are sharded expert-parallel and every rank routes its own 4096 tokens (weak scaling); launch with
torchrun, one rank per GPU.

The JSON line carries:
  value     tokens/s with activations already resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through execute_real_moe_layer with pinned HOST f32 buffers, copies included
  roofline  the routed gate/up + SwiGLU grouped GEMM (the dominant kernel) against the measured bf16 peak
  cpu_baseline  the CPU oracle (a port of the reference's per-token f64 path) on a bounded token sample
`--impl reference` times that CPU path alone, on all host threads.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the routed gate/up + SwiGLU kernel the
# workload selects, from one-pass ncu captures of this command (kernel name -> bytes).
NCU_TRAFFIC_BYTES = {
    # CTA-pair kernel: 1.966 GB read + 228 MB written at 4096 tokens; 1.908 GB + 29.6 MB at 512
    "mixtral:4096:grouped_gemm_2cta_kernel": 2.194e9,
    "mixtral:512:grouped_gemm_2cta_kernel": 1.938e9,
    # single-CTA kernel: 1.95 GB read + 227.5 MB written at 4096 tokens; 1.904 GB + 29.9 MB at 512
    "mixtral:4096:grouped_gemm_tcgen05_kernel": 2.18e9,
    "mixtral:512:grouped_gemm_tcgen05_kernel": 1.934e9,
    # 256-row INT8 kernel: 1.013 GB read + 223 MB written at 4096 tokens
    "mixtral_int8:4096:grouped_gemm_w8_m256_kernel": 1.236e9,
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []  # (host time, fields)
        self.proc = None
        self.thread = None
        self.window = None  # (t0, t1) of the region under load

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        inside = [p for (t, p) in self.samples
                  if self.window is None or (self.window[0] <= t <= self.window[1])]
        for s in inside:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(self.NAMES, s[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_oracle_rate(shape, w, x_host, max_seconds, threads=0, accum=None, ol=None):
    """tokens/s of the CPU oracle (all host threads) on a bounded token sample; `accum` picks the
    reference's accumulation mode (default f64, its certified path; ACC_F32 is its strict path)."""
    from oracle import oracle as orc
    from oracle.from_synth import oracle_layer

    if ol is None:
        ol = oracle_layer(shape, w)
    if accum is None:
        accum = orc.ACC_F64
    cores = orc.max_threads() if threads <= 0 else threads
    n0 = min(x_host.shape[0], max(cores, 4))
    t = time.perf_counter()
    ol.forward(x_host[:n0], accum=accum, nthreads=threads)
    dt = time.perf_counter() - t
    rate = n0 / dt
    n = int(min(x_host.shape[0], max(n0, rate * max_seconds)))
    n = max(cores, n // cores * cores) if n >= cores else n
    n = min(n, x_host.shape[0])
    t = time.perf_counter()
    ol.forward(x_host[:n], accum=accum, nthreads=threads)
    dt = time.perf_counter() - t
    return n / dt, cores, n, ol


def run_stack_bench(args):
    """Decode benchmark: a stack of W8A16 Mixtral-shaped MoE-FFN layers with a residual add between
    layers (attention omitted), Zipf-skewed routing, small batches.  One step = one pass of the batch
    through all layers (replayed from a CUDA graph on a side stream)."""
    import ctypes as C

    import numpy as np
    import torch

    from ateniaengine_b200 import _lib, synth
    from ateniaengine_b200.moe import RealMoeStack

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    shape = synth.SHAPES["mixtral_int8"]
    B = args.tokens or 8
    n_layers = args.layers
    # expert parallelism for decode: every rank holds the same batch and E / world experts of each layer
    el = shape.num_experts // world
    ws = [synth.make_weights(shape, 5 + l, dev, experts=(rank * el, el) if world > 1 else None) for l in range(n_layers)]
    layers = [synth.build_layer(shape, w, max_tokens=max(B, 1), ep_rank=rank, ep_world=world) for w in ws]
    if world > 1:
        nb = _lib.lib().atenia_moe_ep_unique_id_bytes()
        idt = torch.zeros(nb, dtype=torch.uint8, device=dev)
        if rank == 0:
            buf = C.create_string_buffer(nb)
            _lib.check(_lib.lib().atenia_moe_ep_get_unique_id(buf), "ep_get_unique_id")
            idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).to(dev)
        dist.broadcast(idt, 0)
        layers[0].ep_init(bytes(idt.cpu().numpy().tobytes()))
        for l in layers[1:]:
            l.ep_attach(layers[0])
        for l in layers:
            l.ep_replicated_tokens(True)
    stack = RealMoeStack(layers, residual=2)
    x = synth.make_activations(shape, 5, dev, tokens=B, dtype=torch.float32)
    out = torch.empty_like(x)
    # experts touched per layer (weights that must cross HBM): one eager pass with routing outputs
    cur = x
    touched = []
    gemm_ms = 0.0
    for l in layers:
        l.enable_timing(True)
        xn = cur * torch.rsqrt((cur * cur).mean(dim=1, keepdim=True) + 1e-5)
        y, aux = l.forward(xn, out_dtype=torch.float32, aux=True, sync=True)
        touched.append(int(torch.unique(aux["topk_idx"]).numel()))
        gemm_ms += l.last_gemm_ms(0) + l.last_gemm_ms(1)
        l.enable_timing(False)
        cur = cur + y
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(max(args.warmup, 3)):
            stack.forward(x, out=out)
        side.synchronize()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        time.sleep(0.8)
        for _ in range(3):  # every rank replays the same graphs: each one holds a collective per layer
            stack.forward(x, out=out)
        side.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        launches0 = _lib.lib().atenia_moe_counter(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(args.steps):
            stack.forward(x, out=out)
        e1.record(side)
        side.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        launches = int(_lib.lib().atenia_moe_counter(1) - launches0)
        sampler.window = (t0, time.perf_counter())
        clocks = sampler.stop() if rank == 0 else None
    _lib.check(_lib.lib().atenia_moe_stack_check(stack._h, None), "stack_check")
    assert torch.isfinite(out).all()
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return 0
    peaks, peak_src = load_peaks()
    wbytes = sum(t * 3 * shape.d_model * shape.d_ff for t in touched)  # one byte per weight
    # the rank that owns the most touched experts sets the pace; with an even split each streams 1 / world
    achieved = wbytes / world / (ms * 1e-3) / 1e9
    line = {"metric": "moe_ffn_stack_tokens_per_s", "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "int8 weights, bf16 operands, f32 residual stream (W8A16)",
            "data": "synthetic",
            "config": {"workload": f"mixtral_int8 stack: {n_layers} layers, d_model={shape.d_model} d_ff={shape.d_ff} "
                                   f"experts={shape.num_experts} top_k={shape.top_k}, pre-norm residual blocks x + MoE(rmsnorm(x)), batch={B}",
                       "routing_skew": "zipf(1.1)", "experts_touched_per_layer": touched,
                       "parallelism": "single GPU" if world == 1 else
                       f"expert-parallel ep{world}, the batch replicated on every rank, one NCCL all-reduce per layer",
                       "l2_policy": f"inputs larger than L2: {wbytes / 1e6:.0f} MB of expert weights per step"},
            "roofline": {"bound": "hbm", "kernel": "whole step (weights of the touched experts, once per step)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peak_src, "traffic": None,
                         "eager_gemm_ms_per_step": gemm_ms},
            "cpu_baseline": None, "e2e": None, "clocks": clocks, "gpu_launches": launches,
            "note": "launches replayed from a CUDA graph are counted once per layer"}
    print(json.dumps(line))
    return 0


def arm_watchdog(seconds, what):
    """A rank that waits for a peer that died would wait for ever: end the process instead."""
    def fire():
        sys.stderr.write(f"bench.py: {what} exceeded {seconds:.0f} s, giving up\n")
        sys.stderr.flush()
        os._exit(3)
    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


def host_threads():
    """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm
    must not inherit that, so the count is passed to the oracle explicitly."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def layer_roofline(shape, T, touched, peaks, int8):
    """Whole-forward target on one GPU: the slower of the expert flops at the measured tensor peak and
    the bytes that must cross HBM (weights of the experts that got a row, router, activations in and
    out) at the measured copy rate."""
    d, F, Fs, E, k = shape.d_model, shape.d_ff, shape.shared_d_ff, shape.num_experts, shape.top_k
    flops = T * (k * 6.0 * d * F + 6.0 * d * Fs + 2.0 * d * E)
    b = 1 if int8 else 2
    wbytes = touched * 3.0 * d * F * b + 3.0 * d * Fs * b + E * d * 4.0
    if int8:
        wbytes += touched * (2 * F + d) * 4.0 + (2 * Fs + d) * 4.0 * (1 if Fs else 0)
    abytes = 2.0 * T * d * 2
    t_c = flops / (peaks["bf16_tflops"] * 1e12)
    t_h = (wbytes + abytes) / (peaks["hbm_gbs"] * 1e9)
    return {"flops": flops, "hbm_bytes": wbytes + abytes, "t_tensor_ms": t_c * 1e3, "t_hbm_ms": t_h * 1e3,
            "bound": "tensor" if t_c >= t_h else "hbm", "target_ms": max(t_c, t_h) * 1e3}


class EpGroup:
    """torch.distributed plumbing of one benchmark process (one rank per GPU)."""

    def __init__(self, gpus):
        import torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if gpus > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def sync(self):
        import torch
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, v):
        import torch
        if self.dist is None:
            return float(v)
        t = torch.tensor([float(v)], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather_floats(self, vals):
        """[world, len(vals)] list of every rank's values."""
        import torch
        t = torch.tensor([float(v) for v in vals], device=self.dev)
        if self.dist is None:
            return [t.tolist()]
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [o.tolist() for o in out]

    def join_ep(self, layer, direct=False):
        """Joins the layer to the expert-parallel group; with `direct` also maps the peers' buffers for the
        peer-store exchange.  Returns True when every rank has the direct exchange set up, False when the
        layer is on the NCCL send/receive exchange."""
        import ctypes as C

        import torch
        from ateniaengine_b200 import _lib
        nb = _lib.lib().atenia_moe_ep_unique_id_bytes()
        idt = torch.zeros(nb, dtype=torch.uint8, device=self.dev)
        if self.rank == 0:
            buf = C.create_string_buffer(nb)
            _lib.check(_lib.lib().atenia_moe_ep_get_unique_id(buf), "ep_get_unique_id")
            idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).to(self.dev)
        self.dist.broadcast(idt, 0)
        layer.ep_init(bytes(idt.cpu().numpy().tobytes()))
        if not direct:
            return False
        mine = torch.frombuffer(bytearray(layer.ep_ipc_export()), dtype=torch.uint8).to(self.dev)
        blobs = [torch.empty_like(mine) for _ in range(self.world)]
        self.dist.all_gather(blobs, mine)
        ok = 1.0
        try:
            layer.ep_ipc_import(b"".join(bytes(b.cpu().numpy().tobytes()) for b in blobs))
        except Exception as e:  # no peer access between these GPUs, or IPC refused
            sys.stderr.write(f"bench.py: rank {self.rank}: direct exchange unavailable ({e})\n")
            ok = 0.0
        t = torch.tensor([ok], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    def make_ep_layer(self, shape, w, max_tokens, direct):
        """An expert-parallel layer of this rank with the direct exchange if every rank can have it, else
        (all ranks together) a fresh layer on the NCCL exchange."""
        from ateniaengine_b200 import synth
        layer = synth.build_layer(shape, w, max_tokens=max_tokens, ep_rank=self.rank, ep_world=self.world)
        if self.join_ep(layer, direct=direct) or not direct:
            return layer, direct
        layer.close()
        layer = synth.build_layer(shape, w, max_tokens=max_tokens, ep_rank=self.rank, ep_world=self.world)
        self.join_ep(layer, direct=False)
        return layer, False

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def time_steps(grp, fn, steps, host=None):
    """ms per step of `steps` calls of fn, CUDA events on the current stream, barrier + device sync on
    both sides, max over ranks.  `host` (a list) receives this rank's wall-clock ms per step spent ISSUING
    the calls: when it is close to the device figure the step is bound by the host's launch rate."""
    import torch
    grp.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    t1 = time.perf_counter()
    e1.record()
    grp.sync()
    if host is not None:
        host.append((t1 - t0) * 1e3 / steps)
    return grp.max_over_ranks(e0.elapsed_time(e1) / steps)


def measure_record(grp, name, T_total, args, peaks, seed=2, direct=False):
    """One extra workload measured like the headline one (warm-up, K steps, CUDA events, max over
    ranks): tokens/s of the whole job and the fraction of the single-GPU-equivalent roofline.  At N > 1
    the batch of T_total tokens is split over the ranks (strong scaling) and rank 0 also times the
    unsharded layer on the whole batch in the same run."""
    import torch
    from ateniaengine_b200 import synth
    shape = synth.SHAPES[name]
    G = grp.world if grp.dist is not None else 1
    T = T_total // G
    el = shape.num_experts // G
    w = synth.make_weights(shape, seed, grp.dev, experts=(grp.rank * el, el) if G > 1 else None)
    x = synth.make_activations(shape, seed + grp.rank, grp.dev, tokens=T)
    if G > 1:
        layer, direct = grp.make_ep_layer(shape, w, T, direct)
    else:
        layer = synth.build_layer(shape, w, max_tokens=T)
    out = torch.empty_like(x)
    fn = lambda: layer.forward(x, out=out)
    for _ in range(args.warmup):
        fn()
    layer.check()
    layer.enable_timing(True)
    host = []
    ms = time_steps(grp, fn, args.steps, host)
    layer.check()
    phases = [layer.last_phase_ms(i) for i in range(6)]
    recv_rows = layer.last_recv_rows() if G > 1 else T * shape.top_k
    layer.enable_timing(False)
    _, aux = layer.forward(x, aux=True, sync=True)
    touched = int(torch.unique(aux["topk_idx"]).numel())
    per_rank = grp.gather_floats([recv_rows] + phases)
    rec = {"workload": f"{shape.name}: d_model={shape.d_model} d_ff={shape.d_ff} experts={shape.num_experts} "
                       f"top_k={shape.top_k} shared_d_ff={shape.shared_d_ff}",
           "tokens_per_step": T * G, "n_gpus": G, "scaling": "strong" if G > 1 else "single GPU",
           "dtype": "int8 weights, bf16 activations (W8A16)" if shape.int8 else "bf16",
           "ms_per_step": ms, "tokens_per_s": T * G / (ms * 1e-3),
           "host_issue_ms_per_step": grp.max_over_ranks(host[0])}
    rl = layer_roofline(shape, T * G, shape.num_experts if G > 1 else touched, peaks, shape.int8)
    rec["roofline"] = {"bound": rl["bound"], "target_ms_one_gpu": rl["target_ms"], "t_tensor_ms": rl["t_tensor_ms"],
                       "t_hbm_ms": rl["t_hbm_ms"], "frac": rl["target_ms"] / G / ms,
                       "note": "target = slower of expert flops at the measured bf16 peak and touched weight + "
                               "activation bytes at the measured HBM rate, divided by the GPU count"}
    slow = max(range(len(per_rank)), key=lambda r: per_rank[r][0])
    names = ("route_permute_gather", "rows_out", "routed_gemms", "rows_back", "shared_combine", "forward")
    rec["phases_ms_slowest_rank"] = {n: per_rank[slow][1 + i] for i, n in enumerate(names)}
    if G > 1:
        rows = [r[0] for r in per_rank]
        rec["rows_received_per_rank"] = {"max": max(rows), "mean": sum(rows) / len(rows),
                                         "imbalance_max_over_mean": max(rows) / max(sum(rows) / len(rows), 1.0)}
        flags = os.environ.get("ATENIA_MOE_EP_FLAGS", "0") not in ("", "0")
        rec["exchange"] = (("peer stores over NVLink (direct), " + ("ordered by flags in peer memory" if flags
                                                                       else "NCCL for counts and ordering"))
                           if direct else "NCCL send/recv groups")
        # the same batch on one GPU, timed by rank 0 in this very run (the others wait at the barrier)
        single = None
        if grp.rank == 0:
            wf = synth.make_weights(shape, seed, grp.dev)
            xs = [synth.make_activations(shape, seed + r, grp.dev, tokens=T) for r in range(G)]
            xf = torch.cat(xs)
            full = synth.build_layer(shape, wf, max_tokens=T * G)
            of = torch.empty_like(xf)
            for _ in range(args.warmup):
                full.forward(xf, out=of)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                full.forward(xf, out=of)
            e1.record()
            torch.cuda.synchronize()
            single = e0.elapsed_time(e1) / args.steps
            full.check()
            # the sharded run must give the unsharded run's rows (same rows, same experts, same order)
            rec["max_abs_diff_vs_one_gpu_rank0_rows"] = float((of[:T].float() - out.float()).abs().max())
            full.close()
            del wf, xf, of
        grp.sync()
        # the same forward replayed as one CUDA graph (a one-layer stack on a side stream): the direct
        # exchange reads nothing on the host, so kernels, collectives and the second stream's fork and
        # join are all captured, and the host issues one launch per step
        gms = None
        if direct:
            from ateniaengine_b200.moe import RealMoeStack
            st1 = RealMoeStack([layer], residual=False)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                gfn = lambda: st1.forward(x, out=out)
                for _ in range(max(args.warmup, 3)):  # eager, capture, replays
                    gfn()
                layer.check()
                gms = time_steps(grp, gfn, args.steps)
                layer.check()
            torch.cuda.current_stream().wait_stream(side)
            st1.close()
        if grp.rank == 0:
            rec["one_gpu_ms_same_run"] = single
            rec["speedup_vs_one_gpu_same_run"] = single / ms
            if gms is not None:
                rec["graph_replay"] = {"ms_per_step": gms, "tokens_per_s": T * G / (gms * 1e-3),
                                       "speedup_vs_one_gpu_same_run": single / gms,
                                       "frac": rl["target_ms"] / G / gms,
                                       "note": "the same forward replayed as one CUDA graph through a "
                                               "one-layer atenia_moe_stack: one host launch per step"}
    layer.close()
    del w, x, out
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per rank (default: the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--layers", type=int, default=32, help="layers of the mixtral_int8_stack workload")
    ap.add_argument("--windows", type=int, default=25, help="further K-step windows timed after the first (0: none)")
    ap.add_argument("--no-records", action="store_true", help="skip the extra workloads of the default line")
    args = ap.parse_args()
    arm_watchdog(float(os.environ.get("ATENIA_BENCH_WATCHDOG_S", "600" if args.impl == "reference" else "420")),
                 "the whole run")
    if args.workload == "mixtral_int8_stack":
        return run_stack_bench(args)
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        args.gpus = world

    import numpy as np
    import torch

    from ateniaengine_b200 import synth

    shape = synth.SHAPES[args.workload]
    T = args.tokens or shape.tokens
    dtype_name = "int8 weights, bf16 activations (W8A16)" if shape.int8 else "bf16"
    config = {"workload": f"{shape.name}: d_model={shape.d_model} d_ff={shape.d_ff} experts={shape.num_experts} "
                          f"top_k={shape.top_k} shared_d_ff={shape.shared_d_ff} tokens_per_rank={T}",
              "tokens_per_step": T * max(args.gpus, 1),
              "routing_skew": shape.bias,
              "parallelism": "single GPU" if args.gpus == 1 else f"expert-parallel ep{args.gpus}, NCCL send/recv all-to-all",
              "l2_policy": "inputs larger than L2: every step streams the expert weights "
                           f"({3 * shape.d_model * shape.d_ff * shape.num_experts * (1 if shape.int8 else 2) / 1e6:.0f} MB)"}

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return 0
        dev = "cuda:0" if torch.cuda.is_available() else "cpu"
        if dev == "cpu" and shape.int8:
            print(json.dumps({"impl": "reference", "unavailable": "int8 synthetic weights are quantised on the GPU"}))
            return 0
        w = synth.make_weights(shape, 2, dev)
        x = synth.make_activations(shape, 2, dev, tokens=min(T, 512)).float().cpu().numpy()
        from oracle.from_synth import oracle_layer
        ol = oracle_layer(shape, w)
        del w
        cores = host_threads()  # all host cores, whatever OMP_NUM_THREADS the launcher exported
        # size one step to about 2 s of CPU work; the sizing run and one more step are the warm-up
        # (CPU steps have no clocks or caches to settle beyond that)
        n0 = min(x.shape[0], max(cores, 4))
        t = time.perf_counter()
        ol.forward(x[:n0], nthreads=cores)
        rate0 = n0 / (time.perf_counter() - t)
        # about 2 s per step, less when many steps are asked for: the whole run stays near two minutes
        per_step_s = min(2.0, 120.0 / (args.steps + 1))
        n = int(min(x.shape[0], max(1, rate0 * per_step_s)))
        ol.forward(x[:n], nthreads=cores)
        t = time.perf_counter()
        for _ in range(args.steps):
            ol.forward(x[:n], nthreads=cores)
        dt = time.perf_counter() - t
        val = n * args.steps / dt
        line = {"metric": METRIC, "value": val, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64 accumulate",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                                 "sample": f"{n} tokens per step, CPU oracle (C restatement of the reference's "
                                           f"per-token f64 path), {cores} OpenMP threads"},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------------ our arm (GPU)
    import ateniaengine_b200 as ae
    from ateniaengine_b200 import _lib

    grp = EpGroup(args.gpus)
    dev, dist = grp.dev, grp.dist
    local_rank = grp.local_rank
    # rows travel by the library's own peer-store kernels over NVLink (the direct exchange);
    # ATENIA_BENCH_EP_DIRECT=0 times the NCCL send/recv exchange instead
    direct = args.gpus > 1 and os.environ.get("ATENIA_BENCH_EP_DIRECT", "1") != "0"
    E = shape.num_experts
    el = E // args.gpus
    w = synth.make_weights(shape, 2, dev, experts=(rank * el, el))
    x = synth.make_activations(shape, 2 + rank, dev, tokens=T)
    if args.gpus > 1:
        layer, direct = grp.make_ep_layer(shape, w, T, direct)
    else:
        layer = synth.build_layer(shape, w, max_tokens=T)
    if args.gpus > 1:
        if direct:
            flags = os.environ.get("ATENIA_MOE_EP_FLAGS", "0") not in ("", "0")
            config["parallelism"] = (f"expert-parallel ep{args.gpus}, rows stored peer to peer over NVLink, "
                                     + ("counts and ordering by flags in peer memory" if flags
                                        else "NCCL for counts and ordering"))
    out = torch.empty_like(x)
    fwd = lambda: layer.forward(x, out=out)

    for _ in range(args.warmup):
        fwd()
    layer.check()
    grp.sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    time.sleep(0.8)  # nvidia-smi needs a moment before its first reading
    # every rank runs the same forwards: under expert parallelism each one is a set of collectives.
    # The library's CUDA events (grouped GEMMs, phases) are recorded inside the timed forwards: the
    # figures below are those of the last timed step, not of a separate pass.
    layer.enable_timing(True)
    for _ in range(args.warmup):
        fwd()
    t_load0 = time.perf_counter()
    launches0 = _lib.lib().atenia_moe_counter(1)
    ms = time_steps(grp, fwd, args.steps)
    launches = int(_lib.lib().atenia_moe_counter(1) - launches0)
    layer.check()
    gemm1_ms, gemm2_ms = layer.last_gemm_ms(0), layer.last_gemm_ms(1)
    phases = [layer.last_phase_ms(i) for i in range(6)]
    recv_rows = layer.last_recv_rows() if args.gpus > 1 else T * shape.top_k
    layer.enable_timing(False)
    t_load1 = time.perf_counter()
    per_rank = grp.gather_floats([recv_rows, gemm1_ms, gemm2_ms] + phases)
    _, aux = layer.forward(x, aux=True, sync=True)
    touched = int(torch.unique(aux["topk_idx"]).numel())

    # ---- end to end at N > 1: every rank copies its own tokens from pinned host memory, runs the
    # expert-parallel forward and copies its result back; same forwards on every rank, max over ranks
    e2e_multi = None
    if args.gpus > 1:
        hin = torch.empty((T, shape.d_model), dtype=torch.float32).pin_memory()
        hin.copy_(x.float().cpu())
        hout = torch.empty_like(hin).pin_memory()
        xd = torch.empty((T, shape.d_model), dtype=torch.float32, device=dev)
        od = torch.empty_like(xd)

        def one_step():
            xd.copy_(hin, non_blocking=True)
            layer.forward(xd, out=od)
            hout.copy_(od, non_blocking=True)

        for _ in range(3):
            one_step()
        grp.sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            one_step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / args.steps
        layer.check()
        dt = grp.max_over_ranks(dt)
        nfl = T * shape.d_model
        e2e_multi = {"value": T * args.gpus / dt, "unit": UNIT, "h2d_bytes_per_step": nfl * 4 * args.gpus,
                     "d2h_bytes_per_step": nfl * 4 * args.gpus, "ms_per_step": dt * 1e3,
                     "api": "atenia_moe_forward per rank (expert parallel), pinned host f32 in/out on every rank"}

    peaks, peak_src = load_peaks()

    # ---- N > 1: a sample of rank 0's rows against the CPU oracle, outside the timed regions
    parity = None
    if args.gpus > 1 and not shape.int8:
        if rank == 0:
            from oracle.from_synth import oracle_layer, rel_l2
            wf = synth.make_weights(shape, 2, dev)
            ol = oracle_layer(shape, wf)
            del wf
            torch.cuda.empty_cache()
            ns = min(32, T)
            ref = ol.forward(x[:ns].float().cpu().numpy(), nthreads=host_threads())
            parity = {"tokens": ns, "rel_l2_vs_cpu_oracle": rel_l2(out[:ns].float().cpu().numpy(), ref), "bar": 1e-2}
            del ol
        grp.sync()

    # ---- extra records of the line: the other named workloads, each measured like the headline
    records = {}
    if not args.no_records and args.workload == "mixtral" and not args.tokens:
        # release the headline layer first (N = 1 keeps it for the e2e leg below)
        if args.gpus == 1:
            records["w8a16_mixtral_4096"] = measure_record(grp, "mixtral_int8", 4096, args, peaks, seed=5)
            records["deepseek_v2_lite_ep"] = measure_record(grp, "deepseek_v2_lite", 8192, args, peaks, seed=4)
            records["qwen15_moe_2048"] = measure_record(grp, "qwen_moe", 2048, args, peaks, seed=3)
        else:
            records["deepseek_v2_lite_ep"] = measure_record(grp, "deepseek_v2_lite", 8192, args, peaks, seed=4,
                                                            direct=direct)
            if args.gpus == 2:  # the Qwen-shaped layer is named for 1 and 2 GPUs (60 experts: 30 per rank)
                records["qwen15_moe_2048_ep"] = measure_record(grp, "qwen_moe", 2048, args, peaks, seed=3,
                                                               direct=direct)

    # further windows of exactly K steps of the headline workload, back to back, after everything else:
    # the first window above is a burst after an idle moment, the median of these is what a loaded GPU
    # sustains (clocks settle under the power cap).  The clock record covers the timed region and these.
    win = []
    t_win0 = time.perf_counter()
    for _ in range(max(args.windows, 0)):
        win.append(time_steps(grp, fwd, args.steps))
    if rank == 0:
        # the timed region is tens of milliseconds (two or three samples); the record runs from its
        # start to the end of the measurements that follow it, all of them under load
        sampler.window = (t_load0, max(t_load1, t_win0))
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0 and win:
        sampler.window = (t_win0, time.perf_counter())
        clocks_windows = sampler.stop()
    else:
        clocks_windows = None

    if rank != 0:
        grp.close()
        return 0

    slow = max(range(len(per_rank)), key=lambda r: per_rank[r][0])
    rows_slow = per_rank[slow][0]
    g1_slow, g2_slow = per_rank[slow][1], per_rank[slow][2]
    groups = (shape.num_experts // args.gpus) * (args.gpus if args.gpus > 1 and not direct else 1)
    if shape.int8:
        kname = "grouped_gemm_w8_tmem_kernel" if rows_slow < 256 * groups else "grouped_gemm_w8_m256_kernel"
    else:
        kname = "grouped_gemm_2cta_kernel" if rows_slow >= 512 * groups else "grouped_gemm_tcgen05_kernel"
    # dominant kernel: the routed gate/up + SwiGLU grouped GEMM of the rank with the most rows
    flops1 = 4.0 * rows_slow * shape.d_model * shape.d_ff  # gate and up: 2 * 2 * rows * d * F
    achieved = flops1 / (g1_slow * 1e-3) / 1e12
    rl = layer_roofline(shape, T, touched if args.gpus == 1 else shape.num_experts // args.gpus, peaks, shape.int8)
    names = ("route_permute_gather", "rows_out", "routed_gemms", "rows_back", "shared_combine", "forward")
    roofline = {"bound": "tensor", "kernel": kname + "<kSwiGLU> (routed gate/up + SwiGLU)",
                "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"], "peak_source": f"{peak_src} (burst cuBLAS bf16)",
                "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
                "traffic": NCU_TRAFFIC_BYTES.get(f"{shape.name}:{T}:{kname}") if args.gpus == 1 else None,
                "rows": rows_slow, "launch_ms": g1_slow, "down_gemm_ms": g2_slow,
                "down_gemm_tflops": 2.0 * rows_slow * shape.d_model * shape.d_ff / (g2_slow * 1e-3) / 1e12,
                "timed_inside": "the last step of the timed region (events on the launching stream)",
                "phases_ms": {n: per_rank[slow][3 + i] for i, n in enumerate(names)},
                "layer_frac_of_tensor_roofline": (T * shape.top_k * 6.0 * shape.d_model * shape.d_ff +
                                                  T * 6.0 * shape.d_model * shape.shared_d_ff) /
                                                 (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    if args.gpus == 1:
        roofline["layer"] = {"bound": rl["bound"], "target_ms": rl["target_ms"], "frac": rl["target_ms"] / ms}
    windows = None
    if win:
        med = statistics.median(win)
        windows = {"count": len(win), "steps_each": args.steps, "ms_per_step_median": med, "ms_per_step_min": min(win),
                   "ms_per_step_max": max(win), "tokens_per_s_median": T * args.gpus / (med * 1e-3),
                   "first_window_ms_per_step": ms, "clocks": clocks_windows,
                   "layer_frac_of_sustained_tensor_peak": (T * shape.top_k * 6.0 * shape.d_model * shape.d_ff +
                                                           T * 6.0 * shape.d_model * shape.shared_d_ff) /
                                                          (med * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                   "note": "value / ms_per_step are the first window after warm-up (a burst); these windows "
                           "follow it back to back, so their median is the sustained figure under the power cap"}

    # ---- end to end through the operator registry with pinned host buffers (N = 1 only)
    e2e = e2e_multi
    if args.gpus == 1:
        lid = ae.register_resident_moe_layer(layer)
        hin = torch.empty((T, shape.d_model), dtype=torch.float32).pin_memory()
        hin.copy_(x.float().cpu())
        hout = torch.empty_like(hin).pin_memory()
        from ateniaengine_b200.moe import execute_real_moe_layer_ptr
        nfl = T * shape.d_model
        for _ in range(3):
            rc = execute_real_moe_layer_ptr(lid, hin.data_ptr(), nfl, hout.data_ptr())
            _lib.check(rc, "execute_real_moe_layer")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            rc = execute_real_moe_layer_ptr(lid, hin.data_ptr(), nfl, hout.data_ptr())
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / args.steps
        _lib.check(rc, "execute_real_moe_layer")
        assert torch.isfinite(hout).all()
        e2e = {"value": T / dt, "unit": UNIT, "h2d_bytes_per_step": nfl * 4, "d2h_bytes_per_step": nfl * 4,
               "ms_per_step": dt * 1e3, "api": "atenia_execute_real_moe_layer (host f32 in/out, pinned)"}

    # ---- CPU baseline on a bounded sample (N = 1 only)
    cpu = None
    if args.gpus == 1 and not args.no_cpu_baseline:
        xs = x[: min(T, 512)].float().cpu().numpy()
        from oracle import oracle as orc
        cores = host_threads()
        rate, cores, n, ol = cpu_oracle_rate(shape, w, xs, args.cpu_seconds * 0.6, threads=cores)
        rate32, _, n32, _ = cpu_oracle_rate(shape, w, xs, args.cpu_seconds * 0.4, threads=cores, accum=orc.ACC_F32, ol=ol)
        cpu = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{n} of the step's {T} tokens, CPU oracle (C restatement of the reference's per-token "
                         f"f64 path), {cores} OpenMP threads",
               "f32_accumulate": {"value": rate32, "unit": UNIT,
                                  "sample": f"{n32} tokens, the same oracle accumulating in f32 (the reference's "
                                            "strict mode)"}}

    value = T * args.gpus / (ms * 1e-3)
    if args.gpus > 1:
        # whole-forward target of the rank with the most rows: the slower of its expert flops at the
        # measured GEMM rate and the bytes it must move over NVLink (rows it receives from the other
        # ranks, there and back) at the measured peer-copy rate of this pool
        G = args.gpus
        rows = [r[0] for r in per_rank]
        flops = rows_slow * 6.0 * shape.d_model * shape.d_ff + T * 6.0 * shape.d_model * shape.shared_d_ff
        t_compute = flops / (peaks["bf16_tflops"] * 1e12)
        link_bytes = rows_slow * (G - 1) / G * shape.d_model * 2
        nvlink_gbs = 770.0
        t_link = link_bytes / (nvlink_gbs * 1e9)
        target = max(t_compute, t_link)
        roofline["expert_parallel"] = {
            "rows_received_per_rank": rows, "rows_max": max(rows), "rows_mean": sum(rows) / len(rows),
            "imbalance_max_over_mean": max(rows) / max(sum(rows) / len(rows), 1.0),
            "efficiency_bound_from_imbalance": (sum(rows) / len(rows)) / max(rows),
            "slowest_rank": slow, "t_compute_ms": t_compute * 1e3, "t_nvlink_ms": t_link * 1e3,
            "nvlink_bytes_in_per_phase": link_bytes, "nvlink_gbs_per_direction": nvlink_gbs,
            "target_ms": target * 1e3, "frac": target / (ms * 1e-3),
            "note": "every rank routes its own tokens; the rank that owns the most popular experts sets the step"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype_name, "data": "synthetic", "config": config,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "gpu_launches": launches,
            "tensor_core_launches_per_step": 2 + (2 if shape.shared_d_ff else 0),
            "windows": windows, "records": records or None, "parity": parity}
    print(json.dumps(line))
    grp.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
