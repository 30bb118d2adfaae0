#!/usr/bin/env python
"""Benchmark of the fused causal attention path (forward + backward) on B200.

  python bench.py --gpus N --steps K --warmup W            # this library's CUDA path
  python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU attention, timed on host cores

A step is one forward + backward pass of the attention op over one batch of synthetic input
in the GPT-2-small layer configuration (B=8, H=12, S=1024, D=64, causal, fp32 API / TF32 MMA).
FLOPs per step = 2.5 x (2*B*H*S^2*D), the causal accounting of the headline metric.

One JSON line is printed by rank 0.  value     = device-timed throughput, inputs resident in HBM
                                      e2e       = same metric through the C ABI from pinned host buffers,
                                                  host<->device copies inside the timed region
                                      roofline  = dominant kernel against the tensor-core peak
                                      cpu_baseline = the CPU oracle timed on this box's host cores
With N > 1 (torchrun) every rank runs its own batch of the same size: the path shards by
batch x heads with no communication, so the scaling reported is weak.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=8, H=12, S=1024, D=64)
# DRAM bytes (read + write) of one launch of each kernel of the step at exactly the benchmark size, from one ncu
# capture; TRAFFIC_CAPTURE names the build the capture was taken from
TRAFFIC = {"fwd": 91.9e6, "dq": 148.3e6, "dkdv": 125.7e6}
TRAFFIC_CAPTURE = "ncu --set full of bench.py --kernel-case fwd / bwd --batch 8 --seq 1024, backward kernels as of commit 875fe8b, forward as of 4239d77 (unchanged since)"
METRIC = "causal_attention_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def fwd_flops(B, H, S, D):
    return 2.0 * B * H * S * S * D  # causal accounting: 2*B*H*S^2*D


def raw_step_calls(pkg, s, B, H, S, D, scale, stream):
    """[(C function, argument tuple)] of one forward + backward on the tensors of `s` (q, k, v, go, out, lse, delta, dq,
    dk, dv; contiguous, on the GPU), for loops that must not time the host."""
    L = pkg.lib()
    st = stream.cuda_stream
    P = lambda name: s[name].data_ptr()
    for name in ("q", "k", "v", "go", "out", "lse", "delta", "dq", "dk", "dv"):
        assert s[name].is_cuda and s[name].is_contiguous(), name
    fwd = (P("q"), P("k"), P("v"), P("out"), P("lse"), B, H, S, D, float(scale), 1, st)
    bwd = (P("q"), P("k"), P("v"), P("out"), P("go"), P("lse"), P("dq"), P("dk"), P("dv"), P("delta"), B, H, S, D, float(scale), 1, st)
    return [(L.df_attn_forward, fwd), (L.df_attn_backward, bwd)]


def step_flops(B, H, S, D):
    return 2.5 * fwd_flops(B, H, S, D)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(int(r[1]) for r in self.rows if len(r) >= 9 and r[1].isdigit())
        mx = [int(r[2]) for r in self.rows if len(r) >= 9 and r[2].isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# reference arm: the reference's CPU attention (oracle port), all host threads, bounded sample
# ----------------------------------------------------------------------------------------------
class QuietStdout:
    """Routes everything written to file descriptor 1 (Python prints and native libraries alike: NCCL announces its
    version there) to stderr while the benchmark runs, so that stdout carries the one JSON line and nothing else."""

    def __init__(self):
        sys.stdout.flush()
        self.real = os.dup(1)
        os.dup2(2, 1)

    def emit(self, text):
        sys.stdout.flush()
        os.write(self.real, (text + "\n").encode())


def host_threads():
    """Host threads this process may use: its CPU affinity mask (torchrun exports OMP_NUM_THREADS=1, which
    says nothing about the cores that are there)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample(orc, n_seq, steps, warmup, threads=None):
    """Times fwd+bwd of `n_seq` sequences of the benchmark configuration on the host cores; returns
    (TFLOP/s, seconds per run, threads used)."""
    import numpy as np
    H, S, D = CFG["H"], CFG["S"], CFG["D"]
    threads = threads or host_threads()
    orc.set_threads(threads)
    q, k, v, go = (orc.fill_normal((n_seq, S, H * D), 0xDF02, st) for st in range(4))
    scale = 1.0 / math.sqrt(D)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        orc.forward(q, k, v, H, scale, True)
        orc.backward(q, k, v, go, H, scale, True)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = float(np.mean(times))
    return step_flops(n_seq, H, S, D) / sec / 1e12, sec, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle.attn_oracle import Oracle
    orc = Oracle()
    n_seq = 1  # bounded sample: one sequence of the B=8 batch per step
    tflops, sec, cores = cpu_sample(orc, n_seq, args.steps, args.warmup)
    sample = f"fwd+bwd of {n_seq} of {CFG['B']} sequences per step (H=12,S=1024,D=64), fp32, {cores} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "GPT-2-small layer attention fwd+bwd, B=8,H=12,S=1024,D=64, causal", "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's CPU attention is Rust and cannot be built here; this is its C restatement (oracle/)",
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# this library's arm
# ----------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    quiet = QuietStdout()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = load_package()
    pkg.lib()  # raises if the CUDA library is missing: no fallback

    B, H, S, D = CFG["B"], CFG["H"], CFG["S"], CFG["D"]
    scale = 1.0 / math.sqrt(D)
    n = B * S * H * D
    gen = torch.Generator(device=dev)
    gen.manual_seed(0xDF02 + rank)
    # rotating input sets so that consecutive steps never re-read the same bytes from L2:
    # one set = 8 tensors x 24 MiB = 192 MiB, four sets = 768 MiB > 126 MB L2
    n_sets = 4
    sets = []
    for _ in range(n_sets):
        q, k, v, go = (torch.randn((B, S, H * D), device=dev, generator=gen) for _ in range(4))
        sets.append(dict(q=q, k=k, v=v, go=go, out=torch.empty_like(q), lse=torch.empty((B, H, S), device=dev),
                         delta=torch.empty((B, H, S), device=dev), dq=torch.empty_like(q), dk=torch.empty_like(q),
                         dv=torch.empty_like(q)))
    stream = torch.cuda.current_stream()

    # The timed loop calls the two C entry points with argument tuples prepared once per input set: the Python wrappers
    # (tensor checks, keyword handling) take about as long on the host as the 0.17 ms step takes on the GPU, and with
    # eight ranks sharing the host's cores the loop then measured the host (0.21 ms per step at N = 8).
    step_calls = {id(s_): raw_step_calls(pkg, s_, B, H, S, D, scale, stream) for s_ in sets}

    def step(s):
        for fn, a in step_calls[id(s)]:
            st = fn(*a)
            if st != 0:
                raise RuntimeError(f"attention call failed with status {st}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-timed region ----------------
    for w in range(args.warmup):
        step(sets[w % n_sets])
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    pkg.launch_count(reset=True)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record(stream)
    for it in range(args.steps):
        step(sets[it % n_sets])
    ev1.record(stream)
    barrier()
    launches = pkg.launch_count()
    ms_total = ev0.elapsed_time(ev1)
    status = pkg.sync_status()
    if status != 0:
        raise RuntimeError(f"device status {status}")
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = world * step_flops(B, H, S, D) / (ms_step * 1e-3) / 1e12

    # ---------------- end to end: pinned host buffers in, results out, through the C ABI ----------------
    host_in = [torch.randn((B, S, H * D), generator=torch.Generator().manual_seed(7 + i)).pin_memory() for i in range(4)]
    host_out = [[torch.empty((B, S, H * D)).pin_memory() for _ in range(4)] for _ in range(2)]

    # The batch is fed in chunks of sequences over three streams (upload, compute, download) so that the
    # PCIe uplink, the kernels and the PCIe downlink of consecutive chunks overlap; every chunk is an
    # ordinary call of the public entry points on its slice of the caller-owned device buffers. Consecutive
    # steps alternate between two sets of device and pinned host buffers, so that the upload of one step
    # runs under the download of the step before it; every step still moves all of its inputs up and all of
    # its results (O, dQ, dK, dV) down inside the timed region.
    n_chunks = args.e2e_chunks if B % args.e2e_chunks == 0 else 4
    cb = B // n_chunks
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_up = [[torch.cuda.Event() for _ in range(n_chunks)] for _ in range(2)]
    ev_done = [[torch.cuda.Event() for _ in range(n_chunks)] for _ in range(2)]
    ev_computed = [torch.cuda.Event() for _ in range(2)]   # the step's kernels have read the inputs of the set
    ev_drained = [torch.cuda.Event() for _ in range(2)]    # the step's results have left the set
    used = [False, False]
    e2e_count = [0]

    def e2e_step():
        w = e2e_count[0] % 2
        e2e_count[0] += 1
        sd, ho = sets[w], host_out[w]
        if used[w]:
            up.wait_event(ev_computed[w])      # the set's previous inputs are no longer needed
            stream.wait_event(ev_drained[w])   # the set's previous results are on the host
        else:
            ev_free = torch.cuda.Event()
            ev_free.record(stream)             # earlier work on these buffers is ordered before the first upload
            up.wait_event(ev_free)
        for c in range(n_chunks):
            sl = slice(c * cb, (c + 1) * cb)
            with torch.cuda.stream(up):
                for name, src in zip(("q", "k", "v", "go"), host_in):
                    sd[name][sl].copy_(src[sl], non_blocking=True)
                ev_up[w][c].record(up)
            stream.wait_event(ev_up[w][c])
            pkg.forward(sd["q"][sl], sd["k"][sl], sd["v"][sl], H, scale, True, out=sd["out"][sl], lse=sd["lse"][sl],
                        stream=stream)
            pkg.backward(sd["q"][sl], sd["k"][sl], sd["v"][sl], sd["out"][sl], sd["go"][sl], sd["lse"][sl], H, scale, True,
                         d_q=sd["dq"][sl], d_k=sd["dk"][sl], d_v=sd["dv"][sl], delta_buf=sd["delta"][sl], stream=stream)
            ev_done[w][c].record(stream)
            down.wait_event(ev_done[w][c])
            with torch.cuda.stream(down):
                for name, dst in zip(("out", "dq", "dk", "dv"), ho):
                    dst[sl].copy_(sd[name][sl], non_blocking=True)
        ev_computed[w].record(stream)
        ev_drained[w].record(down)
        used[w] = True

    def e2e_finish():
        stream.wait_stream(down)          # the run ends when its last result byte is on the host

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    e2e_finish()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_finish()
    e1.record(stream)
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / e2e_steps
    e2e_value = world * step_flops(B, H, S, D) / (e2e_ms * 1e-3) / 1e12

    # The floor of that number: the same bytes moved both ways at once over the same two streams with no kernel
    # in between (all ranks at the same time, as above).
    def copies_only():
        with torch.cuda.stream(up):
            for name, src in zip(("q", "k", "v", "go"), host_in):
                sets[0][name].copy_(src, non_blocking=True)
        with torch.cuda.stream(down):
            for name, dst in zip(("out", "dq", "dk", "dv"), host_out[1]):
                dst.copy_(sets[1][name], non_blocking=True)
    up.wait_stream(stream)
    down.wait_stream(stream)
    copies_only()
    stream.wait_stream(up)
    stream.wait_stream(down)
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record(stream)
    up.wait_event(c0)
    down.wait_event(c0)
    for _ in range(5):
        copies_only()
    stream.wait_stream(up)
    stream.wait_stream(down)
    c1.record(stream)
    barrier()
    tc = torch.tensor([c0.elapsed_time(c1)], device=dev)
    if world > 1:
        dist.all_reduce(tc, op=dist.ReduceOp.MAX)
    copy_only_ms = float(tc.item()) / 5
    clocks = sampler.stop() if rank == 0 else None

    def run_extras():
        """The path's multi-GPU workloads at this N (all ranks take part). They run after rank 0's single-GPU
        measurements: the ring keeps a GPU at its power cap for seconds, and kernels timed right after it read low."""
        extras = {}
        if args.no_extras:
            return extras
        import importlib
        _init_dist(torch, dist, world, dev)
        ring = importlib.import_module("dark_forest_b200.ring")
        for key, fn in (("strong", lambda: strong_measure(pkg, torch, dist, world, rank, dev, max(5, min(args.steps, 20)), 3)),
                        ("long_forward", lambda: long_forward_measure(pkg, torch, dist, world, rank, dev, 131072, 2, 1)),
                        ("ring", lambda: ring_measure(pkg, ring, torch, dist, world, rank, dev, 65536 * world, True, "balanced",
                                                      2, 1)),
                        ("ring_zigzag_rows", lambda: ring_measure(pkg, ring, torch, dist, world, rank, dev, 65536 * world, True,
                                                                  "zigzag", 2, 1))):
            try:
                extras[key] = fn()
            except torch.cuda.OutOfMemoryError as exc:  # a shared GPU short of memory: report, keep the headline
                extras[key] = {"error": str(exc)[:120]}
            torch.cuda.empty_cache()
        return extras

    if rank != 0:
        run_extras()  # waits in its first collective until rank 0 has finished its single-GPU measurements
        if dist.is_initialized():
            dist.destroy_process_group()
        return

    # ---------------- per-kernel timing for the roofline (rank 0, same stream, CUDA events) ----------------
    def time_call(fn, iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(3):
            fn(sets[i % n_sets])
        torch.cuda.synchronize()
        a.record(stream)
        for i in range(iters):
            fn(sets[i % n_sets])
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters

    ms_fwd = time_call(lambda s: pkg.forward(s["q"], s["k"], s["v"], H, scale, True, out=s["out"], lse=s["lse"],
                                             stream=stream), 20)
    ms_delta = time_call(lambda s: pkg.delta(s["out"], s["go"], H, delta_buf=s["delta"], stream=stream), 20)
    ms_bwd = time_call(lambda s: pkg.backward(s["q"], s["k"], s["v"], s["out"], s["go"], s["lse"], H, scale, True,
                                              d_q=s["dq"], d_k=s["dk"], d_v=s["dv"], delta_buf=s["delta"],
                                              stream=stream), 20)
    # per-kernel times of the backward: the profiling entry point launches each of its two kernels four times back
    # to back between events and returns the time per launch (the dQ kernel of a whole-sequence backward also
    # computes the delta row sums). An event pair around every single launch read 10-12 % more than the kernels take
    # inside a step. Each profiled backward is queued behind the forward of the same input set, as in a timed
    # step, and the input sets rotate from call to call. (Taken here, before the cuBLAS and long-sequence measurements:
    # those leave the GPU at its power cap for a while, and 70-microsecond kernels timed right after them read long.)
    dq_t, dkdv_t = [], []
    for i in range(3 + 20):
        sx = sets[i % n_sets]
        pkg.forward(sx["q"], sx["k"], sx["v"], H, scale, True, out=sx["out"], lse=sx["lse"], stream=stream)
        _, _, _, a_ms, b_ms = pkg.backward_profile(sx["q"], sx["k"], sx["v"], sx["out"], sx["go"], sx["lse"], H, scale, True,
                                                   d_q=sx["dq"], d_k=sx["dk"], d_v=sx["dv"], delta_buf=sx["delta"],
                                                   stream=stream)
        if i >= 3:
            dq_t.append(a_ms)
            dkdv_t.append(b_ms)
    ms_dq, ms_dkdv = sum(dq_t) / len(dq_t), sum(dkdv_t) / len(dkdv_t)

    s0 = sets[0]
    uses_tensor = bool(pkg.lib().df_attn_forward_uses_tensor_cores(s0["q"].data_ptr(), s0["k"].data_ptr(),
                                                                     s0["v"].data_ptr(), s0["out"].data_ptr(), H, S, S, D))

    # TF32 dense peak is not in MEASURED_PEAKS.json: cuBLAS TF32 is measured here with that file's protocol
    peaks, peak_kind = measured_peaks()
    # (the burst figure now; the 4 s sustained loop runs at the very end, after everything else has been timed: it
    # leaves the GPU power-capped for a while, and a forward sweep timed right after it read 25 % low)
    tf32 = measure_tf32_peaks(torch, dev, local, sustained=False)
    tf32["half_of_measured_bf16_burst"] = 0.5 * peaks["bf16_tflops"]
    tf32["half_of_measured_bf16_sustained"] = 0.5 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    tf32_peak = tf32["cublas_tf32_burst"]

    def fracs(tflops):
        """The same achieved figure against the TF32 denominators on record (the sustained one is added at the end)."""
        return {"tflops": tflops, "of_cublas_tf32_burst": tflops / tf32["cublas_tf32_burst"],
                "of_half_measured_bf16_burst": tflops / tf32["half_of_measured_bf16_burst"]}

    # long-sequence forward sweep (B=1, H=12, D=64), the configuration of the reference's bench_sequence_limit
    sweep = []
    for S_long, iters in ((8192, 10), (32768, 3), (131072, 2)):
        try:
            ql, kl, vl = (torch.randn((1, S_long, H * D), device=dev, generator=gen) for _ in range(3))
            ol = torch.empty_like(ql)
            ll = torch.empty((1, H, S_long), device=dev)
            f = lambda _s: pkg.forward(ql, kl, vl, H, scale, True, out=ol, lse=ll, stream=stream)
            x, y = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f(None)
            torch.cuda.synchronize()
            x.record(stream)
            for _ in range(iters):
                f(None)
            y.record(stream)
            torch.cuda.synchronize()
            ms = x.elapsed_time(y) / iters
            tf = fwd_flops(1, H, S_long, D) / (ms * 1e-3) / 1e12
            sweep.append({"S": S_long, "fwd_ms": ms, "fwd_tflops": tf, "frac_of_tf32_peak": tf / tf32_peak,
                          "fracs": fracs(tf)})
            del ql, kl, vl, ol, ll
        except Exception as exc:  # out of memory on a shared GPU: report, do not fail the bench
            sweep.append({"S": S_long, "error": str(exc)[:80]})

    # Roofline of the dominant kernel of the step, k_attn_bwd_dkdv_tf32_d64: four of the seven GEMM units of the
    # backward (S^T, dP^T, dV, dK), i.e. 4 * (2*D*S^2/2) = 2 x the forward's FLOPs per (batch, head).
    # traffic: dram__bytes_read.sum + dram__bytes_write.sum of one launch at exactly this size, literals from the
    # ncu capture named in TRAFFIC_CAPTURE (they do not follow later kernel changes by themselves).
    fwd_tf = fwd_flops(B, H, S, D) / (ms_fwd * 1e-3) / 1e12
    dkdv_tf = 2.0 * fwd_flops(B, H, S, D) / (ms_dkdv * 1e-3) / 1e12
    dq_tf = 1.5 * fwd_flops(B, H, S, D) / (ms_dq * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "k_attn_bwd_dkdv_tf32_d64" if uses_tensor else "k_generic_bwd_dkdv",
                "achieved": dkdv_tf, "peak": tf32_peak, "unit": "TFLOP/s", "frac": dkdv_tf / tf32_peak,
                "fracs": fracs(dkdv_tf), "peaks": tf32,
                "traffic": TRAFFIC["dkdv"] if uses_tensor else None, "traffic_capture": TRAFFIC_CAPTURE,
                "algorithmic_bytes": 6.0 * n * 4 + 2.0 * B * H * S * 4,  # Q,K,V,dO in, dK,dV out, lse+delta
                "peak_source": "cuBLAS TF32 8192^3 burst (best of 10) measured in this run; 4 s sustained figure and half of "
                               f"MEASURED_PEAKS.json's bf16 burst ({peaks.get('bf16_tflops')} TFLOP/s {peak_kind}) in `peaks`",
                "ms_per_launch": ms_dkdv,
                "other_kernels": {"k_attn_fwd_persist_tf32_d64": {"ms": ms_fwd, "tflops": fwd_tf, "frac": fwd_tf / tf32_peak,
                                                                 "fracs": fracs(fwd_tf), "traffic": TRAFFIC["fwd"]},
                                  "k_attn_bwd_dq_tf32_d64": {"ms": ms_dq, "tflops": dq_tf, "frac": dq_tf / tf32_peak,
                                                             "fracs": fracs(dq_tf), "traffic": TRAFFIC["dq"],
                                                             "note": "also computes the delta row sums"}}}
    delta_bytes = 2.0 * n * 4 + B * H * S * 4
    delta_gbs = delta_bytes / (ms_delta * 1e-3) / 1e9

    # one-token decode over a 32K-token cache (the adjacent HBM-bound path of the same API object)
    try:
        decode_line = decode_case(pkg, torch, dev, H, 32768, D, 3)
        decode_line["frac_of_hbm_peak"] = decode_line["splitk_gbs"] / peaks["hbm_gbs"]
    except Exception as exc:  # a shared GPU short of memory: report, do not fail the bench
        decode_line = {"error": str(exc)[:80]}

    # the projections on either side of the attention op (the next step of the same layer), at the full-step shape
    try:
        projection = linear_case(pkg, torch, dev, 8 * 4096, 768, 3)
        projection["frac_of_cublas_tf32_burst"] = projection["ours_tflops"] / tf32_peak
    except Exception as exc:
        projection = {"error": str(exc)[:120]}

    # the attention calls of the full static step (12 layers, S = 4096, one sequence: the reference's engine has no batch
    # dimension), made as its engine makes them, against this library and against the reference's own kernels
    static_step = static_step_case()
    try:
        loss_head = loss_ce_case(pkg, torch, dev, 512, 50257, 2)
    except Exception as exc:
        loss_head = {"error": str(exc)[:120]}

    try:
        step_kernels = step_kernels_case(pkg, torch, dev, 8 * 4096, 768, 2)
    except Exception as exc:
        step_kernels = {"error": str(exc)[:120]}
    torch.cuda.empty_cache()

    try:
        reference_gpu = reference_gpu_case(pkg, torch, dev, stream)
    except Exception as exc:
        reference_gpu = {"error": str(exc)[:120]}

    # ---------------- CPU baseline on a bounded sample (rank 0 only) ----------------
    from oracle.attn_oracle import Oracle
    orc = Oracle()
    cpu_tf, cpu_sec, cpu_threads = cpu_sample(orc, 1, 3, 1)
    cpu_baseline = {"value": cpu_tf, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                    "sample": f"fwd+bwd of 1 of {B} sequences (H=12,S=1024,D=64), 3 timed runs, {cpu_sec:.2f} s each"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "tf32 (fp32 API, TF32 tensor-core MMA, fp32 accumulate)" if uses_tensor else "f32", "data": "synthetic",
        "config": {"workload": "GPT-2-small layer attention fwd+bwd: B=8,H=12,S=1024,D=64, causal, N(0,1) seeded",
                   "parallelism": f"batch x heads sharded, B=8 per GPU, {world} GPU(s), no collective",
                   "l2": "4 rotating input sets of 192 MiB (> 126 MB L2)", "flops_per_step": step_flops(B, H, S, D)},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * n * 4, "d2h_bytes_per_step": 4 * n * 4,
                "ms_per_step": e2e_ms, "copies_only_ms_per_step": copy_only_ms,
                "copies_only_note": "the step's 100 MB up and 100 MB down moved at the same time with no kernel between them: the floor of ms_per_step on this host",
                "pipeline": f"{n_chunks} chunks of {cb} sequences over upload/compute/download streams, two buffer sets alternating between steps"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "kernels": {"fwd_ms": ms_fwd, "fwd_tflops": fwd_tf, "delta_ms": ms_delta, "delta_gbs": delta_gbs,
                    "delta_frac_of_hbm": delta_gbs / peaks["hbm_gbs"], "bwd_ms_incl_delta": ms_bwd, "dkdv_ms": ms_dkdv, "dq_ms": ms_dq,
                    "fwd_bwd_tflops_conventional_3.5x": 3.5 * fwd_flops(B, H, S, D) / ((ms_fwd + ms_bwd) * 1e-3) / 1e12},
        "long_sequence_forward": sweep,
        "decode": decode_line,
        "reference_gpu": reference_gpu,
        "projection": projection,
        "loss_head": loss_head,
        "step_kernels": step_kernels,
        "static_step_attention": static_step,
    }
    for sset in sets:
        sset.clear()
    del host_in, host_out
    torch.cuda.empty_cache()
    line.update(run_extras())
    # last of all: the sustained cuBLAS TF32 figure, and every fraction against it
    sus = measure_tf32_peaks(torch, dev, local, sustained=True)
    tf32.update({k: v for k, v in sus.items() if k != "cublas_tf32_burst"})
    tf32["cublas_tf32_burst_second_measurement"] = sus["cublas_tf32_burst"]

    def add_sustained(node):
        if isinstance(node, dict):
            if "of_cublas_tf32_burst" in node and "tflops" in node:
                node["of_cublas_tf32_sustained"] = node["tflops"] / tf32["cublas_tf32_sustained"]
            for v in node.values():
                add_sustained(v)
        elif isinstance(node, list):
            for v in node:
                add_sustained(v)

    add_sustained(line)
    quiet.emit(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


def measure_tf32_peaks(torch, dev, gpu_index, sustained=True):
    """cuBLAS TF32 8192^3 GEMM on this GPU: burst (best of 10 after 2 warm-ups) and, when asked, sustained (back to
    back for 4 s, with the SM clock sampled meanwhile) - the protocol MEASURED_PEAKS.json uses for bf16."""
    torch.backends.cuda.matmul.allow_tf32 = True
    a = torch.randn((8192, 8192), device=dev)
    b = torch.randn((8192, 8192), device=dev)
    c = torch.empty((8192, 8192), device=dev)
    flop = 2.0 * 8192 ** 3
    best = 1e9
    for i in range(12):
        x, y = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        x.record()
        torch.matmul(a, b, out=c)
        y.record()
        torch.cuda.synchronize()
        if i >= 2:
            best = min(best, x.elapsed_time(y))
    if not sustained:
        del a, b, c
        return {"cublas_tf32_burst": flop / (best * 1e-3) / 1e12}
    sampler = ClockSampler(gpu_index)
    sampler.start()
    x, y = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    n = 0
    x.record()
    while time.perf_counter() - t0 < 4.0:
        for _ in range(20):
            torch.matmul(a, b, out=c)
        n += 20
        torch.cuda.synchronize()
    y.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    sustained = n * flop / (x.elapsed_time(y) * 1e-3) / 1e12
    del a, b, c
    return {"cublas_tf32_burst": flop / (best * 1e-3) / 1e12, "cublas_tf32_sustained": sustained,
            "sustained_sm_mhz": clocks.get("sm_mhz"), "sustained_reasons": clocks.get("reasons")}


def reference_gpu_case(pkg, torch, dev, stream):
    """The kernel to beat: the reference's own CUDA attention, compiled unmodified for sm_100a (oracle/_ref, the
    checker's library - it is timed here, never called by the product path), beside this library on the same
    inputs. Forward at S = 8192 (B=1, H=12, D=64; one timed launch after one warm-up, the protocol of the
    reference's bench_sequence_limit) and forward + backward on one sequence of the benchmark batch (S = 1024;
    the reference's backward needs its H*2*S*S-float scratch)."""
    from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
    if not os.path.exists(REFERENCE_SO):
        return {"unavailable": "oracle/_ref was not built (reference source tree absent at build time)"}
    ref = ReferenceKernels()
    H, D = CFG["H"], CFG["D"]
    scale = 1.0 / math.sqrt(D)
    g = torch.Generator(device=dev)
    g.manual_seed(0xBEA7)
    res = {}

    def timed(fn):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3

    def ours_ms(fn, iters=5):
        fn()
        x, y = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        x.record(stream)
        for _ in range(iters):
            fn()
        y.record(stream)
        torch.cuda.synchronize()
        return x.elapsed_time(y) / iters

    S = 8192
    q, k, v = (torch.randn((S, H * D), device=dev, generator=g) for _ in range(3))
    ref.mha_forward(q, k, v, H, scale, True)  # warm-up
    ms_ref = timed(lambda: ref.mha_forward(q, k, v, H, scale, True))
    q3, k3, v3 = (x[None] for x in (q, k, v))
    o3, l3 = torch.empty_like(q3), torch.empty((1, H, S), device=dev)
    ms_our = ours_ms(lambda: pkg.forward(q3, k3, v3, H, scale, True, out=o3, lse=l3, stream=stream))
    o_ref = ref.mha_forward(q, k, v, H, scale, True)
    res["forward_S8192"] = {"reference_ms": ms_ref, "ours_ms": ms_our, "speedup": ms_ref / ms_our,
                            "reference_tflops": fwd_flops(1, H, S, D) / (ms_ref * 1e-3) / 1e12,
                            "ours_tflops": fwd_flops(1, H, S, D) / (ms_our * 1e-3) / 1e12,
                            "max_abs_diff_o": float((o3[0] - o_ref).abs().max())}
    del q, k, v, q3, k3, v3, o3, l3, o_ref
    S = CFG["S"]
    q, k, v, go = (torch.randn((S, H * D), device=dev, generator=g) for _ in range(4))

    def ref_step():
        ref.mha_forward(q, k, v, H, scale, True)
        return ref.mha_backward(q, k, v, go, H, scale, True)

    ref_step()
    ms_ref = timed(ref_step)
    q3, k3, v3, g3 = (x[None] for x in (q, k, v, go))
    o3, l3, d3 = torch.empty_like(q3), torch.empty((1, H, S), device=dev), torch.empty((1, H, S), device=dev)
    grads = [torch.empty_like(q3) for _ in range(3)]

    def our_step():
        pkg.forward(q3, k3, v3, H, scale, True, out=o3, lse=l3, stream=stream)
        pkg.backward(q3, k3, v3, o3, g3, l3, H, scale, True, d_q=grads[0], d_k=grads[1], d_v=grads[2], delta_buf=d3,
                     stream=stream)

    ms_our = ours_ms(our_step, 20)
    rq, rk, rv = ref_step()
    rel = max(float((a[0] - b).abs().max() / max(float(b.abs().max()), 0.25)) for a, b in zip(grads, (rq, rk, rv)))
    res["fwd_bwd_one_sequence_S1024"] = {"reference_ms": ms_ref, "ours_ms": ms_our, "speedup": ms_ref / ms_our,
                                         "max_rel_diff_grad": rel,
                                         "note": "reference timed by host clock around launch + synchronize (it launches "
                                                 "on the legacy stream and memsets two gradients per call)"}
    return res


def loss_ce_case(pkg, torch, dev, rows, cols, iters):
    """The loss head's fused softmax + cross-entropy on one chunk of logits ([512, 50257] in the static step), HBM-bound:
    algorithmic bytes = 1 read + 2 writes of the chunk (training form), 1 read (eval form); eight chunks rotate so that
    every launch reads from DRAM. Beside it the reference's own kernel (oracle/_ref) on the same data."""
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    n_sets = 8
    zs = [torch.randn((rows, cols), device=dev, generator=g) * 3.0 for _ in range(n_sets)]
    grad = torch.empty((rows, cols), device=dev)
    tg = torch.randint(0, cols, (rows,), device=dev, generator=g, dtype=torch.int32)
    loss = torch.zeros(1, device=dev)
    chunk_bytes = rows * cols * 4.0

    def timed(fn):
        for i in range(n_sets):
            fn(zs[i])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters * n_sets):
            fn(zs[i % n_sets])
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (iters * n_sets)

    variants = {}
    for name, v in (("resident_row", 1), ("second_pass_from_l2", 2)):
        prev = pkg.set_option(pkg.OPT_CE_VARIANT, v)
        variants[name + "_ms"] = timed(lambda z: pkg.chunked_logit_ce(z, tg, loss, rows, grad_logits=grad))
        pkg.set_option(pkg.OPT_CE_VARIANT, prev)
    ms_train = timed(lambda z: pkg.chunked_logit_ce(z, tg, loss, rows, grad_logits=grad))
    ms_eval = timed(lambda z: pkg.chunked_logit_ce(z, tg, loss, rows))
    assert pkg.sync_status() == 0
    peaks, _ = measured_peaks()
    res = {"kernel_case": "loss_ce", "rows": rows, "cols": cols, "train_ms": ms_train, "train_gbs": 3 * chunk_bytes / (ms_train * 1e-3) / 1e9,
           "train_frac_of_hbm": 3 * chunk_bytes / (ms_train * 1e-3) / 1e9 / peaks["hbm_gbs"], "eval_ms": ms_eval,
           "eval_gbs": chunk_bytes / (ms_eval * 1e-3) / 1e9, "eval_frac_of_hbm": chunk_bytes / (ms_eval * 1e-3) / 1e9 / peaks["hbm_gbs"],
           "algorithmic_bytes_train": 3 * chunk_bytes, "variants": variants}
    try:
        from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
        if os.path.exists(REFERENCE_SO):
            ref = ReferenceKernels()
            if ref.has_ce:
                def ref_call(z):
                    ref.lib.launch_fused_chunked_logit_ce(z.data_ptr(), tg.data_ptr(), grad.data_ptr(), loss.data_ptr(), rows, cols, rows)
                torch.cuda.synchronize()
                ms_ref = timed(ref_call)
                res["reference_train_ms"] = ms_ref
                res["speedup_vs_reference_kernel"] = ms_ref / ms_train
    except Exception as exc:
        res["reference_error"] = str(exc)[:100]
    return res


def step_kernels_case(pkg, torch, dev, rows=32768, d_model=768, iters=3):
    """LayerNorm, GELU and AdamW of the training step at the static step's shapes (32768 rows = 8 x 4096 tokens, d_model
    768, MLP width 3072; AdamW over the tensors of GPT-2 small), all HBM-bound. Algorithmic bytes: LayerNorm forward 1
    read + 1 write of [rows, d_model], backward 2 reads + 1 write; GELU forward 1 + 1, backward 2 + 1 of [rows, 4 d_model];
    AdamW 4 reads + 3 writes per parameter. Input sets rotate so that every launch reads from DRAM. Beside each the
    reference's own kernel (oracle/_ref) on the same data; the reference's AdamW is one launch per tensor."""
    g = torch.Generator(device=dev)
    g.manual_seed(6)
    peaks, _ = measured_peaks()

    def timed(fn, n_sets, reps):
        for i in range(n_sets):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(reps * n_sets):
            fn(i % n_sets)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * n_sets)

    ref = None
    try:
        from oracle.attn_oracle import REFERENCE_SO, ReferenceKernels
        if os.path.exists(REFERENCE_SO):
            r = ReferenceKernels()
            ref = r if r.has_step else None
    except Exception:
        ref = None

    def entry(ms, nbytes, ms_ref=None):
        e = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
             "algorithmic_bytes": nbytes}
        if ms_ref is not None:
            e["reference_ms"] = ms_ref
            e["speedup_vs_reference_kernel"] = ms_ref / ms
        return e

    res = {"kernel_case": "step_kernels", "rows": rows, "d_model": d_model}
    # ---- LayerNorm: [rows, d_model] = 100 MB; four input sets
    n_sets = 4
    xs = [torch.randn((rows, d_model), device=dev, generator=g) for _ in range(n_sets)]
    gos = [torch.randn((rows, d_model), device=dev, generator=g) for _ in range(n_sets)]
    gamma, beta = torch.randn(d_model, device=dev, generator=g), torch.randn(d_model, device=dev, generator=g)
    out = torch.empty((rows, d_model), device=dev)
    means, rstds = torch.empty(rows, device=dev), torch.empty(rows, device=dev)
    gg, gb = torch.zeros(d_model, device=dev), torch.zeros(d_model, device=dev)
    act = rows * d_model * 4.0
    # (the timed loops call the C entry points with ready-made pointers: the Python wrappers' argument checks take longer
    # than a 30-microsecond kernel runs, and the loop would time the host)
    L = pkg.lib()
    P = lambda t: t.data_ptr()
    ms = timed(lambda i: L.df_layernorm_forward(P(xs[i]), P(gamma), P(beta), P(out), P(means), P(rstds), rows, d_model, None), n_sets, iters)
    ms_ref = timed(lambda i: ref.lib.launch_layernorm(xs[i].data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                                       means.data_ptr(), rstds.data_ptr(), rows, d_model), n_sets, iters) if ref else None
    res["layernorm_forward"] = entry(ms, 2 * act, ms_ref)
    pkg.layernorm(xs[0], gamma, beta, out=out, means=means, rstds=rstds)
    ms = timed(lambda i: L.df_layernorm_backward(P(gos[i]), P(xs[0]), P(gamma), P(means), P(rstds), P(out), P(gg), P(gb), rows, d_model,
                                                 None), n_sets, iters)
    ms_ref = timed(lambda i: ref.lib.launch_layernorm_backward(gos[i].data_ptr(), xs[0].data_ptr(), gamma.data_ptr(), means.data_ptr(),
                                                                rstds.data_ptr(), out.data_ptr(), gg.data_ptr(), gb.data_ptr(), rows,
                                                                d_model), n_sets, iters) if ref else None
    res["layernorm_backward"] = entry(ms, 3 * act, ms_ref)
    del xs, gos
    # ---- GELU: [rows, 4 d_model] = 403 MB; two input sets
    n = rows * 4 * d_model
    hs = [torch.randn(n, device=dev, generator=g) for _ in range(2)]
    ds = [torch.randn(n, device=dev, generator=g) for _ in range(2)]
    y = torch.empty(n, device=dev)
    ms = timed(lambda i: L.df_gelu_forward(P(hs[i]), P(y), n, None), 2, iters)
    ms_ref = timed(lambda i: ref.lib.launch_gelu(hs[i].data_ptr(), y.data_ptr(), n), 2, iters) if ref else None
    res["gelu_forward"] = entry(ms, 2 * n * 4.0, ms_ref)
    ms = timed(lambda i: L.df_gelu_backward(P(ds[i]), P(hs[i]), P(y), n, None), 2, iters)
    ms_ref = timed(lambda i: ref.lib.launch_gelu_backward(ds[i].data_ptr(), hs[i].data_ptr(), y.data_ptr(), n), 2, iters) if ref else None
    res["gelu_backward"] = entry(ms, 3 * n * 4.0, ms_ref)
    del hs, ds, y
    # ---- AdamW over the parameter tensors of GPT-2 small (12 layers, d_model 768, vocabulary 50257, 1024 positions):
    # 196 tensors, 124 M parameters, 3.5 GB of traffic per step
    d, v, pos, layers = d_model, 50257, 1024, 12
    shapes = [v * d, pos * d, d, d]
    for _ in range(layers):
        shapes += [d, d, d * d, d, d * d, d, d * d, d, d * d, d, d, d, 4 * d * d, 4 * d, 4 * d * d, d]
    tensors = [tuple(torch.randn(sz, device=dev, generator=g) * sc for sc in (1.0, 0.1, 0.01, 1.0)) for sz in shapes]
    for t in tensors:
        t[2].abs_()
    hyper = (3e-4, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** 10, 1 - 0.999 ** 10)
    total = float(sum(shapes))
    plan = pkg.AdamwPlan(tensors)
    ms = timed(lambda i: plan.step(*hyper), 1, max(3, iters))

    ptrs = [tuple(P(a) for a in t) for t in tensors]

    def per_tensor(i):
        for (pp, mm, vv, gg_), sz in zip(ptrs, shapes):
            L.df_adamw_update(pp, mm, vv, gg_, sz, *hyper, None)
    ms_each = timed(per_tensor, 1, max(3, iters))

    def ref_per_tensor(i):
        for (pp, mm, vv, gg_), sz in zip(ptrs, shapes):
            ref.lib.launch_adamw_update(pp, mm, vv, gg_, sz, *hyper)
    ms_ref = timed(ref_per_tensor, 1, max(3, iters)) if ref else None
    res["adamw_all_parameters"] = entry(ms, 7 * total * 4.0, ms_ref)
    res["adamw_all_parameters"].update({"tensors": len(shapes), "parameters": int(total), "launches": 1,
                                        "one_launch_per_tensor_ms": ms_each})
    assert pkg.sync_status() == 0
    return res


def static_step_case(layers=12, seq=4096):
    """Runs dark-forest_b200/lib/static_step (C++: pre-allocated per-layer buffers, legacy symbols, one sync per step)
    for this library and, when oracle/_ref exists, for the reference's own kernels; returns its JSON."""
    lib_dir = os.path.join(ROOT, "dark-forest_b200", "lib")
    exe = os.path.join(lib_dir, "static_step")
    if not os.path.exists(exe):
        return {"unavailable": "static_step was not built"}
    cmd = [exe, "--ours", os.path.join(lib_dir, "libdarkforest_kernels.so"), "--layers", str(layers), "--seq", str(seq), "--steps", "3"]
    ref = os.path.join(ROOT, "oracle", "_ref", "libdf_reference_kernels.so")
    if os.path.exists(ref):
        cmd += ["--ref", ref]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
        return json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 else {"error": (r.stdout + r.stderr)[-200:]}
    except Exception as exc:
        return {"error": str(exc)[:120]}


def linear_case(pkg, torch, dev, rows, d_model, iters):
    """The Q/K/V projection of one layer (three GEMMs + three bias passes in the reference) as one launch of this
    library, beside torch/cuBLAS doing the reference's sequence (three matmuls, three bias adds) in TF32 and in the
    reference's own full-fp32 arithmetic (cublasSgemm). Four input sets rotate (activations > L2 at 32768 rows)."""
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    n_sets = 4
    xs = [torch.randn((rows, d_model), device=dev, generator=g) for _ in range(n_sets)]
    ws = [torch.randn((d_model, d_model), device=dev, generator=g) * 0.02 for _ in range(3)]
    bs = [torch.randn((d_model,), device=dev, generator=g) * 0.02 for _ in range(3)]
    outs = [torch.empty((rows, d_model), device=dev) for _ in range(3)]
    flop = 3 * 2.0 * rows * d_model * d_model

    def timed(fn):
        for i in range(3):
            fn(xs[i % n_sets])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters * n_sets):
            fn(xs[i % n_sets])
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (iters * n_sets)

    ms_ours = timed(lambda x: pkg.linear_qkv(x, *ws, *bs, q=outs[0], k=outs[1], v=outs[2]))
    assert pkg.sync_status() == 0
    ours = [o.clone() for o in outs]

    def torch_seq(x):
        for w, b, o in zip(ws, bs, outs):
            torch.matmul(x, w.t(), out=o)
            o.add_(b)

    torch.backends.cuda.matmul.allow_tf32 = True
    ms_tf32 = timed(torch_seq)
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_fp32 = timed(torch_seq)
    torch_seq(xs[(iters * n_sets - 1) % n_sets])
    err = max(float((a - b).abs().max()) for a, b in zip(ours, outs))
    torch.backends.cuda.matmul.allow_tf32 = True
    # the MLP's first projection [rows, d] x [d, 4d] with GELU: one launch (pre-activation and activation written by the
    # epilogue) against this library's projection followed by its GELU kernel, and against cuBLAS TF32 + bias + torch GELU
    mlp = {}
    try:
        w1 = torch.randn((4 * d_model, d_model), device=dev, generator=g) * 0.02
        b1 = torch.randn((4 * d_model,), device=dev, generator=g) * 0.02
        pre, act = torch.empty((rows, 4 * d_model), device=dev), torch.empty((rows, 4 * d_model), device=dev)
        mlp["fused_ms"] = timed(lambda x: pkg.linear_gelu(x, w1, b1, pre_activation=pre, out=act))
        fused_act = act.clone()
        mlp["separate_ms"] = timed(lambda x: (pkg.linear(x, w1, b1, out=pre), pkg.gelu(pre, out=act)))
        mlp["same_bits_as_separate"] = bool(torch.equal(fused_act, act))

        def torch_mlp(x):
            torch.matmul(x, w1.t(), out=pre)
            pre.add_(b1)
            torch.nn.functional.gelu(pre, approximate="tanh")
        mlp["cublas_tf32_bias_gelu_ms"] = timed(torch_mlp)
        mlp["flop"] = 2.0 * rows * d_model * 4 * d_model
        mlp["fused_tflops"] = mlp["flop"] / (mlp["fused_ms"] * 1e-3) / 1e12
        assert pkg.sync_status() == 0
    except Exception as exc:
        mlp["error"] = str(exc)[:120]
    return {"kernel_case": "linear_qkv", "rows": rows, "d_model": d_model, "flop": flop, "ours_ms": ms_ours, "mlp_up_gelu": mlp,
            "ours_tflops": flop / (ms_ours * 1e-3) / 1e12, "cublas_tf32_3gemm_3bias_ms": ms_tf32,
            "cublas_tf32_tflops": flop / (ms_tf32 * 1e-3) / 1e12, "cublas_fp32_3gemm_3bias_ms": ms_fp32,
            "speedup_vs_reference_arithmetic": ms_fp32 / ms_ours, "speedup_vs_cublas_tf32": ms_tf32 / ms_ours,
            "max_abs_diff_vs_cublas_fp32": err,
            "algorithmic_bytes": 4.0 * rows * d_model * 4 + 3 * d_model * d_model * 4}


def decode_case(pkg, torch, dev, H, T, D, iters):
    """One-token decode over a contiguous fp32 KV cache of T tokens (HBM-bound: K and V are read once): the
    scratch-free form (clusters of 8 CTAs per head) and the split form with caller scratch for chunk_size 256.
    Eight caches are rotated so that every launch reads from DRAM (8 x 2 x T x H x D x 4 bytes > L2 for T >= 4096)."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(2)
    n_sets = 8
    q = torch.randn((H * D,), device=dev, generator=gen)
    caches = [(torch.randn((T, H * D), device=dev, generator=gen), torch.randn((T, H * D), device=dev, generator=gen))
              for _ in range(n_sets)]
    out = torch.empty_like(q)
    chunks = (T + 255) // 256
    parts = (torch.empty(H * chunks, device=dev), torch.empty(H * chunks, device=dev), torch.empty(H * chunks * D, device=dev))
    scale = 1.0 / math.sqrt(D)
    res = {"kernel_case": "decode", "H": H, "T": T, "D": D, "bytes_per_launch": 2.0 * T * H * D * 4}
    for name, kw in (("cluster", {}), ("splitk", {"partials": parts, "max_chunks": chunks})):
        for i in range(n_sets):
            pkg.decode(q, caches[i][0], caches[i][1], H, T, scale, out=out, **kw)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters * n_sets):
            pkg.decode(q, caches[i % n_sets][0], caches[i % n_sets][1], H, T, scale, out=out, **kw)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / (iters * n_sets)
        res[name + "_ms"] = ms
        res[name + "_gbs"] = res["bytes_per_launch"] / (ms * 1e-3) / 1e9
    assert pkg.sync_status() == 0
    return res


def run_kernel_case(args):
    """One kernel of the path on a small case, a few launches: the command that ncu captures."""
    import torch
    from __graft_entry__ import load_package
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    pkg = load_package()
    B, H, S, D = args.batch, args.heads or CFG["H"], args.seq, args.dhead
    scale = 1.0 / math.sqrt(D)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)
    if args.kernel_case == "decode":
        print(json.dumps(decode_case(pkg, torch, dev, H, S, D, args.iters)))
        return
    if args.kernel_case == "loss_ce":
        print(json.dumps(loss_ce_case(pkg, torch, dev, args.seq if args.seq != 16384 else 512, 50257, args.iters)))
        return
    if args.kernel_case == "linear_qkv":
        print(json.dumps(linear_case(pkg, torch, dev, B * S, H * D, args.iters)))
        return
    if args.kernel_case == "step_kernels":
        print(json.dumps(step_kernels_case(pkg, torch, dev, B * S, H * D, args.iters)))
        return
    q, k, v, go = (torch.randn((B, S, H * D), device=dev, generator=gen) for _ in range(4))
    if args.kernel_case == "fwd_bf16":
        qb, kb, vb = (x.to(torch.bfloat16) for x in (q, k, v))
        ob, lb = pkg.forward_bf16(qb, kb, vb, H, scale, True)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            pkg.forward_bf16(qb, kb, vb, H, scale, True, out=ob, lse=lb)
        b.record()
        torch.cuda.synchronize()
        assert pkg.sync_status() == 0
        print(json.dumps({"kernel_case": args.kernel_case, "B": B, "H": H, "S": S, "D": D, "ms": a.elapsed_time(b) / args.iters,
                          "fwd_flops": fwd_flops(B, H, S, D)}))
        return
    out, lse = pkg.forward(q, k, v, H, scale, True)
    delta = torch.empty((B, H, S), device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iters):
        if args.kernel_case == "fwd":
            pkg.forward(q, k, v, H, scale, True, out=out, lse=lse)
        elif args.kernel_case == "delta":
            pkg.delta(out, go, H, delta_buf=delta)
        else:
            pkg.backward(q, k, v, out, go, lse, H, scale, True, d_q=dq, d_k=dk, d_v=dv, delta_buf=delta)
    b.record()
    torch.cuda.synchronize()
    assert pkg.sync_status() == 0
    ms = a.elapsed_time(b) / args.iters
    print(json.dumps({"kernel_case": args.kernel_case, "B": B, "H": H, "S": S, "D": D, "ms": ms,
                      "fwd_flops": fwd_flops(B, H, S, D)}))


# ----------------------------------------------------------------------------------------------
# checker for sequences too long for the CPU oracle: float64 attention on sampled rows (torch, on the GPU's
# float64 units; none of this touches the library under test)
# ----------------------------------------------------------------------------------------------
def _rel(got, ref):
    """max|got - ref| / max(max|ref|, 0.25), the gradient error measure of the parity tests."""
    return float((got.double() - ref).abs().max() / max(float(ref.abs().max()), 0.25))


def sampled_rows_check(torch, full, H, scale, rows_g, out_rows, lse_rows, grads=None, chunk=32768):
    """full = (Q, K, V, dO) [S, H*D] of the WHOLE sequence in the library's input dtype; rows_g: global row indices
    (LongTensor on the device). Compares the library's rows of O and lse - and, with grads = (dQ rows, dK rows, dV rows,
    lse_all [H, S], delta_all [H, S]), of the three gradients - with float64 causal attention. dK/dV of a key row need
    the row statistics of every later query: those come from the library's own lse and delta = rowsum(dO o O), which
    the O / lse rows checked here vouch for. Returns a dict of error figures."""
    Q, K, V, G = full
    S, dm = K.shape
    D = dm // H
    n = rows_g.numel()
    dev = K.device
    ar = torch.arange(S, device=dev)
    f64 = lambda t: t.double().view(-1, H, D).transpose(0, 1)  # [H, rows, D]
    qg, gg = f64(Q[rows_g]), f64(G[rows_g])
    s = torch.empty((H, n, S), dtype=torch.float64, device=dev)
    dp = torch.empty((H, n, S), dtype=torch.float64, device=dev)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        s[:, :, c0:c1] = torch.einsum("hid,hjd->hij", qg, f64(K[c0:c1])) * scale
        dp[:, :, c0:c1] = torch.einsum("hid,hjd->hij", gg, f64(V[c0:c1]))
    s.masked_fill_(ar[None, None, :] > rows_g[None, :, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                      # [H, n]
    p = torch.exp(s - lse[..., None])
    o = torch.zeros((H, n, D), dtype=torch.float64, device=dev)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        o += torch.einsum("hij,hjd->hid", p[:, :, c0:c1], f64(V[c0:c1]))
    back = lambda t: t.transpose(0, 1).reshape(n, dm)
    res = {"rows": int(n), "max_abs_err_o": float((out_rows.double() - back(o)).abs().max()),
           "max_abs_err_lse": float((lse_rows.double() - lse).abs().max())}
    if grads is None:
        return res
    dq_rows, dk_rows, dv_rows, lse_all, delta_all = grads
    dlt = (o * gg).sum(-1)                                # [H, n]
    ds = p * (dp - dlt[..., None])
    dq = torch.zeros((H, n, D), dtype=torch.float64, device=dev)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        dq += scale * torch.einsum("hij,hjd->hid", ds[:, :, c0:c1], f64(K[c0:c1]))
    del s, dp, p, ds
    # the sampled rows as KEYS against every query
    kg, vg = f64(K[rows_g]), f64(V[rows_g])
    dk = torch.zeros((H, n, D), dtype=torch.float64, device=dev)
    dv = torch.zeros((H, n, D), dtype=torch.float64, device=dev)
    for c0 in range(0, S, chunk):
        c1 = min(S, c0 + chunk)
        qc, gc = f64(Q[c0:c1]), f64(G[c0:c1])
        st = torch.einsum("hid,hjd->hij", qc, kg) * scale   # [H, queries, n]
        st.masked_fill_(rows_g[None, None, :] > ar[None, c0:c1, None], float("-inf"))
        pt = torch.exp(st - lse_all[:, c0:c1, None].double())
        dpt = torch.einsum("hid,hjd->hij", gc, vg)
        dst = pt * (dpt - delta_all[:, c0:c1, None].double())
        dv += torch.einsum("hij,hid->hjd", pt, gc)
        dk += scale * torch.einsum("hij,hid->hjd", dst, qc)
    res["max_rel_err_grad"] = max(_rel(dq_rows, back(dq)), _rel(dk_rows, back(dk)), _rel(dv_rows, back(dv)))
    return res


def _allmax(dist, world, res):
    if world > 1:
        got = [None] * world
        dist.all_gather_object(got, res)
        res = {k: (max(g[k] for g in got) if k != "rows" else sum(g[k] for g in got)) for k in res}
    return res


# ----------------------------------------------------------------------------------------------
# multi-GPU workloads (also run inside the default benchmark under torchrun)
# ----------------------------------------------------------------------------------------------
def ring_measure(pkg, ring, torch, dist, world, rank, dev, S, bf16, layout, steps, warmup, heads=None, n_check=24,
                 oracle_check=False, impl="c"):
    """Sequence-parallel ring attention fwd+bwd over all ranks: B=1, the sequence of S rows split over the ranks, K/V
    blocks and dK/dV accumulators exchanged by NCCL send/recv. impl "c": the hop loop of libdarkforest_ring behind the
    C ABI (df_ring_forward / df_ring_backward); "python": the torch.distributed driver of dark-forest_b200/ring.py over
    the block entry points. layout "balanced": every rank holds CONTIGUOUS rows and the re-layout into the balanced
    zigzag order and back is inside the timed call; "zigzag": the caller already holds zigzag rows; "contiguous": plain.
    Every rank draws the WHOLE Q, K, V, dO from one seed (so any row can be checked anywhere) and hands its own rows to
    the ring. Timed with CUDA events per rank, max over ranks. Afterwards sampled rows of O, lse, dQ, dK, dV of every
    rank are compared with float64 attention over the whole sequence."""
    import importlib
    H, D = heads or (16 if bf16 else 12), (128 if bf16 else 64)
    scale = 1.0 / math.sqrt(D)
    if S % (2 * world):
        raise SystemExit("the ring sequence length must be a multiple of 2 * world size")
    L = S // world
    dt = torch.bfloat16 if bf16 else torch.float32
    g = torch.Generator(device=dev)
    g.manual_seed(0xDF05)
    full = []
    for _ in range(4):
        x = torch.randn((S, H * D), device=dev, generator=g)
        full.append(x.to(dt) if bf16 else x)
        del x
    if layout == "zigzag":
        c = S // (2 * world)
        mine = torch.cat([torch.arange(a * c, (a + 1) * c, device=dev) for a in (rank, 2 * world - 1 - rank)])
    else:
        mine = torch.arange(rank * L, (rank + 1) * L, device=dev)
    tq, tk, tv, tg = (x[mine][None].contiguous() for x in full)
    out, lse = torch.empty_like(tq), torch.empty((1, H, L), device=dev)
    dq, dk, dv = (torch.empty_like(tq) for _ in range(3))
    if impl == "c":
        rc = importlib.import_module("dark_forest_b200.ring_c")
        uid = [rc.unique_id() if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(uid, src=0)
        ra = rc.Ring(uid[0], rank, world, layout, H, L, D, bf16, scale, True, timeout_ms=120000, device=dev)
        run_fwd = lambda: ra.forward(tq, tk, tv, out, lse)
        run_bwd = lambda: ra.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
    else:
        if layout == "balanced":
            raise SystemExit("the balanced layout exists in the C ring only")
        backend = ring.CudaBackendBf16(pkg, H, scale) if bf16 else ring.CudaBackend(pkg, H, scale)
        ra = ring.RingAttention(backend, L, H, D, dev, causal=True, layout=layout)
        run_fwd = lambda: ra.forward(tq, tk, tv, out, lse)
        run_bwd = lambda: ra.backward(tq, tk, tv, out, tg, lse, dq, dk, dv)
    fwd_ms, bwd_ms = [], []
    for it in range(warmup + steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        run_fwd()
        e1.record()
        run_bwd()
        e2.record()
        if impl == "c" and ra.wait(timeout_ms=120000) != 0:
            raise RuntimeError("ring wait failed")
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if it >= warmup:
            fwd_ms.append(float(t[0]))
            bwd_ms.append(float(t[1]))
    assert pkg.sync_status() == 0
    f, bw = sum(fwd_ms) / len(fwd_ms), sum(bwd_ms) / len(bwd_ms)
    res = {"workload": f"ring attention fwd+bwd, B=1,H={H},S={S},D={D}, {'bf16' if bf16 else 'fp32/TF32'}, {layout} rows, "
                       f"{world} GPU(s), NCCL send/recv, " + ("C ABI (df_ring_*)" if impl == "c" else "python driver"),
           "n_gpus": world, "fwd_ms": f, "bwd_ms": bw, "fwd_tflops": fwd_flops(1, H, S, D) / (f * 1e-3) / 1e12,
           "fwd_bwd_tflops_2.5x": 2.5 * fwd_flops(1, H, S, D) / ((f + bw) * 1e-3) / 1e12}
    # ---- sampled rows against float64 (every rank checks rows it owns)
    if impl == "c":
        ra.close()
    del ra
    lse_all = torch.empty((H, S), device=dev)
    delta_all = torch.empty((H, S), device=dev)
    my_delta = (out[0].float() * tg[0].float()).view(L, H, D).sum(-1).t().contiguous()   # [H, L]
    if world > 1:
        gl = [torch.empty((H, L), device=dev) for _ in range(world)]
        gd = [torch.empty((H, L), device=dev) for _ in range(world)]
        gi = [torch.empty((L,), dtype=torch.long, device=dev) for _ in range(world)]
        dist.all_gather(gl, lse[0].contiguous())
        dist.all_gather(gd, my_delta)
        dist.all_gather(gi, mine)
        for l_, d_, i_ in zip(gl, gd, gi):
            lse_all[:, i_] = l_
            delta_all[:, i_] = d_
    else:
        lse_all[:, mine] = lse[0]
        delta_all[:, mine] = my_delta
    rs = torch.Generator(device="cpu")
    rs.manual_seed(1234 + rank)
    loc = torch.unique(torch.cat([torch.tensor([0, 1, L // 2 - 1, L // 2, L - 2, L - 1]),
                                  torch.randint(0, L, (max(1, n_check - 6),), generator=rs)])).to(dev)
    chk = sampled_rows_check(torch, full, H, scale, mine[loc], out[0, loc], lse[0][:, loc],
                             grads=(dq[0, loc], dk[0, loc], dv[0, loc], lse_all, delta_all))
    chk = _allmax(dist, world, chk)
    tol_o, tol_g = (2e-2, 2e-2) if bf16 else (2e-3, 5e-3)
    chk["tolerance_o"], chk["tolerance_grad_rel"] = tol_o, tol_g
    chk["pass"] = bool(chk["max_abs_err_o"] <= tol_o and chk["max_rel_err_grad"] <= tol_g)
    res["check"] = chk
    res["max_abs_err_o"], res["max_rel_err_grad"] = chk["max_abs_err_o"], chk["max_rel_err_grad"]
    if oracle_check and S <= 2048 and not bf16:
        from oracle.attn_oracle import Oracle
        import numpy as np
        orc = Oracle()
        orc.set_threads(max(1, host_threads() // world))
        q, k, v, go = (x.float().cpu().numpy()[None] for x in full)
        o_ref, _ = orc.forward(q, k, v, H, scale, True)
        g_ref = orc.backward(q, k, v, go, H, scale, True)
        idx = mine.cpu().numpy()
        e = {"oracle_max_abs_err_o": float(np.abs(out.float().cpu().numpy() - o_ref[:, idx]).max()),
             "oracle_max_rel_err_grad": max(float(np.abs(a.float().cpu().numpy() - r[:, idx]).max() / max(np.abs(r).max(), 0.25))
                                            for a, r in zip((dq, dk, dv), g_ref))}
        res.update(_allmax(dist, world, e))
    # ---- one GPU running a whole sequence with the same kernels: the efficiency denominator
    S1 = min(S, 65536 if bf16 else 32768)
    q1, k1, v1, g1 = (x[:S1][None].contiguous() for x in full)
    o1, l1, d1 = torch.empty_like(q1), torch.empty((1, H, S1), device=dev), torch.empty((1, H, S1), device=dev)
    gr = [torch.empty_like(q1) for _ in range(3)]

    def one():
        if bf16:
            pkg.forward_bf16(q1, k1, v1, H, scale, True, out=o1, lse=l1)
            pkg.backward_bf16(q1, k1, v1, o1, g1, l1, H, scale, True, d_q=gr[0], d_k=gr[1], d_v=gr[2], delta_buf=d1)
        else:
            pkg.forward(q1, k1, v1, H, scale, True, out=o1, lse=l1)
            pkg.backward(q1, k1, v1, o1, g1, l1, H, scale, True, d_q=gr[0], d_k=gr[1], d_v=gr[2], delta_buf=d1)

    one()
    torch.cuda.synchronize()
    x, y = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x.record()
    for _ in range(2):
        one()
    y.record()
    torch.cuda.synchronize()
    t1 = torch.tensor([x.elapsed_time(y) / 2], device=dev)
    if world > 1:
        dist.all_reduce(t1, op=dist.ReduceOp.MAX)
    one_tf = 2.5 * fwd_flops(1, H, S1, D) / (float(t1) * 1e-3) / 1e12
    res["one_gpu_whole_sequence"] = {"S": S1, "fwd_bwd_ms": float(t1), "fwd_bwd_tflops_2.5x": one_tf}
    res["efficiency_vs_n_times_one_gpu"] = res["fwd_bwd_tflops_2.5x"] / (world * one_tf)
    return res


def long_forward_measure(pkg, torch, dist, world, rank, dev, S, steps, warmup, heads=None, n_check=24):
    """Long-context forward in isolation (B=1, H=12, D=64, fp32 API) over all ranks without any exchange: the heads do
    not divide by 8, so the unit is (head, query block). Every rank holds the whole K and V (drawn in place from the
    global seed) and owns two query chunks, r and 2W-1-r of 2W, which gives every rank the same causal work; each
    chunk is one df_attn_forward_block call with the causal shift of its first row."""
    H, D = heads or 12, 64
    scale = 1.0 / math.sqrt(D)
    if S % (2 * world):
        raise SystemExit("--seq must be a multiple of 2 * world size")
    c = S // (2 * world)
    chunks = [rank, 2 * world - 1 - rank]
    g = torch.Generator(device=dev)
    g.manual_seed(0xDF03)  # the same tensors on every rank
    tq_full, tk, tv = (torch.randn((1, S, H * D), device=dev, generator=g) for _ in range(3))
    tqs = [tq_full[:, a * c:(a + 1) * c].contiguous() for a in chunks]
    outs = [torch.empty_like(x) for x in tqs]
    lses = [torch.empty((1, H, c), device=dev) for _ in chunks]

    def step():
        for a, tq, o, l in zip(chunks, tqs, outs, lses):
            kv = (a + 1) * c
            pkg.forward(tq, tk[:, :kv], tv[:, :kv], H, scale, True, out=o, lse=l, causal_shift=a * c)

    times = []
    for it in range(warmup + steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if it >= warmup:
            times.append(float(t[0]))
    assert pkg.sync_status() == 0
    ms = sum(times) / len(times)
    res = {"workload": f"long-context forward, B=1,H={H},S={S},D={D}, fp32/TF32, (head, query block) units over {world} "
                       "GPU(s), no exchange",
           "n_gpus": world, "fwd_ms": ms, "fwd_tflops": fwd_flops(1, H, S, D) / (ms * 1e-3) / 1e12}
    rs = torch.Generator(device="cpu")
    rs.manual_seed(77 + rank)
    loc = torch.unique(torch.cat([torch.tensor([0, c - 1]), torch.randint(0, c, (max(1, n_check // 2 - 2),), generator=rs)])).to(dev)
    worst = None
    full = (tq_full[0], tk[0], tv[0], tq_full[0])
    for a, o, l in zip(chunks, outs, lses):
        chk = sampled_rows_check(torch, full, H, scale, loc + a * c, o[0, loc], l[0][:, loc])
        worst = chk if worst is None else {k: (max(worst[k], chk[k]) if k != "rows" else worst[k] + chk[k]) for k in chk}
    worst = _allmax(dist, world, worst)
    worst["tolerance_o"] = 2e-3
    worst["pass"] = bool(worst["max_abs_err_o"] <= 2e-3 and worst["max_abs_err_lse"] <= 2e-3)
    res["check"] = worst
    res["max_abs_err_o"], res["max_abs_err_lse"] = worst["max_abs_err_o"], worst["max_abs_err_lse"]
    return res


def strong_measure(pkg, torch, dist, world, rank, dev, steps, warmup):
    """Strong scaling of the benchmark configuration: ONE B=8 problem (96 (batch, head) units) split over the ranks by
    sequences, no exchange; T_N = max over ranks of the device time of the local share, beside T_1 = the whole problem
    on one GPU timed in the same process. efficiency = T_1 / (N * T_N)."""
    B, H, S, D = CFG["B"], CFG["H"], CFG["S"], CFG["D"]
    if B % world:
        return {"skipped": f"B={B} sequences do not divide over {world} ranks"}
    scale = 1.0 / math.sqrt(D)
    g = torch.Generator(device=dev)
    g.manual_seed(0xDF02)
    n_sets = 4
    sets = []
    for _ in range(n_sets):
        q, k, v, go = (torch.randn((B, S, H * D), device=dev, generator=g) for _ in range(4))
        sets.append(dict(q=q, k=k, v=v, go=go, out=torch.empty_like(q), lse=torch.empty((B, H, S), device=dev),
                         delta=torch.empty((B, H, S), device=dev), dq=torch.empty_like(q), dk=torch.empty_like(q),
                         dv=torch.empty_like(q)))
    bl = B // world
    sl = slice(rank * bl, (rank + 1) * bl)

    calls = {}

    def step(s_, sel):
        key = (id(s_), sel.start, sel.stop)
        if key not in calls:  # argument tuples prepared once: the loop times the GPU, not the Python wrappers
            view = {name: t[sel] for name, t in s_.items()}
            calls[key] = raw_step_calls(pkg, view, sel.stop - sel.start, H, S, D, scale, torch.cuda.current_stream())
        for fn, a in calls[key]:
            st = fn(*a)
            if st != 0:
                raise RuntimeError(f"attention call failed with status {st}")

    def timed(sel):
        for w in range(max(3, warmup)):
            step(sets[w % n_sets], sel)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for it in range(steps):
            step(sets[it % n_sets], sel)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    tn = timed(sl)
    t1 = timed(slice(0, B))
    assert pkg.sync_status() == 0
    return {"workload": f"B=8,H=12,S=1024,D=64 fwd+bwd, one problem, {bl} sequence(s) = {bl * H} (batch, head) units per GPU, "
                        f"{world} GPU(s), no exchange",
            "n_gpus": world, "ms_per_step": tn, "tflops_2.5x": step_flops(B, H, S, D) / (tn * 1e-3) / 1e12,
            "one_gpu_ms_per_step_same_process": t1, "efficiency_t1_over_n_tn": t1 / (world * tn)}


def _init_dist(torch, dist, world, dev):
    if world > 1:
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    elif not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("gloo", rank=0, world_size=1)


def run_ring(args):
    """--workload ring: see ring_measure. --ring-dtype bf16 is the bf16 D=128 ring configuration (bf16 operands, fp32
    partial results); the default is fp32 API / TF32 MMA with D=64. Prints one JSON line on rank 0."""
    import importlib
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    quiet = QuietStdout()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _init_dist(torch, dist, world, dev)
    pkg = load_package()
    ring = importlib.import_module("dark_forest_b200.ring")
    res = ring_measure(pkg, ring, torch, dist, world, rank, dev, args.seq, args.ring_dtype == "bf16", args.ring_layout,
                       args.steps, args.warmup, heads=args.heads, oracle_check=True, impl=args.ring_impl)
    if rank == 0:
        quiet.emit(json.dumps(res))
    dist.destroy_process_group()


def run_long_forward(args):
    """--workload long_forward: see long_forward_measure. Prints one JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    quiet = QuietStdout()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _init_dist(torch, dist, world, dev)
    pkg = load_package()
    res = long_forward_measure(pkg, torch, dist, world, rank, dev, args.seq, args.steps, args.warmup, heads=args.heads)
    if rank == 0:
        quiet.emit(json.dumps(res))
    dist.destroy_process_group()


def run_gpt2_step(args):
    """Full static GPT-2 training step (12 layers, d_model 768, 12 heads, d_ff 3072, vocab 50257, S=4096, B=8)
    with this library's attention plugged in; reports the attention's share of the step."""
    import importlib
    import torch
    from __graft_entry__ import load_package
    torch.cuda.set_device(0)
    pkg = load_package()
    step = importlib.import_module("dark_forest_b200.gpt2_step")
    res = step.run(pkg, batch=args.batch if args.batch > 1 else 8, seq=args.seq if args.seq != 16384 else 4096,
                   steps=max(1, min(args.steps, 5)), warmup=1)
    assert pkg.sync_status() == 0
    # the same step with torch's LayerNorm, GELU and fused AdamW in place of this library's
    torch.cuda.empty_cache()
    other = step.run(pkg, batch=res["batch"], seq=res["seq"], steps=max(1, min(args.steps, 5)), warmup=1, step_kernels=False)
    res["step_ms_with_torch_layernorm_gelu_adamw"] = other["step_ms"]
    res["loss_first_step_with_torch_layernorm_gelu_adamw"] = other["loss_first_step"]
    H, D = 12, 64
    res["attention_fwd_tflops"] = 12 * fwd_flops(res["batch"], H, res["seq"], D) / (res["attention_fwd_ms"] * 1e-3) / 1e12
    res["workload"] = ("full GPT-2-small training step, fp32 + TF32 GEMMs (torch) + this library's attention, projections, "
                       "LayerNorm, GELU and multi-tensor AdamW")
    print(json.dumps(res))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="attention", choices=["attention", "gpt2_step", "ring", "long_forward"],
                    help="gpt2_step: the full-training-step configuration (attention time share); not the headline metric")
    ap.add_argument("--kernel-case", default=None, choices=["fwd", "bwd", "delta", "fwd_bf16", "decode", "linear_qkv", "loss_ce", "step_kernels"],
                    help="run one kernel of the path a few times on a small case (for ncu) and exit")
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--ring-layout", default="balanced", choices=["balanced", "zigzag", "contiguous"])
    ap.add_argument("--ring-impl", default="c", choices=["c", "python"],
                    help="c: the hop loop behind the C ABI (libdarkforest_ring); python: dark-forest_b200/ring.py")
    ap.add_argument("--ring-dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--heads", type=int, default=None, help="default 12 (16 for the bf16 ring)")
    ap.add_argument("--dhead", type=int, default=CFG["D"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-chunks", type=int, default=4, help="chunks of sequences the end-to-end step is fed in (a divisor of 8)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the strong-scaling, long-context-forward and ring workloads that follow the headline measurement")
    args = ap.parse_args()
    if args.workload == "gpt2_step":
        run_gpt2_step(args)
    elif args.workload == "ring":
        run_ring(args)
    elif args.workload == "long_forward":
        run_long_forward(args)
    elif args.kernel_case:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
