#!/usr/bin/env python
"""Benchmark of the W4A16 group-128 batch-1 decode projection sweep on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one pass of the 28-layer Qwen2.5-1.5B-shaped projection sweep (QKV, O, gate_up +
SwiGLU, down, each with its Q8_1 quantiser in front), run as one CUDA graph through the C ABI
(w4a16_sweep_*).  Weights are seeded synthetic tensors with the benchmark configuration's
distributions; the 675 MB of packed weights streamed per step exceed L2, so every step reads
them from HBM.  Prints ONE JSON line (rank 0).

The oracle (oracle/) is used here only for the cpu_baseline leg / the reference arm and for
a one-layer sanity check of the result.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "W4A16 G128 batch-1 decode projection sweep, achieved HBM bandwidth"
UNIT = "GB/s"
WORKLOAD = ("config 1: 28-layer Qwen2.5-1.5B projection sweep (QKV 1536->2048, O 1536->1536 +res, "
            "gate_up 1536->17920 +SwiGLU, down 8960->1536 +res), W4A16 G128, batch 1, Q8_1 before each GEMV")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--suite", default="sweep", choices=["sweep", "shapes", "single"],
                    help="sweep: the headline line; shapes: per-shape GEMV and M-token GEMM table (configs 0, 3, 4); "
                         "single: a few launches of one kernel (for ncu captures)")
    ap.add_argument("--shape", default="gate_up", help="single: qkv | o | gate_up | down | lm_head | big")
    ap.add_argument("--m", type=int, default=0, help="single: 0 = batch-1 GEMV, else M tokens through the GEMM")
    ap.add_argument("--input", default="q8", choices=["q8", "fp16", "fp16norm"],
                    help="single, batch-1: pre-quantised Q8_1 input, fp16 input, or fp16 input with RMSNorm in the prologue")
    ap.add_argument("--no-shapes", action="store_true", help="skip the per-shape table (configs 0, 3, 4) in the headline line")
    ap.add_argument("--gemv-form", type=int, default=0, choices=[0, 1, 2],
                    help="W4A16_OPT_GEMV_FORM for the run: 0 default, 1 register-held weight loads, 2 bulk copies into shared memory")
    ap.add_argument("--sweep-flags", type=int, default=-1, help="W4A16_SWEEP_* flags of the decode sweep (default: the library's)")
    ap.add_argument("--no-lm-head", action="store_true", help="skip the lm_head / token selection extras (1 GPU only)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 8192 -> 28672 prefill extra")
    ap.add_argument("--m-list", default="1,2,4,8,16,32,64,128,512,1024,4096")
    ap.add_argument("--layers", type=int, default=28, help=argparse.SUPPRESS)
    ap.add_argument("--no-cpu-baseline", action="store_true", help=argparse.SUPPRESS)
    return ap.parse_args()


# ---- synthetic model -----------------------------------------------------------------

def make_layers_np(num_layers: int, seed: int = 0x5EED0001):
    from qwen_engine_b200 import synth
    layers = []
    for l in range(num_layers):
        L = {}
        for name in ("q", "k", "v", "o", "gate_up", "down"):
            N, K = synth.SHAPES[name]
            L[name] = (synth.packed_weights(seed, f"L{l}.{name}", N, K), synth.scales(seed, f"L{l}.{name}", N, K))
        # small norm gains keep the residual stream finite in fp16 over 28 random-weight layers
        L["input_norm"] = np.full(synth.HIDDEN, 0.05, dtype=np.float16)
        L["post_norm"] = np.full(synth.HIDDEN, 0.05, dtype=np.float16)
        layers.append(L)
    return layers


def upload_layers(layers_np):
    import torch
    out = []
    for L in layers_np:
        D = {}
        for k, v in L.items():
            if isinstance(v, tuple):
                D[k] = (torch.from_numpy(v[0].view(np.int32)).cuda(), torch.from_numpy(v[1]).cuda())
            else:
                D[k] = torch.from_numpy(v).cuda()
        out.append(D)
    return out


# ---- clocks ---------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.01, pci_bus_id: str | None = None):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                self.h = pynvml.nvmlDeviceGetHandleByPciBusId(pci_bus_id.encode()) if pci_bus_id else None
            except Exception:
                self.h = None
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self._thr = threading.Thread(target=self._run, args=(period_s,), daemon=True)
        except Exception:
            self.nv = None

    def _run(self, period):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(period)

    def start(self):
        if self._thr:
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=1.0)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU baseline (oracle port) ----------------------------------------------------------

def time_cpu_sweep(layers_np, h0, budget_s: float = 12.0, max_reps: int = 150):
    """Times the oracle's sweep on the host cores.  Returns (GB/s, cores, sample description, last h)."""
    import oracle
    from qwen_engine_b200 import synth
    threads = oracle.default_threads()
    nbytes = synth.layer_algorithmic_bytes() * len(layers_np)
    oracle.decode_sweep(layers_np[:1], h0, threads=threads)  # warm the library and the page cache
    reps, t0, h = 0, time.perf_counter(), None
    while reps < max_reps and (reps == 0 or time.perf_counter() - t0 < budget_s):
        h = oracle.decode_sweep(layers_np, h0, threads=threads)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return nbytes / dt / 1e9, threads, f"{reps} full {len(layers_np)}-layer sweeps of the oracle port, {dt * 1e3:.1f} ms each", h


def bench_config(num_layers, world, nbytes, extra=None):
    """The `config` object both arms print."""
    cfg = {"workload": WORKLOAD, "layers": num_layers, "parallelism": f"replicas x{world}",
           "algorithmic_bytes_per_step": nbytes,
           "l2": "inputs larger than L2: 675 MB of packed weights are streamed per step"}
    if extra:
        cfg.update(extra)
    return cfg


def run_reference_arm(args):
    """The reference's CPU check of this path (tests/test_kernels.cu:308-363, restated in oracle/) on all host
    threads: W warm-up sweeps, then exactly K timed sweeps (one 28-layer sweep = one step, about 0.1 s)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from qwen_engine_b200 import synth
    layers_np = make_layers_np(args.layers)
    h0 = synth.activations(7, "h0", synth.HIDDEN)
    import oracle
    threads = oracle.default_threads()
    nbytes = synth.layer_algorithmic_bytes() * len(layers_np)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    for _ in range(warm):
        oracle.decode_sweep(layers_np, h0, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.decode_sweep(layers_np, h0, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": bench_config(len(layers_np), max(1, args.gpus), nbytes),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{steps} full {len(layers_np)}-layer sweeps",
                         "note": "the reference's CPU check restated in C (tests/test_kernels.cu:308-363), all host "
                                 "threads; the reference has no separately callable CPU implementation of this path"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ---------------------------------------------------------------------------------

def timed_events(torch, stream, fn, steps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1)  # ms


def measured_traffic(kernel_key):
    """DRAM bytes per launch of a kernel as an ncu capture counted them (dram__bytes_read.sum +
    dram__bytes_write.sum): the `traffic_key <kernel> dram_bytes_per_launch <bytes>` line of the committed
    summaries under profiles/; None if no summary holds one."""
    import re
    pat = re.compile(r"traffic_key\s+" + re.escape(kernel_key) + r"\s+dram_bytes_per_launch\s+(\d+)")
    for path in sorted((ROOT / "profiles").glob("*.md")):
        m = pat.search(path.read_text())
        if m:
            return int(m.group(1))
    return None


def kernel_roofline(torch, ops, layers_dev, stream, peaks, reps=20):
    """Average duration of the dominant kernel of the sweep, timed alone and in the form the sweep launches it:
    the gate_up + SwiGLU GEMV with the RMSNorm + Q8_1 of its fp16 input in the prologue.  One CUDA graph of 28
    launches over the 28 layers' distinct weights (397 MB > L2, so every launch streams from HBM), CUDA events
    around each replay."""
    from qwen_engine_b200 import synth
    H, I = synth.HIDDEN, synth.INTER
    x = torch.from_numpy(synth.activations(3, "roof", H)).cuda()
    out = torch.empty(I, dtype=torch.float16, device="cuda")
    with torch.cuda.stream(stream):
        def all_layers():
            for L in layers_dev:
                ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(L["gate_up"][0], L["gate_up"][1], x, L["post_norm"], out, H, I)
        all_layers()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            all_layers()
        for _ in range(3):
            g.replay()
        stream.synchronize()
        ms = timed_events(torch, stream, g.replay, reps)
    per_launch_s = ms * 1e-3 / (reps * len(layers_dev))
    nbytes = synth.gemv_algorithmic_bytes(2 * I, H, n_out=I) - H * 49 // 32 + 2 * H + 2 * H   # fp16 x and gain instead of Q8_1 x
    achieved = nbytes / per_launch_s / 1e9
    peak = peaks.get("hbm_gbs")
    src = "measured" if peak else "fallback"
    peak = peak or 6650.0
    return {"bound": "hbm", "kernel": "gemv_w4_kernel<SwiGLU, fp16 + RMSNorm input> (gate_up 17920x1536)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": measured_traffic("gemv_gate_up_swiglu_rmsnorm"), "peak_source": f"of {src} (burst copy)",
            "bytes_per_launch": nbytes, "us_per_launch": per_launch_s * 1e6,
            "how": f"CUDA graph of {len(layers_dev)} launches over distinct weights, {reps} replays, CUDA events"}


def time_reference_cuda(torch, layers_dev, stream, steps):
    """Second comparison: the reference's own CUDA kernels rebuilt for sm_100a (oracle/_ref), the same
    chain in one CUDA graph.  Returns None when that library is not present."""
    from oracle import RefKernels
    if not RefKernels.available("fastmath"):
        return None
    import ctypes
    from qwen_engine_b200 import synth
    ref = RefKernels("fastmath")
    H, I = synth.HIDDEN, synth.INTER
    h = torch.from_numpy(synth.activations(7, "h0", H)).cuda()
    q = torch.empty(H, dtype=torch.float16, device="cuda")
    k = torch.empty(synth.KV_DIM, dtype=torch.float16, device="cuda")
    v = torch.empty(synth.KV_DIM, dtype=torch.float16, device="cuda")
    mlp = torch.empty(I, dtype=torch.float16, device="cuda")
    q8 = torch.empty(I, dtype=torch.int8, device="cuda")
    xs = torch.empty(I // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(I // 8, dtype=torch.int32, device="cuda")

    def chain(sp):
        for L in layers_dev:
            ref.call("ref_rmsnorm_q8_1", h, L["input_norm"], None, q8, xs, s8, sp, H)
            pod = RefKernels.QKVPod(L["q"][0].data_ptr(), L["q"][1].data_ptr(), q.data_ptr(), L["k"][0].data_ptr(),
                                    L["k"][1].data_ptr(), k.data_ptr(), L["v"][0].data_ptr(), L["v"][1].data_ptr(),
                                    v.data_ptr())
            ref.call("ref_gemv_qkv_w4a8", pod, q8, xs, s8, sp, H, 12, 2, 128)
            ref.call("ref_quantize_fp16_to_q8_1", q, q8, xs, s8, H, sp)
            ref.call("ref_gemv_w4a8", L["o"][0], L["o"][1], q8, xs, s8, h, h, H, H, sp)
            ref.call("ref_rmsnorm_q8_1", h, L["post_norm"], None, q8, xs, s8, sp, H)
            ref.call("ref_gemv_dual_gate_up_swiglu_w4a8", L["gate_up"][0], L["gate_up"][1], q8, xs, s8, mlp, H, I, sp)
            ref.call("ref_quantize_fp16_to_q8_1", mlp, q8, xs, s8, I, sp)
            ref.call("ref_gemv_w4a8", L["down"][0], L["down"][1], q8, xs, s8, h, h, H, I, sp)

    with torch.cuda.stream(stream):
        sp = ctypes.c_void_p(stream.cuda_stream)
        chain(sp)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            chain(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        for _ in range(3):
            g.replay()
        stream.synchronize()
        ms = timed_events(torch, stream, g.replay, steps)
    us = ms * 1e3 / steps
    nbytes = synth.layer_algorithmic_bytes() * len(layers_dev)
    return {"what": "reference CUDA kernels (src/kernels/*.cu) rebuilt for sm_100a with its own flags, same chain "
                    "in one CUDA graph", "us_per_sweep": us, "value": nbytes / (us * 1e-6) / 1e9, "unit": UNIT}


def lm_head_nsplit(torch, dist, ops, rank, world, stream, steps, warmup):
    """Configuration 2: lm_head 1536 -> 151936 split by vocabulary rows over the ranks, fp16 logit slices
    all-gathered over NVLink (NCCL).  Strong scaling: the total work is fixed."""
    from qwen_engine_b200 import nsplit, synth
    N, K = synth.SHAPES["lm_head"]
    slab = nsplit.slab_bounds(N, world, rank)
    rows = slab.rows
    # every rank draws only its own slab of the synthetic matrix
    qw = synth.packed_weights(11, f"lm_head.r{slab.first}", rows, K)
    sc = synth.scales(11, f"lm_head.r{slab.first}", rows, K)
    x = torch.from_numpy(synth.activations(11, "lm_x", K)).cuda()
    q8 = torch.empty(K, dtype=torch.int8, device="cuda")
    xs = torch.empty(K // 128, dtype=torch.float32, device="cuda")
    s8 = torch.empty(K // 8, dtype=torch.int32, device="cuda")
    # rotate over enough copies of the slab that consecutive steps do not hit L2
    copies = max(1, min(24, int(np.ceil(3 * 126e6 / (qw.nbytes + sc.nbytes)))))
    launch = lambda w, s, a, b, c, out, r, k: ops.launch_gemv_w4a8(w, s, a, b, c, None, out, r, k)
    peer_launch = lambda w, s, a, b, c, out, peers, r, k: ops.gemv_w4a8_peers(w, s, a, b, c, out, peers, r, k)
    d_qw, d_sc = torch.from_numpy(qw.view(np.int32)).cuda(), torch.from_numpy(sc).cuda()
    slabs = [(d_qw, d_sc)] + [(d_qw.clone(), d_sc.clone()) for _ in range(copies - 1)]
    nbytes = synth.gemv_algorithmic_bytes(N, K)
    with torch.cuda.stream(stream):
        ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, K)
    stream.synchronize()

    def measure(use_peers):
        shards = [nsplit.NSplitGemv(w, s, N, K, launch, peer_launch=peer_launch if use_peers else None)
                  for w, s in slabs]
        with torch.cuda.stream(stream):
            def one_round():      # one step per weight copy: GEMV on the local slab, then the exchange
                for sh in shards:
                    sh.forward(q8, xs, s8)
            for _ in range(2):
                one_round()
            stream.synchronize()
            result = shards[0].forward(q8, xs, s8).clone()
            # replayed as one CUDA graph where the exchange captures, so the host's launch cost is not timed
            rounds = max(1, (steps + copies - 1) // copies)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_round()
                run, how = graph.replay, "cuda graph"
            except Exception:
                torch.cuda.synchronize()
                run, how = one_round, "eager"
            for _ in range(max(1, warmup // copies)):
                run()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = timed_events(torch, stream, run, rounds)
            torch.cuda.synchronize()
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3 / (rounds * copies)
        return us, how, result

    def measure_signal():
        """The barrier-free form: slices and completion flags written by the GEMV epilogue, a gathering kernel that
        waits for the flags (nsplit.NSplitSignalGemv)."""
        shards = [nsplit.NSplitSignalGemv(w, s, N, K, ops.gemv_w4a8_peers_signal, ops.gather_after_signals) for w, s in slabs]
        with torch.cuda.stream(stream):
            def one_round():
                for sh in shards:
                    sh.forward(q8, xs, s8)
            for _ in range(2):
                one_round()
            stream.synchronize()
            result = shards[0].forward(q8, xs, s8).clone()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            rounds = max(1, (steps + copies - 1) // copies)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_round()
                run, how = graph.replay, "cuda graph"
            except Exception:
                torch.cuda.synchronize()
                run, how = one_round, "eager"
            for _ in range(max(1, warmup // copies)):
                run()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = timed_events(torch, stream, run, rounds)
            torch.cuda.synchronize()
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        timeouts = int(sum(int(sh.status.item()) != 0 for sh in shards))
        if timeouts:
            raise RuntimeError(f"{timeouts} signal waits ran out")
        return float(t.item()) * 1e3 / (rounds * copies), how, result

    us_nccl, how_nccl, y_nccl = measure(False)
    out = {"workload": f"config 2: lm_head {K}->{N}, rows split over {world} GPU(s)", "rows_per_gpu": rows,
           "unit": UNIT, "scaling": "strong", "weight_copies_rotated": copies,
           "nccl_all_gather": {"us_per_step": us_nccl, "value": nbytes / (us_nccl * 1e-6) / 1e9, "timed_as": how_nccl}}
    best = us_nccl
    if world > 1:
        try:
            us_peer, how_peer, y_peer = measure(True)
            out["peer_store_epilogue"] = {"us_per_step": us_peer, "value": nbytes / (us_peer * 1e-6) / 1e9,
                                          "timed_as": how_peer, "equals_nccl_result": bool(torch.equal(y_nccl, y_peer))}
            best = min(best, us_peer)
        except Exception as e:   # no peer access / symmetric memory on this box
            out["peer_store_epilogue"] = {"unavailable": str(e)[:200]}
        try:
            us_sig, how_sig, y_sig = measure_signal()
            out["peer_store_signal"] = {"us_per_step": us_sig, "value": nbytes / (us_sig * 1e-6) / 1e9,
                                        "timed_as": how_sig, "equals_nccl_result": bool(torch.equal(y_nccl, y_sig))}
            best = min(best, us_sig)
        except Exception as e:
            out["peer_store_signal"] = {"unavailable": str(e)[:200]}
    out["us_per_step"] = best
    out["value"] = nbytes / (best * 1e-6) / 1e9
    out["gpus"] = world
    if world > 1:
        # strong-scaling efficiency against the whole matrix on ONE GPU, timed in this same run (random weights of the
        # full height: the timing does not depend on their values), = t(1 GPU) / (world * t(world GPUs))
        try:
            full = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device="cuda"),
                     (torch.rand((N, K // 128), device="cuda") * 0.018 + 0.002).half()) for _ in range(4)]
            y_full = torch.empty(N, dtype=torch.float16, device="cuda")
            with torch.cuda.stream(stream):
                def full_round():
                    for w, s in full:
                        ops.launch_gemv_w4a8(w, s, q8, xs, s8, None, y_full, N, K)
                full_round()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    full_round()
                graph.replay()
                stream.synchronize()
                rounds = max(1, steps // 4)
                one_us = timed_events(torch, stream, graph.replay, rounds) * 1e3 / (rounds * 4)
            out["single_gpu_us_per_step"] = one_us
            for key in ("nccl_all_gather", "peer_store_epilogue", "peer_store_signal"):
                if isinstance(out.get(key), dict) and "us_per_step" in out[key]:
                    out[key]["strong_scaling_efficiency"] = one_us / (world * out[key]["us_per_step"])
            out["strong_scaling_efficiency"] = one_us / (world * best)
            del full
        except Exception as e:
            out["single_gpu_us_per_step"] = {"unavailable": str(e)[:200]}

    # ---- token selection after lm_head: logits + stand-alone sampler vs. candidates from the GEMV's epilogue ----
    try:
        slots = ops.sample_slots(rows)
        temperature = 0.8
        ctl_a = ops.make_sample_control(temperature, 1234, 0)
        ctl_b = ops.make_sample_control(temperature, 1234, 0)
        val = torch.empty(256, dtype=torch.float32, device="cuda")
        idx = torch.empty(256, dtype=torch.int32, device="cuda")
        tok_a = torch.zeros(1, dtype=torch.int32, device="cuda")
        gathers = [nsplit.NSplitGemv(w, s, N, K, launch) for w, s in slabs]
        cand = lambda w, s, a, b, c, v, i, ctl, off, r, k: ops.launch_gemv_w4a8_sample_candidates(
            w, s, a, b, c, None, v, i, ctl, off, r, k)
        samplers = [nsplit.NSplitSampler(w, s, N, K, slots, cand, ops.launch_sample_finish) for w, s in slabs]

        def unfused_round():
            for g in gathers:
                logits = g.forward(q8, xs, s8)
                ops.launch_sample_and_advance(logits, val, idx, ctl_a, tok_a, None, N)

        def fused_round():
            for sm in samplers:
                sm.forward(q8, xs, s8, ctl_b)

        def time_rounds(fn):
            with torch.cuda.stream(stream):
                fn()
                stream.synchronize()
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        fn()
                    run, how = graph.replay, "cuda graph"
                except Exception:
                    torch.cuda.synchronize()
                    run, how = fn, "eager"
                rounds = max(1, (steps + copies - 1) // copies)
                for _ in range(2):
                    run()
                stream.synchronize()
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                ms = timed_events(torch, stream, run, rounds)
                torch.cuda.synchronize()
            t = torch.tensor([ms], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) * 1e3 / (rounds * copies), how

        # same control state on both sides: one step each from a fresh control block, tokens compared
        ca, cb = ops.make_sample_control(temperature, 99, 5), ops.make_sample_control(temperature, 99, 5)
        with torch.cuda.stream(stream):
            lg = gathers[0].forward(q8, xs, s8)
            ops.launch_sample_and_advance(lg, val, idx, ca, tok_a, None, N)
            tok_f = samplers[0].forward(q8, xs, s8, cb).clone()
        stream.synchronize()
        tok_ref = int(tok_a.item())
        same = tok_ref == int(tok_f.item())
        us_a, how_a = time_rounds(unfused_round)
        us_b, how_b = time_rounds(fused_round)
        one_launch = None
        if world == 1:
            ctl_e = ops.make_sample_control(temperature, 1234, 0)
            cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
            cv = torch.empty(slots, dtype=torch.float32, device="cuda")
            ci = torch.empty(slots, dtype=torch.int32, device="cuda")
            tok_e = torch.zeros(1, dtype=torch.int32, device="cuda")

            def one_launch_round():
                for w, s in slabs:
                    ops.launch_gemv_w4a8_sample_one_launch(w, s, q8, xs, s8, None, cv, ci, cnt, ctl_e, tok_e, N, K)
            ce = ops.make_sample_control(temperature, 99, 5)
            with torch.cuda.stream(stream):
                ops.launch_gemv_w4a8_sample_one_launch(slabs[0][0], slabs[0][1], q8, xs, s8, None, cv, ci, cnt, ce, tok_e, N, K)
            stream.synchronize()
            same_e = int(tok_e.item()) == tok_ref
            us_e, how_e = time_rounds(one_launch_round)
            one_launch = {"us_per_step": us_e, "timed_as": how_e, "same_token": bool(same_e)}
        peer_result = signal_result = None
        if world > 1:
            try:
                pc = lambda w, s, a, b, c, v, i, pv, pi, ctl, off, r, k: ops.gemv_w4a8_sample_candidates_peers(
                    w, s, a, b, c, v, i, pv, pi, ctl, off, r, k)
                ctl_c = ops.make_sample_control(temperature, 1234, 0)
                psamplers = [nsplit.NSplitSampler(w, s, N, K, slots, cand, ops.launch_sample_finish, peer_candidates=pc)
                             for w, s in slabs]
                cc = ops.make_sample_control(temperature, 99, 5)
                with torch.cuda.stream(stream):
                    tok_p = psamplers[0].forward(q8, xs, s8, cc).clone()
                stream.synchronize()

                def peer_round():
                    for sm in psamplers:
                        sm.forward(q8, xs, s8, ctl_c)
                us_c, how_c = time_rounds(peer_round)
                peer_result = {"us_per_step": us_c, "timed_as": how_c, "exchange_bytes_per_gpu": slots * 8 * (world - 1),
                               "same_token": bool(int(tok_p.item()) == tok_ref)}
            except Exception as e:
                peer_result = {"unavailable": str(e)[:200]}
            try:
                ctl_d = ops.make_sample_control(temperature, 1234, 0)
                ssamplers = [nsplit.NSplitSignalSampler(w, s, N, K, slots, ops.gemv_w4a8_sample_candidates_signal,
                                                        ops.sample_finish_after_signals) for w, s in slabs]
                cd = ops.make_sample_control(temperature, 99, 5)
                with torch.cuda.stream(stream):
                    tok_s = ssamplers[0].forward(q8, xs, s8, cd).clone()
                stream.synchronize()

                def signal_round():
                    for sm in ssamplers:
                        sm.forward(q8, xs, s8, ctl_d)
                us_d, how_d = time_rounds(signal_round)
                torch.cuda.synchronize()
                signal_result = {"us_per_step": us_d, "timed_as": how_d, "exchange_bytes_per_gpu": (slots * 8 + 4) * (world - 1),
                                 "same_token": bool(int(tok_s.item()) == tok_ref),
                                 "wait_timeouts": int(sum(int(sm.status.item()) != 0 for sm in ssamplers))}
            except Exception as e:
                signal_result = {"unavailable": str(e)[:200]}
        out["token_selection"] = {
            "temperature": temperature, "candidates_per_gpu": slots,
            "logits_gather_then_sampler": {"us_per_step": us_a, "timed_as": how_a,
                                           "exchange_bytes_per_gpu": rows * 2 if world > 1 else 0},
            "sampling_epilogue": {"us_per_step": us_b, "timed_as": how_b,
                                  "exchange_bytes_per_gpu": slots * 8 if world > 1 else 0},
            "same_token": bool(same)}
        if one_launch is not None:
            out["token_selection"]["sampling_epilogue_one_launch"] = one_launch
        if peer_result is not None:
            out["token_selection"]["sampling_epilogue_peer_store"] = peer_result
        if signal_result is not None:
            out["token_selection"]["sampling_epilogue_peer_store_signal"] = signal_result
    except Exception as e:
        out["token_selection"] = {"unavailable": str(e)[:200]}
    return out


def prefill_big_nsplit(torch, dist, ops, rank, world, stream, steps):
    """Configuration 4's scaled-up shape: W4A16 prefill GEMM 8192 -> 28672 at 4096 tokens, weight rows split over
    the ranks, every rank ending with the whole [M][N] output.  Strong scaling; TFLOP/s counts 2*M*N*K once."""
    from qwen_engine_b200 import nsplit, synth
    N, K, M = 28672, 8192, 4096
    slab = nsplit.slab_bounds(N, world, rank, 128)
    qw = torch.from_numpy(synth.packed_weights(13, f"big.r{slab.first}", slab.rows, K).view(np.int32)).cuda()
    sc = torch.from_numpy(synth.scales(13, f"big.r{slab.first}", slab.rows, K)).cuda()
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((M, K), device="cuda", generator=g).half()
    launch = lambda w, s_, xx, out, m, rows, k: ops.launch_gemm_prefill_w4a16(w, s_, xx, None, out, m, rows, k)
    block = lambda w, s_, xx, ptr, ldc, peers, m, rows, k: ops.gemm_prefill_w4a16_block(w, s_, xx, None, ptr, ldc, peers, m, rows, k)
    flops = 2.0 * M * N * K
    reps = max(3, min(steps, 10))

    def measure(use_peers):
        op = nsplit.NSplitGemm(qw, sc, N, K, M, launch, block_launch=block if use_peers else None)
        with torch.cuda.stream(stream):
            for _ in range(2):
                y = op.forward(x, M)
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = timed_events(torch, stream, lambda: op.forward(x, M), reps)
            torch.cuda.synchronize()
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3 / reps
        return us, y.clone()        # the whole [M][N] result, compared outside the timed region

    out = {"workload": f"config 4: W4A16 prefill GEMM {K}->{N}, {M} tokens, weight rows split over {world} GPU(s)",
           "rows_per_gpu": slab.rows, "unit": "TFLOP/s", "scaling": "strong", "timed_as": "eager launches, CUDA events"}
    us, y_ref = measure(False)
    out["nccl_all_gather"] = {"us_per_step": us, "value": flops / (us * 1e-6) / 1e12}
    best = us
    if world > 1:
        try:
            us_p, y_peer = measure(True)
            # the peer-store form splits K differently on narrow slabs: every entry within one fp16 step, nearly all equal
            diff = (y_peer.float() - y_ref.float()).abs()
            tol = torch.maximum(y_ref.float().abs(), torch.tensor(1.0, device=y_ref.device)) * 2.0 ** -10
            out["peer_store_epilogue"] = {"us_per_step": us_p, "value": flops / (us_p * 1e-6) / 1e12,
                                          "equals_nccl_result": bool(torch.equal(y_peer, y_ref)),
                                          "all_within_one_fp16_step": bool((diff <= tol).all().item()),
                                          "identical_fraction": float((y_peer == y_ref).float().mean().item())}
            best = min(best, us_p)
        except Exception as e:
            out["peer_store_epilogue"] = {"unavailable": str(e)[:200]}
    out["us_per_step"] = best
    out["value"] = flops / (best * 1e-6) / 1e12
    out["gpus"] = world
    if world > 1:
        # strong-scaling efficiency against the whole contraction on ONE GPU, timed in this same run
        try:
            w_full = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device="cuda")
            s_full = (torch.rand((N, K // 128), device="cuda") * 0.018 + 0.002).half()
            y_full = torch.empty((M, N), dtype=torch.float16, device="cuda")
            with torch.cuda.stream(stream):
                for _ in range(2):
                    ops.launch_gemm_prefill_w4a16(w_full, s_full, x, None, y_full, M, N, K)
                stream.synchronize()
                one_us = timed_events(torch, stream, lambda: ops.launch_gemm_prefill_w4a16(w_full, s_full, x, None, y_full, M, N, K), reps) * 1e3 / reps
            out["single_gpu_us_per_step"] = one_us
            for key in ("nccl_all_gather", "peer_store_epilogue"):
                if isinstance(out.get(key), dict) and "us_per_step" in out[key]:
                    out[key]["strong_scaling_efficiency"] = one_us / (world * out[key]["us_per_step"])
            out["strong_scaling_efficiency"] = one_us / (world * best)
            del w_full, s_full, y_full
        except Exception as e:
            out["single_gpu_us_per_step"] = {"unavailable": str(e)[:200]}
    return out


SHAPES_QWEN = {"qkv": (2048, 1536), "o": (1536, 1536), "gate_up": (17920, 1536), "down": (1536, 8960)}
SHAPE_BIG = (28672, 8192)


def shapes_table(torch, ops, stream, peaks, reps=10, m_small=(1, 2, 4, 8, 16, 32, 64), m_prefill=(128, 512, 1024, 4096)):
    """Configurations 0, 3 and 4 per shape.  Every measurement is one CUDA graph that walks enough distinct weight
    copies that nothing is served from L2, timed with CUDA events on `stream`.
      gemv    batch-1 GEMV on pre-quantised input: us, GB/s of algorithmic bytes, fraction of the measured copy peak
              (config 0 is `down`);
      small_m M in {1..64}: us of the form the dispatcher picks, of the CUDA-core few-token form and of the
              tensor-core form, so the crossover can be read off (config 3);
      prefill M in {128..4096}: us, TFLOP/s and the fraction of the measured bf16 peak (config 4)."""
    from qwen_engine_b200 import synth
    hbm, tf = peaks.get("hbm_gbs") or 6650.0, peaks.get("bf16_tflops") or 1590.0
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": "measured" if peaks.get("hbm_gbs") else "fallback"},
           "gemv": {}, "small_m": {}, "prefill": {}}
    g = torch.Generator(device="cuda").manual_seed(1)

    def weights(N, K, copies):
        return [(torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device="cuda", generator=g),
                 (torch.rand((N, K // 128), device="cuda", generator=g) * 0.018 + 0.002).half()) for _ in range(copies)]

    def timed_graph(fn, n=reps):
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                fn()
            for _ in range(3):
                gr.replay()
            stream.synchronize()
            ms = timed_events(torch, stream, gr.replay, n)
        return ms * 1e3 / n   # us per graph

    shapes = dict(SHAPES_QWEN, big=SHAPE_BIG)
    for name, (N, K) in shapes.items():
        wbytes = synth.weight_bytes(N, K)
        copies = max(2, min(28, int(np.ceil(3 * 126e6 / wbytes))))
        ws = weights(N, K, copies)
        x = torch.randn(K, device="cuda", generator=g).half()
        q8 = torch.empty(K, dtype=torch.int8, device="cuda")
        xs = torch.empty(K // 128, dtype=torch.float32, device="cuda")
        s8 = torch.empty(K // 8, dtype=torch.int32, device="cuda")
        with torch.cuda.stream(stream):
            ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, K)
        n_out = N // 2 if name == "gate_up" else N
        y = torch.empty(n_out, dtype=torch.float16, device="cuda")

        def gemv_all():
            for w, sc in ws:
                if name == "gate_up":
                    ops.launch_gemv_dual_gate_up_swiglu_w4a8(w, sc, q8, xs, s8, y, K, n_out)
                else:
                    ops.launch_gemv_w4a8(w, sc, q8, xs, s8, None, y, N, K)
        us = timed_graph(gemv_all) / copies
        nb = synth.gemv_algorithmic_bytes(N, K, n_out=n_out)
        out["gemv"][name] = {"N": N, "K": K, "us": round(us, 3), "GB/s": round(nb / us / 1e3, 1),
                             "frac_of_hbm_peak": round(nb / us / 1e3 / hbm, 3), "weight_copies": copies}

        def gemm_for(M, use):
            xm = torch.randn((M, K), device="cuda", generator=g).half()
            ym = torch.empty((M, n_out), dtype=torch.float16, device="cuda")

            def run():
                for w, sc in use:
                    if name == "gate_up":
                        ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(w, sc, xm, ym, M, None, K, n_out)
                    else:
                        ops.launch_gemm_prefill_w4a16(w, sc, xm, None, ym, M, N, K)
            return run

        if name != "big":
            for M in m_small:
                row = {}
                # dispatch: what the library picks; cuda_core: the few-token CUDA-core form; mma_sync: the weight-streaming
                # kernel with warp-level MMAs; tensor_core: the tcgen05 kernel
                for label, opt, mma_max in (("dispatch", 0, 0), ("cuda_core", 1 << 20, 1), ("mma_sync", 1, 1 << 20),
                                            ("tensor_core", 1, 1)):
                    ops.set_option(ops.OPT_GEMM_MIN_TOKENS_TENSOR_CORE, opt)
                    ops.set_option(ops.OPT_GEMM_MMA_MAX_TOKENS, mma_max)
                    try:
                        row[label + "_us"] = round(timed_graph(gemm_for(M, ws), n=max(3, reps // 2)) / copies, 3)
                    finally:
                        ops.set_option(ops.OPT_GEMM_MIN_TOKENS_TENSOR_CORE, 0)
                        ops.set_option(ops.OPT_GEMM_MMA_MAX_TOKENS, 0)
                row["GB/s"] = round((wbytes + 2 * M * K + 2 * M * n_out) / row["dispatch_us"] / 1e3, 1)
                out["small_m"][f"{name}.M{M}"] = row
        for M in (m_prefill if name != "big" else (m_prefill[0], m_prefill[-1])):
            use = ws[:2] if M >= 512 else ws
            us = timed_graph(gemm_for(M, use), n=max(3, reps // 2)) / len(use)
            flops = 2.0 * M * N * K
            out["prefill"][f"{name}.M{M}"] = {"us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1),
                                              "frac_of_bf16_peak": round(flops / us / 1e6 / tf, 3)}
        del ws
        torch.cuda.empty_cache()
    # the GEMV -> tensor-core crossover per shape: the smallest M at which the tensor-core form is the faster one
    for name in SHAPES_QWEN:
        cross = None
        for M in m_small:
            r = out["small_m"][f"{name}.M{M}"]
            if min(r["tensor_core_us"], r["mma_sync_us"]) < r["cuda_core_us"]:
                cross = M
                break
        out["small_m"][f"{name}.crossover_M"] = cross
    out["tc_wait_timeouts"] = ops.debug_counter(0)
    return out


def run_shapes_suite(args):
    """`--suite shapes`: the per-shape table alone."""
    import torch
    import qwen_engine_b200 as ops
    torch.cuda.set_device(0)
    ops.init()
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    ops.set_option(ops.OPT_GEMV_FORM, args.gemv_form)
    out = shapes_table(torch, ops, torch.cuda.Stream(), peaks, reps=max(3, min(args.steps, 20)))
    out["suite"] = "shapes"
    out["gemv_form"] = args.gemv_form
    print(json.dumps(out), flush=True)


def run_single(args):
    """A handful of launches of one kernel over distinct weight copies (so DRAM counters mean something)."""
    import torch
    import qwen_engine_b200 as ops
    from qwen_engine_b200 import synth
    torch.cuda.set_device(0)
    ops.init()
    ops.set_option(ops.OPT_GEMV_FORM, args.gemv_form)
    shapes = {"qkv": (2048, 1536), "o": (1536, 1536), "gate_up": (17920, 1536), "down": (1536, 8960),
              "lm_head": (151936, 1536), "big": (28672, 8192)}
    N, K = shapes[args.shape]
    g = torch.Generator(device="cuda").manual_seed(1)
    copies = max(2, min(12, int(np.ceil(2 * 126e6 / synth.weight_bytes(N, K)))))
    ws = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device="cuda", generator=g),
           (torch.rand((N, K // 128), device="cuda", generator=g) * 0.018 + 0.002).half()) for _ in range(copies)]
    n_out = N // 2 if args.shape == "gate_up" else N
    reps = max(1, min(args.steps, 12))
    if args.m == 0:
        x = torch.randn(K, device="cuda", generator=g).half()
        q8 = torch.empty(K, dtype=torch.int8, device="cuda")
        xs = torch.empty(K // 128, dtype=torch.float32, device="cuda")
        s8 = torch.empty(K // 8, dtype=torch.int32, device="cuda")
        y = torch.empty(n_out, dtype=torch.float16, device="cuda")
        ops.launch_quantize_fp16_to_q8_1(x, q8, xs, s8, K)
        gamma = torch.full((K,), 0.05, dtype=torch.float16, device="cuda")
        for i in range(reps):
            w, sc = ws[i % copies]
            if args.shape == "gate_up":
                if args.input == "q8":
                    ops.launch_gemv_dual_gate_up_swiglu_w4a8(w, sc, q8, xs, s8, y, K, n_out)
                elif args.input == "fp16":
                    ops.launch_gemv_dual_gate_up_swiglu_w4a16(w, sc, x, y, K, n_out)
                else:
                    ops.launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(w, sc, x, gamma, y, K, n_out)
            elif args.input == "q8":
                ops.launch_gemv_w4a8(w, sc, q8, xs, s8, None, y, N, K)
            else:
                ops.launch_gemv_rmsnorm_w4a16(w, sc, x, gamma if args.input == "fp16norm" else None, None, y, N, K)
    else:
        M = args.m
        xm = torch.randn((M, K), device="cuda", generator=g).half()
        ym = torch.empty((M, n_out), dtype=torch.float16, device="cuda")
        for i in range(reps):
            w, sc = ws[i % copies]
            if args.shape == "gate_up":
                ops.launch_gemm_prefill_dual_gate_up_swiglu_w4a16(w, sc, xm, ym, M, None, K, n_out)
            else:
                ops.launch_gemm_prefill_w4a16(w, sc, xm, None, ym, M, N, K)
    torch.cuda.synchronize()
    print(json.dumps({"suite": "single", "shape": args.shape, "m": args.m, "input": args.input, "launches": reps, "copies": copies,
                      "tc_wait_timeouts": ops.debug_counter(0)}), flush=True)


def main():
    args = parse()
    if args.suite == "single":
        run_single(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.suite == "shapes":
        run_shapes_suite(args)
        return

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the W4A16 kernels have no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import qwen_engine_b200 as ops
    from qwen_engine_b200 import synth
    ops.init()
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass

    steps, warmup = max(1, args.steps), max(3, args.warmup)
    layers_np = make_layers_np(args.layers)
    layers_dev = upload_layers(layers_np)
    stream = torch.cuda.Stream()
    h0_np = synth.activations(7, "h0", synth.HIDDEN)
    h_in = torch.from_numpy(h0_np).cuda()
    h_out = torch.empty_like(h_in)
    pin_in = torch.from_numpy(h0_np).pin_memory()
    pin_out = torch.empty(synth.HIDDEN, dtype=torch.float16).pin_memory()
    sweep_flags = args.sweep_flags if args.sweep_flags >= 0 else ops.SWEEP_DEFAULT
    ops.set_option(ops.OPT_GEMV_FORM, args.gemv_form)
    with torch.cuda.stream(stream):
        sweep = ops.DecodeSweep(layers_dev, stream=stream, flags=sweep_flags)
    nbytes = synth.layer_algorithmic_bytes() * len(layers_np)

    props = torch.cuda.get_device_properties(local)
    try:
        bus_id = f"{props.pci_domain_id:08X}:{props.pci_bus_id:02X}:{props.pci_device_id:02X}.0"
    except AttributeError:
        bus_id = None
    sampler = ClockSampler(local, pci_bus_id=bus_id)
    sampler.start()

    # ---- device-resident timing: W warm-up, then exactly K steps --------------------------
    for _ in range(warmup):
        sweep.run_device(h_in, h_out, stream)
    stream.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = timed_events(torch, stream, lambda: sweep.run_device(h_in, h_out, stream), steps)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / steps
    value = world * nbytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host buffers, copies and the host's read of the result inside the region ---
    def e2e_step():
        sweep.run_host(pin_in, pin_out, stream)
        stream.synchronize()
        _ = pin_out[0].item()
    for _ in range(3):
        e2e_step()
    if world > 1:
        dist.barrier()
    ms_e2e = timed_events(torch, stream, e2e_step, steps)
    t = torch.tensor([ms_e2e], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * nbytes / (float(t.item()) / steps * 1e-3) / 1e9
    clocks = sampler.stop()

    final = pin_out.numpy().copy()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "us_per_sweep": ms_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": bench_config(len(layers_np), world, nbytes),
        "options": {"pdl": bool(ops.get_option(ops.OPT_PDL)), "sweep_flags": sweep_flags, "gemv_form": args.gemv_form},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": synth.HIDDEN * 2,
                "d2h_bytes_per_step": synth.HIDDEN * 2,
                "how": "w4a16_sweep_run_host: pinned fp16 hidden state in, sweep graph, hidden state out, "
                       "stream synchronise and host read every step; weights resident (model state)"},
        "gpu_launches": sweep.launches * steps, "gpu_launches_per_step": sweep.launches,
        "clocks": clocks,
        "result_finite": bool(np.isfinite(final.astype(np.float32)).all()),
    }

    if rank == 0:
        with torch.cuda.stream(stream):
            line["roofline"] = kernel_roofline(torch, ops, layers_dev, stream, peaks)
        line["roofline_sweep"] = {"achieved": value / world, "peak": peaks.get("hbm_gbs", 6650.0),
                                  "frac": value / world / peaks.get("hbm_gbs", 6650.0), "unit": UNIT,
                                  "note": f"whole sweep ({sweep.launches} dependent launches) per GPU against the copy peak"}
    if world > 1 or not args.no_lm_head:
        lm = lm_head_nsplit(torch, dist, ops, rank, world, stream, min(steps, 200), warmup)
        if rank == 0:
            line["lm_head"] = lm
    if not args.no_prefill:
        try:
            pf = prefill_big_nsplit(torch, dist, ops, rank, world, stream, steps)
        except Exception as e:      # keeps the headline line alive if this extra fails (e.g. memory on a busy GPU)
            pf = {"unavailable": str(e)[:200]}
        if rank == 0:
            line["prefill_big"] = pf
    if rank == 0 and world == 1 and not args.no_shapes:
        try:
            line["roofline"]["per_shape"] = shapes_table(torch, ops, stream, peaks)
        except Exception as e:
            line["roofline"]["per_shape"] = {"unavailable": str(e)[:200]}
    if rank == 0:
        # the driver's record keeps the objects it knows: the extras are also carried inside `roofline`
        line["roofline"]["sweep"] = line["roofline_sweep"]
        for key in ("lm_head", "prefill_big"):
            if key in line:
                line["roofline"][key] = line[key]
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ref_cuda = time_reference_cuda(torch, layers_dev, stream, min(steps, 100))
        if ref_cuda:
            line["reference_cuda_sm100a"] = ref_cuda
        gbs, cores, sample, h_cpu = time_cpu_sweep(layers_np, h0_np)
        line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        if ref_cuda:   # second comparison: the reference's own CUDA kernels rebuilt for sm_100a
            line["cpu_baseline"]["reference_cuda_sm100a"] = ref_cuda
        # sanity: first layer of the device sweep against the oracle on the same input
        import oracle
        one = ops.DecodeSweep(layers_dev[:1], stream=stream)
        one.run_host(pin_in, pin_out, stream)
        stream.synchronize()
        h1 = oracle.decode_sweep(layers_np[:1], h0_np)
        err = np.abs(pin_out.numpy().astype(np.float64) - h1.astype(np.float64))
        line["check_layer0_max_abs_err"] = float(err.max())
        line["check_layer0_rms"] = float(np.sqrt(np.mean(h1.astype(np.float64) ** 2)))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
