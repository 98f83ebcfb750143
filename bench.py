#!/usr/bin/env python
"""Benchmark of the GPTQ QuantLinear forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload: the 3-bit act-order decode GEMV (K=4096, N=11008, group 128,
M=1).  One *step* is `passes_per_step` passes over a pool of distinct layers of that
shape whose packed weights together exceed the L2 cache, so every launch streams its
weights from HBM; the number of passes is chosen so that the timed region lasts at
least half a second (sustained clocks, enough clock samples).  The headline `value`
is weight bytes per second over the whole job with all inputs resident on the device;
`e2e` is the same quantity through `QuantLinear.forward` with the activations starting
in pinned host memory and the results ending there.  Under torchrun every rank runs
its own pool (the layers of a column-parallel linear are independent: no collective
on the data path) and rank 0 reports the sum; the tensor-parallel models
(`llama7b_decode`, `opt66b_decode`) ride on the same line, with a check that the
sharded model computes what the unsharded one computes (`tp_parity`).

`--impl reference` times the reference's CPU dequantise-then-matmul path
(auto_gptq/nn_modules/qlinear.py:197-243: the reference's own file when it has been
staged under oracle/_ref, else the oracle's restatement of it) on the host cores; it
does not load the CUDA library.
"""
from __future__ import annotations

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

import torch  # noqa: E402

WORKLOADS = {
    "gemv_b3_k4096_n11008_act": dict(bits=3, K=4096, N=11008, group_size=128, act_order=True, M=1),
    "gemv_b4_k4096_n4096": dict(bits=4, K=4096, N=4096, group_size=128, act_order=False, M=1),
}
DEFAULT_WORKLOAD = "gemv_b3_k4096_n11008_act"
POOL_BYTES = 320 << 20  # > 2x the 126 MB L2
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised under profiles/
NCU_DRAM_BYTES_PER_LAUNCH = {"gemv_b3_k4096_n11008_act": 17805568, "gemv_b4_k4096_n4096": None}
METRIC = "gemv_weight_GBps"
MIN_TIMED_MS = 500.0   # the timed region of the headline lasts at least this long


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        # nvidia-smi needs a moment before its first line: wait for it, so that samples exist once the load starts
        t_end = time.perf_counter() + 2.0
        while not self.samples and time.perf_counter() < t_end:
            time.sleep(0.01)

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self, t_begin=None, t_end=None):
        """Median SM clock and throttle reasons of the samples taken between ``t_begin`` and ``t_end``
        (host clock around the GPU load; all samples if not given)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        picked = [p for t, p in self.samples
                  if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end + 0.03)]
        for s in picked:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_forward(cfg):
    """``(forward, x, layer, kind)``: the reference's CPU forward of one layer of the workload.  ``kind`` is
    "reference" when the reference's own qlinear.py has been staged under oracle/_ref (oracle/stage_ref.py), else
    "port" (the oracle's restatement, proven bit-identical to it by tests/test_oracle.py)."""
    import contextlib
    import io
    from autogptq.tvm_b200 import synth          # synthetic tensors only: does not load the CUDA library
    from oracle import stage_ref
    layer = synth.make_layer(cfg["bits"], cfg["K"], cfg["N"], cfg["group_size"], cfg["act_order"], seed=1)
    x = synth.make_x(cfg["M"], cfg["K"], seed=1)
    ref = None
    with contextlib.redirect_stdout(io.StringIO()):
        ref = stage_ref.load()
    if ref is not None:
        mod = ref.QuantLinear(cfg["bits"], cfg["group_size"], cfg["K"], cfg["N"], False)
        mod.qweight, mod.qzeros, mod.scales, mod.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx

        def forward():
            with contextlib.redirect_stdout(io.StringIO()):   # the reference prints on every call
                return mod.forward(x)
        return forward, x, layer, "reference"
    from oracle.gptq_oracle import TorchQuantLinearOracle
    orc = TorchQuantLinearOracle(cfg["bits"], layer.qweight, layer.qzeros, layer.scales, layer.g_idx)
    return (lambda: orc.forward(x)), x, layer, "port"


def cpu_baseline(cfg, budget_s=20.0, max_calls=9):
    """Time the reference's CPU path on one layer of the workload."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    forward, x, layer, kind = reference_forward(cfg)
    forward()  # warm-up
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < budget_s and len(times) < max_calls):
        t0 = time.perf_counter()
        forward()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": layer.weight_bytes() / med / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "seconds_per_call": med,
            "sample": f"{len(times)} forward calls of one layer of the workload (median), torch CPU, {cores} threads"}


def time_gemv_workload(name, dev, steps=300):
    """Weight GB/s and roofline fraction of another GEMV workload (same method as the headline)."""
    from autogptq.tvm_b200 import QuantLinear, ops, synth, _lib
    cfg = WORKLOADS[name]
    bits, K, N, gs, M = cfg["bits"], cfg["K"], cfg["N"], cfg["group_size"], cfg["M"]
    proto = synth.make_layer(bits, K, N, gs, cfg["act_order"], seed=77, device=dev)
    P = max(2, -(-POOL_BYTES // proto.weight_bytes()))
    mods = []
    for i in range(P):
        L = proto if i == 0 else synth.make_layer(bits, K, N, gs, cfg["act_order"], seed=77 + i, device=dev)
        m = QuantLinear(bits, gs, K, N, False)
        m.qweight, m.qzeros, m.scales, m.g_idx = L.qweight, L.qzeros, L.scales, L.g_idx
        m = m.to(dev)
        m.post_init()
        mods.append(m)
    x = synth.make_x(M, K, seed=3, device=dev)
    y = torch.empty((P, M, N), dtype=torch.float16, device=dev)
    ws = ops.get_workspace(dev, _lib.workspace_bytes(_lib.OP_GEMV, M, K, N, bits))

    def one_pass():
        for i, m in enumerate(mods):
            ops.gemv(x, m._qweight_run, m.qzeros, m.scales, m._g_idx_run, bits, gs, x_perm=m._x_perm, out=y[i],
                     workspace=ws)
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        one_pass()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        one_pass()
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * P)
    peak, _ = measured_peaks()
    return {"workload": name, "us_per_launch": us, "weight_GBps": proto.weight_bytes() / us / 1e3,
            "algorithmic_GBps": proto.algorithmic_bytes(M) / us / 1e3,
            "frac_of_measured_hbm": proto.algorithmic_bytes(M) / us / 1e3 / peak, "launches": (steps + 4) * P}


def time_gemm_sweep(dev):
    """Config 2: 4-bit, K=4096, N=12288, M in {16,128,512,2048}; TFLOP/s against the measured dense peak."""
    from autogptq.tvm_b200 import ops, synth
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak_tf, kind = 1590.0, "fallback"
    if os.path.isfile(path):
        with open(path) as f:
            peak_tf, kind = float(json.load(f)["bf16_tflops"]), "measured"
    K, N, bits = 4096, 12288, 4
    layers = [synth.make_layer(bits, K, N, 128, False, seed=200 + i, device=dev) for i in range(6)]  # 151 MB > L2
    out, launches = [], 0
    for M in (16, 128, 512, 2048):
        x = synth.make_x(M, K, seed=M, device=dev)
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        for L in layers:
            ops.gemm(x, L.qweight, L.qzeros, L.scales, None, bits, 128, out=y)
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            for L in layers:
                ops.gemm(x, L.qweight, L.qzeros, L.scales, None, bits, 128, out=y)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * len(layers))
        tf = 2.0 * M * K * N / us / 1e6
        launches += (reps + 1) * len(layers)
        out.append({"M": M, "us": us, "TFLOPs": tf, "frac_of_dense_peak": tf / peak_tf,
                    "weight_GBps": layers[0].weight_bytes() / us / 1e3})
    return {"workload": "gemm_b4_k4096_n12288", "peak_TFLOPs": peak_tf, "peak_kind": kind, "sweep": out,
            "launches": launches}


def time_llama_decode(dev, world, prompt_len=512, decode_steps=256):
    """Config 3: Llama-7B architecture, 4-bit g128, batch 1, 512-token prompt, 256 greedy decode steps, TP = world."""
    from autogptq.tvm_b200 import decoder
    return time_decode(dev, world, decoder.LLAMA_7B, "llama7b_arch_int4_g128_bs1_p512_d256", 1, prompt_len, decode_steps)


def time_opt66b_decode(dev, world):
    """Config 4: OPT-66B architecture, 3-bit g128 act-order, batch 1 and 16, 128-token prompts, 128 decode steps."""
    from autogptq.tvm_b200 import decoder
    return [time_decode(dev, world, decoder.OPT_66B, f"opt66b_arch_int3_g128_act_bs{b}_p128_d128", b, 128, 128)
            for b in (1, 16)]


def time_decode(dev, world, cfg, name, batch, prompt_len, decode_steps):
    from autogptq.tvm_b200 import decoder
    # world > 1: the row-parallel linears and the token pick exchange through peer memory inside the library's
    # kernels (up to 8 rows; larger batches use the process group's all-reduce)
    m = decoder.GPTQDecoder(cfg, batch=batch, device=dev, fused_allreduce=world > 1)
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=torch.Generator().manual_seed(11)).to(dev)
    m.prefill(prompt)            # warm-up (builds run-time views, sizes scratch)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    m.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    # load-time tuning, outside the timed region: the GEMV work split per kind of linear layer, measured in the step
    tuning = m.tune()
    m.capture()
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    e0.record()
    toks = m.decode(decode_steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms, prefill_ms], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, prefill_ms = float(t[0]), float(t[1])
    peak, _ = measured_peaks()
    per_tok_s = ms * 1e-3 / decode_steps
    out = {"workload": name, "tp": world, "batch": batch, "decode_tok_s": batch * decode_steps / (ms * 1e-3),
           "ms_per_token": ms / decode_steps, "prefill_ms": prefill_ms,
           "weight_bytes_per_token_per_gpu": m.bytes_per_token(),
           "frac_of_hbm_roofline": m.bytes_per_token() / per_tok_s / 1e9 / peak,
           "last_token": int(toks[-1, 0]), "gemv_tuning": {k: (list(v) if v else None) for k, v in tuning.items()},
           "allreduce": "none" if world == 1 else ("fused peer-memory exchange" if batch <= 8 else "process group")}
    if m.exchange is not None:
        out["exchange_status"] = m.exchange.status()     # 0: no wait of the fused all-reduce ever ran out
    # what one token launches on this rank (one extra step under the activity tracer, after the timed region; every
    # rank runs it, because the step's exchange needs all of them)
    try:
        kernels = m.step_kernels()
        out["step_kernels"] = {k: v for k, v in sorted(kernels.items(), key=lambda kv: -kv[1])}
        out["step_library_collectives"] = sum(v for k, v in kernels.items() if "nccl" in k.lower())
    except Exception as e:   # the tracer is optional evidence, not part of the measurement
        out["step_kernels"] = {"unavailable": repr(e)[:120]}
    m.close()
    return out


def tp_parity_llama(dev):
    """World > 1: the tensor-parallel Llama-7B-architecture model against the same model on rank 0 alone (logits of
    the prompt's last token and of the first decode step; tolerance of the output contract at the vocabulary
    projection)."""
    from autogptq.tvm_b200 import decoder
    prompt = torch.randint(0, decoder.LLAMA_7B.vocab, (1, 64), generator=torch.Generator().manual_seed(12)).to(dev)
    return decoder.tp_parity(decoder.LLAMA_7B, prompt, dev, fused_allreduce=True)


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    forward, x, layer, kind = reference_forward(cfg)
    steps, warmup = args.steps, max(args.warmup, 3)     # the same counts as the GPU arm
    for _ in range(warmup):
        forward()
    t0 = time.perf_counter()
    for _ in range(steps):
        forward()
    dt = (time.perf_counter() - t0) / steps
    val = layer.weight_bytes() / dt / 1e9
    sample = f"each step = one forward of one layer of the workload on the host, {cores} torch threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": args.workload, **cfg},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "cuda_library_loaded": "autogptq.tvm_b200._lib" in sys.modules,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="shortest timed region of the headline (profiling runs pass 0 to keep the launch count small)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip config 0, the GEMM sweep and the decode run")
    ap.add_argument("--no-opt66b", action="store_true",
                    help="skip the OPT-66B-architecture decode runs (config 4)")
    ap.add_argument("--gemm-demo", type=int, default=0, metavar="M",
                    help="only launch the config-2 GEMM a few times with M rows (a small target for ncu) and exit")
    args = ap.parse_args()
    t_program = time.perf_counter()
    cfg = dict(WORKLOADS[args.workload])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return
    if args.gemm_demo:
        from autogptq.tvm_b200 import ops, synth
        dev = torch.device("cuda", local_rank)
        layers = [synth.make_layer(4, 4096, 12288, 128, False, seed=i, device=dev) for i in range(3)]
        x = synth.make_x(args.gemm_demo, 4096, seed=1, device=dev)
        for _ in range(2):
            for L in layers:
                y = ops.gemm(x, L.qweight, L.qzeros, L.scales, None, 4, 128)
        torch.cuda.synchronize()
        print(json.dumps({"gemm_demo_rows": args.gemm_demo, "checksum": float(y.float().abs().sum())}))
        return

    import torch.distributed as dist
    from autogptq.tvm_b200 import QuantLinear, ops, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)

    bits, K, N, gs, M = cfg["bits"], cfg["K"], cfg["N"], cfg["group_size"], cfg["M"]
    proto = synth.make_layer(bits, K, N, gs, cfg["act_order"], seed=1000 * rank, device=dev)
    P = max(2, -(-POOL_BYTES // proto.weight_bytes()))
    mods = []
    for i in range(P):
        L = proto if i == 0 else synth.make_layer(bits, K, N, gs, cfg["act_order"], seed=1000 * rank + i, device=dev)
        m = QuantLinear(bits, gs, K, N, False)
        m.qweight, m.qzeros, m.scales, m.g_idx = L.qweight, L.qzeros, L.scales, L.g_idx
        m = m.to(dev)
        m.post_init()
        mods.append(m)
    x_dev = synth.make_x(M, K, seed=rank, device=dev)
    y_dev = torch.empty((P, M, N), dtype=torch.float16, device=dev)
    from autogptq.tvm_b200 import _lib
    ws = ops.get_workspace(dev, _lib.workspace_bytes(_lib.OP_GEMV, M, K, N, bits))

    def one_pass():
        for i, m in enumerate(mods):
            ops.gemv(x_dev, m._qweight_run, m.qzeros, m.scales, m._g_idx_run, bits, gs, x_perm=m._x_perm,
                     out=y_dev[i], workspace=ws)

    # capture one pass in a CUDA graph: the timed region is then free of host launch gaps
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        one_pass()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        one_pass()

    def barrier():
        if world > 1:
            dist.barrier()

    # passes per step: enough graph replays that the timed region lasts at least half a second
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 10], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    passes = max(1, int(-(-args.min_timed_ms // (float(t[0]) * args.steps))))

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        for _ in range(passes):
            graph.replay()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    t_load = time.perf_counter()      # clock samples are taken between here and the end of the timed steps
    e0.record()
    for _ in range(args.steps):
        for _ in range(passes):
            graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_load, time.perf_counter())
    barrier()

    # ---- end to end through QuantLinear.forward with host buffers ----
    x_host = torch.empty((P, M, K), dtype=torch.float16).pin_memory()
    x_host.copy_(synth.make_x(P * M, K, seed=99).reshape(P, M, K))
    y_host = torch.empty((P, M, N), dtype=torch.float16).pin_memory()
    x_stage = torch.empty((P, M, K), dtype=torch.float16, device=dev)
    e2e_steps = max(3, min(args.steps, 50))

    def e2e_pass():
        x_stage.copy_(x_host, non_blocking=True)
        ys = [m(x_stage[i]) for i, m in enumerate(mods)]
        y_host.copy_(torch.stack(ys), non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(3):
        e2e_pass()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    e2e_s = (time.perf_counter() - t0) / e2e_steps

    t = torch.tensor([ms, e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_s = float(t[0]), float(t[1])

    extras = {}
    if not args.no_extras:
        del mods, graph
        torch.cuda.empty_cache()
        if rank == 0:
            extras["gemv_config0"] = time_gemv_workload("gemv_b4_k4096_n4096", dev)
            extras["gemm_config2"] = time_gemm_sweep(dev)
        torch.cuda.empty_cache()
        barrier()
        extras["llama7b_decode"] = time_llama_decode(dev, world)   # every rank takes part (tensor parallel)
        if world > 1:
            torch.cuda.empty_cache()
            barrier()
            par = tp_parity_llama(dev)
            if rank == 0:
                extras["llama7b_decode"]["tp_parity"] = par
        # config 4 rides on the same line; on one GPU only while the run has taken less than 300 s so far
        if not args.no_opt66b and (world > 1 or time.perf_counter() - t_program < 300.0):
            torch.cuda.empty_cache()
            barrier()
            extras["opt66b_decode"] = time_opt66b_decode(dev, world)

    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_per_step = ms / args.steps
        wbytes = proto.weight_bytes()
        abytes = proto.algorithmic_bytes(M)
        launch_s = ms_per_step * 1e-3 / (P * passes)
        value = world * P * passes * wbytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, **cfg, "pool_layers": P, "passes_per_step": passes,
                       "l2_policy": f"every pass streams {P} distinct layers ({P * wbytes >> 20} MiB of weights) > L2",
                       "act_order_handling": "rows sorted by group once at load; x gathered in-kernel",
                       "launch": "one CUDA graph replay per pass, one layer per kernel launch",
                       "timed_region_ms": ms},
            "roofline": {"bound": "hbm", "achieved": abytes / launch_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": abytes / launch_s / 1e9 / peak, "traffic": None,
                         "peak_kind": peak_kind, "us_per_launch": launch_s * 1e6,
                         "algorithmic_bytes_per_launch": abytes, "weight_bytes_per_launch": wbytes,
                         "frac_of_nominal_8TBps_on_weight_bytes": wbytes / launch_s / 8e12},
            "e2e": {"value": world * P * wbytes / e2e_s / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": P * M * K * 2, "d2h_bytes_per_step": P * M * N * 2,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
            "gpu_launches": args.steps * P * passes + e2e_steps * P + sum(v.get("launches", 0) for v in extras.values() if isinstance(v, dict)),
            "clocks": clocks,
        }
        line["roofline"]["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)
        # sticky status words of the kernels' bounded waits: raises if any wait ever ran out
        try:
            ops.check_status(dev)
            line["bounded_waits_expired"] = False
        except RuntimeError:
            line["bounded_waits_expired"] = True
        line.update(extras)
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
