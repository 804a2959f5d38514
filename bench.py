#!/usr/bin/env python
"""Decode throughput of the quantized-linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one greedily decoded token of a random-init Qwen2.5-32B-shaped decoder with Q4_K
projections (64 layers; 17.99 GB of GGUF blocks per token, far larger than L2, so every step
streams them from HBM) after a 512-token random prompt.  Prints ONE JSON line.
With N > 1 (launched under torchrun) the model is split tensor-parallel over the N GPUs: q/k/v, gate, up
and the head by rows, attention output and down by K with one all-reduce each (the library's own
one-shot kernel over NVLink peer memory, or NCCL with --comm nccl).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s (Q4_K Qwen-shaped)"
UNIT = "tok/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the persistent step, from the ncu captures
# summarised under profiles/ (taken on a cut of few layers and scaled by the weights per step)
MEGAKERNEL_TRAFFIC = {("qwen2.5-32b-q4_k", 1): 18.10e9}   # profiles/decode_megakernel_qwen32b_q4k_2l.md


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            data = json.load(fh)
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = sorted(sm)[len(sm) // 4:]  # drop the idle samples before and after the region
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


def workload_config(name: str):
    from neura_b200 import qwen

    if name == "qwen2.5-32b-q4_k":
        return qwen.QWEN25_32B_Q4K
    if name == "qwen2.5-0.5b-q8_0":
        return qwen.QWEN25_05B_Q8
    if name.startswith("qwen2.5-32b-q4_k-"):
        return qwen.scaled(qwen.QWEN25_32B_Q4K, int(name.rsplit("-", 1)[1].rstrip("l")))
    raise SystemExit(f"unknown workload {name}")


def workload_description(config, prompt: int, rows: int, parallelism: str) -> dict:
    """The `config` object of a line: both arms describe the workload the same way."""
    return {"workload": f"{config.name} decode: {config.layers} layers, hidden {config.hidden}, "
                        f"{config.heads}/{config.key_heads} heads x {config.head_width}, ff {config.feed_forward}, "
                        f"vocab {config.vocab}; {prompt}-token random prompt, greedy",
            "batch": rows, "parallelism": parallelism,
            "l2": f"inputs larger than L2 ({config.weight_bytes() / 1e9:.2f} GB of weights per step)",
            "weight_bytes_per_token": config.weight_bytes()}


def cpu_baseline(config, seconds: float = 12.0):
    """The oracle's product (the reference tests' f32 loop over unpacked blocks) on the host
    cores, on a bounded sample of the token: rows of the up projection of one layer."""
    import numpy as np
    import oracle

    cores = os.cpu_count() or 1
    k = config.hidden
    n = min(config.feed_forward, 4096)
    w = oracle.Stream(23).normal(n * k, 0.0, 0.02).reshape(n, k)
    packed = oracle.pack_rows(config.element, w)
    x = oracle.Stream(29).normal(k).reshape(1, k)
    oracle.linear(config.element, packed, n, k, x, threads=cores)  # warm-up
    runs, spent = 0, 0.0
    while spent < seconds and runs < 4096:
        t0 = time.perf_counter()
        oracle.linear(config.element, packed, n, k, x, threads=cores)
        spent += time.perf_counter() - t0
        runs += 1
    per_weight = spent / runs / (n * k)
    tok_s = 1.0 / (per_weight * config.weight_elements())
    return {"value": tok_s, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{runs} runs of a [{n}x{k}] {('Q4_K' if config.element == 9 else 'Q8_0')} product at batch 1 "
                      f"({spent:.1f} s), scaled by weights per token ({config.weight_elements()})"}


def run_reference(args):
    """The reference has no CPU (or CUDA) implementation of the product; its only executable
    statement of it is the f32 loop of its tests, which the oracle restates.  This arm times
    that on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    config = workload_config(args.workload)
    import numpy as np  # noqa: F401
    import oracle

    cores = os.cpu_count() or 1
    k, n = config.hidden, min(config.feed_forward, 2048)
    w = oracle.Stream(23).normal(n * k, 0.0, 0.02).reshape(n, k)
    packed = oracle.pack_rows(config.element, w)
    x = oracle.Stream(29).normal(k).reshape(1, k)
    for _ in range(max(1, args.warmup)):
        oracle.linear(config.element, packed, n, k, x, threads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear(config.element, packed, n, k, x, threads=cores)
    elapsed = time.perf_counter() - t0
    scale = config.weight_elements() / (n * k)
    ms_per_step = elapsed / args.steps * scale * 1e3
    value = 1e3 / ms_per_step
    sample = (f"each step = a [{n}x{k}] product at batch 1 on {cores} threads, scaled by weights per token "
              f"(x{scale:.0f})")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_description(config, args.prompt, 1, "host cores"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist = None
        torch.cuda.set_device(local)

    import neura_b200 as nb
    from neura_b200 import qwen
    from neura_b200.synthetic import synthetic_norms, synthetic_weights

    config = workload_config(args.workload)
    rows = args.batch
    warmup = max(3, args.warmup)
    capacity = args.prompt + 2 * (warmup + args.steps) + 8
    rt = nb.Runtime(local)
    rt.use_stream(rt.new_stream())
    tstream = torch.cuda.ExternalStream(rt.stream.value, device=torch.device("cuda", local))
    shard = comm = None
    if world > 1:  # tensor parallel: one model split over the ranks
        from neura_b200 import parallel

        shard = parallel.Shard(config, world, rank)
        if args.comm == "peer":   # the library's one-shot all-reduce over NVLink peer memory
            comm = parallel.PeerComm(rt, world, rank, rows * config.hidden, device=torch.device("cuda", local), stream=tstream)
        else:
            comm = parallel.TorchComm(world, rank, device=torch.device("cuda", local), stream=tstream)
    weights = synthetic_weights(rt, config, seed=23 + rank, shard=shard)
    norms = synthetic_norms(rt, config)
    decoder = qwen.Decoder(rt, config, weights, norms, batch=rows, capacity=capacity, shard=shard, comm=comm)

    # the prompt: random token ids, fed one position at a time through the decode step
    prompts = np.random.default_rng(29).integers(0, config.vocab, (rows, args.prompt), dtype=np.uint32)
    decoder.reset()
    rt.write(decoder.tokens, prompts[:, 0].copy())
    persistent = world == 1 and rows <= 2 and args.step == "persistent"
    if persistent:          # the whole step as one cooperative kernel
        decoder.compile()
        decoder.run_token()
        rt.sync()
    else:
        decoder.step()      # eager once: sizes every scratch region before recording
        rt.sync()
        decoder.record()
    launches_per_token = decoder.launches_per_token()
    for at in range(1, args.prompt):
        rt.write(decoder.tokens, prompts[:, at].copy())
        decoder.run_token()
    rt.sync()

    # pinned host buffers of the end-to-end path: token ids in, token ids out
    ids_host = torch.zeros(rows, dtype=torch.int32).pin_memory()
    h2d = d2h = rows * 4

    def barrier():
        rt.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput: ids and cursors stay on the device --------------
    for _ in range(warmup):
        decoder.run_token()
    barrier()
    launches0 = rt.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        time.sleep(0.15)
        start.record(tstream)
        for _ in range(args.steps):
            decoder.run_token()
        stop.record(tstream)
        barrier()
        time.sleep(0.15)
    ms = start.elapsed_time(stop)
    launches = rt.launches - launches0
    clock_summary = clocks.summary()

    # ---- end to end: the host loop of Batch::step — write ids, run, read ids ---------------
    rt._lib.neura_cuda_read(rt._ctx, rt.stream, ids_host.data_ptr(), decoder.tokens.ptr, d2h)
    barrier()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(tstream)
    for _ in range(args.steps):
        rt._lib.neura_cuda_write(rt._ctx, rt.stream, decoder.tokens.ptr, ids_host.data_ptr(), h2d)
        decoder.run_token()
        rt._lib.neura_cuda_read(rt._ctx, rt.stream, ids_host.data_ptr(), decoder.tokens.ptr, d2h)
        rt.sync()
    t_stop.record(tstream)
    barrier()
    e2e_ms = t_start.elapsed_time(t_stop)

    # ---- roofline of the dominant kernel (the Q4_K product), timed on its own ----------
    peak, peak_kind = measured_peaks()
    name, n, k = "ffn_gate_up", decoder.feed_forward, config.hidden   # gate and up as one paired product
    rt.stage(decoder.hidden, config.element)
    reps = 4
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rt.capture_begin()
    for layer in range(config.layers):  # 64 different matrices: 5 GB between reuses, L2 holds none of it
        rt.linear_staged(weights[f"blk.{layer}.{name}.weight"], decoder.held)
    sweep = rt.capture_end()
    rt.run(sweep)
    rt.sync()
    r0.record(tstream)
    for _ in range(reps):
        rt.run(sweep)
    r1.record(tstream)
    rt.sync()
    kernel_ms = r0.elapsed_time(r1) / (reps * config.layers)
    algorithmic = 2 * nb.payload_bytes(config.element, n * k) + 4 * rows * k + 4 * rows * n
    achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
    kernel_name = f"qlinear_stream_kernel<Q4_K> on the paired gate|up [2x{n}x{k}] at batch {rows}"
    product_alone = {"kernel": kernel_name, "algorithmic_bytes": algorithmic, "kernel_ms": kernel_ms,
                     "achieved": achieved, "frac": achieved / peak}

    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel from the ncu capture
    # summarised in profiles/decode_step_qwen32b_q4k_kernels.md (the full-size shape, batch 1, one GPU)
    traffic = 163.4e6 if (config.name.startswith("qwen2.5-32b-q4_k") and rows == 1 and world == 1) else None
    if persistent:
        # the step is one kernel: its algorithmic bytes are those of all its products,
        # payload_bytes(N*K) + 4*B*K + 4*B*N each (the KV cache it also reads is left out)
        shapes = [(nn, kk) for _, nn, kk in config.linears()] * config.layers + [(config.vocab, config.hidden)]
        algorithmic = sum(nb.payload_bytes(config.element, nn * kk) + 4 * rows * (nn + kk) for nn, kk in shapes)
        kernel_ms = ms / args.steps
        achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
        kernel_name = (f"decode_megakernel<{'Q4_K' if config.element == nb.Q4K else 'Q8_0'}>: the whole step "
                       f"({config.layers} layers + head) as one cooperative launch at batch {rows}")
        traffic = MEGAKERNEL_TRAFFIC.get((config.name, rows))
    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=torch.device("cuda", local))
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        tokens = rows * args.steps  # the ranks decode the same sequences together
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_description(config, args.prompt, rows,
                                           f"tp{world} ({args.comm} all-reduce)" if world > 1 else "single GPU"),
            "clocks": clock_summary,
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "kernel": kernel_name,
                         "algorithmic_bytes": algorithmic, "kernel_ms": kernel_ms, "product_alone": product_alone,
                         "step_gbs_per_gpu": (shard.local_bytes_per_token() if shard else config.weight_bytes())
                                             / (ms / args.steps * 1e-3) / 1e9,
                         "launches_per_token": launches_per_token},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(config)
        print(json.dumps(line))
    if dist is not None:
        # (no destroy_process_group: with NCCL kernels held in a recorded program it was seen to wait forever)
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_prefill(args):
    """A secondary line: the tensor-core prefill product (Q4_K, bf16 operands, f32 accumulate) on one GPU,
    ``--workload prefill-MxNxK`` (the reference's prefill shape is 2048x18944x3584).  Device timing only."""
    import torch

    import neura_b200 as nb

    m, n, k = (int(v) for v in args.workload.split("-", 1)[1].split("x"))
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    device = torch.device("cuda", 0)
    tstream = torch.cuda.ExternalStream(rt.stream.value, device=device)
    with torch.cuda.stream(tstream):
        numbers = torch.randn(n * k, device=device) * 0.02
        blocks = torch.empty(nb.payload_bytes(nb.Q4K, n * k) + 16, dtype=torch.uint8, device=device)
        rt.quantize_device(nb.Q4K, numbers.data_ptr(), n * k, blocks.data_ptr())
        weight = rt.seal_device(nb.Q4K, n, k, blocks.data_ptr())
        x = torch.randn(m, k, device=device)
        out = torch.empty(m, n, device=device)
    rt.sync()
    xd = nb.DeviceTensor(x.data_ptr(), x.numel() * 4, (m, k))
    od = nb.DeviceTensor(out.data_ptr(), out.numel() * 4, (m, n))
    warmup = max(3, args.warmup)
    for _ in range(warmup):
        rt.linear_bf16(weight, xd, od)
    rt.sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = rt.launches
    with ClockSampler(0) as clocks:
        time.sleep(0.15)
        start.record(tstream)
        for _ in range(args.steps):
            rt.linear_bf16(weight, xd, od)
        stop.record(tstream)
        rt.sync()
        time.sleep(0.15)
    ms = start.elapsed_time(stop) / args.steps
    flops = 2.0 * m * n * k
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = {}
    if os.path.exists(path):
        with open(path) as fh:
            peaks = json.load(fh)
    peak = float(peaks.get("bf16_tflops", 1590.0))
    print(json.dumps({
        "metric": "prefill TFLOP/s (Q4_K weights dequantised to bf16 tiles, tcgen05)", "value": flops / ms / 1e9,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x bf16 -> f32", "data": "synthetic",
        "config": {"workload": f"[{m} x {k}] f32 activations x Q4_K [{n} x {k}]; a step converts the activations to bf16 "
                               "and runs the product", "l2": "weights, activations and output exceed L2 together"},
        "clocks": clocks.summary(), "gpu_launches": int(rt.launches - launches0),
        "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / ms / 1e9 / peak, "traffic": None,
                     "peak_kind": "measured burst" if peaks else "fallback",
                     "kernel": "gemm_q4k_tcgen05_kernel (+ to_bf16_kernel)"},
    }))
    rt.close()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="qwen2.5-32b-q4_k")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--prompt", type=int, default=512)
    parser.add_argument("--comm", default="peer", choices=["peer", "nccl"])
    parser.add_argument("--no-cpu", action="store_true")
    parser.add_argument("--step", default="graph", choices=["graph", "persistent"],
                        help="a recorded graph of one kernel per operation (the faster of the two as measured), or one "
                             "cooperative kernel per token (one GPU, batch <= 2)")
    args = parser.parse_args()
    if args.workload.startswith("prefill-"):
        run_prefill(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
