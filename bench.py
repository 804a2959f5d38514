#!/usr/bin/env python
"""Decode throughput of the quantized-linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one greedily decoded token of a random-init Qwen2.5-32B-shaped decoder with Q4_K
projections (64 layers; 17.99 GB of GGUF blocks per token, far larger than L2, so every step
streams them from HBM) after a 512-token random prompt.  Prints ONE JSON line.
With N > 1 (launched under torchrun) the model is split tensor-parallel over the N GPUs: q/k/v, gate, up
and the head by rows, attention output and down by K with one all-reduce each (the library's own
one-shot kernel over NVLink peer memory, or NCCL with --comm nccl).
On one GPU the line also carries `secondary`: the other configurations of the baseline (the Q8_0 product of the
0.5B MLP, the 7B MLP product at batch 1/4/16/64, the 0.5B decoder, the prefill product, decode at batch 16),
each timed in the same process with CUDA events.
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
Q8_0, Q4K = 8, 9
BLOCK = {Q8_0: (32, 34), Q4K: (256, 144)}   # elements and bytes of a block (crates/neura-abi/src/element.rs:33-40,145-178)

# The decoders the baseline's configurations name.  Both arms read the shapes from here; the reference arm
# imports nothing else of this repository but the oracle.
WORKLOADS = {
    "qwen2.5-32b-q4_k": dict(layers=64, hidden=5120, heads=40, key_heads=8, head_width=128, feed_forward=27648,
                             vocab=152064, element=Q4K, tied_head=False),
    "qwen2.5-0.5b-q8_0": dict(layers=24, hidden=896, heads=14, key_heads=2, head_width=64, feed_forward=4864,
                              vocab=151936, element=Q8_0, tied_head=True),
}


def workload_shape(name: str) -> dict:
    """The shape table of a workload; `NAME-<n>l` is the same decoder cut to n layers."""
    if name in WORKLOADS:
        return dict(WORKLOADS[name], name=name)
    base, _, cut = name.rpartition("-")
    if base in WORKLOADS and cut.endswith("l") and cut[:-1].isdigit():
        return dict(WORKLOADS[base], layers=int(cut[:-1]), name=name)
    raise SystemExit(f"unknown workload {name}")


def payload(element: int, elements: int) -> int:
    per, size = BLOCK[element]
    return (elements + per - 1) // per * size


def layer_products(shape: dict):
    """(name, n, k) of the seven projections of a layer, in call order (examples/qwen/attention.rs:106-150, mlp.rs:31-34)."""
    q, kv = shape["heads"] * shape["head_width"], shape["key_heads"] * shape["head_width"]
    h, ff = shape["hidden"], shape["feed_forward"]
    return [("attn_q", q, h), ("attn_k", kv, h), ("attn_v", kv, h), ("attn_output", h, q), ("ffn_gate", ff, h),
            ("ffn_up", ff, h), ("ffn_down", h, ff)]


def weight_elements(shape: dict) -> int:
    return shape["layers"] * sum(n * k for _, n, k in layer_products(shape)) + shape["vocab"] * shape["hidden"]


def workload_description(shape: dict, prompt: int, rows: int, parallelism: str) -> dict:
    """The `config` object of a line: both arms describe the workload the same way."""
    weights = payload(shape["element"], weight_elements(shape))
    return {"workload": f"{shape['name']} decode: {shape['layers']} layers, hidden {shape['hidden']}, "
                        f"{shape['heads']}/{shape['key_heads']} heads x {shape['head_width']}, ff {shape['feed_forward']}, "
                        f"vocab {shape['vocab']}; {prompt}-token random prompt, greedy",
            "batch": rows, "parallelism": parallelism,
            "l2": f"inputs larger than L2 ({weights / 1e9:.2f} GB of weights per step)",
            "weight_bytes_per_token": weights}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def recorded_traffic(key: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised beside this file."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as fh:
        return json.load(fh).get(key)


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


# ---- the CPU arm: the oracle's product over one whole layer at its real shapes ----------------------------------
class CpuLayer:
    """The seven projections of one layer (and the head) of a workload as packed GGUF blocks in host memory, every
    matrix at its real shape and with bytes of its own (274 MB a layer for the 32B shapes: nothing stays in the host
    caches between products), multiplied by the oracle's f32 loop over unpacked blocks on all the host cores.
    The blocks come from one random slab per K, repeated down the rows: the time of a product does not depend on
    the values."""

    def __init__(self, shape: dict):
        import numpy as np
        import oracle

        self.oracle, self.shape, self.element = oracle, shape, shape["element"]
        self.cores = os.cpu_count() or 1
        slabs = {}

        def matrix(n: int, k: int):
            row_bytes = payload(self.element, k)
            if k not in slabs:
                slabs[k] = oracle.pack_rows(self.element, oracle.Stream(23 + k).normal(256 * k, 0.0, 0.02).reshape(256, k))
            return np.tile(slabs[k][: 256 * row_bytes], (n + 255) // 256)[: n * row_bytes].copy()

        self.layer = [(n, k, matrix(n, k)) for _, n, k in layer_products(shape)]
        self.head = (shape["vocab"], shape["hidden"], matrix(shape["vocab"], shape["hidden"]))
        self.x = {k: oracle.Stream(29).normal(k).reshape(1, k) for k in {k for _, k, _ in self.layer} | {shape["hidden"]}}

    def run_layer(self) -> float:
        t0 = time.perf_counter()
        for n, k, packed in self.layer:
            self.oracle.linear(self.element, packed, n, k, self.x[k], threads=self.cores)
        return time.perf_counter() - t0

    def run_head(self) -> float:
        n, k, packed = self.head
        t0 = time.perf_counter()
        self.oracle.linear(self.element, packed, n, k, self.x[k], threads=self.cores)
        return time.perf_counter() - t0

    def token_ms(self, layer_seconds: float, head_seconds: float) -> float:
        return (self.shape["layers"] * layer_seconds + head_seconds) * 1e3

    def describe(self, passes: int) -> dict:
        return {"factor": self.shape["layers"],
                "timed": f"{passes} passes over the seven products of ONE layer at their real shapes and the head once, "
                         f"batch 1, {self.cores} threads",
                "token": "layers x (a layer's time) + the head's time; attention, norms and the cache are left out "
                         "(under 1 % of the weights' bytes)"}


def cpu_baseline(shape: dict, seconds: float = 10.0) -> dict:
    """The in-line CPU figure of our own line: the same code as the reference arm, on a bounded number of passes."""
    cpu = CpuLayer(shape)
    cpu.run_layer()
    head = cpu.run_head()
    spent, passes = 0.0, 0
    while spent < seconds and passes < 256:
        spent += cpu.run_layer()
        passes += 1
    ms = cpu.token_ms(spent / passes, head)
    return {"value": 1e3 / ms, "unit": UNIT, "cores": cpu.cores, "kind": "port", "extrapolated": cpu.describe(passes),
            "sample": f"{passes} layer passes ({spent:.1f} s) of the oracle's product, scaled by the layer count"}


def run_reference(args):
    """The reference has no CPU (or CUDA) implementation of the product; its only executable statement of it is the
    f32 loop of its tests, which the oracle restates.  This arm times that on the host cores: a step is one pass over
    one whole layer's seven products at their real shapes; a token is `layers` such passes and the head."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    shape = workload_shape(args.workload)
    cpu = CpuLayer(shape)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu.run_layer()
    head = cpu.run_head()
    steps = max(1, min(args.steps, 64))   # a bounded sample: a pass over a 32B layer takes a tenth of a second
    spent = sum(cpu.run_layer() for _ in range(steps))
    ms_per_token = cpu.token_ms(spent / steps, head)
    value = 1e3 / ms_per_token
    extrapolated = cpu.describe(steps)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_token, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_description(shape, args.prompt, 1, "host cores"),
        "extrapolated": extrapolated,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.cores, "kind": "port", "extrapolated": extrapolated,
                         "sample": f"{steps} layer passes ({spent:.1f} s) of the oracle's product, scaled by the layer count"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---- our arm -------------------------------------------------------------------------------------------------------
def qwen_config(shape: dict):
    from neura_b200 import qwen

    return qwen.Config(shape["name"], shape["layers"], shape["hidden"], shape["heads"], shape["key_heads"], shape["head_width"],
                       shape["feed_forward"], shape["vocab"], shape["element"], tied_head=shape["tied_head"])


def time_products(rt, torch, tstream, weights, rows: int, k: int, n: int, reps: int = 6):
    """Microseconds per product of `rows` activation rows (staging included) against the sealed weights in turn."""
    import numpy as np

    x, out = rt.tensor(rows, k), rt.tensor(rows, n)
    rt.write(x, np.random.default_rng(5).standard_normal((rows, k)).astype(np.float32))
    rt.reserve(rows, n, k)
    for w in weights:
        rt.linear(w, x, out)
    rt.sync()
    rt.capture_begin()
    for w in weights:
        rt.linear(w, x, out)
    program = rt.capture_end()
    for _ in range(3):
        rt.run(program)
    rt.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(tstream)
    for _ in range(reps):
        rt.run(program)
    e1.record(tstream)
    rt.sync()
    rt.program_free(program)
    rt.free(x.ptr)
    rt.free(out.ptr)
    return e0.elapsed_time(e1) * 1e3 / (reps * len(weights))


def sealed_copies(rt, torch, tstream, device, element: int, n: int, k: int, copies: int):
    import neura_b200 as nb

    made = []
    with torch.cuda.stream(tstream):
        numbers = torch.randn(n * k, device=device) * 0.02
        blocks = torch.empty(nb.payload_bytes(element, n * k) + 16, dtype=torch.uint8, device=device)
        rt.quantize_device(element, numbers.data_ptr(), n * k, blocks.data_ptr())
        for _ in range(copies):
            made.append(rt.seal_device(element, n, k, blocks.data_ptr()))
    rt.sync()
    return made


def secondary_lines(rt, torch, tstream, device, peaks, main_weights, main_norms, main_config, args):
    """The baseline's other configurations, each timed here with CUDA events on the launching stream."""
    import numpy as np

    import neura_b200 as nb
    from neura_b200 import qwen
    from neura_b200.synthetic import synthetic_norms, synthetic_weights

    hbm = float(peaks["hbm_gbs"])
    out = {}
    # config 1: the Q8_0 product of the 0.5B MLP's up projection, batch 1: cold (64 copies, 296 MB between reuses)
    # and resident in L2 (one copy)
    n, k = 4864, 896
    copies = sealed_copies(rt, torch, tstream, device, nb.Q8_0, n, k, 64)
    algorithmic = nb.payload_bytes(nb.Q8_0, n * k) + 4 * (k + n)
    cold = time_products(rt, torch, tstream, copies, 1, k, n)
    warm = time_products(rt, torch, tstream, copies[:1] * 64, 1, k, n)
    out["q8_0_gemv_4864x896_b1"] = {"algorithmic_bytes": algorithmic, "cold_us": cold, "cold_gbs": algorithmic / cold / 1e3,
                                    "cold_frac_of_hbm": algorithmic / cold / 1e3 / hbm, "l2_resident_us": warm,
                                    "l2_resident_gbs": algorithmic / warm / 1e3, "includes": "activation staging"}
    for w in copies:
        rt.free(w.ptr)
    # config 2: the 7B MLP product, Q4_K [18944 x 3584], batch 1 / 4 / 16 / 64, 32 copies (1.2 GB between reuses)
    n, k = 18944, 3584
    copies = sealed_copies(rt, torch, tstream, device, nb.Q4K, n, k, 32)
    sweep = {}
    for rows in (1, 4, 16, 64):
        algorithmic = nb.payload_bytes(nb.Q4K, n * k) + 4 * rows * (k + n)
        us = time_products(rt, torch, tstream, copies, rows, k, n)
        sweep[f"b{rows}"] = {"algorithmic_bytes": algorithmic, "us": us, "gbs": algorithmic / us / 1e3,
                             "frac_of_hbm": algorithmic / us / 1e3 / hbm}
    out["q4_k_product_18944x3584"] = dict(sweep, includes="activation staging",
                                          kernels="qlinear_stream_kernel up to 8 rows, skinny_q4k_tcgen05_kernel above")
    # config 4: the prefill product on the same weights, 2048 rows, bf16 operands
    m = 2048
    x, y = rt.tensor(m, k), rt.tensor(m, n)
    rt.write(x, np.random.default_rng(7).standard_normal((m, k)).astype(np.float32))
    for _ in range(3):
        rt.linear_bf16(copies[0], x, y)
    rt.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(tstream)
    for index in range(16):
        rt.linear_bf16(copies[index % len(copies)], x, y)
    e1.record(tstream)
    rt.sync()
    ms = e0.elapsed_time(e1) / 16
    tflops = 2.0 * m * n * k / ms / 1e9
    out["q4_k_prefill_2048x18944x3584"] = {"ms": ms, "tflops": tflops,
                                           "roofline": {"bound": "tensor", "achieved": tflops, "peak": float(peaks["bf16_tflops"]),
                                                        "unit": "TFLOP/s", "frac": tflops / float(peaks["bf16_tflops"]),
                                                        "kernel": "gemm_q4k_tcgen05_kernel (+ to_bf16_kernel)"}}
    rt.free(x.ptr)
    rt.free(y.ptr)
    for w in copies:
        rt.free(w.ptr)
    # config 5 at batch 16: the same 32B weights, sixteen sequences
    if main_config.name.startswith("qwen2.5-32b-q4_k"):
        rows, steps = 16, 20
        decoder = qwen.Decoder(rt, main_config, main_weights, main_norms, batch=rows, capacity=args.prompt + steps + 16)
        prompts = np.random.default_rng(31).integers(0, main_config.vocab, (rows, args.prompt), dtype=np.uint32)
        decoder.reset()
        decoder.prefill(prompts)
        decoder.step()
        rt.sync()
        decoder.record()
        for _ in range(3):
            decoder.run_token()
        rt.sync()
        e0.record(tstream)
        for _ in range(steps):
            decoder.run_token()
        e1.record(tstream)
        rt.sync()
        ms = e0.elapsed_time(e1) / steps
        out["decode_batch16"] = {"ms_per_step": ms, "tok_s": rows / ms * 1e3, "launches_per_step": decoder.launches_per_token()}
    # the 32B head as common GGUF mixes keep it: Q6_K [152064 x 5120] in GGUF order, batch 1 (639 MB, larger than L2)
    n, k = 152064, 5120
    rng = np.random.default_rng(43)
    blocks = rng.integers(0, 256, (n * (k // 256), 210), dtype=np.uint8)
    blocks[:, 208:210] = rng.uniform(-2e-3, 2e-3, blocks.shape[0]).astype(np.float16).view(np.uint8).reshape(-1, 2)
    head = rt.load(nb.Q6K, n, k, blocks.reshape(-1))
    del blocks
    x, y = rt.tensor(1, k), rt.tensor(1, n)
    rt.write(x, rng.standard_normal((1, k)).astype(np.float32))
    for _ in range(3):
        rt.linear(head, x, y)
    rt.sync()
    e0.record(tstream)
    for _ in range(8):
        rt.linear(head, x, y)
    e1.record(tstream)
    rt.sync()
    us = e0.elapsed_time(e1) / 8 * 1e3
    algorithmic = nb.payload_bytes(nb.Q6K, n * k) + 4 * (k + n)
    out["q6_k_head_152064x5120_b1"] = {"algorithmic_bytes": algorithmic, "us": us, "gbs": algorithmic / us / 1e3,
                                       "frac_of_hbm": algorithmic / us / 1e3 / hbm, "kernel": "qlinear_rows_q6k_kernel (GGUF order)"}
    rt.free(head.ptr)
    rt.free(x.ptr)
    rt.free(y.ptr)
    # config 3: the 0.5B decoder, all projections Q8_0, 128-token prompt, 128 tokens
    shape = workload_shape("qwen2.5-0.5b-q8_0")
    config = qwen_config(shape)
    weights = synthetic_weights(rt, config, seed=41)
    decoder = qwen.Decoder(rt, config, weights, synthetic_norms(rt, config), batch=1, capacity=128 + 128 + 16)
    prompts = np.random.default_rng(37).integers(0, config.vocab, (1, 128), dtype=np.uint32)
    decoder.reset()
    decoder.prefill(prompts)
    decoder.step()
    rt.sync()
    decoder.record()
    for _ in range(3):
        decoder.run_token()
    rt.sync()
    e0.record(tstream)
    for _ in range(124):
        decoder.run_token()
    e1.record(tstream)
    rt.sync()
    ms = e0.elapsed_time(e1) / 124
    out["decode_qwen2.5-0.5b-q8_0"] = {"ms_per_step": ms, "tok_s": 1e3 / ms,
                                       "step_gbs": payload(Q8_0, weight_elements(shape)) / ms / 1e6,
                                       "launches_per_step": decoder.launches_per_token()}
    return out


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

    shape = workload_shape(args.workload)
    config = qwen_config(shape)
    rows = args.batch
    warmup = max(3, args.warmup)
    capacity = args.prompt + 2 * (warmup + args.steps) + 8
    device = torch.device("cuda", local)
    rt = nb.Runtime(local)
    rt.use_stream(rt.new_stream())
    tstream = torch.cuda.ExternalStream(rt.stream.value, device=device)
    shard = comm = None
    if world == 1 and args.rank_of:   # a diagnostic: one rank's share of an N-way split, timed alone without exchanges
        from neura_b200 import parallel

        shard = parallel.Shard(config, args.rank_of, 0, attention=args.attention)
        comm = parallel.NullComm(args.rank_of, 0)
    if world > 1:  # tensor parallel: one model split over the ranks
        from neura_b200 import parallel

        shard = parallel.Shard(config, world, rank, attention=args.attention)
        if args.comm == "peer":   # the library's one-shot all-reduce over NVLink peer memory
            comm = parallel.PeerComm(rt, world, rank, rows * config.hidden, device=device, stream=tstream)
        else:
            comm = parallel.TorchComm(world, rank, device=device, stream=tstream)
    weights = synthetic_weights(rt, config, seed=23 + rank, shard=shard)
    norms = synthetic_norms(rt, config)
    wide = 512 if shard is None and config.element == nb.Q4K else 0   # (rows of a tensor-core prompt chunk)
    decoder = qwen.Decoder(rt, config, weights, norms, batch=rows, capacity=capacity, shard=shard, comm=comm, wide=wide)
    decoder.fold = args.fold == "on"

    # the prompt: random token ids; in chunks where the decoder fills in chunks, else one position at a time
    prompts = np.random.default_rng(29).integers(0, config.vocab, (rows, args.prompt), dtype=np.uint32)
    decoder.reset()
    persistent = rows <= 2 and args.step == "persistent" and ((world == 1 and shard is None) or (world > 1 and args.comm == "peer" and args.attention == "split"))
    prompt_fill = None
    if decoder.chunks:
        fed = args.prompt - 1
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed_fill(through_tensor_cores: bool) -> float:
            for _ in range(2):   # (not timed: the first use of a chunk size makes buffers and loads kernels, the second records its program)
                decoder.prefill(prompts, wide=through_tensor_cores)
                rt.sync()
                decoder.reset()
            p0.record(tstream)
            decoder.prefill(prompts, wide=through_tensor_cores)
            p1.record(tstream)
            rt.sync()
            return p0.elapsed_time(p1)

        tensor_fill = None
        if decoder.wide and decoder.wide_tokens(args.prompt):
            tensor_ms = timed_fill(True)
            decoder.reset()
            tensor_fill = {"tokens": rows * fed, "ms": tensor_ms, "tok_s": rows * fed / tensor_ms * 1e3,
                           "rows_a_chunk": decoder.wide, "tokens_through_bf16": rows * decoder.wide_tokens(args.prompt),
                           "how": "Decoder.prefill(wide=True): the prompt's head through the tcgen05 product with bf16 operands, the chunk a recorded program that is replayed"}
        fill_ms = timed_fill(False)   # the cache the timed decode reads is the one the f32 chunks leave
        prompt_fill = {"tokens": rows * fed, "ms": fill_ms, "tok_s": rows * fed / fill_ms * 1e3,
                       "chunks": list(decoder.chunks), "how": "Decoder.prefill(wide=False): one chunk after another, each chunk size a recorded program that is replayed",
                       "tensor_cores": tensor_fill}
    else:
        rt.write(decoder.tokens, prompts[:, 0].copy())
        fed = 0
    if persistent:          # the whole step as one cooperative kernel
        decoder.compile()
        decoder.run_token()
        rt.sync()
    else:
        decoder.step()      # eager once: sizes every scratch region before recording
        rt.sync()
        decoder.record()
    launches_per_token = decoder.launches_per_token()
    for at in range(fed + 1, args.prompt):
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

    # ---- roofline of the dominant kernel (the streaming product on the paired gate|up), timed on its own ----------
    peaks, peak_kind = measured_peaks()
    peak = float(peaks["hbm_gbs"])
    name, n, k = "ffn_gate_up", decoder.feed_forward, config.hidden   # gate and up as one paired product
    rt.staging_select(0)
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
    tag = "Q4_K" if config.element == nb.Q4K else "Q8_0"
    kernel_key = f"qlinear_stream_kernel<{tag}> gate|up [2x{n}x{k}] b{rows}"
    kernel_name = f"qlinear_stream_kernel<{tag}> on the paired gate|up [2x{n}x{k}] at batch {rows}"
    product_alone = {"kernel": kernel_name, "algorithmic_bytes": algorithmic, "kernel_ms": kernel_ms,
                     "achieved": achieved, "frac": achieved / peak}
    traffic = recorded_traffic(kernel_key) if world == 1 and shard is None else None
    if persistent:
        # the step is one kernel: its algorithmic bytes are those of all its products,
        # payload_bytes(N*K) + 4*B*K + 4*B*N each (the KV cache it also reads is left out)
        shapes = [(nn, kk) for _, nn, kk in config.linears()] * config.layers + [(config.vocab, config.hidden)]
        algorithmic = sum(nb.payload_bytes(config.element, nn * kk) + 4 * rows * (nn + kk) for nn, kk in shapes)
        if shard is not None:   # a rank streams its shares only
            algorithmic = shard.local_bytes_per_token()
        kernel_ms = ms / args.steps
        achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
        kernel_name = f"decode_megakernel<{tag}>: the whole step ({config.layers} layers + head) as one cooperative launch at batch {rows}"
        traffic = recorded_traffic(f"decode_megakernel<{tag}> {config.name} b{rows}") if shard is None else None
    secondary = None
    if world == 1 and shard is None and not persistent and not args.no_secondary and rows == 1:
        secondary = secondary_lines(rt, torch, tstream, device, peaks, weights, norms, config, args)
    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        tokens = rows * args.steps  # the ranks decode the same sequences together
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_description(shape, args.prompt, rows,
                                           f"tp{world} ({args.comm} all-reduce; " + ("MLP and head split, attention whole on every rank" if args.attention == "whole" else "attention, MLP and head split") + ")" if world > 1 else "single GPU"),
            "clocks": clock_summary,
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "traffic_source": "an ncu capture of this kernel, recorded in profiles/traffic.json (not measured live)"
                                           if traffic else None,
                         "peak_kind": peak_kind,
                         "kernel": kernel_name,
                         "algorithmic_bytes": algorithmic, "kernel_ms": kernel_ms, "product_alone": product_alone,
                         "step_gbs_per_gpu": (shard.local_bytes_per_token() if shard else config.weight_bytes())
                                             / (ms / args.steps * 1e-3) / 1e9,
                         "launches_per_token": launches_per_token},
        }
        if secondary is not None:
            line["secondary"] = secondary
        if prompt_fill is not None:
            line["prompt_fill"] = prompt_fill
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(shape)
        print(json.dumps(line))
    if dist is not None:
        # (no destroy_process_group: with NCCL kernels held in a recorded program it was seen to wait forever)
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_prefill(args):
    """A line of its own for the tensor-core prefill product (Q4_K, bf16 operands, f32 accumulate) on one GPU,
    ``--workload prefill-MxNxK`` (the baseline's prefill shape is 2048x18944x3584).  Device timing only."""
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
    peaks, kind = measured_peaks()
    peak = float(peaks["bf16_tflops"])
    print(json.dumps({
        "metric": "prefill TFLOP/s (Q4_K weights dequantised to bf16 tiles, tcgen05)", "value": flops / ms / 1e9,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x bf16 -> f32", "data": "synthetic",
        "config": {"workload": f"[{m} x {k}] f32 activations x Q4_K [{n} x {k}]; a step converts the activations to bf16 "
                               "and runs the product", "l2": "weights, activations and output exceed L2 together"},
        "clocks": clocks.summary(), "gpu_launches": int(rt.launches - launches0),
        "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / ms / 1e9 / peak, "traffic": None,
                     "peak_kind": "measured burst" if kind == "measured" else "fallback",
                     "kernel": "gemm_q4k_tcgen05_kernel (+ to_bf16_kernel)"},
    }))
    rt.close()


def run_product(args):
    """A line of its own for ONE product shape on one GPU, ``--workload product-q4_k-NxK-bB`` (or ``q8_0``): B rows of
    f32 activations against a sealed [N x K] weight, staging included; a step walks as many copies of the weight as
    make 1.2 GB, so every launch streams its weight from HBM.  Device timing only."""
    import torch

    import neura_b200 as nb

    _, kind, shape, batch = args.workload.split("-")
    element = {"q4_k": nb.Q4K, "q8_0": nb.Q8_0}[kind]
    n, k = (int(v) for v in shape.split("x"))
    rows = int(batch.lstrip("b"))
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    device = torch.device("cuda", 0)
    tstream = torch.cuda.ExternalStream(rt.stream.value, device=device)
    copies = sealed_copies(rt, torch, tstream, device, element, n, k, max(2, min(64, int(1.2e9 // nb.payload_bytes(element, n * k)))))
    warmup = max(3, args.warmup)
    launches0 = rt.launches
    with ClockSampler(0) as clocks:
        us = time_products(rt, torch, tstream, copies, rows, k, n, reps=max(1, args.steps))
    peaks, peak_kind = measured_peaks()
    algorithmic = nb.payload_bytes(element, n * k) + 4 * rows * (k + n)
    achieved = algorithmic / us / 1e3
    kernel = "skinny_q4k_tcgen05_kernel (+ skinny_prep_kernel)" if element == nb.Q4K and rows > 8 else "qlinear_stream_kernel (+ prep_kernel)"
    print(json.dumps({
        "metric": "product GB/s of algorithmic bytes", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": us * len(copies) / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{rows} rows x {kind} [{n} x {k}], {len(copies)} copies of the weight in turn",
                   "l2": "the copies exceed L2 together", "us_per_product": us},
        "clocks": clocks.summary(), "gpu_launches": int(rt.launches - launches0),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                     "frac": achieved / float(peaks["hbm_gbs"]), "traffic": None, "peak_kind": peak_kind, "kernel": kernel,
                     "algorithmic_bytes": algorithmic},
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
    parser.add_argument("--no-secondary", action="store_true", help="skip the other configurations of the baseline")
    parser.add_argument("--fold", default="off", choices=["on", "off"],
                        help="fold norms, stagings and (tensor parallel) exchanges into the products' epilogues: fewer, "
                             "longer launches (measured slower at every split, so off)")
    parser.add_argument("--attention", default="whole", choices=["whole", "split"],
                        help="tensor parallel: every rank keeps the whole attention block and only the MLP and the head are "
                             "split (one exchange a layer; the faster split as measured), or the attention block is split by heads "
                             "as well (two exchanges a layer)")
    parser.add_argument("--rank-of", type=int, default=0,
                        help="diagnostic, one GPU: time rank 0's share of a split over this many ranks, no exchanges")
    parser.add_argument("--step", default="graph", choices=["graph", "persistent"],
                        help="a recorded graph of one kernel per operation (the faster of the two as measured), or one "
                             "cooperative kernel per token (one GPU, batch <= 2)")
    args = parser.parse_args()
    if args.workload.startswith("prefill-"):
        run_prefill(args)
    elif args.workload.startswith("product-"):
        run_product(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
