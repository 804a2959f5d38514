"""Synthetic decoder weights made on the GPU: N(0, 0.02) numbers (torch's generator, used
only as a source of random f32), quantised by the library's device packer and sealed.
The benchmark uses this in place of a GGUF file; the tests use the oracle's packer."""
from __future__ import annotations

from typing import Dict

from .qwen import Config
from .runtime import Runtime, Weight, payload_bytes


def synthetic_weights(rt: Runtime, config: Config, seed: int = 23, deviation: float = 0.02,
                      fuse_qkv: bool = True, with_embedding: bool = True, shard=None) -> Dict[str, Weight]:
    """``shard`` (parallel.Shard): make only that rank's shares, in the shapes a sharded load gives
    (the values are fresh random numbers, not slices of one model: the benchmark needs the bytes)."""
    import torch

    device = torch.device("cuda", rt.device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    stream = torch.cuda.ExternalStream(rt.stream.value, device=device) if rt.stream.value else torch.cuda.current_stream(device)
    shapes = config.linears()
    vocab = config.vocab
    if shard is not None:
        qw, kw = shard.query_width, shard.key_width
        shapes = [("attn_q", qw, config.hidden), ("attn_k", kw, config.hidden), ("attn_v", kw, config.hidden),
                  ("attn_output", config.hidden, shard.window(config.query_width, shard.whole).k),
                  ("ffn_gate", shard.feed_forward, config.hidden), ("ffn_up", shard.feed_forward, config.hidden),
                  ("ffn_down", config.hidden, shard.window(config.feed_forward).k)]
        vocab = shard.vocab
    else:
        qw, kw = config.query_width, config.key_width
    biggest = max(max(n * k for _, n, k in shapes), 16 * 1024 * config.hidden)
    numbers = torch.empty(biggest, dtype=torch.float32, device=device)
    blocks = torch.empty(payload_bytes(config.element, biggest) + 16, dtype=torch.uint8, device=device)
    weights: Dict[str, Weight] = {}

    def make(n: int, k: int, dst=None) -> Weight:
        with torch.cuda.stream(stream):
            view = numbers[: n * k]
            view.normal_(0.0, deviation, generator=gen)
            rt.quantize_device(config.element, view.data_ptr(), n * k, blocks.data_ptr())
            return rt.seal_device(config.element, n, k, blocks.data_ptr(), dst)

    for layer in range(config.layers):
        for name, n, k in shapes:
            if fuse_qkv and name in ("attn_k", "attn_v"):
                continue
            if fuse_qkv and name == "attn_q":
                parts = [qw, kw, kw]
                assert all(p % 32 == 0 for p in parts)
                total = sum(parts)
                base = rt.alloc(rt.sealed_bytes(config.element, total, k))
                at = base
                for p in parts:
                    make(p, k, at)
                    at += rt.sealed_bytes(config.element, p, k)
                weights[f"blk.{layer}.attn_qkv.weight"] = Weight(base, config.element, 1, total, k, at - base)
                continue
            if name == "ffn_gate":   # gate and up sealed as a pair
                with torch.cuda.stream(stream):
                    both = torch.empty(2 * payload_bytes(config.element, n * k) + 32, dtype=torch.uint8, device=device)
                    half = (payload_bytes(config.element, n * k) + 15) // 16 * 16
                    for part in range(2):
                        view = numbers[: n * k]
                        view.normal_(0.0, deviation, generator=gen)
                        rt.quantize_device(config.element, view.data_ptr(), n * k, both.data_ptr() + part * half)
                    weights[f"blk.{layer}.ffn_gate_up.weight"] = rt.seal_pair_device(
                        config.element, n, k, both.data_ptr(), both.data_ptr() + half)
                    rt.sync()
                    del both
                continue
            if name == "ffn_up":
                continue
            weights[f"blk.{layer}.{name}.weight"] = make(n, k)
    # the head in slabs of rows so that the scratch stays small
    k = config.hidden
    total = vocab
    base = rt.alloc(rt.sealed_bytes(config.element, total, k))
    at, done = base, 0
    while done < total:
        rows = min(16 * 1024, total - done)
        make(rows, k, at)
        at += rt.sealed_bytes(config.element, rows, k)
        done += rows
    weights["output.weight"] = Weight(base, config.element, 1, total, k, at - base)
    if with_embedding:
        if config.tied_head and shard is None:
            weights["token_embd.weight"] = weights["output.weight"]
        else:  # a table of its own, kept in GGUF order (only rows are gathered from it)
            total = config.vocab
            row_bytes = payload_bytes(config.element, k)
            table = rt.alloc(row_bytes * total)
            done = 0
            with torch.cuda.stream(stream):
                while done < total:
                    rows = min(16 * 1024, total - done)
                    view = numbers[: rows * k]
                    view.normal_(0.0, deviation, generator=gen)
                    rt.quantize_device(config.element, view.data_ptr(), rows * k, table + done * row_bytes)
                    done += rows
            weights["token_embd.weight"] = Weight(table, config.element, 0, total, k, row_bytes * total)
    rt.sync()
    del numbers, blocks
    return weights


def synthetic_norms(rt: Runtime, config: Config):
    """RMSNorm weights of 1, as a random-init model has them."""
    import numpy as np

    ones = np.ones(config.hidden, dtype=np.float32)
    norms = {}
    names = ["output_norm.weight"]
    for layer in range(config.layers):
        names += [f"blk.{layer}.attn_norm.weight", f"blk.{layer}.ffn_norm.weight"]
    for name in names:
        norms[name] = rt.tensor(config.hidden)
        rt.write(norms[name], ones)
    return norms
