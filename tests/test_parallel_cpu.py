"""The tensor-parallel split on the CPU: shard arithmetic, GGUF slicing, and the two exchanges
over a world of 2 gloo ranks (no GPU needed)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shares_partition_rows_and_cover_k_in_whole_blocks():
    from neura_b200 import parallel, qwen

    c = qwen.QWEN25_32B_Q4K
    for world in (1, 2, 4, 8):
        covered = []
        for rank in range(world):
            s = parallel.Shard(c, world, rank)
            assert s.heads * world == c.heads and s.key_heads * world == c.key_heads
            assert s.rows(c.feed_forward) == (rank * c.feed_forward // world, (rank + 1) * c.feed_forward // world)
            w = s.window(c.feed_forward)
            assert w.k % 256 == 0 and w.lo % 64 == 0 and w.hi - w.lo == c.feed_forward // world
            covered.append((w.first_block * 256 + w.lo, w.first_block * 256 + w.hi))
        assert covered[0][0] == 0 and covered[-1][1] == c.feed_forward
        assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    # at 8 ranks a share of the attention output's K is 2.5 super-blocks: both neighbours keep the straddled one
    a, b = parallel.Shard(c, 8, 0).window(c.query_width), parallel.Shard(c, 8, 1).window(c.query_width)
    assert (a.k, a.lo, a.hi, a.first_block) == (768, 0, 640, 0)
    assert (b.k, b.lo, b.hi, b.first_block) == (768, 128, 768, 2)
    assert sum(parallel.Shard(c, 1, 0).local_bytes_per_token() for _ in range(1)) == c.weight_bytes()
    with pytest.raises(ValueError):
        parallel.Shard(qwen.QWEN25_05B_Q8, 4, 0)   # 14 query heads over 2 key heads do not split in 4


def test_a_group_may_keep_the_attention_block_whole():
    from neura_b200 import parallel, qwen

    c = qwen.QWEN25_32B_Q4K
    for world in (2, 4, 8):
        s = parallel.Shard(c, world, 1, attention="whole")
        assert (s.heads, s.key_heads, s.query_width) == (c.heads, c.key_heads, c.query_width)   # every head on every rank
        assert s.rows(c.query_width, whole=True) == (0, c.query_width)
        w = s.window(c.query_width, whole=True)
        assert (w.k, w.lo, w.hi, w.first_block) == (c.query_width, 0, c.query_width, 0)
        assert s.feed_forward == c.feed_forward // world and s.vocab == c.vocab // world      # the MLP and the head are split
        split = parallel.Shard(c, world, 1)
        assert s.local_bytes_per_token() > split.local_bytes_per_token()
    # the heads need not divide by the ranks when the attention stays whole: 14 query heads over 2 key heads on 4 ranks
    small = qwen.Config("whole-tp", 2, 896, 14, 2, 64, 4864, 151936, qwen.Q8_0)
    assert parallel.Shard(small, 4, 3, attention="whole").heads == 14
    with pytest.raises(ValueError):
        parallel.Shard(c, 2, 0, attention="some")


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle
    from neura_b200 import parallel, qwen

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    config = qwen.Config("tp-cpu", 1, 512, 4, 2, 128, 768, 256, oracle.Q4K)
    shard = parallel.Shard(config, world, rank)
    n, k = config.hidden, config.feed_forward           # the down projection: split along K (1.5 super-blocks each)
    w = oracle.Stream(23).normal(n * k, 0.0, 0.02).reshape(n, k)
    packed = oracle.pack_rows(config.element, w)
    x = oracle.Stream(29).normal(2 * k).reshape(2, k)
    full = oracle.linear(config.element, packed, n, k, x)
    window = shard.window(k)
    local = np.zeros((2, window.k), dtype=np.float32)
    share = k // world
    local[:, window.lo: window.hi] = x[:, rank * share: (rank + 1) * share]
    partial = torch.from_numpy(oracle.linear(config.element, shard.slice_columns(packed, n, k), n, window.k, local))
    dist.all_reduce(partial)
    row_ok = float(np.abs(partial.numpy() - full).max()) <= 1e-3 * float(np.sqrt(np.mean(full ** 2)))
    # the gate projection: split along its rows, shares gathered side by side
    n2, k2 = config.feed_forward, config.hidden
    w2 = oracle.Stream(31).normal(n2 * k2, 0.0, 0.02).reshape(n2, k2)
    packed2 = oracle.pack_rows(config.element, w2)
    x2 = oracle.Stream(37).normal(k2).reshape(1, k2)
    full2 = oracle.linear(config.element, packed2, n2, k2, x2)
    mine = torch.from_numpy(oracle.linear(config.element, shard.slice_rows(packed2, n2, k2), n2 // world, k2, x2))
    gathered = torch.empty(world * (n2 // world))
    dist.all_gather_into_tensor(gathered, mine.reshape(-1))
    col_ok = np.array_equal(gathered.numpy().reshape(-1).view(np.uint32), full2.reshape(-1).view(np.uint32))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write(f"{int(row_ok)} {int(col_ok)}")
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_device_products(tmp_path):
    import torch.multiprocessing as mp

    world, port = 2, 29611 + os.getpid() % 200
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        row_ok, col_ok = open(tmp_path / f"rank{rank}.txt").read().split()
        assert row_ok == "1", "the all-reduced K shares leave the single-device product"
        assert col_ok == "1", "the gathered row shares are not the single-device product bit for bit"


def test_the_decoder_and_the_oracle_stepper_agree_on_what_goes_through_the_wide_path():
    # the head of a prompt that goes through the tensor-core chunks: all but the last token, in chunks of `wide`, unless
    # fewer than WIDE_FROM tokens would be left for the last wide chunk (those take the ordinary chunks)
    import types

    from neura_b200.qwen import Decoder
    from oracle.decoder import OracleDecoder

    for wide, start in ((0, 64), (512, 64), (128, 64), (8, 5), (100, 64)):
        one = types.SimpleNamespace(wide=wide, WIDE_FROM=start)
        for length in (1, 2, 5, 13, 64, 65, 66, 129, 150, 200, 330, 512, 513, 700):
            got = Decoder.wide_tokens(one, length)
            assert got == OracleDecoder.wide_tokens(one, length)
            fed = length - 1
            if not wide or fed < start:
                assert got == 0
            else:
                assert got in (fed, fed - fed % wide) and (fed - got == 0 or fed - got < start)
