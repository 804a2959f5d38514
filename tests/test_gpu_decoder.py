"""The decoder step and its parts against the CPU oracle (needs a B200)."""
import dataclasses

import numpy as np
import pytest

import neura_b200 as nb
from neura_b200 import qwen

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_embedding_rows_are_the_dequantised_table_rows(runtime, oracle):
    for element, width in ((nb.Q8_0, 896), (nb.Q4K, 1024)):
        vocab = 320
        table = oracle.Stream(3).normal(vocab * width, 0.0, 0.02).reshape(vocab, width)
        packed = oracle.pack_rows(element, table)
        tokens = np.array([0, 5, 319, 64, 5], dtype=np.uint32)
        expected = oracle.embed(element, packed, width, tokens)
        tok = runtime.tensor_u32(tokens.size)
        runtime.write(tok, tokens)
        out = runtime.tensor(tokens.size, width)
        for seal in (False, True):
            runtime.embed(runtime.load(element, vocab, width, packed, seal=seal), tok, out)
            assert np.array_equal(bits(runtime.read(out)), bits(expected))


def test_rms_norm_matches_and_its_staging_feeds_the_product(runtime, oracle):
    rows, k, n = 3, 1024, 96
    x = oracle.Stream(5).normal(rows * k).reshape(rows, k) * 3.0
    weight = oracle.Stream(6).uniform(k, 0.5, 1.5)
    expected = oracle.rms_norm(x, weight, 1e-6)
    xd, wd, nd = runtime.tensor(rows, k), runtime.tensor(k), runtime.tensor(rows, k)
    runtime.write(xd, x)
    runtime.write(wd, weight)
    w = oracle.Stream(7).normal(n * k, 0.0, 0.02).reshape(n, k)
    for element in (nb.Q4K, nb.Q8_0):
        packed = oracle.pack_rows(element, w)
        runtime.rms_norm_stage(xd, wd, 1e-6, element, normed=nd)
        assert np.abs(runtime.read(nd) - expected).max() <= 2e-6 * np.abs(expected).max()
        out = runtime.tensor(rows, n)
        runtime.linear_staged(runtime.load(element, n, k, packed), out)
        want = oracle.linear(element, packed, n, k, expected)
        assert np.abs(runtime.read(out) - want).max() <= 1e-3 * np.sqrt(np.mean(want ** 2))


def test_rope_and_cache_write(runtime, oracle):
    batch, heads, key_heads, width, capacity = 3, 4, 2, 64, 32
    row = (heads + 2 * key_heads) * width
    qkv = oracle.Stream(8).normal(batch * row).reshape(batch, row)
    position = np.array([0, 7, 31], dtype=np.uint32)
    qd, pd = runtime.tensor(batch, row), runtime.tensor_u32(batch)
    keys = runtime.tensor(batch * key_heads * capacity * width)
    values = runtime.tensor(batch * key_heads * capacity * width)
    runtime.write(qd, qkv)
    runtime.write(pd, position)
    runtime.write(keys, np.zeros(keys.shape, np.float32))
    runtime.write(values, np.zeros(values.shape, np.float32))
    runtime.rope_cache(qd, pd, 1e6, heads, key_heads, width, capacity, keys, values)
    got = runtime.read(qd)
    q = oracle.rope(qkv[:, : heads * width].reshape(batch, heads, width), position, 1e6)
    k = oracle.rope(qkv[:, heads * width: (heads + key_heads) * width].reshape(batch, key_heads, width), position, 1e6)
    assert np.abs(got[:, : heads * width] - q.reshape(batch, -1)).max() <= 2e-5
    assert np.abs(got[:, heads * width: (heads + key_heads) * width] - k.reshape(batch, -1)).max() <= 2e-5
    kc = runtime.read(keys).reshape(batch, key_heads, capacity, width)
    vc = runtime.read(values).reshape(batch, key_heads, capacity, width)
    v = qkv[:, (heads + key_heads) * width:].reshape(batch, key_heads, width)
    for b in range(batch):
        assert np.abs(kc[b, :, position[b]] - k[b]).max() <= 2e-5
        assert np.array_equal(bits(vc[b, :, position[b]]), bits(v[b]))
        untouched = np.delete(kc[b], position[b], axis=1)
        assert not untouched.any()


@pytest.mark.parametrize("heads,key_heads,width,capacity,positions", [
    (6, 2, 64, 96, (0, 70)),        # two splits in one cluster
    (10, 2, 128, 600, (599, 301)),  # five splits of 128 in one cluster
    (4, 4, 128, 1100, (1099, 5)),   # nine splits: merged through global memory
])
def test_attention_over_the_cache(runtime, oracle, heads, key_heads, width, capacity, positions):
    batch = 2
    q = oracle.Stream(9).normal(batch * heads * width).reshape(batch, heads, width)
    keys = oracle.Stream(10).normal(batch * key_heads * capacity * width).reshape(batch, key_heads, capacity, width)
    values = oracle.Stream(11).normal(keys.size).reshape(keys.shape)
    position = np.array(positions, dtype=np.uint32)
    expected = oracle.attend(q, keys, values, position + 1, 0.125)
    qd, out = runtime.tensor(batch, heads * width), runtime.tensor(batch, heads * width)
    kd, vd, pd = runtime.tensor(keys.size), runtime.tensor(values.size), runtime.tensor_u32(batch)
    runtime.write(qd, q.reshape(batch, -1))
    runtime.write(kd, keys.reshape(-1))
    runtime.write(vd, values.reshape(-1))
    runtime.write(pd, position)
    runtime.attend(qd, kd, vd, pd, 0.125, heads, key_heads, width, capacity, out)
    assert np.abs(runtime.read(out) - expected.reshape(batch, -1)).max() <= 1e-5


def test_attention_of_many_sequences_takes_the_small_tiles(runtime, oracle):
    # 20 sequences x 8 key heads x two 128-position tiles are more tiles than the GPU has SMs: the launcher then takes
    # tiles of 64 positions (three CTAs an SM) and merges the splits through global memory
    batch, heads, key_heads, width, capacity = 20, 16, 8, 128, 200
    q = oracle.Stream(19).normal(batch * heads * width).reshape(batch, heads, width)
    keys = oracle.Stream(20).normal(batch * key_heads * capacity * width).reshape(batch, key_heads, capacity, width)
    values = oracle.Stream(21).normal(keys.size).reshape(keys.shape)
    position = (np.arange(batch, dtype=np.uint32) * 37 + 3) % capacity
    expected = oracle.attend(q, keys, values, position + 1, 0.125)
    qd, out = runtime.tensor(batch, heads * width), runtime.tensor(batch, heads * width)
    kd, vd, pd = runtime.tensor(keys.size), runtime.tensor(values.size), runtime.tensor_u32(batch)
    runtime.write(qd, q.reshape(batch, -1))
    runtime.write(kd, keys.reshape(-1))
    runtime.write(vd, values.reshape(-1))
    runtime.write(pd, position)
    runtime.attend(qd, kd, vd, pd, 0.125, heads, key_heads, width, capacity, out)
    assert np.abs(runtime.read(out) - expected.reshape(batch, -1)).max() <= 1e-5


@pytest.mark.parametrize("rows,heads,key_heads,width,capacity,start", [
    (64, 8, 2, 128, 96, 0), (100, 40, 8, 128, 200, 37), (511, 10, 2, 128, 640, 0), (77, 14, 2, 64, 130, 50), (130, 16, 2, 64, 140, 3)])
def test_attention_of_a_wide_prompt_chunk_matches_the_oracle(runtime, oracle, rows, heads, key_heads, width, capacity, start):
    # 64 rows and more of one sequence: blocks of 16 rows walk the cache tile by tile with a running softmax; row r sees the
    # positions up to its own cursor start + r (the last block is ragged, the last tile of a block partly masked)
    q = oracle.Stream(51).normal(rows * heads * width).reshape(rows, heads, width)
    keys = oracle.Stream(52).normal(key_heads * capacity * width).reshape(1, key_heads, capacity, width)
    values = oracle.Stream(53).normal(keys.size).reshape(keys.shape)
    position = np.minimum(start + np.arange(rows, dtype=np.uint32), capacity - 1).astype(np.uint32)
    expected = np.concatenate([oracle.attend(q[r: r + 1], keys, values, position[r: r + 1] + 1, 0.09) for r in range(rows)])
    stride = heads * width + 2 * key_heads * width   # the queries sit at the head of q|k|v rows
    rowsd = np.zeros((rows, stride), dtype=np.float32)
    rowsd[:, : heads * width] = q.reshape(rows, -1)
    qd, out = runtime.tensor(rows, stride), runtime.tensor(rows, heads * width)
    kd, vd, pd = runtime.tensor(keys.size), runtime.tensor(values.size), runtime.tensor_u32(rows)
    runtime.write(qd, rowsd)
    runtime.write(kd, keys.reshape(-1))
    runtime.write(vd, values.reshape(-1))
    runtime.write(pd, position)
    runtime.attend_rows(qd, kd.ptr, vd.ptr, pd, 0.09, rows, heads, key_heads, width, capacity, out)
    assert np.abs(runtime.read(out) - expected.reshape(rows, -1)).max() <= 1e-5


def test_argmax_takes_the_lowest_index_on_ties(runtime, oracle):
    x = oracle.Stream(12).normal(3 * 5000).reshape(3, 5000)
    x[0, 4000] = x[0, 17] = 9.0
    x[1, 4999] = 8.0
    x[2] = -1.0
    xd, out = runtime.tensor(3, 5000), runtime.tensor_u32(3)
    runtime.write(xd, x)
    runtime.argmax(xd, out)
    assert list(runtime.read(out, dtype=np.uint32)) == [17, 4999, 0]
    assert list(oracle.argmax(x)) == [17, 4999, 0]


def load_model(rt, config, packed, norms):
    from neura_b200.parallel import load_decoder_weights

    return load_decoder_weights(rt, config, packed, norms)


SMALL = {
    "q8_0": qwen.Config("tiny-q8_0", 2, 896, 14, 2, 64, 4864, 2048, nb.Q8_0, tied_head=True),
    "q4_k": qwen.Config("tiny-q4_k", 2, 1024, 8, 2, 128, 2816, 2048, nb.Q4K),
}


@pytest.mark.parametrize("name,batch", [("q8_0", 1), ("q4_k", 1), ("q4_k", 3), ("q4_k-folded", 2), ("q8_0-folded", 1)])
def test_greedy_tokens_match_the_oracle_for_64_steps(oracle, name, batch):
    from oracle.decoder import OracleDecoder, synthetic_model

    name, _, folded = name.partition("-")   # "-folded": norms and stagings in the products' epilogues
    config = SMALL[name]
    packed, norms = synthetic_model(config, seed=23)
    prompts = (oracle.Stream(29).uniform(batch * 16, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(batch, 16)
    want, margins = OracleDecoder(config, packed, norms, batch=batch, capacity=96).generate(prompts, 64)
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=batch, capacity=96)
        decoder.fold = bool(folded)
        assert decoder.folded() == bool(folded)
        eager = decoder.generate(prompts, 64)
        decoder.record()
        replayed = decoder.generate(prompts, 64)
    finally:
        rt.close()
    assert np.array_equal(eager, replayed), "a recorded step decodes what the eager step decodes"
    differs = np.argwhere(eager != want)
    if differs.size:
        b, at = differs[0]
        pytest.fail(f"sequence {b} leaves the oracle at step {at}: {eager[b, at]} for {want[b, at]}, "
                    f"the oracle's margin there is {margins[b, at]:.3e}")


@pytest.mark.parametrize("name,batch,length", [("q4_k", 1, 45), ("q4_k", 2, 70), ("q4_k", 1, 110), ("q8_0", 1, 45), ("q8_0", 3, 21)])
def test_a_prompt_fed_in_chunks_decodes_what_the_oracle_decodes(oracle, name, batch, length):
    # Batch::prefill (crates/neura-generate/src/batch.rs:1595-1599): chunks of 32 and 8 (16 and 8 for Q8_0), the rest alone.
    # (70 tokens: the second chunk of 32 is recorded and replayed; 110 tokens: the third replays the recorded program)
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL[name]
    packed, norms = synthetic_model(config, seed=23)
    prompts = (oracle.Stream(43).uniform(batch * length, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(batch, length)
    want, margins = OracleDecoder(config, packed, norms, batch=batch, capacity=length + 40).generate(prompts, 32)
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=batch, capacity=length + 40)
        decoder.record()
        launches = rt.launches
        one_by_one = decoder.generate(prompts, 32)
        stepped, launches = rt.launches - launches, rt.launches
        chunked = decoder.generate(prompts, 32, chunked=True)
        fed = rt.launches - launches
        decoder.release()   # the step's and the chunks' programs go back; the decoder steps eagerly from here on
        assert decoder.program is None and np.array_equal(decoder.generate(prompts, 4, chunked=True), chunked[:, :4])
    finally:
        rt.close()
    assert fed < stepped, "the chunks take fewer launches than the tokens one by one"
    assert np.array_equal(chunked, one_by_one), "a prompt fed in chunks leaves the cache the decode steps leave"
    differs = np.argwhere(chunked != want)
    if differs.size:
        b, at = differs[0]
        pytest.fail(f"sequence {b} leaves the oracle at step {at}: {chunked[b, at]} for {want[b, at]}, "
                    f"the oracle's margin there is {margins[b, at]:.3e}")


@pytest.mark.parametrize("rows,k,stride", [(1, 896, 896), (70, 1024, 1024), (300, 5120, 5200)])
def test_rms_norm_of_many_rows_matches_the_oracle(oracle, rows, k, stride):
    x = oracle.Stream(83).normal(rows * stride).reshape(rows, stride).astype(np.float32)
    gain = oracle.Stream(85).uniform(k, 0.5, 1.5).astype(np.float32)
    want = oracle.rms_norm(np.ascontiguousarray(x[:, :k]), gain, 1e-6)
    with nb.Runtime(0) as rt:
        xd, gd, od = rt.tensor(rows, stride), rt.tensor(k), rt.tensor(rows, stride)
        rt.write(xd, x)
        rt.write(gd, gain)
        rt.write(od, np.zeros((rows, stride), dtype=np.float32))
        rt.rms_norm(xd, gd, 1e-6, od, k=k)
        got = rt.read(od).reshape(rows, stride)
    assert np.abs(got[:, :k] - want).max() <= 1e-5 * np.abs(want).max()
    assert not got[:, k:].any(), "the columns past k stay as they were"


@pytest.mark.parametrize("batch,length,wide", [(1, 200, 128), (2, 150, 128), (1, 330, 512)])
def test_a_prompt_fed_through_the_tensor_cores_decodes_what_the_oracle_decodes(oracle, batch, length, wide):
    # the head of the prompt in chunks of up to `wide` rows through the bf16 product (200: 128 + 71 rows; 150: 128 rows,
    # then 21 tokens through the f32 chunks; 330: one chunk of 329 rows); the oracle rounds the same products' operands
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL["q4_k"]
    packed, norms = synthetic_model(config, seed=23)
    prompts = (oracle.Stream(47).uniform(batch * length, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(batch, length)
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=batch, capacity=length + 72, wide=wide)
        through = decoder.wide_tokens(length)
        decoder.record()
        got = decoder.generate(prompts, 64, chunked=True)
        again = decoder.generate(prompts, 64, chunked=True)
    finally:
        rt.close()
    assert through == {200: 199, 150: 128, 330: 329}[length]
    want, margins = OracleDecoder(config, packed, norms, batch=batch, capacity=length + 72).generate(prompts, 64, bf16_tokens=through)
    assert np.array_equal(got, again), "the same prompt fills the cache the same way twice"
    differs = np.argwhere(got != want)
    if differs.size:
        b, at = differs[0]
        pytest.fail(f"sequence {b} leaves the oracle at step {at}: {got[b, at]} for {want[b, at]}, "
                    f"the oracle's margin there is {margins[b, at]:.3e}")


def test_a_decoder_read_from_a_gguf_file_decodes_what_the_poured_tensors_decode(oracle, tmp_path):
    from neura_b200 import gguf
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL["q4_k"]
    packed, norms = synthetic_model(config, seed=23)
    norms["blk.1.attn_norm.weight"] = oracle.Stream(4).uniform(config.hidden, 0.5, 1.5)
    path = tmp_path / "tiny.gguf"
    path.write_bytes(gguf.write_decoder(config, packed, norms))
    prompts = (oracle.Stream(31).uniform(8, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(1, 8)
    want, margins = OracleDecoder(config, packed, norms, batch=1, capacity=48).generate(prompts, 32)
    rt = nb.Runtime(0)
    try:
        decoder = qwen.Decoder.from_gguf(rt, str(path), batch=1, capacity=48)
        assert decoder.config == dataclasses.replace(config, floor=float(np.float32(config.floor)))  # stored as f32
        got = decoder.generate(prompts, 32)
    finally:
        rt.close()
    assert np.array_equal(got, want), f"smallest oracle margin {margins.min():.3e}"


def test_continuous_batching_decodes_each_sequence_as_the_oracle_decodes_it_alone(oracle):
    from neura_b200.generate import Batch
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL["q8_0"]
    packed, norms = synthetic_model(config, seed=23)
    draws = (oracle.Stream(37).uniform(24, 0.0, 1.0) * config.vocab).astype(np.uint32)
    prompts = [list(draws[:9]), list(draws[9:10]), list(draws[10:16]), list(draws[16:24])]
    steps = 12
    alone = [OracleDecoder(config, packed, norms, batch=1, capacity=40).generate(np.array([p]), steps)[0][0].tolist()
             for p in prompts]
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=3, capacity=40)
        decoder.record()
        batch = Batch(decoder)
        got = {i: [] for i in range(len(prompts))}
        plane, waiting = {}, list(range(len(prompts)))
        for _ in range(3):
            index = waiting.pop(0)
            plane[batch.admit(prompts[index])] = index
            for slot, token in batch.step():  # every sequence joins a step after the one before it
                got[plane[slot]].append(token)
        for _ in range(200):
            for slot, token in batch.step():
                got[plane[slot]].append(token)
            for slot in list(batch.occupied()):
                if len(got[plane[slot]]) >= steps:
                    batch.finish(slot)
                    if waiting:
                        index = waiting.pop(0)
                        plane[batch.admit(prompts[index])] = index
            if not list(batch.occupied()):
                break
    finally:
        rt.close()
    assert [got[i][:steps] for i in range(len(prompts))] == alone


def test_continuous_batching_feeds_a_long_prompt_through_the_tensor_cores(oracle):
    # Batch::prefill over a decoder built with wide rows: the long prompt's head goes through fill_wide (100 of its 120
    # tokens in one chunk; the 19 left in chunks of 8 and alone), the short prompt through the f32 chunks only
    from neura_b200.generate import Batch
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL["q4_k"]
    packed, norms = synthetic_model(config, seed=23)
    draws = (oracle.Stream(39).uniform(160, 0.0, 1.0) * config.vocab).astype(np.uint32)
    prompts = [list(draws[:120]), list(draws[120:160])]
    steps = 16
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=2, capacity=160, wide=100)
        through = [decoder.wide_tokens(len(p)) for p in prompts]
        decoder.record()
        batch = Batch(decoder)
        plane = {batch.admit(p): i for i, p in enumerate(prompts)}
        got = {0: [], 1: []}
        for _ in range(60):
            for slot, token in batch.step():
                got[plane[slot]].append(token)
            if min(len(tokens) for tokens in got.values()) >= steps:
                break
    finally:
        rt.close()
    assert through == [100, 0]
    alone = [OracleDecoder(config, packed, norms, batch=1, capacity=160).generate(np.array([p]), steps, bf16_tokens=t)[0][0].tolist()
             for p, t in zip(prompts, through)]
    assert [got[i][:steps] for i in range(2)] == alone


def test_the_whole_half_billion_decoder_decodes_the_golden_tokens(oracle):
    """Qwen2.5-0.5B shapes, every projection Q8_0, tied head: 128 prompt tokens, 128 greedy tokens,
    against the ids the CPU oracle decoded (tests/golden/make_decoder_golden.py)."""
    import os

    from oracle.decoder import synthetic_model

    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "qwen05b_q8_0_greedy.npz"))
    config = qwen.QWEN25_05B_Q8
    packed, norms = synthetic_model(config, seed=int(golden["seeds"][0]))
    prompts, want, margins = golden["prompt"], golden["tokens"], golden["margins"]
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        del packed
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=1, capacity=256)
        decoder.record()
        got = decoder.generate(prompts, want.shape[1])
    finally:
        rt.close()
    differs = np.argwhere(got != want)
    if differs.size:
        _, at = differs[0]
        pytest.fail(f"the decoder leaves the golden ids at step {at}: {got[0, at]} for {want[0, at]}; "
                    f"the oracle's margin there is {margins[0, at]:.3e}, the smallest before it {margins[0, :at + 1].min():.3e}")


def test_a_recording_cut_short_by_a_refusal_is_ended_when_the_context_closes(runtime, oracle):
    packed = oracle.pack_rows(nb.Q8_0, oracle.Stream(2).normal(64 * 4096, 0.0, 0.02).reshape(64, 4096))
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weight = rt.load(nb.Q8_0, 64, 4096, packed)
        x, out = rt.tensor(1, 4096), rt.tensor(1, 64)
        rt.capture_begin()
        with pytest.raises(nb.NeuraCudaError, match="may not grow the scratch"):
            rt.linear(weight, x, out)
    finally:
        rt.close()
    probe = runtime.tensor(16)          # the thread is out of capture mode: allocation works again
    runtime.write(probe, np.arange(16, dtype=np.float32))
    assert runtime.read(probe).tolist() == list(range(16))


@pytest.mark.parametrize("name,batch,prompt,steps,capacity", [
    ("q8_0", 1, 16, 64, 96), ("q4_k", 1, 16, 64, 96), ("q4_k", 2, 16, 64, 96),
    ("q4_k", 1, 200, 24, 256),    # four splits of the cached positions to merge
])
def test_the_persistent_step_decodes_what_the_oracle_decodes(oracle, name, batch, prompt, steps, capacity):
    from oracle.decoder import OracleDecoder, synthetic_model

    config = SMALL[name]
    packed, norms = synthetic_model(config, seed=23)
    prompts = (oracle.Stream(41).uniform(batch * prompt, 0.0, 1.0) * config.vocab).astype(np.uint32).reshape(batch, prompt)
    want, margins = OracleDecoder(config, packed, norms, batch=batch, capacity=capacity).generate(prompts, steps)
    rt = nb.Runtime(0)
    rt.use_stream(rt.new_stream())
    try:
        weights, dnorms = load_model(rt, config, packed, norms)
        decoder = qwen.Decoder(rt, config, weights, dnorms, batch=batch, capacity=capacity)
        decoder.compile()
        assert decoder.launches_per_token() == 1
        got = decoder.generate(prompts, steps)
        again = decoder.generate(prompts, steps)
        kinds, nanos = decoder.trace()
        decoder.release()
    finally:
        rt.close()
    assert np.array_equal(got, again), "the persistent step decodes the same ids twice"
    # embedding, staging, five phases a layer, head, argmax; every phase took some time
    assert kinds.tolist() == [1, 4] + [2, 3, 2, 2, 2] * config.layers + [2, 5] and (nanos > 0).all()
    differs = np.argwhere(got != want)
    if differs.size:
        b, at = differs[0]
        pytest.fail(f"sequence {b} leaves the oracle at step {at}: {got[b, at]} for {want[b, at]}, "
                    f"the oracle's margin there is {margins[b, at]:.3e}")


@pytest.mark.parametrize("heads,key_heads,width,capacity,positions", [
    (6, 2, 64, 96, (0, 70)), (10, 2, 128, 600, (599, 301)), (4, 4, 128, 1100, (1099, 5)), (8, 2, 128, 64, (70, 63)),
])
def test_rope_and_attention_in_one_launch_equal_the_two_launches(runtime, oracle, heads, key_heads, width, capacity, positions):
    batch = len(positions)
    row = (heads + 2 * key_heads) * width
    qkv = oracle.Stream(51).normal(batch * row).reshape(batch, row)
    cache = batch * key_heads * capacity * width
    filled_k = oracle.Stream(52).normal(cache)
    filled_v = oracle.Stream(53).normal(cache)
    position = np.array(positions, dtype=np.uint32)     # (70 in a cache of 64: the cache is full, nothing is written)
    qd, pd = runtime.tensor(batch, row), runtime.tensor_u32(batch)
    runtime.write(pd, position)
    outs, caches = [], []
    for fused in (False, True):
        keys, values, out = runtime.tensor(cache), runtime.tensor(cache), runtime.tensor(batch, heads * width)
        runtime.write(keys, filled_k)
        runtime.write(values, filled_v)
        runtime.write(qd, qkv)
        if fused:
            angles = runtime.tensor(batch, width // 2, 2)
            runtime.rope_table(pd, 1e6, width, angles)
            runtime.rope_attend(qd, pd, angles, 0.125, heads, key_heads, width, capacity, keys, values, out)
            assert np.array_equal(bits(runtime.read(qd)), bits(qkv)), "the fused launch leaves q | k | v as they were"
        else:
            runtime.rope_cache(qd, pd, 1e6, heads, key_heads, width, capacity, keys, values)
            runtime.attend(qd, keys, values, pd, 0.125, heads, key_heads, width, capacity, out)
        outs.append(runtime.read(out))
        caches.append((runtime.read(keys), runtime.read(values)))
    assert np.array_equal(bits(outs[0]), bits(outs[1]))
    assert np.array_equal(bits(caches[0][0]), bits(caches[1][0])) and np.array_equal(bits(caches[0][1]), bits(caches[1][1]))
