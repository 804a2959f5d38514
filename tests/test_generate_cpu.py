"""The continuous-batching bookkeeping (generate.Batch) over the oracle's decoder as the stepper:
the emission rule and the refusals of crates/neura-generate/src/batch.rs, and that ragged
admissions decode, plane by plane, what a batch of one decodes."""
import numpy as np
import pytest

from neura_b200.generate import Batch, BatchError, Emitted
from neura_b200.qwen import Config
from neura_b200.runtime import Q8_0
from oracle.decoder import OracleDecoder, synthetic_model

CONFIG = Config("nano", 2, 128, 4, 2, 32, 256, 160, Q8_0, tied_head=True)


class Echo:
    """A stepper whose choice is token + cursor: the bookkeeping shows in the numbers."""
    batch, capacity = 3, 16

    def __init__(self):
        self.calls = []

    def answer(self, tokens, cursors):
        self.calls.append((tokens.copy(), cursors.copy()))
        return tokens + cursors


def test_a_plane_emits_its_feed_one_step_after_it_was_chosen():
    echo = Echo()
    batch = Batch(echo)
    assert batch.step() == [] and not echo.calls
    slot = batch.admit([10, 20])
    assert slot == 0 and list(batch.active()) == [0] and batch.cursor(0) == 0 and batch.remaining(0) == 16
    assert batch.step() == []            # feeds 10 at cursor 0
    assert batch.step() == []            # feeds 20 at cursor 1: choice 21 becomes the feed
    assert batch.step() == [Emitted(0, 21)]   # feeds 21 at cursor 2: choice 23
    assert batch.step() == [Emitted(0, 23)]
    assert batch.cursor(0) == 4
    tokens = [int(c[0][0]) for c in echo.calls]
    cursors = [int(c[1][0]) for c in echo.calls]
    assert tokens == [10, 20, 21, 23] and cursors == [0, 1, 2, 3]


def test_planes_join_leave_suspend_and_resume():
    echo = Echo()
    batch = Batch(echo)
    a, b = batch.admit([1]), batch.admit([5, 6, 7])
    assert (a, b) == (0, 1)
    assert batch.step() == []                       # a: feed 1; b feeds 5
    assert batch.step() == [Emitted(0, 1)]          # a emits 1 (1+0), feeds it at cursor 1 -> 2
    batch.suspend(a)
    assert list(batch.active()) == [1] and list(batch.occupied()) == [0, 1]
    assert batch.step() == []                       # b feeds 7 at cursor 2 -> feed 9
    assert echo.calls[-1][0][0] == 0 and echo.calls[-1][1][0] == 2   # the suspended plane rides at its cursor
    assert batch.cursor(a) == 2
    batch.resume(a, [40])
    c = batch.admit([100])
    assert c == 2
    emitted = batch.step()                          # a feeds 40 at 2 -> 42; b emits 9; c feeds 100
    assert emitted == [Emitted(1, 9)]
    emitted = batch.step()
    assert emitted == [Emitted(0, 42), Emitted(1, 12), Emitted(2, 100)]
    batch.finish(b)
    assert list(batch.occupied()) == [0, 2] and batch.admit([3]) == 1
    assert batch.advance(2) == [Emitted(0, 45), Emitted(2, 101), Emitted(0, 49), Emitted(1, 3), Emitted(2, 103)]


def test_the_calls_the_reference_refuses_are_refused():
    batch = Batch(Echo())
    with pytest.raises(BatchError, match="at least one token"):
        batch.admit([])
    with pytest.raises(BatchError, match="16 tokens where this batch holds 16"):
        batch.admit(list(range(16)))
    with pytest.raises(BatchError, match="names no plane 3"):
        batch.restart(3, [1])
    with pytest.raises(BatchError, match="holds no sequence"):
        batch.suspend(1)
    slot = batch.admit([1, 2])
    with pytest.raises(BatchError, match="still holds 2 prompt tokens"):
        batch.suspend(slot)
    with pytest.raises(BatchError, match="resumes only after it is suspended"):
        batch.resume(slot, [3])
    batch.advance(2)
    batch.suspend(slot)
    with pytest.raises(BatchError, match="already suspended"):
        batch.suspend(slot)
    with pytest.raises(BatchError, match="at least one token"):
        batch.resume(slot, [])
    with pytest.raises(BatchError, match="resumes with 14 tokens"):
        batch.resume(slot, list(range(14)))
    batch.admit([1]), batch.admit([1])
    with pytest.raises(BatchError, match="all 3 planes"):
        batch.admit([1])
    with pytest.raises(BatchError, match="at least one wave"):
        batch.advance(0)
    with pytest.raises(BatchError, match="does not fit a cache"):
        Batch(Echo(), context=17)


def test_a_full_context_is_refused_before_the_device_runs():
    batch = Batch(Echo(), context=4)
    batch.admit([1, 2, 3])
    batch.advance(4)
    with pytest.raises(BatchError, match="filled its context of 4"):
        batch.step()


def test_ragged_admissions_decode_what_a_batch_of_one_decodes():
    packed, norms = synthetic_model(CONFIG, seed=11)
    prompts = [[3, 9, 27, 81], [5], [7, 49, 11]]
    alone = []
    for prompt in prompts:
        want, _ = OracleDecoder(CONFIG, packed, norms, batch=1, capacity=24, threads=2).generate(np.array([prompt]), 6)
        alone.append([int(t) for t in want[0]])
    batch = Batch(OracleDecoder(CONFIG, packed, norms, batch=2, capacity=24, threads=2))
    got = {0: [], 1: [], 2: []}
    plane = {batch.admit(prompts[0]): 0}
    batch.step()                       # sequence 1 joins a step late
    plane[batch.admit(prompts[1])] = 1
    joined = False
    for _ in range(40):
        for slot, token in batch.step():
            got[plane[slot]].append(token)
        for slot in list(batch.occupied()):
            if len(got[plane[slot]]) >= 6:
                batch.finish(slot)
                if not joined:   # sequence 2 takes the first plane that frees
                    joined = True
                    plane[batch.admit(prompts[2])] = 2
        if not list(batch.occupied()):
            break
    assert [got[i][:6] for i in range(3)] == alone


def test_a_stepper_with_a_wide_path_takes_the_head_of_a_long_prompt_through_it():
    # Batch::prefill with a stepper that offers the tensor path: 13 prompt tokens, wide chunks of 8 from 5 tokens up:
    # 12 are fed, 8 in one wide chunk (bf16 operands), the other 4 as a chunk of 4; the last goes through the step
    packed, norms = synthetic_model(CONFIG, seed=11)
    prompt = [3, 9, 27, 81, 5, 7, 49, 11, 2, 4, 8, 16, 32]
    alone = OracleDecoder(CONFIG, packed, norms, batch=1, capacity=24, threads=2)
    want, _ = alone.generate(np.array([prompt]), 6, bf16_tokens=8)
    stepper = OracleDecoder(CONFIG, packed, norms, batch=2, capacity=24, threads=2)
    stepper.wide, stepper.WIDE_FROM = 8, 5
    assert stepper.wide_tokens(len(prompt)) == 8
    calls = []
    fill_wide, fill = stepper.fill_wide, stepper.fill
    stepper.fill_wide = lambda slot, tokens, start: (calls.append(("wide", len(tokens), start)), fill_wide(slot, tokens, start))[1]
    stepper.fill = lambda slot, tokens, start: (calls.append(("fill", len(tokens), start, stepper.bf16)), fill(slot, tokens, start))[1]
    batch = Batch(stepper)
    slot = batch.admit(prompt)
    got = []
    for _ in range(8):
        got += [token for s, token in batch.step() if s == slot]
    assert calls == [("wide", 8, 0), ("fill", 8, 0, True), ("fill", 4, 8, False)]
    assert got[:6] == [int(t) for t in want[0]]
