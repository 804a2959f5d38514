"""Continuous batching over the decode step: the host side of the reference's ``Batch``.

Mirrors the plane bookkeeping of crates/neura-generate/src/batch.rs: ``admit`` (1000-1013),
``restart`` (1056-1105), ``resume`` (1015-1054), ``suspend`` (1107-1123), ``step`` (1125-1135),
``finish`` (1137-1148) and the emission rule of ``complete_answer`` (1676-1714): a plane that feeds
its last prompt token keeps the chosen token as its feed and emits nothing; a generating plane emits
its feed and keeps the new choice.  Greedy choice only (the reference's default ``Sampling``).
A stepper that offers ``fill`` takes the prompts in chunks first (``Batch::prefill``, batch.rs:1595-1599,
:298-325): all but a prompt's last token, which goes through the decode step like every generated one.

The device work is one call per step: ``stepper.answer(tokens, cursors) -> chosen`` over all planes
(``qwen.Decoder.answer``).  A plane that is empty or suspended rides along with token 0 at its own
cursor: what it writes lands in the cache row its next real token overwrites.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Iterator, List, NamedTuple, Optional, Sequence

import numpy as np


class Emitted(NamedTuple):
    slot: int
    token: int


PROMPTING, GENERATING, SUSPENDED = "feeding", "answering", "holding"


@dataclass
class _Slot:
    cursor: int
    phase: str
    prompt: Deque[int]
    feed: int = 0

    @property
    def running(self) -> bool:
        return self.phase != SUSPENDED


class BatchError(RuntimeError):
    """A call the reference's Batch refuses with a panic."""


class Batch:
    def __init__(self, stepper, context: Optional[int] = None):
        """``stepper``: ``.batch`` planes, ``.capacity`` cache rows a plane, ``.answer(tokens, cursors)``.
        ``context``: the longest sequence a plane holds (at most the cache's capacity)."""
        self.stepper = stepper
        self.batch = int(stepper.batch)
        self.context = int(context or stepper.capacity)
        if self.context > stepper.capacity:
            raise BatchError(f"a context of {self.context} does not fit a cache of {stepper.capacity} rows a plane")
        self.slots: List[Optional[_Slot]] = [None] * self.batch

    # -- planes ------------------------------------------------------------------------
    def _held(self, slot: int) -> _Slot:
        self._named(slot)
        held = self.slots[slot]
        if held is None:
            raise BatchError(f"plane {slot} of this batch holds no sequence")
        return held

    def _named(self, slot: int) -> None:
        if not 0 <= slot < self.batch:
            raise BatchError(f"a batch of {self.batch} planes names no plane {slot}")

    def admit(self, tokens: Sequence[int]) -> int:
        for slot, held in enumerate(self.slots):
            if held is None:
                self.restart(slot, tokens)
                return slot
        raise BatchError(f"all {self.batch} planes of this batch hold a sequence")

    def restart(self, slot: int, tokens: Sequence[int]) -> None:
        self._named(slot)
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise BatchError("a batch admits a prompt of at least one token")
        if len(tokens) >= self.context:
            raise BatchError(f"the prompt holds {len(tokens)} tokens where this batch holds {self.context} of context")
        self.slots[slot] = _Slot(0, PROMPTING, deque(tokens))

    def resume(self, slot: int, tokens: Sequence[int]) -> None:
        held = self._held(slot)
        if held.phase != SUSPENDED:
            raise BatchError(f"plane {slot} resumes only after it is suspended, and it is still {held.phase} its sequence")
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise BatchError("a sequence resumes with at least one token")
        if held.cursor >= self.context:
            raise BatchError(f"a sequence at cursor {held.cursor} of a context of {self.context} resumes only after "
                             "the application restarts or releases it")
        if len(tokens) >= self.context - held.cursor:
            raise BatchError(f"a sequence at cursor {held.cursor} resumes with {len(tokens)} tokens where this batch "
                             f"holds {self.context} of context")
        self.slots[slot] = _Slot(held.cursor, PROMPTING, deque(tokens))

    def suspend(self, slot: int) -> None:
        held = self._held(slot)
        if held.phase == PROMPTING:
            raise BatchError(f"a sequence suspends after it has fed its prompt, and plane {slot} still holds "
                             f"{len(held.prompt)} prompt tokens")
        if held.phase == SUSPENDED:
            raise BatchError(f"plane {slot} of this batch is already suspended")
        held.phase = SUSPENDED

    def finish(self, slot: int) -> None:
        self._named(slot)
        self.slots[slot] = None

    def active(self) -> Iterator[int]:
        return (slot for slot, held in enumerate(self.slots) if held is not None and held.running)

    def occupied(self) -> Iterator[int]:
        return (slot for slot, held in enumerate(self.slots) if held is not None)

    def cursor(self, slot: int) -> Optional[int]:
        held = self.slots[slot]
        return None if held is None else held.cursor

    def remaining(self, slot: int) -> Optional[int]:
        cursor = self.cursor(slot)
        return None if cursor is None else self.context - cursor

    # -- one step ------------------------------------------------------------------------
    def step(self) -> List[Emitted]:
        """One decode step over every running plane; the tokens the generating planes emit."""
        if next(self.active(), None) is None:
            return []
        tokens = np.zeros(self.batch, dtype=np.uint32)
        cursors = np.zeros(self.batch, dtype=np.uint32)
        for slot, held in enumerate(self.slots):
            if held is None:
                continue
            cursors[slot] = min(held.cursor, self.stepper.capacity - 1)
            if held.phase == PROMPTING:
                tokens[slot] = held.prompt[0]
            elif held.phase == GENERATING:
                tokens[slot] = held.feed
            if held.running and held.cursor >= self.context:
                raise BatchError(f"plane {slot} has filled its context of {self.context}; finish, suspend or restart it")
        self._prefill()
        for slot, held in enumerate(self.slots):   # (a fill moved the cursors of the planes it fed)
            if held is not None:
                cursors[slot] = min(held.cursor, self.stepper.capacity - 1)
                if held.phase == PROMPTING:
                    tokens[slot] = held.prompt[0]
        chosen = self.stepper.answer(tokens, cursors)
        emitted: List[Emitted] = []
        for slot, held in enumerate(self.slots):
            if held is None or not held.running:
                continue
            token = int(chosen[slot])
            if held.phase == PROMPTING:
                held.prompt.popleft()
                if not held.prompt:
                    held.phase, held.feed = GENERATING, token
            else:
                emitted.append(Emitted(slot, held.feed))
                held.feed = token
            held.cursor += 1
        return emitted

    def _prefill(self) -> None:
        """Batch::prefill: every feeding plane hands all but the last token of its prompt to the stepper's ``fill`` in
        the chunk sizes it names (largest first); what is left over, fewer tokens than the smallest chunk, goes
        through the decode steps."""
        chunks = tuple(getattr(self.stepper, "chunks", ()) or ())
        if not chunks or not hasattr(self.stepper, "fill"):
            return
        for slot, held in enumerate(self.slots):
            if held is None or held.phase != PROMPTING:
                continue
            # (a stepper built for it takes the head of a long prompt in wide chunks through the tensor-core product)
            wide = int(getattr(self.stepper, "wide", 0) or 0)
            through = self.stepper.wide_tokens(len(held.prompt)) if wide and hasattr(self.stepper, "fill_wide") else 0
            while through > 0:
                size = min(wide, through)
                self.stepper.fill_wide(slot, [held.prompt.popleft() for _ in range(size)], held.cursor)
                held.cursor += size
                through -= size
            while True:
                size = next((c for c in chunks if c <= len(held.prompt) - 1), None)
                if size is None:
                    break
                self.stepper.fill(slot, [held.prompt.popleft() for _ in range(size)], held.cursor)
                held.cursor += size

    def advance(self, waves: int) -> List[Emitted]:
        """``waves`` steps in a row (batch.rs:1174-1190 walks them as one frame)."""
        if waves <= 0:
            raise BatchError("a batch walks at least one wave a frame")
        emitted: List[Emitted] = []
        for _ in range(waves):
            emitted += self.step()
        return emitted
