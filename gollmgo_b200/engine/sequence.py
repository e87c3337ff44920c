"""A request on its way through the scheduler.

States and transitions are the reference's (internal/scheduler/sequence.go:13-45):
WAITING -> PREFILLING (-> itself for every further portion) -> DECODING ->
FINISHED, and DECODING -> PREEMPTED -> WAITING; here a sequence can also be
preempted while it is still prefilling, and a sequence that waits (again) for
admission can finish: a token of its that was still on the device when it was
preempted may turn out to end it, and a failed step ends what it held.
"""
from __future__ import annotations

import enum
import time
from typing import List, Optional

from ..sampling.params import SamplingParams


PENDING = -1       # in Sequence.output: a token sampled on the device that the host has not read yet


class SeqState(enum.Enum):
    WAITING = "WAITING"
    PREFILLING = "PREFILLING"
    DECODING = "DECODING"
    FINISHED = "FINISHED"
    PREEMPTED = "PREEMPTED"


_VALID = {
    SeqState.WAITING: {SeqState.PREFILLING, SeqState.FINISHED},
    SeqState.PREFILLING: {SeqState.PREFILLING, SeqState.DECODING, SeqState.PREEMPTED, SeqState.FINISHED},
    SeqState.DECODING: {SeqState.FINISHED, SeqState.PREEMPTED},
    SeqState.PREEMPTED: {SeqState.WAITING},
    SeqState.FINISHED: set(),
}


class InvalidTransition(RuntimeError):
    pass


class Sequence:
    def __init__(self, seq_id: int, request_id: str, prompt: List[int], params: SamplingParams):
        self.id = seq_id
        self.request_id = request_id
        self.prompt = list(prompt)
        self.output: List[int] = []
        self.params = params
        self.state = SeqState.WAITING
        self.num_computed = 0              # tokens whose keys and values are in the cache
        self.preemptions = 0
        self.finish_reason: Optional[str] = None
        self.created_at = time.perf_counter()
        self.first_token_at: Optional[float] = None
        self.last_token_at: Optional[float] = None
        self.token_times: List[float] = []
        self.resolved = 0                  # tokens of `output` whose value the host knows
        self.pending_row = -1              # row of the unknown token in the sampler's device buffer
        self.dropped = False               # ended by an end-of-sequence token; later samples are void
        self.error: Optional[str] = None   # why it ended, if a step it took part in failed

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_slice(self, lo: int, hi: int) -> List[int]:
        """tokens[lo:hi] without building the whole list."""
        n = len(self.prompt)
        if lo >= n:
            return self.output[lo - n:hi - n]
        if hi <= n:
            return self.prompt[lo:hi]
        return self.prompt[lo:] + self.output[:hi - n]

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens not yet in the cache.  After a preemption this is prompt and
        generated tokens together: they are recomputed as one prompt."""
        return self.total_len - self.num_computed

    def transition(self, to: SeqState) -> None:
        if to not in _VALID[self.state]:
            raise InvalidTransition(f"{self.state.value} -> {to.value}")
        self.state = to

    @property
    def finished(self) -> bool:
        return self.state is SeqState.FINISHED
