"""Per-request state (torch-free).

Parity: ``Sequence`` / ``SequenceStatus`` / ``RequestMetrics``
(servelab/engine/sequence.py:11-113).  One deliberate difference: after a
recompute-preemption the reference makes prompt + generated tokens the new
prompt (sequence.py:102-109), so ``max_tokens`` starts again and earlier output
is dropped from the result; here the prompt length never changes and only the
computed counter is reset.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(str, Enum):
    WAITING = "WAITING"
    RUNNING = "RUNNING"
    FINISHED_EOS = "FINISHED_EOS"
    FINISHED_LENGTH = "FINISHED_LENGTH"
    FINISHED_ABORTED = "FINISHED_ABORTED"


FINISHED_STATES = frozenset({SequenceStatus.FINISHED_EOS, SequenceStatus.FINISHED_LENGTH,
                             SequenceStatus.FINISHED_ABORTED})


@dataclass
class RequestMetrics:
    arrival_time: float = 0.0
    first_scheduled_time: float = 0.0
    first_token_time: float = 0.0
    finished_time: float = 0.0
    num_preemptions: int = 0
    num_steps: int = 0                    # steps this request took part in

    @property
    def ttft(self) -> float:
        return self.first_token_time - self.arrival_time

    @property
    def e2e_latency(self) -> float:
        return self.finished_time - self.arrival_time

    def to_dict(self) -> dict:
        return {"ttft": self.ttft, "latency": self.e2e_latency,
                "preemptions": self.num_preemptions,
                "queue_time": max(0.0, self.first_scheduled_time - self.arrival_time),
                "steps": self.num_steps}


class Sequence:
    """Prompt plus generated tokens of one request.

    ``num_computed_tokens`` counts tokens whose keys/values (and state) are in
    the cache.  A step feeds tokens [num_computed, num_computed + n); logits are
    wanted only when the portion reaches the last token.  While decoding,
    num_computed == len - 1 after every step (the sampled token is fed by the
    next step; tests/test_engine_smoke.py:113-127 in the reference).
    """

    def __init__(self, request_id: str, prompt_token_ids: List[int],
                 sampling_params: SamplingParams, priority: int = 0,
                 arrival_time: float = 0.0, stream_id: int = 0):
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.token_ids: List[int] = list(prompt_token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_computed_tokens = 0
        self.sampling_params = sampling_params
        self.priority = priority
        self.arrival_time = arrival_time
        self.stream_id = stream_id            # random stream of this request
        self.status = SequenceStatus.WAITING
        self.abort_reason: Optional[str] = None     # set with FINISHED_ABORTED
        self.metrics = RequestMetrics(arrival_time=arrival_time)

    @property
    def num_output_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def output_token_ids(self) -> List[int]:
        return self.token_ids[self.num_prompt_tokens:]

    def get_len(self) -> int:
        return len(self.token_ids)

    def num_uncomputed(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    def is_decoding(self) -> bool:
        """One token left to feed: the step is a single decoded token (or the
        only token of a one-token prompt)."""
        return self.num_uncomputed() == 1

    def is_finished(self) -> bool:
        return self.status in FINISHED_STATES

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))

    def on_preempt_recompute(self) -> None:
        self.num_computed_tokens = 0
        self.metrics.num_preemptions += 1
        self.status = SequenceStatus.WAITING

    def __repr__(self) -> str:  # pragma: no cover
        return (f"Sequence({self.request_id}, len={self.get_len()}, "
                f"computed={self.num_computed_tokens}, {self.status.value})")
