"""Results handed to the caller.

The field names are the reference's result schema (``RequestOutput`` /
``CompletionOutput``, servelab/engine/output.py:9-41), so code written against it
reads these objects unchanged: ``finish_reason`` is "eos", "length" or "aborted".
Beyond the reference: an aborted request says why (``abort_reason``: it could never
fit in the cache pool, it exceeds the position limit, or the caller aborted it; the
reference drops such requests without an output), and the metrics carry what this
engine counts (time spent waiting, steps the request took part in, generated tokens
across preemptions).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

from .sequence import Sequence, SequenceStatus

_REASONS = {SequenceStatus.FINISHED_EOS: "eos", SequenceStatus.FINISHED_LENGTH: "length",
            SequenceStatus.FINISHED_ABORTED: "aborted"}


@dataclass
class CompletionOutput:
    index: int = 0
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    abort_reason: Optional[str] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: str = ""
    prompt_token_ids: List[int] = field(default_factory=list)
    outputs: List[CompletionOutput] = field(default_factory=list)
    finished: bool = False
    metrics: Optional[dict] = None

    @classmethod
    def from_sequence(cls, seq: Sequence,
                      detokenize: Optional[Callable[[List[int]], str]] = None) -> "RequestOutput":
        reason = _REASONS.get(seq.status)                  # None while the request still runs
        generated = seq.token_ids[seq.num_prompt_tokens:]
        completion = CompletionOutput(token_ids=generated, finish_reason=reason,
                                      text=detokenize(generated) if detokenize else "",
                                      abort_reason=seq.abort_reason if reason == "aborted" else None)
        metrics = seq.metrics.to_dict()
        metrics["generated_tokens"] = len(generated)
        return cls(seq.request_id, prompt_token_ids=seq.token_ids[:seq.num_prompt_tokens],
                   outputs=[completion], finished=reason is not None, metrics=metrics)
