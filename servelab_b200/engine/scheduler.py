"""Continuous batching with chunked prefill and recompute-preemption (torch-free).

Each ``schedule()`` call shares one token budget (``max_num_batched_tokens``)
among, in this order (servelab/engine/scheduler.py:150-243):

  1. single decoded tokens of running requests, in running order, at most
     ``max_num_seqs`` of them (scheduler.py:176-188);
  2. the next portion of prompts already in flight, in policy order: a portion
     is min(remaining, budget) tokens (scheduler.py:190-198,246-265);
  3. admission of waiting requests in policy order (FCFS = arrival time then
     id, scheduler.py:37-41; "priority" puts the priority value first,
     scheduler.py:44-48) while fewer than ``max_num_seqs`` are running and budget
     is left; the first request that cannot get pages blocks those behind it
     (scheduler.py:200-241).

Pages are reserved here, before the step runs.  When pages run out for a running
request, the latest-arrived running request that is not yet part of this step
loses its pages and goes back to the front of the waiting queue with its
computed counter reset (recompute, scheduler.py:276-316); this repeats until the
reservation fits (the reference preempts one victim and lets the requester idle
a step).  With no victim left the requester itself is preempted.  A waiting
request that does not fit simply stays waiting.  A request that could never fit
in the pool, or is longer than the model's position limit, finishes as
"aborted" and IS reported (the reference drops it silently, scheduler.py:211-215).

``chunked_prefill=False`` keeps the reference's older mode: whole prompts in
one portion regardless of the budget, and no decodes while anything waits
(scheduler.py:177,255-258).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from ..cache.manager import CacheManager
from ..config.engine import SchedulerConfig
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledPortion:
    """Tokens [start, start + num_tokens) of ``seq`` run in this step."""
    seq: Sequence
    start: int
    num_tokens: int

    @property
    def wants_logits(self) -> bool:
        return self.start + self.num_tokens == self.seq.get_len()

    @property
    def is_decode(self) -> bool:
        return self.num_tokens == 1 and self.start >= self.seq.num_prompt_tokens


@dataclass
class SchedulerOutput:
    portions: List[ScheduledPortion] = field(default_factory=list)
    preempted: List[str] = field(default_factory=list)
    aborted: List[Sequence] = field(default_factory=list)

    def is_empty(self) -> bool:
        return not self.portions

    @property
    def num_batched_tokens(self) -> int:
        return sum(p.num_tokens for p in self.portions)

    def has(self, seq: Sequence) -> bool:
        return any(p.seq is seq for p in self.portions)


def _order(policy: str, seqs: List[Sequence]) -> List[Sequence]:
    if policy == "priority":
        return sorted(seqs, key=lambda s: (s.priority, s.arrival_time, s.request_id))
    return sorted(seqs, key=lambda s: (s.arrival_time, s.request_id))


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager,
                 clock: Callable[[], float], eos_token_ids=(), max_model_len: int = 1 << 30):
        self.cfg = config
        self.cache = cache
        self.clock = clock
        self.eos_token_ids = frozenset(int(e) for e in eos_token_ids)
        self.max_model_len = max_model_len
        self.waiting: List[Sequence] = []
        self.running: List[Sequence] = []
        self.num_preemptions = 0

    # ------------------------------------------------------------ intake
    def add_request(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def abort_request(self, request_id: str) -> Optional[Sequence]:
        for queue in (self.waiting, self.running):
            for i, s in enumerate(queue):
                if s.request_id == request_id:
                    queue.pop(i)
                    self.cache.release(request_id)
                    s.status = SequenceStatus.FINISHED_ABORTED
                    s.abort_reason = "aborted by the caller"
                    s.metrics.finished_time = self.clock()
                    return s
        return None

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------- schedule
    def schedule(self) -> SchedulerOutput:
        now = self.clock()
        out = SchedulerOutput()
        budget = self.cfg.max_num_batched_tokens

        # 1) single decoded tokens (held back in the unchunked mode while anything waits)
        decodes_held = not self.cfg.chunked_prefill and bool(self.waiting)
        if not decodes_held:
            budget = self._schedule_decodes(out, budget)

        # 2) prompts in flight
        for seq in _order(self.cfg.policy, [s for s in self.running if not s.is_decoding()]):
            if budget <= 0:
                break
            if seq not in self.running or out.has(seq):
                continue
            n = self._portion(seq, budget)
            if self._reserve(seq, n, out):
                budget -= n

        # 3) admission
        self.waiting = _order(self.cfg.policy, self.waiting)
        while self.waiting and len(self.running) < self.cfg.max_num_seqs and budget > 0:
            seq = self.waiting[0]
            too_long = seq.get_len() > self.max_model_len
            if too_long or not self.cache.can_ever_hold(seq.get_len(), self._max_portion()):
                self.waiting.pop(0)
                seq.status = SequenceStatus.FINISHED_ABORTED
                seq.abort_reason = (f"{seq.get_len()} tokens exceed the position limit "
                                    f"{self.max_model_len}" if too_long else
                                    f"{seq.get_len()} tokens can never fit in the cache pool")
                seq.metrics.finished_time = now
                out.aborted.append(seq)
                continue
            n = self._portion(seq, budget)
            if not self.cache.open(seq.request_id):
                break                             # no state slot free
            if not self.cache.ensure(seq.request_id, n, for_admission=True):
                self.cache.release(seq.request_id)
                break                             # head-of-line blocking
            self.waiting.pop(0)
            seq.status = SequenceStatus.RUNNING
            seq.metrics.first_scheduled_time = seq.metrics.first_scheduled_time or now
            self.running.append(seq)
            out.portions.append(ScheduledPortion(seq, 0, n))
            budget -= n

        # The unchunked mode held the decodes back for the waiting requests; if none of
        # those could be admitted (no pages while the running ones hold them), the step
        # would be empty for ever: the running requests decode instead, finish and free
        # their pages.  The reference gets out of the same corner by preempting a running
        # request when admission fails (scheduler.py:232-237,276-298).
        if decodes_held and not out.portions and not out.aborted:
            self._schedule_decodes(out, budget)
        return out

    def _schedule_decodes(self, out: SchedulerOutput, budget: int) -> int:
        """Phase 1: one token for every running request that is decoding; returns the
        budget that is left."""
        num_decodes = 0
        for seq in list(self.running):
            if seq not in self.running or not seq.is_decoding():
                continue                      # preempted a moment ago / still in prompt
            if num_decodes >= self.cfg.max_num_seqs or budget < 1:
                break
            if self._reserve(seq, 1, out):
                num_decodes += 1
                budget -= 1
        return budget

    def _max_portion(self) -> int:
        return self.cfg.max_num_batched_tokens if self.cfg.chunked_prefill else 1 << 30

    def _portion(self, seq: Sequence, budget: int) -> int:
        remaining = seq.num_uncomputed()
        return max(1, min(remaining, budget)) if self.cfg.chunked_prefill else max(1, remaining)

    def _reserve(self, seq: Sequence, n: int, out: SchedulerOutput) -> bool:
        """Reserve room for ``n`` more tokens of a running request, preempting
        others (latest arrival first) while it does not fit."""
        target = seq.num_computed_tokens + n
        while not self.cache.ensure(seq.request_id, target):
            victim = next((v for v in reversed(_order(self.cfg.policy, self.running))
                           if v is not seq and not out.has(v)), None)
            if victim is None:
                self._preempt(seq, out)
                return False
            self._preempt(victim, out)
        out.portions.append(ScheduledPortion(seq, seq.num_computed_tokens, n))
        return True

    def _preempt(self, seq: Sequence, out: SchedulerOutput) -> None:
        self.running.remove(seq)
        self.cache.release(seq.request_id)
        seq.on_preempt_recompute()
        self.num_preemptions += 1
        self.waiting.insert(0, seq)
        out.preempted.append(seq.request_id)

    # ---------------------------------------------------- after the step
    def update_after_exec(self, out: SchedulerOutput, sampled: Dict[str, int],
                          now: Optional[float] = None) -> List[Sequence]:
        """Advance computed counters, give back pages a window has passed,
        append sampled tokens, apply stop conditions (EOS or stop ids unless
        ignore_eos, then max_tokens, scheduler.py:319-349; also the position
        limit), release finished requests.  Returns those that finished."""
        now = self.clock() if now is None else now
        finished: List[Sequence] = []
        for p in out.portions:
            seq = p.seq
            seq.num_computed_tokens = p.start + p.num_tokens
            seq.metrics.num_steps += 1
            self.cache.trim(seq.request_id, seq.num_computed_tokens)
            if seq.request_id not in sampled:
                continue
            token = int(sampled[seq.request_id])
            seq.append_token(token)
            if seq.metrics.first_token_time == 0.0:
                seq.metrics.first_token_time = now
            sp = seq.sampling_params
            is_stop = token in self.eos_token_ids or token in sp.stop_token_ids
            if is_stop and not sp.ignore_eos:
                seq.status = SequenceStatus.FINISHED_EOS
            elif seq.num_output_tokens >= sp.max_tokens or seq.get_len() >= self.max_model_len:
                seq.status = SequenceStatus.FINISHED_LENGTH
            if seq.is_finished():
                finished.append(seq)
        for seq in finished:
            self.running.remove(seq)
            self.cache.release(seq.request_id)
            seq.metrics.finished_time = now
        return finished

    # ------------------------------------------------------------- stats
    def stats(self) -> dict:
        return {"waiting": len(self.waiting), "running": len(self.running),
                "gpu_cache_usage": round(self.cache.usage(), 4),
                "num_preemptions_total": self.num_preemptions}
