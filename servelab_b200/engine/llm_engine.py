"""The Python entry point: ``LLMEngine`` ties scheduler, cache, step function and
sampler together, in the manner of the reference's engine
(servelab/engine/engine.py:42-297):

    engine = LLMEngine("path/to/model")              # or a typed config + weights
    engine.add_request(prompt_token_ids=[...], sampling_params=SamplingParams(...))
    while engine.has_unfinished():
        for out in engine.step(): ...
    outputs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams.greedy(8))

Method names and meanings are the reference's: add_request (engine.py:138),
abort_request (:162), has_unfinished (:165), step (:169, returns the requests
that finished in this step), generate (:249, outputs in input order), stats
(:290).  Differences: requests that can never run are returned as "aborted"
outputs instead of vanishing; ``max_tokens`` counts all generated tokens also
across a preemption; prompts are checked against the vocabulary and the
position limit.

Look-ahead: while every running request is decoding and none can end by its length
in the current step, the engine launches step N+1 before it reads the tokens of
step N.  Step N+1 takes its input tokens from the sampler's result on the device,
so the GPU never waits for the host between two decode steps; the host reads the
tokens of step N while N+1 runs.  A request that turns out to have ended in step N
(an EOS or stop token) has run one step too many: that result is dropped (the page
it wrote is already given back; later steps come later on the stream).  ``step()``
still returns the requests that finished in the step whose tokens it read.
"""

from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence as Seq, Union

import torch

from ..config.engine import CacheConfig, SchedulerConfig
from ..config.registry import load_config
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.source import FolderSource, WeightSource
from .outputs import RequestOutput
from .runner import ModelRunner
from .scheduler import ScheduledPortion, Scheduler, SchedulerOutput
from .sequence import Sequence, SequenceStatus


class LLMEngine:
    def __init__(self, model: Union[str, object], cache_config: Optional[CacheConfig] = None,
                 scheduler_config: Optional[SchedulerConfig] = None, seed: int = 1234,
                 dtype: str = "bfloat16", device: str = "cuda:0", tokenizer=None,
                 clock: Optional[Callable[[], float]] = None,
                 weights: Optional[WeightSource] = None, cuda_graphs: bool = True,
                 max_model_len: Optional[int] = None, lookahead: bool = True):
        """``model``: a model folder (config.json + safetensors), or a typed
        architecture config together with ``weights``."""
        if isinstance(model, str):
            config, weights = load_config(model), weights or FolderSource(model)
        else:
            config = model
            if weights is None:
                raise ValueError("a typed config needs weights= (a WeightSource)")
        self.model_config = config
        self.cache_config = cache_config or CacheConfig()
        self.scheduler_config = scheduler_config or SchedulerConfig()
        self.tokenizer = tokenizer
        self.clock = clock or time.monotonic
        self.runner = ModelRunner(config, weights, dtype=dtype, cache_config=self.cache_config,
                                  max_num_seqs=self.scheduler_config.max_num_seqs, device=device,
                                  cuda_graphs=cuda_graphs, max_model_len=max_model_len)
        spec = self.runner.spec
        self.scheduler = Scheduler(self.scheduler_config, self.runner.cache, self.clock,
                                   eos_token_ids=spec.eos_token_ids,
                                   max_model_len=self.runner.max_model_len)
        self.sampler = Sampler(seed, device)
        self._req_counter = 0
        self.num_steps = 0
        self.lookahead = lookahead
        self._ahead = None                 # (requests, their tokens on the way) of a step launched ahead
        self.num_lookahead_steps = 0
        # measurements: a list that receives, per step, (tokens run, cached keys read = the sum
        # of the requests' context lengths, query-key pairs scored, rows of logits)
        self.step_trace: Optional[list] = None

    # -------------------------------------------------------------- intake
    def add_request(self, prompt: Optional[str] = None,
                    sampling_params: Optional[SamplingParams] = None,
                    prompt_token_ids: Optional[Seq[int]] = None,
                    request_id: Optional[str] = None, priority: int = 0) -> str:
        if prompt_token_ids is None:
            if self.tokenizer is None or prompt is None:
                raise ValueError("need prompt_token_ids, or a tokenizer + prompt")
            prompt_token_ids = self.tokenizer.encode(prompt)
        prompt_token_ids = [int(t) for t in prompt_token_ids]
        if not prompt_token_ids:
            raise ValueError("empty prompt")
        self.runner.check_tokens(prompt_token_ids)
        self._req_counter += 1
        request_id = request_id or f"req-{self._req_counter}"
        seq = Sequence(request_id, prompt_token_ids, sampling_params or SamplingParams(),
                       priority=priority, arrival_time=self.clock(), stream_id=self._req_counter)
        self.scheduler.add_request(seq)
        return request_id

    def abort_request(self, request_id: str) -> bool:
        return self.scheduler.abort_request(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------- stepping
    def step(self) -> List[RequestOutput]:
        """One scheduler step; returns the requests that finished in it."""
        outputs: List[RequestOutput] = []
        adopted = self._adopt_ahead()
        if adopted is not None:
            plan, rows, pending = adopted          # launched by the previous call
            logit_seqs = [p.seq for p in plan.portions]
        else:
            plan = self.scheduler.schedule()
            outputs = [RequestOutput.from_sequence(s, self._detokenize) for s in plan.aborted]
            if plan.is_empty():
                return outputs
            entries, logit_seqs = [], []
            for p in plan.portions:
                seq = p.seq
                want = (p.num_tokens - 1,) if p.wants_logits else ()
                entries.append(self.runner.entry(seq.request_id,
                                                 seq.token_ids[p.start:p.start + p.num_tokens],
                                                 p.start, want))
                if p.wants_logits:
                    logit_seqs.append(seq)
            logits = self.runner.step(entries)
            pending = self.sampler.sample_async(logits, logit_seqs)
            rows = list(range(len(logit_seqs)))
        self._launch_ahead(plan, logit_seqs, rows, pending)
        tokens = pending.wait()
        sampled: Dict[str, int] = {s.request_id: tokens[r] for s, r in zip(logit_seqs, rows)}
        if self.step_trace is not None:
            self.step_trace.append((
                sum(p.num_tokens for p in plan.portions),
                sum(p.start + p.num_tokens for p in plan.portions),
                sum(p.num_tokens * p.start + p.num_tokens * (p.num_tokens + 1) // 2 for p in plan.portions),
                len(logit_seqs)))
        finished = self.scheduler.update_after_exec(plan, sampled, now=self.clock())
        self.num_steps += 1
        return outputs + [RequestOutput.from_sequence(s, self._detokenize) for s in finished]

    # ------------------------------------------------------------ look-ahead
    def _launch_ahead(self, plan: SchedulerOutput, seqs: List[Sequence], rows: List[int],
                      pending) -> None:
        """Launch the decode step after ``plan`` now, with the tokens ``pending`` holds on
        the device, if that step is certain except for stop tokens."""
        self._ahead = None
        sch, runner = self.scheduler, self.runner
        if (not self.lookahead or not seqs or sch.waiting or plan.preempted
                or len(plan.portions) != len(sch.running) or len(seqs) != len(plan.portions)
                or not runner.replays_graph(len(seqs))):
            return
        for p in plan.portions:
            seq, sp = p.seq, p.seq.sampling_params
            if (p.num_tokens != 1 or not p.wants_logits                 # a prompt portion
                    or seq.num_output_tokens + 1 >= sp.max_tokens        # ends by its length
                    or seq.get_len() + 1 >= sch.max_model_len):
                return
        # every request gets one more token; its position is the current length.  (Windowed
        # groups: the pages that step N's bookkeeping gives back afterwards are still read by
        # the step launched here; whoever gets them next writes them in a later step, which
        # the stream runs after this one.)
        for seq in seqs:
            if not runner.cache.ensure(seq.request_id, seq.get_len() + 1):
                return                              # no page: the scheduler decides next step
        entries = [runner.entry(seq.request_id, [0], seq.get_len(), (0,)) for seq in seqs]
        ids = pending.device
        if rows != list(range(ids.shape[0])):
            ids = ids[torch.tensor(rows, dtype=torch.long, device=ids.device)]
        logits = runner.step(entries, token_ids_from=ids)
        self._ahead = (list(seqs), self.sampler.sample_async(logits, seqs, ahead=1))
        self.num_lookahead_steps += 1

    def _adopt_ahead(self):
        """The step launched ahead, as a plan over the requests that are still running
        (others ended meanwhile; their rows are dropped): (plan, rows, pending) or None."""
        ahead, self._ahead = self._ahead, None
        if ahead is None:
            return None
        seqs, pending = ahead
        running = {id(s) for s in self.scheduler.running}
        plan, rows = SchedulerOutput(), []
        for r, seq in enumerate(seqs):
            if id(seq) in running and seq.status == SequenceStatus.RUNNING:
                plan.portions.append(ScheduledPortion(seq, seq.get_len() - 1, 1))
                rows.append(r)
        if not rows:
            return None
        return plan, rows, pending

    def _detokenize(self, token_ids: List[int]) -> str:
        return "" if self.tokenizer is None else self.tokenizer.decode(token_ids)

    # ------------------------------------------------------------- generate
    def generate(self, prompts: List, sampling_params: Optional[SamplingParams] = None,
                 verbose: bool = False) -> List[RequestOutput]:
        """Offline batch generation; prompts are strings (needs a tokenizer) or
        lists of token ids.  Outputs come back in input order."""
        params = sampling_params or SamplingParams()
        ids = [self.add_request(prompt=p if isinstance(p, str) else None,
                                prompt_token_ids=None if isinstance(p, str) else list(p),
                                sampling_params=params) for p in prompts]
        results: Dict[str, RequestOutput] = {}
        while self.has_unfinished():
            for out in self.step():
                results[out.request_id] = out
            if verbose:
                st = self.scheduler.stats()
                print(f"[step] running={st['running']} waiting={st['waiting']} "
                      f"cache={st['gpu_cache_usage']:.0%}")
        return [results.get(i) for i in ids]

    # ----------------------------------------------------------------- misc
    def stats(self) -> dict:
        return {**self.scheduler.stats(), **self.runner.cache.stats(),
                "num_blocks": self.runner.num_pages, "block_size": self.runner.page_size,
                "dtype": str(self.runner.dtype).replace("torch.", ""),
                "device": self.runner.device, "steps": self.num_steps}
