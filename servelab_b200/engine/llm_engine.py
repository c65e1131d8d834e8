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
"""

from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence as Seq, Union

from ..config.engine import CacheConfig, SchedulerConfig
from ..config.registry import load_config
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.source import FolderSource, WeightSource
from .outputs import RequestOutput
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import Sequence


class LLMEngine:
    def __init__(self, model: Union[str, object], cache_config: Optional[CacheConfig] = None,
                 scheduler_config: Optional[SchedulerConfig] = None, seed: int = 1234,
                 dtype: str = "bfloat16", device: str = "cuda:0", tokenizer=None,
                 clock: Optional[Callable[[], float]] = None,
                 weights: Optional[WeightSource] = None, cuda_graphs: bool = True,
                 max_model_len: Optional[int] = None):
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
        tokens = self.sampler.sample(logits, logit_seqs)
        sampled: Dict[str, int] = {s.request_id: t for s, t in zip(logit_seqs, tokens)}
        finished = self.scheduler.update_after_exec(plan, sampled, now=self.clock())
        self.num_steps += 1
        return outputs + [RequestOutput.from_sequence(s, self._detokenize) for s in finished]

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
