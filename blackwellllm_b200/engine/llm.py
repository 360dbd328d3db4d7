"""The Python entry point, in the manner of the reference's public API
(include/blackwell/engine.h:104-204, docs/INFERENCE_API.md:173-244).

:class:`BlackwellEngine` keeps the reference's names and meanings where it has
them: ``InferenceConfig(max_context_length, max_batch_size, temperature, top_p)``,
position-addressed ``forward(token_id, pos, ...)`` that returns the next sampled
token, ``prefill(token_ids, start_pos, ...)`` that consumes a prompt and samples
only after its last token, ``forward_batch`` (one token each of distinct
sequences, greedy), ``forward_eval`` and ``last_token_probability`` (log
probability of a given next token), ``rewind`` and ``release_sequence``.  Beyond the reference,
``generate`` runs many requests with continuous batching through the scheduler.

Token ids in, token ids out: the engine holds no tokenizer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Union

import torch

from ..config.registry import load_config, parse_config
from ..kernels import ops
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .engine import Engine, EngineError, EngineOptions
from .scheduler import Scheduler


@dataclass
class InferenceConfig:
    """What a caller asks for (the reference's tier-2 request,
    include/blackwell/runtime_config.h:87-137, same names and defaults)."""
    max_context_length: int = 2048
    max_batch_size: int = 1
    temperature: float = 0.6
    top_p: float = 0.9


@dataclass
class DecodeRequest:
    """One row of ``forward_batch`` (include/blackwell/engine.h: DecodeRequest{seq, token, pos})."""
    seq_id: int
    token_id: int
    pos: int


@dataclass
class GenerationResult:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    preemptions: int = 0


class BlackwellEngine:
    def __init__(self, model: Optional[str] = None, request: Optional[InferenceConfig] = None, *,
                 config: Optional[Mapping[str, object]] = None, random_seed: int = 0, random_std: float = 0.02,
                 dtype: str = "bfloat16", page_size: int = 16, num_pages: Optional[int] = None,
                 max_batch_tokens: int = 2048, chunk: Optional[int] = None, kv_fraction: Optional[float] = None,
                 seed: int = 0, device: str = "cuda:0", cuda_graphs: bool = True, ignore_unexpected: bool = False):
        """``model``: a folder with config.json and model.safetensors.  Or ``config``
        (the config.json object) for random weights from ``random_seed``.  The cache
        holds ``max_batch_size`` sequences of ``max_context_length`` tokens unless
        ``num_pages`` or ``kv_fraction`` (of free device memory) says otherwise.
        ``ignore_unexpected``: tensors of the checkpoint that the model does not use are
        passed over with a note instead of being an error."""
        self.request = request or InferenceConfig()
        rq = self.request
        if rq.max_context_length <= 0 or rq.max_batch_size < 1:
            raise EngineError("max_context_length must be > 0 and max_batch_size >= 1")
        if num_pages is None and kv_fraction is None:
            num_pages = rq.max_batch_size * -(-rq.max_context_length // page_size)
        opts = EngineOptions(dtype=dtype, page_size=page_size, num_pages=num_pages,
                             kv_fraction=kv_fraction or 0.6, max_requests=max(rq.max_batch_size, 1),
                             max_batch_tokens=max(max_batch_tokens, rq.max_batch_size), device=device,
                             max_context=rq.max_context_length, cuda_graphs=cuda_graphs,
                             ignore_unexpected=ignore_unexpected)
        if (model is None) == (config is None):
            raise EngineError("give either a model folder or a config for random weights")
        # the context is checked against the model before any weight is read
        # (the reference's plan does the same, src/core/runtime_config.cpp:59-65)
        mc = load_config(model) if model is not None else parse_config(config)
        if mc.max_position_embeddings and rq.max_context_length > mc.max_position_embeddings:
            raise EngineError(f"max_context_length {rq.max_context_length} exceeds the model's "
                              f"max_position_embeddings {mc.max_position_embeddings}")
        if model is not None:
            self.engine = Engine.from_folder(model, options=opts)
        else:
            self.engine = Engine.from_config(config, seed=random_seed, std=random_std, options=opts)
        self.sampler = Sampler(self.engine.device)
        self.seed = seed
        self.chunk = chunk
        self.max_batch_tokens = max_batch_tokens
        self._last_logits: Dict[int, torch.Tensor] = {}   # rows of the LAST step's logits, by sequence
        self.scheduler = self._new_scheduler()

    def _new_scheduler(self) -> Scheduler:
        return Scheduler(self.engine.cache, max_batch_tokens=self.max_batch_tokens,
                         max_running=self.request.max_batch_size, chunk=self.chunk,
                         max_context=self.request.max_context_length,
                         eos_token_ids=self.engine.config.eos_token_ids, seed=self.seed)

    @property
    def vocab_size(self) -> int:
        return self.engine.config.vocab_size

    # ------------------------------------------------------------------ position-addressed calls
    def _seq(self, seq_id: int):
        return ("seq", int(seq_id))

    def _reconcile(self, seq_id: int, pos: int) -> None:
        """pos < length rewinds to pos; pos > length is a gap and an error
        (src/core/kv_cache/paged_kv_manager.cpp:72-92)."""
        rid = self._seq(seq_id)
        cache = self.engine.cache
        length = cache.length(rid) if cache.has(rid) else 0
        if pos > length:
            raise EngineError(f"sequence {seq_id}: position {pos} leaves a gap after its {length} cached tokens")
        if pos < length:
            cache.truncate(rid, pos)
        if pos >= self.request.max_context_length:
            raise EngineError(f"position {pos} is outside max_context_length {self.request.max_context_length}")

    def _pick(self, logits: torch.Tensor, seq_ids: Sequence[int], temperature: float, top_p: float) -> List[int]:
        # The random number of a draw is a function of (seed, sequence, position of the sampled token):
        # the same prompt on the same sequence id gives the same tokens again, whatever ran before.
        p = SamplingParams(temperature=temperature, top_p=top_p)
        draws = [self.engine.cache.length(self._seq(s)) for s in seq_ids]
        seeds = [self.seed * 1_000_003 + s for s in seq_ids]
        return self.sampler.sample(logits, [p] * len(seq_ids), seeds, draws)

    def forward(self, token_id: int, pos: int, temperature: float = 0.6, top_p: float = 0.9,
                seq_id: int = 0) -> int:
        """One auto-regressive step: writes the cache at ``pos``, returns the next token."""
        return self.prefill([token_id], pos, temperature, top_p, seq_id)

    def prefill(self, token_ids: Sequence[int], start_pos: int = 0, temperature: float = 0.6,
                top_p: float = 0.9, seq_id: int = 0) -> int:
        """Consumes the tokens from ``start_pos`` and samples only the continuation after
        the last one (the reference's prefill_status, src/core/engine.cpp:1520-1552)."""
        ids = list(token_ids)
        if not ids:
            raise EngineError("prefill needs at least one token")
        if start_pos + len(ids) > self.request.max_context_length:
            raise EngineError("the tokens do not fit max_context_length")
        self._reconcile(seq_id, start_pos)
        rid = self._seq(seq_id)
        at, logits = 0, None
        while at < len(ids):
            n = min(len(ids) - at, self.max_batch_tokens)
            last = at + n == len(ids)
            logits = self.engine.step([StepEntry(rid, ids[at:at + n], [n - 1] if last else [])])
            at += n
        self._last_logits = {seq_id: logits[0]}
        return self._pick(logits, [seq_id], temperature, top_p)[0]

    def forward_eval(self, token_id: int, pos: int, target_token_id: int, seq_id: int = 0) -> float:
        """Feeds ``token_id`` at ``pos`` and returns ln P(target_token_id) of the next token,
        for perplexity (the reference's forward_eval_status, src/core/engine.cpp:1557-1570)."""
        self._check_token(target_token_id)
        self._reconcile(seq_id, pos)
        logits = self.engine.step([StepEntry(self._seq(seq_id), [token_id], [0])])
        self._last_logits = {seq_id: logits[0]}
        return self._log_prob(logits[:1], target_token_id)

    def last_token_probability(self, token_id: int, seq_id: int = 0) -> float:
        """P(token_id) under the logits that the last forward, prefill, forward_batch or
        forward_eval left for the sequence, without a model step; 0 for an id outside the
        vocabulary or a sequence that was not in that last call (the reference reads its one
        logits buffer as the last step left it, src/core/engine.cpp:1618-1630)."""
        row = self._last_logits.get(seq_id)
        if row is None or not 0 <= token_id < self.vocab_size:
            return 0.0
        return min(1.0, max(0.0, math.exp(self._log_prob(row[None, :], token_id))))

    def _check_token(self, token_id: int) -> None:
        if not 0 <= token_id < self.vocab_size:
            raise EngineError(f"token id {token_id} is outside the vocabulary of {self.vocab_size}")

    def _log_prob(self, logits: torch.Tensor, token_id: int) -> float:
        target = torch.tensor([token_id], dtype=torch.int32, device=logits.device)
        return float(ops.log_prob(logits, target).item())

    def forward_batch(self, requests: Sequence[DecodeRequest]) -> List[int]:
        """One token each of distinct sequences, greedy (src/core/engine.cpp:1576-1616)."""
        if not requests:
            raise EngineError("forward_batch needs at least one request")
        seqs = [r.seq_id for r in requests]
        if len(set(seqs)) != len(seqs):
            raise EngineError("forward_batch: a sequence appears twice")
        for r in requests:
            self._reconcile(r.seq_id, r.pos)
        logits = self.engine.step([StepEntry(self._seq(r.seq_id), [r.token_id], [0]) for r in requests])
        self._last_logits = {s: logits[i] for i, s in enumerate(seqs)}
        return self._pick(logits, seqs, 0.0, 1.0)

    def rewind(self, seq_id: int, pos: int) -> None:
        rid = self._seq(seq_id)
        if not self.engine.cache.has(rid):
            raise EngineError(f"unknown sequence {seq_id}")
        self.engine.cache.truncate(rid, pos)

    def release_sequence(self, seq_id: int) -> None:
        rid = self._seq(seq_id)
        if self.engine.cache.has(rid):
            self.engine.cache.free_request(rid)
        self._last_logits.pop(seq_id, None)

    def reset_state(self, seq_id: int = 0) -> None:
        """Forgets the sequence (cache and any fixed-size state)."""
        self.release_sequence(seq_id)

    # ------------------------------------------------------------------ continuous batching
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        if params is None:
            params = SamplingParams(temperature=self.request.temperature, top_p=self.request.top_p)
        return self.scheduler.add_request(prompt_token_ids, params).rid

    def step(self) -> List[GenerationResult]:
        """One scheduler step; returns the requests that finished in it."""
        plan = self.scheduler.plan()
        if not plan.entries:
            return []
        entries = [StepEntry(e.request.rid, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                   for e in plan.entries]
        self._last_logits = {}
        logits = self.engine.step(entries)
        samplers = [e.request for e in plan.entries if e.samples]
        sampled: Dict[int, int] = {}
        if samplers:
            toks = self.sampler.sample(logits, [r.params for r in samplers], [r.seed for r in samplers],
                                       [len(r.generated) for r in samplers], [r.generated for r in samplers])
            sampled = {r.rid: t for r, t in zip(samplers, toks)}
        done = self.scheduler.commit(plan, sampled)
        for r in done:   # handed to the caller here: a long-lived engine keeps no finished request
            self.scheduler.finished.pop(r.rid, None)
        return [GenerationResult(r.rid, r.prompt, r.generated, r.finish_reason, r.preemptions) for r in done]

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[GenerationResult]:
        """Generates for one prompt or many (lists of token ids); results in the order given."""
        single = bool(prompts) and isinstance(prompts[0], int)
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if params is None or isinstance(params, SamplingParams):
            pl = [params] * len(plist)
        else:
            pl = list(params)
            if len(pl) != len(plist):
                raise EngineError("one SamplingParams per prompt")
        rids = [self.add_request(p, sp) for p, sp in zip(plist, pl)]
        results: Dict[int, GenerationResult] = {}
        while self.scheduler.has_work():
            before = self.scheduler.stats.steps
            for res in self.step():
                results[res.request_id] = res
            if self.scheduler.stats.steps == before and self.scheduler.has_work():
                raise EngineError("the scheduler made no progress (cache too small for the waiting request)")
        return [results[r] for r in rids]


LLM = BlackwellEngine
