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


_GREEDY = SamplingParams(temperature=0.0, top_p=1.0)
FROM_LAST = -1   # DecodeRequest.token_id: the token that the previous forward_batch sampled for the sequence


class PendingTokens:
    """Tokens that the device is still choosing: the read-back into pinned memory is queued behind the
    sampler; :meth:`result` waits for it."""

    def __init__(self, picked: torch.Tensor, host: Optional[torch.Tensor] = None, done: bool = False):
        """``host``: pinned memory into which the read-back is already queued (``done``: and complete)."""
        if host is None:
            host = torch.empty(picked.shape, dtype=picked.dtype, pin_memory=picked.is_cuda)
            host.copy_(picked, non_blocking=True)
        self._host = host
        self._event = None
        if picked.is_cuda and not done:
            self._event = torch.cuda.Event()
            self._event.record()

    def result(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()


class _RowsOf:
    """The rows of a step's logits by sequence, looked up when asked for (a graph replay's logits are
    overwritten by the next step of the same batch size: ask before it)."""

    def __init__(self, logits: torch.Tensor, seqs: Sequence[int]):
        self._logits, self._index = logits, {s: i for i, s in enumerate(seqs)}

    def get(self, seq_id, default=None):
        i = self._index.get(seq_id)
        return default if i is None else self._logits[i]

    def pop(self, seq_id, default=None):
        self._index.pop(seq_id, None)


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
        self._fed = None            # (sequences, their sampled tokens on the device) of the last forward_batch
        self._ahead = None          # (plan, prepared step) of the next scheduler step, made while the last one ran
        self.pipeline = True        # prepare decode steps ahead (see step())
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

    def _drop_ahead(self) -> None:
        """Takes back a scheduler step that was prepared ahead (another kind of call comes first)."""
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            self.engine.cancel_prepared(ahead[1])

    def _reconcile(self, seq_id: int, pos: int) -> None:
        """pos < length rewinds to pos; pos > length is a gap and an error
        (src/core/kv_cache/paged_kv_manager.cpp:72-92)."""
        self._drop_ahead()
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
        return self.forward_batch_async(requests, wait=True).result()

    def forward_batch_async(self, requests: Sequence[DecodeRequest], wait: bool = False) -> "PendingTokens":
        """:meth:`forward_batch` without waiting for its tokens: the step and the read-back of the
        sampled tokens are queued on the device and a handle is returned; ``handle.result()`` waits
        and gives the tokens.  A request whose ``token_id`` is :data:`FROM_LAST` takes the token that
        the previous ``forward_batch`` call sampled for its sequence, straight from the device (all
        requests of the call, the same sequences in the same order as in that call).  So a decode loop
        can queue step n + 1 before it reads step n's tokens, and the device never waits for the host:

            pending = llm.forward_batch_async([DecodeRequest(s, first[s], pos) for s in seqs])
            while ...:
                pos += 1
                nxt = llm.forward_batch_async([DecodeRequest(s, FROM_LAST, pos) for s in seqs])
                tokens = pending.result()          # step n's tokens, while step n + 1 runs
                pending = nxt
        """
        if not requests:
            raise EngineError("forward_batch needs at least one request")
        self._drop_ahead()
        seqs = [r.seq_id for r in requests]
        if len(set(seqs)) != len(seqs):
            raise EngineError("forward_batch: a sequence appears twice")
        fed = [r.token_id == FROM_LAST for r in requests]
        source = None
        if any(fed):
            if not all(fed) or self._fed is None or self._fed[0] != seqs:
                raise EngineError("forward_batch: FROM_LAST needs every request of the call to use it, for the "
                                  "same sequences in the same order as the call before")
            source = self._fed[1]
        cache, limit = self.engine.cache, self.request.max_context_length
        rids = [("seq", int(r.seq_id)) for r in requests]
        # the hot path: one C call does the whole step (see csrc/decode_step.h); it declines what it does
        # not take (a new sequence, no captured graph yet, any refusal), and the ordinary path below explains
        native = self.engine.decode_native(rids, [0 if source is not None else r.token_id for r in requests],
                                           [r.pos for r in requests], source, wait=wait) \
            if all(0 <= r.pos < limit for r in requests) else None
        if native is not None:
            logits, picked, host = native
            self._last_logits = _RowsOf(logits, seqs)
            self._fed = (seqs, picked)
            return PendingTokens(picked, host, done=wait)
        entries = []
        for r, rid in zip(requests, rids):
            length = cache.length(rid) if cache.has(rid) else 0
            if r.pos != length:
                if r.pos > length:
                    raise EngineError(f"sequence {r.seq_id}: position {r.pos} leaves a gap after its {length} cached tokens")
                cache.truncate(rid, r.pos)
            if r.pos >= limit:
                raise EngineError(f"position {r.pos} is outside max_context_length {limit}")
            entries.append(StepEntry(rid, [0 if source is not None else r.token_id], [0]))
        logits = self.engine.step(entries, token_source=source)
        self._last_logits = _RowsOf(logits, seqs)
        picked = self.sampler.sample_async(logits, [_GREEDY] * len(seqs), seqs, seqs)   # greedy, as the reference's batched decode
        self._fed = (seqs, picked)
        return PendingTokens(picked)

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
        """One scheduler step; returns the requests that finished in it.

        While the GPU runs a step after which every running request decodes, the host prepares the
        next one (the same requests, one token each: pages reserved, block tables and positions
        packed), so that only the sampled tokens have to be filled in before it is launched.  If the
        step turns out differently (a request ended on an end-of-sequence token, one arrived), what
        was prepared is taken back and the step is planned the ordinary way."""
        ahead, self._ahead = self._ahead, None
        if ahead is not None and (self.scheduler.waiting or [e.request for e in ahead[0].entries] != self.scheduler.running):
            self.engine.cancel_prepared(ahead[1])
            ahead = None
        if ahead is not None:
            plan, prep = ahead
            logits = self.engine.launch_prepared(prep, [e.tokens[0] for e in plan.entries])
        else:
            plan = self.scheduler.plan()
            if not plan.entries:
                return []
            entries = [StepEntry(e.request.rid, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                       for e in plan.entries]
            logits = self.engine.step(entries)
        self._last_logits = {}
        samplers = [e.request for e in plan.entries if e.samples]
        sampled: Dict[int, int] = {}
        picked = None
        if samplers:
            picked = self.sampler.sample_async(logits, [r.params for r in samplers], [r.seed for r in samplers],
                                               [len(r.generated) for r in samplers], [r.generated for r in samplers])
        nxt = self._prepare_ahead(plan)        # host work while the GPU runs this step
        if picked is not None:
            sampled = {r.rid: t for r, t in zip(samplers, picked.tolist())}     # waits for the step
        try:
            done = self.scheduler.commit(plan, sampled)
        except BaseException:
            if nxt is not None:
                self.engine.cancel_prepared(nxt[1])
            raise
        if nxt is not None:
            if done or self.scheduler.waiting:
                self.engine.cancel_prepared(nxt[1])
            else:
                for e in nxt[0].entries:    # the tokens that were being sampled while the step was prepared
                    e.tokens = [sampled[e.request.rid]]
                self._ahead = nxt
        for r in done:   # handed to the caller here: a long-lived engine keeps no finished request
            self.scheduler.finished.pop(r.rid, None)
        return [GenerationResult(r.rid, r.prompt, r.generated, r.finish_reason, r.preemptions) for r in done]

    def _prepare_ahead(self, plan):
        """The next step, prepared while this one runs, if it is certain to be "one token for each
        running request": every running request samples in this step, none of them reaches its limit
        of new tokens or of context with the token being sampled, nobody waits.  (A request may still
        end on an end-of-sequence token: then what is prepared here is cancelled.)"""
        sch = self.scheduler
        if not self.pipeline or sch.waiting or not plan.entries or len(plan.entries) != len(sch.running):
            return None
        for e in plan.entries:
            r = e.request
            if not e.samples or len(r.generated) + 1 >= r.params.max_new_tokens:
                return None
            if sch.max_context is not None and len(r.prompt) + len(r.generated) + 1 >= sch.max_context:
                return None
        prep = self.engine.prepare_decode_ahead([r.rid for r in sch.running])
        if prep is None:
            return None
        from .scheduler import PlannedEntry, StepPlan
        return StepPlan([PlannedEntry(r, [0], True) for r in sch.running], []), prep

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
