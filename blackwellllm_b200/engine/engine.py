"""The engine: a model, its cache, and ONE step function.

``Engine.step(entries)`` takes a batch of (request, its next tokens): portions of
prompts beside single decoded tokens, cut anywhere.  It runs only those tokens,
reading everything earlier from the cache, and returns the float32 logits at the
places asked for.  The reference has three disjoint widths instead (one token,
one chunk of one sequence, one token each of B sequences:
src/core/engine.cpp:822, 895, 1304); here they are one call.

Pages for every token of the step are reserved before anything runs, so a step
either runs whole or raises :class:`OutOfPages` with nothing changed (the
reference budgets pages before compute likewise:
src/core/engine_prefill_coordinator.cpp:160-169).
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import (ERR_BAD_TOKEN, ERR_BAD_WANT, ERR_NO_SLOT, ERR_OUT_OF_PAGES, ERR_TOO_MANY_TOKENS,
                             ERR_TOO_SMALL, CacheManager, native)
from ..cache.pages import OutOfPages
from ..config.registry import load_config, parse_config
from ..config.specs import ModelConfig
from ..models.decoder import DecoderModel
from ..parts.base import BuildContext, PagedKVRequest
from ..weights.loader import bind_tensors, load_weights
from ..weights.random_init import random_tensors
from .batch import BatchBuilder, StepBatch, StepEntry

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16,
           "bf16": torch.bfloat16, torch.float32: torch.float32, torch.bfloat16: torch.bfloat16}


class EngineError(RuntimeError):
    pass


@dataclass
class EngineOptions:
    dtype: object = "bfloat16"      # "bfloat16" | "float32"
    page_size: int = 16
    num_pages: Optional[int] = None  # pages per cache group; None: from max_tokens or kv_fraction
    max_tokens: Optional[int] = None  # tokens the cache holds (each request rounded up to a page)
    kv_fraction: float = 0.6         # of the memory free after the weights, if neither is given
    max_requests: int = 64
    max_batch_tokens: int = 8192
    max_context: Optional[int] = None  # longest request; None: what the pool holds
    ignore_unexpected: bool = False  # tensors of a checkpoint that the model does not use: pass over, no error
    cuda_graphs: bool = True         # replay decode-only steps from a CUDA graph per batch size
    graph_after: int = 3             # a batch size is recorded at its n-th decode-only step (a recording costs about
                                     # two uncaptured steps; batch sizes that pass by once or twice never pay it)
    native_decode: bool = True       # greedy decode-only steps of live requests go through the C entry point
    max_graph_batch: int = 256
    device: str = "cuda:0"


def require_cuda(device: torch.device) -> None:
    if device.type != "cuda" or not torch.cuda.is_available():
        raise EngineError("blackwellllm_b200 runs on a CUDA device (B200, sm_100a) only; "
                          "there is no CPU path")


@dataclass
class PreparedDecode:
    """A decode-only step whose bookkeeping is done and whose token ids are still to come."""
    rids: list
    host: torch.Tensor        # the packed step in pinned memory; its first len(rids) words are the token ids
    total: int
    slot: dict                # the graph of this batch size and its device buffer
    ring_slot: int            # where the pinned buffer sits in the uploader's ring
    rids_done: bool = False   # launched or cancelled


class Engine:
    def __init__(self, config: ModelConfig, model: DecoderModel, options: EngineOptions):
        self.config = config
        self.model = model
        self.options = options
        self.device = torch.device(options.device)
        self.dtype = _DTYPES[options.dtype]
        requests = model.cache_requests()
        num_pages = self._decide_num_pages(options, requests)
        self.cache = CacheManager(requests, options.page_size, num_pages, options.max_requests,
                                  dtype=self.dtype, device=self.device)
        self._builder = BatchBuilder(self.device)
        self._graphs: Dict[int, dict] = {}
        self._graph_uses: Dict[int, int] = {}   # decode-only steps seen per batch size that has no graph yet
        self._capture_stream = None
        self._grown = None
        longest = options.max_context or num_pages * options.page_size
        self._graph_width = -(-longest // options.page_size)
        self.steps_run = 0
        self.tokens_run = 0
        self.native_steps = 0      # steps that went through the C entry point (csrc/decode_step.h)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _options(opts: Mapping[str, object]) -> EngineOptions:
        o = opts.get("options")
        if o is not None:
            return o
        return EngineOptions(**{k: v for k, v in opts.items() if k != "options"})

    @classmethod
    def _build(cls, config: ModelConfig, options: EngineOptions):
        if options.dtype not in _DTYPES:
            raise EngineError(f"dtype must be 'bfloat16' or 'float32', got {options.dtype!r}")
        device = torch.device(options.device)
        require_cuda(device)
        torch.cuda.set_device(device)
        ctx = BuildContext(device, _DTYPES[options.dtype])
        return DecoderModel(config, ctx), ctx

    @classmethod
    def from_folder(cls, model_dir: str, **opts) -> "Engine":
        """A folder with config.json and model.safetensors (or an index and shards)."""
        options = cls._options(opts)
        config = load_config(model_dir)
        model, ctx = cls._build(config, options)
        model.bind(load_weights(model_dir, model.param_specs(), ctx.dtype, ctx.device, options.ignore_unexpected))
        return cls(config, model, options)

    @classmethod
    def from_tensors(cls, raw_config: Mapping[str, object], tensors: Mapping[str, torch.Tensor],
                     **opts) -> "Engine":
        options = cls._options(opts)
        config = parse_config(raw_config)
        model, ctx = cls._build(config, options)
        model.bind(bind_tensors(tensors, model.param_specs(), ctx.dtype, ctx.device,
                                ignore_unexpected=options.ignore_unexpected))
        return cls(config, model, options)

    @classmethod
    def from_config(cls, raw_config: Mapping[str, object], seed: int = 0, std: float = 0.02,
                    bias_std: Optional[float] = None, **opts) -> "Engine":
        """Random weights made on the device (no folder is written)."""
        options = cls._options(opts)
        config = parse_config(raw_config)
        model, ctx = cls._build(config, options)
        specs = model.param_specs()
        tensors = random_tensors(specs, seed, std, bias_std, dtype=ctx.dtype, device=ctx.device)
        model.bind(bind_tensors(tensors, specs, ctx.dtype, ctx.device))
        return cls(config, model, options)

    def _decide_num_pages(self, o: EngineOptions, requests) -> int:
        if o.num_pages is not None:
            return int(o.num_pages)
        if o.max_tokens is not None:
            return max(1, -(-int(o.max_tokens) // o.page_size))
        groups: Dict[PagedKVRequest, int] = {}
        for r in requests:
            if isinstance(r, PagedKVRequest):
                groups[r] = groups.get(r, 0) + 1
        if not groups:
            return 1
        esize = 4 if self.dtype == torch.float32 else 2
        per_page = sum(n * 2 * r.num_kv_heads * o.page_size * r.head_dim * esize for r, n in groups.items())
        free, _ = torch.cuda.mem_get_info(self.device)
        return max(1, int(free * o.kv_fraction) // per_page)

    # ------------------------------------------------------------------ requests
    def add_request(self, rid) -> None:
        self.cache.add_request(rid)

    def end_request(self, rid) -> None:
        """The request is finished: its pages and its state slot are given back."""
        self.cache.free_request(rid)

    def has_request(self, rid) -> bool:
        return self.cache.has(rid)

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry], min_blocks: int = 0, into=None,
                replay_width: Optional[int] = None, defer_send: bool = False):
        """Checks the entries, reserves pages for all their tokens (all or nothing)
        and uploads the batch.  The checks, the page bookkeeping and the packing of the
        step's buffer are one call into the C++ host runtime."""
        cache = self.cache
        R = len(entries)
        rids = [e.rid for e in entries]
        if len(set(rids)) != R:
            twice = next(r for i, r in enumerate(rids) if r in rids[:i])
            raise EngineError(f"request {twice!r} appears twice in one step")
        handles = np.fromiter(map(cache.handle, rids), dtype=np.int32, count=R)
        n_tok = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=R)
        n_want = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=R)
        T, W = int(n_tok.sum()), int(n_want.sum())
        if T == R:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        else:
            tokens = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T)
        want = np.fromiter((w for e in entries for w in e.want), dtype=np.int64, count=W)
        V = self.config.vocab_size
        if T and (tokens.min() < 0 or tokens.max() >= V):     # also keeps the ids inside int32
            self._explain(entries, ERR_BAD_TOKEN)
        if W and (want.min() < 0 or want.max() >= 2 ** 31):
            self._explain(entries, ERR_BAD_WANT)
        tokens, want = tokens.astype(np.int32), want.astype(np.int32)
        G = len(cache.groups)
        blocks_bound = max(min_blocks, self._graph_width + -(-self.options.max_batch_tokens // cache.page_size) + 1)
        cap = 3 * T + 4 * R + 1 + W + G * R * blocks_bound
        meta = np.zeros(4 + max(G, 1), dtype=np.int64)
        new_slots = np.zeros(max(R, 1), dtype=np.int32)
        was_new = handles < 0
        for attempt in range(2):
            host = self._builder.pinned(cap)
            total = native().bwh_pack_step(cache._h, R, handles.ctypes.data, n_tok.ctypes.data, tokens.ctypes.data,
                                           n_want.ctypes.data, want.ctypes.data, V, min_blocks,
                                           self.options.max_batch_tokens, host.data_ptr(), cap, meta.ctypes.data,
                                           new_slots.ctypes.data)
            if total != ERR_TOO_SMALL:
                break
            # a request longer than max_context: no table is longer than its group's pool (nothing changed yet)
            cap = 3 * T + 4 * R + 1 + W + G * R * (max([min_blocks] + [g.num_pages for g in cache.groups]) + 1)
        if total < 0:
            self._explain(entries, int(total))
        k = 0
        for i in np.nonzero(was_new)[0]:
            cache.adopt(entries[i].rid, int(handles[i]))
            cache.zero_state(int(new_slots[k]))
            k += 1
        self._grown = (entries, was_new)     # what to take back if the model fails after this point
        widths = {g: int(meta[4 + g]) for g in range(G)}
        if replay_width is not None:
            # a graph replay: the captured kernels read the buffer at its fixed address, no views needed
            if any(w != replay_width for w in widths.values()):
                raise EngineError("a request outgrew max_context: its block table no longer fits the graph")
            if defer_send:
                return host, int(total)     # the caller sends it later (a step prepared ahead)
            self._builder.send(host, int(total), into)
            return None
        return self._builder.finish(host, T, R, W, widths, rids, into)

    def _explain(self, entries: Sequence[StepEntry], code: int) -> None:
        """Raises the error that the host runtime's code stands for, with the offending entry named."""
        V = self.config.vocab_size
        T = sum(len(e.tokens) for e in entries)
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise EngineError(f"request {e.rid!r}: a step entry needs at least one token")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise EngineError(f"request {e.rid!r}: token id {t} is outside [0, {V})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise EngineError(f"request {e.rid!r}: wanted place {w} is outside its {n} tokens")
        if code == ERR_TOO_MANY_TOKENS:
            raise EngineError(f"step of {T} tokens exceeds max_batch_tokens={self.options.max_batch_tokens}")
        if code == ERR_NO_SLOT:
            new = sum(1 for e in entries if not self.cache.has(e.rid))
            raise OutOfPages(f"{new} new requests but {self.cache.slots.num_free} request slots are free")
        if code == ERR_OUT_OF_PAGES:
            ps = self.cache.page_size
            need = [0] * len(self.cache.groups)
            for e in entries:
                pn = self.cache.pages_needed(e.rid, len(e.tokens)) if self.cache.has(e.rid) \
                    else [-(-len(e.tokens) // ps)] * len(need)
                need = [a + b for a, b in zip(need, pn)]
            raise OutOfPages(f"step needs {need} pages per group, {self.cache.free_pages()} are free")
        raise EngineError(f"the host runtime refused the step (code {code})")

    # A decode-only step (one token and one wanted place per request) has the same
    # shapes every time: its kernels are captured once per batch size in a CUDA graph
    # and replayed.  Everything that changes from step to step (tokens, positions,
    # block tables, lengths) lives in one device buffer at a fixed address that is
    # overwritten before each replay.
    def _graph_key(self, entries: Sequence[StepEntry]):
        if not self.options.cuda_graphs or len(entries) > self.options.max_graph_batch:
            return None
        if not all(getattr(b.mixer, "graph_safe", True) for b in self.model.blocks):
            return None  # a mixer that works on the host between kernels cannot be captured
        for e in entries:
            if len(e.tokens) != 1 or list(e.want) != [0]:
                return None
        return len(entries)

    @contextlib.contextmanager
    def _capture(self, graph):
        """Records what runs inside into ``graph`` on a stream of its own.  (``torch.cuda.graph`` does the same
        after a full garbage collection, 25 to 40 ms with a model's worth of Python objects: more than the
        recording itself.)"""
        if not hasattr(graph, "capture_begin"):          # a stand-in graph of the tests
            with torch.cuda.graph(graph):
                yield
            return
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        side = self._capture_stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            graph.capture_begin()
            try:
                yield
            finally:
                graph.capture_end()
        torch.cuda.current_stream(self.device).wait_stream(side)

    def _step_graph(self, entries: Sequence[StepEntry], R: int, token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        width = self._graph_width
        slot = self._graphs.get(R)
        if slot is None:
            n_groups = len(self.cache.groups)
            total = 3 * R + (R + 1) + 3 * R + R + n_groups * R * width
            slot = {"buf": torch.zeros(total, dtype=torch.int32, device=self.device), "graph": None,
                    "logits": None, "kernels": 0}
            self._graphs[R] = slot
        if slot["graph"] is not None:
            self.prepare(entries, min_blocks=width, into=slot["buf"], replay_width=width)
            if token_source is not None:
                slot["buf"][:R].copy_(token_source)     # the token ids lead the packed layout
            slot["graph"].replay()
            return slot["logits"]
        # No graph of this batch size yet.  Its first ``graph_after`` - 1 decode-only steps run uncaptured, on
        # the batch as a replay would see it (block tables of the graph's width, the key bound of the graph), so
        # that every kernel and buffer of the graph has been used once; the next one records.  Whichever way,
        # the model runs ONCE for the step (a mixer with state of its own must not see a step twice): the
        # step that records after uncaptured ones captures (a capture executes nothing) and replays; a step
        # that records as the very first of its size runs uncaptured, which is its result, and then captures.
        uses = self._graph_uses.get(R, 0) + 1
        self._graph_uses[R] = uses
        batch = self.prepare(entries, min_blocks=width, into=slot["buf"])
        if any(t.shape[1] != width for t in batch.block_tables.values()):
            raise EngineError("a request outgrew max_context: its block table no longer fits the graph")
        batch.static_bound = width * self.cache.page_size
        # what the host derives from the batch's shape and the bound alone (attention work lists) is made by the
        # first of these steps and shared by the later ones and the graph: nothing is copied to the device inside a capture
        batch.static_extras = slot.setdefault("static_extras", {})
        if token_source is not None:
            batch.token_ids.copy_(token_source)
        from ..kernels import ops
        record = uses >= self.options.graph_after
        logits = None
        if not record or uses == 1:
            logits = self.model.forward(batch, self.cache.views)
            if not record:
                return logits
            torch.cuda.synchronize(self.device)
            batch.extras.clear()   # what depends on this step's values is recomputed inside the graph
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with self._capture(graph):
            slot["logits"] = self.model.forward(batch, self.cache.views)
        slot["kernels"] = ops.launches - before
        slot["graph"] = graph
        slot["batch"] = batch   # keeps the per-step tensors that the captured kernels read alive
        if logits is None:
            graph.replay()
            logits = slot["logits"]
        return logits

    def graph_kernel_count(self, batch_size: int) -> int:
        """Launcher calls captured in the decode graph of this batch size (0: none yet)."""
        slot = self._graphs.get(batch_size)
        return slot["kernels"] if slot else 0

    # ------------------------------------------------------------------ a decode step prepared ahead
    # While the GPU runs step n, the host can already do step n + 1's bookkeeping if it is a decode-only
    # step of known requests: check, reserve pages, grow the requests, pack block tables, positions and
    # lengths into pinned memory.  Only the token ids are missing (they are being sampled).  Once they are
    # known they are written into the packed buffer and the step is launched: one small copy and a graph
    # replay stand between the read-back of step n's tokens and the start of step n + 1.
    def prepare_decode_ahead(self, rids: Sequence[object]) -> Optional["PreparedDecode"]:
        """Reserves and packs a step of one token (still unknown) for each request.  None if such a
        step cannot be prepared ahead: no captured graph for this batch size yet, a cache with
        fixed-size state (a reservation there cannot be taken back), or no pages (the scheduler then
        decides whom to preempt).  The requests are longer by one token until the step is launched
        or cancelled."""
        R = len(rids)
        slot = self._graphs.get(R)
        if (slot is None or slot["graph"] is None or self.cache._states
                or self._graph_key([StepEntry(r, [0], [0]) for r in rids]) != R):
            return None
        entries = [StepEntry(r, [0], [0]) for r in rids]
        try:
            host, total = self.prepare(entries, min_blocks=self._graph_width, into=slot["buf"],
                                       replay_width=self._graph_width, defer_send=True)
        except (OutOfPages, EngineError):
            return None
        return PreparedDecode(list(rids), host, total, slot, self._builder.last_ring_slot)

    def launch_prepared(self, prep: "PreparedDecode", tokens: Sequence[int]) -> torch.Tensor:
        """Fills in the tokens of a step prepared ahead and runs it (a graph replay)."""
        V = self.config.vocab_size
        if len(tokens) != len(prep.rids) or any(not 0 <= int(t) < V for t in tokens):
            self.cancel_prepared(prep)
            raise EngineError(f"a prepared step needs one token id in [0, {V}) per request")
        prep.host[:len(tokens)] = torch.as_tensor(list(tokens), dtype=torch.int32)   # token ids lead the packed layout
        try:
            with torch.cuda.device(self.device):
                self._builder.send(prep.host, prep.total, prep.slot["buf"], ring_slot=prep.ring_slot)
                prep.slot["graph"].replay()
        except BaseException:
            self.cancel_prepared(prep)
            raise
        prep.rids_done = True
        self.cache.release_passed_many(prep.rids)
        self.steps_run += 1
        self.tokens_run += len(prep.rids)
        return prep.slot["logits"]

    def cancel_prepared(self, prep: "PreparedDecode") -> None:
        """Takes a prepared step back: every request that is still live loses the token it was grown by."""
        if prep.rids_done:
            return
        prep.rids_done = True
        for rid in prep.rids:
            if self.cache.has(rid):
                self.cache.truncate(rid, self.cache.length(rid) - 1)

    def decode_native(self, rids: Sequence[object], tokens: Sequence[int], positions: Sequence[int],
                      token_source: Optional[torch.Tensor] = None, wait: bool = True):
        """A decode-only greedy step of live requests through the C entry point (``csrc/decode_step.h``):
        one token each at the given positions (a lower position than a request's length rewinds it first).
        Returns (logits, sampled tokens on the device, the same in pinned host memory), or None when the
        step is not one the C path takes (no captured graph of this batch size yet, a request the cache
        does not hold, a refusal): the caller then takes :meth:`step`, which explains a refusal."""
        R = len(rids)
        slot = self._graphs.get(R)
        if (not self.options.native_decode or slot is None or slot["graph"] is None or self.cache._states
                or not all(getattr(b.mixer, "graph_safe", True) for b in self.model.blocks)):
            return None
        from . import native_step
        nat = slot.get("native")
        if nat is None:
            nat = slot["native"] = native_step.NativeDecodeSlot(self, R, slot)
        with torch.cuda.device(self.device):
            rc, host = native_step.decode_step(self, nat, rids, tokens, positions, token_source, wait)
        if rc != native_step.SUCCESS:
            return None
        self.cache.release_passed_many(rids)
        self.steps_run += 1
        self.tokens_run += R
        self.native_steps += 1
        return slot["logits"], nat.sampled, host

    def step(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one batch; returns float32 logits [wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``.  The result of a graph
        replay is overwritten by the next step of the same batch size.

        ``token_source``: an int32 tensor on the device with one token id per token of the step, used
        INSTEAD of the entries' own ids (which are then placeholders): the tokens a sampler has just
        chosen go into the next step without a round trip through the host.  Their range is the
        sampler's responsibility (it chooses among the vocabulary).

        A step that fails changes nothing: a refusal (bad entries, no pages) comes before
        anything is reserved, and if the model raises after the requests have grown, they are
        rolled back to their lengths before the step and requests that the step created are
        freed (the reference rolls a failed chunk back to a coherent prefix likewise:
        src/core/engine_prefill_coordinator.cpp:296-304)."""
        if not entries:
            return torch.empty((0, self.config.vocab_size), dtype=torch.float32, device=self.device)
        self._grown = None
        try:
            with torch.cuda.device(self.device):
                R = self._graph_key(entries)
                if R is not None:
                    logits = self._step_graph(entries, R, token_source)
                    T = R
                else:
                    batch = self.prepare(entries)
                    if token_source is not None:
                        batch.token_ids.copy_(token_source)
                    logits = self.model.forward(batch, self.cache.views)
                    T = batch.T
        except BaseException:
            self._roll_back()
            raise
        self.cache.release_passed_many([e.rid for e in entries])
        self.steps_run += 1
        self.tokens_run += T
        return logits

    def _roll_back(self) -> None:
        """Puts every request of a failed step back to its length before the step; a request
        the step created is freed.  A request whose fixed-size state may have been advanced
        cannot go back by part of its length: it is freed too (its owner starts it again).
        Nothing to do if the step failed before the requests were grown."""
        grown, self._grown = self._grown, None
        if grown is None:
            return
        cache = self.cache
        entries, was_new = grown
        for e, new in zip(entries, was_new):
            if not cache.has(e.rid):
                continue
            if new:
                cache.free_request(e.rid)
                continue
            try:
                cache.truncate(e.rid, cache.length(e.rid) - len(e.tokens))
            except ValueError:
                cache.free_request(e.rid)
