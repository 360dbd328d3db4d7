"""The step function's host side without a GPU: what ``Engine.step`` checks, reserves, packs and
gives back.  The model is a stand-in that runs no kernel: it records the batch it is handed and
returns a logits row per wanted place that names the token and its position, so the test can see
that the right tokens arrive at the right positions with the right block tables.  (The kernels
behind the same call are covered by the GPU tests.)"""
import contextlib

import pytest
import torch

import tiny
from blackwellllm_b200.cache.pages import OutOfPages
from blackwellllm_b200.config.registry import parse_config
from blackwellllm_b200.engine.engine import Engine, EngineError, EngineOptions, StepEntry
from blackwellllm_b200.parts.base import FixedStateRequest, PagedKVRequest

WINDOW = 24


class StandInModel:
    """Two cache groups (all keys; a window) and one fixed-size state, no arithmetic."""

    def __init__(self, vocab):
        self.vocab = vocab
        self.blocks = []          # no mixer objects: nothing forbids a graph, graphs are switched off anyway
        self.batches = []

    def cache_requests(self):
        return [PagedKVRequest(2, 16, None), PagedKVRequest(1, 16, WINDOW), FixedStateRequest((3,), torch.float32), None]

    def forward(self, batch, views):
        self.batches.append(batch)
        rows = batch.logit_rows.tolist()
        out = torch.zeros((len(rows), self.vocab), dtype=torch.float32)
        for i, t in enumerate(rows):
            out[i, 0] = float(batch.token_ids[t])
            out[i, 1] = float(batch.positions[t])
            out[i, 2] = float(batch.req_of_token[t])
        return out


@pytest.fixture
def engine(monkeypatch):
    # the step selects its CUDA device around the kernels; there is none here and the stand-in needs none
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    cfg = parse_config(tiny.CONFIGS["llama"][0])
    model = StandInModel(cfg.vocab_size)
    opts = EngineOptions(dtype="float32", page_size=8, num_pages=12, max_requests=3, max_batch_tokens=64,
                         cuda_graphs=False, device="cpu")
    return Engine(cfg, model, opts), model


def test_a_mixed_step_arrives_whole(engine):
    eng, model = engine
    lg = eng.step([StepEntry("a", [5, 6, 7, 8, 9, 10, 11, 12, 13, 14], [0, 9]), StepEntry("b", [3, 4], [])])
    assert lg[:, :3].tolist() == [[5, 0, 0], [14, 9, 0]]
    lg = eng.step([StepEntry("b", [7], [0]), StepEntry("a", [1, 2, 3], [2]), StepEntry("c", [9, 9], [1])])
    assert lg[:, :3].tolist() == [[7, 2, 0], [3, 12, 1], [9, 1, 2]]          # order of the entries and of want
    b = model.batches[-1]
    assert (b.T, b.R) == (6, 3) and b.cu_q.tolist() == [0, 1, 4, 6]
    assert b.token_ids.tolist() == [7, 1, 2, 3, 9, 9] and b.positions.tolist() == [2, 10, 11, 12, 0, 1]
    assert b.q_start.tolist() == [2, 10, 0] and b.kv_len.tolist() == [3, 13, 2] and b.rids == ["b", "a", "c"]
    assert sorted(b.state_slot.tolist()) == [0, 1, 2]
    for g in (0, 1):   # every request's block-table row, padded with -1, as the cache manager holds it
        for r, rid in enumerate(b.rids):
            row = b.block_tables[g][r].tolist()
            held = eng.cache.block_table(rid, g)
            assert row[:len(held)] == held and all(p == -1 for p in row[len(held):])
    assert eng.steps_run == 2 and eng.tokens_run == 18
    eng.cache.check_invariants()


def test_the_window_gives_pages_back_after_the_step(engine):
    eng, _ = engine
    eng.step([StepEntry("a", list(range(40)), [39])])
    assert eng.cache.block_table("a", 0) == [0, 1, 2, 3, 4]                   # all keys: 5 pages of 8
    assert eng.cache.block_table("a", 1)[:2] == [-1, -1]                       # the window of 24 has passed 2 pages
    assert eng.cache.free_pages() == [7, 9]
    eng.end_request("a")
    assert eng.cache.free_pages() == [12, 12] and not eng.has_request("a")


def test_state_is_zeroed_when_a_slot_is_handed_out_again(engine):
    eng, _ = engine
    eng.step([StepEntry("a", [1], [])])
    slot = eng.cache.slot("a")
    eng.cache.views[2].state[slot] = 7.0
    eng.end_request("a")
    eng.step([StepEntry("b", [1], [])])
    assert eng.cache.slot("b") == slot and eng.cache.views[2].state[slot].tolist() == [0.0, 0.0, 0.0]


def test_refusals_change_nothing(engine):
    eng, model = engine
    eng.step([StepEntry("a", list(range(40)), [39])])       # 5 of the 12 pages of the first group
    before = (eng.cache.free_pages(), eng.cache.length("a"), eng.cache.slots.num_free, len(model.batches))
    bad = [
        ([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])], EngineError, "twice"),
        ([StepEntry("a", [], [])], EngineError, "at least one token"),
        ([StepEntry("a", [1, 999], [0])], EngineError, "token id 999"),
        ([StepEntry("a", [-1], [0])], EngineError, "token id -1"),
        ([StepEntry("a", [1, 2], [2])], EngineError, "wanted place 2"),
        ([StepEntry("n", [1], [-1])], EngineError, "wanted place -1"),
        ([StepEntry("a", [1] * 65, [])], EngineError, "max_batch_tokens=64"),
        ([StepEntry("a", [1], [0]), StepEntry("n", [1] * 63, [])], OutOfPages, "pages per group"),       # 1 + 8 pages, 7 are free
        ([StepEntry("n1", [1], []), StepEntry("n2", [1], []), StepEntry("n3", [1], [])], OutOfPages, "request slots"),
    ]
    for entries, err, text in bad:
        with pytest.raises(err, match=text):
            eng.step(entries)
        assert (eng.cache.free_pages(), eng.cache.length("a"), eng.cache.slots.num_free, len(model.batches)) == before
        assert not any(eng.has_request(r) for r in ("n", "n1", "n2", "n3"))
    eng.cache.check_invariants()
    assert eng.step([]).shape == (0, eng.config.vocab_size)                   # an empty step is no step
    assert eng.steps_run == 1


class NoStateModel(StandInModel):
    """One cache group, no fixed-size state; fails on demand after the requests have grown."""
    fail = None

    def cache_requests(self):
        return [PagedKVRequest(2, 16, None)]

    def forward(self, batch, views):
        if self.fail is not None:
            raise self.fail
        return super().forward(batch, views)


def test_a_forward_that_raises_leaves_lengths_and_pages_as_they_were(monkeypatch):
    """The model fails after the step's pages were reserved and the requests grown (a kernel refusing a
    size, a CUDA error): every request is back at its length before the step, a request the step created
    is gone, no page is lost; the next step runs as if nothing had happened."""
    from blackwellllm_b200.kernels.ops import KernelError
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    cfg = parse_config(tiny.CONFIGS["llama"][0])
    model = NoStateModel(cfg.vocab_size)
    eng = Engine(cfg, model, EngineOptions(dtype="float32", page_size=8, num_pages=12, max_requests=3,
                                           max_batch_tokens=64, cuda_graphs=False, device="cpu"))
    eng.step([StepEntry("a", list(range(20)), [19]), StepEntry("b", [1, 2, 3], [])])
    before = (eng.cache.free_pages(), eng.cache.length("a"), eng.cache.length("b"), eng.cache.slots.num_free,
              eng.cache.block_table("a", 0), eng.steps_run)
    model.fail = KernelError("attention: refused")
    with pytest.raises(KernelError, match="refused"):
        eng.step([StepEntry("a", [5, 6, 7, 8, 9], [4]), StepEntry("n", list(range(17)), []), StepEntry("b", [4], [0])])
    assert (eng.cache.free_pages(), eng.cache.length("a"), eng.cache.length("b"), eng.cache.slots.num_free,
            eng.cache.block_table("a", 0), eng.steps_run) == before
    assert not eng.has_request("n")
    eng.cache.check_invariants()
    model.fail = None
    lg = eng.step([StepEntry("a", [5], [0])])
    assert lg[0, :2].tolist() == [5, 20]                                       # position 20: nothing of the failed step stayed


def test_a_failed_step_frees_a_request_whose_state_cannot_go_back(engine):
    """Fixed-size state cannot be rolled back by part of a request's length: such a request is freed."""
    eng, model = engine
    eng.step([StepEntry("a", list(range(10)), [])])

    def boom(batch, views):
        raise RuntimeError("boom")
    model.forward = boom
    with pytest.raises(RuntimeError, match="boom"):
        eng.step([StepEntry("a", [1, 2], [1]), StepEntry("n", [3], [0])])
    assert not eng.has_request("a") and not eng.has_request("n")
    assert eng.cache.free_pages() == [12, 12] and eng.cache.slots.num_free == 3
    eng.cache.check_invariants()


def test_the_first_step_of_a_decode_batch_size_runs_the_model_once(monkeypatch):
    """Decode-only steps are replayed from a graph per batch size.  The step that records the graph must run
    the model once, not twice: a mixer with state of its own would otherwise advance its state twice for
    one token.  The graph here is a stand-in that records what a capture records (the launches, without
    running them) and runs them at replay; the model counts what actually ran."""
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    capturing = []

    class FakeGraph:
        def __init__(self):
            self.recorded = []

        def replay(self):
            for fn in self.recorded:
                fn()

    @contextlib.contextmanager
    def fake_capture(graph):
        capturing.append(graph)
        try:
            yield
        finally:
            capturing.pop()
    monkeypatch.setattr(torch.cuda, "CUDAGraph", FakeGraph)
    monkeypatch.setattr(torch.cuda, "graph", fake_capture)

    class StatefulModel(StandInModel):
        """Per request slot a count of the tokens it has seen (its 'state'), bumped by every run."""

        def __init__(self, vocab):
            super().__init__(vocab)
            self.seen = torch.zeros(8, dtype=torch.int64)
            self.runs = 0

        def cache_requests(self):
            return [PagedKVRequest(2, 16, None)]

        def _run(self, batch, out):
            self.runs += 1
            for t in range(batch.T):
                self.seen[int(batch.state_slot[int(batch.req_of_token[t])])] += 1
            for i, t in enumerate(batch.logit_rows.tolist()):
                out[i, 0], out[i, 1] = float(batch.token_ids[t]), float(batch.positions[t])

        def forward(self, batch, views):
            out = torch.zeros((len(batch.logit_rows), self.vocab), dtype=torch.float32)
            if capturing:
                capturing[-1].recorded.append(lambda: self._run(batch, out))    # recorded, not run
            else:
                self._run(batch, out)
            return out

    cfg = parse_config(tiny.CONFIGS["llama"][0])
    model = StatefulModel(cfg.vocab_size)
    eng = Engine(cfg, model, EngineOptions(dtype="float32", page_size=8, num_pages=12, max_requests=3,
                                           max_batch_tokens=64, cuda_graphs=True, graph_after=1, device="cpu"))
    eng.step([StepEntry("a", [1, 2, 3], []), StepEntry("b", [4], [])])      # prompts: not a decode-only step
    assert model.runs == 1 and eng.graph_kernel_count(2) == 0
    slot_a, slot_b = eng.cache.slot("a"), eng.cache.slot("b")
    lg = eng.step([StepEntry("a", [7], [0]), StepEntry("b", [8], [0])])     # the first decode step of batch size 2
    assert model.runs == 2                                                   # once: not a warm-up run and a replay
    assert model.seen[slot_a] == 4 and model.seen[slot_b] == 2
    assert lg[:, :2].tolist() == [[7, 3], [8, 1]]
    lg = eng.step([StepEntry("b", [9], [0]), StepEntry("a", [6], [0])])     # replayed
    assert model.runs == 3 and model.seen[slot_a] == 5 and model.seen[slot_b] == 3
    assert lg[:, :2].tolist() == [[9, 2], [6, 4]]

    # A batch size recorded at its third decode-only step: two uncaptured steps, then a step that captures (which
    # runs nothing) and replays, then replays.  Every step runs the model once.
    model = StatefulModel(cfg.vocab_size)
    eng = Engine(cfg, model, EngineOptions(dtype="float32", page_size=8, num_pages=12, max_requests=3,
                                           max_batch_tokens=64, cuda_graphs=True, graph_after=3, device="cpu"))
    eng.step([StepEntry("a", [1, 2, 3], []), StepEntry("b", [4], [])])
    slot_a, slot_b = eng.cache.slot("a"), eng.cache.slot("b")
    for k, (ta, tb) in enumerate([(7, 8), (9, 6), (5, 4), (3, 2)]):
        lg = eng.step([StepEntry("a", [ta], [0]), StepEntry("b", [tb], [0])])
        assert model.runs == 2 + k and model.seen[slot_a] == 4 + k and model.seen[slot_b] == 2 + k
        assert lg[:, :2].tolist() == [[ta, 3 + k], [tb, 1 + k]]
        assert (eng.graph_kernel_count(2) > 0 or eng._graphs[2]["graph"] is not None) == (k >= 2)


def test_no_device_no_engine():
    cfg = tiny.CONFIGS["llama"][0]
    with pytest.raises(EngineError, match="no CPU path"):
        Engine.from_config(cfg, device="cpu")
    with pytest.raises(EngineError, match="dtype must be"):
        Engine.from_config(cfg, dtype="float16")


# ---------------------------------------------------------------- the Python entry point above the step function
class RuleModel(StandInModel):
    """Logits that make greedy decoding follow a rule: after a token t at position p the best next
    token is (t + p) % vocab."""

    def cache_requests(self):
        return [PagedKVRequest(2, 16, None)]

    def forward(self, batch, views):
        self.batches.append(batch)
        rows = batch.logit_rows.tolist()
        out = torch.zeros((len(rows), self.vocab), dtype=torch.float32)
        for i, t in enumerate(rows):
            out[i, (int(batch.token_ids[t]) + int(batch.positions[t])) % self.vocab] = 1.0
        return out


class ArgmaxSampler:
    def __init__(self, device):
        pass

    def sample_async(self, logits, params, seeds, draw_index, generated=None):
        assert all(p.greedy for p in params)
        return logits.argmax(dim=1)

    def sample(self, logits, params, seeds, draw_index, generated=None):
        return self.sample_async(logits, params, seeds, draw_index, generated).tolist()


def rule_continuation(prompt, n, vocab):
    out, last, pos = [], prompt[-1], len(prompt) - 1
    for _ in range(n):
        last = (last + pos) % vocab
        pos += 1
        out.append(last)
    return out


@pytest.fixture
def llm(monkeypatch):
    import dataclasses

    from blackwellllm_b200.engine import llm as llm_module
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    models = []

    def from_config(raw, seed=0, std=0.02, options=None):
        cfg = parse_config(raw)
        models.append(RuleModel(cfg.vocab_size))
        return Engine(cfg, models[-1], dataclasses.replace(options, device="cpu", cuda_graphs=False))
    monkeypatch.setattr(llm_module.Engine, "from_config", staticmethod(from_config))
    monkeypatch.setattr(llm_module, "Sampler", ArgmaxSampler)

    def make(**kw):
        from blackwellllm_b200 import BlackwellEngine, InferenceConfig
        rq = InferenceConfig(max_context_length=kw.pop("ctx", 96), max_batch_size=kw.pop("batch", 3))
        e = BlackwellEngine(None, rq, config=tiny.CONFIGS["llama"][0], page_size=8, **kw)
        return e, models[-1]
    return make


def test_generate_batches_requests_and_returns_them_in_order(llm):
    from blackwellllm_b200 import SamplingParams
    e, model = llm(max_batch_tokens=16)
    V = e.vocab_size
    prompts = [[3, 4, 5], list(range(10, 40)), [7], [9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 1, 2, 3, 4, 5, 6, 7]]
    res = e.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))
    assert [r.prompt_token_ids for r in res] == prompts
    for p, r in zip(prompts, res):
        assert r.token_ids == rule_continuation(p, 6, V) and r.finish_reason == "limit"
    assert all(b.T <= 16 for b in model.batches)                              # the token budget of a step
    assert any(b.R > 1 and max(b.h_q_len) > 1 and min(b.h_q_len) == 1 for b in model.batches)   # portions beside decoded tokens
    assert e.engine.cache.free_pages() == [3 * 12] and e.scheduler.finished == {} and not e.scheduler.has_work()
    # one prompt, one SamplingParams per prompt, and the wrong number of them
    one = e.generate([3, 4, 5], SamplingParams(temperature=0.0, max_new_tokens=2))
    assert len(one) == 1 and one[0].token_ids == rule_continuation([3, 4, 5], 2, V)
    with pytest.raises(EngineError, match="one SamplingParams per prompt"):
        e.generate(prompts, [SamplingParams(temperature=0.0)])


def test_generate_with_too_few_pages_preempts_and_still_follows_the_rule(llm):
    from blackwellllm_b200 import SamplingParams
    e, _ = llm(max_batch_tokens=32, num_pages=7, ctx=48)
    V = e.vocab_size
    prompts = [list(range(1, 18)), list(range(2, 20)), list(range(5, 15))]
    res = e.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=14, ignore_eos=True))
    for p, r in zip(prompts, res):
        assert r.token_ids == rule_continuation(p, 14, V)
    assert e.scheduler.stats.preemptions > 0 and sum(r.preemptions for r in res) == e.scheduler.stats.preemptions
    assert e.engine.cache.free_pages() == [7]
    e.engine.cache.check_invariants()


def test_decode_steps_prepared_ahead_give_the_same_tokens_and_are_taken_back_on_a_surprise(monkeypatch):
    """generate() prepares the next decode step while the current one runs.  With stand-ins for the graph
    (what a capture records runs at replay) and a model that follows a rule: the tokens are those of the
    unpipelined run; a request that ends on an end-of-sequence token (which nobody could know ahead)
    makes the engine take the prepared step back, and no page or slot is lost."""
    import dataclasses

    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, SamplingParams
    from blackwellllm_b200.engine import llm as llm_module
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    capturing = []

    class FakeGraph:
        def __init__(self):
            self.recorded = []

        def replay(self):
            for fn in self.recorded:
                fn()

    @contextlib.contextmanager
    def fake_capture(graph):
        capturing.append(graph)
        try:
            yield
        finally:
            capturing.pop()
    monkeypatch.setattr(torch.cuda, "CUDAGraph", FakeGraph)
    monkeypatch.setattr(torch.cuda, "graph", fake_capture)

    class CapturableRuleModel(RuleModel):
        def forward(self, batch, views):
            out = torch.zeros((len(batch.logit_rows), self.vocab), dtype=torch.float32)

            def run():
                out.zero_()
                for i, t in enumerate(batch.logit_rows.tolist()):
                    out[i, (int(batch.token_ids[t]) + int(batch.positions[t])) % self.vocab] = 1.0
            if capturing:
                capturing[-1].recorded.append(run)
            else:
                self.batches.append(batch)
                run()
            return out

    engines = []

    def from_config(raw, seed=0, std=0.02, options=None):
        cfg = parse_config(raw)
        engines.append(Engine(cfg, CapturableRuleModel(cfg.vocab_size), dataclasses.replace(options, device="cpu")))
        return engines[-1]
    monkeypatch.setattr(llm_module.Engine, "from_config", staticmethod(from_config))
    monkeypatch.setattr(llm_module, "Sampler", ArgmaxSampler)

    def run(pipeline, eos):
        raw = dict(tiny.CONFIGS["llama"][0], eos_token_id=eos)
        e = BlackwellEngine(None, InferenceConfig(max_context_length=96, max_batch_size=3), config=raw, page_size=8,
                            max_batch_tokens=32, cuda_graphs=True)
        e.pipeline = pipeline
        e.engine.options.graph_after = 1     # every batch size is recorded at its first decode step
        launched = {"ahead": 0, "cancelled": 0}
        real_launch, real_cancel = e.engine.launch_prepared, e.engine.cancel_prepared

        def launch(prep, tokens):
            launched["ahead"] += 1
            return real_launch(prep, tokens)

        def cancel(prep):
            launched["cancelled"] += 0 if prep.rids_done else 1
            return real_cancel(prep)
        e.engine.launch_prepared, e.engine.cancel_prepared = launch, cancel
        prompts = [[3, 4, 5], list(range(10, 27)), [7, 8]]
        res = e.generate(prompts, [SamplingParams(temperature=0.0, max_new_tokens=n) for n in (20, 12, 16)])
        assert e.engine.cache.free_pages() == [3 * 12] and e.engine.cache.slots.num_free == 3
        e.engine.cache.check_invariants()
        return [(r.token_ids, r.finish_reason) for r in res], launched

    V = tiny.CONFIGS["llama"][0]["vocab_size"]
    plain, n0 = run(False, eos=None)
    piped, n1 = run(True, eos=None)
    assert piped == plain and n0["ahead"] == 0 and n1["ahead"] >= 10       # most decode steps were prepared ahead
    assert [t for t, _ in plain][0] == rule_continuation([3, 4, 5], 20, V)
    # the sixth token of the first request is now an end-of-sequence token: nobody knows before it is sampled
    eos = plain[0][0][5]
    plain_eos, _ = run(False, eos=eos)
    piped_eos, n2 = run(True, eos=eos)
    assert piped_eos == plain_eos and plain_eos[0][1] == "eos" and len(plain_eos[0][0]) <= 6
    assert n2["cancelled"] >= 1 and n2["ahead"] >= 5


def test_position_addressed_calls_reconcile_the_cache(llm):
    from blackwellllm_b200 import DecodeRequest
    e, model = llm(max_batch_tokens=8, batch=2)
    V = e.vocab_size
    ids = list(range(20, 41))                                                  # 21 tokens: three steps of at most 8
    nxt = e.prefill(ids, 0, 0.0, 1.0, 0)
    assert nxt == rule_continuation(ids, 1, V)[0] and [b.T for b in model.batches] == [8, 8, 5]
    assert [len(b.logit_rows) for b in model.batches] == [0, 0, 1]            # logits only after the last token
    nxt2 = e.forward(nxt, 21, 0.0, 1.0, 0)
    assert [nxt, nxt2] == rule_continuation(ids, 2, V)
    # an earlier position rewinds the sequence to it; a later one would leave a gap
    again = e.forward(ids[10], 10, 0.0, 1.0, 0)
    assert again == (ids[10] + 10) % V and e.engine.cache.length(("seq", 0)) == 11
    with pytest.raises(EngineError, match="gap"):
        e.forward(1, 13, 0.0, 1.0, 0)
    with pytest.raises(EngineError, match="do not fit max_context_length"):
        e.prefill([1] * 97, 0, 0.0, 1.0, 1)
    # one token each of distinct sequences
    out = e.forward_batch([DecodeRequest(0, 5, 11), DecodeRequest(1, 6, 0)])
    assert out == [(5 + 11) % V, 6 % V]
    with pytest.raises(EngineError, match="twice"):
        e.forward_batch([DecodeRequest(0, 5, 12), DecodeRequest(0, 6, 13)])
    with pytest.raises(EngineError, match="at least one request"):
        e.forward_batch([])
    e.rewind(0, 4)
    assert e.engine.cache.length(("seq", 0)) == 4
    with pytest.raises(EngineError, match="unknown sequence"):
        e.rewind(5, 0)
    e.release_sequence(0); e.reset_state(1); e.release_sequence(7)            # the last one never existed
    assert e.engine.cache.live == [] and e.engine.cache.free_pages() == [2 * 12]


def test_sampler_uploads_what_the_kernels_expect(monkeypatch):
    """The sampler's host side: the (temperature, top_p, uniform number) rows and the penalized ids with their
    row boundaries, as the kernels receive them.  The kernels are stand-ins that record their arguments, and
    pinned memory is ordinary memory here."""
    import types

    from blackwellllm_b200 import SamplingParams
    from blackwellllm_b200.sampling import sampler as S
    from blackwellllm_b200.sampling.params import uniform
    seen = {}

    def empty(*size, pin_memory=False, **kw):
        return torch.empty(*size, **kw)
    shim = types.SimpleNamespace(**{k: getattr(torch, k) for k in ("float32", "int32", "Tensor", "device", "tensor")}, empty=empty)
    monkeypatch.setattr(S, "torch", shim)
    monkeypatch.setattr(S.ops, "sample", lambda logits, t, p, u: seen.update(sample=(t, p, u)) or torch.zeros(logits.shape[0], dtype=torch.int32))
    monkeypatch.setattr(S.ops, "repetition_penalty", lambda logits, ids, begin, pen: seen.update(pen=(ids, begin, pen)))
    sm = S.Sampler(torch.device("cpu"))
    logits = torch.zeros((4, 16))
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, top_p=0.5),
              SamplingParams(temperature=1.3, top_p=1.0, repetition_penalty=1.5, repetition_window=2),
              SamplingParams(temperature=0.0, repetition_penalty=2.0, repetition_window=0)]
    seeds, draws = [11, 12, 13, 14], [0, 5, 9, 2]
    out = sm.sample(logits, params, seeds, draws, [[1, 2], [3], [4, 5, 6], [7, 8, 9, 7]])
    assert out == [0, 0, 0, 0]
    t, p, u = seen["sample"]
    assert t.tolist() == pytest.approx([0.0, 0.7, 1.3, 0.0]) and p.tolist() == pytest.approx([0.9, 0.5, 1.0, 0.9])
    assert u.tolist() == pytest.approx([0.0, uniform(12, 5), uniform(13, 9), 0.0])     # greedy rows draw nothing
    ids, begin, pen = seen["pen"]
    assert ids.tolist() == [5, 6, 7, 8, 9, 7] and begin.tolist() == [0, 0, 0, 2, 6]     # window 2; window 0: everything emitted
    assert pen.tolist() == pytest.approx([1.0, 1.0, 1.5, 2.0])
    # all greedy, no penalty: nothing is uploaded
    seen.clear()
    sm.sample(logits[:2], [SamplingParams(temperature=0.0)] * 2, [1, 2], [0, 0], [[1], [2]])
    assert seen == {"sample": (None, None, None)}
    with pytest.raises(ValueError, match="one SamplingParams per logits row"):
        sm.sample(logits, params[:2], seeds, draws)
