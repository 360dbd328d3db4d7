"""The cache manager's bookkeeping and the scheduler's decisions (no GPU: the
manager runs without tensors, and a fake step stands in for the model)."""
import random

import pytest
from hypothesis import example, given, settings, strategies as st

from blackwellllm_b200.cache.manager import CacheManager
from blackwellllm_b200.cache.pages import OutOfPages
from blackwellllm_b200.engine.scheduler import RequestRefused, Scheduler
from blackwellllm_b200.parts.base import FixedStateRequest, PagedKVRequest
from blackwellllm_b200.sampling.params import SamplingParams, philox4x32, uniform

FULL = PagedKVRequest(2, 16, None)
WIN = PagedKVRequest(2, 16, 20)


def test_allocator_basics():
    """Pages through the manager: all or nothing, lowest ids first, the page just freed is used again first."""
    cm = CacheManager([FULL], page_size=8, num_pages=4, max_requests=2)
    cm.add_request("a")
    assert cm.append("a", 24) == 0
    assert cm.block_table("a", 0) == [0, 1, 2] and cm.free_pages() == [1]
    cm.add_request("b")
    with pytest.raises(OutOfPages):
        cm.append("b", 9)                        # needs two pages, one is free
    assert cm.free_pages() == [1] and cm.length("b") == 0 and cm.block_table("b", 0) == []   # never a part of them
    cm.truncate("a", 16)                         # gives page 2 back
    assert cm.free_pages() == [2]
    assert cm.append("b", 8) == 0
    assert cm.block_table("b", 0) == [2]         # LIFO: the page just freed is used again first
    cm.check_invariants()
    with pytest.raises(ValueError):
        cm.append("a", 0)
    with pytest.raises(KeyError):
        cm.free_request("never added")
    with pytest.raises(ValueError):
        CacheManager([FULL], page_size=8, num_pages=0, max_requests=2)


def test_slots():
    cm = CacheManager([FULL], page_size=8, num_pages=4, max_requests=2)
    a, b = cm.add_request("a"), cm.add_request("b")
    assert {a, b} == {0, 1} and cm.slots.num_free == 0
    with pytest.raises(OutOfPages):
        cm.add_request("c")
    with pytest.raises(ValueError):
        cm.add_request("a")                      # already live
    cm.free_request("a")
    assert cm.slots.num_free == 1
    with pytest.raises(KeyError):
        cm.free_request("a")                     # not twice
    assert cm.add_request("c") == a              # the slot just freed is used again
    cm.check_invariants()


def test_groups_by_need():
    cm = CacheManager([FULL, WIN, FULL, None, FixedStateRequest((4,)), WIN], page_size=8,
                      num_pages=[10, 6], max_requests=3)
    assert len(cm.groups) == 2
    assert cm.groups[0].entries == [0, 2] and cm.groups[1].entries == [1, 5]
    assert cm.views[0].group == 0 and cm.views[1].group == 1 and cm.views[3] is None


def test_append_all_or_nothing_and_free():
    cm = CacheManager([FULL, WIN], page_size=8, num_pages=[10, 2], max_requests=2)
    cm.add_request("a")
    assert cm.pages_needed("a", 17) == [3, 3]
    with pytest.raises(OutOfPages):
        cm.append("a", 17)  # group 1 has 2 pages: nothing may change
    assert cm.free_pages() == [10, 2] and cm.length("a") == 0
    assert cm.append("a", 16) == 0
    assert cm.free_pages() == [8, 0] and cm.length("a") == 16
    cm.check_invariants()
    cm.free_request("a")
    assert cm.free_pages() == [10, 2] and not cm.has("a")
    cm.check_invariants()


def test_window_gives_pages_back():
    cm = CacheManager([WIN], page_size=8, num_pages=5, max_requests=1)
    cm.add_request("a")
    total_freed = 0
    for _ in range(100):   # 100 tokens through a pool of 5 pages of 8: only the window stays
        cm.append("a", 1)
        total_freed += cm.release_passed("a")
        cm.check_invariants()
        held = [p for p in cm.block_table("a", 0) if p >= 0]
        # the next query at position L needs keys >= L - 19
        first_needed = max(0, cm.length("a") - 19) // 8
        assert cm.block_table("a", 0)[:first_needed] == [-1] * first_needed
        assert all(p >= 0 for p in cm.block_table("a", 0)[first_needed:])
        assert len(held) <= 4
    assert total_freed > 5  # pages were used again
    with pytest.raises(ValueError, match="released"):
        cm.truncate("a", 10)


def test_truncate_rewinds_pages():
    cm = CacheManager([FULL], page_size=8, num_pages=6, max_requests=1)
    cm.add_request("a")
    cm.append("a", 30)
    assert cm.free_pages() == [2]
    cm.truncate("a", 9)
    assert cm.length("a") == 9 and cm.free_pages() == [4]
    cm.check_invariants()
    cm.truncate("a", 0)
    assert cm.free_pages() == [6]


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 5), st.integers(0, 3), st.integers(1, 40)), min_size=1, max_size=80),
       st.integers(4, 24))
def test_no_page_lost_or_held_twice_under_random_orders(ops, num_pages):
    """Random admissions, growths, window releases, rewinds and ends: after every
    operation, held + free pages are exactly the pool and no page has two owners."""
    cm = CacheManager([FULL, WIN], page_size=8, num_pages=[num_pages, num_pages], max_requests=4)
    for rid, op, n in ops:
        if op == 0 and not cm.has(rid):
            try:
                cm.add_request(rid)
            except OutOfPages:
                assert cm.slots.num_free == 0
        elif op == 1 and cm.has(rid):
            before = (cm.free_pages(), cm.length(rid))
            try:
                cm.append(rid, n)
                cm.release_passed(rid)
            except OutOfPages:
                assert (cm.free_pages(), cm.length(rid)) == before
        elif op == 2 and cm.has(rid):
            cm.free_request(rid)
        elif op == 3 and cm.has(rid) and cm.length(rid) > 0:
            try:
                cm.truncate(rid, max(0, cm.length(rid) - n))
            except ValueError:
                pass
        cm.check_invariants()
    for rid in cm.live:
        cm.free_request(rid)
    assert cm.free_pages() == [num_pages, num_pages] and cm.slots.num_free == 4


# ------------------------------------------------------------------ scheduler

class FakeEngine:
    """Stands in for Engine.step: grows the cache as the engine does and 'samples'
    a token that is a function of the request's tokens so far, so a recompute
    after preemption must give the same continuation."""

    def __init__(self, cache):
        self.cache = cache
        self.batches = []

    def run(self, sched, plan):
        sampled = {}
        need = [0] * len(self.cache.groups)
        for e in plan.entries:
            rid = e.request.rid
            if not self.cache.has(rid):
                self.cache.add_request(rid)
            assert self.cache.length(rid) == e.request.num_computed
            self.cache.append(rid, len(e.tokens))  # raises OutOfPages if the plan was wrong
            self.cache.release_passed(rid)
            if e.samples:
                seen = e.request.tokens[: e.request.num_computed + len(e.tokens)]
                sampled[rid] = (sum(seen) * 31 + len(seen)) % 97 + 3
        self.batches.append([(e.request.rid, len(e.tokens)) for e in plan.entries])
        self.cache.check_invariants()
        return sched.commit(plan, sampled)


def drive(sched, fake, limit=10_000):
    out = []
    for _ in range(limit):
        if not sched.has_work():
            return out
        plan = sched.plan()
        assert plan.entries, "no progress"
        assert sum(len(e.tokens) for e in plan.entries) <= sched.max_batch_tokens
        out += fake.run(sched, plan)
    raise AssertionError("scheduler did not finish")


def expected_continuation(prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        t = (sum(toks) * 31 + len(toks)) % 97 + 3
        out.append(t)
        toks.append(t)
    return out


def test_portions_under_budget_and_chunk():
    cm = CacheManager([FULL], page_size=8, num_pages=64, max_requests=4)
    s = Scheduler(cm, max_batch_tokens=16, chunk=12)
    fake = FakeEngine(cm)
    r = s.add_request(list(range(1, 41)), SamplingParams(temperature=0, max_new_tokens=3))
    done = drive(s, fake)
    assert [b for b in fake.batches] == [[(0, 12)], [(0, 12)], [(0, 12)], [(0, 4)], [(0, 1)], [(0, 1)]]
    assert done[0].generated == expected_continuation(r.prompt, 3) and done[0].finish_reason == "limit"
    assert cm.free_pages() == [64]


def test_mixed_batches_decode_beside_portions():
    cm = CacheManager([FULL], page_size=8, num_pages=64, max_requests=4)
    s = Scheduler(cm, max_batch_tokens=16, chunk=12)
    fake = FakeEngine(cm)
    a = s.add_request([5] * 9, SamplingParams(temperature=0, max_new_tokens=6))
    b = s.add_request([7] * 40, SamplingParams(temperature=0, max_new_tokens=2))
    drive(s, fake)
    # first step: a's whole prompt (9) plus the first 7 tokens of b (budget 16)
    assert fake.batches[0] == [(0, 9), (1, 7)]
    # later: a decodes (1 token) beside portions of b
    assert fake.batches[1] == [(0, 1), (1, 12)]
    assert s.finished[a.rid].generated == expected_continuation(a.prompt, 6)
    assert s.finished[b.rid].generated == expected_continuation(b.prompt, 2)


def test_eos_and_context_limit():
    cm = CacheManager([FULL], page_size=8, num_pages=64, max_requests=2)
    first = expected_continuation([4, 4, 4], 1)[0]
    s = Scheduler(cm, eos_token_ids=[first])
    drive(s, FakeEngine(cm))
    r = s.add_request([4, 4, 4], SamplingParams(temperature=0, max_new_tokens=50))
    drive(s, FakeEngine(cm))
    assert r.finish_reason == "eos" and r.generated == [first]
    s2 = Scheduler(cm, max_context=6)
    r2 = s2.add_request([4, 4, 4], SamplingParams(temperature=0, max_new_tokens=50))
    drive(s2, FakeEngine(cm))
    assert r2.finish_reason == "ctx" and len(r2.prompt) + len(r2.generated) == 6
    r3 = s2.add_request([4, 4, 4], SamplingParams(temperature=0, max_new_tokens=50, ignore_eos=True))
    assert r3.params.ignore_eos
    with pytest.raises(RequestRefused, match="max_context"):
        s2.add_request([1] * 6)


def test_refused_when_it_could_never_run_alone():
    cm = CacheManager([FULL], page_size=8, num_pages=4, max_requests=2)
    s = Scheduler(cm)
    with pytest.raises(RequestRefused, match="pages"):
        s.add_request([1] * 30, SamplingParams(max_new_tokens=10))  # 39 cached tokens > 32
    s.add_request([1] * 30, SamplingParams(max_new_tokens=3))       # 32 cached tokens fit
    with pytest.raises(RequestRefused):
        s.add_request([])


def test_pages_run_out_preempts_latest_and_recomputes_the_same_tokens():
    # two requests of 14 + 12 tokens each need 4 pages of 8 at the end; the pool has 6
    cm = CacheManager([FULL], page_size=8, num_pages=6, max_requests=4)
    s = Scheduler(cm, max_batch_tokens=64)
    fake = FakeEngine(cm)
    a = s.add_request([3] * 14, SamplingParams(temperature=0, max_new_tokens=12))
    b = s.add_request([9] * 14, SamplingParams(temperature=0, max_new_tokens=12))
    drive(s, fake)
    assert s.stats.preemptions >= 1
    assert b.preemptions >= 1 and a.preemptions == 0   # the most recently admitted one yields
    assert a.generated == expected_continuation(a.prompt, 12)
    assert b.generated == expected_continuation(b.prompt, 12)  # recompute reproduces it
    assert cm.free_pages() == [6] and cm.slots.num_free == 4
    # the preempted request came back at the front and recomputed prompt + generated in one portion
    assert any(n > 14 for step in fake.batches for rid, n in step if rid == b.rid)


def test_admission_waits_for_slots_and_pages():
    cm = CacheManager([FULL], page_size=8, num_pages=8, max_requests=2)
    s = Scheduler(cm, max_batch_tokens=64)
    fake = FakeEngine(cm)
    reqs = [s.add_request([i + 1] * 10, SamplingParams(temperature=0, max_new_tokens=4)) for i in range(5)]
    drive(s, fake)
    assert max(len(b) for b in fake.batches) <= 2  # never more than the slots
    for r in reqs:
        assert r.generated == expected_continuation(r.prompt, 4)
    assert s.stats.admitted == 5 + s.stats.preemptions and s.stats.finished == 5


@settings(max_examples=25, deadline=None)
@given(st.integers(0, 10_000))
@example(512)   # every running request in its prompt, each needing a page, none free: one must yield
def test_scheduler_random_loads_always_finish_right(seed):
    rng = random.Random(seed)
    cm = CacheManager([FULL, WIN], page_size=8, num_pages=[rng.randint(8, 20)] * 2, max_requests=rng.randint(1, 4))
    s = Scheduler(cm, max_batch_tokens=rng.randint(4, 40), chunk=rng.choice([None, 3, 12]))
    fake = FakeEngine(cm)
    reqs = []
    for _ in range(rng.randint(1, 8)):
        p = [rng.randint(1, 50) for _ in range(rng.randint(1, 30))]
        reqs.append(s.add_request(p, SamplingParams(temperature=0, max_new_tokens=rng.randint(1, 20))))
    drive(s, fake)
    for r in reqs:
        assert r.generated == expected_continuation(r.prompt, r.params.max_new_tokens)
    assert cm.free_pages() == [g.num_pages for g in cm.groups] and cm.slots.num_free == cm.max_requests


def test_philox_stream():
    # Philox4x32-10 known-answer vectors (counter, key -> output) from the Random123 test suite
    assert philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    assert philox4x32((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    us = [uniform(7, i) for i in range(1000)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.45 < sum(us) / 1000 < 0.55
    assert uniform(7, 3) == us[3] and uniform(8, 3) != us[3]


def test_sampling_params_checks_and_penalty_window():
    with pytest.raises(ValueError):
        SamplingParams(temperature=-0.1)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(max_new_tokens=0)
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=0.0)
    with pytest.raises(ValueError):
        SamplingParams(repetition_window=-1)
    assert SamplingParams(temperature=0.0).greedy and SamplingParams(temperature=9e-6).greedy
    assert not SamplingParams(temperature=0.1).greedy
    gen = list(range(100))
    assert SamplingParams().penalized(gen) == ()                                   # off by default
    assert SamplingParams(repetition_penalty=1.0).penalized(gen) == ()             # <= 1 is off
    assert list(SamplingParams(repetition_penalty=1.2).penalized(gen)) == gen[-64:]
    assert list(SamplingParams(repetition_penalty=1.2, repetition_window=3).penalized(gen)) == [97, 98, 99]
    assert list(SamplingParams(repetition_penalty=1.2, repetition_window=0).penalized(gen)) == gen
    assert SamplingParams(repetition_penalty=1.2).penalized([]) == ()


def test_request_span_is_a_slice_of_prompt_plus_generated():
    from blackwellllm_b200.engine.scheduler import Request
    r = Request(0, [1, 2, 3, 4], SamplingParams(), 0, generated=[10, 11, 12])
    whole = r.tokens
    assert whole == [1, 2, 3, 4, 10, 11, 12]
    for start in range(len(whole) + 1):
        for n in range(len(whole) - start + 1):
            assert r.span(start, n) == whole[start:start + n], (start, n)


# ---------------------------------------------------------------------------------------------
# The host runtime's packed step against the same step put together call by call

def _pack(cm, entries, vocab=1000, min_blocks=0, max_tokens=10 ** 6, cap=1 << 16):
    import numpy as np
    from blackwellllm_b200.cache.manager import native
    R = len(entries)
    handles = np.array([cm.handle(r) for r, _, _ in entries], dtype=np.int32)
    n_tok = np.array([len(t) for _, t, _ in entries], dtype=np.int32)
    n_want = np.array([len(w) for _, _, w in entries], dtype=np.int32)
    tokens = np.array([x for _, t, _ in entries for x in t], dtype=np.int32)
    want = np.array([x for _, _, w in entries for x in w], dtype=np.int32)
    out = np.full(cap, -7, dtype=np.int32)
    meta = np.zeros(4 + len(cm.groups), dtype=np.int64)
    new_slots = np.zeros(R, dtype=np.int32)
    total = native().bwh_pack_step(cm._h, R, handles.ctypes.data, n_tok.ctypes.data, tokens.ctypes.data,
                                   n_want.ctypes.data, want.ctypes.data, vocab, min_blocks, max_tokens,
                                   out.ctypes.data, cap, meta.ctypes.data, new_slots.ctypes.data)
    if total >= 0:
        for (rid, _, _), h in zip(entries, handles):
            if not cm.has(rid):
                cm.adopt(rid, int(h))
    return int(total), out, meta


@pytest.mark.parametrize("seed", range(6))
def test_packed_step_equals_the_step_built_call_by_call(seed):
    import torch
    from blackwellllm_b200.cache import manager as M
    from batch_packer import pack_batch
    from blackwellllm_b200.engine.batch import BatchBuilder
    rng = random.Random(seed)
    pages = rng.randint(12, 30)
    a = CacheManager([FULL, WIN, FULL], page_size=8, num_pages=[pages, pages], max_requests=4)   # packed
    b = CacheManager([FULL, WIN, FULL], page_size=8, num_pages=[pages, pages], max_requests=4)   # call by call
    live, next_id = [], 0
    for step in range(40):
        entries = []
        for rid in list(live):
            if rng.random() < 0.6:
                n = rng.choice([1, 1, 1, 2, 5, 13])
                entries.append((rid, [rng.randrange(1000) for _ in range(n)], sorted(rng.sample(range(n), rng.randint(0, min(n, 2))))))
        while len(live) + sum(1 for e in entries if e[0] not in live) < 4 and rng.random() < 0.5:
            n = rng.randint(1, 30)
            entries.append((f"r{next_id}", [rng.randrange(1000) for _ in range(n)], [n - 1]))
            next_id += 1
        if not entries:
            continue
        rng.shuffle(entries)
        min_blocks = rng.choice([0, 0, 7])
        before = (a.free_pages(), a.slots.num_free, {r: a.length(r) for r in live})
        total, out, meta = _pack(a, entries, min_blocks=min_blocks)
        # the same step, call by call, on the twin
        need = [0, 0]
        for rid, t, _ in entries:
            pn = b.pages_needed(rid, len(t)) if b.has(rid) else [-(-len(t) // 8)] * 2
            need = [x + y for x, y in zip(need, pn)]
        if any(n > f for n, f in zip(need, b.free_pages())):
            assert total == M.ERR_OUT_OF_PAGES
            assert (a.free_pages(), a.slots.num_free, {r: a.length(r) for r in live}) == before   # nothing changed
            victim = rng.choice(live)                      # make room and go on
            a.free_request(victim); b.free_request(victim); live.remove(victim)
            continue
        assert total > 0
        segs, rows, t0 = [], [], 0
        for rid, t, w in entries:
            if not b.has(rid):
                b.add_request(rid)
                live.append(rid)
            q0 = b.append(rid, len(t))
            segs.append((rid, t, q0, q0 + len(t), b.slot(rid)))
            rows += [t0 + x for x in w]
            t0 += len(t)
        block_rows = {g: [b.block_table(rid, g) for rid, _, _ in entries] for g in range(2)}
        ref = pack_batch(BatchBuilder(torch.device("cpu")), segs, rows, block_rows, min_blocks=min_blocks)
        T, R = ref.T, ref.R
        flat = torch.cat([ref.token_ids, ref.positions, ref.req_of_token, ref.cu_q, ref.q_start, ref.kv_len,
                          ref.state_slot, ref.logit_rows] + [ref.block_tables[g].reshape(-1) for g in range(2)])
        assert total == flat.numel() == meta[2] and meta[0] == T and meta[1] == len(rows)
        assert [int(meta[4]), int(meta[5])] == [ref.block_tables[0].shape[1], ref.block_tables[1].shape[1]]
        assert out[:total].tolist() == flat.tolist()
        assert int(out[total]) == -7                       # nothing written past the end
        for rid, _, _ in entries:
            assert a.release_passed(rid) == b.release_passed(rid)
        a.check_invariants(); b.check_invariants()
        assert a.free_pages() == b.free_pages()
        for rid in list(live):
            if rng.random() < 0.15:
                a.free_request(rid); b.free_request(rid); live.remove(rid)


def test_packed_step_refusals_change_nothing():
    from blackwellllm_b200.cache import manager as M
    cm = CacheManager([FULL], page_size=8, num_pages=4, max_requests=2)
    cm.add_request("a")
    cm.append("a", 5)
    state = (cm.free_pages(), cm.slots.num_free, cm.length("a"))
    assert _pack(cm, [("a", [1, 2000], [0])])[0] == M.ERR_BAD_TOKEN
    assert _pack(cm, [("a", [1, -1], [0])])[0] == M.ERR_BAD_TOKEN
    assert _pack(cm, [("a", [1, 2], [2])])[0] == M.ERR_BAD_WANT
    assert _pack(cm, [("a", [1, 2], [0]), ("a", [3], [0])])[0] == M.ERR_TWICE
    assert _pack(cm, [("a", [1] * 9, [0])], max_tokens=8)[0] == M.ERR_TOO_MANY_TOKENS
    assert _pack(cm, [("a", [1], [0]), ("n1", [1], [0]), ("n2", [1], [0])])[0] == M.ERR_NO_SLOT
    assert _pack(cm, [("a", [1] * 20, [0]), ("n1", [1] * 9, [0])])[0] == M.ERR_OUT_OF_PAGES
    assert _pack(cm, [("a", [1], [0])], cap=5)[0] == M.ERR_TOO_SMALL
    assert (cm.free_pages(), cm.slots.num_free, cm.length("a")) == state and not cm.has("n1")
    cm.check_invariants()
