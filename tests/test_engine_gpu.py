"""The engine through its Python entry point, against the plain implementation:
greedy generation, long decoding, the first tokens of a sequence, sampling with
temperature and nucleus against the CPU twin, the position-addressed calls, and
what happens when pages run out."""
import math

import pytest
import torch

import tiny
from plain_model import load_plain_weights, plain_greedy, plain_logits
from plain_sampling import plain_log_prob, plain_repetition_penalty, plain_sample

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {(n, d): tiny.make_folder(n, d, root) for n in tiny.CONFIGS for d in ("float32", "bfloat16")}


def make(folder, dtype, ctx=512, batch=4, **kw):
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig
    return BlackwellEngine(folder, InferenceConfig(max_context_length=ctx, max_batch_size=batch), dtype=dtype, **kw)


def check_greedy_path(raw, W, prompt, tokens, dtype):
    """float32: the plain greedy continuation, token for token.  bfloat16: every token
    is the plain implementation's best or within the rounding bound of it."""
    if dtype == "float32":
        assert tokens == plain_greedy(raw, W, prompt, len(tokens))
        return
    seq = list(prompt)
    for t in tokens:
        lg = plain_logits(raw, W, seq)[-1]
        assert float(lg.max() - lg[t]) <= tiny.TOL["bfloat16"] * float(lg.abs().max())
        seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["llama", "qwen"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from blackwellllm_b200 import SamplingParams
    raw, _, page = tiny.CONFIGS[name]
    folder = folders[(name, dtype)]
    W = load_plain_weights(folder)
    llm = make(folder, dtype, page_size=page)
    prompts = [tiny.prompt(n, raw["vocab_size"], 40 + n) for n in (5, 17, 33)]
    res = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=8))
    for p, r in zip(prompts, res):
        assert r.finish_reason == "limit" and len(r.token_ids) == 8 and r.prompt_token_ids == p
        check_greedy_path(raw, W, p, r.token_ids, dtype)
    assert llm.engine.cache.free_pages() == [g.num_pages for g in llm.engine.cache.groups]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """A one-token prompt, then 150 tokens decoded one by one (graph replay), checked
    against the plain implementation at every position."""
    from blackwellllm_b200 import StepEntry
    raw, _, page = tiny.CONFIGS["llama3"]
    folder = folders[("llama3", dtype)]
    W = load_plain_weights(folder)
    llm = make(folder, dtype, page_size=page, ctx=256, batch=1)
    ids = tiny.prompt(151, raw["vocab_size"], 9)
    ref = plain_logits(raw, W, ids)
    eng = llm.engine
    worst = 0.0
    for i, t in enumerate(ids):
        lg = eng.step([StepEntry("a", [t], [0])])[0].double().cpu()
        worst = max(worst, float((lg - ref[i]).abs().max()) / float(ref.abs().max()))
    assert worst <= tiny.TOL[dtype], worst
    assert eng.graph_kernel_count(1) > 0      # the decode steps ran from the captured graph


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["llama", "qwen"])
def test_one_wrong_page_in_one_layer_exceeds_the_logit_bound(folders, name, dtype):
    """Negative control of the whole-model bound: after a prompt, ONE page of ONE layer's cache gets the
    contents of another page (what a stale block-table entry would read there).  The next token's logits
    must then miss the plain implementation by more than the bound that every parity test allows, and
    stay within it when the page is put right again."""
    from blackwellllm_b200 import Engine, StepEntry
    raw, _, page = tiny.CONFIGS[name]
    folder = folders[(name, dtype)]
    W = load_plain_weights(folder)
    ids = tiny.prompt(3 * page + 2, raw["vocab_size"], 77)
    ref = plain_logits(raw, W, ids)
    scale = float(ref.abs().max())
    eng = Engine.from_folder(folder, dtype=dtype, page_size=page, max_tokens=256, cuda_graphs=False)
    eng.step([StepEntry("a", ids[:-1], [])])
    pool = eng.cache.groups[0].pool                   # [entries (layers), 2, pages, kv heads, page, head]
    table = eng.cache.block_table("a", 0)
    layer = pool.shape[0] - 1
    saved = pool[layer, :, table[1]].clone()
    pool[layer, :, table[1]] = pool[layer, :, table[0]]
    bad = eng.step([StepEntry("a", [ids[-1]], [0])])[0].double().cpu()
    assert float((bad - ref[-1]).abs().max()) / scale > tiny.TOL[dtype], "the bound cannot see a wrong page"
    eng.cache.truncate("a", len(ids) - 1)
    pool[layer, :, table[1]] = saved
    good = eng.step([StepEntry("a", [ids[-1]], [0])])[0].double().cpu()
    assert float((good - ref[-1]).abs().max()) / scale <= tiny.TOL[dtype]


def test_sampling_kernel_matches_the_cpu_twin():
    from blackwellllm_b200.kernels import ops
    from blackwellllm_b200.sampling.params import uniform
    g = torch.Generator().manual_seed(0)
    V = 1000
    logits = (torch.randn(64, V, generator=g) * 3).to(DEV)
    temps = [0.0, 0.3, 0.6, 1.0, 1.7] * 13
    tops = [1.0, 0.9, 0.5, 0.99, 0.2, 1.0, 0.7] * 10
    R = 64
    t = torch.tensor(temps[:R], device=DEV)
    p = torch.tensor(tops[:R], device=DEV)
    us = [uniform(5, i) for i in range(R)]
    u = torch.tensor(us, device=DEV)
    got = ops.sample(logits, t, p, u).tolist()
    checked = 0
    for r in range(R):
        want, margin = plain_sample(logits[r].cpu(), temps[r], tops[r], us[r])
        if margin > 1e-4:   # a draw that close to a CDF edge may fall either way in float32
            assert got[r] == want, (r, temps[r], tops[r])
            checked += 1
    assert checked >= 60
    # greedy: lowest index wins a tie
    tie = torch.zeros(2, 50, device=DEV)
    tie[0, 7] = tie[0, 30] = 2.0
    tie[1, 49] = 1.0
    assert ops.sample(tie, None, None, None).tolist() == [7, 49]


def test_sampling_distribution_and_nucleus():
    from blackwellllm_b200.kernels import ops
    probs = torch.tensor([0.5, 0.25, 0.15, 0.07, 0.03])
    logits = probs.log().repeat(4000, 1).to(DEV)
    u = torch.rand(4000, generator=torch.Generator().manual_seed(1)).to(DEV)
    ones = torch.ones(4000, device=DEV)
    full = ops.sample(logits, ones, ones, u)
    freq = torch.bincount(full.long().cpu(), minlength=5).double() / 4000
    assert float((freq - probs.double()).abs().max()) < 0.03
    nucleus = ops.sample(logits, ones, ones * 0.8, u)   # 0.5 + 0.25 + 0.15 reach 0.8: three tokens stay
    assert set(nucleus.tolist()) == {0, 1, 2}


def test_temperature_generation_is_seeded_and_independent_of_the_batch(folders):
    """Chunked prefill (chunk 12) mixed with decoding, temperature 1.0: the tokens
    follow the CPU twin on the plain logits, and a request's tokens do not depend on
    which other requests share its batches."""
    from blackwellllm_b200 import SamplingParams
    from blackwellllm_b200.sampling.params import uniform
    raw, _, page = tiny.CONFIGS["qwen"]
    folder = folders[("qwen", "float32")]
    W = load_plain_weights(folder)
    prompts = [tiny.prompt(n, raw["vocab_size"], 70 + n) for n in (1, 9, 40, 70)]
    sp = SamplingParams(temperature=1.0, top_p=1.0, max_new_tokens=6)
    llm = make(folder, "float32", page_size=page, chunk=12, max_batch_tokens=32, seed=2)
    res = llm.generate(prompts, sp)
    for rid, (p, r) in enumerate(zip(prompts, res)):
        seq = list(p)
        for i, t in enumerate(r.token_ids):
            want, margin = plain_sample(plain_logits(raw, W, seq)[-1], 1.0, 1.0, uniform(2 * 1_000_003 + rid, i))
            if margin > 1e-4:
                assert t == want
            seq.append(t)
    alone = make(folder, "float32", page_size=page, seed=2)
    solo = alone.generate([prompts[0]], sp)[0]          # request number 0 again, with no company
    assert solo.token_ids == res[0].token_ids


def test_repetition_penalty_and_log_prob_kernels_match_the_cpu_twins():
    from blackwellllm_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    R, V = 5, 1003
    base = torch.randn(R, V + 5, generator=g) * 4
    logits = base.to(DEV)[:, :V]                       # rows with a stride that is not their width
    hist = [[10, 20, 10, 10, 999, 20], [], [7] * 300 + [8, 9], [-1, V, V + 3, 5], list(range(0, V, 3))]
    pens = [1.15, 1.5, 2.0, 1.3, 1.0]                  # the last row: penalty off
    flat = [t for h in hist for t in h]
    begin = [0]
    for h in hist:
        begin.append(begin[-1] + len(h))
    out = ops.repetition_penalty(logits, torch.tensor(flat, dtype=torch.int32, device=DEV),
                                 torch.tensor(begin, dtype=torch.int32, device=DEV),
                                 torch.tensor(pens, dtype=torch.float32, device=DEV)).cpu()
    for r in range(R):
        want = plain_repetition_penalty(base[r, :V], hist[r], pens[r])
        assert torch.equal(out[r], want), r
    assert torch.equal(logits.cpu(), out)              # in place
    targets = [0, V - 1, 500, 7, 123]
    lp = ops.log_prob(logits, torch.tensor(targets, dtype=torch.int32, device=DEV)).cpu()
    for r in range(R):
        assert abs(float(lp[r]) - plain_log_prob(out[r], targets[r])) < 1e-4, r


def test_generation_with_a_repetition_penalty_follows_the_plain_rule(folders):
    """Greedy with a strong penalty over a window of 3: every token is the argmax of the plain
    logits after the plain penalty on the last three generated tokens."""
    from blackwellllm_b200 import SamplingParams
    raw, _, page = tiny.CONFIGS["llama"]
    folder = folders[("llama", "float32")]
    W = load_plain_weights(folder)
    llm = make(folder, "float32", page_size=page)
    prompts = [tiny.prompt(n, raw["vocab_size"], 30 + n) for n in (5, 17)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=10, repetition_penalty=50.0, repetition_window=3,
                        ignore_eos=True)
    res = llm.generate(prompts, sp)
    for p, r in zip(prompts, res):
        seq, gen = list(p), []
        for t in r.token_ids:
            lg = plain_repetition_penalty(plain_logits(raw, W, seq)[-1].float(), gen[-3:], 50.0)
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-4:
                assert t == int(lg.argmax())
            seq.append(t); gen.append(t)


def test_forward_eval_and_last_token_probability(folders):
    from blackwellllm_b200 import EngineError
    raw, _, page = tiny.CONFIGS["qwen"]
    folder = folders[("qwen", "float32")]
    W = load_plain_weights(folder)
    llm = make(folder, "float32", page_size=page)
    ids = tiny.prompt(12, raw["vocab_size"], 4)
    ref = plain_logits(raw, W, ids)
    total = 0.0
    for i in range(len(ids) - 1):                       # the perplexity loop of the reference's evaluation
        lp = llm.forward_eval(ids[i], i, ids[i + 1])
        assert abs(lp - plain_log_prob(ref[i], ids[i + 1])) < 1e-4
        total += lp
    assert total < 0
    prob = llm.last_token_probability(ids[5])
    assert abs(prob - math.exp(plain_log_prob(ref[len(ids) - 2], ids[5]))) < 1e-5
    assert llm.last_token_probability(raw["vocab_size"]) == 0.0 and llm.last_token_probability(3, seq_id=9) == 0.0
    with pytest.raises(EngineError, match="vocabulary"):
        llm.forward_eval(ids[0], 0, raw["vocab_size"])
    nxt = llm.prefill(ids, 0, 0.0, 1.0)                  # rewinds to 0 and leaves the last position's logits
    assert abs(llm.last_token_probability(nxt) - math.exp(plain_log_prob(ref[-1], nxt))) < 1e-5


def test_position_addressed_calls(folders):
    from blackwellllm_b200 import DecodeRequest, EngineError
    raw, _, page = tiny.CONFIGS["llama"]
    folder = folders[("llama", "float32")]
    W = load_plain_weights(folder)
    llm = make(folder, "float32", page_size=page)
    p = tiny.prompt(20, raw["vocab_size"], 3)
    want = plain_greedy(raw, W, p, 3)
    nxt = llm.prefill(p, 0, 0.0, 1.0, seq_id=0)
    got = [nxt]
    for i in range(2):
        nxt = llm.forward(nxt, len(p) + i, 0.0, 1.0, seq_id=0)
        got.append(nxt)
    assert got == want
    # the per-token loop gives the same continuation as the chunked prefill
    for i, t in enumerate(p):
        last = llm.forward(t, i, 0.0, 1.0, seq_id=1)
    assert last == want[0]
    # re-decoding an earlier position rewinds; a gap is an error, not a fault
    assert llm.forward(p[10], 10, 0.0, 1.0, seq_id=1) == plain_greedy(raw, W, p[:11], 1)[0]
    with pytest.raises(EngineError, match="gap"):
        llm.forward(1, 50, 0.0, 1.0, seq_id=1)
    with pytest.raises(EngineError, match="twice"):
        llm.forward_batch([DecodeRequest(0, 1, 22), DecodeRequest(0, 2, 22)])
    # batched decode of distinct sequences equals the sequential calls
    llm.rewind(0, len(p))
    llm.prefill(p[:11], 0, 0.0, 1.0, seq_id=2)
    both = llm.forward_batch([DecodeRequest(0, want[0], len(p)), DecodeRequest(2, 7, 11)])
    assert both[0] == want[1] and both[1] == plain_greedy(raw, W, p[:11] + [7], 1)[0]
    llm.release_sequence(0); llm.release_sequence(1); llm.release_sequence(2)
    assert llm.engine.cache.free_pages() == [g.num_pages for g in llm.engine.cache.groups]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forward_batch_async_feeds_the_sampled_tokens_on_the_device(folders, dtype):
    """A decode loop that queues step n + 1 before it reads step n's tokens (FROM_LAST: the token ids go
    from the sampler into the next step on the device) gives the tokens of the loop that waits every step."""
    from blackwellllm_b200 import FROM_LAST, DecodeRequest, EngineError
    raw, _, page = tiny.CONFIGS["qwen"]
    folder = folders[("qwen", dtype)]
    llm = make(folder, dtype, page_size=page)
    llm.engine.options.graph_after = 1       # the batch size is recorded at its first decode step
    prompts = {0: tiny.prompt(20, raw["vocab_size"], 3), 2: tiny.prompt(11, raw["vocab_size"], 4), 5: tiny.prompt(33, raw["vocab_size"], 6)}

    def decode(pipelined, steps=7):
        first = {s: llm.prefill(p, 0, 0.0, 1.0, seq_id=s) for s, p in prompts.items()}
        seqs = list(prompts)
        out = {s: [first[s]] for s in seqs}
        pos = {s: len(prompts[s]) for s in seqs}
        if not pipelined:
            for _ in range(steps):
                toks = llm.forward_batch([DecodeRequest(s, out[s][-1], pos[s]) for s in seqs])
                for s, t in zip(seqs, toks):
                    out[s].append(t); pos[s] += 1
            return out
        pending = llm.forward_batch_async([DecodeRequest(s, first[s], pos[s]) for s in seqs])
        for _ in range(steps - 1):
            for s in seqs:
                pos[s] += 1
            nxt = llm.forward_batch_async([DecodeRequest(s, FROM_LAST, pos[s]) for s in seqs])
            for s, t in zip(seqs, pending.result()):
                out[s].append(t)
            pending = nxt
        for s, t in zip(seqs, pending.result()):
            out[s].append(t)
        return out

    waited = decode(False)
    assert llm.engine.native_steps >= 5          # once the graph of this batch size exists, the C entry point runs the steps
    assert decode(True) == waited
    before = llm.engine.native_steps
    llm.engine.options.native_decode = False     # the same loops through the Python path
    assert decode(False) == waited and decode(True) == waited and llm.engine.native_steps == before
    llm.engine.options.native_decode = True
    if dtype == "float32":
        W = load_plain_weights(folder)
        for s, p in prompts.items():
            assert waited[s] == plain_greedy(raw, W, p, 8)
    with pytest.raises(EngineError, match="FROM_LAST"):
        llm.forward_batch_async([DecodeRequest(2, FROM_LAST, 18), DecodeRequest(0, FROM_LAST, 27), DecodeRequest(5, FROM_LAST, 40)])
    with pytest.raises(EngineError, match="FROM_LAST"):
        llm.forward_batch_async([DecodeRequest(0, FROM_LAST, 27), DecodeRequest(2, 3, 18), DecodeRequest(5, FROM_LAST, 40)])


def test_sampled_tokens_of_the_position_addressed_calls_do_not_depend_on_what_ran_before(folders):
    """Temperature 1: the same prompt from position 0 on the same sequence id gives the same tokens again
    (the draw is a function of seed, sequence and position, not of how many draws came before)."""
    raw, _, page = tiny.CONFIGS["qwen"]
    llm = make(folders[("qwen", "float32")], "float32", page_size=page, seed=5)
    p = tiny.prompt(15, raw["vocab_size"], 8)

    def run():
        out = [llm.prefill(p, 0, 1.0, 1.0, seq_id=0)]
        for i in range(5):
            out.append(llm.forward(out[-1], len(p) + i, 1.0, 1.0, seq_id=0))
        return out
    first = run()
    llm.forward(3, 4, 1.0, 1.0, seq_id=0)        # something else in between, on the same sequence
    assert run() == first
    assert len(set(first)) > 1


def test_pages_run_out_preemption_reproduces_the_tokens(folders):
    from blackwellllm_b200 import SamplingParams
    raw, _, page = tiny.CONFIGS["llama"]
    folder = folders[("llama", "float32")]
    W = load_plain_weights(folder)
    prompts = [tiny.prompt(30, raw["vocab_size"], 200 + i) for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=40)
    # 3 requests x 69 cached tokens need 15 pages of 16; the pool has 9
    llm = make(folder, "float32", page_size=16, num_pages=9, ctx=512, batch=3)
    res = llm.generate(prompts, sp)
    assert llm.scheduler.stats.preemptions >= 1
    for p, r in zip(prompts, res):
        assert r.token_ids == plain_greedy(raw, W, p, 40)
    assert llm.engine.cache.free_pages() == [9]
    from blackwellllm_b200.engine.scheduler import RequestRefused
    with pytest.raises(RequestRefused):
        llm.add_request(tiny.prompt(120, raw["vocab_size"], 1), SamplingParams(max_new_tokens=100))


def test_no_cpu_path_and_bad_tokens(folders):
    from blackwellllm_b200 import Engine, EngineError, StepEntry
    from blackwellllm_b200.kernels import ops
    folder = folders[("llama", "float32")]
    with pytest.raises(EngineError, match="CUDA"):
        Engine.from_folder(folder, dtype="float32", device="cpu")
    with pytest.raises(ops.KernelError, match="CUDA tensor"):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.float32)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=64)
    with pytest.raises(EngineError, match="outside"):
        eng.step([StepEntry("a", [256], [0])])
    with pytest.raises(EngineError, match="wanted place"):
        eng.step([StepEntry("a", [1, 2], [2])])
    from blackwellllm_b200.cache.pages import OutOfPages
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", [1] * 65, [])])
    assert not eng.has_request("a") and eng.cache.free_pages() == [4]   # nothing was changed


def test_command_line_one_shot_and_gen_protocol(folders, capsys, monkeypatch):
    """The command line on a model folder: `--prompt-ids` prints the greedy continuation, and the
    GEN line protocol of `--serve` (src/main.cpp's `GEN <bytes> <max_new> <max_in> <temp> <top_p>`
    followed by the payload) answers with RESULT / TEXT / END; a bad request does not end the loop."""
    import io
    from blackwellllm_b200 import cli
    folder = folders[("llama", "float32")]
    raw, _, _ = tiny.CONFIGS["llama"]
    W = load_plain_weights(folder)
    prompt = [5, 17, 3, 200, 41, 7, 7, 9]
    want = plain_greedy(raw, W, prompt, 6)
    rc = cli.main(["-m", folder, "--dtype", "float32", "--ctx", "128", "--temperature", "0", "--max-new-tokens", "6",
                   "--prompt-ids", ",".join(map(str, prompt)), "--stats"])
    cap = capsys.readouterr()
    assert rc == 0 and [int(t) for t in cap.out.strip().splitlines()[0].split()] == want
    assert "[stats] prompt=8 new=6" in cap.err

    payload = " ".join(map(str, prompt)).encode()
    script = b"GEN %d 6 0 0.0 1.0 0\n" % len(payload) + payload + b"\nNONSENSE\n" + \
             b"GEN %d 4 0 0.0 1.0 0\n" % len(payload) + payload + b"\nQUIT\n"

    class Stdin:
        buffer = io.BytesIO(script)
    monkeypatch.setattr("sys.stdin", Stdin)
    rc = cli.main(["-m", folder, "--dtype", "float32", "--ctx", "128", "--serve"])
    lines = capsys.readouterr().out.strip().splitlines()
    assert rc == 0
    results = [ln for ln in lines if ln.startswith("<<<RESULT")]
    texts = [ln for ln in lines if ln.startswith("TEXT ")]
    assert len(results) == 2 and "prompt_tokens=8 gen_tokens=6" in results[0] and "gen_tokens=4" in results[1]
    assert [int(t) for t in texts[0][5:].split()] == want and [int(t) for t in texts[1][5:].split()] == want[:4]
    assert any(ln.startswith("<<<ERROR") for ln in lines) and lines.count("<<<END>>>") == 2
