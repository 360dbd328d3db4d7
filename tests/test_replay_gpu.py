"""bin/trace_run against the plain implementation: the same requests whole, with the
last 32 tokens one by one, in portions of changing size, and mixed with other
requests in a pool so small that pages are used again; in 32-bit and in bfloat16;
on tiny configurations that differ in every size and option."""
import pytest

import replay
import tiny
from plain_model import load_plain_weights, plain_logits

pytestmark = pytest.mark.gpu

LENGTHS = [40, 97, 50, 70, 130, 65]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    return {(n, d): tiny.make_folder(n, d, root) for n in tiny.CONFIGS for d in ("float32", "bfloat16")}


_plain_cache = {}


def requests_and_plain(name, dtype, folder):
    key = (name, dtype)
    if key not in _plain_cache:
        raw = tiny.CONFIGS[name][0]
        reqs = {f"r{i}": tiny.prompt(n, raw["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS)}
        W = load_plain_weights(folder)
        plain = {rid: plain_logits(raw, W, ids) for rid, ids in reqs.items()}
        _plain_cache[key] = (reqs, plain)
    return _plain_cache[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay(folders, name, dtype, family):
    raw, _, page = tiny.CONFIGS[name]
    folder = folders[(name, dtype)]
    reqs, plain = requests_and_plain(name, dtype, folder)
    if family == "whole":
        steps, max_tokens = replay.trace_whole(reqs)
    elif family == "tail":
        steps, max_tokens = replay.trace_tail(reqs)
    elif family == "portions":
        steps, max_tokens = replay.trace_portions(reqs)
    else:
        max_tokens = 384  # 6 requests of 64..192 rounded tokens: at most four live, never all
        steps = replay.trace_mixed(reqs, max_tokens, seed=3)
        assert max(len(s["entries"]) for s in steps) >= 3
    rows = replay.run_trace(folder, dtype, steps, max_tokens, raw["vocab_size"], page_size=page)
    replay.compare(rows, plain, tiny.TOL[dtype], label=f"{name} {dtype} {family}", min_cosine=tiny.MIN_COSINE[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_changes_only_rounding(folders, dtype):
    """The same positions under two ways of cutting agree far more closely than
    either agrees with the plain implementation's bound."""
    name = "qwen"
    raw, _, page = tiny.CONFIGS[name]
    folder = folders[(name, dtype)]
    reqs, _ = requests_and_plain(name, dtype, folder)
    s1, m1 = replay.trace_whole(reqs)
    s2, m2 = replay.trace_portions(reqs)
    a = replay.run_trace(folder, dtype, s1, m1, raw["vocab_size"], page_size=page)
    b = replay.run_trace(folder, dtype, s2, m2, raw["vocab_size"], page_size=page)
    worst = max(float((a[k] - b[k]).abs().max()) / float(a[k].abs().max()) for k in a)
    assert worst <= tiny.TOL[dtype], worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_pages_of_24_tokens(folders, dtype):
    """A page size that does not divide 64 (nor the kernels' key tiles): mixed steps in a pool where pages
    are used again."""
    name = "llama3"
    raw = tiny.CONFIGS[name][0]
    folder = folders[(name, dtype)]
    reqs, plain = requests_and_plain(name, dtype, folder)
    steps = replay.trace_mixed(reqs, 384, seed=8)
    rows = replay.run_trace(folder, dtype, steps, 384, raw["vocab_size"], page_size=24)
    replay.compare(rows, plain, tiny.TOL[dtype], label=f"{name} {dtype} mixed, pages of 24")
