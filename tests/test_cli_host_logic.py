"""The command line's host logic without a GPU: option names and defaults of the reference's
program (src/apps/main.cpp:42-60, 90-160), the generation loop's stop reasons (main.cpp:410-439),
head-and-tail truncation (main.cpp:305-315), line escaping (main.cpp:289-303) and the ``GEN``
request / ``<<<RESULT>>>`` reply framing (main.cpp:262-276).  The engine is a stand-in that follows
a fixed rule (next token = (last token + position) % 50) and records its calls; generation through
the real engine is covered by the GPU tests."""
import io
import types

import pytest

from blackwellllm_b200 import cli


class StandIn:
    """Position-addressed calls of the entry point, with a rule instead of a model."""

    def __init__(self):
        self.calls = []

    def reset_state(self, seq_id=0):
        self.calls.append(("reset", seq_id))

    def prefill(self, ids, start_pos, temperature, top_p, seq_id):
        self.calls.append(("prefill", list(ids), start_pos, temperature, top_p, seq_id))
        return (ids[-1] + start_pos + len(ids) - 1) % 50

    def forward(self, tok, pos, temperature, top_p, seq_id):
        self.calls.append(("forward", tok, pos, temperature, top_p, seq_id))
        return (tok + pos) % 50


def rule(ids, n):
    out, last, pos = [], ids[-1], len(ids) - 1
    for _ in range(n):
        last = (last + pos) % 50
        pos += 1
        out.append(last)
    return out


def test_options_and_defaults_of_the_reference_program():
    ap = cli.build_parser()
    a = ap.parse_args([])
    assert (a.ctx, a.kv_mode, a.prefill, a.chat, a.serve, a.gpu_layers) == (16384, "paged", "fast", False, False, None)
    assert (a.temperature, a.top_p, a.max_new_tokens) == (0.6, 0.9, 1024)     # scripts/cli_chat.py:77-85
    a = ap.parse_args(["-m", "DIR", "--system", "s", "--ctx", "4096", "--gpu-layers", "3", "--chat", "--serve",
                       "--kv-mode", "continuous", "--prefill", "loop"])
    assert (a.model, a.system, a.ctx, a.gpu_layers, a.chat, a.serve, a.kv_mode, a.prefill) == \
        ("DIR", "s", 4096, 3, True, True, "continuous", "loop")
    assert ap.parse_args(["DIR"]).model_pos == "DIR"                             # the folder without -m
    with pytest.raises(SystemExit):
        ap.parse_args(["--kv-mode", "ring"])
    with pytest.raises(SystemExit, match="paged"):
        cli.make_engine(ap.parse_args(["-m", "DIR", "--kv-mode", "continuous"]))
    with pytest.raises(SystemExit, match="--model"):
        cli.make_engine(ap.parse_args([]))
    with pytest.raises(SystemExit, match="--config"):
        cli.make_engine(ap.parse_args(["--random-weights"]))


def test_small_helpers():
    assert cli.parse_ids("1, 2,3  4") == [1, 2, 3, 4]
    with pytest.raises(ValueError):
        cli.parse_ids("1 x")
    assert cli.escape_line("a\\b\nc\rd\te") == "a\\\\b\\nc\\rd\\te"
    ids = list(range(10))
    assert cli.middle_truncate(ids, 0) == (ids, False) and cli.middle_truncate(ids, 10) == (ids, False)
    assert cli.middle_truncate(ids, 5) == ([0, 1, 7, 8, 9], True)               # head = budget // 2, the rest from the tail
    assert cli.middle_truncate(ids, 1) == ([9], True)


def test_generation_loop_stop_reasons_and_calls():
    e = StandIn()
    ids = [3, 4, 5]
    out, stop, _, _ = cli.generate_once(e, ids, 6, 0.7, 0.8, False, 100, set())
    assert (out, stop) == (rule(ids, 6), "limit")
    assert e.calls[0] == ("reset", 0) and e.calls[1] == ("prefill", ids, 0, 0.7, 0.8, 0)
    # every emitted token is fed back at the next position; the last sampled one is not emitted
    assert [c[1:3] for c in e.calls[2:]] == [(t, 3 + i) for i, t in enumerate(out)]
    # an end-of-sequence token stops before it is emitted
    want = rule(ids, 6)
    out, stop, _, _ = cli.generate_once(StandIn(), ids, 6, 0.0, 1.0, False, 100, {want[2]})
    assert (out, stop) == (want[:2], "eos")
    # the context ends generation: positions 0..ctx-1 exist
    out, stop, _, _ = cli.generate_once(StandIn(), ids, 6, 0.0, 1.0, False, 5, set())
    assert (out, stop) == (want[:2], "ctx")
    # --prefill loop: one greedy forward per prompt token, the same continuation
    e = StandIn()
    seen = []
    out, stop, _, _ = cli.generate_once(e, ids, 4, 0.5, 0.9, True, 100, set(), seen.append)
    assert out == rule(ids, 4) == seen
    assert e.calls[1:4] == [("forward", 3, 0, 0.0, 1.0, 0), ("forward", 4, 1, 0.0, 1.0, 0), ("forward", 5, 2, 0.0, 1.0, 0)]


def test_gen_protocol_framing(monkeypatch, capsys):
    def request(payload, *fields):
        body = payload.encode()
        return (" ".join(["GEN", str(len(body))] + [str(f) for f in fields]) + "\n").encode() + body

    stream = io.BytesIO(
        b"\n"                                                    # an empty line is skipped
        + request("3 4 5", 4, 0, 0.0, 1.0, 0)                   # ids, since there is no tokenizer
        + b"\n" + request(" ".join(str(i) for i in range(40)), 2, 6, 0.0, 1.0, 0)   # truncated to 6 ids
        + b"\nHELLO 1\n"                                         # not a request: an error line, the loop goes on
        + request("1 x", 2)                                      # a payload that is no list of ids
        + request("7", 3)                                        # defaults: greedy, no input cap
        + b"QUIT\n" + request("9", 1))                           # nothing after QUIT is read
    monkeypatch.setattr(cli.sys, "stdin", types.SimpleNamespace(buffer=stream))
    args = cli.build_parser().parse_args(["--ctx", "64", "--serve"])
    e = StandIn()
    assert cli.serve(e, None, args, set()) == 0
    lines = capsys.readouterr().out.splitlines()
    blocks = [ln for ln in lines if ln.startswith("<<<")]
    assert lines[0].startswith("<<<RESULT prompt_tokens=3 gen_tokens=4 ") and " stop=limit trunc=0 prefill=fast>>>" in lines[0]
    assert lines[1] == "TEXT " + " ".join(str(t) for t in rule([3, 4, 5], 4)) and lines[2] == "<<<END>>>"
    kept = [0, 1, 2, 37, 38, 39]
    assert lines[3].startswith("<<<RESULT prompt_tokens=6 gen_tokens=2 ") and " trunc=1 " in lines[3]
    assert lines[4] == "TEXT " + " ".join(str(t) for t in rule(kept, 2))
    assert lines[6].startswith("<<<ERROR expected: GEN ")
    assert lines[7].startswith("<<<ERROR ") and "invalid literal" in lines[7]
    assert lines[8].startswith("<<<RESULT prompt_tokens=1 gen_tokens=3 ") and lines[10] == "<<<END>>>"
    assert len(lines) == 11 and len(blocks) == 8
    prefills = [c for c in e.calls if c[0] == "prefill"]
    assert [c[1] for c in prefills] == [[3, 4, 5], kept, [7]]
    assert all(c[3:5] == (0.0, 1.0) for c in prefills)           # temperature 0: greedy
    assert stream.read() == request("9", 1)                      # left unread


def test_gen_protocol_caps_the_prompt_to_the_context(monkeypatch, capsys):
    body = " ".join(str(i % 50) for i in range(100)).encode()
    stream = io.BytesIO(b"GEN %d 8 0 0 1 0\n" % len(body) + body)
    monkeypatch.setattr(cli.sys, "stdin", types.SimpleNamespace(buffer=stream))
    args = cli.build_parser().parse_args(["--ctx", "48", "--serve", "--prefill", "loop"])
    e = StandIn()
    assert cli.serve(e, None, args, set()) == 0
    first = capsys.readouterr().out.splitlines()[0]
    # ctx - (max_new + 8) = 32 prompt tokens survive (main.cpp: the hard cap of a request)
    assert "prompt_tokens=32 gen_tokens=8 " in first and "trunc=1 prefill=loop>>>" in first
    assert sum(1 for c in e.calls if c[0] == "forward") == 32 + 8 and not any(c[0] == "prefill" for c in e.calls)


def test_entry_point_refuses_before_anything_is_loaded(tmp_path):
    """The request's checks of the reference's plan (src/core/runtime_config.cpp:53-65) come before any
    weight is read or any device is asked for, so they show without a GPU."""
    import json

    import tiny
    from blackwellllm_b200 import BlackwellEngine, EngineError, InferenceConfig
    raw = dict(tiny.CONFIGS["llama"][0], max_position_embeddings=64)
    with pytest.raises(EngineError, match="max_context_length must be > 0"):
        BlackwellEngine(None, InferenceConfig(max_context_length=0), config=raw)
    with pytest.raises(EngineError, match="max_batch_size >= 1"):
        BlackwellEngine(None, InferenceConfig(max_batch_size=0), config=raw)
    with pytest.raises(EngineError, match="either a model folder or a config"):
        BlackwellEngine(None, InferenceConfig())
    with pytest.raises(EngineError, match="either a model folder or a config"):
        BlackwellEngine(str(tmp_path), InferenceConfig(), config=raw)
    with pytest.raises(EngineError, match="exceeds the model's max_position_embeddings 64"):
        BlackwellEngine(None, InferenceConfig(max_context_length=65), config=raw)
    (tmp_path / "config.json").write_text(json.dumps(raw))               # a folder: the same check from its config.json
    with pytest.raises(EngineError, match="exceeds the model's max_position_embeddings 64"):
        BlackwellEngine(str(tmp_path), InferenceConfig(max_context_length=128))
