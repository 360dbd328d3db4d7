"""Command line in the manner of the reference's ``blackwell_llm`` (src/apps/main.cpp:42-60,
90-160) and of scripts/cli_chat.py: the same option names with the same meanings
where it has them.

    python -m blackwellllm_b200.cli --model DIR [--ctx N] [--chat | --serve] [--prefill fast|loop]

* ``-m/--model DIR``  checkpoint folder (also the first positional argument)
* ``--system TEXT``   system prompt of the conversation (needs a tokenizer.json)
* ``--ctx N``         max context length in tokens (default 16384)
* ``--gpu-layers N``  accepted; every layer is resident on this GPU, so it changes nothing
* ``--chat``          interactive loop (the default); ``exit`` / ``quit`` leave it
* ``--serve``         the ``GEN`` line protocol (main.cpp:259-284), one request at a time
* ``--kv-mode``       ``paged`` (the only cache here; ``continuous`` is refused)
* ``--prefill``       ``fast``: the prompt in portions; ``loop``: one ``forward`` per token

Added: ``--config JSON --random-weights`` (a model from a configuration and
``--seed``), ``--dtype``, ``--page-size``, ``--num-pages``, ``--max-batch-tokens``,
``--temperature`` (0.6), ``--top-p`` (0.9), ``--max-new-tokens`` (1024),
``--prompt-ids 1,2,3`` (one shot, no loop), ``--stats``.

Without a ``tokenizer.json`` in the model folder (or without the ``tokenizers``
package) prompts and replies are lists of token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="blackwellllm_b200", description="Llama/Qwen2 inference on one B200")
    ap.add_argument("model_pos", nargs="?", default=None, help=argparse.SUPPRESS)
    ap.add_argument("-m", "--model", default=None, help="checkpoint directory (weights + config [+ tokenizer])")
    ap.add_argument("--system", default="You are a helpful, smart, and concise AI assistant.",
                    help="system prompt for the conversation prelude")
    ap.add_argument("--ctx", type=int, default=16384, help="max context length in tokens (default 16384)")
    ap.add_argument("--gpu-layers", type=int, default=None, help="accepted for compatibility; all layers are resident")
    ap.add_argument("--chat", action="store_true", help="interactive chat (the default mode)")
    ap.add_argument("--serve", action="store_true", help="GEN line protocol on stdin/stdout")
    ap.add_argument("--kv-mode", choices=["continuous", "paged"], default="paged")
    ap.add_argument("--prefill", choices=["fast", "loop"], default="fast")
    ap.add_argument("--config", default=None, help="config.json for --random-weights")
    ap.add_argument("--random-weights", action="store_true", help="random weights from --config and --seed")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--max-new-tokens", type=int, default=1024)
    ap.add_argument("--repetition-penalty", type=float, default=1.0,
                    help="> 1 makes tokens already generated less likely (with --prompt-ids; default off)")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids: generate once and exit")
    ap.add_argument("--stats", action="store_true", help="print timing and scheduler counters")
    ap.add_argument("--ignore-unexpected-tensors", action="store_true",
                    help="pass over tensors of the checkpoint that the model does not use (default: an error)")
    return ap


def load_tokenizer(model_dir: Optional[str]):
    if not model_dir:
        return None
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def escape_line(text: str) -> str:
    return text.replace("\\", "\\\\").replace("\n", "\\n").replace("\r", "\\r").replace("\t", "\\t")


def middle_truncate(ids: List[int], budget: int):
    """Keep head and tail, drop the middle (main.cpp:305-315)."""
    if budget == 0 or len(ids) <= budget:
        return ids, False
    head = budget // 2
    return ids[:head] + ids[len(ids) - (budget - head):], True


def make_engine(args):
    from .engine.llm import BlackwellEngine, InferenceConfig
    if args.kv_mode == "continuous":
        raise SystemExit("--kv-mode continuous: this engine has only the paged cache")
    req = InferenceConfig(max_context_length=args.ctx, max_batch_size=1,
                          temperature=args.temperature, top_p=args.top_p)
    kw = dict(dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
              max_batch_tokens=args.max_batch_tokens, seed=args.seed)
    if args.random_weights:
        if not args.config:
            raise SystemExit("--random-weights needs --config JSON")
        with open(args.config, "r", encoding="utf-8") as f:
            raw = json.load(f)
        return BlackwellEngine(None, req, config=raw, random_seed=args.seed, **kw)
    model = args.model or args.model_pos
    if not model:
        raise SystemExit("give --model DIR (or --config JSON --random-weights)")
    return BlackwellEngine(model, req, ignore_unexpected=args.ignore_unexpected_tensors, **kw)


def generate_once(engine, ids: List[int], max_new: int, temperature: float, top_p: float,
                  prefill_loop: bool, ctx: int, eos: set, on_token=None):
    """prefill, then one forward per token until eos / limit / ctx (main.cpp:410-439)."""
    engine.reset_state(0)
    t0 = time.perf_counter()
    if prefill_loop:
        nxt = -1
        for pos, tok in enumerate(ids):
            nxt = engine.forward(tok, pos, 0.0, 1.0, 0)
    else:
        nxt = engine.prefill(ids, 0, temperature, top_p, 0)
    t1 = time.perf_counter()
    pos, out, stop = len(ids), [], "limit"
    while len(out) < max_new:
        if nxt in eos:
            stop = "eos"
            break
        if pos >= ctx:
            stop = "ctx"
            break
        out.append(nxt)
        if on_token:
            on_token(nxt)
        nxt = engine.forward(nxt, pos, temperature, top_p, 0)
        pos += 1
    t2 = time.perf_counter()
    return out, stop, (t1 - t0) * 1e3, (t2 - t1) * 1e3


def serve(engine, tok, args, eos) -> int:
    stdin = sys.stdin.buffer
    while True:
        line = stdin.readline()
        if not line:
            return 0
        parts = line.decode("utf-8", "replace").split()
        if not parts:
            continue
        if parts[0] == "QUIT":
            return 0
        try:
            if parts[0] != "GEN" or len(parts) < 2:
                raise ValueError("expected: GEN <byte_len> <max_new> <max_input_tokens> <temp> <top_p> <chat>")
            nbytes = int(parts[1])
            max_new = int(parts[2]) if len(parts) > 2 else 64
            max_in = int(parts[3]) if len(parts) > 3 else 0
            temp = float(parts[4]) if len(parts) > 4 else 0.0
            top_p = float(parts[5]) if len(parts) > 5 else 1.0
            payload = stdin.read(nbytes).decode("utf-8", "replace")
            ids = tok.encode(payload).ids if tok else parse_ids(payload)
            hard_cap = max(1, args.ctx - (max_new + 8))
            budget = hard_cap if max_in == 0 or max_in > hard_cap else max_in
            ids, trunc = middle_truncate(ids, budget)
            out, stop, pre_ms, dec_ms = generate_once(engine, ids, max_new, temp, top_p,
                                                      args.prefill == "loop", args.ctx, eos)
            text = tok.decode(out) if tok else " ".join(str(t) for t in out)
            print(f"<<<RESULT prompt_tokens={len(ids)} gen_tokens={len(out)} prefill_ms={pre_ms:.1f} "
                  f"decode_ms={dec_ms:.1f} stop={stop} trunc={int(trunc)} prefill={args.prefill}>>>")
            print(f"TEXT {escape_line(text)}\n<<<END>>>", flush=True)
        except Exception as e:  # one bad request must not end the loop (main.cpp:272-274)
            print(f"<<<ERROR {escape_line(str(e))}>>>", flush=True)


def chat(engine, tok, args, eos) -> int:
    print("[System] Type 'exit' or 'quit' to end the session.")
    if tok is None:
        print("[System] No tokenizer: enter token ids separated by spaces or commas.")
    history: List[int] = []
    if tok is not None and args.system:
        history = tok.encode(args.system + "\n").ids
    while True:
        try:
            user = input("\n[User]: ")
        except EOFError:
            return 0
        if user.lower().strip() in ("exit", "quit"):
            print("\n[System] Closing chat session. Goodbye!")
            return 0
        if not user.strip():
            continue
        try:
            ids = tok.encode(user + "\n").ids if tok else parse_ids(user)
        except ValueError:
            print("[System] token ids must be integers")
            continue
        prompt = history + ids
        print("\n[Model]: ", end="", flush=True)

        def show(t):
            print(tok.decode([t]) if tok else f"{t} ", end="", flush=True)

        out, stop, pre_ms, dec_ms = generate_once(engine, prompt, args.max_new_tokens, args.temperature,
                                                  args.top_p, args.prefill == "loop", args.ctx, eos, show)
        print()
        history = prompt + out
        if args.stats:
            print(f"[stats] prompt={len(prompt)} new={len(out)} prefill_ms={pre_ms:.1f} "
                  f"decode_ms={dec_ms:.1f} stop={stop}")


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    engine = make_engine(args)
    tok = load_tokenizer(args.model or args.model_pos)
    eos = set(engine.engine.config.eos_token_ids)
    if args.gpu_layers is not None:
        print("[System] --gpu-layers: all layers are resident on this GPU", file=sys.stderr)
    if args.prompt_ids is not None:
        from .sampling.params import SamplingParams
        ids = parse_ids(args.prompt_ids)
        t0 = time.perf_counter()
        res = engine.generate(ids, SamplingParams(temperature=args.temperature, top_p=args.top_p,
                                                  max_new_tokens=args.max_new_tokens,
                                                  repetition_penalty=args.repetition_penalty))[0]
        dt = time.perf_counter() - t0
        print(" ".join(str(t) for t in res.token_ids))
        if args.stats:
            st = engine.scheduler.stats
            print(f"[stats] prompt={len(ids)} new={len(res.token_ids)} stop={res.finish_reason} "
                  f"seconds={dt:.3f} steps={st.steps} admitted={st.admitted} preemptions={st.preemptions} "
                  f"pages_free={engine.engine.cache.free_pages()}", file=sys.stderr)
        return 0
    if args.serve:
        return serve(engine, tok, args, eos)
    return chat(engine, tok, args, eos)


if __name__ == "__main__":
    sys.exit(main())
