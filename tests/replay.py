"""Drives bin/trace_run as a user would and collects logits by (request, position).
Also builds the families of traces the tests replay."""
import json
import os
import random
import subprocess
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def run_trace(model_dir, dtype, steps, max_tokens, vocab, page_size=None, timeout=600):
    """steps: list of {"step", "entries", "end"}.  Returns {(id, position): row}."""
    out_dir = tempfile.mkdtemp(prefix="trace_out_")
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    pos = {}
    rows = {}
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {st['step']}", f"trace_run said {line!r} (exit {proc.poll()})"
            wanted = []
            for e in st["entries"]:
                p0 = pos.get(e["id"], 0)
                wanted += [(e["id"], p0 + w) for w in e.get("want", [])]
                pos[e["id"]] = p0 + len(e["tokens"])
            for rid in st.get("end", []):
                pos.pop(rid, None)
            path = os.path.join(out_dir, f"{st['step']}.f32")
            if wanted:
                arr = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
                for k, row in zip(wanted, arr):
                    assert k not in rows, f"{k} wanted twice"
                    rows[k] = torch.from_numpy(row.copy())
            else:
                assert not os.path.exists(path)
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return rows


def rounded(n, to=64):
    return -(-n // to) * to


def trace_whole(requests):
    """Each request alone and whole, every position wanted."""
    steps = []
    for i, (rid, ids) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [rid]})
    return steps, max(rounded(len(v)) for v in requests.values())


def trace_tail(requests, tail=32):
    """Most of it in one step and the last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = len(ids) - tail
        assert head >= 1
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head],
                                                        "want": list(range(head))}], "end": []})
        for j in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[j]], "want": [0]}],
                          "end": [rid] if j == len(ids) - 1 else []})
    return steps, max(rounded(len(v)) for v in requests.values())


def trace_portions(requests, sizes=(7, 2, 13, 3, 5, 2, 16, 17, 4, 31, 2)):
    """Portions of changing size, down to two tokens, one request at a time."""
    steps = []
    k = 0
    for rid, ids in requests.items():
        at = 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[at:at + n],
                                                            "want": list(range(n))}],
                          "end": [rid] if at + n == len(ids) else []})
            at += n
    return steps, max(rounded(len(v)) for v in requests.values())


def trace_mixed(requests, max_tokens, seed=0, max_live=4, decode_tail=9):
    """Up to ``max_live`` live requests; portions of some beside single tokens of
    others; some requests sit a step out.  A request is admitted only while the
    live ones (each rounded up to 64 tokens) fit in ``max_tokens``, so later
    requests get the pages of earlier ones."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}  # rid -> position
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting[0]
            held = sum(rounded(len(requests[r])) for r in live)
            if held + rounded(len(ids)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = 0
        assert live, "max_tokens too small for the next request"
        entries, end = [], []
        order = list(live)
        rng.shuffle(order)
        for rid in order:
            if len(order) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            ids = requests[rid]
            at = live[rid]
            if at < len(ids) - decode_tail:
                n = min(rng.choice([2, 3, 5, 8, 13, 21]), len(ids) - decode_tail - at)
            else:
                n = 1
            entries.append({"id": rid, "tokens": ids[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if at + n == len(ids):
                end.append(rid)
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            del live[rid]
    return steps


REPORT = []   # lines for the summary at the end of the run (conftest.py prints them)


def compare(rows, plain, tol_rel, label=None, min_cosine=None):
    """rows: {(id, pos): tensor}; plain: {id: [T, V] tensor}.  Returns the worst
    error relative to the request's largest logit and where it is.  With a ``label`` the
    lowest cosine between a returned row and the plain row, and the share of rows whose
    largest logit is at the same token, go into the run's summary."""
    worst = (0.0, None)
    low_cos, same_top = 1.0, 0
    for (rid, p), row in rows.items():
        ref = plain[rid]
        scale = float(ref.abs().max())
        got, want = row.double(), ref[p].double()
        err = float((got - want).abs().max()) / scale
        if err > worst[0] or err != err:
            worst = (err, (rid, p))
        low_cos = min(low_cos, float(torch.dot(got, want) / (got.norm() * want.norm())))
        same_top += int(torch.argmax(got) == torch.argmax(want))
    missing = [(rid, p) for rid, ref in plain.items() for p in range(ref.shape[0]) if (rid, p) not in rows]
    assert not missing, f"positions never returned: {missing[:5]}"
    if label is not None:
        REPORT.append(f"{label}: worst error {worst[0]:.2e} of the logit scale (bound {tol_rel:.1e}), lowest cosine "
                      f"{low_cos:.6f}, same top-1 token at {same_top} of {len(rows)} positions")
    assert worst[0] <= tol_rel, f"worst error {worst[0]:.3e} of the logit scale at {worst[1]} (bound {tol_rel})"
    if min_cosine is not None:
        assert low_cos >= min_cosine, f"cosine {low_cos} below {min_cosine}"
    return worst
