#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

Default run: the layer sizes of the Llama-3.1-8B shape with random bfloat16 weights,
decode at batch 8 and context 8,192 (K timed steps after W warm-up steps), plus
prefill of 2,048 tokens and decode at batch 1 and 64.  A "step" is one decode step.
``value`` is decoded tokens per second timed on the device; ``e2e`` is the same
through the Python entry point with host token lists in and out.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 14336, "num_hidden_layers": 32, "vocab_size": 128256,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072,
}
# the other two big shapes: for --shape, not for the default run
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "intermediate_size": 18944, "num_hidden_layers": 28, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 131072,
}
QWEN25_14B = dict(QWEN25_7B, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                  intermediate_size=13824, num_hidden_layers=48)
SHAPES = {"llama-3.1-8b": ("Llama-3.1-8B", LLAMA_8B, 3), "qwen2.5-7b": ("Qwen2.5-7B", QWEN25_7B, 4),
          "qwen2.5-14b": ("Qwen2.5-14B", QWEN25_14B, 5)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    weight_elems = layers * per_layer + V * H  # embedding rows read are negligible
    kv_per_token = layers * 2 * nkv * hd
    return per_layer, weight_elems, kv_per_token


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES),
                    help="layer sizes (default: the Llama-3.1-8B shape of the headline number)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64", help="other decode batch sizes to report")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (for profiling); the JSON line then lacks the other part")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "fxslava/BlackwellLLM has no Python package or build metadata (pip install finds no "
                          "setup.py/pyproject.toml); it is a Windows/MSVC CMake project built for sm_120 only"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported"}))
        return 2

    import torch
    from blackwellllm_b200 import BlackwellEngine, DecodeRequest, InferenceConfig, StepEntry
    from blackwellllm_b200.kernels import ops

    shape_name, shape_cfg, weight_seed = SHAPES[args.shape]
    full_layers = shape_cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(shape_cfg, num_hidden_layers=args.layers)
    pk = peaks()
    page = 16
    sizes = sorted({args.batch, *[int(x) for x in args.points.split(",") if x]})
    max_b = max(sizes)
    room = args.context + args.warmup + args.steps * 2 + 64
    num_pages = max_b * -(-room // page) + -(-args.prefill_tokens // page) + 8
    llm = BlackwellEngine(None, InferenceConfig(max_context_length=room + 64, max_batch_size=max_b + 1),
                          config=cfg, random_seed=weight_seed, random_std=0.02, dtype="bfloat16", page_size=page,
                          num_pages=num_pages, max_batch_tokens=max(args.prefill_tokens, max_b), seed=0,
                          cuda_graphs=not args.no_graphs)
    eng = llm.engine
    dev = eng.device
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1234)
    per_layer, weight_elems, kv_per_token = model_bytes_and_flops(cfg, args.layers)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------- prefill of T tokens (one step, logits at the last position)
    T = args.prefill_tokens
    prompt = torch.randint(0, V, (T,), generator=gen).tolist()
    pre_ms = []
    for it in range(3 if args.only != "decode" else 0):
        s, e = ev(), ev()
        torch.cuda.synchronize()
        s.record()
        eng.step([StepEntry("prefill", prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        pre_ms.append(s.elapsed_time(e))
        eng.end_request("prefill")
    prefill_ms = min(pre_ms[1:]) if pre_ms else None
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    prefill_flops = 2.0 * T * args.layers * per_layer + 2.0 * V * cfg["hidden_size"] \
        + args.layers * 4.0 * nh * hd * T * (T + 1) / 2
    prefill = {"value": None, "tokens": T, "ms": None, "frac": None} if prefill_ms is None else \
        {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
         "frac": prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---------------- decode at context C: caches of B requests filled with random keys and values
    def fill_cache(B):
        for rid in list(eng.cache.live):
            eng.cache.free_request(rid)
        for g in eng.cache.groups:
            g.pool.normal_(0.0, 0.5)
        for b in range(B):
            eng.cache.add_request(("seq", b))
            eng.cache.append(("seq", b), args.context - 1)

    def decode_device(B, steps, warmup):
        fill_cache(B)
        toks = torch.randint(0, V, (B,), generator=gen).tolist()

        def one():
            return eng.step([StepEntry(("seq", b), [toks[b]], [0]) for b in range(B)])
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        l0 = ops.launches
        s, e = ev(), ev()
        s.record()
        for _ in range(steps):
            one()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / steps, (ops.launches - l0)

    def decode_e2e(B, steps, warmup):
        fill_cache(B)
        toks = torch.randint(0, V, (B,), generator=gen).tolist()
        pos = args.context - 1
        for _ in range(warmup):
            toks = llm.forward_batch([DecodeRequest(b, toks[b], pos) for b in range(B)])
            pos += 1
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            toks = llm.forward_batch([DecodeRequest(b, toks[b], pos) for b in range(B)])
            pos += 1
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / steps

    points = {}
    if args.only == "prefill":
        print(json.dumps({"prefill": prefill}))
        return 0
    for B in sizes:
        if B == args.batch:
            continue
        ms, _ = decode_device(B, max(5, args.steps // 2), args.warmup)
        points[f"decode_b{B}"] = B / (ms / 1e3)

    sampler = ClockSampler()
    sampler.start()
    B = args.batch
    ms_step, launches = decode_device(B, args.steps, args.warmup)
    clocks = sampler.stop()
    e2e_ms = decode_e2e(B, args.steps, args.warmup)
    graph_launches = getattr(eng, "graph_kernel_count", lambda n: 0)(B)
    if graph_launches:
        launches = graph_launches * args.steps
    status = ops.gemm_tc_status()

    bytes_step = weight_elems * 2 + B * args.context * kv_per_token * 2
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    blocks_w = -(-(args.context + 1) // page)
    out = {
        "metric": f"decode tok/s at batch {B}, context {args.context} ({shape_name} shape, bf16)",
        "value": B / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{shape_name} shape, random weights N(0,0.02) seed {weight_seed}", "global_batch": B,
                   "seq_len": args.context, "parallelism": "single GPU", "layers": args.layers,
                   "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": nh,
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": V, "page_size": page, "kv_dtype": "bf16",
                   "kv_fill": "random keys/values at context-1 tokens", "l2": "inputs larger than L2",
                   "cuda_graphs": not args.no_graphs, "peaks": pk["source"]},
        "e2e": {"value": B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 4 * (3 * B + (B + 1) + 3 * B + B + B * blocks_w),
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clocks,
        "kernel_status": status,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
