#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

Default run: the layer sizes of the Llama-3.1-8B shape with random bfloat16 weights,
decode at batch 8 and context 8,192 (K timed steps after W warm-up steps), plus
prefill of 2,048 tokens, decode at batch 1 and 64, steps of 512 and 1,024 tokens, the
share of each kernel in a decode step and in the prefill step, and two serving
workloads through ``generate()`` (Qwen2.5-7B sizes: 32 requests with prompts of 512 to
4,096 tokens mixed with decoding; Qwen2.5-14B sizes: 16 prompts of 16,384 tokens, then
256 tokens each).  A "step" is one decode step.  ``value`` is decoded tokens per second
timed on the device; ``e2e`` is the same through the Python entry point with host
token lists in and out.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

``--impl reference`` runs the unmodified reference (fxslava/BlackwellLLM's dense core, built for
sm_100a by ``baseline/build_reference.sh`` into ``baseline/_ref``) on the same sizes through its
own public calls, and prints the same line with ``"impl": "reference"``.
"""
import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import tempfile
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
# the other two big shapes: for --shape and for the serving workloads
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
# the serving workloads: (shape, requests, shortest prompt, longest prompt, new tokens each)
SERVE = {"qwen2.5-7b": (32, 512, 4096, 128), "qwen2.5-14b": (16, 16384, 16384, 256)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "bf16_tflops_burst": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id="0"):
        self.proc = None
        self.gpu_id = gpu_id      # the UUID of the CUDA device that is timed, not an nvidia-smi index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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


def device_uuid():
    """``GPU-<uuid>`` of CUDA device 0 (what ``nvidia-smi -i`` takes; its own index 0 may be another GPU
    on a shared machine)."""
    import torch
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(0).uuid)
    except Exception:
        return "0"


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    weight_elems = layers * per_layer + V * H  # embedding rows read are negligible
    kv_per_token = layers * 2 * nkv * hd
    return per_layer, weight_elems, kv_per_token


def config_record(shape_name, weight_seed, cfg, args, full_layers, pk, **more):
    """``config`` of the JSON line: flat, at most 20 keys."""
    rec = {"model": f"{shape_name} shape, random weights N(0,0.02) seed {weight_seed}", "global_batch": args.batch,
           "seq_len": args.context, "parallelism": "single GPU", "layers": args.layers,
           "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
           "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": 16, "kv_dtype": "bf16",
           "kv_fill": "random keys/values at context-1 tokens", "l2": "inputs larger than L2",
           "cuda_graphs": not args.no_graphs, "peaks": pk["source"]}
    rec.update(more)
    assert len(rec) <= 20
    return rec


# ---------------------------------------------------------------------------------------------- the reference arm

def reference_arm(args):
    """Runs ``baseline/_ref/ref_bench`` (the reference's own engine behind its public calls) on a random
    checkpoint of the same sizes and prints the line; any obstacle becomes the ``unavailable`` line."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if args.gpus != 1:
        return unavailable("the reference's engine runs on one GPU")
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_bench")
    if not os.path.isfile(exe):
        ref_src = os.environ.get("BLACKWELLLLM_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
        script = os.path.join(ROOT, "baseline", "build_reference.sh")
        if os.path.isdir(os.path.join(ref_src, "src", "core")):
            built = subprocess.run(["sh", script, ref_src], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if built.returncode != 0:
                return unavailable("baseline/build_reference.sh failed: " + built.stdout.strip().splitlines()[-1][:300])
        if not os.path.isfile(exe):
            return unavailable("baseline/_ref/ref_bench is not built and no reference checkout is beside the "
                               "repository (run baseline/build_reference.sh <checkout>)")
    import torch
    from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
    from blackwellllm_b200.weights.safetensors_io import write_file
    shape_name, shape_cfg, weight_seed = SHAPES[args.shape]
    full_layers = shape_cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    args.layers = layers
    cfg = dict(shape_cfg, num_hidden_layers=layers, torch_dtype="bfloat16")
    pk = peaks()
    with tempfile.TemporaryDirectory(prefix="reference_model_") as folder:
        # the same random tensors as our own arm (same seed, same order), made on the GPU, stored as bfloat16
        tensors = random_tensors(model_param_specs(cfg), seed=weight_seed, std=0.02, dtype=torch.bfloat16, device="cuda:0")
        tensors = {k: v.cpu() for k, v in tensors.items()}
        torch.cuda.empty_cache()
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_file(os.path.join(folder, "model.safetensors"), tensors)
        del tensors
        sampler = ClockSampler(device_uuid())
        sampler.start()
        cmd = [exe, os.path.join(folder, "model.safetensors"), str(args.batch), str(args.context), str(args.steps),
               str(args.warmup), str(args.prefill_tokens), str(cfg["vocab_size"])]
        try:
            run = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=1500)
        except subprocess.TimeoutExpired:
            sampler.stop()
            return unavailable("the reference did not finish within 1500 s at these sizes")
        clocks = sampler.stop()
    fields = {}
    for line in run.stdout.splitlines():
        if "status=" in line:
            fields = dict(kv.split("=", 1) for kv in line.split() if "=" in kv)
    if run.returncode != 0 or fields.get("status") != "ok":
        tail = (run.stderr.strip().splitlines() or [""])[-1][:200]
        return unavailable(f"the reference's engine failed (exit {run.returncode}, {fields.get('status', 'no status line')}) {tail}")
    ms_step, prefill_ms = float(fields["decode_ms_per_step"]), float(fields["prefill_ms"])
    B, T = args.batch, args.prefill_tokens
    per_layer, weight_elems, kv_per_token = model_bytes_and_flops(cfg, layers)
    achieved = (weight_elems * 2 + B * args.context * kv_per_token * 2) / (ms_step / 1e3) / 1e9
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2.0 * T * layers * per_layer + 2.0 * cfg["vocab_size"] * cfg["hidden_size"] + layers * 4.0 * nh * hd * T * (T + 1) / 2
    blocks_w = -(-(args.context + 1) // 16)
    print(json.dumps({
        "metric": f"decode tok/s at batch {B}, context {args.context} ({shape_name} shape, bf16)",
        "value": B / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": config_record(shape_name, weight_seed, cfg, args, full_layers, pk, cuda_graphs=False,
                                kv_fill="each sequence prefilled with its own random tokens after a shared first page"),
        # the reference's calls take host tokens and return host tokens: its only number IS end to end
        "e2e": {"value": B / (ms_step / 1e3), "unit": "tokens/s", "ms_per_step": ms_step,
                "h2d_bytes_per_step": 4 * (4 * B + B * blocks_w), "d2h_bytes_per_step": 4 * B},
        "prefill": {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
                    "frac": flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                    "frac_burst": flops / (prefill_ms / 1e3) / (pk["bf16_tflops_burst"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "timing": "host wall clock around the reference's blocking calls (prefill_status, forward_batch)",
        "fill_seconds": float(fields.get("fill_s", 0.0)), "clocks": clocks}))
    return 0


# ---------------------------------------------------------------------------------------------- kernel shares

def kernel_shares(ops, run_step):
    """Share of each launcher in one step: the step runs once more, uncaptured, with a CUDA-event timer
    around every launcher call (each call synchronised, so the times are of kernels alone, cold; shares,
    not absolutes).  Launchers are named by what they compute in the model."""
    ops.enable_timing(True)
    try:
        run_step()
    finally:
        report = ops.timing_report()
        ops.enable_timing(False)
    total = sum(ms for _, ms in report.values()) or 1.0
    groups = {}
    for name, (calls, ms) in report.items():
        groups[name] = groups.get(name, 0.0) + ms
    return {k: round(v / total, 4) for k, v in sorted(groups.items(), key=lambda kv: -kv[1])}


def name_launchers(cfg):
    """Maps a launcher's timing tag to the model's name for it (by the product's shape)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (nh + 2 * nkv) * hd

    def rename(tag):
        fn, _, shape = tag.partition(" ")
        if fn in ("bw_gemm_tc", "bw_gemm_tc_rope", "bw_gemm_tc_planes") and shape:
            dims = shape.replace("rope", "").replace("planes", "").split("x")
            N, K = int(dims[1]), int(dims[2])
            if fn == "bw_gemm_tc_rope" or (N, K) == (qkv, H):
                return "gemm_qkv" + ("+rope+append" if fn == "bw_gemm_tc_rope" else "")
            if (N, K) == (H, nh * hd):
                return "gemm_o+residual"
            if (N, K) == (2 * I, H):
                return "gemm_gate_up+swiglu"
            if (N, K) == (H, I):
                return "gemm_down+residual"
            if (N, K) == (V, H):
                return "gemm_lm_head"
        return {"bw_attention_tc": "attention_prefill_tcgen05", "bw_attention_mma": "attention_decode_mma",
                "bw_rmsnorm": "rmsnorm", "bw_add_rmsnorm": "rmsnorm", "bw_rope_table": "rope_table", "bw_kv_slots": "kv_slots",
                "bw_rope_append": "rope_append", "bw_embed_gather": "embed_gather"}.get(fn, fn)
    return rename


# ---------------------------------------------------------------------------------------------- serving workloads

def serve_workload(shape_key, steps_cap=None):
    """BASELINE workloads 4 and 5: N requests with random prompts through ``generate()`` (the scheduler's
    continuous batching, token budget 2,048, greedy, no end-of-sequence): wall-clock tokens per second."""
    import torch
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, SamplingParams
    shape_name, cfg, seed = SHAPES[shape_key]
    n_req, lo, hi, new = SERVE[shape_key]
    rng = random.Random(seed)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(lo, hi))] for _ in range(n_req)]
    ctx = hi + new + 16
    llm = BlackwellEngine(None, InferenceConfig(max_context_length=ctx, max_batch_size=n_req), config=cfg,
                          random_seed=seed, random_std=0.02, dtype="bfloat16", page_size=16, max_batch_tokens=2048, seed=0)
    sp = SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True)
    llm.generate([prompts[0][:64]], SamplingParams(temperature=0.0, max_new_tokens=4, ignore_eos=True))   # warm-up
    torch.cuda.synchronize()
    steps0 = llm.scheduler.stats.steps
    t0 = time.perf_counter()
    res = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_prompt, n_new = sum(len(p) for p in prompts), sum(len(r.token_ids) for r in res)
    out = {"requests": n_req, "prompt_tokens": n_prompt, "new_tokens": n_new, "seconds": round(dt, 3),
           "tokens_per_s": (n_prompt + n_new) / dt, "new_tokens_per_s": n_new / dt,
           "steps": llm.scheduler.stats.steps - steps0, "preemptions": llm.scheduler.stats.preemptions}
    del llm, res
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


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
    ap.add_argument("--step-widths", default="512,1024", help="steps of this many prompt tokens to report (ms)")
    ap.add_argument("--workload", default="default", choices=["default", "serve", "none"],
                    help="serve: only the shape's serving workload through generate(); none: leave the serving "
                         "workloads out of the default run")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (for profiling); the JSON line then lacks the other part")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported"}))
        return 2
    if args.workload == "serve":
        if args.shape not in SERVE:
            print(json.dumps({"error": f"no serving workload for --shape {args.shape}; one of {sorted(SERVE)}"}))
            return 2
        print(json.dumps({"workload": f"serve {args.shape}", **serve_workload(args.shape)}))
        return 0

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
    widths = [int(x) for x in args.step_widths.split(",") if x]
    max_b = max(sizes)
    room = args.context + args.warmup + args.steps * 2 + 64
    num_pages = max_b * -(-room // page) + -(-args.prefill_tokens // page) + 8
    llm = BlackwellEngine(None, InferenceConfig(max_context_length=room + 64, max_batch_size=max_b + 1),
                          config=cfg, random_seed=weight_seed, random_std=0.02, dtype="bfloat16", page_size=page,
                          num_pages=num_pages, max_batch_tokens=max(args.prefill_tokens, max_b), seed=0,
                          cuda_graphs=not args.no_graphs)
    eng = llm.engine
    eng.options.graph_after = 1   # the decode measurements' batch sizes are recorded in their first warm-up step
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1234)
    per_layer, weight_elems, kv_per_token = model_bytes_and_flops(cfg, args.layers)
    rename = name_launchers(cfg)

    def renamed(shares):
        out = {}
        for tag, frac in shares.items():
            out[rename(tag)] = round(out.get(rename(tag), 0.0) + frac, 4)
        return out

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------- prefill of T tokens (one step, logits at the last position)
    def time_prompt_step(n_tokens, reps=3):
        prompt = torch.randint(0, V, (n_tokens,), generator=gen).tolist()
        times = []
        for _ in range(reps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            eng.step([StepEntry("prefill", prompt, [n_tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
            eng.end_request("prefill")
        return min(times[1:]), prompt

    T = args.prefill_tokens
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    prefill = {"value": None, "tokens": T, "ms": None, "frac": None}
    kernels = {}
    step_points = {}
    if args.only != "decode":
        prefill_ms, prompt = time_prompt_step(T)
        prefill_flops = 2.0 * T * args.layers * per_layer + 2.0 * V * cfg["hidden_size"] \
            + args.layers * 4.0 * nh * hd * T * (T + 1) / 2
        prefill = {"value": T / (prefill_ms / 1e3), "tokens": T, "ms": prefill_ms,
                   "frac": prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                   "frac_burst": prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_burst"] * 1e12)}

        def one_prefill():
            eng.step([StepEntry("prefill", prompt, [T - 1])])
            eng.end_request("prefill")
        kernels["prefill"] = renamed(kernel_shares(ops, one_prefill))
        for w in widths:
            if w <= eng.options.max_batch_tokens:
                step_points[f"step_{w}_tokens_ms"] = time_prompt_step(w)[0]

    # ---------------- decode at context C: caches of B requests filled with random keys and values
    def fill_cache(B, context=None):
        for rid in list(eng.cache.live):
            eng.cache.free_request(rid)
        for g in eng.cache.groups:
            g.pool.normal_(0.0, 0.5)
        for b in range(B):
            eng.cache.add_request(("seq", b))
            eng.cache.append(("seq", b), (context or args.context) - 1)

    def decode_device(B, steps, warmup, context=None):
        fill_cache(B, context)
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
        """Every step: host token ids in (they go to the device in the step's packed buffer, from pinned
        memory), host token ids out (read back before the next step is made)."""
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

    def decode_e2e_pipelined(B, steps, warmup):
        """The same loop as a server runs it: step n + 1 is queued (its packed buffer from pinned memory,
        its token ids taken on the device from step n's sampler) before step n's tokens are read on the
        host; every step's tokens still reach the host, one step late."""
        from blackwellllm_b200 import FROM_LAST
        fill_cache(B)
        toks = torch.randint(0, V, (B,), generator=gen).tolist()
        pos = args.context - 1
        pending = llm.forward_batch_async([DecodeRequest(b, toks[b], pos) for b in range(B)])
        got = 0
        for i in range(warmup + steps):
            if i == warmup:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
            pos += 1
            nxt = llm.forward_batch_async([DecodeRequest(b, FROM_LAST, pos) for b in range(B)])
            got += len(pending.result())
            pending = nxt
        pending.result()
        torch.cuda.synchronize()
        assert got == (warmup + steps) * B
        return (time.perf_counter() - t0) * 1e3 / steps

    def generate_decode_steps(B, prompt_len, pipeline, steps=40):
        """Wall-clock ms per decode-only step of ``generate()``'s own loop (scheduler, sampler, read-back of
        the tokens) at batch B: what the host adds shows against the device-only time of the same step."""
        from blackwellllm_b200 import SamplingParams
        for rid in list(eng.cache.live):
            eng.cache.free_request(rid)
        llm.pipeline = pipeline
        sp = SamplingParams(temperature=0.0, max_new_tokens=steps + 20, ignore_eos=True)
        for b in range(B):
            llm.add_request(torch.randint(0, V, (prompt_len,), generator=gen).tolist(), sp)
        sch = llm.scheduler
        while sch.waiting or any(r.remaining > 1 for r in sch.running):
            llm.step()
        for _ in range(8):      # the first decode step of this batch size records its graph
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / steps
        while sch.has_work():
            llm.step()
        llm.pipeline = True
        return ms

    points = dict(step_points)
    if args.only == "prefill":
        print(json.dumps({"prefill": prefill, "kernels": kernels, "points": points}))
        return 0
    for B in sizes:
        if B == args.batch:
            continue
        ms, _ = decode_device(B, max(5, args.steps // 2), args.warmup)
        points[f"decode_b{B}"] = B / (ms / 1e3)

    sampler = ClockSampler(device_uuid())
    sampler.start()
    B = args.batch
    ms_step, launches = decode_device(B, args.steps, args.warmup)
    e2e_ms = decode_e2e(B, args.steps, args.warmup)
    e2e_pipe_ms = decode_e2e_pipelined(B, args.steps, args.warmup)
    clocks = sampler.stop()      # over the three timed decode regions (device, end to end, pipelined)
    graph_launches = getattr(eng, "graph_kernel_count", lambda n: 0)(B)
    if graph_launches:
        launches = graph_launches * args.steps

    # what the host adds to a decode step of generate() at batch 32 (short contexts, where it weighs most)
    if 32 <= max_b and args.only == "all":
        points["generate_b32_ms_per_step"] = generate_decode_steps(32, 512, True)
        points["generate_b32_ms_per_step_unpipelined"] = generate_decode_steps(32, 512, False)
        points["generate_b32_device_ms_per_step"] = decode_device(32, 20, args.warmup, context=512 + 40)[0]

    # the share of each kernel in a decode step: one more step, uncaptured and timed launcher by launcher
    fill_cache(B)
    toks = torch.randint(0, V, (B,), generator=gen).tolist()
    graphs_on, eng.options.cuda_graphs = eng.options.cuda_graphs, False
    try:
        kernels["decode"] = renamed(kernel_shares(ops, lambda: eng.step([StepEntry(("seq", b), [toks[b]], [0]) for b in range(B)])))
    finally:
        eng.options.cuda_graphs = graphs_on
    status = ops.gemm_tc_status() | ops.attention_tc_status()

    bytes_step = weight_elems * 2 + B * args.context * kv_per_token * 2
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    blocks_w = -(-(args.context + 1) // page)
    out = {
        "metric": f"decode tok/s at batch {B}, context {args.context} ({shape_name} shape, bf16)",
        "value": B / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": config_record(shape_name, weight_seed, cfg, args, full_layers, pk),
        "e2e": {"value": B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 4 * (3 * B + (B + 1) + 3 * B + B + B * blocks_w),
                "d2h_bytes_per_step": 4 * B},
        # a server's loop: the next step is queued before this step's tokens are read (they are fed on the device)
        "e2e_pipelined": {"value": B / (e2e_pipe_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_pipe_ms,
                          "h2d_bytes_per_step": 4 * (3 * B + (B + 1) + 3 * B + B + B * blocks_w), "d2h_bytes_per_step": 4 * B},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "kernels": kernels,
        "clocks": clocks,
        "kernel_status": status,
    }
    # ---------------- the serving workloads of the other two shapes, through generate()
    if args.workload == "default" and args.only == "all" and args.shape == "llama-3.1-8b" and args.layers == full_layers:
        del llm, eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for key in SERVE:
            try:
                r = serve_workload(key)
                out["points"][f"serve_{key}_tokens_per_s"] = r["tokens_per_s"]
                out["points"][f"serve_{key}_new_tokens_per_s"] = r["new_tokens_per_s"]
                out["points"][f"serve_{key}_seconds"] = r["seconds"]
            except Exception as e:   # the headline number stands even if a side workload cannot run
                out["points"][f"serve_{key}_error"] = f"{type(e).__name__}: {e}"[:200]
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
