#!/usr/bin/env python3
"""Benchmark of lumenllm_b200 on one B200: decode tokens per second of a
Qwen3-8B-shaped model (random bfloat16 weights, synthetic token ids) at batch 8,
with prefill of 2,048 tokens, batch-1 and batch-64 decode, an end-to-end number
through the Python entry point, time to the first token of short prompts, and the
HBM roofline of the decode step.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--timings]

`--shape` runs the same measurement at the two larger workloads (their batch, prompt
lengths, context and sampling); `--timings` adds, from a separate pass that is not
timed as a whole, each kernel class's share of a decode step and of a prompt step.
One JSON line goes to standard output. More than one GPU is not built: the
program says so and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_key_value_heads=8, head_dim=128,
              vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
              tie_word_embeddings=False)
# The benchmark shape (Qwen3-8B) and the two larger workloads: layer sizes, and per workload the
# batch, the range of prompt lengths, the context length and how tokens are chosen.
WORKLOADS = {
    "8b": dict(model=dict(COMMON, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                          intermediate_size=12288),
               batch=8, prompt=(1024, 2048), context=4096, temperature=0.0),
    "14b": dict(model=dict(COMMON, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40,
                           intermediate_size=17408),
                batch=16, prompt=(256, 6144), context=8192, temperature=0.0),
    "32b": dict(model=dict(COMMON, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                           intermediate_size=25600),
                batch=8, prompt=(128, 2048), context=4096, temperature=0.7),
}
SHAPE = WORKLOADS["8b"]["model"]
CONTEXT = 4096
PROMPT_LO, PROMPT_HI = 1024, 2048
PREFILL_TOKENS = 2048
TEMPERATURE = 0.0
SAMPLING_SEED = 1234


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class Clocks:
    """Samples nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def mark(self):
        return time.perf_counter()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not any(a <= t <= b for a, b in windows):
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])); mx = max(mx, float(f[1]))
            except (ValueError, IndexError):
                continue
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qw = cfg["num_attention_heads"] * cfg["head_dim"]
    kvw = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = H * (qw + 2 * kvw) + qw * H + 3 * H * I
    return {"layer_params": per_layer * layers, "head_params": V * H,
            "kv_bytes_per_token": 2 * layers * kvw * 2}


def sampling_for(B):
    """Options of the B sequences and a function step -> their uniform numbers: greedy, or at the
    workload's temperature with one seeded stream of uniforms per sequence (made on the host and
    passed to the device sampler every step, as generation does)."""
    from lumenllm_b200.sampling import SamplingConfig, uniform
    if TEMPERATURE <= 0.0:
        return [SamplingConfig()] * B, (lambda step: [0.0] * B)
    cfgs = [SamplingConfig(temperature=TEMPERATURE, seed=SAMPLING_SEED + i) for i in range(B)]
    return cfgs, (lambda step: [uniform(SAMPLING_SEED + i, 0, step) for i in range(B)])


def decode_run(eng, B, steps, warmup, seed):
    """Prefills B prompts (lengths uniform in [PROMPT_LO, PROMPT_HI]), then decodes
    with the sampled tokens fed back on the device. Returns per-step ms and bytes read."""
    import torch
    from lumenllm_b200 import StepEntry
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(PROMPT_LO, PROMPT_HI + 1, (B,), generator=g).tolist()
    prompts = [torch.randint(0, eng.vocab_size, (n,), generator=g).tolist() for n in lens]
    slots = [eng.alloc_slot() for _ in range(B)]
    logits = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    cfgs, uniforms = sampling_for(B)
    tok = eng.sampler.pick(logits, cfgs, uniforms(0))
    entries = [(s, [0]) for s in slots]
    for k in range(warmup):
        tok = eng.run_device(entries, cfgs, uniforms(1 + k), tokens_on_device=tok)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for k in range(steps):
        tok = eng.run_device(entries, cfgs, uniforms(1 + warmup + k), tokens_on_device=tok)
    ev1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    eng.check_kernels()
    ms = ev0.elapsed_time(ev1) / steps
    mean_len = sum(lens) / B + warmup + steps / 2
    launches = getattr(eng.graphs, "last", None)
    per = launches.kernels_per_replay if launches is not None else 0
    for s in slots:
        eng.free_slot(s)
    return {"ms": ms, "mean_len": mean_len, "window": (t0, t1), "kernels_per_step": per,
            "tok_s": B * 1000.0 / ms}


def first_token_run(eng, n_tokens, runs=7):
    """Milliseconds from the call with a prompt of n_tokens host tokens to its first sampled
    token on the host (median of `runs`, after two untimed ones)."""
    import torch
    g = torch.Generator().manual_seed(100 + n_tokens)
    prompt = torch.randint(0, eng.vocab_size, (n_tokens,), generator=g).tolist()
    cfgs, uniforms = sampling_for(1)
    times = []
    for it in range(2 + runs):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.run([(s, prompt)], cfgs, uniforms(0))
        times.append((time.perf_counter() - t0) * 1e3)
        eng.free_slot(s)
    return statistics.median(times[2:])


def timings_pass(eng, B, model_cfg):
    """Each kernel class's share of one decode step at batch B and of one 2,048-token prompt
    step, from a pass of its own: every launch is bracketed by two CUDA events (which also
    keeps kernels from overlapping, so the shares are of the sum of the kernels' own times,
    not of the step's time). After crates/aegisllm-cuda/src/executor/prefill/timings.rs:1-39."""
    import torch
    from lumenllm_b200 import StepEntry
    from lumenllm_b200.ops import native
    H, I = model_cfg["hidden_size"], model_cfg["intermediate_size"]
    qw = model_cfg["num_attention_heads"] * model_cfg["head_dim"]
    kvw = model_cfg["num_key_value_heads"] * model_cfg["head_dim"]
    products = {(qw + 2 * kvw, H): "qkv", (H, qw): "o", (2 * I, H): "gate_up", (H, I): "down",
                (model_cfg["vocab_size"], H): "head"}
    if qw == I:      # cannot happen for the shapes here; keeps the table honest if it does
        products[(H, qw)] = "o_or_down"
    names = {"lumen_add_rmsnorm": "norm", "lumen_qk_norm_rope_store": "qk_norm_rope_store",
             "lumen_rope_table": "rope_table", "lumen_silu_mul": "silu_mul", "lumen_embed": "embed",
             "lumen_attn_decode": "attention", "lumen_attn_decode_qkv": "attention + rotary",
             "lumen_embed_tiled": "embed", "lumen_attn_prefill_tc": "attention",
             "lumen_attn_prefill": "attention", "lumen_attn_generic": "attention",
             "lumen_argmax": "sampling", "lumen_sample": "sampling", "lumen_gemm_tc_qkv": "qkv"}

    def label(name, args):
        if name == "lumen_gemm_tc":
            return products.get((int(args[4]), int(args[5])), "other_product")
        return names.get(name, name)

    def shares(run):
        rec = []
        native.instrument(lambda name, args: rec.append([label(name, args), torch.cuda.Event(enable_timing=True),
                                                         torch.cuda.Event(enable_timing=True)]) or rec[-1])
        try:
            run()
            torch.cuda.synchronize()
        finally:
            native.instrument(None)
        total, by = 0.0, {}
        for lab, e0, e1 in rec:
            ms = e0.elapsed_time(e1)
            by[lab] = by.get(lab, 0.0) + ms
            total += ms
        out = {k: round(v / total, 4) for k, v in sorted(by.items(), key=lambda kv: -kv[1])}
        out["sum_ms"] = round(total, 3)
        out["launches"] = len(rec)
        return out

    g = torch.Generator().manual_seed(5)
    lens = torch.randint(PROMPT_LO, PROMPT_HI + 1, (B,), generator=g).tolist()
    slots = [eng.alloc_slot() for _ in range(B)]
    eng.step([StepEntry(s, torch.randint(0, eng.vocab_size, (n,), generator=g).tolist(), [])
              for s, n in zip(slots, lens)])
    cfgs, uniforms = sampling_for(B)
    was = eng.use_graphs
    eng.use_graphs = False            # launch by launch, so that every kernel can be bracketed
    try:
        for _ in range(2):
            eng.run_device([(s, [1]) for s in slots], cfgs, uniforms(0))
        decode = shares(lambda: eng.run_device([(s, [1]) for s in slots], cfgs, uniforms(1)))
    finally:
        eng.use_graphs = was
    for s in slots:
        eng.free_slot(s)
    prompt = torch.randint(0, eng.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
    s = eng.alloc_slot()
    prefill = shares(lambda: eng.step([StepEntry(s, prompt, [PREFILL_TOKENS - 1])]))
    eng.free_slot(s)
    return {"decode": decode, "prefill": prefill}


def prefill_run(eng, warmup, runs=5):
    import torch
    from lumenllm_b200 import StepEntry
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, eng.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
    times, windows = [], []
    for it in range(warmup + runs):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        eng.step([StepEntry(s, prompt, [PREFILL_TOKENS - 1])])
        ev1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        eng.free_slot(s)
        if it >= warmup:
            times.append(ev0.elapsed_time(ev1))
            windows.append((t0, t1))
    return statistics.median(times), windows


def e2e_run(built, B, steps, warmup, seed):
    """The same decode through the public entry point: host token lists in, host token
    lists out, one host<->device round trip per step. As with the device-timed steps the
    first `warmup` decode steps after the prompts are not timed (the GPU's clocks come back
    from the prompts' power draw over the first ten or twenty): the timed region runs from the
    moment the host holds every sequence's token of step `warmup` to the moment it holds the
    tokens of step `warmup + steps`, taken where `generate` hands the tokens over."""
    import torch
    from lumenllm_b200 import GenerateRequest
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(PROMPT_LO, PROMPT_HI + 1, (B,), generator=g).tolist()
    prompts = [torch.randint(0, built.engine.vocab_size, (n,), generator=g).tolist() for n in lens]
    cfgs, _ = sampling_for(B)
    reqs = [GenerateRequest(p, warmup + steps + 1, c) for p, c in zip(prompts, cfgs)]
    stamps = []          # when the last sequence's k-th token reached the host

    def on_token(i, tok):
        if i == B - 1:
            stamps.append(time.perf_counter())

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = built.generate(reqs, eos_token_ids=[], max_batch=B, on_token=on_token)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if len(stamps) != warmup + steps + 1 or any(o.completion_tokens != warmup + steps + 1 for o in outs):
        raise RuntimeError("e2e: generate did not return the tokens asked for")
    timed = stamps[warmup + steps] - stamps[warmup]
    whole = max(o.decode_s for o in outs)
    return {"tok_s": B * steps / timed, "decode_s": timed, "window": (t0, t1),
            "whole_tok_s": (sum(o.completion_tokens for o in outs) - B) / whole}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(WORKLOADS),
                    help="layer sizes and workload (default: the benchmark configuration, 8b)")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the shape has, for small memory (named in config)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--points", default="1,64", metavar="B,B",
                    help="batch sizes of the further decode points (default 1,64)")
    ap.add_argument("--timings", action="store_true",
                    help="add each kernel class's share of a decode and of a prompt step")
    ap.add_argument("--context", type=int, default=None,
                    help="context length (default: the workload's)")
    ap.add_argument("--prompt-len", default=None, metavar="LO:HI",
                    help="prompt lengths are drawn uniformly from this range")
    args = ap.parse_args()
    wl = WORKLOADS[args.shape]
    shape = wl["model"]
    globals()["CONTEXT"] = args.context or wl["context"]
    lo, _, hi = (args.prompt_len or f"{wl['prompt'][0]}:{wl['prompt'][1]}").partition(":")
    globals()["PROMPT_LO"], globals()["PROMPT_HI"] = int(lo), int(hi or lo)
    globals()["TEMPERATURE"] = wl["temperature"]
    layers = args.layers or shape["num_hidden_layers"]
    if not 1 <= PROMPT_LO <= PROMPT_HI or PROMPT_HI + 64 + max(3, args.warmup) + max(1, args.steps) + 64 > CONTEXT:
        print("bench.py: prompts, warm-up and steps must fit the context", file=sys.stderr)
        return 2
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is Rust + NVRTC CUDA for SM120; no Rust toolchain on "
                          "this image, so it cannot be built or installed offline"}))
        return 0
    if args.gpus != 1:
        print("bench.py: lumenllm_b200 is a single-GPU library; --gpus > 1 is not built")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch
    from lumenllm_b200.engine import BuiltEngine, Engine
    from lumenllm_b200.config import SamplingDefaults
    from lumenllm_b200.ops import native
    pk = peaks()
    cfg = dict(shape, num_hidden_layers=layers)
    B = args.batch or wl["batch"]
    point_batches = [] if args.no_points else [int(x) for x in args.points.split(",") if x.strip()]
    top_b = max([B] + point_batches)
    max_tokens = max(B * CONTEXT, top_b * (PROMPT_HI + 64 + warmup + steps + 64))
    nums = model_numbers(cfg, layers)
    need = max_tokens * nums["kv_bytes_per_token"] + 2 * (nums["layer_params"] + 2 * nums["head_params"])
    if need > 165e9:
        print(f"bench.py: {need / 1e9:.0f} GB of weights and cache do not fit; use --no-points, a "
              "smaller --batch or --context, or fewer --layers", file=sys.stderr)
        return 2
    eng = Engine.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", max_tokens=max_tokens,
                             max_slots=max(top_b, 8), context_size=CONTEXT)
    eng.graphs.min_width = CONTEXT // 64
    built = BuiltEngine(eng, SamplingDefaults(temperature=TEMPERATURE, seed=SAMPLING_SEED), B)
    clocks = Clocks()
    clocks.start()

    # the prompt measurement first: it is the one compared with a burst figure (the peak that
    # a GEMM reaches before the power cap settles the clocks), so it runs before the long
    # decode loops have warmed the GPU
    pre_ms, pre_windows = prefill_run(eng, warmup=3)
    ttft = {str(n): round(first_token_run(eng, n), 3) for n in (128, 512)}

    launches0 = native.launches
    main_run = decode_run(eng, B, steps, warmup, seed=1)
    eager_launches = native.launches - launches0
    ms = main_run["ms"]
    weight_bytes = 2 * (nums["layer_params"] + nums["head_params"])
    kv_bytes = B * main_run["mean_len"] * nums["kv_bytes_per_token"]
    achieved = (weight_bytes + kv_bytes) / (ms * 1e-3) / 1e9

    T = PREFILL_TOKENS
    flops = 2 * T * nums["layer_params"] + 2 * nums["head_params"] \
        + layers * 2 * T * T * cfg["head_dim"] * cfg["num_attention_heads"]
    pre_frac = flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

    # three runs, the median: a run is a quarter of a second, and host jitter shows in it
    e2e_runs = sorted((e2e_run(built, B, steps, warmup, seed=2) for _ in range(3)), key=lambda r: r["tok_s"])
    e2e = e2e_runs[1]
    e2e["window"] = (min(r["window"][0] for r in e2e_runs), max(r["window"][1] for r in e2e_runs))
    points, points_frac, windows = {}, {}, [main_run["window"], e2e["window"]] + pre_windows
    if point_batches:
        for b in point_batches:
            r = decode_run(eng, b, min(steps, 32), warmup, seed=10 + b)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            got = (weight_bytes + b * r["mean_len"] * nums["kv_bytes_per_token"]) / (r["ms"] * 1e-3) / 1e9
            points_frac[f"decode_b{b}"] = round(got / pk["hbm_gbs"], 4)
            windows.append(r["window"])
    time.sleep(0.3)
    clocks.stop()
    timings = timings_pass(eng, B, cfg) if args.timings else None
    sampled = TEMPERATURE > 0.0
    # per step and host to device: the step's metadata, and with sampling its options and
    # uniform numbers; device to host: the sampled tokens and the kernels' error flag
    meta_bytes = 4 * (9 * 4 * ((B + 3) // 4 + 1) + B * (CONTEXT // 64)) + (20 * B if sampled else 0)
    out = {
        "metric": "decode_tokens_per_s", "value": round(main_run["tok_s"], 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {"model": f"qwen3-{args.shape}-shape", "layers": layers,
                   "layers_of_shape": shape["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied_head": False, "global_batch": B,
                   "seq_len": CONTEXT, "prompt_len": f"{PROMPT_LO}..{PROMPT_HI}",
                   "parallelism": "single", "weights": "random N(0,0.02)",
                   "sampling": f"temperature {TEMPERATURE} seeded" if sampled else "greedy",
                   "l2": "inputs_larger_than_l2", "peaks": pk["source"]},
        "clocks": clocks.summary(windows),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": 4 * B + 4,
                "untimed_first_steps": warmup, "with_first_steps": round(e2e["whole_tok_s"], 1)},
        "gpu_launches": int(main_run["kernels_per_step"] * steps) or int(eager_launches),
        "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(pre_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "points_roofline_frac": points_frac,     # the same bytes-over-time figure as "roofline"
        "first_token_ms": ttft,                  # prompts of 128 and 512 tokens, host to host
    }
    if timings is not None:
        out["timings"] = timings
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
