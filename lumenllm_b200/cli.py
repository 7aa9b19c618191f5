"""Command line in the manner of the reference's `aegisllm generate` (flags:
crates/aegisllm/src/cli/parse.rs:637-704; engine flags crates/aegisllm/src/cli/
flags.rs:74-161): `--config|--parameters`, `--model`, `--ctx-size`,
`--cuda-device`, `--max-tokens` (default 32), `--temp|--temperature`, `--top-k`,
`--top-p`. Flags override the parameters file. The reference takes text
(`--prompt`); this library has no tokenizer and takes token ids:

  lumenllm generate --config parameters.json --prompt-tokens 1,2,3 [--prompt-tokens 4,5]
                    [--prompt-file prompts.json] [--max-tokens N] [--temperature T] [--top-k K]
                    [--top-p P] [--min-p M] [--seed S] [--eos id,id] [--stop id,id]
                    [--dtype bfloat16|float32] [--format text|json]
  lumenllm bench-generate --config ... --prompt-tokens ... [--warmup W] [--runs R] [--format text|json]
  lumenllm random-model --config-json config.json --out DIR [--seed S] [--std X] [--norm-jitter A]
                        [--dtype bfloat16|float32]
  lumenllm replay --model DIR --dtype ... --out DIR --max-tokens N      (same as bin/trace_run)

`generate` prints the produced token ids, one request a line, to standard output
and `finish=... prompt_tokens=... completion_tokens=...` to standard error
(crates/aegisllm/src/cli/run.rs:213-218).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _ids(text):
    text = text.strip()
    return [int(x) for x in text.replace(",", " ").split()] if text else []


def _engine_flags(ap):
    ap.add_argument("--config", "--parameters", dest="parameters")
    ap.add_argument("--model")
    ap.add_argument("--ctx-size", type=int)
    ap.add_argument("--cuda-device", type=int)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"])
    ap.add_argument("--kv-max-tokens", type=int, help="tokens the cache holds (default ctx x batch)")
    ap.add_argument("--batch-size", type=int)
    ap.add_argument("--allow-extra-tensors", action="store_true",
                    help="warn about stored tensors that no part of the model reads instead of refusing them")


def _generate_flags(ap):
    ap.add_argument("--prompt-tokens", action="append", default=[],
                    help="token ids of one prompt, comma separated; repeat for a batch")
    ap.add_argument("--prompt-file", help="JSON file: a list of token-id lists")
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--temp", "--temperature", dest="temperature", type=float)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--top-p", type=float)
    ap.add_argument("--min-p", type=float)
    ap.add_argument("--seed", type=int)
    ap.add_argument("--eos", help="token ids that end a request without being kept")
    ap.add_argument("--stop", help="token ids that end a request and are kept")
    ap.add_argument("--format", choices=["text", "json"], default="text")


def _build(args):
    from .engine import EngineConfig, build
    return build(EngineConfig(model_path=args.model, parameters=args.parameters, dtype=args.dtype,
                              context_size=args.ctx_size, max_tokens=args.kv_max_tokens,
                              max_batch=args.batch_size, device=args.cuda_device,
                              strict_weights=not args.allow_extra_tensors))


def _requests(args, built):
    from .engine import GenerateRequest
    prompts = [_ids(p) for p in args.prompt_tokens]
    if args.prompt_file:
        prompts += [list(map(int, p)) for p in json.loads(open(args.prompt_file).read())]
    if not prompts:
        raise SystemExit("generate requires --prompt-tokens or --prompt-file")
    sampling = built.default_sampling(temperature=args.temperature, top_k=args.top_k,
                                      top_p=args.top_p, min_p=args.min_p, seed=args.seed)
    stop = _ids(args.stop) if args.stop else []
    return [GenerateRequest(p, args.max_tokens, sampling, stop) for p in prompts]


def cmd_generate(args):
    built = _build(args)
    reqs = _requests(args, built)
    eos = _ids(args.eos) if args.eos is not None else None
    outs = built.generate(reqs, eos_token_ids=eos)
    if args.format == "json":
        print(json.dumps([{"tokens": o.tokens, "prompt_tokens": o.prompt_tokens,
                           "completion_tokens": o.completion_tokens,
                           "finish_reason": o.finish_reason} for o in outs]))
    else:
        for o in outs:
            print(",".join(str(t) for t in o.tokens))
    for o in outs:
        print(f"finish={o.finish_reason} prompt_tokens={o.prompt_tokens} "
              f"completion_tokens={o.completion_tokens}", file=sys.stderr)
    return 0


def cmd_bench_generate(args):
    """Warm-up runs, measured runs, mean prefill and decode time, tokens per second
    (crates/aegisllm/src/engine/bench.rs:53-180)."""
    import torch
    built = _build(args)
    reqs = _requests(args, built)
    rows = []
    for it in range(args.warmup + args.runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = built.generate(reqs, eos_token_ids=[])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if it >= args.warmup:
            rows.append((dt, outs))
    n_prompt = sum(o.prompt_tokens for o in rows[0][1])
    n_out = sum(o.completion_tokens for o in rows[0][1])
    prefill = sum(max(o.prefill_s for o in outs) for _, outs in rows) / len(rows)
    total = sum(dt for dt, _ in rows) / len(rows)
    decode = max(total - prefill, 1e-9)
    rec = {"runs": len(rows), "prompt_tokens": n_prompt, "completion_tokens": n_out,
           "prefill_s": prefill, "decode_s": decode, "prefill_tok_s": n_prompt / max(prefill, 1e-9),
           "decode_tok_s": max(n_out - len(reqs), 0) / decode}
    if args.format == "json":
        print(json.dumps(rec))
    else:
        print(" ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in rec.items()))
    return 0


def cmd_random_model(args):
    from .weights import write_random_model
    cfg = json.loads(open(args.config_json).read())
    out = write_random_model(cfg, args.out, seed=args.seed, std=args.std,
                             norm_jitter=args.norm_jitter, dtype=args.dtype)
    print(out)
    return 0


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    ap = argparse.ArgumentParser(prog="lumenllm", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate")
    _engine_flags(g)
    _generate_flags(g)
    g.set_defaults(fn=cmd_generate)
    b = sub.add_parser("bench-generate")
    _engine_flags(b)
    _generate_flags(b)
    b.add_argument("--warmup", type=int, default=1)
    b.add_argument("--runs", type=int, default=3)
    b.set_defaults(fn=cmd_bench_generate)
    r = sub.add_parser("random-model")
    r.add_argument("--config-json", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-jitter", type=float, default=0.0)
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.set_defaults(fn=cmd_random_model)
    args = ap.parse_args(argv)
    from .config import ConfigError
    from .engine import GenerationError, StepError
    from .weights import WeightError
    try:
        return args.fn(args)
    except (ConfigError, WeightError, StepError, GenerationError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
