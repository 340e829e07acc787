"""Command line: model folder in, generated token ids out.

The reference's programs take the model file as their only argument and compile every
other option in (test/main.cu:18-67: ``_use_f16``, ``_kv_data_type``, ``_n_output``,
``max_batches``, ``n_predict = 64``; example/load_model/load_model.cu:9-25).  The same
names are flags here, with the reference's values as defaults where it has them.

    python -m tffinfer_b200 MODEL_DIR --prompt-ids 1,2,3 --n-predict 64
    python -m tffinfer_b200 MODEL_DIR --prompt-len 128 --max-batches 8 --temperature 0.7 --seed 1
    python -m tffinfer_b200 --random-config cfg.json --random-seed 0 --save-model DIR   (writes a model folder)
    python -m tffinfer_b200 MODEL_DIR --load-only                                       (as example/load_model)
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tffinfer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="model folder (config.json + model.safetensors)")
    g = ap.add_argument_group("model options (ModelConfig of the reference)")
    g.add_argument("--use-f16", dest="use_f16", action="store_true", default=True,
                   help="16-bit serving kernels (bfloat16 here); the reference's _use_f16 (default on)")
    g.add_argument("--no-use-f16", dest="use_f16", action="store_false", help="true 32-bit path")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], help="same choice by name; overrides --use-f16")
    g.add_argument("--n-ctx", type=int, default=None, help="longest sequence (_n_ctx); default from config.json")
    g.add_argument("--n-predict", type=int, default=64, help="tokens to generate per prompt (n_predict)")
    g.add_argument("--max-batches", type=int, default=1, help="number of prompts with --prompt-len (max_batches)")
    s = ap.add_argument_group("sampling (SamplingConfig of the reference)")
    s.add_argument("--sample-type", default=None, choices=["greedy", "random", "top_k", "top_p"],
                   help="_type; default greedy, or random when a temperature is given")
    s.add_argument("--temperature", type=float, default=None, help="_temperature (0 = greedy)")
    s.add_argument("--top-k", type=int, default=0, help="_top_k (0 = off)")
    s.add_argument("--top-p", type=float, default=1.0, help="_top_p (1 = off)")
    s.add_argument("--min-p", type=float, default=0.0, help="_min_p (0 = off)")
    s.add_argument("--repetition-penalty", type=float, default=1.0, help="_repetition_penalty (1 = off)")
    s.add_argument("--seed", type=int, default=0, help="_seed")
    s.add_argument("--eos", type=int, action="append", default=[], help="token id that ends a request (repeatable)")
    p = ap.add_argument_group("prompts (token ids; the engine has no tokenizer)")
    p.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    p.add_argument("--prompt-file", help="file with one prompt a line, ids separated by spaces or commas")
    p.add_argument("--prompt-len", type=int, help="random prompts of this length (with --max-batches, --seed)")
    e = ap.add_argument_group("engine")
    e.add_argument("--page-size", type=int, default=16)
    e.add_argument("--max-cache-tokens", type=int, default=None)
    e.add_argument("--max-live", type=int, default=64)
    e.add_argument("--max-tokens-per-step", type=int, default=2048)
    e.add_argument("--no-cuda-graphs", action="store_true")
    e.add_argument("--log-level", default=None, choices=["error", "warning", "info", "debug"],
                   help="threshold of the log lines on stderr (default: TFFINFER_LOG, else warning)")
    e.add_argument("--kernel-trace", metavar="FILE",
                   help="time every kernel call of the run (CUDA graphs off) and write a Chrome trace to FILE; "
                        "the totals per kind of call go to stderr")
    r = ap.add_argument_group("random weights")
    r.add_argument("--random-config", help="config.json to make random weights for")
    r.add_argument("--random-seed", type=int, default=0)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    r.add_argument("--save-model", help="folder to write config.json and model.safetensors to")
    ap.add_argument("--load-only", action="store_true", help="load the model and exit (example/load_model)")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    return ap


def _parse_ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import tffinfer_b200 as tff
    from tffinfer_b200.config import EngineConfig
    from tffinfer_b200.sampling import SamplingParams

    if args.random_config:
        if not args.save_model:
            print("--random-config needs --save-model DIR", file=sys.stderr)
            return 2
        with open(args.random_config) as f:
            cj = json.load(f)
        arch = tff.get_architecture(cj["architectures"][0])
        cfg = arch.read_config(cj)
        tff.write_random_model(args.save_model, cfg, seed=args.random_seed, store_dtype=args.store_dtype)
        print(f"wrote {args.save_model} (seed {args.random_seed}, {args.store_dtype})")
        if not args.model:
            return 0
    if not args.model:
        print("a model folder is needed (or --random-config with --save-model)", file=sys.stderr)
        return 2

    if args.log_level:
        tff.log.set_level(args.log_level)
    dtype = args.dtype or ("bfloat16" if args.use_f16 else "float32")
    ecfg = EngineConfig(dtype=dtype, page_size=args.page_size, max_cache_tokens=args.max_cache_tokens,
                        max_live_requests=args.max_live, max_tokens_per_step=args.max_tokens_per_step,
                        max_model_len=args.n_ctx, use_cuda_graphs=not (args.no_cuda_graphs or args.kernel_trace),
                        seed=args.seed)
    t0 = time.time()
    engine = tff.Engine(args.model, ecfg)
    t_load = time.time() - t0
    if args.load_only:
        print(f"loaded {args.model} in {t_load:.2f} s")
        return 0

    prompts = [_parse_ids(t) for t in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_parse_ids(line) for line in f if line.strip()]
    if args.prompt_len:
        rng = random.Random(args.seed)
        vocab = engine.runner.desc.vocab_size
        prompts += [[rng.randrange(vocab) for _ in range(args.prompt_len)] for _ in range(args.max_batches)]
    if not prompts:
        print("no prompt given (--prompt-ids, --prompt-file or --prompt-len)", file=sys.stderr)
        return 2

    temperature = args.temperature if args.temperature is not None else (0.0 if args.sample_type in (None, "greedy") else 1.0)
    if args.sample_type == "greedy":
        temperature = 0.0
    sp = SamplingParams.make(temperature=temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                             repetition_penalty=args.repetition_penalty, seed=args.seed,
                             max_new_tokens=args.n_predict, eos_token_ids=tuple(args.eos))
    t0 = time.time()
    if args.kernel_trace:
        from tffinfer_b200.kernels.trace import KernelTrace
        with KernelTrace(engine.runner.ops) as trace:
            reqs = engine.generate(prompts, sp, return_requests=True)
        trace.write_chrome_trace(args.kernel_trace)
        for name, calls, ms in trace.summary():
            print(f"  {name:28s} {calls:7d} calls {ms:10.3f} ms", file=sys.stderr)
    else:
        reqs = engine.generate(prompts, sp, return_requests=True)
    dt = time.time() - t0
    n_new = sum(len(r.generated) for r in reqs)
    if args.json:
        print(json.dumps({"outputs": [r.generated for r in reqs], "finish_reasons": [r.finish_reason for r in reqs],
                          "seconds": dt, "generated_tokens": n_new, "stats": engine.stats()}))
    else:
        for i, r in enumerate(reqs):
            print(f"[{i}] prompt {len(r.prompt)} tokens -> {len(r.generated)} tokens ({r.finish_reason}): "
                  + " ".join(str(t) for t in r.generated))
        print(f"{n_new} token decode time: {dt:.3f} s ({n_new / dt:.1f} tok/s); load {t_load:.2f} s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
