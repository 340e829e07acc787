#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second at the Qwen3-8B shape
(random bfloat16 weights, batch 8, 2048-token prompts, 16-token cache pages), with the
prefill rate of one 2048-token prompt, decode at batch 1 and 64, the same decode
measured end to end through the Python entry point, and roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline configuration: the Qwen3-8B shape
SHAPE = dict(num_layers=36, hidden_size=4096, num_heads=32, num_kv_heads=8, head_dim=128,
             intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, max_position=40960)
CONTEXT = 4096
PROMPT_LEN = 2048
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    out = dict(FALLBACK_PEAKS)
    out["source"] = "fallback"
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.samples.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_engine(layers: int, max_live: int, cache_tokens: int, seed: int = 0, graphs: bool = True,
                context: int = CONTEXT, step_tokens: int = PROMPT_LEN):
    import torch
    import tffinfer_b200 as tff
    from tffinfer_b200.config import Qwen3Config
    from tffinfer_b200.weights import random_tensors_on_device
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", tie_word_embeddings=False,
                      layer_types=("full_attention",) * layers, **{**SHAPE, "num_layers": layers}).validate()
    tensors = random_tensors_on_device(cfg, seed, "cuda", "bfloat16")
    ecfg = tff.EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=cache_tokens,
                            max_live_requests=max_live, max_tokens_per_step=step_tokens, max_model_len=context,
                            use_cuda_graphs=graphs)
    runner = tff.ModelRunner(config=cfg, tensors=tensors, engine_config=ecfg)
    del tensors
    torch.cuda.empty_cache()
    return tff.Engine(runner=runner), cfg


def model_bytes(cfg) -> dict:
    H, L, I, V = cfg.hidden_size, cfg.num_layers, cfg.intermediate_size, cfg.vocab_size
    qw, kvw = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    per_layer = (qw + 2 * kvw) * H + H * qw + 3 * I * H
    return {"layer_params": per_layer, "weights_read_per_step": 2 * (per_layer * L + V * H),
            "kv_bytes_per_token": 2 * L * cfg.num_kv_heads * cfg.head_dim * 2}


def decode_run(engine, batch: int, steps: int, warmup: int, seed: int, sampler=None, prompt_len: int = PROMPT_LEN):
    """Prefills ``batch`` prompts of ``prompt_len`` tokens, then times ``steps`` decode steps
    after ``warmup`` untimed ones.  Returns device-timed and wall-clock figures."""
    import torch
    from tffinfer_b200 import SamplingParams
    rng = random.Random(seed)
    vocab = engine.runner.desc.vocab_size
    # earlier requests decode while later ones prefill, a step's token budget at a time
    budget = max(1, engine.runner.ecfg.max_tokens_per_step)
    sp = SamplingParams(max_new_tokens=warmup + steps + 8 + batch * -(-prompt_len // budget))
    ids = [engine.add_request([rng.randrange(vocab) for _ in range(prompt_len)], sp,
                              request_id=f"b{batch}_{prompt_len}_{i}", key=i)
           for i in range(batch)]
    # prefill: until every request has produced its first token
    while any(len(engine.requests[i].generated) == 0 for i in ids):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    ops = engine.runner.ops
    launches0 = ops.launches
    ctx0 = sum(len(engine.requests[i]) for i in ids) / batch
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    engine.step_events = None
    if sampler is not None:
        sampler.start()
    t0 = time.perf_counter()
    for k in range(steps):
        engine.step_events = ev[k]
        outs = engine.step()
        assert len(outs) == batch
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if sampler is not None:
        sampler.stop()
    engine.step_events = None
    per_step = sorted(a.elapsed_time(b) for a, b in ev)
    dev_ms = sum(per_step)
    ctx1 = sum(len(engine.requests[i]) for i in ids) / batch
    launches = ops.launches - launches0
    ops.check_errors()
    h2d = engine.runner.last_h2d_bytes
    for i in ids:                                   # stop the requests and give their pages back
        engine.abort(i)
    return {"tok_s": batch * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps,
            "e2e_tok_s": batch * steps / wall, "launches": launches, "mean_context": (ctx0 + ctx1) / 2,
            "h2d_bytes": h2d, "d2h_bytes": 4 * batch + 4,      # drawn tokens and the kernels' error word
            "p50_ms": per_step[len(per_step) // 2], "p99_ms": per_step[min(len(per_step) - 1, int(0.99 * len(per_step)))],
            "max_ms": per_step[-1]}


def prefill_run(engine, iters: int, warmup: int, seed: int, prompt_len: int = PROMPT_LEN):
    import torch
    from tffinfer_b200 import StepEntry
    rng = random.Random(seed)
    vocab = engine.runner.desc.vocab_size
    runner = engine.runner
    times = []
    for it in range(warmup + iters):
        toks = [rng.randrange(vocab) for _ in range(prompt_len)]
        rid = f"prefill{prompt_len}_{it}"
        runner.add_request(rid)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        batch = runner.make_batch([StepEntry(rid, toks, [prompt_len - 1])])
        torch.cuda.synchronize()
        a.record()
        logits = runner.run_batch(batch)
        b.record()
        torch.cuda.synchronize()
        runner.cache.commit(rid, prompt_len)
        runner.finish_request(rid)
        if it >= warmup:
            times.append(a.elapsed_time(b))
        assert logits.shape[0] == 1
    runner.ops.check_errors()
    return statistics.median(times)


# whole-workload runs through the scheduler (a 14B shape with mixed prompts, a 32B shape with long prompts)
WORKLOADS = {
    "mixed14b": dict(shape=dict(num_layers=40, hidden_size=5120, num_heads=40, num_kv_heads=8, head_dim=128,
                                intermediate_size=17408, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                max_position=40960),
                     requests=32, prompt_lens=(128, 4096), new_tokens=128, chunk=512, context=4352),
    "long32b": dict(shape=dict(num_layers=64, hidden_size=5120, num_heads=64, num_kv_heads=8, head_dim=128,
                               intermediate_size=25600, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                               max_position=40960),
                    requests=16, prompt_lens=(8192, 8192), new_tokens=256, chunk=2048, context=8448),
    # many short requests: 512 prompts of 64 to 512 tokens, 64 new tokens each, at most 256 live at a time
    "chat8b": dict(shape=dict(SHAPE), requests=512, prompt_lens=(64, 512), new_tokens=64, chunk=2048, context=1024, live=256),
    # the headline shape in true 32-bit (FFMA products, float32 attention and cache) on short prompts
    "fp32_short": dict(shape=dict(SHAPE), requests=4, prompt_lens=(64, 192), new_tokens=16, chunk=256, context=512,
                       dtype="float32"),
}


def run_workload(name: str, layers: int = 0) -> int:
    """Runs a whole workload (prompts prefilled in portions while others decode) and prints its totals."""
    import torch
    import tffinfer_b200 as tff
    from tffinfer_b200.config import Qwen3Config
    from tffinfer_b200.weights import random_tensors_on_device
    w = WORKLOADS[name]
    shape = dict(w["shape"])
    if layers:
        shape["num_layers"] = layers
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", tie_word_embeddings=False,
                      layer_types=("full_attention",) * shape["num_layers"], **shape).validate()
    rng = random.Random(0)
    lens = [rng.randint(*w["prompt_lens"]) for _ in range(w["requests"])]
    live = w.get("live", w["requests"])
    cache_tokens = sum(sorted((-(-(n + w["new_tokens"] + 1) // PAGE_SIZE) * PAGE_SIZE for n in lens), reverse=True)[:live])
    dtype = w.get("dtype", "bfloat16")
    ecfg = tff.EngineConfig(dtype=dtype, page_size=PAGE_SIZE, max_cache_tokens=cache_tokens,
                            max_live_requests=live, max_tokens_per_step=w["chunk"], max_model_len=w["context"])
    tensors = random_tensors_on_device(cfg, 0, "cuda", dtype)
    engine = tff.Engine(runner=tff.ModelRunner(config=cfg, tensors=tensors, engine_config=ecfg))
    del tensors
    torch.cuda.empty_cache()
    sp = tff.SamplingParams(max_new_tokens=w["new_tokens"])
    warm = engine.generate([[1, 2, 3, 4]], tff.SamplingParams(max_new_tokens=4))       # builds kernels, first graphs
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ids = [engine.add_request(p, sp, key=i) for i, p in enumerate(prompts)]
    steps = 0
    first_token_at = {}
    step_s = []
    while engine.has_unfinished():
        t_step = time.perf_counter()
        for o in engine.step():
            if o.token is not None and o.request_id not in first_token_at:
                first_token_at[o.request_id] = time.perf_counter() - t0
        step_s.append(time.perf_counter() - t_step)       # host time of a step: with steps launched ahead, the
        steps += 1                                        # device time of the step before
    step_s.sort()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    engine.runner.ops.check_errors()
    gen = sum(len(engine.requests[i].generated) for i in ids)
    st = engine.stats()
    print(json.dumps({"workload": name, "layers": cfg.num_layers, "requests": len(ids), "prompt_tokens": sum(lens),
                      "generated_tokens": gen, "seconds": round(dt, 3), "steps": steps,
                      "total_tok_s": round((sum(lens) + gen) / dt, 1), "generated_tok_s": round(gen / dt, 1),
                      "step_ms_p50": round(1e3 * step_s[len(step_s) // 2], 3),
                      "step_ms_p99": round(1e3 * step_s[min(len(step_s) - 1, int(0.99 * len(step_s)))], 3),
                      "mean_time_to_first_token_s": round(sum(first_token_at.values()) / max(1, len(first_token_at)), 3),
                      "pages_high_water": st["pages_high_water"], "pages_total": st["pages_total"],
                      "preemptions": st["preemptions"], "dtype": "bf16" if dtype == "bfloat16" else "fp32",
                      "data": "synthetic"}))
    return 0


# decode and prefill of the headline shape at other batch sizes and context lengths than the headline's
SWEEP_DECODE = [(1, 512), (1, 8192), (1, 32768), (8, 512), (8, 8192), (8, 32768), (64, 512), (64, 8192), (256, 1024)]
SWEEP_PREFILL = [512, 1024, 4096, 8192]


def prefill_flops(cfg, mb, T: int) -> float:
    """Products of the layers for T tokens, the causal half of the attention's two products, the output matrix
    for the one wanted row."""
    return (2 * T * mb["layer_params"] * cfg.num_layers
            + 2 * T * T * cfg.head_dim * cfg.num_heads * cfg.num_layers + 2 * cfg.vocab_size * cfg.hidden_size)


def run_sweep(layers: int, steps: int, warmup: int) -> int:
    """One JSON line a point: decode steps (bytes that must be read / time / measured copy rate) and whole-prompt
    prefill steps (flops / time / measured product rate) of the Qwen3-8B shape at further sizes."""
    import torch
    peaks = load_peaks()
    steps = min(steps, 24)
    need = max(b * (n + warmup + steps + 72 + b * -(-n // max(SWEEP_PREFILL))) for b, n in SWEEP_DECODE)
    engine, cfg = make_engine(layers, max(b for b, _ in SWEEP_DECODE), need, context=SHAPE["max_position"],
                              step_tokens=max(SWEEP_PREFILL + [PROMPT_LEN]))
    mb = model_bytes(cfg)
    for b, n in SWEEP_DECODE:
        run = decode_run(engine, b, steps, warmup, seed=10 + b, prompt_len=n)
        byts = mb["weights_read_per_step"] + b * run["mean_context"] * mb["kv_bytes_per_token"]
        print(json.dumps({"point": "decode", "batch": b, "context": round(run["mean_context"]), "layers": cfg.num_layers,
                          "tok_s": round(run["tok_s"], 1), "ms_per_step": round(run["ms_per_step"], 4),
                          "p99_ms": round(run["p99_ms"], 4), "gbytes_per_step": round(byts / 1e9, 2),
                          "hbm_frac": round(byts / (run["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4),
                          "peaks": peaks["source"]}), flush=True)
    for T in SWEEP_PREFILL:
        pms = prefill_run(engine, iters=3, warmup=2, seed=T, prompt_len=T)
        fl = prefill_flops(cfg, mb, T)
        print(json.dumps({"point": "prefill", "tokens": T, "layers": cfg.num_layers, "ms": round(pms, 3),
                          "tok_s": round(T / (pms / 1e3), 1), "tflops": round(fl / (pms / 1e3) / 1e12, 1),
                          "frac": round(fl / (pms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                          "frac_sustained": round(fl / (pms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12), 4),
                          "peaks": peaks["source"]}), flush=True)
    torch.cuda.synchronize()
    return 0


# layer sizes of other models of the family (layers, hidden, query heads, feed-forward; 8 key/value heads of 128 all)
OTHER_SHAPES = {"0.6B": (28, 1024, 16, 3072), "1.7B": (28, 2048, 16, 6144), "4B": (36, 2560, 32, 9728),
                "14B": (40, 5120, 40, 17408), "32B": (64, 5120, 64, 25600)}


def run_shapes(steps: int, warmup: int) -> int:
    """Decode at batch 1 and 8 (2048-token prompts) and a 2048-token prefill at the layer sizes of the other
    models of the family, one JSON line a shape: small models are bound by the latency of a layer's chain of
    kernels, large ones by their bytes."""
    import torch
    peaks = load_peaks()
    steps = min(steps, 24)
    for name, (layers, hidden, heads, inter) in OTHER_SHAPES.items():
        SHAPE.update(num_layers=layers, hidden_size=hidden, num_heads=heads, intermediate_size=inter)
        engine, cfg = make_engine(layers, 8, 8 * (PROMPT_LEN + warmup + steps + 96))
        mb = model_bytes(cfg)
        line = {"point": "shape", "model": f"Qwen3-{name} shape", "layers": layers, "hidden": hidden, "heads": heads,
                "intermediate": inter, "peaks": peaks["source"]}
        for b in (1, 8):
            run = decode_run(engine, b, steps, warmup, seed=b)
            byts = mb["weights_read_per_step"] + b * run["mean_context"] * mb["kv_bytes_per_token"]
            line[f"decode_b{b}"] = {"tok_s": round(run["tok_s"], 1), "ms_per_step": round(run["ms_per_step"], 4),
                                    "hbm_frac": round(byts / (run["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
        pms = prefill_run(engine, iters=3, warmup=2, seed=4)
        fl = prefill_flops(cfg, mb, PROMPT_LEN)
        line["prefill"] = {"tokens": PROMPT_LEN, "ms": round(pms, 3), "tok_s": round(PROMPT_LEN / (pms / 1e3), 1),
                           "frac": round(fl / (pms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        print(json.dumps(line), flush=True)
        del engine
        torch.cuda.empty_cache()
    return 0


ATTN_DECODE_POINTS = [(1, 529), (1, 8209), (1, 32785), (8, 529), (8, 2069), (8, 8213), (64, 531), (64, 2069), (256, 1057)]


def run_attn_decode(iters: int = 50) -> int:
    """The decode attention of the headline shape alone (one layer's cache, scattered pages, one new token a request):
    one JSON line a point with the time of a call (its kernel and the merge of the key shares), L2 flushed between
    calls, against the bytes of keys and values at the measured copy rate."""
    import math
    import numpy as np
    import torch
    from tffinfer_b200.engine.batch import StepBatch
    from tffinfer_b200.kernels.library import CudaKernels
    ops = CudaKernels()
    peaks = load_peaks()
    nq, nkv, d, page = SHAPE["num_heads"], SHAPE["num_kv_heads"], SHAPE["head_dim"], PAGE_SIZE
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for B, ctx in ATTN_DECODE_POINTS:
        rng = random.Random(B * 100003 + ctx)
        blocks = -(-(ctx + 1) // page)
        ids = list(range(B * blocks + 5))
        rng.shuffle(ids)
        table = torch.tensor([ids[i * blocks:(i + 1) * blocks] for i in range(B)], dtype=torch.int32, device=dev)
        cache = torch.randn((len(ids), 1, 2, nkv, page, d), device=dev, dtype=torch.bfloat16)
        q = torch.randn((B, nq * d), device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        full = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        ones = np.ones(B, dtype=np.int32)
        batch = StepBatch(num_tokens=B, num_requests=B, num_logit_rows=B, max_q_len=1, max_kv_len=ctx + 1,
                          token_ids=torch.zeros(B, dtype=torch.int32, device=dev), positions=full, tok_req=ar[:B],
                          q_start=ar, pos_start=full, kv_len=full + 1, slots=ar[:B], logit_rows=ar[:B], req_order=ar[:B],
                          block_tables=[table], h_q_lens=ones, h_pos_start=ones * ctx, h_sorted_q_lens=ones,
                          h_sorted_kv_lens=ones * (ctx + 1), all_decode=True, real_requests=B, real_logit_rows=B)
        byts = B * (ctx + 1) * 2 * nkv * d * 2

        def call():
            ops.attention_bf16(q, batch, table, cache, 0, page, out, nq, nkv, d, 1 / math.sqrt(d), 0)
        for _ in range(3):
            call()
        times = []
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            call()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        ops.check_errors()
        us = statistics.median(times)
        print(json.dumps({"point": "attn_decode", "requests": B, "context": ctx, "mbytes": round(byts / 1e6, 1),
                          "us": round(us, 1), "us_at_copy_rate": round(byts / peaks["hbm_gbs"] / 1e3, 1),
                          "key_shares": ops.attention_splits(B, 1, nq, nkv), "peaks": peaks["source"]}), flush=True)
        del cache
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="headline", choices=["headline", "sweep", "attn_decode", "shapes"] + sorted(WORKLOADS),
                    help="headline: the decode/prefill benchmark; sweep: the same shape at further batch sizes and "
                         "context lengths; attn_decode: the decode attention alone; shapes: the layer sizes of the other "
                         "models of the family; else a whole workload through "
                         "the scheduler")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE["num_layers"],
                    help="fewer layers than the shape has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (no batch 1 / 64, no prefill)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profilers)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "NKKdev/TFFinfer is a CMake C++/CUDA project without Python packaging whose dependencies "
                          "(glog, Taskflow, libdivide) are fetched from the network; it loads GGUF Q8_0 files only and "
                          "has no sm_100 build: it cannot be installed offline here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    if args.workload == "sweep":
        return run_sweep(args.layers, args.steps, warmup)
    if args.workload == "attn_decode":
        return run_attn_decode()
    if args.workload == "shapes":
        return run_shapes(args.steps, warmup)
    if args.workload != "headline":
        return run_workload(args.workload, 0 if args.layers == SHAPE["num_layers"] else args.layers)

    import torch
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device", file=sys.stderr)
        return 1
    peaks = load_peaks()
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    tokens_needed = max_batch * (PROMPT_LEN + warmup + args.steps + max_batch + 64)
    engine, cfg = make_engine(args.layers, max_batch, tokens_needed, graphs=not args.no_graphs)
    mb = model_bytes(cfg)

    clocks = ClockSampler()
    main_run = decode_run(engine, args.batch, args.steps, warmup, seed=1, sampler=clocks)
    points = {}
    points_roofline = {}
    prefill = None

    def hbm_fraction(run, batch):
        """bytes the step has to read (every weight once, the cache of the live requests) / its time / the peak"""
        b = mb["weights_read_per_step"] + batch * run["mean_context"] * mb["kv_bytes_per_token"]
        return b / (run["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]

    if not args.skip_points:
        small_steps = min(args.steps, 32)
        for name, b, seed in (("decode_b1", 1, 2), ("decode_b64", 64, 3)):
            run = decode_run(engine, b, small_steps, warmup, seed=seed)
            points[name] = round(run["tok_s"], 1)
            points_roofline[name] = {"ms_per_step": round(run["ms_per_step"], 4), "hbm_frac": round(hbm_fraction(run, b), 4),
                                     "p50_ms": round(run["p50_ms"], 4), "p99_ms": round(run["p99_ms"], 4)}
        pms = prefill_run(engine, iters=5, warmup=3, seed=4)
        T = PROMPT_LEN
        flops = prefill_flops(cfg, mb, T)
        prefill = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(flops / (pms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                   "tflops": round(flops / (pms / 1e3) / 1e12, 1)}

    step_s = main_run["ms_per_step"] / 1e3
    bytes_step = mb["weights_read_per_step"] + args.batch * main_run["mean_context"] * mb["kv_bytes_per_token"]
    achieved = bytes_step / step_s / 1e9
    out = {
        "metric": "decode tok/s (Qwen3-8B shape, bf16, batch 8, 2048-token prompts)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random N(0,0.02) weights)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": cfg.num_layers, "layers_of_shape": SHAPE["num_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE_SIZE,
                   "parallelism": "1 GPU", "l2": "inputs larger than L2 (15 GB of weights read per step)",
                   "cuda_graphs": not args.no_graphs},
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": main_run["h2d_bytes"], "d2h_bytes_per_step": main_run["d2h_bytes"]},
        "gpu_launches": main_run["launches"],
        "latency_ms": {"p50": round(main_run["p50_ms"], 4), "p99": round(main_run["p99_ms"], 4),
                       "max": round(main_run["max_ms"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "clocks": clocks.summary(),
    }
    if prefill is not None:
        out["prefill"] = prefill
        out["points"] = points
        out["points_roofline"] = points_roofline
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
