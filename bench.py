#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of requests (default 8) whose contexts end at
the benchmark's context length (4096).  Prints ONE JSON line: decoded tokens per
second timed on the device with CUDA events (``value``), the same through the Python
entry point with host tokens in and out (``e2e``), the prefill of 2,048 tokens,
the decode step's share of the HBM roofline, and decode at batch 1 and 64.
``--workload serve-0.5b | serve-32b`` runs one of the baseline's serving workloads through
``LLM.generate`` instead and prints a record of its own (wall clock, prompt and generated
tokens a second).
Weights are random (drawn on the device), token ids uniform random: there is no
dataset.  The decode step reads every weight once (15 GB, far more than the 126 MB
L2), so successive steps cannot be served from cache.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the baseline's third configuration: Qwen2.5-7B sizes
CONFIG_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
    "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 32768, "tie_word_embeddings": False,
    "hidden_act": "silu",
}
FULL_LAYERS = 28
PAGE_SIZE = 16          # tokens per cache page as the baseline configuration states (--page-size); 64 is measured as a point
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi's clocks and throttle reasons, sampled every 200 ms while a timed
    region runs.  Reading only; no setting of the GPU is touched."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 8:
                        continue
                    try:
                        sm.append(float(parts[0]))
                        mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[4:8]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


class DeviceTimer:
    """Sums the device time of the parts of steps bracketed by start()/stop(), with CUDA
    events on the launching stream."""

    def __init__(self):
        import torch
        self.torch = torch
        self.pairs = []
        self._open = None

    def start(self):
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = ev

    def stop(self):
        if self._open is None:
            return
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record()
        self.pairs.append((self._open, ev))
        self._open = None

    def total_ms(self, first=None):
        """Device time of the first ``first`` bracketed parts (all by default)."""
        self.torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.pairs[:first])


def flops_of_step(cfg, tokens_per_req, ctx_before, logits_rows):
    """FLOPs of one step: 2 per multiply-add of every matrix product, and the causal
    attention's q.k and p.v products over the keys each query sees."""
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nq, nkv, hd, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    per_layer = (nq + 2 * nkv) * hd * H + nq * hd * H + 3 * I * H
    T = sum(tokens_per_req)
    fl = 2.0 * T * per_layer * L + 2.0 * logits_rows * V * H
    for n, c in zip(tokens_per_req, ctx_before):
        keys = n * c + n * (n + 1) / 2.0
        fl += 4.0 * keys * hd * nq * L
    return fl


def decode_run(model, cfg, batch, context, steps, warmup, seed=0, graphs=True):
    """Prefill `batch` requests through the entry point, then time `steps` decode steps."""
    import numpy as np
    import torch

    from sllm_b200 import ops
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    prompt_len = context - (steps + warmup)
    page = PAGE_SIZE
    pages = batch * (-(-(context + 1) // page))
    # every request gets a portion in every step, so that all prompts end in the same step
    chunk = 512
    llm = LLM(model=model, block_size=page, num_pages=pages, max_num_seqs=batch, max_batch_tokens=batch * chunk,
              chunk_size=chunk, max_model_len=context + 1, policy="reserve", cuda_graphs=graphs)
    rng = np.random.default_rng(seed)
    for i in range(batch):
        llm.add_request(rng.integers(0, cfg["vocab_size"], prompt_len).tolist(),
                        SamplingParams(max_new=steps + warmup))
    while any(r.pending > 1 or r.num_computed == 0 for r in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()                                    # prompts, in portions under the token budget
    for _ in range(warmup - 1):                       # the step that ended the prompts made token 1
        llm.step()
    torch.cuda.synchronize()
    timer = DeviceTimer()
    clocks = ClockSampler()
    clocks.start()
    before = dict(ops.launches)
    def copied_bytes():
        return (llm.engine.h2d_bytes + llm.sampler.h2d_bytes, llm.engine.d2h_bytes + llm.sampler.d2h_bytes)
    copied, launched = copied_bytes(), llm.engine.steps_run
    t0 = time.perf_counter()
    for _ in range(steps):
        _, sampled = llm.step(device_timer=timer)
        assert len(sampled) == batch
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    dev_ms = timer.total_ms(steps)        # a step queued ahead of the last one read is not among the K
    clk = clocks.stop()
    launches = {k: ops.launches[k] - before[k] for k in before}
    # bytes the step has to read: every weight once, and the live requests' cache
    ctx_mean = prompt_len + warmup + (steps - 1) / 2.0
    kv_bytes = llm.engine.cache.bytes_per_token(2 if model.dtype == torch.bfloat16 else 4) * ctx_mean * batch
    step_bytes = model.weight_bytes() + kv_bytes
    # per step: the packed batch description (one pinned buffer: ids, positions, slots, block tables, sampling
    # inputs) goes up, the sampled ids come down; counted from the tensors the engine copied
    # (per step the device ran: with a step queued ahead, the window may hold one launch more or less than `steps`)
    ran = max(1, llm.engine.steps_run - launched)
    h2d = (copied_bytes()[0] - copied[0]) // ran
    d2h = (copied_bytes()[1] - copied[1]) // ran
    for r in list(llm.scheduler.running):
        llm.abort(r.req_id)
    del llm
    torch.cuda.empty_cache()
    return {"ms_per_step": dev_ms / steps, "tok_s": batch * steps / (dev_ms / 1e3),
            "e2e_tok_s": batch * steps / wall, "e2e_ms_per_step": wall * 1e3 / steps,
            "step_bytes": step_bytes, "clocks": clk, "launches": launches, "h2d": h2d, "d2h": d2h,
            "prompt_len": prompt_len}


def prefill_run(model, cfg, tokens, reps=5, seed=1, warmup=3):
    import numpy as np
    import torch

    from sllm_b200.engine import Engine, StepEntry
    eng = Engine(model, page_size=PAGE_SIZE, num_pages=-(-tokens // PAGE_SIZE) + 1, max_requests=2)
    rng = np.random.default_rng(seed)
    times = []
    for i in range(reps + warmup):
        ids = rng.integers(0, cfg["vocab_size"], tokens).tolist()
        entries = [StepEntry(i, ids, [tokens - 1])]
        ctx = eng.prepare(entries)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.run(ctx, entries)
        b.record()
        torch.cuda.synchronize()
        eng.finish(i)
        if i >= warmup:
            times.append(a.elapsed_time(b))
    del eng
    torch.cuda.empty_cache()
    return statistics.median(times)


# The baseline's serving workloads (its fourth and fifth configurations): many requests of mixed length through
# the scheduler, prompt portions beside decoded tokens, timed by wall clock around `LLM.generate`.
SERVING = {
    "serve-0.5b": {
        "name": "Qwen2.5-Coder-0.5B sizes",
        "config": {"num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
                   "head_dim": 64, "intermediate_size": 4864, "vocab_size": 151936, "rms_norm_eps": 1e-6,
                   "tie_word_embeddings": True},
        "batch": 32, "prompt_lens": (128, 4096), "max_new": 128, "temperature": 0.7, "chunk": 512, "context": 8192,
    },
    "serve-32b": {
        "name": "Qwen2.5-32B sizes",
        "config": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
                   "head_dim": 128, "intermediate_size": 27648, "vocab_size": 152064, "rms_norm_eps": 1e-5,
                   "tie_word_embeddings": False},
        "batch": 16, "prompt_lens": (512, 6144), "max_new": 256, "temperature": 0.0, "chunk": 1024, "context": 8192,
    },
}


def serving_run(which: str, layers: int | None = None) -> dict:
    """One JSON record for a serving workload: the wall time of `LLM.generate` over the whole batch of
    requests (second of two runs: the first captures the decode graphs), host tokens in and out."""
    import numpy as np
    import torch

    from sllm_b200 import ops
    from sllm_b200.engine import build_random_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    w = SERVING[which]
    cfg = dict(CONFIG_7B)
    cfg.update(w["config"])
    full = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    model, _ = build_random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", std=0.02)
    rng = np.random.default_rng(0)
    lo, hi = w["prompt_lens"]
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(rng.integers(lo, hi + 1))).tolist() for _ in range(w["batch"])]
    llm = LLM(model=model, block_size=PAGE_SIZE, max_num_seqs=w["batch"], chunk_size=w["chunk"],
              max_batch_tokens=w["batch"] * w["chunk"], max_model_len=w["context"])     # the reference bounds a step's
    # tokens by requests x portion (runtime/scheduler.py:57-58): every running request may bring a portion
    runs = []
    for rep in range(2):
        params = [SamplingParams(max_new=w["max_new"], temperature=w["temperature"], seed=100 * rep + i)
                  for i in range(len(prompts))]
        sampler = ClockSampler()
        sampler.start()
        before = dict(ops.launches)
        steps0 = llm.steps
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = llm.generate(prompts, params)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        runs.append({"s": dt, "clocks": sampler.stop(), "steps": llm.steps - steps0,
                     "own": ops.launches["own"] - before["own"], "library": ops.launches["library"] - before["library"],
                     "out": sum(len(r.ids) for r in res)})
    ops.check_tcgen05_status()
    llm.engine.cache.check()
    n_in = sum(len(p) for p in prompts)
    r = runs[-1]
    return {
        "metric": f"tokens/s through LLM.generate ({w['name']}, bf16, {w['batch']} requests, prompts of "
                  f"{lo}..{hi} tokens, {w['max_new']} new tokens each, prompt portions of {w['chunk']} beside decoded tokens)",
        "value": round((n_in + r["out"]) / r["s"], 1), "unit": "tokens/s (prompt and generated)", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "wall_s": round(r["s"], 3), "first_run_s": round(runs[0]["s"], 3), "prompt_tokens": n_in, "generated_tokens": r["out"],
        "generated_tok_s": round(r["out"] / r["s"], 1), "steps": r["steps"],
        "config": {"model": w["name"], "layers": cfg["num_hidden_layers"], "layers_full": full, "hidden": cfg["hidden_size"],
                   "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": w["batch"],
                   "seq_len": w["context"], "chunk": w["chunk"], "step_token_budget": w["batch"] * w["chunk"], "temperature": w["temperature"], "page_size": PAGE_SIZE,
                   "kv_dtype": "bf16", "parallelism": "1 GPU"},
        "gpu_launches": r["own"], "library_launches": r["library"], "clocks": r["clocks"],
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=("decode",) + tuple(SERVING), default="decode",
                    help="decode: the default run; serve-*: the baseline's serving workloads through LLM.generate")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer than the configuration has, only where memory or time needs it")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64 and the prefill")
    ap.add_argument("--prefill-only", action="store_true", help="run the 2,048-token prefill alone (for profilers)")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    args = ap.parse_args(argv)
    globals()["PAGE_SIZE"] = args.page_size

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "skfine24/sLLM has no setup.py or pyproject.toml: pip cannot install it offline "
                          "(\"Neither 'setup.py' nor 'pyproject.toml' found\"), and its CUDA path is built for "
                          "sm_121 with one-token decode only"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from sllm_b200.engine import build_random_model
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    if args.workload != "decode":
        print(json.dumps(serving_run(args.workload, args.layers)))
        return 0
    args.layers = args.layers or FULL_LAYERS
    peaks, peaks_kind = load_peaks()
    cfg = dict(CONFIG_7B)
    cfg["num_hidden_layers"] = args.layers
    model, _ = build_random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", std=0.02)
    torch.cuda.synchronize()

    if args.prefill_only:
        ms = prefill_run(model, cfg, PREFILL_TOKENS, reps=2)
        fl = flops_of_step(cfg, [PREFILL_TOKENS], [0], 1)
        print(json.dumps({"prefill_only": True, "layers": args.layers, "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                          "tflops": round(fl / (ms / 1e3) / 1e12, 1)}))
        return 0
    # The prefill is timed first: after the decode runs the GPU sits at its power cap and the same
    # step takes about a tenth longer (26 against 23 ms); its own clocks are recorded beside it.
    prefill = None
    if not args.no_points:
        sampler = ClockSampler()
        sampler.start()
        ms = prefill_run(model, cfg, PREFILL_TOKENS)
        fl = flops_of_step(cfg, [PREFILL_TOKENS], [0], 1)
        prefill = {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                   "frac": round(fl / (ms / 1e3) / 1e12 / peaks["bf16_tflops"], 4),
                   "tflops": round(fl / (ms / 1e3) / 1e12, 1), "peak_tflops": peaks["bf16_tflops"],
                   # eight steps back to back run at the power cap: the fraction of the sustained library rate too
                   "frac_of_sustained": round(fl / (ms / 1e3) / 1e12 / peaks["bf16_tflops_sustained"], 4),
                   "peak_tflops_sustained": peaks["bf16_tflops_sustained"], "clocks": sampler.stop()}
    main_run = decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup, graphs=not args.no_graphs)
    points = {}
    if not args.no_points:
        if PAGE_SIZE != 64:
            # the same run with pages of 64 tokens: the TMA-fed attention kernels issue one box per page
            globals()["PAGE_SIZE"] = 64
            r = decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup, graphs=not args.no_graphs)
            points[f"decode_b{args.batch}_page64"] = round(r["tok_s"], 1)
            globals()["PAGE_SIZE"] = args.page_size
        for b in (1, 64):
            r = decode_run(model, cfg, b, args.context, max(8, args.steps // 2), 3, seed=b)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)

    achieved = main_run["step_bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": "decode tok/s (Qwen2.5-7B sizes, bf16, batch 8, context 4096)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {
            "model": "Qwen2.5-7B sizes", "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": args.context, "prompt_len": main_run["prompt_len"],
            "page_size": PAGE_SIZE, "kv_dtype": "bf16", "parallelism": "1 GPU", "cuda_graphs": not args.no_graphs,
            "l2": "inputs larger than L2 (15 GB of weights read per step)", "peaks": peaks_kind,
        },
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s",
                "ms_per_step": round(main_run["e2e_ms_per_step"], 4),
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"]["own"],
        "library_launches": main_run["launches"]["library"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
    }
    if prefill:
        out["prefill"] = prefill
    if points:
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
