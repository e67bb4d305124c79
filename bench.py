#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of requests (default 8) whose contexts end at
the benchmark's context length (4096).  Prints ONE JSON line: decoded tokens per
second timed on the device with CUDA events (``value``), the same through the Python
entry point with host tokens in and out (``e2e``), the prefill of 2,048 tokens,
the decode step's share of the HBM roofline, decode at batch 1 and 64, the baseline's
stated run (prompts of 2,048 tokens, then 256 greedy tokens, at batch 1, 8 and 64) and
the verdict of a logit check against the plain implementation under ``tests/plain``.
The K steps are timed ``--repeats`` times in a row (default 5): ``ms_per_step`` is the
median region's, the smallest and largest stand beside it, and the clocks are sampled
over all of them.
``--impl reference`` runs skfine24/sLLM's own device-resident decode on the same sizes
(``baseline/reference_arm.py``) and prints the same keys.
``--workload serve-0.5b | serve-32b`` runs one of the baseline's serving workloads through
``LLM.generate`` instead and prints a record of its own (wall clock, prompt and generated
tokens a second).  ``--kernel-times`` adds the device time per kernel entry point of one
decode step and one prefill launched kernel by kernel.
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
    """nvidia-smi's clocks and throttle reasons, sampled every 50 ms while a timed
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
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
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


def decode_run(model, cfg, batch, context, steps, warmup, seed=0, graphs=True, repeats=1):
    """Prefill `batch` requests through the entry point, then time `steps` decode steps, `repeats`
    times in a row; the last region's contexts end at `context`.  The median region is the result."""
    import numpy as np
    import torch

    from sllm_b200 import ops
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    total_steps = warmup + repeats * steps
    prompt_len = context - total_steps
    page = PAGE_SIZE
    pages = batch * (-(-(context + 1) // page))
    # every request gets a portion in every step, so that all prompts end in the same step
    chunk = 512
    llm = LLM(model=model, block_size=page, num_pages=pages, max_num_seqs=batch, max_batch_tokens=batch * chunk,
              chunk_size=chunk, max_model_len=context + 1, policy="reserve", cuda_graphs=graphs,
              row_tile=0)                             # (no portion is shortened: the prompts are to end together)
    rng = np.random.default_rng(seed)
    for i in range(batch):
        llm.add_request(rng.integers(0, cfg["vocab_size"], prompt_len).tolist(),
                        SamplingParams(max_new=total_steps))
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
    walls = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            _, sampled = llm.step(device_timer=timer)
            assert len(sampled) == batch
        torch.cuda.synchronize()
        walls.append(time.perf_counter() - t0)
    # device time of each region of K consecutive steps (a step queued ahead of the last one read is
    # not among them)
    torch.cuda.synchronize()
    per = [a.elapsed_time(b) for a, b in timer.pairs]
    # (the last region may hold a pair fewer, its last step being the one queued ahead: a region's time is the mean of
    # the steps it holds times K, not the sum of however many there are)
    dev = [steps * statistics.mean(per[r * steps:(r + 1) * steps]) for r in range(repeats)]
    clk = clocks.stop()
    launches = {k: (ops.launches[k] - before[k]) // repeats for k in before}
    # bytes the step has to read: every weight once, and the live requests' cache (the median region's contexts)
    mid = sorted(range(repeats), key=lambda r: dev[r])[repeats // 2]
    ctx_mean = prompt_len + warmup + mid * steps + (steps - 1) / 2.0
    kv_bytes = llm.engine.cache.bytes_per_token(2 if model.dtype == torch.bfloat16 else 4) * ctx_mean * batch
    step_bytes = model.weight_bytes() + kv_bytes
    # per step: the packed batch description (one pinned buffer: ids, positions, slots, block tables, sampling
    # inputs) goes up, the sampled ids come down; counted from the tensors the engine copied
    # (per step the device ran: with a step queued ahead, the window may hold one launch more or less)
    ran = max(1, llm.engine.steps_run - launched)
    h2d = (copied_bytes()[0] - copied[0]) // ran
    d2h = (copied_bytes()[1] - copied[1]) // ran
    for r in list(llm.scheduler.running):
        llm.abort(r.req_id)
    llm.drain()
    del llm
    torch.cuda.empty_cache()
    dev_ms, wall = dev[mid], statistics.median(walls)
    return {"ms_per_step": dev_ms / steps, "tok_s": batch * steps / (dev_ms / 1e3),
            "ms_min": min(dev) / steps, "ms_max": max(dev) / steps,
            "e2e_tok_s": batch * steps / wall, "e2e_ms_per_step": wall * 1e3 / steps,
            "step_bytes": step_bytes, "clocks": clk, "launches": launches, "h2d": h2d, "d2h": d2h,
            "prompt_len": prompt_len}


def stated_run(model, cfg, batch, prompt_len=2048, new_tokens=256, seed=5):
    """The baseline's stated decode run: `batch` prompts of `prompt_len` uniform random ids, then
    `new_tokens` greedy tokens each, through the entry point.  Run twice (the first captures the graph
    and warms the kernels up); of the second, every decode step after the prompts is timed: on the device
    (CUDA events around each step's device part) and by wall clock.  Returns (device tok/s, wall tok/s)."""
    import numpy as np
    import torch

    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    context = prompt_len + new_tokens
    llm = LLM(model=model, block_size=PAGE_SIZE, num_pages=batch * (-(-(context + 1) // PAGE_SIZE)), max_num_seqs=batch,
              max_batch_tokens=max(batch * 512, prompt_len), chunk_size=512, max_model_len=context + 1, policy="reserve",
              row_tile=0)
    rng = np.random.default_rng(seed)
    out = None
    for rep in range(2):
        reqs = [llm.add_request(rng.integers(0, cfg["vocab_size"], prompt_len).tolist(), SamplingParams(max_new=new_tokens))
                for _ in range(batch)]
        while any(r.pending > 1 or r.num_computed == 0 for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        torch.cuda.synchronize()
        timer = DeviceTimer()
        steps = 0
        t0 = time.perf_counter()
        while any(r.status != "finished" for r in reqs):
            llm.step(device_timer=timer)
            steps += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        llm.drain()
        out = (batch * steps / (timer.total_ms(steps) / 1e3), batch * steps / wall, steps)
    del llm
    torch.cuda.empty_cache()
    return out


def prefill_run(model, cfg, tokens, reps=9, seed=1, warmup=3):
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


def logit_check(cfg, tokens=64, layers=2, seed=11):
    """Does the engine at these layer sizes give the plain implementation's logits?  A model folder of the
    benchmark's widths, `layers` deep, is written with seeded random weights; the plain implementation under
    tests/plain (numpy, whole sequence, no cache) reads it and computes the logits of one prompt of `tokens`
    ids; the engine runs the same prompt from the same folder in float32 and in bfloat16, most of it as one
    portion and the last 8 tokens one by one.  float32 must agree to 1e-4 (relative to the largest logit),
    bfloat16 to 2 % rms and 8 % at worst of the logits' spread, and the greedy token of the last position
    must be the same (the bounds the tests use at these widths).  The timed model itself has other (device-drawn)
    weights and all its layers; this checks the kernels chosen at its widths."""
    import numpy as np
    import torch

    from sllm_b200.engine import Engine, StepEntry, build_model
    from sllm_b200.weights import write_random_model
    from tests.plain import qwen2_plain as plain
    small = dict(cfg)
    small["num_hidden_layers"] = layers
    t0 = time.perf_counter()
    out = {"tokens": tokens, "layers": layers, "against": "tests/plain (numpy float32, whole sequence)"}
    with tempfile.TemporaryDirectory() as d:
        folder = write_random_model(os.path.join(d, "m"), small, seed, std=0.02, bias_std=0.2, gain_std=0.1)
        c, w = plain.load_model(folder)
        ids = np.random.default_rng(seed).integers(0, small["vocab_size"], tokens).tolist()
        want = plain.forward(ids, w, c)
        spread = float(want.std())
        ok = True
        for dtype in ("float32", "bfloat16"):
            model, _ = build_model(folder, dtype, "cuda:0")
            eng = Engine(model, page_size=PAGE_SIZE, num_pages=-(-tokens // PAGE_SIZE) + 1, max_requests=1)
            head = tokens - 8
            rows = [eng.step([StepEntry("r", ids[:head], list(range(head)))]).cpu().numpy()]
            for t in range(head, tokens):
                rows.append(eng.step([StepEntry("r", ids[t:t + 1], [0])]).cpu().numpy())
            got = np.concatenate(rows)
            eng.finish("r")
            err = np.abs(got - want)
            if dtype == "float32":
                out["float32_max_rel"] = float(err.max() / np.abs(want).max())
                good = out["float32_max_rel"] <= 1e-4
            else:
                out["bfloat16_rms_of_spread"] = round(float(np.sqrt((err ** 2).mean()) / spread), 5)
                out["bfloat16_max_of_spread"] = round(float(err.max() / spread), 4)
                good = out["bfloat16_rms_of_spread"] <= 0.02 and out["bfloat16_max_of_spread"] <= 0.08
            good = good and int(got[-1].argmax()) == int(want[-1].argmax())
            ok = ok and bool(good)
            del eng, model
            torch.cuda.empty_cache()
    out["ok"] = ok
    out["s"] = round(time.perf_counter() - t0, 1)
    return out


def kernel_times(model, cfg, batch, context):
    """Device milliseconds per kernel entry point for one decode step of `batch` requests at `context`
    and for one prefill of PREFILL_TOKENS, both launched kernel by kernel with events around every launch."""
    import numpy as np
    import torch

    from sllm_b200 import ops
    from sllm_b200.engine import Engine, StepEntry
    eng = Engine(model, page_size=PAGE_SIZE, num_pages=batch * (-(-(context + 1) // PAGE_SIZE)) + PREFILL_TOKENS // PAGE_SIZE + 1,
                 max_requests=batch + 1)
    rng = np.random.default_rng(3)
    for b in range(batch):
        ids = rng.integers(0, cfg["vocab_size"], context - 2).tolist()
        for i in range(0, len(ids), 2048):
            eng.step([StepEntry(b, ids[i:i + 2048], [])])
    out = {}
    for name, make in (("decode", lambda: [StepEntry(b, [1], [0]) for b in range(batch)]),
                       ("prefill", lambda: [StepEntry("p", rng.integers(0, cfg["vocab_size"], PREFILL_TOKENS).tolist(), [PREFILL_TOKENS - 1])])):
        if name == "decode":
            eng.step(make())                       # warm
        else:
            eng.step(make())
            eng.finish("p")
        torch.cuda.synchronize()
        with ops.KernelTimes() as kt:
            eng.step(make())
        out[name] = {k.replace("sllm_", ""): [n, round(ms, 4)] for k, (n, ms) in sorted(kt.table().items(), key=lambda kv: -kv[1][1])}
    return out


def graph_times(cfg, batch, context) -> dict:
    """Microseconds per launch of the kernels of one decode layer at `batch` tokens, each kind repeated in a CUDA
    graph of its own with its weights (or keys and values) cycled over copies larger than L2 together, so that
    every launch streams from HBM and runs behind a launch of its own kind, as it does inside a step.  Products
    in the forms the dispatch knows (`ws`: warp-split with the residual epilogue; `stream`: k-split partial sums;
    `tc`: tensor-memory streaming; `pair`: CTA pairs; `library`: torch.mm), decode attention with its merge at the
    number of ranges the engine picks and its neighbours."""
    import torch

    from sllm_b200 import ops
    dev = "cuda:0"
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(9):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3 / reps)
        return round(statistics.median(ts), 2)

    out = {}
    M = batch
    for name, N, K, silu in (("qkv", (nq + 2 * nkv) * hd, H, False), ("o_proj", H, nq * hd, False),
                             ("gate_up", 2 * I, H, True), ("down", H, I, False)):
        copies = max(3, -(-400_000_000 // (N * K * 2)))
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(M, K, device=dev).bfloat16()
        res = torch.zeros(M, N, device=dev)
        turn = [0]

        def w():
            turn[0] += 1
            return ws[turn[0] % copies]
        forms = {}
        if silu:
            forms["dispatch"] = lambda: ops.linear_silu_mul(x, w(), 8, torch.bfloat16)
            if M <= 32:
                forms["stream"] = lambda: ops.linear_stream(x, w(), None, torch.bfloat16, silu=True)
            if M <= 128:
                forms["tc"] = lambda: ops.linear_tc(x, w(), None, torch.bfloat16, silu=True)
            forms["pair"] = lambda: ops.gemm_pair(x, w(), None, torch.bfloat16, silu=True, wide=False)
        else:
            forms["dispatch"] = lambda: ops.linear(x, w(), None, torch.float32, allow_partials=True)
            if ops.ws_supports(M, N, K):
                forms["ws"] = lambda: ops.linear_ws(x, w(), None, torch.float32, residual=res)
            if M <= 32:
                forms["stream"] = lambda: ops.linear_stream(x, w(), None, torch.float32, splits=ops._stream_splits(N, K))
            if M <= 128:
                forms["tc"] = lambda: ops.linear_tc(x, w(), None, torch.float32, splits=ops._tc_splits(N, K))
            forms["library"] = lambda: torch.mm(x, w().t(), out_dtype=torch.float32)
            if M > 128:                           # a prompt portion: the CTA-pair product plain, with the residual epilogue, cut along K
                gain = torch.ones(N, device=dev)
                forms["pair"] = lambda: ops.gemm_pair(x, w(), None, torch.float32, wide=False)
                forms["pair_residual_and_next_norm"] = lambda: ops.gemm_pair(x, w(), None, torch.float32, residual=res, next_gain=gain)
                for cut in (2, 3, 5):
                    forms[f"pair_{cut}_slices"] = lambda cut=cut: ops.gemm_pair(x, w(), None, torch.float32, splits=cut)
                for cols in (256, 512, 448, 384, 320):      # the tile widths, plain and with the residual epilogue
                    wide = False if cols == 256 else True if cols == 512 else cols
                    forms[f"pair_{cols}_wide"] = lambda wide=wide: ops.gemm_pair(x, w(), None, torch.float32, wide=wide)
                    forms[f"pair_{cols}_wide_residual_and_next_norm"] = lambda wide=wide: ops.gemm_pair(
                        x, w(), None, torch.float32, wide=wide, residual=res, next_gain=gain)
        rec = {"bytes_alone_us": round(N * K * 2 / 1e6 / (load_peaks()[0]["hbm_gbs"] / 1e3), 2)}
        for form, fn in forms.items():
            try:
                rec[form] = timed(fn, reps=3 * copies)
            except Exception as e:      # noqa: BLE001  (a form that refuses these sizes says so in the record)
                rec[form] = f"{type(e).__name__}"
        if not silu:
            rec["slices_picked"] = ops.pair_splits(M, N, K) if M > 128 else 1
            if M > 128:
                rec["tile_form_picked"] = ops.pair_wide_cols(M, N)      # False: 256 wide, True: 512, else the width
        out[name] = rec
        del ws
        torch.cuda.empty_cache()
    if batch > 128:                               # (rows of a prompt portion: no decode attention of that many requests)
        ops.check_tcgen05_status()
        return out
    # decode attention over `context` keys a request, pages with consecutive ids
    ps = PAGE_SIZE
    per = -(-context // ps)
    copies = 3 if batch * context * nkv * hd * 4 < 1.2e9 else 2
    caches = []
    for _ in range(copies):
        kc = torch.randn(batch * per + 1, nkv, ps, hd, device=dev).bfloat16()
        caches.append((kc, torch.randn_like(kc)))
    bt = torch.arange(batch * per, device=dev, dtype=torch.int32).reshape(batch, per)
    q = torch.randn(batch, nq * hd, device=dev).bfloat16()
    q_start = torch.arange(batch + 1, device=dev, dtype=torch.int32)
    ctx_len = torch.full((batch,), context, device=dev, dtype=torch.int32)
    small, _ = ops.attention_tiles([1] * batch, nq // nkv, dev)
    picked = ops.choose_splits(batch, nkv, context, ops._tma_ctas_per_sm(hd))
    rec = {"bytes_alone_us": round(batch * context * nkv * hd * 4 / 1e6 / (load_peaks()[0]["hbm_gbs"] / 1e3), 2), "picked_ranges": picked}
    turn = [0]
    for s in sorted({max(1, picked - 1), picked, min(32, picked + 1)}):
        def attend(s=s):
            turn[0] += 1
            kc, vc = caches[turn[0] % copies]
            ops.attention_tma_decode(q, kc, vc, bt, q_start, ctx_len, small, s, nq, nkv, hd, hd ** -0.5, None)
        rec[f"ranges_{s}"] = timed(attend, reps=2 * copies)
    out["attention_and_merge"] = rec
    ops.check_tcgen05_status()
    return out


def reference_main(args) -> int:
    """The reference arm: the same metric, sizes, batch, context and number of steps through skfine24/sLLM's own
    device-resident decode (see baseline/reference_arm.py)."""
    from baseline import reference_arm
    cfg = dict(CONFIG_7B)
    cfg["num_hidden_layers"] = args.layers or FULL_LAYERS
    try:
        r = reference_arm.run(cfg, batch=args.batch, context=args.context, steps=args.steps, warmup=max(args.warmup, 3),
                              repeats=args.repeats, clock_sampler=ClockSampler())
    except reference_arm.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    except Exception as e:       # noqa: BLE001  (whatever the reference raised: the line says what)
        print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))
        return 0
    config = base_config(cfg, args, r["prompt_len"])
    config.update({"prompts": "one random prompt; its numpy prefill cache copied to every sequence",
                   "timing": "wall clock around the steps (the reference's step synchronises and mirrors the cache to the host inside)",
                   "host_weights": "one layer's tensors shared by all layers" if r["shared_layers"] else "every tensor drawn"})
    if r["shortened"]:
        config["prompt_shortened"] = "the numpy prefill of the full prompt does not fit this arm's time"
    out = {
        "impl": "reference",
        "metric": f"decode tok/s (Qwen2.5-7B sizes, bf16, batch {args.batch}, context {args.context})",
        "value": round(r["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(r["ms_per_step"], 3), "ms_per_step_min": round(r["ms_min"], 3), "ms_per_step_max": round(r["ms_max"], 3),
        "repeats": r["repeats"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "config": config,
        "e2e": {"value": round(r["tok_s"], 2), "unit": "tokens/s", "ms_per_step": round(r["ms_per_step"], 3),
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                "note": "the same measurement: the reference's public step is host to host"},
        "gpu_launches": r["launches_per_step"] * args.steps, "clocks": r["clocks"],
        "prefill": r["prefill"], "points": {"decode_b1": round(r["decode_b1"], 2)},
        "reference_self_check": r["agree"],
    }
    print(json.dumps(out))
    return 0


def base_config(cfg, args, prompt_len) -> dict:
    """The keys of `config` that both arms share (sizes, batch, context)."""
    return {
        "model": "Qwen2.5-7B sizes", "layers": cfg["num_hidden_layers"], "layers_full": FULL_LAYERS,
        "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
        "global_batch": args.batch, "seq_len": args.context, "prompt_len": prompt_len, "kv_dtype": "bf16",
        "parallelism": "1 GPU", "l2": "inputs larger than L2 (15 GB of weights read per step)",
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=("decode",) + tuple(SERVING), default="decode",
                    help="decode: the default run; serve-*: the baseline's serving workloads through LLM.generate")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--repeats", type=int, default=5, help="how many times the K steps are timed in a row (the median is reported)")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer than the configuration has, only where memory or time needs it")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64, the stated runs, the prefill and the logit check")
    ap.add_argument("--prefill-only", action="store_true", help="run the prefill alone (for profilers, and for portions of other sizes)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="tokens of the timed prompt portion (the record's is 2,048)")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    ap.add_argument("--kernel-times", action="store_true", help="add device time per kernel entry point (a step launched kernel by kernel)")
    ap.add_argument("--graph-times", action="store_true",
                    help="print microseconds per launch of one decode layer's kernels at --batch and --context, each kind in a graph of its own, and exit")
    args = ap.parse_args(argv)
    globals()["PAGE_SIZE"] = args.page_size
    globals()["PREFILL_TOKENS"] = max(2, args.prefill_tokens)
    args.repeats = max(1, args.repeats)

    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    if args.impl == "reference":
        return reference_main(args)
    if args.warmup < 3:
        args.warmup = 3
    while args.context - (args.warmup + args.repeats * args.steps) < 16 and args.repeats > 1:
        args.repeats -= 1

    import torch

    from sllm_b200.engine import build_random_model
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    if args.workload != "decode":
        print(json.dumps(serving_run(args.workload, args.layers)))
        return 0
    if args.graph_times:
        print(json.dumps({"graph_times_us": graph_times(CONFIG_7B, args.batch, args.context), "batch": args.batch,
                          "context": args.context, "page_size": PAGE_SIZE}))
        return 0
    args.layers = args.layers or FULL_LAYERS
    peaks, peaks_kind = load_peaks()
    cfg = dict(CONFIG_7B)
    cfg["num_hidden_layers"] = args.layers
    check = None
    if not args.no_points and not args.prefill_only:
        try:
            check = logit_check(cfg)
        except Exception as e:      # noqa: BLE001  (the record says that the check did not run, and why)
            check = {"ok": False, "error": f"{type(e).__name__}: {str(e)[:200]}"}
    model, _ = build_random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0", std=0.02)
    torch.cuda.synchronize()

    if args.prefill_only:
        ms = prefill_run(model, cfg, PREFILL_TOKENS, reps=2 if PREFILL_TOKENS == 2048 else 5)     # (few launches for a profiler)
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
    main_run = decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup, graphs=not args.no_graphs,
                          repeats=args.repeats)
    points = {}
    if not args.no_points:
        if PAGE_SIZE != 64:
            # the same run with pages of 64 tokens: the TMA-fed attention kernels issue one box per page
            globals()["PAGE_SIZE"] = 64
            r = decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup, graphs=not args.no_graphs,
                           repeats=min(3, args.repeats))
            points[f"decode_b{args.batch}_page64"] = round(r["tok_s"], 1)
            globals()["PAGE_SIZE"] = args.page_size
        for b in (1, 64):
            r = decode_run(model, cfg, b, args.context, args.steps, 3, seed=b, repeats=min(3, args.repeats))
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_e2e"] = round(r["e2e_tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        # between them, where the dispatch changes kernels (up to 16 tokens, up to 32, up to 128)
        for b in (16, 32, 128):
            r = decode_run(model, cfg, b, args.context, args.steps, 3, seed=b, repeats=min(3, args.repeats))
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        # long contexts, where the cache is most of what a step reads (the attention kernels are compared with their
        # float32 statement at these lengths in tests/test_long_context_gpu.py)
        for b, ctx in ((8, 16384), (1, 32768)):
            r = decode_run(model, cfg, b, ctx, args.steps, 3, seed=ctx, repeats=min(3, args.repeats))
            points[f"decode_b{b}_ctx{ctx}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_ctx{ctx}_hbm_frac"] = round(r["step_bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        # the baseline's stated run: prompts of 2,048 tokens, then 256 greedy tokens, every decode step timed
        for b in (1, 8, 64):
            dev, wall, n = stated_run(model, cfg, b)
            points[f"decode_b{b}_prompt2048_new256"] = round(dev, 1)
            points[f"decode_b{b}_prompt2048_new256_e2e"] = round(wall, 1)

    achieved = main_run["step_bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    config = base_config(cfg, args, main_run["prompt_len"])
    config.update({"page_size": PAGE_SIZE, "cuda_graphs": not args.no_graphs, "peaks": peaks_kind, "repeats": args.repeats,
                   "timed_contexts": f"{main_run['prompt_len'] + args.warmup}..{args.context}"})
    out = {
        "metric": f"decode tok/s (Qwen2.5-7B sizes, bf16, batch {args.batch}, context {args.context})",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "ms_per_step_min": round(main_run["ms_min"], 4), "ms_per_step_max": round(main_run["ms_max"], 4),
        "repeats": args.repeats, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": config,
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
    if check is not None:
        out["logit_check"] = check
    if args.kernel_times:
        out["kernel_times"] = kernel_times(model, cfg, args.batch, args.context)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
