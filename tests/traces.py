"""Traces for replay tests: the same requests cut into steps in different ways.

A trace is a list of step records in the replay program's input format, each with
an extra key ``expect`` (dropped before it is sent): the (request, position) of
every wanted logits row, in output order.  `max_tokens` of a trace is the peak,
over steps, of the live requests' token counts each rounded up to 64.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Trace:
    def __init__(self):
        self.steps = []
        self.held = {}          # live request -> tokens in the cache
        self.peak = 0

    def step(self, entries, end=()):
        """entries: list of (req, start, tokens, want)."""
        rec = {"step": len(self.steps), "entries": [], "end": list(end), "expect": []}
        for req, start, tokens, want in entries:
            assert self.held.get(req, 0) == start, "a request's tokens must be fed in order"
            rec["entries"].append({"id": req, "tokens": [int(t) for t in tokens], "want": [int(w) for w in want]})
            rec["expect"].extend((req, start + w) for w in want)
            self.held[req] = start + len(tokens)
        self.peak = max(self.peak, sum(-(-n // 64) * 64 for n in self.held.values()))
        for r in end:
            del self.held[r]
        self.steps.append(rec)

    @property
    def max_tokens(self):
        return self.peak

    def lines(self):
        return "".join(json.dumps({k: v for k, v in s.items() if k != "expect"}) + "\n" for s in self.steps)


def whole(reqs: dict, t: Trace | None = None) -> Trace:
    """Each request alone and whole in one step, every position wanted."""
    t = t or Trace()
    for r, ids in reqs.items():
        t.step([(r, 0, ids, range(len(ids)))], end=[r])
    return t


def tail_decode(reqs: dict, tail: int = 32, t: Trace | None = None) -> Trace:
    """Most of each request in one step, the last `tail` tokens one by one."""
    t = t or Trace()
    for r, ids in reqs.items():
        head = max(1, len(ids) - tail)
        t.step([(r, 0, ids[:head], [head - 1])])
        for p in range(head, len(ids)):
            t.step([(r, p, ids[p:p + 1], [0])], end=[r] if p == len(ids) - 1 else [])
        if head == len(ids):
            t.step([], end=[r])
    return t


def portions(reqs: dict, sizes=(7, 2, 13, 2, 5, 3, 2, 16, 2, 11), t: Trace | None = None) -> Trace:
    """One request at a time in portions of changing size, down to two tokens."""
    t = t or Trace()
    i = 0
    for r, ids in reqs.items():
        p = 0
        while p < len(ids):
            n = min(sizes[i % len(sizes)], len(ids) - p)
            i += 1
            last = p + n == len(ids)
            t.step([(r, p, ids[p:p + n], range(n))], end=[r] if last else [])
            p += n
    return t


def mixed(reqs: dict, live: int = 4, prompt_frac: float = 0.6, sizes=(9, 2, 17, 3, 2, 6),
          t: Trace | None = None) -> Trace:
    """Up to `live` requests at a time: the first part of each as prompt portions of
    changing size, the rest as single tokens, portions of some beside single tokens
    of others; a request that ends makes room (and pages) for the next."""
    t = t or Trace()
    waiting = list(reqs.items())
    running = []                 # [req, ids, pos, prompt_len]
    i = 0
    while waiting or running:
        while waiting and len(running) < live:
            r, ids = waiting.pop(0)
            running.append([r, ids, 0, max(1, int(len(ids) * prompt_frac))])
        entries, end = [], []
        for st in running:
            r, ids, pos, plen = st
            if pos < plen:
                n = min(sizes[i % len(sizes)], plen - pos)
                i += 1
                want = [n - 1] if pos + n == plen else ([0, n - 1] if n > 1 else [0])
            else:
                n, want = 1, [0]
            entries.append((r, pos, ids[pos:pos + n], want))
            st[2] = pos + n
            if st[2] == len(ids):
                end.append(r)
        # a request may sit a step out and go on later
        if len(entries) > 2 and len(t.steps) % 5 == 3 and entries[1][0] not in end and entries[1][1] > 0:
            skipped = entries.pop(1)
            for st in running:
                if st[0] == skipped[0]:
                    st[2] -= len(skipped[2])
        t.step(entries, end=end)
        running = [st for st in running if st[0] not in end]
    return t


def replay_subprocess(trace: Trace, model_dir: str, dtype: str, out_dir: str, page_size: int,
                      max_tokens: int | None = None, timeout: float = 600.0):
    """Run bin/trace_run as a user would; returns {step: array [wanted, vocab]}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens or trace.max_tokens), "--page-size", str(page_size)]
    r = subprocess.run(cmd, input=trace.lines(), capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"trace_run exited {r.returncode}:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [ln for ln in r.stdout.splitlines() if ln.startswith("done ")]
    assert [int(d.split()[1]) for d in done] == list(range(len(trace.steps)))
    return read_outputs(trace, out_dir)


def read_outputs(trace: Trace, out_dir: str):
    out = {}
    for s in trace.steps:
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if s["expect"]:
            a = np.fromfile(path, dtype="<f4")
            out[s["step"]] = a.reshape(len(s["expect"]), -1)
        else:
            assert not os.path.exists(path)
    return out


def replay_engine(trace: Trace, engine):
    """The same steps through an Engine in this process."""
    from sllm_b200.engine import StepEntry
    out = {}
    for s in trace.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                out[s["step"]] = logits.float().cpu().numpy()
        for r in s["end"]:
            engine.finish(r)
    return out


def compare(trace: Trace, outputs: dict, want: dict, rtol: float, atol: float, what: str = ""):
    """Every wanted row against the plain implementation's row; on a difference, say
    where the first wrong row lies."""
    worst = 0.0
    for s in trace.steps:
        if not s["expect"]:
            continue
        got = outputs[s["step"]]
        for row, (req, pos) in enumerate(s["expect"]):
            ref = want[req][pos]
            err = np.abs(got[row] - ref)
            tol = atol + rtol * np.abs(ref)
            if not (err <= tol).all():
                j = int(np.argmax(err - tol))
                raise AssertionError(
                    f"{what}: first wrong row at step {s['step']}, request {req!r}, position {pos} "
                    f"(entries {[(e['id'], len(e['tokens'])) for e in s['entries']]}): "
                    f"logit {j} is {got[row][j]:.6g}, plain gives {ref[j]:.6g}, |diff| {err[j]:.3g}")
            worst = max(worst, float((err / (atol + rtol * np.abs(ref))).max()))
    return worst


def all_modes(reqs: dict) -> Trace:
    """The four cuttings one after the other in one trace (request ids tagged by mode)."""
    t = Trace()
    whole({f"w.{r}": v for r, v in reqs.items()}, t=t)
    tail_decode({f"t.{r}": v for r, v in reqs.items()}, t=t)
    portions({f"p.{r}": v for r, v in reqs.items()}, t=t)
    mixed({f"m.{r}": v for r, v in reqs.items()}, t=t)
    return t


def tagged(want: dict) -> dict:
    return {f"{tag}.{r}": v for tag in "wtpm" for r, v in want.items()}
