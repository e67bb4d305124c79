"""Sampling over the logits a step returns.

Greedy and temperature sampling run on the device for all rows at once
(`ops.sample_rows`); only the chosen ids cross to the host.  Rows that ask for
top-k, top-p or a repetition penalty are taken to the host and sampled in float64
exactly as the reference does (runtime/sampler.py:12-88).  Either way a sampled
token consumes one uniform from the request's own ``numpy.random.default_rng(seed)``
(runtime/sampler.py:86; serving/executor.py:358), so equal logits give the
reference's tokens.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


def apply_repetition_penalty(logits: np.ndarray, seen_ids, penalty) -> np.ndarray:
    """Seen ids: logit / penalty if positive, * penalty if negative; a copy; ids outside
    the vocabulary ignored (runtime/sampler.py:12-33)."""
    out = np.asarray(logits, dtype=np.float64).copy()
    if penalty is None or penalty <= 0 or penalty == 1.0 or seen_ids is None:
        return out
    ids = np.asarray(list(seen_ids), dtype=np.int64)
    ids = ids[(ids >= 0) & (ids < out.size)]
    if ids.size:
        vals = out[ids]
        out[ids] = np.where(vals < 0, vals * penalty, vals / penalty)
    return out


def sample_host(logits: np.ndarray, params: SamplingParams, rng: np.random.Generator) -> int:
    """The reference's sampler (runtime/sampler.py:36-88) on one row."""
    logits = np.asarray(logits, dtype=np.float64)
    if params.temperature is None or params.temperature <= 0:
        return int(np.argmax(logits))
    logits = logits / params.temperature
    probs = np.exp(logits - logits.max())
    probs = probs / probs.sum()
    if params.top_k is not None:
        k = min(int(params.top_k), probs.size)
        keep = np.argsort(probs)[-k:]
        mask = np.zeros(probs.shape, dtype=bool)
        mask[keep] = True
        probs = np.where(mask, probs, 0.0)
        s = probs.sum()
        if s > 0:
            probs = probs / s
    if params.top_p is not None:
        order = np.argsort(probs)[::-1]
        cutoff = int(np.searchsorted(np.cumsum(probs[order]), params.top_p) + 1)
        mask = np.zeros(probs.shape, dtype=bool)
        mask[order[:cutoff]] = True
        probs = np.where(mask, probs, 0.0)
    total = probs.sum()
    if total <= 0 or not np.isfinite(total):
        return int(np.argmax(logits))
    probs = probs / total
    idx = int(np.searchsorted(np.cumsum(probs), rng.random()))
    return min(idx, probs.size - 1)


class Sampler:
    """Picks one token per logits row.  ``rows`` pairs each row with its request's
    parameters, generator and the ids seen so far (for the penalty)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._pin = self.device.type == "cuda"

    @staticmethod
    def host_inputs(rows):
        """(temperatures float32[R], uniforms float64[R]) for rows that all sample on the
        device; a sampled (non-greedy) row draws its one uniform here."""
        temps = np.zeros(len(rows), dtype=np.float32)
        unis = np.zeros(len(rows), dtype=np.float64)
        for i, (p, rng, _) in enumerate(rows):
            t = float(p.temperature or 0.0)
            if t > 0:
                temps[i] = t
                unis[i] = rng.random()
        return temps, unis

    def sample(self, logits: torch.Tensor, rows, device_timer=None) -> list[int]:
        """rows: list of (SamplingParams, numpy Generator, seen ids or None)."""
        R = logits.shape[0]
        if R != len(rows):
            raise ValueError(f"{R} logits rows for {len(rows)} requests")
        if R == 0:
            if device_timer is not None:
                device_timer.stop()
            return []
        any_temp = any(p.temperature and p.temperature > 0 for p, _, _ in rows)
        host_rows = [i for i, (p, _, _) in enumerate(rows) if not p.on_device]
        temps = uni = None
        if any_temp:
            buf = torch.empty(R, dtype=torch.float32, pin_memory=self._pin)
            ubuf = torch.zeros(R, dtype=torch.float64, pin_memory=self._pin)
            for i, (p, rng, _) in enumerate(rows):
                t = float(p.temperature or 0.0)
                buf[i] = t if p.on_device else 0.0
                if p.on_device and t > 0:
                    ubuf[i] = rng.random()          # one uniform per sampled token
            temps = buf.to(self.device, non_blocking=True)
            uni = ubuf.to(self.device, non_blocking=True)
        picked = ops.sample_rows(logits, temps, uni)
        if device_timer is not None:
            device_timer.stop()
        ids = picked.cpu().tolist()
        for i in host_rows:
            p, rng, seen = rows[i]
            row = logits[i].float().cpu().numpy()
            row = apply_repetition_penalty(row, seen, p.repetition_penalty)
            ids[i] = sample_host(row, p, rng)
        return [int(t) for t in ids]
