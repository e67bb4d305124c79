"""Sampling over the logits a step returns.

Every row is sampled on the device, all rows at once (`ops.sample_rows`): greedy,
temperature, top-k and top-p as runtime/sampler.py:36-88 defines them, after the
repetition penalty (runtime/sampler.py:12-33) has changed the seen ids' logits in
place: from the engine's table of seen ids on the device (`ops.penalty_from_seen_`,
what `LLM` uses: it needs nothing from the host and is part of a captured decode
step), or from the lists of seen ids a caller of `Sampler.sample` hands over
(`ops.repetition_penalty_`).  Only the chosen ids cross to the host.  A sampled
token consumes one uniform from the request's own ``numpy.random.default_rng(seed)``
(runtime/sampler.py:86; serving/executor.py:358), so equal logits give the
reference's tokens.
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    """Picks one token per logits row on the device.  ``rows`` pairs each row with its
    request's parameters, generator and the ids seen so far (for the penalty)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._pin = self.device.type == "cuda"
        self.h2d_bytes = 0          # bytes of sampling inputs copied to the device so far (measurement)
        self.d2h_bytes = 0          # bytes of sampled ids copied back so far

    @staticmethod
    def host_inputs(rows):
        """(temperatures float32[R], uniforms float64[R], top_k int32[R], top_p float32[R]) as
        the sampling kernel takes them: temperature 0 is greedy, top_k 0 and top_p -1 filter
        nothing; a sampled (non-greedy) row draws its one uniform here."""
        n = len(rows)
        temps = np.zeros(n, dtype=np.float32)
        unis = np.zeros(n, dtype=np.float64)
        top_k = np.zeros(n, dtype=np.int32)
        top_p = np.full(n, -1.0, dtype=np.float32)
        for i, (p, rng, _) in enumerate(rows):
            t = float(p.temperature or 0.0)
            if t > 0:
                temps[i] = t
                unis[i] = rng.random()              # one uniform per sampled token
                if p.top_k is not None:
                    top_k[i] = min(int(p.top_k), 2 ** 31 - 1)
                if p.top_p is not None:
                    top_p[i] = max(float(p.top_p), 0.0)
        return temps, unis, top_k, top_p

    @staticmethod
    def penalties(params_list):
        """float32[R] repetition penalties (1 where a request has none), or None if no request has one."""
        if not any(p.penalised for p in params_list):
            return None
        return np.array([p.repetition_penalty if p.penalised else 1.0 for p in params_list], dtype=np.float32)

    @staticmethod
    def penalty_pairs(rows):
        """(row, id, penalty) arrays naming each seen id of each penalised row once, or None."""
        r, t, q = [], [], []
        for i, (p, _, seen) in enumerate(rows):
            if p.penalised and seen is not None and len(seen):
                ids = np.unique(np.asarray(list(seen), dtype=np.int64))
                r.append(np.full(ids.size, i, dtype=np.int32))
                t.append(ids.astype(np.int32))
                q.append(np.full(ids.size, p.repetition_penalty, dtype=np.float32))
        if not r:
            return None
        return np.concatenate(r), np.concatenate(t), np.concatenate(q)

    def _to_device(self, *arrays):
        out = []
        for a in arrays:
            h = torch.from_numpy(a)
            if self._pin:
                h = h.pin_memory()
            out.append(h.to(self.device, non_blocking=True))
            self.h2d_bytes += h.numel() * h.element_size()
        return out

    def sample(self, logits: torch.Tensor, rows, device_timer=None) -> list[int]:
        """rows: list of (SamplingParams, numpy Generator, seen ids or None).  The penalty
        changes ``logits`` in place."""
        R = logits.shape[0]
        if R != len(rows):
            raise ValueError(f"{R} logits rows for {len(rows)} requests")
        if R == 0:
            if device_timer is not None:
                device_timer.stop()
            return []
        pairs = self.penalty_pairs(rows)
        if pairs is not None:
            ops.repetition_penalty_(logits, *self._to_device(*pairs))
        temps, unis, top_k, top_p = self.host_inputs(rows)
        if not (temps > 0).any():
            picked = ops.sample_rows(logits)
        elif not top_k.any() and not (top_p >= 0).any():
            picked = ops.sample_rows(logits, *self._to_device(temps, unis))
        else:
            picked = ops.sample_rows(logits, *self._to_device(temps, unis, top_k, top_p))
        if device_timer is not None:
            device_timer.stop()
        self.d2h_bytes += picked.numel() * picked.element_size()
        return [int(t) for t in picked.cpu().tolist()]
