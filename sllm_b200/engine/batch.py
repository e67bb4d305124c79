"""The description of one step's batch, packed into one int32 buffer.

A step is described to the kernels by a handful of int32 arrays: token ids, positions,
the request of each token, cumulative starts, context lengths, state slots, wanted rows
and, per cache group, where each new token is written and which pages each request reads.
They lie in ONE buffer so that one copy brings them to the device.  `BatchLayout` says
where each array lies; `pack` fills a host buffer from the cache manager's books;
`context` wraps a device copy of it as the `StepContext` the parts see.

Both ways of running a step use these three: a step launched kernel by kernel packs into a
fresh pinned buffer of exactly the step's sizes; a step replayed from a CUDA graph packs
into the graph's fixed buffer, with rows of padding beyond the live requests.  A field added
to `StepContext` is added here once.
"""

from __future__ import annotations

import numpy as np

from ..parts.base import GroupView, StepContext


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class BatchLayout:
    """Offsets of the arrays of a step with ``T`` tokens, ``S`` requests (rows), ``R`` wanted rows
    and ``pages[g]`` block-table columns in cache group g.  ``extras`` names further int32 sections
    (a caller's own: sampler inputs of a captured step) and their lengths in 32-bit words."""

    FIELDS = ("token_ids", "positions", "seq_of_token", "q_start", "ctx_len", "state_slots", "logit_rows")

    def __init__(self, T: int, S: int, R: int, pages, extras=None):
        self.T, self.S, self.R = int(T), int(S), int(R)
        self.pages = [int(p) for p in pages]
        sizes = {"token_ids": T, "positions": T, "seq_of_token": T, "q_start": S + 1, "ctx_len": S,
                 "state_slots": S, "logit_rows": R}
        for gi, mp in enumerate(self.pages):
            sizes[f"slot_mapping{gi}"] = T
            sizes[f"block_tables{gi}"] = S * mp
        for k, n in (extras or {}).items():
            if k in sizes:
                raise ValueError(f"section {k!r} is the layout's own")
            sizes[k] = int(n)
        self.sizes = sizes
        self.offs, total = {}, 0
        for k, n in sizes.items():
            self.offs[k] = total
            total += _pad4(max(n, 1))
        self.total = total

    def sec(self, buf, key):
        """The section ``key`` of ``buf`` (a numpy array or a torch tensor of `total` int32)."""
        o = self.offs[key]
        return buf[o:o + self.sizes[key]]


def pack(layout: BatchLayout, h: np.ndarray, cache, entries, totals, *, tokens_from_host: bool = True) -> None:
    """Write the step's description into the host buffer ``h`` (int32, `layout.total` long).

    ``entries`` bring ``req_id``, ``tokens`` and ``want``; ``totals[i]`` is the number of tokens
    request i holds after the step, so its tokens stand at positions ``totals[i] - n .. totals[i] - 1``.
    The requests' pages must be reserved already.  Rows of the layout beyond the entries are padding:
    one token each (id 0, position 0), no context, no page to write to (slot mapping -1), block table
    all -1, the cache's spare state slot; their logits are wanted like the others' so that the shapes
    stay those of the layout.  With ``tokens_from_host`` false the token ids are left for the caller
    to put there on the device.
    """
    n_live = len(entries)
    S, T = layout.S, layout.T
    ps = cache.page_size
    sec = layout.sec
    tok, pos, sot = sec(h, "token_ids"), sec(h, "positions"), sec(h, "seq_of_token")
    q_start, ctx_len, slots, rows = sec(h, "q_start"), sec(h, "ctx_len"), sec(h, "state_slots"), sec(h, "logit_rows")
    tables = [sec(h, f"block_tables{gi}").reshape(S, mp) if mp else None for gi, mp in enumerate(layout.pages)]
    maps = [sec(h, f"slot_mapping{gi}") for gi in range(len(layout.pages))]
    t0 = r0 = 0
    q_start[0] = 0
    for si, (e, tot) in enumerate(zip(entries, totals)):
        n = len(e.tokens)
        req = cache.requests[e.req_id]
        if n == 1:
            tok[t0] = e.tokens[0] if tokens_from_host else 0
            pos[t0] = tot - 1
        else:
            tok[t0:t0 + n] = np.asarray(e.tokens, dtype=np.int32) if tokens_from_host else 0
            pos[t0:t0 + n] = np.arange(tot - n, tot, dtype=np.int32)
        sot[t0:t0 + n] = si
        q_start[si + 1] = t0 + n
        ctx_len[si] = tot
        slots[si] = req.slot
        for w in e.want:
            rows[r0] = t0 + w
            r0 += 1
        for gi, bt in enumerate(tables):
            table = req.tables[gi]
            m = len(table)
            if bt is not None:
                bt[si, :m] = table
                bt[si, m:] = -1
            if n == 1:
                page = table[(tot - 1) // ps]
                if page < 0:
                    raise RuntimeError(f"request {e.req_id!r}: a token would be written to a page given back")
                maps[gi][t0] = page * ps + (tot - 1) % ps
            else:
                p = np.arange(tot - n, tot, dtype=np.int64)
                pages = np.asarray(table, dtype=np.int64)[p // ps]
                if (pages < 0).any():
                    raise RuntimeError(f"request {e.req_id!r}: a token would be written to a page given back")
                maps[gi][t0:t0 + n] = (pages * ps + p % ps).astype(np.int32)
        t0 += n
    pad = S - n_live
    if pad:
        if t0 + pad != T or r0 + pad != layout.R:
            raise ValueError("padding rows bring one token and one wanted row each; the layout does not fit")
        tok[t0:] = 0
        pos[t0:] = 0
        sot[t0:] = np.arange(n_live, S, dtype=np.int32)
        q_start[n_live + 1:] = np.arange(t0 + 1, T + 1, dtype=np.int32)
        ctx_len[n_live:] = 0
        slots[n_live:] = cache.padding_slot
        rows[r0:] = np.arange(t0, T, dtype=np.int32)
        for gi, bt in enumerate(tables):
            if bt is not None:
                bt[n_live:] = -1
            maps[gi][t0:] = -1
    elif t0 != T or r0 != layout.R:
        raise ValueError(f"the entries bring {t0} tokens and {r0} wanted rows, the layout holds {T} and {layout.R}")


def context(layout: BatchLayout, dev, page_size: int, q_lens, ctx_lens, **flags) -> StepContext:
    """The `StepContext` over ``dev``, the device copy of a packed buffer.  ``q_lens`` and ``ctx_lens``
    are the host's copies, which only launch shapes are taken from."""
    sec = layout.sec
    groups = [GroupView(page_size, sec(dev, f"block_tables{gi}").view(layout.S, mp), sec(dev, f"slot_mapping{gi}"))
              for gi, mp in enumerate(layout.pages)]
    return StepContext(
        num_tokens=layout.T, num_seqs=layout.S, token_ids=sec(dev, "token_ids"), positions=sec(dev, "positions"),
        seq_of_token=sec(dev, "seq_of_token"), q_start=sec(dev, "q_start"), ctx_len=sec(dev, "ctx_len"),
        state_slots=sec(dev, "state_slots"), logit_rows=sec(dev, "logit_rows"), groups=groups,
        q_lens=list(q_lens), ctx_lens=[int(c) for c in ctx_lens], max_q_len=max(q_lens), max_ctx_len=int(max(ctx_lens)),
        **flags)


def pages_missing(cache, entries, totals) -> list[int]:
    """Per cache group: the pages the step's requests need beyond those they hold, all together."""
    out = []
    for gi in range(len(cache.groups)):
        need = 0
        for e, tot in zip(entries, totals):
            req = cache.requests.get(e.req_id)
            need += max(0, cache.pages_for(tot) - (len(req.tables[gi]) if req else 0))
        out.append(need)
    return out
