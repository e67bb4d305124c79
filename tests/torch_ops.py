"""Plain PyTorch float32 statements of the package's operations, with the same
signatures as `sllm_b200.ops`.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared
with, on the GPU, at sizes other than the engine's; (2) patched over
`sllm_b200.ops` (fixture `cpu_ops`), they let the step function, the cache and
the scheduler be exercised on a machine without a GPU.  The product never
imports this file; without its kernels it raises.
"""

from __future__ import annotations

import torch


def embed_gather(table, ids):
    return table[ids.long()].float()


def add_rmsnorm(residual, delta, weight, eps, out_dtype):
    if delta is not None:
        d = delta.float()
        if d.dim() == 3:
            d = d.sum(0)
        residual += d
    var = (residual * residual).mean(-1, keepdim=True)
    return (residual * (var + eps) ** -0.5 * weight).to(out_dtype)


def linear(x, w, bias, out_dtype, allow_partials=False):
    out = x.float() @ w.float().t()
    if bias is not None:
        out = out + bias
    return out.to(out_dtype)


def can_accumulate(x, w):
    return x.dtype == torch.bfloat16 and x.shape[0] <= 8 and x.shape[1] % 32 == 0 and 16 <= w.shape[0] <= 8192


def linear_accumulate(x, w, bias, residual):
    residual += linear(x, w, bias, torch.float32)


def silu_mul(gu, interleave, out_dtype):
    T, two_i = gu.shape
    I = two_i // 2
    v = gu.float().reshape(T, I // interleave, 2, interleave)
    g, u = v[:, :, 0, :], v[:, :, 1, :]
    return (g * (1.0 / (1.0 + torch.exp(-g))) * u).reshape(T, I).to(out_dtype)


def linear_silu_mul(x, w_gate_up, interleave, out_dtype):
    return silu_mul(linear(x, w_gate_up, None, x.dtype), interleave, out_dtype)


def rope_kv_write(qkv, bias, positions, table, rotary_dim, nq, nkv, hd, slot_mapping, k_cache, v_cache, out_dtype):
    x = qkv.float()
    if x.dim() == 3:
        x = x.sum(0)
    T = x.shape[0]
    if bias is not None:
        x = x + bias
    x = x.reshape(T, nq + 2 * nkv, hd)
    if rotary_dim:
        half = rotary_dim // 2
        cs = table[positions.long()]                     # [T, 2, half]
        c, s = cs[:, None, 0, :], cs[:, None, 1, :]
        qk = x[:, :nq + nkv]
        x1, x2 = qk[..., :half], qk[..., half:rotary_dim]
        rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, qk[..., rotary_dim:]], dim=-1)
        x = torch.cat([rot, x[:, nq + nkv:]], dim=1)
    q = x[:, :nq].reshape(T, nq * hd).to(out_dtype)
    if slot_mapping is not None:
        ps = k_cache.shape[2]
        page, off = slot_mapping.long() // ps, slot_mapping.long() % ps
        k_cache[page, :, off, :] = x[:, nq:nq + nkv].to(k_cache.dtype)
        v_cache[page, :, off, :] = x[:, nq + nkv:].to(v_cache.dtype)
    return q


def attention_simt(q, k_cache, v_cache, block_tables, positions, seq_of_token, nq, nkv, hd, scale, window):
    T = q.shape[0]
    ps = k_cache.shape[2]
    out = torch.empty((T, nq, hd), dtype=torch.float32, device=q.device)
    qf = q.float().reshape(T, nq, hd)
    rep = nq // nkv
    for t in range(T):
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        j = torch.arange(lo, pos + 1, device=q.device)
        pages = block_tables[int(seq_of_token[t])].long()[j // ps]
        k = k_cache[pages, :, j % ps, :].float()          # [n, nkv, hd]
        v = v_cache[pages, :, j % ps, :].float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", qf[t], k) * scale
        p = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", p, v)
    return out.reshape(T, nq * hd).to(q.dtype)


def paged_attention(q, k_cache, v_cache, step, group, nq, nkv, hd, scale, window):
    g = step.groups[group]
    return attention_simt(q, k_cache, v_cache, g.block_tables, step.positions, step.seq_of_token,
                          nq, nkv, hd, scale, window)


def gather_rows(x, rows):
    if x.dim() == 3:
        return x[:, rows.long()].sum(0)
    return x[rows.long()].clone()


def sample_rows(logits, temperature=None, uniform=None, top_k=None, top_p=None):
    from tests.plain import qwen2_plain as plain
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    for r in range(R):
        t = float(temperature[r]) if temperature is not None else 0.0
        k = int(top_k[r]) if top_k is not None and int(top_k[r]) > 0 else None
        p = float(top_p[r]) if top_p is not None and float(top_p[r]) >= 0 else None
        out[r] = plain.sample(logits[r].double().cpu().numpy(), t, k, p, u=float(uniform[r]) if t > 0 else None)
    return out


def repetition_penalty_(logits, pair_row, pair_id, pair_penalty):
    V = logits.shape[1]
    for r, i, q in zip(pair_row.tolist(), pair_id.tolist(), pair_penalty.tolist()):
        if 0 <= i < V:
            v = float(logits[r, i])
            logits[r, i] = v * q if v < 0 else v / q
    return logits


def mark_seen(seen, step):
    slots = step.state_slots[step.seq_of_token[:step.num_tokens].long()].long()
    ids = step.token_ids[:step.num_tokens].long()
    ok = (ids >= 0) & (ids < seen.shape[1]) & (slots >= 0) & (slots < seen.shape[0])
    seen[slots[ok], ids[ok]] = 1


def penalty_from_seen_(logits, seen, step, penalty):
    for r in range(logits.shape[0]):
        q = float(penalty[r])
        if not q > 0 or q == 1.0:
            continue
        slot = int(step.state_slots[step.seq_of_token[step.logit_rows[r]]])
        mine = seen[slot].bool()
        row = logits[r].double()
        logits[r] = torch.where(mine, torch.where(row < 0, row * q, row / q), row).float()
    return logits


ALL = ["embed_gather", "add_rmsnorm", "linear", "can_accumulate", "linear_accumulate", "silu_mul", "linear_silu_mul", "rope_kv_write",
       "attention_simt", "paged_attention", "gather_rows", "sample_rows", "repetition_penalty_", "mark_seen", "penalty_from_seen_"]
