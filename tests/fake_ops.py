"""A stand-in for the CUDA extension, in torch on the CPU, for tests of the host-side logic
(cache manager, batching, run order, scheduler) on a machine without a GPU.

It has the functions of the extension module with the same arguments and the same
in-place effects.  It is test equipment: the package never selects it; a test installs it
with ``vt_transformer_b200.ops.use_backend``.  Kernels themselves are tested on the GPU
against the plain implementation, not against this file.
"""
from __future__ import annotations

import torch


def embedding(table, ids, out, status=None, scale=1.0):
    idx = ids.long()
    ok = (idx >= 0) & (idx < table.shape[0])
    out.zero_()
    out[ok] = table[idx[ok]].float() * scale
    if status is not None and bool((idx >= table.shape[0]).any()):
        status[0] = 1


def logits_scale_cap(logits, scale, cap):
    logits.mul_(scale)
    if cap > 0:
        logits.copy_(cap * torch.tanh(logits / cap))


def rmsnorm(x, delta, weight, eps, out, rows=None, status=None):
    idx = torch.arange(x.shape[0]) if rows is None else rows.long()
    v = x[idx]
    if delta is not None:
        v = v + delta[idx].float()
        x[idx] = v
    r = torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + eps)
    out.copy_((weight * v * r).to(out.dtype))


def silu_mul(gu, out, interleave=0):
    inter = out.shape[1]
    if interleave:
        pairs = gu.view(gu.shape[0], inter // 8, 2, 8).float()
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
    else:
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def _rotate(x, cs):
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = cs[:, None, :, 0], cs[:, None, :, 1]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rope_store(qkv, positions, cos_sin, k_cache, v_cache, token_seq, block_table, heads, kv_heads, head_dim,
               store, status=None):
    T = qkv.shape[0]
    live = token_seq >= 0
    qd, kd = heads * head_dim, kv_heads * head_dim
    page_size = k_cache.shape[2]
    q = qkv[:, :qd].view(T, heads, head_dim)
    k = qkv[:, qd:qd + kd].view(T, kv_heads, head_dim)
    v = qkv[:, qd + kd:].view(T, kv_heads, head_dim)
    pos = positions.long().clamp(min=0)
    if cos_sin is not None:
        cs = cos_sin[pos]
        q_rot = _rotate(q, cs).to(qkv.dtype)
        k_rot = _rotate(k, cs).to(qkv.dtype)
        q[live] = q_rot[live]
    else:
        k_rot = k
    if not store:
        return
    for t in range(T):
        if not bool(live[t]):
            continue
        p = int(positions[t])
        page = int(block_table[int(token_seq[t]), p // page_size])
        assert 0 <= page < k_cache.shape[0], "bad page"
        k_cache[page, :, p % page_size, :] = k_rot[t]
        v_cache[page, :, p % page_size, :] = v[t]


def gemm_simt(a, w, bias, c):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias
    c.copy_(y.to(c.dtype))


def attention_simt(qkv, out, k_cache, v_cache, positions, token_seq, block_table, heads, kv_heads, head_dim,
                   window, scale, status=None):
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    g = heads // kv_heads
    q = qkv[:, :heads * head_dim].view(T, heads, head_dim).float()
    for t in range(T):
        s = int(token_seq[t])
        if s < 0:
            out[t] = 0
            continue
        p = int(positions[t])
        first = max(0, p - window + 1) if window > 0 else 0
        js = torch.arange(first, p + 1)
        pages = block_table[s, (js // page_size)].long()
        assert bool((pages >= 0).all()), "attention reads a page that is not held"
        keys = k_cache[pages, :, js % page_size, :].float()      # [J, kv_heads, d]
        vals = v_cache[pages, :, js % page_size, :].float()
        for h in range(heads):
            sc = (keys[:, h // g, :] @ q[t, h]) * scale
            pr = torch.softmax(sc, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (pr @ vals[:, h // g, :]).to(out.dtype)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def sample(logits, temperature, top_k, top_p, u, out):
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        k = int(top_k[r])
        if not t > 0 or k == 1:
            out[r] = int(torch.argmax(logits[r]))
            continue
        z = logits[r].double() / t
        keep = torch.ones_like(z, dtype=torch.bool)
        if 0 < k < z.numel():
            keep &= z >= torch.topk(z, k).values[-1]
        e = torch.where(keep, torch.exp(z - z.max()), torch.zeros_like(z))
        p = float(top_p[r])
        if p < 1.0:
            order = torch.argsort(e, descending=True)
            c = torch.cumsum(e[order], 0)
            n = int(torch.searchsorted(c, torch.tensor(p * float(c[-1]), dtype=torch.float64))) + 1
            thr = e[order[min(n, z.numel()) - 1]]
            e = torch.where(e >= thr, e, torch.zeros_like(e))
        c = torch.cumsum(e, 0)
        idx = int(torch.searchsorted(c, torch.tensor(float(u[r]) * float(c[-1]), dtype=torch.float64), right=True))
        out[r] = min(idx, z.numel() - 1)
