"""Plain torch restatements of every kernel entry point in `rust_deeplearning_b200.kernels.ops`,
with the same signatures, computed in float64 with Python loops.

Two uses, both in tests only:
  * each CUDA kernel is compared with its function here, at sizes of the tests' choosing;
  * `install(monkeypatch)` swaps them in for the CUDA entry points so that the engine's
    host logic (batching, paging, slots, schedules) can be exercised on a machine without a GPU.
They share no code with the kernels; formulas are cited in tests/plain_gemma2.py.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def embed_rows(table, ids, scale, status=None):
    ids = ids.long()
    bad = (ids < 0) | (ids >= table.shape[0])
    out = table[ids.clamp(0, table.shape[0] - 1)].to(F64) * float(torch.tensor(scale, dtype=torch.float32))
    out[bad] = float("nan")
    if status is not None and bool(bad.any()):
        status[0] = 1
    return out.to(torch.float32)


def _rms(v, p):
    w, eps, off = p
    ms = (v * v).mean(dim=-1, keepdim=True)
    return v / torch.sqrt(ms + eps) * (w.to(F64) + off)


def norm_residual_norm(x, *, first=None, residual=None, second=None, out_dtype=None, row_index=None, want_output=True):
    v = x.to(F64)
    if row_index is not None:
        v = v[row_index.long()]
    t = _rms(v, first) if first is not None else v
    if residual is not None:
        h = residual.to(F64) + t
        residual.copy_(h.to(torch.float32))
    else:
        h = t
    if not want_output:
        return None
    y = _rms(h, second) if second is not None else h
    return y.to(out_dtype or x.dtype)


def gated_activation(gate_up, activation):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].to(F64), gate_up[:, inter:].to(F64)
    if activation in ("gelu_pytorch_tanh", "gelu_tanh"):
        a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    elif activation == "silu":
        a = g / (1.0 + torch.exp(-g))
    else:
        raise ValueError(activation)
    return (a * u).to(gate_up.dtype)


def softcap_(z, cap):
    z.copy_((cap * torch.tanh(z.to(F64) / cap)).to(z.dtype))
    return z


def residual_add_(residual, x):
    residual.copy_((residual.to(F64) + x.to(F64)).to(torch.float32))
    return residual


def convert_rows(x, out_dtype, row_index=None):
    v = x if row_index is None else x[row_index.long()]
    return v.to(out_dtype)


def linear(x, weight, out_dtype=None, softcap=None, status=None):
    z = x.to(F64) @ weight.to(F64).t()
    if softcap is not None:
        z = softcap * torch.tanh(z / softcap)
    return z.to(out_dtype or x.dtype)


def linear_gated(x, weight_gate_up, activation, status=None):
    return gated_activation(x.to(F64) @ weight_gate_up.to(F64).t(), activation).to(x.dtype)


def _cache_index(table_row, pos, page_size, ring_pages):
    logical = pos // page_size
    return int(table_row[logical % ring_pages]), pos - logical * page_size


def _swizzle_index(r, head_dim, element_size):
    """Where the elements of a row lie inside a cache page: the row's 16-byte chunks are stored at
    chunk c ^ (r & 7), r being the row's place in its page; chunks of the last incomplete group of
    eight, and rows whose size is no multiple of 16 bytes, are stored plainly."""
    epc = 16 // element_size
    idx = torch.arange(head_dim)
    if head_dim % epc:
        return idx
    chunks = head_dim // epc
    c = idx // epc
    c_stored = torch.where((c | 7) < chunks, c ^ (r & 7), c)
    return c_stored * epc + idx % epc


def cache_store(dst_row, values, r):
    """Write a key or value row into its place `r` of a cache page."""
    dst_row[_swizzle_index(r, values.numel(), values.element_size()).to(dst_row.device)] = values


def cache_load(src_row, r):
    """Read the key or value row at place `r` of a cache page."""
    return src_row[_swizzle_index(r, src_row.numel(), src_row.element_size()).to(src_row.device)]


def rope_cache(qkv, n_heads, n_kv_heads, head_dim, *, tok_seq, tok_pos, cos=None, sin=None, rotary_dim=0,
               pages=None, seq_end=None):
    T = qkv.shape[0]
    total = n_heads + 2 * n_kv_heads
    rows = qkv.view(T, total, head_dim)
    half = rotary_dim // 2
    for t in range(T):
        pos = int(tok_pos[t])
        if pos < 0:
            continue
        if cos is not None:
            c, s = cos[pos].to(F64), sin[pos].to(F64)
            for h in range(n_heads + n_kv_heads):
                x1, x2 = rows[t, h, :half].to(F64), rows[t, h, half:rotary_dim].to(F64)
                rows[t, h, :half] = (x1 * c - x2 * s).to(qkv.dtype)
                rows[t, h, half:rotary_dim] = (x1 * s + x2 * c).to(qkv.dtype)
        if pages is not None and n_kv_heads > 0:
            seq = int(tok_seq[t])
            if pos + pages.ring_pages * pages.page_size < int(seq_end[seq]):
                continue
            page, r = _cache_index(pages.tables[seq], pos, pages.page_size, pages.ring_pages)
            for g in range(n_kv_heads):
                cache_store(pages.k[page, g, r], rows[t, n_heads + g], r)
                cache_store(pages.v[page, g, r], rows[t, n_heads + n_kv_heads + g], r)
    return qkv


def attention(q, b, pages, *, n_heads, n_kv_heads, head_dim, score_scale, softcap, window, new_kv=None,
              kind="auto", scratch=None, keys_per_split=None, status=None, rotate_and_write=None):
    if rotate_and_write is not None:
        # the step's rows as the projection left them: rotate a copy, write the cache, then read everything from it
        cos, sin, rotary_dim = rotate_and_write
        assert new_kv is not None and new_kv[0] is q and q.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
        q = q.clone()
        rope_cache(q, n_heads, n_kv_heads, head_dim, tok_seq=b.tok_seq, tok_pos=b.tok_pos, cos=cos if rotary_dim else None,
                   sin=sin if rotary_dim else None, rotary_dim=rotary_dim, pages=pages, seq_end=b.seq_cached)
    T = q.shape[0]
    out = torch.zeros((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    group = n_heads // n_kv_heads
    for t in range(b.n_tokens):
        p = int(b.tok_pos[t])
        if p < 0:
            continue
        seq = int(b.tok_seq[t])
        cached = int(b.seq_cached[seq])
        row0 = int(b.seq_start[seq]) - int(b.seq_past[seq])
        lo = max(0, p - window + 1) if window else 0
        for h in range(n_heads):
            g = h // group
            qv = q[t, h * head_dim:(h + 1) * head_dim].to(F64)
            ks, vs = [], []
            for j in range(lo, p + 1):
                if j < cached:
                    page, r = _cache_index(pages.tables[seq], j, pages.page_size, pages.ring_pages)
                    ks.append(cache_load(pages.k[page, g, r], r))
                    vs.append(cache_load(pages.v[page, g, r], r))
                else:
                    rows, k_col, v_col = new_kv
                    ks.append(rows[row0 + j, k_col + g * head_dim:k_col + (g + 1) * head_dim])
                    vs.append(rows[row0 + j, v_col + g * head_dim:v_col + (g + 1) * head_dim])
            K, V = torch.stack(ks).to(F64), torch.stack(vs).to(F64)
            s = (K @ qv) * float(torch.tensor(score_scale, dtype=torch.float32))
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            a = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (a @ V).to(q.dtype)
    return out


def attention_vectorised(q, b, pages, *, n_heads, n_kv_heads, head_dim, score_scale, softcap, window, new_kv=None):
    """The same function as `attention`, a sequence at a time with whole matrices (float64 on the tensors'
    device): for cases of thousands of keys, where the loop above over every key of every head takes minutes.
    `tests/test_attention_random_gpu.py` holds the two against each other on small cases."""
    def logical(stored):        # every row of every page in its logical order
        n_pages, n_kv, rows, hd = stored.shape
        idx = torch.stack([_swizzle_index(r, hd, stored.element_size()) for r in range(rows)]).to(stored.device)
        return torch.gather(stored, 3, idx[None, None].expand(n_pages, n_kv, rows, hd))
    k_all, v_all = logical(pages.k), logical(pages.v)
    out = torch.zeros((q.shape[0], n_heads * head_dim), dtype=q.dtype, device=q.device)
    group = n_heads // n_kv_heads
    ps, ring = pages.page_size, pages.ring_pages
    scale = float(torch.tensor(score_scale, dtype=torch.float32))
    for i in range(b.n_seqs):
        r0, r1 = int(b.seq_start[i]), int(b.seq_start[i + 1])
        if r1 == r0:
            continue
        past, cached = int(b.seq_past[i]), int(b.seq_cached[i])
        total = past + (r1 - r0)
        j = torch.arange(total, device=q.device)
        page = pages.tables[i][((j // ps) % ring).long()].long()
        # (in a ring the rows of positions that have been overwritten are wrong here; the window masks them below)
        K = k_all[page, :, (j % ps).long(), :].to(F64)           # [positions, kv heads, head_dim]
        V = v_all[page, :, (j % ps).long(), :].to(F64)
        if cached < total:
            rows, k_col, v_col = new_kv
            width = n_kv_heads * head_dim
            K[cached:] = rows[r0 + (cached - past):r1, k_col:k_col + width].reshape(-1, n_kv_heads, head_dim).to(F64)
            V[cached:] = rows[r0 + (cached - past):r1, v_col:v_col + width].reshape(-1, n_kv_heads, head_dim).to(F64)
        Q = q[r0:r1, :n_heads * head_dim].reshape(-1, n_kv_heads, group, head_dim).to(F64)
        p = b.tok_pos[r0:r1].long()
        s = torch.einsum("tkgd,jkd->tkgj", Q, K) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        seen = j[None, :] <= p[:, None]
        if window:
            seen &= j[None, :] > p[:, None] - window
        a = torch.softmax(s.masked_fill(~seen[:, None, None, :], -math.inf), dim=-1)
        out[r0:r1] = torch.einsum("tkgj,jkd->tkgd", a, V).reshape(r1 - r0, -1).to(q.dtype)
    return out


def sample(logits, *, temperature, top_k=None, top_p=None, repetition_penalty=None, seed=0, row_stream=None,
           row_step=None, history=None, history_start=None, out=None, host_out=None):
    """Follows the kernel's stated semantics (ties at the top-p threshold kept), in float32 like the
    reference's sampling functions; the penalty once per occurrence in the history, each in float32."""
    from rust_deeplearning_b200.sampling.sampler import uniform_for
    rows, vocab = logits.shape
    res = torch.zeros(rows, dtype=torch.int32, device=logits.device)
    for r in range(rows):
        x = logits[r].to(torch.float32).clone()
        if temperature < 1e-7:
            res[r] = int(torch.argmax(x))       # torch returns the first maximum
            continue
        if repetition_penalty not in (None, 1.0) and history is not None:
            hb, he = int(history_start[r]), int(history_start[r + 1])
            for tok in (int(v) for v in history[hb:he]):
                if 0 <= tok < vocab:
                    v = x[tok]
                    x[tok] = v / repetition_penalty if v > 0 else v * repetition_penalty
        w = x / temperature
        if top_k and top_k < vocab:
            thr = torch.sort(w).values[vocab - top_k]
            w[w < thr] = -math.inf
        if top_p is not None and top_p < 1.0:
            e = torch.exp(w - w.max())
            order = torch.argsort(-e, stable=True)
            c = torch.cumsum(e[order], 0)
            n_keep = int((c < top_p * e.sum()).sum()) + 1
            thr = w[order[min(n_keep, vocab) - 1]]
            w[w < thr] = -math.inf
        e = torch.exp(w - w.max())
        u = uniform_for(seed, int(row_stream[r]) if row_stream is not None else r,
                        int(row_step[r]) if row_step is not None else 0)
        c = torch.cumsum(e, 0)
        hit = (u * c[-1] < c).nonzero()
        res[r] = int(hit[0]) if len(hit) else int((w > -math.inf).nonzero()[-1])
    if host_out is not None:
        host_out[:rows] = res.cpu()
    if out is not None:
        out.copy_(res)
        return out
    return res


def upload_batch(dst, src_pinned, n_ints, fed=None):
    dst[:n_ints] = src_pinned[:n_ints].to(dst.device)
    if fed is not None:
        sampled, src_at, tok_at, n_fed = fed
        rows = src_pinned[src_at:src_at + n_fed].long().to(dst.device)
        dst[tok_at:tok_at + n_fed] = sampled[rows]


_NAMES = ["embed_rows", "norm_residual_norm", "gated_activation", "softcap_", "residual_add_", "convert_rows",
          "linear", "linear_gated", "rope_cache", "attention", "sample", "upload_batch"]


def install(monkeypatch):
    """Replace the CUDA entry points by the functions above (tests without a GPU only)."""
    from rust_deeplearning_b200.kernels import ops
    for name in _NAMES:
        monkeypatch.setattr(ops, name, globals()[name])
