"""Plain, slow Gemma 2 in numpy: the oracle the engine is compared with.

Whole sequences, no cache, no batching, one function per part, float64 by
default.  It shares no code with the package: it reads config.json and the
safetensors file itself, and every formula is written from the reference's
source (sweengineeringlabs/rust-deeplearning, crate paths below are relative to
`rustml/`).  The reference is CPU Rust and no Rust toolchain exists where this
build runs, so nothing here was compared with a compiled reference: it rests on
the formulas.

Where the reference's own Gemma 2 route deviates from the architecture (two
norms per block, SiLU, no final soft-cap, head_dim = hidden/heads, window
ignored for single-token steps) this file follows the architecture and cites
the shared layer code that implements the right formula.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------

def read_config(folder):
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def _bf16_to_f32(raw):
    # bf16 -> f32 is a 16-bit left shift: hub/main/src/core/safetensors.rs:272-274
    u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32)
    return (u16 << 16).view(np.float32)


def read_safetensors(path):
    """u64 LE header length, JSON header, data: hub/main/src/core/safetensors.rs:59-121."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[base + b:base + e]
        if info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "BF16":
            arr = _bf16_to_f32(raw)
        elif info["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"]).astype(np.float64)
    return out


def load_folder(folder):
    return read_config(folder), read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(table, ids, hidden_size):
    """x[t] = E[id_t] * sqrt(H): nn/main/src/core/embedding.rs:50-76 (gather),
    nlp/main/src/core/model.rs:896-900 (scale), nlp/main/src/api/types.rs:618 (value)."""
    ids = np.asarray(ids)
    if ids.min() < 0 or ids.max() >= table.shape[0]:
        raise IndexError("token id out of range")
    return table[ids] * np.float64(np.float32(math.sqrt(hidden_size)))


def rms_norm(x, w, eps, offset=1.0):
    """y = x / sqrt(mean(x^2) + eps) * (w + offset): core/main/src/core/tensor/ops.rs:735-743,
    offset added to the weight in nn/main/src/core/rms_norm.rs:43-50."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * (w + offset)


def rope_tables(head_dim, n_pos, theta):
    """inv_i = theta^(-2i/hd), angle = pos * inv_i: nn/main/src/core/rope.rs:93-108."""
    half = head_dim // 2
    inv = 1.0 / (np.float64(theta) ** (2.0 * np.arange(half, dtype=np.float64) / head_dim))
    ang = np.arange(n_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang), np.sin(ang)


def rope_apply(x, cos, sin):
    """Half-split rotation of [T, heads, hd] rows at positions 0..T-1:
    out[i] = x[i] cos - x[i+hd/2] sin; out[i+hd/2] = x[i] sin + x[i+hd/2] cos
    (nn/main/src/core/rope.rs:188-191)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)


def attention_mask(T, window):
    """keep j <= p, and p - j < window on local layers:
    core/main/src/core/tensor/ops.rs:905-922 (causal), :932-952 (window test :939)."""
    p = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    keep = j <= p
    if window is not None:
        keep &= (p - j) < window
    return keep


def attention(n, wq, wk, wv, wo, cos, sin, *, n_heads, n_kv_heads, head_dim,
              query_pre_attn_scalar, softcap, window):
    """Whole-sequence grouped-query attention, nn/main/src/core/attention.rs:372-448:
    projections without bias (:372-374), RoPE on q and k (:394-398), consecutive query
    heads share a KV head (core/main/src/core/tensor/ops.rs:980-987), scores divided by
    sqrt(query_pre_attn_scalar) (:415-416, nlp/main/src/core/model.rs:692), soft-cap
    cap*tanh(s/cap) after the scale and before the mask (:419-423), -inf mask, softmax
    (core/main/src/core/tensor/ops.rs:598-608), P.V (:442-446), output projection (:448).
    The mask is applied for every length (the reference skips it for a single new
    token, attention.rs:429; the architecture does not)."""
    T = n.shape[0]
    q = (n @ wq.T).reshape(T, n_heads, head_dim)
    k = (n @ wk.T).reshape(T, n_kv_heads, head_dim)
    v = (n @ wv.T).reshape(T, n_kv_heads, head_dim)
    q = rope_apply(q, cos[:T], sin[:T])
    k = rope_apply(k, cos[:T], sin[:T])
    group = n_heads // n_kv_heads
    keep = attention_mask(T, window)
    out = np.zeros((T, n_heads, head_dim))
    for h in range(n_heads):
        g = h // group
        s = q[:, h, :] @ k[:, g, :].T
        s = s / math.sqrt(query_pre_attn_scalar)
        if softcap is not None:
            s = softcap * np.tanh(s / softcap)
        s = np.where(keep, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        e = np.exp(s)
        a = e / e.sum(axis=-1, keepdims=True)
        out[:, h, :] = a @ v[:, g, :]
    return out.reshape(T, n_heads * head_dim) @ wo.T


def gelu_tanh(x):
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))): core/main/src/core/tensor/ops.rs:433-438."""
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def feed_forward(n, wg, wu, wd):
    """down(gelu(gate(x)) * up(x)): nn/main/src/core/feed_forward.rs:151-161."""
    return (gelu_tanh(n @ wg.T) * (n @ wu.T)) @ wd.T


def block(x, w, prefix, cfg, cos, sin, window):
    """h = x + post_attn_norm(attn(input_norm(x))); y = h + post_ffn_norm(mlp(pre_ffn_norm(h))):
    nn/main/src/core/transformer_block.rs:324-355."""
    eps = cfg["rms_norm_eps"]
    n1 = rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    a = attention(
        n1,
        w[prefix + "self_attn.q_proj.weight"], w[prefix + "self_attn.k_proj.weight"],
        w[prefix + "self_attn.v_proj.weight"], w[prefix + "self_attn.o_proj.weight"],
        cos, sin,
        n_heads=cfg["num_attention_heads"],
        n_kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
        head_dim=cfg["head_dim"],
        query_pre_attn_scalar=cfg["query_pre_attn_scalar"],
        softcap=cfg.get("attn_logit_softcapping"),
        window=window,
    )
    h = x + rms_norm(a, w[prefix + "post_attention_layernorm.weight"], eps)
    n2 = rms_norm(h, w[prefix + "pre_feedforward_layernorm.weight"], eps)
    f = feed_forward(n2, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                     w[prefix + "mlp.down_proj.weight"])
    return h + rms_norm(f, w[prefix + "post_feedforward_layernorm.weight"], eps)


def layer_window(cfg, i):
    """Even layers are local, odd layers global: nlp/main/src/core/model.rs:175-179."""
    if cfg.get("sliding_window") is None:
        return None
    return cfg["sliding_window"] if i % 2 == 0 else None


def lm_head(n, table, final_softcap):
    """Tied output projection (nlp/main/src/core/model.rs:829-834, :936) and the final
    soft-cap cap*tanh(z/cap), which the reference lacks (llmforge/BACKLOG.md:248,255)
    and the architecture has."""
    z = n @ table.T
    if final_softcap is not None:
        z = final_softcap * np.tanh(z / final_softcap)
    return z


def forward(cfg, w, ids):
    """Logits [T, V] of one whole sequence: nlp/main/src/core/model.rs:847-887."""
    T = len(ids)
    if T > cfg["max_position_embeddings"]:
        raise ValueError("sequence longer than max_position_embeddings")  # model.rs:906-913
    table = w["model.embed_tokens.weight"]
    x = embed(table, ids, cfg["hidden_size"])
    cos, sin = rope_tables(cfg["head_dim"], T, cfg["rope_theta"])
    for i in range(cfg["num_hidden_layers"]):
        x = block(x, w, f"model.layers.{i}.", cfg, cos, sin, layer_window(cfg, i))
    n = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = table if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return lm_head(n, head, cfg.get("final_logit_softcapping"))


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------

def argmax(logits):
    """First maximum wins (strict >): nlp/main/src/core/sampling.rs:8-18."""
    best, mx = 0, -math.inf
    for i, v in enumerate(logits):
        if v > mx:
            best, mx = i, v
    return best


def apply_repetition_penalty(logits, past, penalty):
    """Positive logits divided, others multiplied, once per occurrence in the history:
    nlp/main/src/core/sampling.rs:23-34."""
    out = np.array(logits, dtype=np.float32)
    for t in past:
        if 0 <= t < len(out):
            out[t] = out[t] / np.float32(penalty) if out[t] > 0 else out[t] * np.float32(penalty)
    return out


def apply_top_k(logits, k):
    """Keep values >= the k-th largest, ties kept: nlp/main/src/core/sampling.rs:38-52."""
    out = np.array(logits, dtype=np.float32)
    if k >= len(out):
        return out
    thr = np.sort(out)[len(out) - k]
    out[out < thr] = -np.inf
    return out


def softmax32(logits):
    x = np.asarray(logits, dtype=np.float32)
    e = np.exp(x - x.max())
    return e / e.sum(dtype=np.float32)


def apply_top_p(logits, p):
    """Smallest descending prefix whose cumulative probability reaches p, crossing token
    included: nlp/main/src/core/sampling.rs:56-87."""
    out = np.array(logits, dtype=np.float32)
    if p >= 1.0:
        return out
    probs = softmax32(out)
    order = np.argsort(-probs, kind="stable")
    keep = np.zeros(len(out), dtype=bool)
    c = np.float32(0.0)
    for idx in order:
        c += probs[idx]
        keep[idx] = True
        if c >= p:
            break
    out[~keep] = -np.inf
    return out


def sample_categorical(logits, r):
    """Stable softmax, first index with r < cumulative sum, else the last index:
    nlp/main/src/core/sampling.rs:91-106.  `r` in [0, 1) is given by the caller."""
    probs = softmax32(logits)
    c = np.float32(0.0)
    for i, pr in enumerate(probs):
        c += pr
        if r < c:
            return i
    return len(probs) - 1


def sample_token(logits, past, r, *, temperature, top_k=None, top_p=None, repetition_penalty=None):
    """penalty -> /temperature -> top-k -> top-p -> draw; temperature < 1e-7 is greedy:
    nlp/main/src/core/generator.rs:176-201."""
    if temperature < 1e-7:
        return argmax(logits)
    x = np.array(logits, dtype=np.float32)
    if repetition_penalty is not None:
        x = apply_repetition_penalty(x, past, repetition_penalty)
    x = x / np.float32(temperature)
    if top_k is not None:
        x = apply_top_k(x, top_k)
    if top_p is not None:
        x = apply_top_p(x, top_p)
    return sample_categorical(x, r)


def generate_greedy(cfg, w, prompt, max_new_tokens, stop_ids=()):
    """Prefill, sample, then feed each sampled token back; a stop token ends the sequence
    and is not returned; at most max_new_tokens tokens: nlp/main/src/core/generator.rs:243-273.
    Re-runs the whole sequence for every token, as the cache-less loop in
    nlp/main/src/core/generation.rs:48-95 does."""
    tokens = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        logits = forward(cfg, w, tokens)[-1]
        t = argmax(logits.astype(np.float32))
        if t in stop_ids:
            break
        tokens.append(t)
        new.append(t)
    return new
