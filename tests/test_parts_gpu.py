"""Each part alone on the GPU against the plain implementation's function for it: norm and residual
stream, rotary tables and rotation, feed-forward, embedding and head, the attention mixer over a
cache (whole prompt, then token by token), the block."""
import math

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
from rust_deeplearning_b200.cache.cache import Cache, RunNeeds
from rust_deeplearning_b200.engine.batch import BatchLayout, batch_from_buffer, count_tiles, fill_batch
from rust_deeplearning_b200.kernels import ops
from rust_deeplearning_b200.parts.registry import BuildContext, build_part
from rust_deeplearning_b200.parts.norm import ResidualStream, RMSNorm
from rust_deeplearning_b200.parts.spec import LayerSpec, PartSpec, TensorSpec
from rust_deeplearning_b200.parts.model import build_block

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def as_dtype(t, dtype):
    """A tensor as the device holds it, and the float64 values that stands for."""
    d = t.to(dtype).to(DEV)
    return d, d.double().cpu().numpy()


def close(got, want, dtype, what="", rel=6.0):
    got = got.double().cpu().numpy()
    scale = max(float(np.abs(want).max()), 1e-6)
    tol = (3e-5 if dtype is torch.float32 else rel * 2.0 ** -8) * scale
    err = float(np.abs(got - want).max())
    assert got.shape == want.shape and np.isfinite(got).all()
    assert err <= tol, f"{what}: {err:.3e} > {tol:.3e}"


def make_batch(cache, slots, tokens_per_seq, want="all"):
    lens = [len(t) for t in tokens_per_seq]
    past = [cache.length(s) for s in slots]
    cache.reserve(slots, lens)
    tables = [g.table_rows(slots) for g in cache.kv_groups]
    widths = [g.table_width for g in cache.kv_groups]
    wants = [list(range(l)) for l in lens]
    layout = BatchLayout(sum(lens), len(slots), sum(lens), count_tiles(lens, ops.PREFILL_QUERY_TILE), widths, ops.PREFILL_QUERY_TILE)
    host = np.zeros(layout.size, dtype=np.int32)
    real, n_want, n_tiles = fill_batch(host, layout, tokens=tokens_per_seq, past=past, slots=slots, want=wants, tables=tables)
    dev = torch.from_numpy(host).to(DEV)
    b = batch_from_buffer(dev, layout, real_tokens=real, real_seqs=len(slots), n_want=n_want, n_tiles=n_tiles,
                          is_decode=max(lens) == 1, max_total_len=max(p + l for p, l in zip(past, lens)))
    b.cache_owner_of, b.shared_runs = {0: 0}, frozenset()
    cache.advance(slots, lens)
    return b


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_and_residual_stream(dtype):
    H = 96
    w1, w1f = as_dtype(rnd((H,), 1, 0.3), dtype)
    w2, w2f = as_dtype(rnd((H,), 2, 0.3), dtype)
    n1, n2 = RMSNorm(w1, 1e-5, 1.0), RMSNorm(w2, 1e-6, 0.0)
    x, xf = as_dtype(rnd((7, H), 3, 2.0), torch.float32)
    close(n1.apply(x, dtype), plain.rms_norm(xf, w1f, 1e-5, 1.0), dtype, "apply")
    branch, bf = as_dtype(rnd((7, H), 4), dtype)
    stream = ResidualStream(x.clone())
    stream.add(branch, n1)
    y = stream.normed(n2, dtype)
    h = xf + plain.rms_norm(bf, w1f, 1e-5, 1.0)
    close(stream.value(), h, torch.float32, "residual sum")
    close(y, plain.rms_norm(h, w2f, 1e-6, 0.0), dtype, "fused norm")
    stream.add(branch, None)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    close(stream.normed_rows(n2, rows, dtype), plain.rms_norm((h + bf)[[5, 0]], w2f, 1e-6, 0.0), dtype, "rows")

    class Centered:                     # some other norm kind: the stream takes the unfused route
        def apply(self, v, out_dtype):
            return (v.float() - v.float().mean(-1, keepdim=True)).to(out_dtype)
    stream = ResidualStream(x.clone())
    stream.add(branch, Centered())
    close(stream.normed(n2, dtype), plain.rms_norm(xf + (bf - bf.mean(-1, keepdims=True)), w2f, 1e-6, 0.0), dtype, "unfused")


def test_rotary_tables_and_rotation():
    ctx = BuildContext({}, torch.float32, DEV)
    spec = PartSpec("rotary", {"theta": 1e6, "head_dim": 32, "rotary_dim": 32, "max_positions": 3000})
    rot = build_part("position", spec, ctx)
    assert build_part("position", spec, ctx) is rot                       # one table for all layers
    cos, sin = plain.rope_tables(32, 3000, 1e6)
    assert np.abs(rot.cos.double().cpu().numpy() - cos).max() < 1e-7     # float32 rounding of exact angles
    assert np.abs(rot.sin.double().cpu().numpy() - sin).max() < 1e-7
    T, nh, nkv = 9, 3, 1
    rows, rf = as_dtype(rnd((T, (nh + 2 * nkv) * 32), 5), torch.float32)
    pos = torch.tensor([0, 1, 2, 2999, 17, 1024, 5, 6, 7], dtype=torch.int32, device=DEV)

    class B: tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV); tok_pos = pos
    rot.rotate(rows, nh, nkv, 32, B)
    want = rf.reshape(T, nh + 2 * nkv, 32).copy()
    p = pos.cpu().numpy()
    want[:, :nh + nkv] = plain.rope_apply(want[:, :nh + nkv][None].repeat(1, 0)[0], cos[p], sin[p])
    close(rows, want.reshape(T, -1), torch.float32, "rotation")            # values are untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [5, 40])
def test_gated_mlp_embedding_and_head(dtype, rows):
    H, I, V = 80, 112, 131
    tensors = {"g": rnd((I, H), 6, 0.1), "u": rnd((I, H), 7, 0.1), "d": rnd((H, I), 8, 0.1), "e": rnd((V, H), 9, 0.1)}
    dev = {k: as_dtype(v, dtype) for k, v in tensors.items()}
    ctx = BuildContext({k: v[0] for k, v in dev.items()}, dtype, DEV)
    ff = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_pytorch_tanh"},
                                              {"gate": TensorSpec("g", (I, H)), "up": TensorSpec("u", (I, H)), "down": TensorSpec("d", (H, I))}), ctx)
    x, xf = as_dtype(rnd((rows, H), 10), dtype)
    close(ff.forward(x), plain.feed_forward(xf, dev["g"][1], dev["u"][1], dev["d"][1]), dtype, "gated mlp", rel=10.0)
    emb = build_part("embedding", PartSpec("scaled_embedding", {"scale": math.sqrt(H)}, {"table": TensorSpec("e", (V, H))}), ctx)
    ids = torch.tensor([0, 130, 7], dtype=torch.int32, device=DEV)
    close(emb.forward(ids), plain.embed(dev["e"][1], [0, 130, 7], H), torch.float32, "embedding")
    head = build_part("head", PartSpec("linear_head", {"softcap": 2.0}, {"weight": TensorSpec("e", (V, H))}), ctx)
    logits = head.forward(x)
    assert logits.dtype is torch.float32
    close(logits, plain.lm_head(xf, dev["e"][1], 2.0), torch.float32 if dtype is torch.float32 else torch.bfloat16, "head")


def attention_spec(H, nh, nkv, hd, qs, cap, window, theta, prefix=""):
    return PartSpec("attention",
                    {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "score_scale": qs ** -0.5,
                     "softcap": cap, "window": window,
                     "position": PartSpec("rotary", {"theta": theta, "head_dim": hd, "rotary_dim": hd, "max_positions": 512})},
                    {"q": TensorSpec(prefix + "q", (nh * hd, H)), "k": TensorSpec(prefix + "k", (nkv * hd, H)),
                     "v": TensorSpec(prefix + "v", (nkv * hd, H)), "o": TensorSpec(prefix + "o", (H, nh * hd))})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window,cap", [(4, 2, 16, 8, 50.0), (6, 1, 32, None, None), (3, 3, 48, 40, 5.0)])
def test_attention_mixer_over_its_cache(dtype, nh, nkv, hd, window, cap):
    H, qs, theta, T = 64, 24.0, 1e4, 70
    w = {"q": rnd((nh * hd, H), 11, 0.2), "k": rnd((nkv * hd, H), 12, 0.2), "v": rnd((nkv * hd, H), 13, 0.2),
         "o": rnd((H, nh * hd), 14, 0.2)}
    dev = {k: as_dtype(v, dtype) for k, v in w.items()}
    ctx = BuildContext({k: v[0] for k, v in dev.items()}, dtype, DEV)
    mixer = build_part("mixer", attention_spec(H, nh, nkv, hd, qs, cap, window, theta), ctx)
    kv, state = mixer.needs()
    assert (kv.n_kv_heads, kv.head_dim, kv.window) == (nkv, hd, window) and state is None
    x, xf = as_dtype(rnd((T, H), 15), dtype)
    cos, sin = plain.rope_tables(hd, T, theta)
    want = plain.attention(xf, dev["q"][1], dev["k"][1], dev["v"][1], dev["o"][1], cos, sin, n_heads=nh, n_kv_heads=nkv,
                           head_dim=hd, query_pre_attn_scalar=qs, softcap=cap, window=window)
    cache = Cache([RunNeeds(kv, None)], max_tokens=256, max_seqs=2, page_size=16, dtype=dtype, device=DEV)
    slot = cache.alloc_slot()
    toks = [0] * T
    got = mixer.forward(x[:50].contiguous(), make_batch(cache, [slot], [toks[:50]]), cache.run_cache(0), 0)
    close(got, want[:50], dtype, "whole prompt", rel=10.0)
    for t in range(50, T):
        got = mixer.forward(x[t:t + 1].contiguous(), make_batch(cache, [slot], [[0]]), cache.run_cache(0), 0)
        close(got, want[t:t + 1], dtype, f"position {t}", rel=10.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sandwich_block(dtype):
    H, nh, nkv, hd, I, T = 64, 4, 2, 16, 128, 33
    cfg = {"rms_norm_eps": 1e-6, "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
           "query_pre_attn_scalar": 16, "attn_logit_softcapping": 50.0}
    p = "model.layers.0."
    names = {p + "self_attn.q_proj.weight": (nh * hd, H), p + "self_attn.k_proj.weight": (nkv * hd, H),
             p + "self_attn.v_proj.weight": (nkv * hd, H), p + "self_attn.o_proj.weight": (H, nh * hd),
             p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
             p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
             p + "pre_feedforward_layernorm.weight": (H,), p + "post_feedforward_layernorm.weight": (H,)}
    dev = {n: as_dtype(rnd(s, 20 + i, 0.15), dtype) for i, (n, s) in enumerate(names.items())}
    ctx = BuildContext({n: v[0] for n, v in dev.items()}, dtype, DEV)
    mixer = attention_spec(H, nh, nkv, hd, 16, 50.0, 8, 1e4)
    mixer = PartSpec(mixer.kind, mixer.params, {r: TensorSpec(p + f"self_attn.{r}_proj.weight", names[p + f"self_attn.{r}_proj.weight"])
                                                for r in "qkvo"})
    ff = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_pytorch_tanh"},
                  {r: TensorSpec(p + f"mlp.{r}_proj.weight", names[p + f"mlp.{r}_proj.weight"]) for r in ("gate", "up", "down")})
    norm = lambda n: PartSpec("rms_norm", {"size": H, "eps": 1e-6, "offset": 1.0}, {"weight": TensorSpec(p + n, (H,), "vector")})
    layer = LayerSpec("sandwich", mixer, ff, {"pre_mixer": norm("input_layernorm.weight"), "post_mixer": norm("post_attention_layernorm.weight"),
                                              "pre_feed_forward": norm("pre_feedforward_layernorm.weight"),
                                              "post_feed_forward": norm("post_feedforward_layernorm.weight")})
    blk = build_block(layer, ctx)
    x, xf = as_dtype(rnd((T, H), 40), torch.float32)
    cos, sin = plain.rope_tables(hd, T, 1e4)
    want = plain.block(xf, {n: v[1] for n, v in dev.items()}, p, cfg, cos, sin, 8)
    kv, _ = blk.mixer.needs()
    cache = Cache([RunNeeds(kv, None)], max_tokens=128, max_seqs=1, page_size=16, dtype=dtype, device=DEV)
    slot = cache.alloc_slot()
    stream = ResidualStream(x.clone())
    blk.forward(stream, make_batch(cache, [slot], [[0] * T]), cache.run_cache(0), 0)
    close(stream.value(), want, torch.float32 if dtype is torch.float32 else torch.bfloat16, "block", rel=10.0)
