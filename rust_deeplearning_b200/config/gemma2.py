"""Gemma 2 (`Gemma2ForCausalLM`): typed configuration and its description as parts.

Keys are the architecture's own config.json keys.  The reference's Gemma 2
struct (`rustml/nlp/main/src/api/types.rs:336-350`, mapping `:597-632`) reads
only a subset (no head_dim, query_pre_attn_scalar, final_logit_softcapping) and
hard-codes the rest; here every size and constant of the model comes from the
file and none stands in code.  What is fixed here is what the architecture
fixes: the (1 + w) norm (`types.rs:619`), the embedding scale sqrt(hidden)
(`types.rs:618`), the four norms around mixer and feed-forward
(`rustml/nn/main/src/core/transformer_block.rs:143-163`), GeGLU
(`rustml/nn/main/src/core/feed_forward.rs:98-111`) and even layers local, odd
layers global (`rustml/nlp/main/src/core/model.rs:175-179`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from .base import Architecture, ConfigReader, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

ARCHITECTURE_NAME = "Gemma2ForCausalLM"
MODEL_TYPE = "gemma2"


@dataclass(frozen=True)
class Gemma2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    query_pre_attn_scalar: float
    max_position_embeddings: int
    hidden_activation: str
    sliding_window: Optional[int]
    attn_logit_softcapping: Optional[float]
    final_logit_softcapping: Optional[float]
    tie_word_embeddings: bool
    layer_types: Tuple[str, ...]          # "sliding_attention" | "full_attention", one per layer
    bos_token_id: Optional[int]
    eos_token_id: Tuple[int, ...]
    torch_dtype: Optional[str]

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "Gemma2Config":
        r = ConfigReader(raw, "Gemma2 config")
        L = r.integer("num_hidden_layers", minimum=1, maximum=65536)
        H = r.integer("hidden_size", minimum=1)
        nh = r.integer("num_attention_heads", minimum=1)
        # optional in the reference too, falling back to the number of heads (types.rs:340, :606)
        nkv = r.integer("num_key_value_heads", default=nh, minimum=1)
        hd = r.integer("head_dim", minimum=2)
        I = r.integer("intermediate_size", minimum=1)
        V = r.integer("vocab_size", minimum=1)
        eps = r.number("rms_norm_eps", positive=True)
        theta = r.number("rope_theta", positive=True)
        qs = r.number("query_pre_attn_scalar", positive=True)
        maxpos = r.integer("max_position_embeddings", minimum=1)
        # older files name the same key 'hidden_act'
        act = r.string("hidden_activation" if raw.get("hidden_activation") is not None or
                       raw.get("hidden_act") is None else "hidden_act")
        window = r.integer("sliding_window", default=None, minimum=1)
        attn_cap = r.number("attn_logit_softcapping", default=None, positive=True)
        final_cap = r.number("final_logit_softcapping", default=None, positive=True)
        tie = r.boolean("tie_word_embeddings", default=True)
        bos = r.integer("bos_token_id", default=None, minimum=0)
        eos = r.id_list("eos_token_id", default=())
        dtype = r.string("torch_dtype", default=raw.get("dtype") if isinstance(raw.get("dtype"), str) else None)

        layer_types = raw.get("layer_types")
        if layer_types is None and L is not None:
            # even layers local, odd layers global: nlp/main/src/core/model.rs:175-179
            layer_types = ["sliding_attention" if (i % 2 == 0 and window is not None) else "full_attention"
                           for i in range(L)]
        elif L is not None:
            ok = (isinstance(layer_types, list) and len(layer_types) == L
                  and all(t in ("sliding_attention", "full_attention") for t in layer_types))
            r.check(ok, f"key 'layer_types' must list 'sliding_attention' or 'full_attention' for each of the {L} layers")
            if ok:
                r.check(window is not None or "sliding_attention" not in layer_types,
                        "'layer_types' has sliding layers but 'sliding_window' is not given")
            else:
                layer_types = []

        if nh and nkv:
            r.check(nh % nkv == 0, f"num_attention_heads ({nh}) must be a multiple of num_key_value_heads ({nkv})")
        if hd:
            r.check(hd % 2 == 0, f"head_dim ({hd}) must be even for the rotary pairing")
        if eos and V:
            r.check(all(0 <= t < V for t in eos), f"eos_token_id {eos} outside the vocabulary of {V}")
        r.finish()
        return Gemma2Config(L, H, nh, nkv, hd, I, V, eps, theta, qs, maxpos, act, window, attn_cap, final_cap,
                            tie, tuple(layer_types), bos, tuple(eos), dtype)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        eos = list(self.eos_token_id)
        d["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        d["architectures"] = [ARCHITECTURE_NAME]
        d["model_type"] = MODEL_TYPE
        return {k: v for k, v in d.items() if v is not None}


def build_spec(cfg: Gemma2Config) -> ModelSpec:
    """The model as parts.  Tensor names are the checkpoint's own
    (`rustml/nlp/main/src/core/weight_map.rs:270-343` lists them for the four-norm layout)."""
    H, hd, nh, nkv, I, V = (cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads,
                            cfg.num_key_value_heads, cfg.intermediate_size, cfg.vocab_size)

    def norm(name):
        return PartSpec("rms_norm", {"size": H, "eps": cfg.rms_norm_eps, "offset": 1.0},
                        {"weight": TensorSpec(name, (H,), "vector")})

    position = PartSpec("rotary", {"theta": cfg.rope_theta, "head_dim": hd, "rotary_dim": hd,
                                   "max_positions": cfg.max_position_embeddings})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        local = cfg.layer_types[i] == "sliding_attention"
        mixer = PartSpec(
            "attention",
            {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd,
             # scores are divided by sqrt(query_pre_attn_scalar): attention.rs:415-416, model.rs:692
             "score_scale": 1.0 / math.sqrt(cfg.query_pre_attn_scalar),
             "softcap": cfg.attn_logit_softcapping,
             "window": cfg.sliding_window if local else None,
             "position": position},
            {"q": TensorSpec(p + "self_attn.q_proj.weight", (nh * hd, H)),
             "k": TensorSpec(p + "self_attn.k_proj.weight", (nkv * hd, H)),
             "v": TensorSpec(p + "self_attn.v_proj.weight", (nkv * hd, H)),
             "o": TensorSpec(p + "self_attn.o_proj.weight", (H, nh * hd))})
        ff = PartSpec(
            "gated_mlp",
            {"hidden_size": H, "intermediate_size": I, "activation": cfg.hidden_activation},
            {"gate": TensorSpec(p + "mlp.gate_proj.weight", (I, H)),
             "up": TensorSpec(p + "mlp.up_proj.weight", (I, H)),
             "down": TensorSpec(p + "mlp.down_proj.weight", (H, I))})
        norms = {"pre_mixer": norm(p + "input_layernorm.weight"),
                 "post_mixer": norm(p + "post_attention_layernorm.weight"),
                 "pre_feed_forward": norm(p + "pre_feedforward_layernorm.weight"),
                 "post_feed_forward": norm(p + "post_feedforward_layernorm.weight")}
        layers.append(LayerSpec("sandwich", mixer, ff, norms))

    table = TensorSpec("model.embed_tokens.weight", (V, H))
    embedding = PartSpec("scaled_embedding", {"vocab_size": V, "hidden_size": H, "scale": math.sqrt(H)},
                         {"table": table})
    head_weight = table if cfg.tie_word_embeddings else TensorSpec("lm_head.weight", (V, H))
    head = PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "softcap": cfg.final_logit_softcapping},
                    {"weight": head_weight})
    spec = ModelSpec(
        architecture=ARCHITECTURE_NAME, hidden_size=H, vocab_size=V,
        max_positions=cfg.max_position_embeddings, embedding=embedding, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"), head=head,
        stop_token_ids=cfg.eos_token_id, bos_token_id=cfg.bos_token_id,
        # buffers some exporters write, and the head's copy of the tied table (model.rs:829-834 ties them)
        ignored_tensors=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ()))
    spec.validate()
    return spec


register_architecture(Architecture(ARCHITECTURE_NAME, MODEL_TYPE, Gemma2Config.from_dict, build_spec), replace=True)
