"""Configurations drawn at random (seeded): every size and option of the architecture varies from case to case -
head sizes from 16 to 256 (one that is no multiple of 16), one to four key/value heads with one to nine query
heads each (nine is more than the fast decode kernel takes), widths that are no multiple of 8, one to three
layers, any vocabulary, windows from 5 keys to none, soft-caps on and off, tied and untied heads, pages of 16, 32
and 64 rows.  Each case runs one to five sequences of unequal length through the engine in both dtypes - whole,
as a prefix with single tokens after it (shorter sequences end earlier), and as chunks of 1 to 59 tokens a step
that mix with one another - and compares every logit with the plain implementation; in float32 the three ways
of cutting also have to give the same bits."""
import tempfile

import numpy as np
import pytest
import torch

import model_helpers as mh
import plain_gemma2 as plain

pytestmark = pytest.mark.gpu


def draw(case: int):
    rng = np.random.default_rng(case)
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 128, 24, 256]))
    n_kv = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 5, 8, 9]))
    window = int(rng.choice([0, 5, 17, 64, 70, 130]))
    cfg = {
        "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
        "num_hidden_layers": int(rng.integers(1, 4)), "hidden_size": int(rng.choice([48, 64, 72, 88, 136, 50, 200])),
        "num_attention_heads": n_kv * group, "num_key_value_heads": n_kv, "head_dim": hd,
        "intermediate_size": int(rng.choice([64, 96, 112, 200, 70])), "vocab_size": int(rng.integers(90, 500)),
        "rms_norm_eps": float(rng.choice([1e-6, 1e-5, 1e-3])), "rope_theta": float(rng.choice([500.0, 10000.0, 1e6])),
        "sliding_window": window or None, "query_pre_attn_scalar": int(rng.choice([hd, 24, 100, 144])),
        "attn_logit_softcapping": float(rng.choice([0, 20.0, 50.0])) or None,
        "final_logit_softcapping": float(rng.choice([0, 15.0, 30.0])) or None, "max_position_embeddings": 1024,
        "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": bool(rng.integers(0, 2)),
        "bos_token_id": 2, "eos_token_id": 1,
    }
    page = int(rng.choice([16, 32, 64]))
    lengths = [int(v) for v in rng.integers(1, 500 if case % 4 == 0 else 230, size=int(rng.integers(1, 6)))]
    return rng, cfg, page, lengths


@pytest.mark.parametrize("case", range(12))
def test_a_configuration_drawn_at_random(case):
    from rust_deeplearning_b200 import Engine, load_model, write_random_model
    rng, cfg, page, lengths = draw(case)
    what = f"heads {cfg['num_attention_heads']}/{cfg['num_key_value_heads']} x {cfg['head_dim']}, width {cfg['hidden_size']}, " \
           f"window {cfg['sliding_window']}, page {page}, lengths {lengths}"
    with tempfile.TemporaryDirectory(prefix="rdl_random_") as folder:
        write_random_model(folder, cfg, case, "bfloat16")
        plain_cfg, plain_weights = plain.load_folder(folder)
        seqs = [mh.prompt(1000 + 10 * case + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]
        want = [plain.forward(plain_cfg, plain_weights, s) for s in seqs]
        for dtype in ("float32", "bfloat16"):
            eng = Engine(load_model(folder, dtype, "cuda:0"), max_tokens=4096, max_seqs=8, page_size=page)
            # whole prompts, one batch, every position
            slots = [eng.new_sequence() for _ in seqs]
            whole = eng.step(slots, seqs, "all").clone()
            mh.assert_logits(whole, np.concatenate(want), dtype, f"{dtype}, whole; {what}")
            first_row = np.concatenate([[0], np.cumsum(lengths)])
            exact = dtype == "float32"          # the 32-bit path gives the same bits however the tokens are cut
            for s in slots:
                eng.release(s)
            # a prefix, then single tokens
            k = int(rng.integers(1, 12))
            cut = [max(1, len(s) - k) for s in seqs]
            slots = [eng.new_sequence() for _ in seqs]
            eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], [[] for _ in seqs])
            for j in range(k):
                live = [i for i, (s, c) in enumerate(zip(seqs, cut)) if c + j < len(s)]
                if not live:
                    break
                got = eng.step([slots[i] for i in live], [[seqs[i][cut[i] + j]] for i in live], "last")
                mh.assert_logits(got, np.stack([want[i][cut[i] + j] for i in live]), dtype, f"{dtype}, single tokens, step {j}; {what}")
                for r, i in enumerate(live):
                    assert not exact or torch.equal(got[r], whole[first_row[i] + cut[i] + j]), \
                        f"float32 bits of position {cut[i] + j} of sequence {i} differ between a single-token step and the whole prompt; {what}"
            for s in slots:
                eng.release(s)
            # chunks of many tokens on a cached prefix, of another length for each sequence and step
            slots = [eng.new_sequence() for _ in seqs]
            pos = [0] * len(seqs)
            while True:
                live = [i for i in range(len(seqs)) if pos[i] < len(seqs[i])]
                if not live:
                    break
                toks = [seqs[i][pos[i]:pos[i] + int(rng.integers(1, 60))] for i in live]
                got = eng.step([slots[i] for i in live], toks, "all")
                mh.assert_logits(got, np.concatenate([want[i][pos[i]:pos[i] + len(t)] for i, t in zip(live, toks)]), dtype,
                                 f"{dtype}, chunks from {pos}; {what}")
                r = 0
                for i, t in zip(live, toks):
                    at = first_row[i] + pos[i]
                    assert not exact or torch.equal(got[r:r + len(t)], whole[at:at + len(t)]), \
                        f"float32 bits of a chunk of {len(t)} at position {pos[i]} of sequence {i} differ from the whole prompt; {what}"
                    r += len(t)
                    pos[i] += len(t)
            for s in slots:
                eng.release(s)
            eng.check_status()
