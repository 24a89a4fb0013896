"""Parts that are not the library's, defined and registered here, built and stepped without a change
to the package: a mixer with per-sequence state of fixed size, a feed-forward with routing, another
position encoding, a norm of another kind; and a schedule that names a layer twice and lets a run
read another run's keys and values.  The toy model is compared with a plain whole-sequence
restatement written below; it is nobody's architecture."""

import numpy as np
import pytest
import torch

from rust_deeplearning_b200 import Engine
from rust_deeplearning_b200.cache.cache import StateRequirement
from rust_deeplearning_b200.config.base import Architecture, register_architecture
from rust_deeplearning_b200.parts.model import Model
from rust_deeplearning_b200.parts.registry import register_part, registered_parts
from rust_deeplearning_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
from rust_deeplearning_b200.weights.loader import random_weights

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
H, V, NH, NKV, HD, DECAY = 48, 97, 4, 2, 16, 0.75


# ---- toy parts (torch on the device; rows of a step are visited sequence by sequence) ----

class DecayMixer:
    """s_t = decay * s_{t-1} + x_t ; y_t = s_t W.  The state s lives in the cache, one row per sequence."""

    def __init__(self, spec, ctx):
        self.w = ctx.tensor(spec.tensors["w"])
        self.decay = spec.params["decay"]

    def needs(self):
        return None, StateRequirement((H,), "float32")

    def forward(self, x, batch, cache, run):
        starts, slots = batch.seq_start.tolist(), batch.slots.tolist()
        out = torch.empty_like(x)
        for i in range(batch.real_seqs):
            s = cache.state[slots[i]]
            for r in range(starts[i], starts[i + 1]):
                s.mul_(self.decay).add_(x[r].float())
                out[r] = (s @ self.w.float().t()).to(x.dtype)
        return out


class RoutedFF:
    """Two experts, each a matrix; a row goes to the expert whose router score is larger, scaled by the score."""

    def __init__(self, spec, ctx):
        self.router, self.e0, self.e1 = (ctx.tensor(spec.tensors[k]).float() for k in ("router", "e0", "e1"))

    def forward(self, x):
        xf = x.float()
        score = xf @ self.router.t()                      # [rows, 2]
        pick = score[:, 1] > score[:, 0]
        y = torch.where(pick[:, None], xf @ self.e1.t(), xf @ self.e0.t()) * torch.sigmoid(score.max(dim=1).values)[:, None]
        return y.to(x.dtype)


class AddedSinusoid:
    """Another position encoding: adds sin(pos * f_i) to every query and key head."""

    def __init__(self, spec, ctx):
        self.freq = torch.tensor([spec.params["base"] ** -(i / HD) for i in range(HD)], dtype=torch.float32, device=ctx.device)

    def rotate(self, rows, n_heads, n_kv_heads, head_dim, batch):
        T = rows.shape[0]
        enc = torch.sin(batch.tok_pos[:T].float()[:, None] * self.freq[None, :])
        view = rows.view(T, -1, head_dim)
        view[:, :n_heads + n_kv_heads] = (view[:, :n_heads + n_kv_heads].float() + enc[:, None, :]).to(rows.dtype)


class MeanShiftNorm:
    def __init__(self, spec, ctx):
        self.w = ctx.tensor(spec.tensors["weight"]).float()

    def apply(self, x, out_dtype):
        xf = x.float()
        return ((xf - xf.mean(-1, keepdim=True)) * (1 + self.w)).to(out_dtype)


def register_toys():
    for role, kind, cls in (("mixer", "toy_decay", DecayMixer), ("feed_forward", "toy_routed", RoutedFF),
                            ("position", "toy_added_sinusoid", AddedSinusoid), ("norm", "toy_mean_shift", MeanShiftNorm)):
        register_part(role, kind, lambda spec, ctx, cls=cls: cls(spec, ctx), replace=True)


def toy_spec() -> ModelSpec:
    rms = lambda n: PartSpec("rms_norm", {"size": H, "eps": 1e-5, "offset": 1.0}, {"weight": TensorSpec(n, (H,), "vector")})
    shift = lambda n: PartSpec("toy_mean_shift", {}, {"weight": TensorSpec(n, (H,), "vector")})
    attention = PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD,
                                       "score_scale": 0.25, "softcap": None, "window": 6,
                                       "position": PartSpec("toy_added_sinusoid", {"base": 50.0})},
                         {r: TensorSpec(f"l0.{r}", s) for r, s in (("q", (NH * HD, H)), ("k", (NKV * HD, H)),
                                                                    ("v", (NKV * HD, H)), ("o", (H, NH * HD)))})
    mlp = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 64, "activation": "silu"},
                   {"gate": TensorSpec("l0.gate", (64, H)), "up": TensorSpec("l0.up", (64, H)), "down": TensorSpec("l0.down", (H, 64))})
    layer0 = LayerSpec("sandwich", attention, mlp, {"pre_mixer": rms("l0.n1"), "post_mixer": shift("l0.n2"),
                                                     "pre_feed_forward": rms("l0.n3")})
    decay = PartSpec("toy_decay", {"decay": DECAY}, {"w": TensorSpec("l1.w", (H, H), init_std=0.1)})
    routed = PartSpec("toy_routed", {}, {"router": TensorSpec("l1.router", (2, H), init_std=0.5),
                                         "e0": TensorSpec("l1.e0", (H, H), init_std=0.1), "e1": TensorSpec("l1.e1", (H, H), init_std=0.1)})
    layer1 = LayerSpec("sandwich", decay, routed, {"pre_mixer": shift("l1.n1"), "pre_feed_forward": rms("l1.n3"),
                                                    "post_feed_forward": rms("l1.n4")})
    table = TensorSpec("embed", (V, H), init_std=0.5)
    # layer 0, layer 1, layer 0 again (its own cache), layer 1 again (its own state), layer 0 reading run 0's keys
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, reads_cache_of=0))
    return ModelSpec("ToyForTests", H, V, 256, PartSpec("scaled_embedding", {"scale": 1.0}, {"table": table}),
                     (layer0, layer1), schedule, rms("final"), PartSpec("linear_head", {"softcap": None}, {"weight": table}))


# ---- the same model, plainly, on whole sequences ----

def plain_forward(w, ids):
    f = lambda n: w[n].double().cpu().numpy()
    rms = lambda x, n, eps=1e-5: x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * (1 + f(n))
    shift = lambda x, n: (x - x.mean(-1, keepdims=True)) * (1 + f(n))
    T = len(ids)
    pos = np.arange(T)
    enc = np.sin(pos[:, None] * np.array([50.0 ** -(i / HD) for i in range(HD)], dtype=np.float32).astype(np.float64)[None, :])

    def project(n):
        q = (n @ f("l0.q").T).reshape(T, NH, HD) + enc[:, None]
        k = (n @ f("l0.k").T).reshape(T, NKV, HD) + enc[:, None]
        v = (n @ f("l0.v").T).reshape(T, NKV, HD)
        return q, k, v

    def attend(q, k, v):
        out = np.zeros((T, NH, HD))
        keep = (pos[None, :] <= pos[:, None]) & (pos[:, None] - pos[None, :] < 6)
        for h in range(NH):
            s = np.where(keep, q[:, h] @ k[:, h // 2].T * 0.25, -np.inf)
            a = np.exp(s - s.max(-1, keepdims=True))
            out[:, h] = (a / a.sum(-1, keepdims=True)) @ v[:, h // 2]
        return out.reshape(T, NH * HD) @ f("l0.o").T

    def layer0(x, shared=None):
        q, k, v = project(rms(x, "l0.n1"))
        if shared is not None:
            k, v = shared
        h = x + shift(attend(q, k, v), "l0.n2")
        n = rms(h, "l0.n3")
        g, u = n @ f("l0.gate").T, n @ f("l0.up").T
        return h + (g / (1 + np.exp(-g)) * u) @ f("l0.down").T, (k, v)

    def layer1(x):
        n = shift(x, "l1.n1")
        s, ys = np.zeros(H), []
        for t in range(T):
            s = DECAY * s + n[t]
            ys.append(s @ f("l1.w").T)
        h = x + np.stack(ys)
        n = rms(h, "l1.n3")
        score = n @ f("l1.router").T
        pick = score[:, 1] > score[:, 0]
        y = np.where(pick[:, None], n @ f("l1.e1").T, n @ f("l1.e0").T) / (1 + np.exp(-score.max(1)))[:, None]
        return h + rms(y, "l1.n4")

    x = f("embed")[ids]
    x, kv0 = layer0(x)
    x = layer1(x)
    x, _ = layer0(x)
    x = layer1(x)
    x, _ = layer0(x, shared=kv0)
    return rms(x, "final") @ f("embed").T


@pytest.fixture(scope="module")
def toy():
    register_toys()
    spec = toy_spec()
    weights = random_weights(spec, 3, torch.float32, DEV)
    kept = {n: t.clone() for n, t in weights.items()}
    return Model(spec, weights, torch.float32, DEV), kept


def check(got, want, what):
    got = got.double().cpu().numpy()
    assert got.shape == want.shape and np.isfinite(got).all()
    err, scale = np.abs(got - want).max(), np.abs(want).max()
    assert err <= 1e-4 * max(1.0, scale), f"{what}: {err:.3e} (scale {scale:.2f})"


def test_toy_parts_are_registered_from_outside():
    register_toys()
    assert "toy_decay" in registered_parts("mixer") and "toy_routed" in registered_parts("feed_forward")
    assert "toy_added_sinusoid" in registered_parts("position") and "toy_mean_shift" in registered_parts("norm")
    register_architecture(Architecture("ToyForTests", "toy", lambda raw: raw, lambda cfg: toy_spec()), replace=True)


def test_cache_gives_each_run_what_it_declares(toy):
    model, _ = toy
    needs = model.needs()
    assert [n.kv is not None for n in needs] == [True, False, True, False, True]
    assert [n.state is not None for n in needs] == [False, True, False, True, False]
    assert needs[4].reads_cache_of == 0
    eng = Engine(model, max_tokens=512, max_seqs=4, use_graphs=False)
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].runs == [0, 2]          # two runs of one layer, storage each
    assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].runs == [1, 3]
    assert tuple(eng.cache.run_cache(1).state.shape) == (4, H)
    assert eng.cache.run_cache(4).k.data_ptr() == eng.cache.run_cache(0).k.data_ptr()


def test_toy_model_whole_and_token_by_token(toy):
    model, w = toy
    eng = Engine(model, max_tokens=512, max_seqs=4, use_graphs=False)
    rng = np.random.default_rng(0)
    ids = [int(v) for v in rng.integers(0, V, size=90)]
    want = plain_forward(w, ids)
    a = eng.new_sequence()
    check(eng.step([a], [ids], "all"), want, "whole")
    b = eng.new_sequence()
    check(eng.step([b], [ids[:70]], "all"), want[:70], "prefix")
    for t in range(70, 90):                                 # state and keys carried from step to step
        check(eng.step([b], [[ids[t]]], "all"), want[t:t + 1], f"position {t}")
    eng.release(a); eng.release(b)
    c = eng.new_sequence()                                  # the slot's state was reset, its pages are stale
    assert c in (a, b)
    check(eng.step([c], [ids[:40]], "all"), want[:40], "reused slot")
    check(eng.step([c], [ids[40:75]], "all"), want[40:75], "a second chunk on state and cache")


def test_toy_model_in_unequal_batches(toy):
    model, w = toy
    eng = Engine(model, max_tokens=512, max_seqs=3, use_graphs=False)
    rng = np.random.default_rng(1)
    for round_ in range(2):
        seqs = [[int(v) for v in rng.integers(0, V, size=n)] for n in (31, 8, 19)]
        lens = [20, 1, 12]
        want = [plain_forward(w, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        check(eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], "all"),
              np.concatenate([x[:n] for x, n in zip(want, lens)]), "prompts")
        pos, live = list(lens), [0, 1, 2]
        while live:
            got = eng.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live], "last")
            check(got, np.stack([want[i][pos[i]] for i in live]), f"decode {pos}")
            for i in live:
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(seqs[i])]:
                eng.release(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]


def test_toy_model_in_bfloat16_single_tokens():
    """The same model in bfloat16, where steps of few rows may carry their norms in the products (parts/norm.py): here
    the attention and the gated feed-forward offer that, the toy parts do not, one post-norm is of a kind that cannot
    take part and one branch has no post-norm at all - every combination must fall back to the same numbers."""
    register_toys()
    spec = toy_spec()
    weights = random_weights(spec, 3, torch.bfloat16, DEV)
    kept = {n: t.clone() for n, t in weights.items()}
    eng = Engine(Model(spec, weights, torch.bfloat16, DEV), max_tokens=512, max_seqs=4, use_graphs=False)
    rng = np.random.default_rng(2)
    seqs = [[int(v) for v in rng.integers(0, V, size=n)] for n in (40, 23, 31)]
    want = [plain_forward(kept, s) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    cut = [len(s) - 8 for s in seqs]
    got = eng.step(slots, [s[:c] for s, c in zip(seqs, cut)], "last").double().cpu().numpy()
    ref0 = np.stack([w[c - 1] for w, c in zip(want, cut)])
    scale = max(np.abs(w).max() for w in want)
    assert np.abs(got - ref0).max() <= 0.03 * scale
    for k in range(8):
        got = eng.step(slots, [[s[c + k]] for s, c in zip(seqs, cut)], "last").double().cpu().numpy()
        ref = np.stack([w[c + k] for w, c in zip(want, cut)])
        assert np.isfinite(got).all() and np.abs(got - ref).max() <= 0.03 * scale, (k, np.abs(got - ref).max(), scale)
