"""bin/trace_run driven as a user drives it: steps on standard input, logits in files.  The same
requests are replayed whole, with the last 32 tokens one by one, and in batches of unequal lengths
whose shorter requests end earlier (one batch after another on a cache that only holds one batch,
so slots and pages are used again); every written position is compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import model_helpers as mh
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(name, dtype, steps, max_tokens, out_dir):
    """Feed `steps` one at a time, waiting for `done <step>` after each, as the protocol asks."""
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", mh.model_folder(name), "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    V = tiny_configs.config(name)[0]["vocab_size"]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, V)
        else:
            assert not os.path.exists(path)
    return out


def check(name, dtype, steps, outputs, seqs):
    """Every wanted place of every step against the plain logits of its request at its position."""
    pos = {rid: 0 for rid in seqs}
    for s in steps:
        rows = []
        for e in s["entries"]:
            want = mh.plain_logits(name, seqs[e["id"]])
            rows += [want[pos[e["id"]] + w] for w in e.get("want", [])]
            pos[e["id"]] += len(e["tokens"])
        if rows:
            got = outputs[s["step"]]
            tol = mh.tolerance(dtype, np.stack(rows))
            err = np.abs(got.astype(np.float64) - np.stack(rows)).max(axis=1)
            assert np.isfinite(got).all()
            assert err.max() <= tol, f"step {s['step']}: error {err.max():.3e} > {tol:.3e}, first bad row {int(np.argmax(err > tol))}"


def requests(name):
    V = tiny_configs.config(name)[0]["vocab_size"]
    lens = {"a": 70, "b": 33, "c": 101, "d": 40, "e": 65}
    return {rid: mh.prompt(500 + i, n, V) for i, (rid, n) in enumerate(lens.items())}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_whole_then_last_32_one_by_one(tmp_path, name, dtype):
    seqs = requests(name)
    steps, k = [], 0
    for rid, ids in seqs.items():                    # each request alone and whole
        steps.append({"step": k, "entries": [{"id": rid + "w", "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [rid + "w"]})
        k += 1
    for rid, ids in seqs.items():                    # each request alone, the last 32 tokens one by one
        cut = len(ids) - 32
        steps.append({"step": k, "entries": [{"id": rid, "tokens": ids[:cut], "want": [0, cut - 1]}], "end": []})
        k += 1
        for t in range(cut, len(ids)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [ids[t]], "want": [0]}],
                          "end": [rid] if t == len(ids) - 1 else []})
            k += 1
    all_seqs = dict(seqs)
    all_seqs.update({rid + "w": ids for rid, ids in seqs.items()})
    out = replay(name, dtype, steps, max_tokens=128, out_dir=str(tmp_path))   # one request of 101 tokens at a time
    check(name, dtype, steps, out, all_seqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_unequal_batches_one_after_another(tmp_path, name, dtype):
    seqs = requests(name)
    prompt_len = {"a": 50, "b": 1, "c": 90, "d": 17, "e": 64}
    steps, k = [], 0
    for members in (["a", "b", "c"], ["d", "e"], ["c", "a", "e", "b"][:3], ["b", "d"]):
        ids = {m: seqs[m] for m in members}
        pos = {m: prompt_len[m] for m in members}
        ending = [m for m in members if pos[m] == len(ids[m])]
        steps.append({"step": k, "entries": [{"id": f"{m}{k}", "tokens": ids[m][:pos[m]], "want": [pos[m] - 1]}
                                             for m in members], "end": [f"{m}{k}" for m in ending]})
        names = {m: f"{m}{k}" for m in members}
        k += 1
        live = [m for m in members if m not in ending]
        while live:
            ending = [m for m in live if pos[m] + 1 == len(ids[m])]
            steps.append({"step": k, "entries": [{"id": names[m], "tokens": [ids[m][pos[m]]],
                                                  "want": [0] if (pos[m] % 3 or m in ending) else []} for m in live],
                          "end": [names[m] for m in ending]})
            k += 1
            for m in live:
                pos[m] += 1
            live = [m for m in live if m not in ending]
        for m in members:
            seqs[names[m]] = ids[m]
    # the largest batch holds 128 + 64 + 128 positions (rounded up to 64): the cache fits one batch only
    out = replay(name, dtype, steps, max_tokens=320, out_dir=str(tmp_path))
    check(name, dtype, steps, out, seqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_portions_and_mixed_steps(tmp_path, name, dtype):
    """Steps the generation loop never forms but the step function takes: a request fed in portions of many
    tokens (7 / 23 / 15, then 70 / 60 for another) and steps that mix a portion or a whole prompt with
    single tokens of requests under way."""
    V = tiny_configs.config(name)[0]["vocab_size"]
    seqs = {"p": mh.prompt(600, 45, V), "q": mh.prompt(601, 130, V), "r": mh.prompt(602, 12, V), "s": mh.prompt(603, 20, V)}
    all_of = lambda rid, a, b: {"id": rid, "tokens": seqs[rid][a:b], "want": list(range(b - a))}
    steps = [
        {"step": 0, "entries": [all_of("p", 0, 7)], "end": []},
        {"step": 1, "entries": [all_of("p", 7, 30), all_of("q", 0, 70)], "end": []},               # a portion beside a prompt
        {"step": 2, "entries": [all_of("p", 30, 45), all_of("q", 70, 130), all_of("r", 0, 11)], "end": ["p", "q"]},
        {"step": 3, "entries": [all_of("r", 11, 12), all_of("s", 0, 19)], "end": ["r"]},           # one token beside a prompt
        {"step": 4, "entries": [all_of("s", 19, 20)], "end": ["s"]},
    ]
    out = replay(name, dtype, steps, max_tokens=384, out_dir=str(tmp_path))
    check(name, dtype, steps, out, seqs)


@pytest.mark.parametrize("case,name,dtype", [(0, "A", "float32"), (1, "B", "bfloat16"), (2, "D", "bfloat16"), (3, "E", "float32")])
def test_replay_of_a_trace_drawn_at_random_with_the_cache_at_its_bound(tmp_path, case, name, dtype):
    """One to four batches of one to five requests of 1 to 149 tokens, prompts cut anywhere, requests ended
    anywhere (also before their last token), logits wanted at random places - and --max-tokens set to exactly
    what the protocol promises: the most that live requests hold at any time, each rounded up to 64."""
    rng = np.random.default_rng(case)
    V = tiny_configs.config(name)[0]["vocab_size"]
    seqs, steps, most = {}, [], 0
    held = lambda lengths: sum(-(-n // 64) * 64 for n in lengths)
    for batch in range(int(rng.integers(1, 5))):
        members = [f"b{batch}r{i}" for i in range(int(rng.integers(1, 6)))]
        for m in members:
            seqs[m] = mh.prompt(int(rng.integers(0, 1 << 30)), int(rng.integers(1, 150)), V)
        pos = {m: int(rng.integers(1, len(seqs[m]) + 1)) for m in members}
        stop_at = {m: int(rng.integers(pos[m], len(seqs[m]) + 1)) for m in members}
        ending = [m for m in members if pos[m] >= stop_at[m]]
        steps.append({"step": len(steps), "end": list(ending), "entries": [
            {"id": m, "tokens": seqs[m][:pos[m]], "want": sorted(set(int(v) for v in rng.integers(0, pos[m], size=int(rng.integers(0, 4)))))}
            for m in members]})
        most = max(most, held(pos[m] for m in members))
        live = [m for m in members if m not in ending]
        while live:
            for m in live:
                pos[m] += 1
            most = max(most, held(pos[m] for m in live))
            ending = [m for m in live if pos[m] >= stop_at[m]]
            steps.append({"step": len(steps), "end": list(ending), "entries": [
                {"id": m, "tokens": [seqs[m][pos[m] - 1]], "want": [0] if rng.integers(0, 3) else []} for m in live]})
            live = [m for m in live if m not in ending]
    out = replay(name, dtype, steps, max_tokens=most, out_dir=str(tmp_path))
    check(name, dtype, steps, out, seqs)


def test_a_step_the_engine_refuses_ends_the_replay_with_a_message(tmp_path):
    """More tokens than --max-tokens promised, an id outside the vocabulary, a line that is no JSON: `done` for the
    steps before, one line on standard error, exit code 1, no file for the refused step."""
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []}]
    for bad in ({"step": 1, "entries": [{"id": "b", "tokens": list(range(100)), "want": [0]}], "end": []},
                {"step": 1, "entries": [{"id": "a", "tokens": [100000], "want": [0]}], "end": []},
                "this is no step"):
        out_dir = tmp_path / f"out{len(os.listdir(tmp_path))}"
        lines = "".join(json.dumps(s) + "\n" for s in steps) + (bad if isinstance(bad, str) else json.dumps(bad)) + "\n"
        r = subprocess.run([sys.executable, TRACE_RUN, "--model", mh.model_folder("A"), "--dtype", "float32", "--out", str(out_dir),
                            "--max-tokens", "64"], input=lines, capture_output=True, text=True, timeout=300)
        assert r.returncode == 1 and r.stdout.split() == ["done", "0"], (r.stdout, r.stderr)
        assert r.stderr.strip().splitlines()[-1].startswith("error: step") and "Traceback" not in r.stderr, r.stderr
        assert sorted(os.listdir(out_dir)) == ["0.f32"]
