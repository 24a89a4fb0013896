"""The command line as a process: `bin/rustml-infer MODEL_DIR ...` prints the tokens that the Python
entry point and the plain implementation give (greedy), streams them one a line, and honours
--max-tokens and --stop-ids.  (The reference's own command-line tests run the built binary in the same
way: rustml/nlp/tests/infer_cli.rs:15-80.)"""
import os
import subprocess
import sys

import pytest

import model_helpers as mh
import plain_gemma2 as plain
import tiny_configs

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INFER = os.path.join(ROOT, "bin", "rustml-infer")


def run(args, stdin=None):
    r = subprocess.run([sys.executable, INFER, *args], input=stdin, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    return r.stdout, r.stderr


def test_greedy_tokens_equal_the_entry_point_and_the_plain_implementation(tmp_path):
    from rust_deeplearning_b200 import Generator
    name = "A"
    cfg, w = mh.plain_model(name)
    V = tiny_configs.config(name)[0]["vocab_size"]
    folder = mh.model_folder(name)
    prompts = [mh.prompt(500 + i, n, V) for i, n in enumerate((6, 13))]
    stops = cfg["eos_token_id"] if isinstance(cfg["eos_token_id"], list) else [cfg["eos_token_id"]]
    want = [plain.generate_greedy(cfg, w, p, 6, frozenset(stops)) for p in prompts]

    # one prompt on the command line: the completion on one line
    out, err = run([folder, "--prompt-ids", ",".join(map(str, prompts[0])), "--max-tokens", "6", "--temperature", "0",
                    "--dtype", "float32", "--max-context", "128"])
    assert [int(t) for t in out.split()] == want[0]
    assert "finished by" in err

    # a file of prompts: one line of tokens for each, in order; the same as the Python entry point
    f = tmp_path / "prompts.txt"
    f.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    out, _ = run([folder, "--prompt-file", str(f), "--max-tokens", "6", "--temperature", "0", "--dtype", "float32",
                  "--max-context", "128"])
    got = [[int(t) for t in line.split()] for line in out.strip().split("\n")]
    assert got == want
    gen = Generator(mh.loaded_model(name, "float32"), max_batch=4, max_context=128).with_temperature(0.0)
    assert [r.tokens for r in gen.generate_batch_results(prompts, 6)] == got

    # --stream prints a token a line as it is made; --stop-ids ends a request at its first stop token
    out, _ = run([folder, "--prompt-ids", " ".join(map(str, prompts[0])), "--max-tokens", "6", "--temperature", "0",
                  "--dtype", "float32", "--max-context", "128", "--stream"])
    assert [int(t) for t in out.split()] == want[0]
    if len(want[0]) >= 3:
        stop = want[0][2]
        out, _ = run([folder, "--prompt-ids", " ".join(map(str, prompts[0])), "--max-tokens", "6", "--temperature", "0",
                      "--dtype", "float32", "--max-context", "128", "--stop-ids", str(stop)])
        first = want[0].index(stop)
        assert [int(t) for t in out.split()] == want[0][:first]


def test_seeded_sampling_is_reproducible_in_bfloat16():
    folder = mh.model_folder("B")
    args = [folder, "--prompt-ids", "3 1 4 1 5", "--max-tokens", "10", "--temperature", "0.9", "--top-k", "20", "--top-p", "0.9",
            "--repetition-penalty", "1.1", "--seed", "11", "--max-context", "128", "--stop-ids", ""]
    a, _ = run(args)
    b, _ = run(args)
    assert a == b and len(a.split()) == 10
    c, _ = run(args[:-4] + ["--seed", "12", "--max-context", "128", "--stop-ids", ""])
    assert c != a


@pytest.mark.parametrize("args,needle", [
    (["--prompt-ids", "3 100000"], "vocabulary"),                       # an id outside the vocabulary
    (["--prompt-ids", "1 2 3 4 5 6", "--max-context", "4"], "context"),   # a prompt longer than the context asked for
    (["--prompt-ids", "1 2", "--temperature", "-1"], "temperature"),
    (["--prompt-ids", "1 2", "--top-k", "0"], "top_k"),
    (["--prompt-ids", "1 2", "--repetition-penalty", "0"], "repetition_penalty"),
])
def test_a_wrong_number_is_one_line_on_standard_error(args, needle):
    r = subprocess.run([sys.executable, INFER, mh.model_folder("A"), "--max-tokens", "3", "--dtype", "float32", *args],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and r.stdout == ""
    last = r.stderr.strip().splitlines()[-1]
    assert last.startswith("error:") and needle in last, r.stderr
    assert "Traceback" not in r.stderr
