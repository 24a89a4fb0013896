"""The command line's option surface and its errors, as the reference tests its own
(rustml/nlp/tests/infer_cli.rs:15-80): help lists every option; bad input is an error message."""
import io

import pytest

from rust_deeplearning_b200 import cli


def test_help_lists_every_option(capsys):
    with pytest.raises(SystemExit) as e:
        cli.main(["--help"])
    assert e.value.code == 0
    out = capsys.readouterr().out
    for opt in ("MODEL_DIR", "--prompt", "--prompt-ids", "--prompt-file", "--max-tokens", "--temperature", "--top-k",
                "--top-p", "--repetition-penalty", "--stream", "--seed", "--dtype", "--stop-ids", "--max-context",
                "--random-config", "--weights-seed", "--timings"):
        assert opt in out, opt
    assert "(0.0 = greedy)" in out
    p = cli.build_parser()
    assert p.get_default("max_tokens") == 256 and p.get_default("temperature") == 0.8     # infer.rs:23-28


def test_prompts():
    p = cli.build_parser()
    assert cli.read_prompts(p.parse_args(["m", "--prompt-ids", "1, 2,3 4"]), io.StringIO()) == [[1, 2, 3, 4]]
    assert cli.read_prompts(p.parse_args(["m", "--prompt", "hé"]), io.StringIO()) == [[104, 195, 169]]
    assert cli.read_prompts(p.parse_args(["m"]), io.StringIO("ab\n")) == [[97, 98, 10]]
    with pytest.raises(SystemExit) as e:
        cli.read_prompts(p.parse_args(["m"]), io.StringIO("  \n"))
    assert "No prompt provided" in str(e.value)
    with pytest.raises(SystemExit):
        cli.read_prompts(p.parse_args(["m", "--prompt-ids", "1,x"]), io.StringIO())
    with pytest.raises(SystemExit):
        cli.read_prompts(p.parse_args(["m", "--prompt", "a", "--prompt-ids", "1"]), io.StringIO())


def test_prompt_file(tmp_path):
    f = tmp_path / "prompts.txt"
    f.write_text("1 2 3\n\n7,8\n")
    p = cli.build_parser()
    assert cli.read_prompts(p.parse_args(["m", "--prompt-file", str(f)]), io.StringIO()) == [[1, 2, 3], [7, 8]]
    with pytest.raises(SystemExit):
        cli.read_prompts(p.parse_args(["m", "--prompt-file", str(tmp_path / "none")]), io.StringIO())


def test_a_bad_model_folder_is_an_error_message(tmp_path, capsys):
    assert cli.main([str(tmp_path / "nowhere"), "--prompt-ids", "1"]) == 1
    assert "error:" in capsys.readouterr().err


def test_model_dir_or_random_config_exactly_one(tmp_path, capsys):
    with pytest.raises(SystemExit) as e:
        cli.main(["--prompt-ids", "1"])
    assert "MODEL_DIR or --random-config" in str(e.value)
    with pytest.raises(SystemExit):
        cli.main([str(tmp_path), "--random-config", str(tmp_path / "c.json"), "--prompt-ids", "1"])
    assert cli.main(["--random-config", str(tmp_path / "missing.json"), "--prompt-ids", "1"]) == 1
    assert "error:" in capsys.readouterr().err
