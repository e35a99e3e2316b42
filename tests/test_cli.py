"""The command line's parsing and the sub-commands that need no GPU."""
import json
import os
import subprocess
import sys

import pytest

from ghost_infer_b200 import cli
from conftest import TINY_A

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = [sys.executable, os.path.join(ROOT, "bin", "ghost-infer")]


def test_option_names_and_defaults_are_the_reference_s():
    o = cli.parse_opts(["m"])
    assert (o.max_new, o.temp, o.top_k, o.top_p, o.prompt_len) == (256, 0.7, 40, 0.9, 256)     # src/main.rs:120-150
    o = cli.parse_opts(["m", "-p", "1,2", "-n", "5", "-t", "0", "--top-k", "3", "--top-p", "0.5", "--seed", "9",
                        "--ctx", "64", "--prompt-len", "7", "--gpu", "--batch", "2", "--dtype", "float32"])
    assert (o.prompt, o.max_new, o.temp, o.top_k, o.top_p, o.seed, o.ctx, o.prompt_len, o.batch, o.dtype) == \
        ("1,2", 5, 0.0, 3, 0.5, 9, 64, 7, 2, "float32")
    o = cli.parse_opts(["m", "--prompt", "4", "--max", "8", "--temp", "1.5"])
    assert (o.prompt, o.max_new, o.temp) == ("4", 8, 1.5)
    with pytest.raises(cli.UsageError, match="unknown option --nope"):
        cli.parse_opts(["m", "--nope"])
    with pytest.raises(cli.UsageError, match="-n needs a value"):
        cli.parse_opts(["m", "-n"])
    with pytest.raises(cli.UsageError, match="is not a number"):
        cli.parse_opts(["m", "-t", "warm"])
    with pytest.raises(cli.UsageError, match="missing model path"):
        cli.parse_opts([])


def test_prompts_are_token_ids():
    assert cli.parse_ids("1,2,3") == [[1, 2, 3]]
    assert cli.parse_ids("1 2;3,4 ; 5") == [[1, 2], [3, 4], [5]]
    with pytest.raises(cli.UsageError):
        cli.parse_ids(" ; ")


def test_usage_random_and_inspect(tmp_path):
    p = subprocess.run(EXE, capture_output=True, text=True)
    assert p.returncode == 2 and "USAGE:" in p.stderr and "--top-k" in p.stderr
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    p = subprocess.run(EXE + ["random", str(cfg), str(out), "--seed", "3", "--dtype", "float32"], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    p = subprocess.run(EXE + ["inspect", str(out)], capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "21 tensors" in p.stdout and "hidden_size" in p.stdout and "F32" in p.stdout
    assert "model.embed_tokens.weight" in p.stdout
    p = subprocess.run(EXE + ["inspect", str(tmp_path / "nowhere")], capture_output=True, text=True)
    assert p.returncode == 1 and p.stderr.startswith("error:")
