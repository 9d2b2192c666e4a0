"""The command line programs on the CPU: what needs no device (option parsing, a model folder that is not there,
a model folder written and inspected), and that a user's mistake is answered in one line, not with a stack trace."""
import json
import subprocess
import sys
from pathlib import Path

import tiny

ROOT = Path(__file__).resolve().parent.parent


def run(*argv, stdin=""):
    return subprocess.run([sys.executable, *map(str, argv)], input=stdin, capture_output=True, text=True, timeout=600)


def test_trace_run_answers_a_missing_model_in_one_line(tmp_path):
    p = run(ROOT / "bin" / "trace_run", "--model", tmp_path / "nope", "--dtype", "float32", "--out", tmp_path / "o",
            "--max-tokens", "64")
    assert p.returncode == 1
    # with a device: the folder is missing; without: there is no device.  Either way one line and no trace.
    assert p.stderr.startswith("trace_run: error: ") and "Traceback" not in p.stderr
    assert "no such file" in p.stderr or "no CUDA device" in p.stderr
    assert p.stdout == ""


def test_trace_run_refuses_an_unknown_dtype(tmp_path):
    p = run(ROOT / "bin" / "trace_run", "--model", tmp_path, "--dtype", "float16", "--out", tmp_path / "o",
            "--max-tokens", "64")
    assert p.returncode == 2 and "invalid choice" in p.stderr


def test_random_model_and_inspect(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(tiny.CONFIG_B))
    p = run(ROOT / "bin" / "flambeau", "random-model", "--config", cfg, "--out", tmp_path / "m", "--seed", "4")
    assert p.returncode == 0, p.stderr
    assert (tmp_path / "m" / "config.json").exists() and (tmp_path / "m" / "model.safetensors").exists()
    p = run(ROOT / "bin" / "flambeau", "inspect", "--model", tmp_path / "m")
    assert p.returncode == 0, p.stderr
    assert "MistralForCausalLM" in p.stdout and "model.layers.2.self_attn.q_proj.weight" in p.stdout


def test_flambeau_answers_mistakes_in_one_line(tmp_path):
    p = run(ROOT / "bin" / "flambeau", "inspect", "--model", tmp_path / "nope")
    assert p.returncode == 1 and p.stderr.startswith("flambeau inspect: error:") and "Traceback" not in p.stderr
    bad = dict(tiny.CONFIG_A, hidden_act="gelu")
    (tmp_path / "config.json").write_text(json.dumps(bad))
    p = run(ROOT / "bin" / "flambeau", "random-model", "--config", tmp_path / "config.json", "--out", tmp_path / "m")
    assert p.returncode == 1 and "hidden_act" in p.stderr and "Traceback" not in p.stderr


def test_bench_subcommand_keeps_the_contract_for_more_than_one_gpu(capsys):
    """`flambeau bench` is bench.py: for more than one GPU it says so in one line and exits with 2; the reference
    arm answers with its `unavailable` line."""
    import json
    from flambeau_b200.cli import main
    assert main(["bench", "--gpus", "4"]) == 2
    out = capsys.readouterr().out.strip().splitlines()
    assert len(out) == 1 and "one GPU" in out[0]
    assert main(["bench", "--impl", "reference"]) == 0
    line = json.loads(capsys.readouterr().out)
    assert line["impl"] == "reference" and "unavailable" in line
