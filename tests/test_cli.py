"""The command line: the part that needs no GPU, and generation through it on one."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

import plain_model

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, "-m", "dryft_flash_infer_b200", *args], cwd=ROOT, capture_output=True, text=True)


def test_random_model_writes_a_loadable_folder(tmp_path):
    from dryft_flash_infer_b200.config import load_config
    from dryft_flash_infer_b200.weights import ModelFiles

    (tmp_path / "c.json").write_text(json.dumps(plain_model.TINY_A))
    done = run("random-model", "--config", str(tmp_path / "c.json"), "--seed", "3", "--out", str(tmp_path / "m"))
    assert done.returncode == 0, done.stderr
    assert load_config(tmp_path / "m").hidden_size == 64
    assert "model.layers.1.mlp.down_proj.weight" in ModelFiles(tmp_path / "m").names()


@pytest.mark.gpu
def test_generate_prints_one_line_per_step(tmp_path):
    (tmp_path / "c.json").write_text(json.dumps(plain_model.TINY_B))
    assert run("random-model", "--config", str(tmp_path / "c.json"), "--out", str(tmp_path / "m")).returncode == 0
    (tmp_path / "p.json").write_text(json.dumps([[1, 2, 3], [4, 5, 6, 7, 8]]))
    done = run("generate", "--model", str(tmp_path / "m"), "--prompt-ids", str(tmp_path / "p.json"),
               "--max-new-tokens", "5", "--temperature", "0.7", "--seed", "2")
    assert done.returncode == 0, done.stderr
    lines = [json.loads(l) for l in done.stdout.strip().splitlines()]
    assert len(lines) == 6 and all(len(row) == 2 for row in lines[:5]) and lines[5]["steps"] == 5
    again = run("generate", "--model", str(tmp_path / "m"), "--prompt-ids", str(tmp_path / "p.json"),
                "--max-new-tokens", "5", "--temperature", "0.7", "--seed", "2", "--cuda-graph", "off")
    assert [json.loads(l) for l in again.stdout.strip().splitlines()][:5] == lines[:5]


@pytest.mark.gpu
def test_generate_from_a_configuration_alone(tmp_path):
    """``--random-config``: a model of random weights without a folder on disk; the same seed, the same tokens."""
    (tmp_path / "c.json").write_text(json.dumps(plain_model.TINY_A))
    args = ("generate", "--random-config", str(tmp_path / "c.json"), "--random-prompts", "3:9", "--max-new-tokens", "4",
            "--seed", "7", "--dtype", "float32")
    first, second = run(*args), run(*args)
    assert first.returncode == 0, first.stderr
    rows = [json.loads(l) for l in first.stdout.strip().splitlines()]
    assert len(rows) == 5 and all(len(r) == 3 for r in rows[:4]) and first.stdout == second.stdout.replace(
        second.stdout.strip().splitlines()[-1], first.stdout.strip().splitlines()[-1])
    both = run("generate", "--random-config", str(tmp_path / "c.json"), "--model", str(tmp_path), "--random-prompts", "1:2",
               "--max-new-tokens", "1")
    assert both.returncode != 0 and "either" in both.stderr


def bench(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, capture_output=True, text=True)


def test_bench_measures_one_gpu_only_and_says_so():
    done = bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert done.returncode == 2
    lines = done.stdout.strip().splitlines()
    assert len(lines) == 1 and "--gpus 2" in lines[0]


def test_bench_reference_arm_without_a_gpu_says_why_in_one_line():
    """On a machine without a CUDA device neither arm can run; the reference arm then prints its
    one-line reason and exits 0 (with a device it runs the reference, which takes minutes: not here)."""
    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("with a CUDA device the arm runs the reference itself")
    done = bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "\n" not in line["unavailable"]
