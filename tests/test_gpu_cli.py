"""The command line run as a user runs it: `python -m somi_inference_b200.entrypoints.generate`
in a process of its own, on the GPU, compared with the plain implementation."""

import json
import os
import subprocess
import sys

import pytest
import torch

from tests.plain import qwen2_plain as plain
from tests.tiny import TINY, make_model, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*argv: str) -> list[dict]:
    r = subprocess.run([sys.executable, "-m", "somi_inference_b200.entrypoints.generate", *argv],
                       cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"exit {r.returncode}\n{r.stdout}\n{r.stderr}"
    return [json.loads(line) for line in r.stdout.strip().splitlines() if line.startswith("{")]


def test_generate_from_a_model_folder(tmp_path):
    d = make_model("A", str(tmp_path), torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    prompt = random_tokens(17, cfg["vocab_size"], 3)
    log = tmp_path / "out.jsonl"
    (rec,) = run_cli("--model-name", d, "--prompt-ids", *map(str, prompt), "--max-new-tokens", "8",
                     "--temperature", "0", "--dtype", "float32", "--num-blocks", "16",
                     "--output-file", str(log))
    assert rec["prompt_ids"] == prompt and rec["output_ids"] == plain.greedy(cfg, w, prompt, 8)
    assert json.loads(log.read_text().strip()) == rec
    # several random prompts run together, drawn from --seed
    recs = run_cli("--model-name", d, "--prompt-lens", "5", "17", "33", "--seed", "0",
                   "--max-new-tokens", "8", "--temperature", "0", "--dtype", "float32",
                   "--num-blocks", "16", "--chunk-size", "16")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (5, 17, 33)]
    assert [r["prompt_len"] for r in recs] == [5, 17, 33]
    assert [r["output_ids"] for r in recs] == [plain.greedy(cfg, w, p, 8) for p in prompts]


def test_config_and_seed_in_tokens_out(tmp_path):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["B"]))
    recs = run_cli("--config", str(cfg_path), "--random-weights", "--seed", "1", "--std", "0.08",
                   "--weights-dtype", "float32", "--dtype", "float32", "--prompt-lens", "9", "40",
                   "--max-new-tokens", "6", "--temperature", "0", "--block-size", "8",
                   "--num-blocks", "32")
    d = make_model("B", str(tmp_path), torch.float32, std=0.08)        # the same seed
    cfg, w = plain.load_folder(d)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (9, 40)]
    assert [r["output_ids"] for r in recs] == [plain.greedy(cfg, w, p, 6) for p in prompts]
    # bfloat16 (the default dtype) runs and gives tokens of the vocabulary
    recs = run_cli("--config", str(cfg_path), "--random-weights", "--seed", "1", "--prompt-lens", "9",
                   "--max-new-tokens", "4", "--temperature", "0.8", "--top-k", "20",
                   "--block-size", "8", "--num-blocks", "32")
    assert len(recs[0]["output_ids"]) == 4
    assert all(0 <= t < cfg["vocab_size"] for t in recs[0]["output_ids"])
