"""The command line (`python -m somi_inference_b200.entrypoints.generate`): its options, the
branch that writes a random model folder, and generation from a folder and from a configuration
plus a seed, run in-process on the CPU with the test-only kernel table.  The same program is run
as a subprocess on the GPU in tests/test_gpu_cli.py."""

import json

import pytest
import torch

from somi_inference_b200.entrypoints import generate
from tests.plain import qwen2_plain as plain
from tests.plain.host_ops import HostOps
from tests.tiny import TINY, make_model, random_tokens


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("cli"))


def test_option_names_and_defaults_follow_the_reference():
    """Names shared with the reference's programs and its `LLM` keep their meaning and defaults
    (benchmarks/bench_decode.py:116-199; somi_inference/entrypoints/llm.py:58-70,126-135)."""
    a = generate.parse_args(["--model-name", "m"])
    assert (a.model_name, a.block_size, a.num_blocks, a.max_concurrent) == ("m", 16, 256, 16)
    assert (a.device, a.dtype, a.seed) == ("auto", "auto", 42)
    assert (a.temperature, a.top_k, a.top_p, a.repetition_penalty) == (1.0, -1, 1.0, 1.0)
    assert a.prompt is None and a.prompt_ids is None and a.prompt_lens is None
    assert a.policy == "preempt" and not a.random_weights and a.output_file is None
    b = generate.parse_args(["--config", "c.json", "--random-weights", "--prompt-lens", "5", "17",
                             "--max-new-tokens", "3", "--dtype", "float32", "--temperature", "0",
                             "--top-k", "7", "--top-p", "0.5", "--repetition-penalty", "1.3",
                             "--chunk-size", "8", "--max-num-batched-tokens", "24",
                             "--policy", "reserve", "--output-file", "o.jsonl"])
    assert b.random_weights and b.config == "c.json" and b.prompt_lens == [5, 17]
    assert (b.max_new_tokens, b.dtype, b.temperature, b.top_k, b.top_p) == (3, "float32", 0.0, 7, 0.5)
    assert (b.repetition_penalty, b.chunk_size, b.max_num_batched_tokens) == (1.3, 8, 24)
    assert b.policy == "reserve" and b.output_file == "o.jsonl"
    with pytest.raises(SystemExit):
        generate.parse_args(["--dtype", "float16"])         # the engine has no float16 path
    with pytest.raises(SystemExit):
        generate.parse_args(["--device", "cpu"])            # nor a CPU path


def test_missing_arguments_are_refused(capsys):
    assert generate.main([]) == 2
    assert generate.main(["--write-random-model", "x"]) == 2
    assert generate.main(["--random-weights", "--prompt-ids", "1"]) == 2
    assert generate.main(["--model-name", "m"]) == 2        # no prompt
    err = capsys.readouterr().err
    assert "--model-name" in err and "--config" in err and "--prompt" in err


def test_write_random_model_then_generate_from_the_folder(root, capsys, tmp_path):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["A"]))
    out_dir = str(tmp_path / "model")
    assert generate.main(["--write-random-model", out_dir, "--config", str(cfg_path), "--seed", "3",
                          "--weights-dtype", "float32", "--std", "0.08"]) == 0
    assert capsys.readouterr().out.strip() == out_dir
    cfg, w = plain.load_folder(out_dir)
    assert cfg["hidden_size"] == 64 and "model.embed_tokens.weight" in w
    prompt = random_tokens(11, 256, 4)
    log = tmp_path / "out.jsonl"
    rc = generate.main(["--model-name", out_dir, "--prompt-ids", *map(str, prompt),
                        "--max-new-tokens", "6", "--temperature", "0", "--dtype", "float32",
                        "--num-blocks", "16", "--output-file", str(log)],
                       ops=HostOps(), device="cpu")
    assert rc == 0
    printed = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert printed["prompt_ids"] == prompt
    assert printed["output_ids"] == plain.greedy(cfg, w, prompt, 6)
    assert json.loads(log.read_text().strip()) == printed


def test_config_and_seed_in_tokens_out(root, capsys, tmp_path):
    """`--config FILE --random-weights --seed N`: one call from a configuration and a seed to
    tokens; the weights are the ones `--write-random-model` writes for the same seed."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["B"]))
    argv = ["--config", str(cfg_path), "--random-weights", "--seed", "1", "--std", "0.08",
            "--weights-dtype", "float32", "--dtype", "float32", "--prompt-lens", "5", "17",
            "--max-new-tokens", "4", "--temperature", "0", "--block-size", "8", "--num-blocks", "32"]
    assert generate.main(argv, ops=HostOps(), device="cpu") == 0
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert [x["prompt_len"] for x in lines] == [5, 17]
    d = make_model("B", root, torch.float32, std=0.08)      # seed 1 as well
    cfg, w = plain.load_folder(d)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (5, 17)]
    assert [x["output_ids"] for x in lines] == [plain.greedy(cfg, w, p, 4) for p in prompts]
