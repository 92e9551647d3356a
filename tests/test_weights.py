"""Weight files: round trip, dtypes, and the one error that lists everything wrong (no GPU)."""

import json
import os

import pytest
import torch

from somi_inference_b200.config import Qwen2Config
from somi_inference_b200.parts import BuildContext, declared_tensors
from somi_inference_b200.weights import (SafetensorsFile, WeightError, load_tensors,
                                         random_tensors, save_safetensors, write_random_model)
from tests.plain import qwen2_plain as plain
from tests.tiny import TINY_A, TINY_B


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(t, p)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c", "e"]
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the independent reader of the plain implementation agrees
    for k, v in plain.read_safetensors(p).items():
        assert torch.equal(v, t[k])
    try:
        from safetensors.torch import load_file
    except ImportError:
        return
    for k, v in load_file(p).items():
        assert torch.equal(v, t[k])


def test_random_model_is_deterministic_and_loads(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    a = random_tensors(cfg, 1, dtype=torch.float32)
    b = random_tensors(cfg, 1, dtype=torch.float32)
    c = random_tensors(cfg, 2, dtype=torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert torch.equal(a["model.norm.weight"], torch.ones(192))
    assert abs(a["model.embed_tokens.weight"].std().item() - 0.02) < 1e-3
    d = write_random_model(cfg, 1, str(tmp_path / "m"), dtype=torch.bfloat16)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    decl = declared_tensors(cfg.to_model_spec())
    loaded = load_tensors(d, decl)
    assert set(loaded) == set(decl)
    assert all(v.dtype == torch.bfloat16 for v in loaded.values())
    assert torch.equal(loaded["lm_head.weight"], a["lm_head.weight"].to(torch.bfloat16))
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]


def test_placement_keeps_precisions():
    ctx = BuildContext(dtype=torch.bfloat16, device=torch.device("cpu"), ops=None)
    assert ctx.place(torch.ones(4, 4, dtype=torch.float32), matrix=True).dtype == torch.bfloat16
    assert ctx.place(torch.ones(4, dtype=torch.float32), matrix=False).dtype == torch.float32
    assert ctx.place(torch.ones(4, dtype=torch.bfloat16), matrix=False).dtype == torch.bfloat16
    assert ctx.place(torch.ones(4, dtype=torch.int64), matrix=False).dtype == torch.int32
    ctx32 = BuildContext(dtype=torch.float32, device=torch.device("cpu"), ops=None)
    assert ctx32.place(torch.ones(4, 4, dtype=torch.bfloat16), matrix=True).dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    t = random_tensors(cfg, 0, dtype=torch.float32)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    t["model.layers.7.extra.weight"] = torch.zeros(2)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # ignored buffer
    os.makedirs(tmp_path / "m")
    save_safetensors(t, str(tmp_path / "m" / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path / "m"), declared_tensors(cfg.to_model_spec()))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(err)
    for part in ("missing (2)", "unexpected (1)", "wrong shape (1)", "(64, 32)", "(64, 64)"):
        assert part in msg


def test_tied_model_tolerates_lm_head_and_untied_needs_it(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    t = random_tensors(cfg, 0, dtype=torch.float32)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    os.makedirs(tmp_path / "tied")
    save_safetensors(t, str(tmp_path / "tied" / "model.safetensors"))
    decl = declared_tensors(cfg.to_model_spec())
    # the tied model's head declares the matrix as a copy that is tolerated and never read
    assert "lm_head.weight" not in load_tensors(str(tmp_path / "tied"), decl)
    t["lm_head.weight"] = torch.zeros(3, 3)                   # but its shape is still checked
    os.makedirs(tmp_path / "tied_bad")
    save_safetensors(t, str(tmp_path / "tied_bad" / "model.safetensors"))
    with pytest.raises(WeightError, match="wrong shape"):
        load_tensors(str(tmp_path / "tied_bad"), decl)
    cfg_b = Qwen2Config.from_dict(TINY_B)
    tb = random_tensors(cfg_b, 1, dtype=torch.float32)
    del tb["lm_head.weight"]
    os.makedirs(tmp_path / "untied")
    save_safetensors(tb, str(tmp_path / "untied" / "model.safetensors"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_tensors(str(tmp_path / "untied"), declared_tensors(cfg_b.to_model_spec()))


def test_optional_tensor_may_be_absent(tmp_path):
    """A declaration marked optional: absent from the file -> absent from the result, no error;
    present -> loaded and shape-checked like any other."""
    from somi_inference_b200.parts.base import TensorDecl
    decl = {"w": TensorDecl("w", (2, 3)), "b": TensorDecl("b", (2,), matrix=False, optional=True)}
    os.makedirs(tmp_path / "without")
    save_safetensors({"w": torch.ones(2, 3)}, str(tmp_path / "without" / "model.safetensors"))
    assert sorted(load_tensors(str(tmp_path / "without"), decl)) == ["w"]
    os.makedirs(tmp_path / "with")
    save_safetensors({"w": torch.ones(2, 3), "b": torch.ones(2)}, str(tmp_path / "with" / "model.safetensors"))
    assert sorted(load_tensors(str(tmp_path / "with"), decl)) == ["b", "w"]
    os.makedirs(tmp_path / "bad")
    save_safetensors({"w": torch.ones(2, 3), "b": torch.ones(5)}, str(tmp_path / "bad" / "model.safetensors"))
    with pytest.raises(WeightError, match="wrong shape"):
        load_tensors(str(tmp_path / "bad"), decl)


def test_sharded_folder(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    t = random_tensors(cfg, 0, dtype=torch.float32)
    names = sorted(t)
    half = len(names) // 2
    d = tmp_path / "m"
    os.makedirs(d)
    save_safetensors({k: t[k] for k in names[:half]}, str(d / "model-00001-of-00002.safetensors"))
    save_safetensors({k: t[k] for k in names[half:]}, str(d / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in names[:half]}
    wm.update({k: "model-00002-of-00002.safetensors" for k in names[half:]})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    loaded = load_tensors(str(d), declared_tensors(cfg.to_model_spec()))
    assert all(torch.equal(loaded[k], t[k]) for k in t)
    with pytest.raises(FileNotFoundError):
        load_tensors(str(tmp_path), declared_tensors(cfg.to_model_spec()))
