"""Compares the plain implementation (tests/plain/qwen2_plain.py) with the reference's own model
code on tiny random models, once, on the CPU, and writes the small outputs kept beside it.

Run where the reference checkout is importable:
    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

What is compared (float32, CPU):
* tiny A (tied head): logits at every position = F.linear(QwenModel(ids), embedding), the
  reference's head (somi_inference/models/qwen2_adapter.py:60-62);
* tiny B (untied head): the final-norm hidden states of QwenModel (the reference cannot
  express an untied head);
* greedy tokens of the reference's QwenAdapter prefill + decode over its own paged cache
  (somi_inference/models/qwen2_adapter.py:64-146) for prompts of 5/17/33 tokens.
The reference's weights are our seeded tensors, renamed by the inverse of its `_map_hf_key`
and with gate/up concatenated (qwen2_adapter.py:149-189).  Written: golden_tiny.json with the
worst differences, the reference's greedy tokens and a few logits rows, so that the test can
check the plain implementation without the reference checkout.
"""

import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from somi_inference.core.paged_attention import KVCacheManager  # noqa: E402  (reference)
from somi_inference.models.qwen2 import ForwardContext, ForwardMode, QwenModel, causal_attention  # noqa: E402
from somi_inference.models.qwen2_adapter import QwenAdapter  # noqa: E402

from somi_inference_b200.config import Qwen2Config  # noqa: E402
from somi_inference_b200.weights import random_tensors  # noqa: E402
from tests.plain import qwen2_plain as plain  # noqa: E402
from tests.tiny import SEEDS, TINY, random_tokens  # noqa: E402

STD = 0.08


def reference_model(cfg: dict, w: dict) -> QwenModel:
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    m = QwenModel(vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
                  intermediate_size=cfg["intermediate_size"],
                  num_hidden_layers=cfg["num_hidden_layers"],
                  num_attention_heads=cfg["num_attention_heads"],
                  num_key_value_heads=cfg["num_key_value_heads"], head_dim=hd,
                  max_seq_size=cfg["max_position_embeddings"], rms_norm_eps=cfg["rms_norm_eps"],
                  rope_theta=cfg["rope_theta"])
    sd = {}
    for k, v in w.items():
        if k == "lm_head.weight":
            continue
        k2 = k.removeprefix("model.")
        k2 = {"embed_tokens.weight": "token_embedding.weight",
              "norm.weight": "final_layernorm.weight"}.get(k2, k2)
        if k2.endswith("mlp.gate_proj.weight") or k2.endswith("mlp.up_proj.weight"):
            continue
        sd[k2] = v
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}.mlp"
        sd[f"layers.{i}.mlp.gate_up_proj.weight"] = torch.cat(
            (w[f"{p}.gate_proj.weight"], w[f"{p}.up_proj.weight"]), dim=0)
    m.load_state_dict(sd, strict=True)
    return m.eval()


def reference_hidden(m: QwenModel, ids: list[int]) -> torch.Tensor:
    ctx = ForwardContext(mode=ForwardMode.PREFILL,
                         attn_fn=lambda q, k, v, layer: causal_attention(q, k, v),
                         posi_idx=torch.arange(len(ids)).unsqueeze(0))
    with torch.no_grad():
        return m(torch.tensor([ids]), ctx)[0]


def reference_greedy(m: QwenModel, cfg: dict, prompt: list[int], n_new: int) -> list[int]:
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    kv = KVCacheManager(num_blocks=16, block_size=16, num_kv_heads=cfg["num_key_value_heads"],
                        head_dim=hd, n_layers=cfg["num_hidden_layers"])
    ad = QwenAdapter(m)
    out = []
    with torch.inference_mode():
        kv.register_sequence(0)
        tok = int(torch.argmax(ad.prefill(torch.tensor([prompt]), kv, 0)[0, 0]))
        out.append(tok)
        for _ in range(n_new - 1):
            tok = int(torch.argmax(ad.decode(torch.tensor([[tok]]), kv, [0])[0, 0]))
            out.append(tok)
    return out


def main() -> None:
    record = {"std": STD, "made_with": "reference QwenModel/QwenAdapter on CPU, float32"}
    for name in ("A", "B"):
        cfg = dict(TINY[name])
        w = {k: v.float() for k, v in random_tensors(Qwen2Config.from_dict(cfg), SEEDS[name],
                                                     std=STD, dtype=torch.float32).items()}
        m = reference_model(cfg, w)
        ids = random_tokens(60, cfg["vocab_size"], 100)
        ref_h = reference_hidden(m, ids)
        ours_h = plain.hidden_states(cfg, w, torch.tensor(ids))
        entry = {"ids": ids, "hidden_max_abs_diff": float((ref_h - ours_h).abs().max()),
                 "hidden_scale": float(ref_h.abs().max())}
        if cfg["tie_word_embeddings"]:
            ref_logits = torch.nn.functional.linear(ref_h, m.token_embedding.weight.detach())
            ours = plain.logits(cfg, w, ids)
            entry["logits_max_abs_diff"] = float((ref_logits - ours).abs().max())
            entry["logits_scale"] = float(ref_logits.abs().max())
            entry["reference_logits_rows"] = {str(p): ref_logits[p, :16].tolist() for p in (0, 31, 59)}
            entry["greedy"] = {}
            for n in (5, 17, 33):
                prompt = random_tokens(n, cfg["vocab_size"], n)
                got = reference_greedy(m, cfg, prompt, 8)
                assert got == plain.greedy(cfg, w, prompt, 8), (n, got)
                entry["greedy"][str(n)] = {"prompt": prompt, "tokens": got}
        else:
            entry["reference_hidden_rows"] = {str(p): ref_h[p, :16].tolist() for p in (0, 31, 59)}
        record[name] = entry
        print(name, {k: v for k, v in entry.items() if k.endswith("diff") or k.endswith("scale")})
    with open(os.path.join(HERE, "golden_tiny.json"), "w") as f:
        json.dump(record, f, indent=1)


if __name__ == "__main__":
    main()
