"""The bfloat16 path against the float32 path at the layer sizes of the large models.

The tiny configurations cannot reach the kernels' large-size variants (rings that are not deep,
more output tiles than SMs, the vocabulary-sized head, token widths of 32 and 64 with long K).
Two layers with the 7B and 0.5B layer sizes, random weights whose values are bfloat16 in both
engines, prompts of different lengths in one step and then decode steps, at batch sizes on both
sides of the kernels' token widths (16, 32, 64).  The float32 engine is the reference; the bounds
are those of the replay tests (root mean square 4e-3, largest difference 4e-2 of the largest logit).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = {
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
               vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "0.5b": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                 vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def weights(request):
    from somi_inference_b200.config import Qwen2Config
    from somi_inference_b200.parts import declared_tensors
    raw = dict(SHAPES[request.param], num_hidden_layers=2, max_position_embeddings=4608,
               architectures=["Qwen2ForCausalLM"], hidden_act="silu", use_sliding_window=False)
    cfg = Qwen2Config.from_dict(raw)
    gen = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, d in declared_tensors(cfg.to_model_spec()).items():
        if d.init == "ones":
            tensors[name] = torch.ones(d.shape, dtype=torch.bfloat16, device="cuda")
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.03, generator=gen)
            tensors[name] = t.to(torch.bfloat16)
    yield request.param, cfg, tensors
    tensors.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("batch", [5, 17, 32, 33, 64])
def test_bfloat16_against_float32_at_large_layer_sizes(weights, batch):
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(batch)
    lens = [int(x) for x in torch.randint(20, 300, (batch,), generator=g)]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    feed = torch.randint(0, cfg.vocab_size, (3, batch), generator=g).tolist()
    outs = []
    for dtype in ("bfloat16", "float32"):
        tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=batch * 320 + 64,
                                  max_requests=batch + 1)
        res = [eng.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])]
        for s in range(3):
            res.append(eng.step([StepEntry(i, [feed[s][i]], [0]) for i in range(batch)]))
        eng.ops.check_errors()
        outs.append(torch.cat([r.float() for r in res]))
        del eng, tt
    got, ref = outs
    scale = ref.abs().max().item()
    rms = ((got - ref) ** 2).mean().sqrt().item()
    assert rms <= 4e-3 * scale, f"{name} batch {batch}: rms {rms / scale:.2e} of the largest logit"
    assert (got - ref).abs().max().item() <= 4e-2 * scale


def test_bfloat16_against_float32_with_thousands_of_chunks(weights):
    """A decode step with more than 16 chunks of 128 keys per SM takes the attention kernel whose
    CTAs walk through several chunks, and a merge over fewer, larger partial results: many
    requests with contexts of a few thousand tokens, of different lengths."""
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    batch, ctx = {"7b": (40, 2100), "0.5b": (48, 4200)}[name]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert -(-ctx // 128) * cfg.num_key_value_heads * batch >= 16 * sms, "the step is meant to be large"
    g = torch.Generator().manual_seed(7)
    lens = [ctx - 37 * (i % 7) for i in range(batch)]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    feed = torch.randint(0, cfg.vocab_size, (4, batch), generator=g).tolist()
    outs = []
    for dtype in ("bfloat16", "float32"):
        tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=sum(lens) + 64 * batch,
                                  max_requests=batch)
        for i, p in enumerate(prompts):
            eng.step([StepEntry(i, p, [])])
        res = [eng.step([StepEntry(i, [feed[s][i]], [0]) for i in range(batch)]) for s in range(4)]
        eng.ops.check_errors()
        outs.append(torch.cat([r.float() for r in res]))
        del eng, tt
    got, ref = outs
    scale = ref.abs().max().item()
    rms = ((got - ref) ** 2).mean().sqrt().item()
    assert rms <= 4e-3 * scale, f"{name}: rms {rms / scale:.2e} of the largest logit"
    assert (got - ref).abs().max().item() <= 4e-2 * scale
