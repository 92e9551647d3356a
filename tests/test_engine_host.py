"""The host side of the engine (batch layout, cache manager, order of runs, scheduler loop)
checked on the CPU by handing the engine the test-only kernel table of tests/plain/host_ops.py.
The product path never runs like this; the same checks run on the GPU with the CUDA kernels in
tests/test_gpu_replay.py and tests/test_gpu_engine.py."""

import pytest
import torch

from somi_inference_b200 import LLM, SamplingParams
from somi_inference_b200.cache import OutOfPages
from somi_inference_b200.config import register_architecture, unregister_architecture
from somi_inference_b200.engine import Engine, StepEntry
from tests import replay, toy_model
from tests.plain import qwen2_plain as plain
from tests.plain.host_ops import HostOps
from tests.tiny import PAGE_SIZES, TINY, make_model, random_tokens
from tests.toy_parts import register_toys, unregister_toys

MODES = {"whole": replay.whole, "last32": replay.last_one_by_one, "portions": replay.portions,
         "mixed": replay.mixed}


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("host"))


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name", list(TINY))
def test_cuts_agree_with_plain(root, name, mode):
    d = make_model(name, root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 10 + i)
            for i, n in enumerate([5, 97, 40, 70, 33, 64])}
    ref = {k: plain.logits(cfg, w, v) for k, v in reqs.items()}
    steps, max_tokens = MODES[mode](reqs)
    eng = Engine(d, dtype="float32", page_size=PAGE_SIZES[name], max_tokens=max_tokens,
                 device="cpu", ops=HostOps())
    got = replay.run_steps(eng, steps)
    replay.compare(got, ref, 3e-5, f"{name}/{mode}")
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


def test_out_of_pages_leaves_the_cache_as_it_was(root):
    d = make_model("A", root, torch.float32, std=0.08)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=4, device="cpu", ops=HostOps())
    eng.step([StepEntry("a", list(range(40)), [39])])
    free = eng.cache.free_pages()
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", [1], [0]), StepEntry("b", list(range(30)), [29])])
    assert eng.cache.free_pages() == free and not eng.has("b") and eng.length("a") == 40
    eng.cache.check_consistency()
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([StepEntry("a", [256], [0])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    assert eng.cache.free_pages() == free


def test_positions_limit(root):
    d = make_model("A", root, torch.float32, std=0.08)       # 128 positions
    eng = Engine(d, dtype="float32", page_size=16, num_pages=16, device="cpu", ops=HostOps())
    eng.step([StepEntry("a", list(range(128)), [])])
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1], [0])])


def test_generation_through_the_entry_point_matches_plain_greedy(root):
    d = make_model("B", root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    llm = LLM(d, num_blocks=40, block_size=8, max_concurrent=3, device="cpu", dtype="float32",
              ops=HostOps(), chunk_size=32, max_num_batched_tokens=48)
    prompts = [random_tokens(n, 1000, 50 + i) for i, n in enumerate([1, 9, 40, 100])]
    outs = llm.generate_many(prompts, max_new_tokens=6,
                             sampling_params=SamplingParams(temperature=0.0),
                             arrival_steps=[0, 0, 1, 3])
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(cfg, w, p, 6)
    assert llm.engine.cache.free_pages() == [40]
    assert llm.generate(prompts[1], max_new_tokens=4, temperature=0.0) == outs[1][:4]


def test_text_in_text_out_through_a_tokenizer_in_the_model_folder(root):
    """`LLM.generate` with a string: the prompt goes through the tokenizer that lies in the model
    folder and the new tokens come back as text (somi_inference/entrypoints/llm.py:118-160).  The
    tokenizer here is a word-level one written by the test (one word per id); a folder without a
    tokenizer refuses text with a clear error."""
    import json
    import os
    import shutil
    tokenizers = pytest.importorskip("tokenizers")
    pytest.importorskip("transformers")
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    src = make_model("A", root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(src)
    bare = LLM(src, num_blocks=16, block_size=8, max_concurrent=1, device="cpu", dtype="float32",
               ops=HostOps())
    with pytest.raises(ValueError, match="no tokenizer"):
        bare.generate("w5 w17", max_new_tokens=2, temperature=0.0)
    d = os.path.join(root, "A_with_tokenizer")
    shutil.copytree(src, d)
    vocab = {f"w{i}": i for i in range(cfg["vocab_size"])}
    tok = tokenizers.Tokenizer(WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = Whitespace()
    tok.save(os.path.join(d, "tokenizer.json"))
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "w0"}, f)
    llm = LLM(d, num_blocks=16, block_size=8, max_concurrent=1, device="cpu", dtype="float32",
              ops=HostOps())
    ids = [5, 17, 3, 200, 41]
    text = llm.generate(" ".join(f"w{i}" for i in ids), max_new_tokens=5, temperature=0.0, ignore_eos=True)
    assert text == " ".join(f"w{i}" for i in plain.greedy(cfg, w, ids, 5))


def test_sampled_generation_matches_the_plain_sampler(root):
    """Tiny B at temperature 0.7 with top-k, top-p and a repetition penalty, portions of 32 mixed
    with decoding: every token is the one the plain pipeline draws with the same (seed, counter)."""
    from tests.plain import generate_plain
    d = make_model("B", root, torch.float32, std=0.02)
    cfg, w = plain.load_folder(d)
    llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=4, device="cpu", dtype="float32",
              ops=HostOps(), chunk_size=32, max_num_batched_tokens=40)
    prompts = [random_tokens(n, 1000, 90 + i) for i, n in enumerate([1, 9, 40, 100])]
    kinds = [dict(temperature=0.7), dict(temperature=0.7, top_k=40),
             dict(temperature=0.7, top_p=0.9), dict(temperature=0.7, repetition_penalty=1.3)]
    sps = [SamplingParams(seed=5 + i, **k) for i, k in enumerate(kinds)]
    outs = llm.generate_many(prompts, max_new_tokens=6, sampling_params=sps, ignore_eos=True,
                             arrival_steps=[0, 0, 1, 2])
    for p, o, sp, k in zip(prompts, outs, sps, kinds):
        assert generate_plain.check_sampled(cfg, w, p, o, seed=sp.seed, **k) == 0
        assert o == generate_plain.generate(cfg, w, p, 6, seed=sp.seed, **k)


def test_end_of_sequence_under_steps_launched_ahead(root):
    """Decode steps are launched before the host has read the ids of the step before.  A request
    that ends on such a token has a row in the step that ran ahead: the row is dropped, the others
    go on, a late arrival is admitted afterwards, and every page comes back, with and without
    running ahead."""
    d = make_model("B", root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 200 + i) for i, n in enumerate([7, 19, 33, 12])]
    free_run = [plain.greedy(cfg, w, p, 16) for p in prompts]
    eos = free_run[1][6]
    want = [o[:o.index(eos) + 1] if eos in o else o for o in free_run]
    assert any(len(o) < 16 for o in want)
    for ahead in (True, False):
        llm = LLM(d, num_blocks=40, block_size=8, max_concurrent=3, device="cpu", dtype="float32",
                  ops=HostOps(), chunk_size=16, eos_token_id=eos)
        llm.run_ahead = ahead
        launched_ahead = 0
        reqs = [llm.make_request(p, max_new_tokens=16, sampling_params=SamplingParams(temperature=0.0))
                for p in prompts]
        pending = [(0, reqs[0]), (0, reqs[1]), (2, reqs[2]), (11, reqs[3])]
        step = 0
        while pending or llm.scheduler.has_unfinished():
            while pending and pending[0][0] <= step:
                llm.scheduler.add_request(pending.pop(0)[1])
            llm.step()
            launched_ahead += llm._ahead is not None
            llm.engine.cache.check_consistency()
            step += 1
        assert [r.output_tokens for r in reqs] == want, f"run_ahead={ahead}"
        assert (launched_ahead > 0) == ahead
        assert (llm.rows_dropped > 0) == ahead
        llm.step()
        assert llm.engine.cache.free_pages() == [40]


def test_preempted_request_generates_the_same_tokens(root):
    d = make_model("A", root, torch.float32, std=0.08)
    prompts = [random_tokens(n, 256, 70 + i) for i, n in enumerate([30, 28, 26])]
    sp = [SamplingParams(temperature=0.8, seed=100 + i) for i in range(3)]
    roomy = LLM(d, num_blocks=64, block_size=4, max_concurrent=3, device="cpu", dtype="float32",
                ops=HostOps())
    want = roomy.generate_many(prompts, max_new_tokens=20, sampling_params=sp, ignore_eos=True)
    tight = LLM(d, num_blocks=28, block_size=4, max_concurrent=3, device="cpu", dtype="float32",
                ops=HostOps())
    reqs = [tight.make_request(p, max_new_tokens=20, sampling_params=s, ignore_eos=True)
            for p, s in zip(prompts, sp)]
    tight.run([(0, r) for r in reqs])
    assert sum(r.num_preemptions for r in reqs) > 0, "the test is meant to run out of pages"
    assert [r.output_tokens for r in reqs] == want
    assert tight.engine.cache.free_pages() == [28]


class FailingOps(HostOps):
    """A kernel table whose attention raises at chosen calls, like a launch that failed."""

    def __init__(self, fail_at: set[int]) -> None:
        super().__init__()
        self.calls = 0
        self.fail_at = set(fail_at)

    def paged_attention(self, *args, **kwargs):
        self.calls += 1
        if self.calls in self.fail_at:
            raise RuntimeError("injected launch failure")
        return super().paged_attention(*args, **kwargs)


def test_a_failed_launch_leaves_nothing_reserved(root):
    """If a step raises after its pages were reserved (a kernel error, out of memory), the
    reservations are cancelled: the engine's step leaves the cache as it was, and the loop of
    the entry point can simply be called again and generates what it would have generated."""
    d = make_model("A", root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=8, device="cpu", ops=FailingOps({3}))
    eng.step([StepEntry("a", random_tokens(20, 256, 1), [])])
    free = eng.cache.free_pages()
    with pytest.raises(RuntimeError, match="injected"):
        eng.step([StepEntry("a", random_tokens(20, 256, 2), []), StepEntry("b", [3, 4, 5], [2])])
    assert eng.cache.free_pages() == free and eng.cache.length("a") == 20
    assert not eng.cache.is_registered("b")
    eng.cache.check_consistency()
    eng.step([StepEntry("a", random_tokens(20, 256, 2), []), StepEntry("b", [3, 4, 5], [2])])

    prompts = [random_tokens(n, 256, 90 + i) for i, n in enumerate([9, 21])]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    layers = cfg["num_hidden_layers"]
    # failures in a prompt step, in a decode step launched ahead, and in a later one
    for fail_at in ({1}, {2 * layers + 1}, {5 * layers + 2}):
        llm = LLM(d, num_blocks=16, block_size=8, max_concurrent=2, device="cpu", dtype="float32",
                  ops=FailingOps(fail_at), chunk_size=32)
        reqs = [llm.make_request(p, max_new_tokens=8, sampling_params=SamplingParams(temperature=0.0))
                for p in prompts]
        for r in reqs:
            llm.scheduler.add_request(r)
        failures = 0
        for _ in range(200):
            if not llm.scheduler.has_unfinished():
                break
            try:
                llm.step()
            except RuntimeError:
                failures += 1
            llm.engine.cache.check_consistency()
        assert failures == 1
        assert [r.output_tokens for r in reqs] == want, fail_at
        llm.step()
        assert llm.engine.cache.free_pages() == [16]


def test_toy_architecture_is_registered_built_and_stepped(root):
    register_toys()
    register_architecture(toy_model.ARCH, toy_model.ToyConfig)
    try:
        d = toy_model.write_toy_model(root + "/toy")
        ids = random_tokens(45, toy_model.V, 3)
        ref = toy_model.plain_logits(d, ids)
        eng = Engine(d, dtype="float32", page_size=8, max_tokens=128, device="cpu", ops=HostOps())
        # full keys (two layers share the group), a window of 6, and keys and values of
        # different widths stored apart
        assert len(eng.cache.groups) == 3
        assert [g.storage is None for g in eng.cache.groups].count(True) == 1
        got = eng.step([StepEntry("w", ids, list(range(45)))])
        assert (got - ref).abs().max().item() < 3e-5
        eng.end("w")
        rows = []
        i = 0
        for c in [5, 2, 11, 1, 1, 9, 16]:
            rows.append(eng.step([StepEntry("p", ids[i:i + c], list(range(c)))]))
            i += c
        assert (torch.cat(rows) - ref).abs().max().item() < 3e-5
        eng.end("p")
        assert all(f == eng.num_pages for f in eng.cache.free_pages())
        # the same model with the tensor that its file may lack (a bias) present
        d2 = toy_model.write_toy_model(root + "/toy_bias", with_optional=True)
        ref2 = toy_model.plain_logits(d2, ids)
        assert (ref2 - ref).abs().max().item() > 1e-3          # the bias matters
        eng2 = Engine(d2, dtype="float32", page_size=8, max_tokens=128, device="cpu", ops=HostOps())
        got2 = torch.cat([eng2.step([StepEntry("q", ids[:30], list(range(30)))]),
                          eng2.step([StepEntry("q", ids[30:], list(range(15)))])])
        assert (got2 - ref2).abs().max().item() < 3e-5
    finally:
        unregister_architecture(toy_model.ARCH)
        unregister_toys()


def test_abort_and_a_stream_that_is_closed_early(root):
    """A request that is aborted between steps leaves the others' tokens unchanged, also when a
    decode step with a row for it is on its way; a stream whose reader stops leaves no request
    and no page behind."""
    d = make_model("B", root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 600 + i) for i, n in enumerate([9, 17, 5])]
    want = [plain.greedy(cfg, w, p, 12) for p in prompts]
    for ahead in (True, False):
        llm = LLM(d, num_blocks=40, block_size=8, max_concurrent=3, device="cpu", dtype="float32",
                  ops=HostOps(), chunk_size=16)
        llm.run_ahead = ahead
        reqs = [llm.make_request(p, max_new_tokens=12, sampling_params=SamplingParams(temperature=0.0),
                                 ignore_eos=True) for p in prompts]
        for r in reqs:
            llm.scheduler.add_request(r)
        steps = 0
        while llm.scheduler.has_unfinished():
            llm.step()
            steps += 1
            if steps == 5:
                assert (llm._ahead is not None) == ahead
                assert llm.abort(reqs[1])
            llm.engine.cache.check_consistency()
        assert reqs[0].output_tokens == want[0] and reqs[2].output_tokens == want[2]
        assert reqs[1].finish_reason == "aborted" and reqs[1].output_tokens == want[1][:len(reqs[1].output_tokens)]
        assert 0 < len(reqs[1].output_tokens) < 12
        llm.step()
        assert llm.engine.cache.free_pages() == [40]
        # a stream read for three tokens only
        llm.scheduler.drain_finished()
        got = []
        stream = llm.generate_stream(prompts[0], max_new_tokens=12, temperature=0.0)
        for t in stream:
            got.append(t)
            if len(got) == 3:
                break
        stream.close()
        assert got == want[0][:3]
        assert not llm.scheduler.has_unfinished()
        llm.step()
        assert llm.engine.cache.free_pages() == [40]
        assert llm.generate(prompts[2], max_new_tokens=12, temperature=0.0, ignore_eos=True) == want[2]


@pytest.mark.parametrize("seed", range(6))
def test_random_schedules_with_ends_aborts_and_late_arrivals(root, seed):
    """Random prompts, arrival steps, token budgets, pool sizes and policies; an end-of-sequence
    token that some requests meet, and one request aborted on the way.  Every other request must
    give plain greedy decoding's tokens (cut at the end-of-sequence token), and the cache must be
    consistent after every step and empty at the end."""
    import random
    rng = random.Random(1000 + seed)
    name = rng.choice(["A", "B"])
    d = make_model(name, root, torch.float32, std=0.08)
    cfg, w = plain.load_folder(d)
    n = rng.randrange(2, 6)
    new = rng.choice([3, 8, 14])
    limit = cfg["max_position_embeddings"] - new - 1
    prompts = [random_tokens(rng.randrange(1, min(limit, 60)), cfg["vocab_size"], 50 * seed + i)
               for i in range(n)]
    free_run = [plain.greedy(cfg, w, p, new) for p in prompts]
    eos = rng.choice(rng.choice(free_run))               # a token that does come up
    want = [o[:o.index(eos) + 1] if eos in o else o for o in free_run]
    page = rng.choice([4, 8, 16])
    need = max(-(-(len(p) + new) // page) for p in prompts)
    llm = LLM(d, num_blocks=rng.choice([need + 1, 2 * need, 64]), block_size=page,
              max_concurrent=rng.choice([1, 2, 4]), device="cpu", dtype="float32", ops=HostOps(),
              chunk_size=rng.choice([2, 7, 16, 64]), max_num_batched_tokens=rng.choice([8, 24, 64]),
              policy=rng.choice(["preempt", "reserve"]), eos_token_id=eos)
    llm.run_ahead = rng.random() < 0.7
    reqs = [llm.make_request(p, max_new_tokens=new, sampling_params=SamplingParams(temperature=0.0))
            for p in prompts]
    pending = sorted(((rng.randrange(0, 8), i) for i in range(n)))
    victim, abort_at = rng.randrange(n), rng.randrange(1, 12)
    step = 0
    while pending or llm.scheduler.has_unfinished():
        while pending and pending[0][0] <= step:
            llm.scheduler.add_request(reqs[pending.pop(0)[1]])
        llm.step()
        step += 1
        if step == abort_at:
            llm.abort(reqs[victim])
        llm.engine.cache.check_consistency()
        assert step < 2000
    llm.step()
    pools = len(llm.engine.cache.groups)
    assert llm.engine.cache.free_pages() == [llm.engine.num_pages] * pools
    for i, r in enumerate(reqs):
        if r.finish_reason == "aborted":
            assert i == victim and r.output_tokens == want[i][:len(r.output_tokens)]
        else:
            assert r.output_tokens == want[i], f"request {i}"
