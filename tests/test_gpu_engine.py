"""Generation through the entry point, long decoding, the first tokens of a sequence, each
part of a layer alone, and the toy architecture, on the GPU with the CUDA kernels."""

import pytest
import torch

from tests import replay, toy_model
from tests.plain import qwen2_plain as plain
from tests.plain.host_ops import HostOps
from tests.tiny import PAGE_SIZES, TINY, make_model, random_tokens
from tests.toy_parts import register_toys, unregister_toys

pytestmark = pytest.mark.gpu
STD = 0.08


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("gpu_engine"))


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_generation_through_the_entry_point(root, name):
    from somi_inference_b200 import LLM, SamplingParams
    d = make_model(name, root, torch.float32, std=STD)
    cfg, w = plain.load_folder(d)
    llm = LLM(d, num_blocks=64, block_size=PAGE_SIZES[name], max_concurrent=4, dtype="float32",
              chunk_size=32, max_num_batched_tokens=64)
    prompts = [random_tokens(n, cfg["vocab_size"], 50 + i) for i, n in enumerate([1, 9, 40, 100, 33])]
    outs = llm.generate_many(prompts, max_new_tokens=12,
                             sampling_params=SamplingParams(temperature=0.0),
                             arrival_steps=[0, 0, 1, 2, 5])
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(cfg, w, p, 12)
    assert llm.engine.cache.free_pages() == [64] * len(llm.engine.cache.groups)
    assert llm.generate(prompts[2], max_new_tokens=5, temperature=0.0) == outs[2][:5]


def test_tiny_b_as_the_benchmark_description_states_it(root):
    """Tiny B of the benchmark description, to the letter: weights N(0, 0.02) from seed 1,
    float32, pages of 8, four prompts of 1/9/40/100 random ids, prompt portions of 32 tokens
    mixed with decoding, 12 tokens each at temperature 0.7 with fixed sampling seeds.  Expected
    ids: plain whole-sequence logits through the plain sampler with the same (seed, counter)
    (the reference checks generation against an independent implementation in
    tests/entrypoints/test_llm_e2e.py:60-71)."""
    from somi_inference_b200 import LLM, SamplingParams
    from tests.plain import generate_plain
    d = make_model("B", root, torch.float32, std=0.02)
    cfg, w = plain.load_folder(d)
    llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=4, dtype="float32", chunk_size=32,
              max_num_batched_tokens=40)
    prompts = [random_tokens(n, 1000, 90 + i) for i, n in enumerate([1, 9, 40, 100])]
    sps = [SamplingParams(temperature=0.7, seed=5 + i) for i in range(4)]
    outs = llm.generate_many(prompts, max_new_tokens=12, sampling_params=sps, ignore_eos=True,
                             arrival_steps=[0, 0, 1, 2])
    boundary = 0
    for p, o, sp in zip(prompts, outs, sps):
        assert len(o) == 12
        boundary += generate_plain.check_sampled(cfg, w, p, o, temperature=0.7, seed=sp.seed)
    assert boundary <= 1          # 48 draws: a draw at a rounding boundary is a rare event
    assert llm.engine.cache.free_pages() == [64]


def test_temperature_generation_is_reproducible_and_batch_independent(root):
    from somi_inference_b200 import LLM, SamplingParams
    d = make_model("B", root, torch.bfloat16, std=STD)
    llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=4, dtype="float32", chunk_size=32)
    prompts = [random_tokens(n, 1000, 90 + i) for i, n in enumerate([1, 9, 40, 100])]
    sps = [SamplingParams(temperature=0.7, seed=5 + i) for i in range(4)]
    together = llm.generate_many(prompts, max_new_tokens=12, sampling_params=sps)
    alone = [llm.generate(p, max_new_tokens=12, temperature=0.7, seed=5 + i)
             for i, p in enumerate(prompts)]
    assert together == alone
    assert len({tuple(o) for o in together}) == 4


def test_end_of_sequence_arrives_while_the_next_step_is_prepared(root):
    """Generation prepares the next decode step while the tokens of the current one are sampled.
    A request that ends on such a token (end of sequence, not foreseeable) must not run on, the
    others must go on unchanged, and every page must come back.  The end-of-sequence token is
    chosen as one that greedy generation does produce, at different steps in different requests."""
    from somi_inference_b200 import LLM, SamplingParams
    d = make_model("B", root, torch.float32, std=STD)
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 200 + i) for i, n in enumerate([7, 19, 33, 12])]
    free_run = [plain.greedy(cfg, w, p, 24) for p in prompts]
    eos = free_run[1][9]                     # request 1 ends at its 10th token at the latest
    want = []
    for o in free_run:
        want.append(o[:o.index(eos) + 1] if eos in o else o)
    for early, ahead in ((True, True), (True, False), (False, False)):
        llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=4, dtype="float32", chunk_size=16,
                  eos_token_id=eos)
        llm.prepare_early, llm.run_ahead = early, ahead
        outs = llm.generate_many(prompts, max_new_tokens=24,
                                 sampling_params=SamplingParams(temperature=0.0))
        assert outs == want, f"prepare_early={early} run_ahead={ahead}"
        assert any(len(o) < 24 for o in outs)
        llm.step()                           # gives back what was prepared for a step that never came
        assert llm.engine.cache.free_pages() == [64] * len(llm.engine.cache.groups)
        llm.engine.cache.check_consistency()


def test_steps_launched_ahead_sample_the_same_tokens(root):
    """A decode step that is launched before the host has read the ids of the step before takes
    them on the device and counts the token on its way for the random numbers: temperature,
    top-k and top-p sampling give the same tokens with and without it, also when requests arrive
    late and when one of them has a repetition penalty (which keeps its steps from running ahead)."""
    from somi_inference_b200 import LLM, SamplingParams
    d = make_model("C", root, torch.float32, std=STD)
    cfg, _ = plain.load_folder(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 400 + i) for i, n in enumerate([5, 21, 40, 9])]
    for penalty in (1.0, 1.3):
        sps = [SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=11 + i,
                              repetition_penalty=penalty if i == 2 else 1.0) for i in range(4)]
        outs = []
        for ahead in (True, False):
            llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=4, dtype="float32", chunk_size=16)
            llm.run_ahead = ahead
            outs.append(llm.generate_many(prompts, max_new_tokens=20, sampling_params=sps,
                                          arrival_steps=[0, 0, 3, 9], ignore_eos=True))
            llm.engine.cache.check_consistency()
            assert llm.engine.cache.free_pages() == [64] * len(llm.engine.cache.groups)
        assert outs[0] == outs[1], f"penalty {penalty}"


def test_a_step_of_another_caller_between_prepared_steps(root):
    """The engine's step function used directly between two steps of generation overwrites the
    descriptor that generation had prepared: generation must notice and build its step again."""
    from somi_inference_b200 import LLM, SamplingParams
    from somi_inference_b200.engine import StepEntry
    d = make_model("B", root, torch.float32, std=STD)
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 300 + i) for i, n in enumerate([11, 23])]
    llm = LLM(d, num_blocks=64, block_size=8, max_concurrent=3, dtype="float32", chunk_size=16)
    reqs = [llm.make_request(p, max_new_tokens=14, sampling_params=SamplingParams(temperature=0.0),
                             ignore_eos=True) for p in prompts]
    for r in reqs:
        llm.scheduler.add_request(r)
    steps = 0
    while llm.scheduler.has_unfinished():
        llm.step()
        steps += 1
        if steps % 3 == 0:
            llm.engine.step([StepEntry("other", random_tokens(5, cfg["vocab_size"], steps), [4])])
            llm.engine.end("other")
    assert [r.output_tokens for r in reqs] == [plain.greedy(cfg, w, p, 14) for p in prompts]


def test_preemption_on_the_gpu_gives_the_same_tokens(root):
    from somi_inference_b200 import LLM, SamplingParams
    d = make_model("A", root, torch.float32, std=STD)
    prompts = [random_tokens(n, 256, 70 + i) for i, n in enumerate([30, 28, 26])]
    sp = [SamplingParams(temperature=0.0) for _ in range(3)]
    roomy = LLM(d, num_blocks=64, block_size=4, max_concurrent=3, dtype="float32")
    want = roomy.generate_many(prompts, max_new_tokens=20, sampling_params=sp, ignore_eos=True)
    tight = LLM(d, num_blocks=28, block_size=4, max_concurrent=3, dtype="float32")
    reqs = [tight.make_request(p, max_new_tokens=20, sampling_params=s, ignore_eos=True)
            for p, s in zip(prompts, sp)]
    tight.run([(0, r) for r in reqs])
    assert sum(r.num_preemptions for r in reqs) > 0
    assert [r.output_tokens for r in reqs] == want


@pytest.mark.parametrize("seed", [0, 1, 2])
@pytest.mark.parametrize("name", ["A", "C"])
def test_serving_with_random_arrivals_few_pages_and_aborts(root, name, seed):
    """A serving run made by a random number generator: requests of random lengths arrive at
    random steps and want random numbers of tokens, the page pool is small enough for
    preemptions, and some requests are taken out half way.  Every request that was left alone
    must have produced exactly the greedy tokens of the plain implementation, an aborted one
    a prefix of them, and no page may be lost.  (float32, so that the largest logit is the
    same on both sides.)"""
    import random
    from somi_inference_b200 import LLM, SamplingParams
    from somi_inference_b200.engine.scheduler import RequestStatus
    d = make_model(name, root, torch.float32, std=STD)
    cfg, w = plain.load_folder(d)
    rng = random.Random(1000 + seed)
    ps = PAGE_SIZES[name]
    n_req = 10
    lens = [rng.choice([1, 2, 3, 7, 17, 31, 45, 64, 80]) for _ in range(n_req)]
    news = [rng.randint(1, 24) for _ in range(n_req)]
    arrivals = sorted(rng.randint(0, 12) for _ in range(n_req))
    # room for the largest request and a little more: requests are admitted while pages are
    # free and preempted when the running ones outgrow the pool
    pages = -(-(max(lens) + max(news)) // ps) + 3
    llm = LLM(d, num_blocks=pages, block_size=ps, max_concurrent=4, dtype="float32",
              chunk_size=rng.choice([8, 16, 32]), max_num_batched_tokens=rng.choice([24, 48, 96]))
    prompts = [random_tokens(n, cfg["vocab_size"], 300 + 10 * seed + i) for i, n in enumerate(lens)]
    reqs = [llm.make_request(p, max_new_tokens=k, sampling_params=SamplingParams(temperature=0.0),
                             ignore_eos=True) for p, k in zip(prompts, news)]
    abort_at = {i: rng.randint(1, max(1, news[i] - 1)) for i in rng.sample(range(n_req), 3)}
    aborted = set()
    pending = list(zip(arrivals, range(n_req)))
    step = 0
    while pending or llm.scheduler.has_unfinished():
        while pending and pending[0][0] <= step:
            llm.scheduler.add_request(reqs[pending.pop(0)[1]])
        llm.step()
        llm.scheduler.drain_finished()
        for i, k in abort_at.items():
            if (i not in aborted and len(reqs[i].output_tokens) >= k
                    and reqs[i].status is not RequestStatus.FINISHED):
                assert llm.abort(reqs[i])
                aborted.add(i)
        llm.engine.cache.check_consistency()
        step += 1
        assert step < 2000, "the serving loop does not come to an end"
    for i, (p, r) in enumerate(zip(prompts, reqs)):
        want = plain.greedy(cfg, w, p, news[i])
        if i in aborted:
            assert r.output_tokens == want[:len(r.output_tokens)] and len(r.output_tokens) >= 1
        else:
            assert r.output_tokens == want, f"request {i} (prompt of {lens[i]} tokens)"
    assert llm.engine.cache.free_pages() == [pages] * len(llm.engine.cache.groups)
    llm.engine.ops.check_errors()
    assert sum(r.num_preemptions for r in reqs) > 0, "the pool was meant to be too small"
    assert aborted, "some requests were meant to be taken out"


@pytest.mark.parametrize("chunks", [2, 3])
def test_decoding_with_several_chunks_per_cta(root, chunks):
    """Steps with thousands of 128-key chunks run decode attention with CTAs that walk through
    several chunks (keys and values in rings).  Tiny models never get there by themselves, so
    the choice is forced: four requests of different lengths, one of them beyond the window of
    the windowed layers, decoded together for 150 steps across chunk and page edges."""
    from somi_inference_b200.engine import Engine, StepEntry
    d = make_model("D", root, torch.bfloat16, std=STD)
    cfg, w = plain.load_folder(d)
    lens = [300, 150, 260, 33]
    steps = 150
    ids = [random_tokens(n + steps, cfg["vocab_size"], 500 + i) for i, n in enumerate(lens)]
    ref = [plain.logits(cfg, w, x) for x in ids]
    scale = max(r.abs().max().item() for r in ref)
    eng = Engine(d, dtype="bfloat16", page_size=16, max_tokens=4 * 512)
    eng.ops.set_decode_ring_chunks(chunks)
    try:
        for i, n in enumerate(lens):
            eng.step([StepEntry(i, ids[i][:n], [])])
        worst, bad, around = 0.0, [], []
        for t in range(steps):
            got = eng.step([StepEntry(i, [ids[i][n + t]], [0]) for i, n in enumerate(lens)]).float().cpu()
            errs = [(got[i] - ref[i][n + t]).abs().max().item() for i, n in enumerate(lens)]
            worst = max(worst, max(errs))
            bad += [(t, i, round(e / scale, 3)) for i, e in enumerate(errs) if not e <= 4e-2 * scale]
            if bad and t <= bad[0][0] + 2:          # every request's error at and after the first bad step
                around.append((t, [round(e / scale, 4) for e in errs]))
        eng.ops.check_errors()
    finally:
        eng.ops.set_decode_ring_chunks(0)
    assert worst <= 4e-2 * scale, (f"chunks per CTA {chunks}: {worst / scale:.3e} of the logits' scale; "
                                   f"{len(bad)} rows off, the first (step, request, error): {bad[:10]}; "
                                   f"all requests around the first: {around}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(root, dtype):
    """A 3-token prompt followed by 300 single-token steps (pages fill and follow one another),
    and the logits of the very first positions."""
    from somi_inference_b200.engine import Engine, StepEntry
    d = make_model("C", root, getattr(torch, dtype), std=STD)
    cfg, w = plain.load_folder(d)
    ids = random_tokens(303, cfg["vocab_size"], 4)
    ref = plain.logits(cfg, w, ids)
    scale = ref.abs().max().item()
    atol = 3e-5 if dtype == "float32" else 4e-2 * scale      # bounds as in test_gpu_replay.py
    eng = Engine(d, dtype=dtype, page_size=16, max_tokens=320)
    rows = [eng.step([StepEntry("x", ids[:3], [0, 1, 2])])]
    for t in ids[3:]:
        rows.append(eng.step([StepEntry("x", [t], [0])]))
    got = torch.cat(rows).float().cpu()
    err = (got - ref).abs().max(dim=1).values
    assert err.max().item() <= atol, f"first wrong position: {int(torch.nonzero(err > atol)[0])}"
    assert err[:3].max().item() <= atol


def test_parts_alone(root):
    """Each part of a layer, built through its registry with its own numbers, against the
    plain formula: norm, feed-forward, embedding and head, attention mixer over a cache."""
    from somi_inference_b200.cache import CacheManager
    from somi_inference_b200.config import PartSpec
    from somi_inference_b200.engine.batch import BatchBuilder, StepEntry
    from somi_inference_b200.ops import cuda_ops
    from somi_inference_b200.parts import (EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                                           BuildContext)
    ops = cuda_ops()

    def dense(t):        # a part may hand on float32 partial sums [splits, T, H] for the next norm
        return t.sum(0) if t.dim() == 3 else t.float()

    g = torch.Generator().manual_seed(0)
    H, I, Vv, T = 96, 200, 301, 23
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), ops=ops)
        # norm with residual sum
        wn = 1 + 0.1 * torch.randn(H, generator=g)
        norm = NORMS.build(PartSpec("rmsnorm", {"size": H, "eps": 2e-5, "names": {"weight": "n"}}),
                           {"n": ctx.place(wn, matrix=False)}, ctx)
        res, delta = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g).to(dtype)
        r = res.clone().cuda()
        out = norm.forward(r, delta.cuda())
        want = plain.rms_norm(res + delta.float(), wn, 2e-5)
        assert (out.float().cpu() - want).abs().max() < tol * 4
        assert torch.equal(r.cpu(), res + delta.float())
        # feed-forward
        ws = {k: 0.1 * torch.randn(s, generator=g) for k, s in
              (("p.mlp.gate_proj.weight", (I, H)), ("p.mlp.up_proj.weight", (I, H)),
               ("p.mlp.down_proj.weight", (H, I)))}
        ws = {k: v.to(dtype).float() for k, v in ws.items()}
        ff = FEED_FORWARDS.build(PartSpec("swiglu", {
            "hidden_size": H, "intermediate_size": I,
            "names": {"gate_weight": "p.mlp.gate_proj.weight", "up_weight": "p.mlp.up_proj.weight",
                      "down_weight": "p.mlp.down_proj.weight"}}),
            {k: ctx.place(v, matrix=True) for k, v in ws.items()}, ctx)
        x = torch.randn(T, H, generator=g).to(dtype)
        y = dense(ff.forward(x.cuda(), None))
        assert (y.cpu() - plain.swiglu(x.float(), ws, "p")).abs().max() < tol * 4
        # embedding and heads (tied and untied)
        table = (0.1 * torch.randn(Vv, H, generator=g)).to(dtype).float()
        head_w = (0.1 * torch.randn(Vv, H, generator=g)).to(dtype).float()
        placed = {"e": ctx.place(table, matrix=True), "h": ctx.place(head_w, matrix=True)}
        emb = EMBEDDINGS.build(PartSpec("token_embedding", {"vocab_size": Vv, "hidden_size": H,
                                                            "names": {"weight": "e"}}), placed, ctx)
        ids = torch.randint(0, Vv, (T,), generator=g, dtype=torch.int32)
        from types import SimpleNamespace
        assert torch.equal(emb.forward(SimpleNamespace(token_ids=ids.cuda())).cpu(), table[ids.long()])
        for tied, wm in ((True, table), (False, head_w)):
            head = HEADS.build(PartSpec("lm_head", {"vocab_size": Vv, "hidden_size": H, "tied": tied,
                                                    "names": {"weight": "h", "tied_to": "e"}}),
                               placed, ctx)
            lg = head.forward(x.cuda())
            assert lg.dtype == torch.float32
            assert (lg.cpu() - x.float() @ wm.T).abs().max() < tol * 4
        # attention mixer: two steps over its own cache against the plain block
        nq, nkv, hd = 6, 2, 16
        cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H}
        wa = {}
        for nme, shp in (("q_proj.weight", (nq * hd, H)), ("k_proj.weight", (nkv * hd, H)),
                         ("v_proj.weight", (nkv * hd, H)), ("o_proj.weight", (H, nq * hd)),
                         ("q_proj.bias", (nq * hd,)), ("k_proj.bias", (nkv * hd,)),
                         ("v_proj.bias", (nkv * hd,))):
            wa[f"p.self_attn.{nme}"] = (0.15 * torch.randn(shp, generator=g)).to(dtype).float()
        names = {f"{a}_{b}": f"p.self_attn.{a}_proj.{b}" for a in "qkvo" for b in ("weight", "bias")}
        mixer = MIXERS.build(PartSpec("attention", {
            "hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": True,
            "out_bias": False, "window": 9, "names": names,
            "position": PartSpec("rope", {"head_dim": hd, "theta": 777.0, "max_positions": 64})}),
            {k: ctx.place(v, matrix=v.dim() == 2) for k, v in wa.items()}, ctx)
        mgr = CacheManager([mixer.cache_needs()], [None], num_pages=8, page_size=4, max_requests=2,
                           max_positions=64, dtype=dtype, device="cuda")
        builder = BatchBuilder(mgr, device="cuda", q_tile_sizes=ops.q_tile_sizes)
        h = torch.randn(T, H, generator=g).to(dtype)
        cos, sin = plain.rope_tables(hd, 777.0, T)
        want = plain.attention_block(h.float(), wa, "p", cfg, cos, sin, 9)
        mgr.register("r")
        outs = []
        for a, b in ((0, 14), (14, 15), (15, T)):
            mgr.reserve("r", b - a)
            batch, _ = builder.build([StepEntry("r", [0] * (b - a), [])])
            outs.append(dense(mixer.forward(h[a:b].cuda(), batch, mgr.view(0), True)))
            mgr.commit("r")
        assert (torch.cat(outs).cpu() - want).abs().max() < tol * 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_on_the_gpu(root, dtype):
    """A mixer with state of its own, a routed feed-forward, another position encoding, an
    embedding that reads positions, a layer with four norms, a layer without a feed-forward and
    a mixer whose values are wider than its keys, all defined by the tests, run through the
    engine with the CUDA kernels for everything else."""
    from somi_inference_b200.config import register_architecture, unregister_architecture
    from somi_inference_b200.engine import Engine, StepEntry
    register_toys()
    register_architecture(toy_model.ARCH, toy_model.ToyConfig)
    try:
        d = toy_model.write_toy_model(root + f"/toy_{dtype}", dtype=getattr(torch, dtype),
                                      n_experts=3 if dtype == "float32" else 1)
        reqs = {f"t{i}": random_tokens(n, toy_model.V, 20 + i) for i, n in enumerate([45, 70, 12, 90, 33])}
        ref = {k: toy_model.plain_logits(d, v) for k, v in reqs.items()}
        scale = max(v.abs().max().item() for v in ref.values())
        atol = 3e-5 if dtype == "float32" else 4e-2 * scale
        rms = 1e-5 if dtype == "float32" else 4e-3 * scale
        for mode in (replay.whole, replay.portions, replay.mixed):
            steps, max_tokens = mode(reqs)
            eng = Engine(d, dtype=dtype, page_size=8, max_tokens=max_tokens)
            assert len(eng.cache.groups) == 3
            got = replay.run_steps(eng, steps)
            replay.compare(got, ref, atol, f"toy/{dtype}/{mode.__name__}", rms)
            assert all(f == eng.num_pages for f in eng.cache.free_pages())
    finally:
        unregister_architecture(toy_model.ARCH)
        unregister_toys()
