"""Each CUDA kernel alone against its plain reference (tests/plain/host_ops.py, on the CPU in
float32), at sizes other than the engine's tiny models: widths that are no power of two, head
sizes 16..256 in steps of 16, odd group counts, several page sizes, windows."""

import pytest
import torch

from tests.gpu_util import attention_case, batch_to_cpu
from tests.plain.host_ops import HostOps

pytestmark = pytest.mark.gpu
HOST = HostOps()
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(1000, 80, 7), (517, 896, 33), (3001, 3584, 5)])
def test_embed(ops, dtype, V, H, T):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    ids[0], ids[-1] = 0, V - 1
    out = torch.empty(T, H, dtype=torch.float32, device="cuda")
    ops.embed(ids.cuda(), table.cuda(), out)
    ref = torch.empty(T, H)
    HOST.embed(ids, table, ref)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("N,H", [(9, 80), (4, 896), (3, 3584), (2, 5120), (5, 8192),
                                 # more than 32 rows: a warp per row up to 2,048 columns
                                 (70, 896), (45, 1540), (33, 80), (100, 2048), (41, 2052)])
def test_add_rmsnorm(ops, dtype, wdtype, N, H):
    g = torch.Generator().manual_seed(2)
    res = torch.randn(N, H, generator=g) * 3
    delta = torch.randn(N, H, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(wdtype)
    eps = 3e-5
    for use_delta in (True, False):
        r_gpu = res.clone().cuda()
        out = torch.empty(N, H, dtype=dtype, device="cuda")
        ops.add_rmsnorm(r_gpu, delta.cuda() if use_delta else None, w.cuda(), eps, out)
        r_ref = res.clone()
        ref = torch.empty(N, H, dtype=dtype)
        HOST.add_rmsnorm(r_ref, delta if use_delta else None, w, eps, ref)
        torch.testing.assert_close(r_gpu.cpu(), r_ref, rtol=0, atol=0)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))
    # selected rows: residual untouched, rows gathered
    rows = torch.tensor([N - 1, 0, N // 2], dtype=torch.int32)
    r_gpu = res.clone().cuda()
    out = torch.empty(3, H, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r_gpu, delta.cuda(), w.cuda(), eps, out, rows.cuda())
    ref = torch.empty(3, H, dtype=dtype)
    HOST.add_rmsnorm(res.clone(), delta, w, eps, ref, rows)
    assert torch.equal(r_gpu.cpu(), res)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(3, 176), (17, 4864), (2, 18944)])
def test_silu_mul(ops, dtype, T, I):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(T, 2 * I, generator=g) * 4).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    ops.silu_mul(gu.cuda(), out)
    ref = torch.empty(T, I, dtype=dtype)
    HOST.silu_mul(gu, ref)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (14, 2, 64, 64, 16),
                                             (28, 4, 128, 128, 16), (3, 1, 48, 48, 8),
                                             (6, 3, 80, 32, 32), (2, 2, 256, 256, 64),
                                             (5, 5, 32, 0, 16)])
def test_rope_store(ops, dtype, nq, nkv, hd, rot, ps):
    g = torch.Generator().manual_seed(4)
    T, pages = 37, 12
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, generator=g).to(dtype)
    positions = torch.randint(0, 30000, (T,), generator=g, dtype=torch.int32)
    positions[0] = 0
    theta = 1e6
    inv_freq = (1.0 / (theta ** (torch.arange(0, max(rot, 2), 2) / max(rot, 2)))).float()
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, nkv, ps, hd, dtype=dtype)
    vc = torch.zeros(pages, nkv, ps, hd, dtype=dtype)
    q_gpu, kc_gpu, vc_gpu = qkv.clone().cuda(), kc.clone().cuda(), vc.clone().cuda()
    ops.rope_store(q_gpu, positions.cuda(), inv_freq.cuda(), nq, nkv, hd, rot, slots.cuda(),
                   kc_gpu, vc_gpu)
    q_ref = qkv.clone()
    HOST.rope_store(q_ref, positions, inv_freq, nq, nkv, hd, rot, slots, kc, vc)
    # angles reach 3e4 rad: sin/cos of the device and of the host differ by float32 rounding of
    # the reduced argument, a few 1e-7 absolute on values of size ~4
    t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(q_gpu.cpu().float(), q_ref.float(), **t)
    torch.testing.assert_close(kc_gpu.cpu().float(), kc.float(), **t)
    assert torch.equal(vc_gpu.cpu(), vc)
    # without a slot map nothing is stored
    kc2 = torch.zeros_like(kc_gpu)
    ops.rope_store(qkv.clone().cuda(), positions.cuda(), inv_freq.cuda(), nq, nkv, hd, rot, None,
                   kc2, kc2)
    assert kc2.abs().sum().item() == 0


ATT_CASES = [
    # nq nkv hd ps window requests(ctx, q)
    (4, 2, 16, 16, None, [(0, 5), (0, 17), (0, 33)]),
    (14, 2, 64, 16, None, [(0, 70), (100, 1), (37, 2), (15, 1), (64, 16)]),
    (28, 4, 128, 16, None, [(300, 1), (0, 40), (255, 1), (256, 1), (1, 1)]),
    (3, 1, 48, 8, None, [(9, 31), (0, 1), (8, 8)]),
    (6, 3, 32, 16, 24, [(0, 70), (50, 1), (23, 1), (24, 1), (25, 3), (5, 30)]),
    (5, 5, 80, 32, 7, [(40, 9), (6, 1), (7, 1)]),
    (2, 1, 256, 64, None, [(100, 3), (63, 2)]),
    (8, 1, 112, 4, 130, [(200, 20), (129, 1), (130, 1), (131, 1)]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATT_CASES, ids=[f"c{i}" for i in range(len(ATT_CASES))])
def test_paged_attention(ops, dtype, case):
    nq, nkv, hd, ps, window, reqs = case
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=ps,
                                              window=window, requests=reqs, dtype=dtype)
    out = torch.full((batch.num_tokens, nq * hd), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd,
                        hd ** -0.5, window, out)
    ref = torch.empty(batch.num_tokens, nq * hd, dtype=dtype)
    HOST.paged_attention(qkv.cpu(), view.keys.cpu(), view.values.cpu(), batch_to_cpu(batch),
                         batch_to_cpu(batch).groups[0], nq, nkv, hd, hd ** -0.5, window, ref)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 50])
def test_attention_far_key_and_window_edge(ops, dtype, window):
    """One key is made to dominate: the output must be its value, or must not see it at all.

    The dominating key is put (a) far back among hundreds, (b) in the first slot of a page,
    (c) in the last slot of a page, (d) exactly on the window's edge (seen) and (e) one position
    beyond it (hidden)."""
    nq, nkv, hd, ps = 4, 2, 64, 16
    ctx = 400
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=ps,
                                              window=window, requests=[(ctx, 1)], dtype=dtype)
    qpos = ctx
    spots = [3, 16 * 7, 16 * 9 - 1] if window is None else [qpos - window + 1, qpos - window]
    table = batch.groups[0].block_table[0].cpu()
    q = qkv.view(1, nq + 2 * nkv, hd)
    for spot in spots:
        keys = view.keys.clone()
        page, off = int(table[spot // ps]), spot % ps
        for h in range(nkv):
            keys[page, h, off] = (q[0, h * (nq // nkv)].float() * 20).to(dtype)
        out = torch.empty(1, nq * hd, dtype=dtype, device="cuda")
        store = view.storage.clone()       # the TMA kernel reads through the group's storage
        ks, vs = store[0, 0], store[0, 1]
        ks.copy_(keys)
        ops.paged_attention(qkv, ks, vs, batch, batch.groups[0], nq, nkv, hd,
                            hd ** -0.5, window, out, storage=store)
        ops.check_errors()
        got = out.view(nq, hd)[0].float()
        planted = view.values[page, 0, off].float()
        seen = window is None or spot > qpos - window
        close = torch.allclose(got, planted, rtol=2e-2, atol=2e-2)
        assert close == seen, f"key at {spot}: seen={seen}, output equals its value: {close}"


@pytest.fixture(params=["pingpong", "tcgen05"])
def prefill_kernel(request, ops):
    """Run a prompt-attention test on the two-tile tcgen05 kernel (whatever the step's size) or on
    the one-tile kernel."""
    was = ops.use_pp_prefill, ops.pp_prefill_min_ctas
    ops.use_pp_prefill, ops.pp_prefill_min_ctas = request.param == "pingpong", 0
    yield request.param
    ops.use_pp_prefill, ops.pp_prefill_min_ctas = was


@pytest.mark.parametrize("window", [None, 130])
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 128), (6, 2, 64)])
def test_prefill_attention_far_key_and_window_edge(ops, prefill_kernel, nq, nkv, hd, window):
    """The same for a prompt portion (the tcgen05 kernels): one key is made to dominate for one
    query row; that row's output must be the key's value, or must not see it.  Rows at the first
    and last position of the portion and on both sides of a 128-row tile edge; keys far back, on
    both sides of the 128-key tile edges, in the first and last slot of a page, on the diagonal,
    one beyond the diagonal (hidden), on the window's edge (seen) and one beyond it (hidden)."""
    ps, ctx, qn = 16, 300, 200
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=ps,
                                              window=window, requests=[(ctx, qn)],
                                              dtype=torch.bfloat16, seed=3)
    table = batch.groups[0].block_table[0].cpu()
    q = qkv.view(qn, nq + 2 * nkv, hd)
    G = nq // nkv
    for r in (0, 127, 128, qn - 1):
        qpos = ctx + r
        if window is None:
            spots = [5, 127, 128, 255, 256, 16 * 20, 16 * 21 - 1, qpos, qpos + 1]
        else:
            spots = [qpos - window + 1, qpos - window, qpos]
        for spot in spots:
            if spot >= ctx + qn:
                continue
            keys = view.keys.clone()
            page, off = int(table[spot // ps]), spot % ps
            for h in range(nkv):
                keys[page, h, off] = (q[r, h * G].float() * 20).to(torch.bfloat16)
            out = torch.empty(qn, nq * hd, dtype=torch.bfloat16, device="cuda")
            store = view.storage.clone()
            ks, vs = store[0, 0], store[0, 1]
            ks.copy_(keys)
            ops.paged_attention(qkv, ks, vs, batch, batch.groups[0], nq, nkv, hd, hd ** -0.5,
                                window, out, storage=store)
            ops.check_errors()
            got = out.view(qn, nq, hd)[r, 0].float()
            planted = view.values[page, 0, off].float()
            seen = spot <= qpos and (window is None or spot > qpos - window)
            close = torch.allclose(got, planted, rtol=2e-2, atol=2e-2)
            assert close == seen, (f"row {r} (position {qpos}), key at {spot}: seen={seen}, "
                                   f"output equals its value: {close}")


DECODE_CASES = [
    # nq nkv hd ps window ctx lengths (each request brings one token)
    (14, 2, 64, 16, None, [0, 1, 126, 127, 128, 129, 255, 256, 1000, 2047]),
    (28, 4, 128, 16, None, [5, 127, 128, 700, 2048]),
    (16, 1, 64, 8, None, [300, 17]),
    (3, 3, 32, 64, None, [130, 64, 63]),
    (14, 2, 64, 16, 200, [10, 199, 200, 201, 500, 383, 384, 385]),
    (8, 4, 128, 32, 128, [127, 128, 129, 1000]),
    # long contexts: many chunks per request
    (14, 2, 64, 16, None, [3900, 100, 2300]),
    (4, 2, 128, 16, None, [5000, 3]),
    # more than 32 chunks: the merge in which the warps share the chunks, also with a window
    # (the first chunks are skipped) and at head size 32
    (14, 2, 64, 16, None, [9000, 70, 4224, 4225]),
    (6, 2, 64, 16, 6000, [9000, 6100, 5999, 12]),
    (3, 3, 32, 64, None, [4500, 129]),
]


@pytest.mark.parametrize("tma", [True, False, 2, 3, 8], ids=["tma", "cp_async", "ring2", "ring3", "ring8"])
@pytest.mark.parametrize("case", DECODE_CASES, ids=[f"d{i}" for i in range(len(DECODE_CASES))])
def test_split_kv_decode_attention(ops, case, tma):
    """Single-token requests around the 128-key chunk edges, with and without a window, beside
    one prompt portion; bfloat16 goes through the split-KV kernel: the one with a chunk per
    CTA, and the one whose CTAs walk through 2, 3 or 8 chunks with keys and values in rings
    (which a step chooses by itself only when it has thousands of chunks)."""
    nq, nkv, hd, ps, window, ctxs = case
    ring = 0 if isinstance(tma, bool) else tma
    tma = bool(tma)
    if ring and not ops.lib.somi_decode_tma_supported(nq, nkv, hd, ps):
        pytest.skip("the ring kernel is part of the TMA path")
    assert ops.decode_supported(nq, nkv, hd, torch.bfloat16)
    reqs = [(c, 1) for c in ctxs] + [(40, 9)]
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=ps,
                                              window=window, requests=reqs, dtype=torch.bfloat16,
                                              seed=7)
    out = torch.full((batch.num_tokens, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    before = ops.launches
    ops.use_tma_decode = tma
    ops.set_decode_ring_chunks(ring if ring else 1)
    try:
        ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd,
                            hd ** -0.5, window, out, storage=view.storage)
        ops.check_errors()
    finally:
        ops.use_tma_decode = True
        ops.set_decode_ring_chunks(0)
    assert ops.launches - before >= 2      # one kernel for the portion, the split kernel for the rest
    ref = torch.empty(batch.num_tokens, nq * hd, dtype=torch.bfloat16)
    cb = batch_to_cpu(batch)
    HOST.paged_attention(qkv.cpu(), view.keys.cpu(), view.values.cpu(), cb, cb.groups[0], nq, nkv,
                         hd, hd ** -0.5, window, ref)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(torch.bfloat16))


PREFILL_CASES = [
    # nq nkv hd ps window requests (ctx, q)
    (14, 2, 64, 16, None, [(0, 200), (100, 64), (37, 2), (63, 65), (0, 1), (500, 3)]),
    (28, 4, 128, 16, None, [(0, 130), (1000, 70), (64, 64)]),
    (6, 3, 32, 8, 24, [(0, 90), (50, 30), (23, 2), (5, 70)]),
    (4, 1, 64, 32, 100, [(0, 300), (150, 129)]),
    (2, 2, 128, 64, None, [(3, 61), (0, 64), (0, 65)]),
    (7, 1, 64, 16, None, [(0, 700), (1500, 100)]),
    (4, 2, 128, 8, 70, [(0, 400), (333, 90)]),
    # long key ranges (more than 1,024 keys for a block of queries)
    (4, 2, 128, 8, 1200, [(900, 400), (2000, 130)]),
    (3, 1, 64, 16, None, [(0, 1300), (1100, 50)]),
]


@pytest.mark.parametrize("path", ["pingpong", "tcgen05", "tma", "cp_async"])
@pytest.mark.parametrize("case", PREFILL_CASES, ids=[f"p{i}" for i in range(len(PREFILL_CASES))])
def test_tensor_core_prefill_attention(ops, case, path):
    """Portions with and without cached context, around the 64-row and 64-key tile edges,
    windows shorter and longer than a tile; bfloat16 goes through the tensor-core kernel."""
    nq, nkv, hd, ps, window, reqs = case
    assert ops.prefill_supported(nq, nkv, hd, torch.bfloat16)
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=ps,
                                              window=window, requests=reqs, dtype=torch.bfloat16,
                                              seed=11)
    out = torch.full((batch.num_tokens, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.use_pp_prefill = path == "pingpong"
    ops.pp_prefill_min_ctas, min_ctas = 0, ops.pp_prefill_min_ctas     # the tests' steps are small
    ops.use_tc_prefill = path == "tcgen05"
    ops.use_tma_prefill = path != "cp_async"
    try:
        ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd,
                            hd ** -0.5, window, out, storage=view.storage)
        ops.check_errors()
    finally:
        ops.use_tma_prefill = ops.use_tc_prefill = ops.use_pp_prefill = True
        ops.pp_prefill_min_ctas = min_ctas
    ref = torch.empty(batch.num_tokens, nq * hd, dtype=torch.bfloat16)
    cb = batch_to_cpu(batch)
    HOST.paged_attention(qkv.cpu(), view.keys.cpu(), view.values.cpu(), cb, cb.groups[0], nq, nkv,
                         hd, hd ** -0.5, window, ref)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("N", [7, 50])
def test_add_rmsnorm_sums_partial_deltas(ops, N):
    g = torch.Generator().manual_seed(5)
    H, S = 896, 5
    res = torch.randn(N, H, generator=g)
    parts = torch.randn(S, N, H, generator=g)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    r_gpu = res.clone().cuda()
    out = torch.empty(N, H, dtype=torch.bfloat16, device="cuda")
    ops.add_rmsnorm(r_gpu, parts.cuda(), w.cuda(), 1e-6, out)
    r_ref = res.clone()
    ref = torch.empty(N, H, dtype=torch.bfloat16)
    HOST.add_rmsnorm(r_ref, parts, w, 1e-6, ref)
    torch.testing.assert_close(r_gpu.cpu(), r_ref, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(torch.bfloat16))
    rows = torch.tensor([6, 2], dtype=torch.int32)
    out2 = torch.empty(2, H, dtype=torch.bfloat16, device="cuda")
    ops.add_rmsnorm(res.clone().cuda(), parts.cuda(), w.cuda(), 1e-6, out2, rows.cuda())
    torch.testing.assert_close(out2.cpu().float(), ref[rows.long()].float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("nq,nkv,hd,rot,ps", [(14, 2, 64, 64, 16), (28, 4, 128, 128, 16), (6, 3, 80, 32, 32)])
@pytest.mark.parametrize("store", [True, False])
def test_rope_store_from_partial_sums(ops, nq, nkv, hd, rot, ps, store):
    g = torch.Generator().manual_seed(6)
    T, pages, S = 9, 4, 3
    width = (nq + 2 * nkv) * hd
    parts = torch.randn(S, T, width, generator=g)
    bias = torch.randn(width, generator=g).to(torch.bfloat16)
    positions = torch.randint(0, 5000, (T,), generator=g, dtype=torch.int32)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, rot, 2) / rot))).float()
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, nkv, ps, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_gpu = torch.zeros(T, width, dtype=torch.bfloat16, device="cuda")
    kc_gpu, vc_gpu = kc.clone().cuda(), vc.clone().cuda()
    ops.rope_store(q_gpu, positions.cuda(), inv_freq.cuda(), nq, nkv, hd, rot,
                   slots.cuda() if store else None, kc_gpu, vc_gpu, partials=parts.cuda(),
                   bias=bias.cuda())
    # reference: the summed projection in float32, rotated, then rounded once
    full = (parts.sum(0) + bias.float())
    q_ref = full.clone()
    kc_ref, vc_ref = kc.float(), vc.float()
    HOST.rope_store(q_ref, positions, inv_freq, nq, nkv, hd, rot, slots if store else None,
                    kc_ref, vc_ref)
    t = dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(q_gpu.cpu().float()[:, :nq * hd], q_ref[:, :nq * hd], **t)
    if store:
        torch.testing.assert_close(kc_gpu.cpu().float(), kc_ref, **t)
        torch.testing.assert_close(vc_gpu.cpu().float(), vc_ref, **t)
    else:
        assert kc_gpu.abs().sum().item() == 0 and vc_gpu.abs().sum().item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(3, 176), (5, 4864), (2, 90)])
def test_silu_mul_interleaved(ops, dtype, T, I):
    g = torch.Generator().manual_seed(8)
    gu = (torch.randn(T, 2 * I, generator=g) * 3).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    ops.silu_mul(gu.cuda(), out, interleaved=True)
    ref = torch.empty(T, I, dtype=dtype)
    HOST.silu_mul(gu, ref, interleaved=True)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("nq,nkv,hd,reqs", [
    (4, 2, 128, [(300, 200), (0, 129)]),          # prompt portions: the tcgen05 kernel
    (6, 2, 64, [(0, 300), (100, 64)]),
    (14, 2, 64, [(2047, 1), (128, 1), (5, 1)]),    # single tokens: the split-KV kernel and its merge
    (8, 4, 128, [(1000, 1), (127, 1)]),
])
def test_attention_launched_alone_many_times(ops, nq, nkv, hd, reqs):
    """Each launch on an idle GPU with a synchronisation before and after: whatever a kernel's
    warps hand to one another without an order would show as a result that changes from launch
    to launch, or as a wait that runs out."""
    mgr, batch, qkv, view, _ = attention_case(ops, nq=nq, nkv=nkv, hd=hd, page_size=16, window=None,
                                              requests=reqs, dtype=torch.bfloat16, seed=21)
    first = None
    for i in range(30):
        out = torch.full((batch.num_tokens, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        ops.paged_attention(qkv, view.keys, view.values, batch, batch.groups[0], nq, nkv, hd,
                            hd ** -0.5, None, out, storage=view.storage)
        torch.cuda.synchronize()
        if first is None:
            first = out.clone()
            assert not torch.isnan(first.float()).any()
        else:
            assert torch.equal(out, first), f"launch {i} differs from the first"
    ops.check_errors()
