"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it (the GPU's
memory belongs to their own pool, or an allocation's device-wide synchronisation is not
acceptable where they are).  `somi_paged_attention_decode_static` serves them: same inputs and
outputs as `somi_paged_attention_decode`, with the scratch in a fixed device array inside the
library.  This test calls the symbol with ctypes and compares its output with a plain float32
attention computed on the CPU (and, bit for bit, with the ordinary entry point), twice in a row
(the array keeps the first call's contents, which must not matter), checks that free device
memory does not move across a call, a call that fills the array to its last slot, and the
refusal of calls that do not fit.  The file is named so that it is collected last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from somi_inference_b200.ops.build import build
    lib = ctypes.CDLL(build())
    lib.somi_paged_attention_decode_static_capacity.restype = ctypes.c_longlong
    lib.somi_paged_attention_decode_static_strerror.restype = ctypes.c_char_p
    return lib


def _case(seed, n_req, nq, nkv, hd, ps, ctxs):
    g = torch.Generator().manual_seed(seed)
    pages_per_req = [-(-(c + 1) // ps) for c in ctxs]
    n_pages = sum(pages_per_req) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(pages_per_req)
    table = torch.full((n_req, width), -1, dtype=torch.int32)
    k = 0
    for r, n in enumerate(pages_per_req):
        table[r, :n] = torch.tensor(perm[k:k + n], dtype=torch.int32)
        k += n
    kc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(n_pages, nkv, ps, hd, generator=g).to(torch.bfloat16).cuda()
    qkv = torch.randn(n_req, (nq + 2 * nkv) * hd, generator=g).to(torch.bfloat16).cuda()
    ctx = torch.tensor(ctxs, dtype=torch.int32).cuda()
    return qkv, kc, vc, table.cuda(), ctx, width


def _plain(qkv, kc, vc, table, ctx, nq, nkv, hd, ps, window):
    """Attention of one new token per request over its cached keys and its own, in float32 on
    the CPU: the new token's key and value are already in the cache at position ctx."""
    qkv, kc, vc, table = qkv.float().cpu(), kc.float().cpu(), vc.float().cpu(), table.cpu()
    out = torch.zeros(qkv.shape[0], nq * hd)
    for r, c in enumerate(ctx.cpu().tolist()):
        n = c + 1
        first = max(0, n - window) if window else 0
        pos = torch.arange(first, n)
        pages = table[r, pos // ps].long()
        for h in range(nq):
            kvh = h // (nq // nkv)
            q = qkv[r, h * hd:(h + 1) * hd]
            k = kc[pages, kvh, pos % ps]                  # [keys, hd]
            v = vc[pages, kvh, pos % ps]
            p = torch.softmax((k @ q) * hd ** -0.5, dim=0)
            out[r, h * hd:(h + 1) * hd] = p @ v
    return out


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(lib, static, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits):
    n = qkv.shape[0]
    out = torch.full((n, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [_p(qkv), ctypes.c_int(qkv.shape[1]), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(n),
              _p(kc), _p(vc), _p(table), ctypes.c_int(width), _p(ctx), ctypes.c_int(nq),
              ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(ps), ctypes.c_float(hd ** -0.5),
              ctypes.c_int(window)]
    if static:
        rc = lib.somi_paged_attention_decode_static(*common, ctypes.c_int(max_splits), _p(out), stream)
    else:
        part_o = torch.empty(n * nq * max_splits * hd, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(n * nq * max_splits * 2, dtype=torch.float32, device="cuda")
        rc = lib.somi_paged_attention_decode(*common, _p(part_o), _p(part_ml),
                                             ctypes.c_int(max_splits), _p(out), stream)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_entry_point_matches_plain_attention():
    lib = _lib()
    assert lib.somi_paged_attention_decode_static_capacity() == 2 << 20
    nq, nkv, hd, ps = 14, 2, 64, 16
    # two different batches in a row: the second call finds the first call's partial results
    for seed, ctxs, window in ((1, [700, 5, 129, 1023, 256], 0), (2, [90, 2047, 300], 200)):
        qkv, kc, vc, table, ctx, width = _case(seed, len(ctxs), nq, nkv, hd, ps, ctxs)
        max_splits = -(-width * ps // 128)
        want = _plain(qkv, kc, vc, table, ctx, nq, nkv, hd, ps, window)
        rc, got = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits)
        assert rc == 0, lib.somi_paged_attention_decode_static_strerror(rc)
        assert not torch.isnan(got.float()).any()
        # the tolerance the kernel tests use for bfloat16 against a float32 reference
        torch.testing.assert_close(got.float().cpu(), want, rtol=1.6e-2, atol=1e-2)
        # the ordinary entry point runs the same kernels over caller-provided scratch: same bits
        rc_ref, ref = _call(lib, False, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits)
        assert rc_ref == 0 and torch.equal(got, ref)
        # a second call in a row, with free device memory read before and after it
        torch.cuda.synchronize()
        out = torch.full_like(got, float("nan"))
        n = qkv.shape[0]
        args = [_p(qkv), ctypes.c_int(qkv.shape[1]), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(n),
                _p(kc), _p(vc), _p(table), ctypes.c_int(width), _p(ctx), ctypes.c_int(nq),
                ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(ps), ctypes.c_float(hd ** -0.5),
                ctypes.c_int(window), ctypes.c_int(max_splits), _p(out),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)]
        free_before = torch.cuda.mem_get_info()[0]
        rc2 = lib.somi_paged_attention_decode_static(*args)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before      # it allocated nothing
        assert rc2 == 0 and torch.equal(out, got)


def test_static_scratch_filled_to_its_last_slot():
    """31 requests x 5 heads x 205 chunks x (64 + 2) floats is the largest call that fits
    (31,775 slots of 66 floats in 2 Mi floats); one chunk more is refused."""
    lib = _lib()
    nq, nkv, hd, ps = 5, 1, 64, 16
    assert 31 * nq * 205 == (2 << 20) // (hd + 2)
    ctxs = [(37 * i) % 900 + 1 for i in range(31)]
    qkv, kc, vc, table, ctx, width = _case(4, 31, nq, nkv, hd, ps, ctxs)
    want = _plain(qkv, kc, vc, table, ctx, nq, nkv, hd, ps, 0)
    rc, got = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, 0, 205)
    assert rc == 0, lib.somi_paged_attention_decode_static_strerror(rc)
    torch.testing.assert_close(got.float().cpu(), want, rtol=1.6e-2, atol=1e-2)
    rc, out = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, 0, 206)
    assert rc == 10002 and torch.isnan(out.float()).all()


def test_static_scratch_refuses_what_does_not_fit():
    lib = _lib()
    nq, nkv, hd, ps = 14, 2, 64, 16
    qkv, kc, vc, table, ctx, width = _case(3, 2, nq, nkv, hd, ps, [10, 20])
    too_many = (2 << 20) // (2 * nq * (hd + 2)) + 1
    rc, out = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, 0, too_many)
    assert rc == 10002
    assert b"static scratch" in lib.somi_paged_attention_decode_static_strerror(rc)
    assert torch.isnan(out.float()).all()          # nothing was launched
    # sizes whose product wraps around 64 bits must not pass the capacity test
    rc, out = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, 0, 2 ** 31 - 1)
    assert rc == 10002 and torch.isnan(out.float()).all()
    rc, _ = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, 48, ps, 0, 1)
    assert rc == 10001
