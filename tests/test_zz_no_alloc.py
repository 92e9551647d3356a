"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it (the GPU's
memory belongs to their own pool, or an allocation's device-wide synchronisation is not
acceptable where they are).  `somi_paged_attention_decode_static` serves them: same inputs and
outputs as `somi_paged_attention_decode`, with the scratch in a fixed device array inside the
library.  This test calls both symbols with ctypes on the same inputs, twice in a row (the
array keeps the first call's contents, which must not matter), and checks the refusal of a
call that does not fit.  The file is named so that it is collected last.
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


def test_static_scratch_entry_point_matches_the_ordinary_one():
    lib = _lib()
    assert lib.somi_paged_attention_decode_static_capacity() == 2 << 20
    nq, nkv, hd, ps = 14, 2, 64, 16
    # two different batches in a row: the second call finds the first call's partial results
    for seed, ctxs, window in ((1, [700, 5, 129, 1023, 256], 0), (2, [90, 2047, 300], 200)):
        qkv, kc, vc, table, ctx, width = _case(seed, len(ctxs), nq, nkv, hd, ps, ctxs)
        max_splits = -(-width * ps // 128)
        rc_ref, ref = _call(lib, False, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits)
        rc, got = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits)
        assert rc_ref == 0 and rc == 0, lib.somi_paged_attention_decode_static_strerror(rc)
        assert not torch.isnan(got.float()).any()
        # the tolerance the kernel tests use for bfloat16; the two paths run the same kernels
        torch.testing.assert_close(got.float(), ref.float(), rtol=1.6e-2, atol=1e-2)
        rc2, again = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, window, max_splits)
        assert rc2 == 0 and torch.equal(again, got)


def test_static_scratch_refuses_what_does_not_fit():
    lib = _lib()
    nq, nkv, hd, ps = 14, 2, 64, 16
    qkv, kc, vc, table, ctx, width = _case(3, 2, nq, nkv, hd, ps, [10, 20])
    too_many = (2 << 20) // (2 * nq * (hd + 2)) + 1
    rc, out = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, hd, ps, 0, too_many)
    assert rc == 10002
    assert b"static scratch" in lib.somi_paged_attention_decode_static_strerror(rc)
    assert torch.isnan(out.float()).all()          # nothing was launched
    rc, _ = _call(lib, True, qkv, kc, vc, table, ctx, width, nq, nkv, 48, ps, 0, 1)
    assert rc == 10001
