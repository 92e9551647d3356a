"""The kernel table restated with elementary tensor operations on the CPU.

Test-only.  It serves two purposes: (1) each function is the plain reference
that the matching CUDA kernel is compared with, at sizes other than the
engine's; (2) handed to `Engine(ops=HostOps())` it lets the host-side logic
(batch layout, cache manager, schedule of runs) be tested without a GPU.  The
product path never imports this file.
"""

from __future__ import annotations

import torch


class HostOps:
    name = "host"
    generic_q_tile = 16
    q_tile_sizes = (16, 64, 128)
    launches = 0

    def check_attention_geometry(self, num_heads, num_kv_heads, head_dim) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("heads not divisible by kv heads")

    def embed(self, ids, table, out) -> None:
        out.copy_(table[ids.long()].float())

    def skinny_supported(self, M, N, K, dtype) -> bool:
        return False

    def check_errors(self) -> None:
        pass

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None) -> None:
        if delta is not None and delta.dim() == 3:
            delta = delta.sum(0)
        if rows is None:
            if delta is not None:
                residual += delta.float()
            r = residual
        else:
            r = residual[rows.long()]
            if delta is not None:
                r = r + delta[rows.long()].float()
        inv = 1.0 / torch.sqrt(r.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((r * inv * weight.float()).to(out.dtype))

    def rope_store(self, qkv, positions, inv_freq, nq, nkv, hd, rotary_dim, slot_map, kcache,
                   vcache, partials=None, bias=None) -> None:
        T = qkv.shape[0]
        if partials is not None:
            full = partials.sum(0) + (bias.float() if bias is not None else 0.0)
            qkv.copy_(full.to(qkv.dtype))
        x = qkv.view(T, nq + 2 * nkv, hd)
        if rotary_dim:
            ang = positions.float().unsqueeze(1) * inv_freq.unsqueeze(0)     # [T, rot/2]
            c, s = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
            half = rotary_dim // 2
            qk = x[:, :nq + nkv, :rotary_dim].float()
            a, b = qk[..., :half], qk[..., half:]
            x[:, :nq + nkv, :rotary_dim] = torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)
        if slot_map is not None:
            ps = kcache.shape[2]
            page, off = slot_map.long() // ps, slot_map.long() % ps
            kcache[page, :, off, :] = x[:, nq:nq + nkv, :]
            vcache[page, :, off, :] = x[:, nq + nkv:, :]

    def paged_attention(self, qkv, kcache, vcache, batch, group, nq, nkv, hd, scale, window,
                        out, storage=None) -> None:
        T = qkv.shape[0]
        q = qkv.view(T, nq + 2 * nkv, hd)[:, :nq].float()
        ps = kcache.shape[2]
        cu, ctx = batch.cu_q.tolist(), batch.ctx_len.tolist()
        rep = nq // nkv
        for r in range(batch.num_requests):
            a, b = cu[r], cu[r + 1]
            n_kv = ctx[r] + (b - a)
            first = 0
            if window:
                first = max(0, ctx[r] - window + 1)
            pos = torch.arange(first, n_kv)
            pages = group.block_table[r].long()[pos // ps]
            assert (pages >= 0).all(), "attention would read a page that was given back"
            k = kcache[pages, :, pos % ps, :].float()      # [n, nkv, hd]
            v = vcache[pages, :, pos % ps, :].float()
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
            s = torch.einsum("thd,nhd->htn", q[a:b], k) * scale
            qpos = torch.arange(ctx[r], n_kv).view(1, -1, 1)
            kpos = pos.view(1, 1, -1)
            hide = kpos > qpos
            if window:
                hide = hide | (kpos <= qpos - window)
            s = s.masked_fill(hide, float("-inf"))
            o = torch.einsum("htn,nhd->thd", torch.softmax(s, -1), v)
            out[a:b] = o.reshape(b - a, nq * hd).to(out.dtype)

    def silu_mul(self, gu, out, interleaved=False) -> None:
        I = out.shape[1]
        if interleaved:
            g, u = gu[:, 0::2].float(), gu[:, 1::2].float()
        else:
            g, u = gu[:, :I].float(), gu[:, I:].float()
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    def sample(self, logits, temperature, top_k, top_p, penalty, seed, counter, hist_off,
               hist_tok, out) -> None:
        from tests.plain.sampler_plain import sample_row
        seeds = seed.cpu().numpy().view("uint64")
        counters = counter.cpu().numpy().view("uint32")
        for r in range(logits.shape[0]):
            hist = hist_tok[int(hist_off[r]):int(hist_off[r + 1])].tolist()
            tok, _, _ = sample_row(logits[r].cpu(), float(temperature[r]), int(top_k[r]),
                                   float(top_p[r]), float(penalty[r]), hist, int(seeds[r]),
                                   int(counters[r]))
            out[r] = tok
