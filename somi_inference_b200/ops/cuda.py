"""The kernel table of the product path: thin ctypes wrappers over `csrc/`.

Every method checks what its kernel cannot check (devices, dtypes, contiguity),
launches on torch's current stream and raises if the launch failed.  There is no
other implementation behind these calls: without a CUDA device or without the
compiled library, construction fails.
"""

from __future__ import annotations

import ctypes

import torch

from . import trace
from .build import build as _build_library

_F32, _BF16 = 0, 1
ERR_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("the kernels of this engine run on a CUDA device only; got a "
                              f"{t.device} tensor")
        if not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


class CudaOps:
    name = "cuda"

    def __init__(self) -> None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
        self.lib_path = _build_library()
        self.lib = ctypes.CDLL(self.lib_path)
        self.lib.somi_attention_generic_q_tile.restype = ctypes.c_int
        self.generic_q_tile = int(self.lib.somi_attention_generic_q_tile())
        self.lib.somi_prefill_q_tile.restype = ctypes.c_int
        self.prefill_q_tile = int(self.lib.somi_prefill_q_tile())
        self.lib.somi_prefill_tc_q_tile.restype = ctypes.c_int
        self.prefill_tc_q_tile = int(self.lib.somi_prefill_tc_q_tile())
        self.lib.somi_prefill_pp_q_tile.restype = ctypes.c_int
        self.prefill_pp_q_tile = int(self.lib.somi_prefill_pp_q_tile())
        self.q_tile_sizes = (self.generic_q_tile, self.prefill_q_tile, self.prefill_tc_q_tile,
                             self.prefill_pp_q_tile)
        self.use_pp_prefill = True
        self.pp_prefill_min_ctas = torch.cuda.get_device_properties(0).multi_processor_count
        self.use_tc_prefill = True
        self._q_maps: dict = {}
        self.lib.somi_decode_chunk.restype = ctypes.c_int
        self.decode_chunk = int(self.lib.somi_decode_chunk())
        self._workspace = None
        self._device_index = torch.cuda.current_device()
        self._tensor_maps: dict = {}
        self.use_tma_decode = True
        self.lib.somi_decode_ring_chunks.argtypes = [ctypes.c_int]
        self.lib.somi_decode_ring_chunks.restype = None
        self.use_tma_prefill = True
        self._gemm_maps: dict = {}
        self.use_skinny_gemm = True
        self.skinny_max_tokens = int(self.lib.somi_skinny_gemm_max_tokens())
        self._retired: list = []
        self.launches = 0     # kernels of this library launched so far

    # ------------------------------------------------------------------ util
    def _stream(self) -> ctypes.c_void_p:
        # the raw handle of the current stream, without the Python stream object in between:
        # that path costs microseconds per launch, which a step of hundreds of launches feels
        return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(self._device_index))

    def _done(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc == ERR_UNSUPPORTED:
            raise KernelError(f"{what}: these sizes are not supported by the kernel")
        if rc != 0:
            raise KernelError(f"{what}: CUDA error {rc}")

    def check_attention_geometry(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"head_dim {head_dim} is not supported: the attention kernels take "
                              "multiples of 16 from 16 to 256")
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise KernelError(f"{num_heads} query heads cannot be grouped over {num_kv_heads} "
                              "key/value heads")

    # --------------------------------------------------------------- kernels
    def embed(self, ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
        _check(ids, table, out)
        assert ids.dtype == torch.int32 and out.dtype == torch.float32
        rc = self.lib.somi_embed(_ptr(ids), _ptr(table), _code(table), _ptr(out),
                                 ctypes.c_int(ids.shape[0]), ctypes.c_int(table.shape[1]),
                                 self._stream())
        self._done(rc, "embed")
        if trace.active():
            n = ids.shape[0] * table.shape[1]
            trace.note("embed", n * (table.element_size() + 4))

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None) -> None:
        """residual += delta (float32, in place); out = rmsnorm(residual) * weight.

        `delta` is [N, H] in the compute dtype, or float32 [splits, N, H] partial sums that are
        added in order.  With `rows`, only those rows are produced and residual is not written.
        """
        _check(residual, delta, weight, out, rows)
        assert residual.dtype == torch.float32
        H = residual.shape[1]
        n_out = out.shape[0]
        splits, stride = 1, 0
        if delta is not None and delta.dim() == 3:
            assert delta.dtype == torch.float32
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        rc = self.lib.somi_add_rmsnorm(
            _ptr(residual), _ptr(delta), _code(delta) if delta is not None else _F32,
            ctypes.c_int(splits), ctypes.c_longlong(stride),
            _ptr(weight), _code(weight), ctypes.c_float(eps), _ptr(out), _code(out), _ptr(rows),
            ctypes.c_int(n_out), ctypes.c_int(H), ctypes.c_int(0 if rows is not None else 1),
            self._stream())
        self._done(rc, "add_rmsnorm")
        if trace.active():
            n = n_out * H
            moved = n * (4 + out.element_size()) + H * weight.element_size()
            if delta is not None:
                moved += splits * n * delta.element_size()
            if rows is None:
                moved += n * 4
            trace.note("add_rmsnorm", moved, detail=f"splits={splits}" if splits > 1 else "")

    def rope_store(self, qkv, positions, inv_freq, nq, nkv, hd, rotary_dim, slot_map, kcache,
                   vcache, partials=None, bias=None) -> None:
        """Rotate q and k of `qkv` in place and store k, v at their cache slots.

        With `partials` (float32 [splits, T, width], the output of a split-K projection) the
        projection is summed here, `bias` added, and `qkv` (bfloat16) only receives the queries.
        """
        _check(qkv, positions, inv_freq, slot_map, kcache, vcache, partials, bias)
        page_size = kcache.shape[2] if kcache is not None else 1
        if kcache is not None and slot_map is not None:
            assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
        if partials is not None:
            assert partials.dtype == torch.float32 and qkv.dtype == torch.bfloat16
            rc = self.lib.somi_rope_store_partial(
                _ptr(partials), ctypes.c_int(partials.shape[0]),
                ctypes.c_longlong(partials.shape[1] * partials.shape[2]), _ptr(bias),
                _code(bias) if bias is not None else _F32, _ptr(qkv), _ptr(positions),
                _ptr(inv_freq), ctypes.c_int(qkv.shape[0]), ctypes.c_int(nq), ctypes.c_int(nkv),
                ctypes.c_int(hd), ctypes.c_int(rotary_dim), _ptr(slot_map), _ptr(kcache),
                _ptr(vcache), ctypes.c_int(page_size), self._stream())
            self._done(rc, "rope_store_partial")
            if trace.active():
                n = qkv.shape[0] * qkv.shape[1]
                trace.note("rope_store", partials.shape[0] * n * 4 + n * 2, detail="from partial sums")
            return
        rc = self.lib.somi_rope_store(
            _ptr(qkv), _code(qkv), _ptr(positions), _ptr(inv_freq), ctypes.c_int(qkv.shape[0]),
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(rotary_dim),
            _ptr(slot_map), _ptr(kcache), _ptr(vcache), ctypes.c_int(page_size), self._stream())
        self._done(rc, "rope_store")
        if trace.active():
            n = qkv.shape[0] * qkv.shape[1]
            trace.note("rope_store", n * qkv.element_size() * 2)

    def _scratch(self, n_floats: int, device) -> torch.Tensor:
        """Float32 scratch that outlives the call (kernels of a captured graph keep its address)."""
        if self._workspace is None or self._workspace.numel() < n_floats:
            if self._workspace is not None:
                self._retired.append(self._workspace)
            self._workspace = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        return self._workspace

    def prefill_supported(self, nq: int, nkv: int, hd: int, dtype) -> bool:
        return dtype == torch.bfloat16 and bool(self.lib.somi_prefill_supported(
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd)))

    def decode_supported(self, nq: int, nkv: int, hd: int, dtype) -> bool:
        return dtype == torch.bfloat16 and bool(self.lib.somi_decode_supported(
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd)))

    def _kv_tensor_map(self, storage: torch.Tensor, hd: int, page_size: int):
        """A TMA tensor map over a cache group's whole storage, seen as [rows, hd] bfloat16."""
        key = (storage.data_ptr(), storage.numel(), hd, page_size)
        entry = self._tensor_maps.get(key)
        if entry is None:
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_kv_tensor_map(ctypes.c_void_p(addr), _ptr(storage),
                                                  ctypes.c_longlong(storage.numel() // hd),
                                                  ctypes.c_int(hd), ctypes.c_int(page_size))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over the cache (code {rc})")
            entry = (raw, addr)
            self._tensor_maps[key] = entry
        return entry[1]

    def set_decode_ring_chunks(self, chunks: int) -> None:
        """Chunks of 128 keys that one CTA of the TMA decode kernel walks through: 0 lets the
        launcher choose from the step's size (the default), 1 forces the one-chunk kernel,
        2..8 the ring kernel with that many."""
        self.lib.somi_decode_ring_chunks(int(chunks))

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for all kernels of the library (on by default)."""
        self.lib.somi_set_pdl(ctypes.c_int(1 if on else 0))

    def _q_tensor_map(self, qkv: torch.Tensor) -> int:
        key = (qkv.data_ptr(), qkv.shape[0], qkv.shape[1])
        entry = self._q_maps.get(key)
        if entry is None:
            if len(self._q_maps) > 4096:
                self._q_maps.clear()
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_q_tensor_map(ctypes.c_void_p(addr), _ptr(qkv),
                                                 ctypes.c_longlong(qkv.shape[0]),
                                                 ctypes.c_longlong(qkv.shape[1]))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over the projection buffer (code {rc})")
            entry = (raw, addr)
            self._q_maps[key] = entry
        return entry[1]

    def check_errors(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out (synchronises)."""
        if int(self.lib.somi_decode_tma_error()) != 0:
            raise KernelError("the TMA decode attention kernel gave up waiting for a copy; "
                              "its results are not valid")
        if int(self.lib.somi_prefill_tma_error()) != 0:
            raise KernelError("the TMA prefill attention kernel gave up waiting for a copy; "
                              "its results are not valid")
        if int(self.lib.somi_prefill_pp_error()) != 0:
            raise KernelError("the two-tile tcgen05 prefill attention kernel gave up waiting on a "
                              "barrier; its results are not valid")
        if int(self.lib.somi_prefill_tc_error()) != 0:
            raise KernelError("the tcgen05 prefill attention kernel gave up waiting on a barrier; "
                              "its results are not valid")
        if int(self.lib.somi_gemm_error()) != 0:
            raise KernelError("the tcgen05 matrix product gave up waiting on a barrier; "
                              "its results are not valid")

    @staticmethod
    def _attention_work(batch, first: int, last: int, nq: int, nkv: int, hd: int, elt: int,
                        window: int) -> tuple[float, float]:
        """Bytes and flops of attention for requests [first, last) of the batch: every key and
        value of a request's context once, queries in and outputs out; two products per
        (query, key) pair that the mask leaves."""
        moved = flops = 0.0
        cu, ctx = batch.host.cu_q, batch.host.ctx_len
        for r in range(first, last):
            q, c = int(cu[r + 1] - cu[r]), int(ctx[r])
            pairs = q * c + q * (q + 1) // 2
            kv = c + q
            if window:
                pairs = sum(min(c + i + 1, window) for i in range(q)) if q < 4096 else min(pairs, q * window)
                kv = min(kv, window + q - 1)
            moved += 2 * kv * nkv * hd * elt + 2 * q * nq * hd * elt
            flops += 4.0 * nq * hd * pairs
        return moved, flops

    def paged_attention(self, qkv, kcache, vcache, batch, group, nq, nkv, hd, scale, window,
                        out, storage=None) -> None:
        """Attention of every token of the step over the cache (keys/values already stored).

        In bfloat16 with head sizes 32/64/128, portions of prompts go to the tensor-core
        prefill kernel and single-token requests to the split-KV kernel (at most 16 query
        heads per kv head); float32 and every other size go to the generic kernel.
        """
        _check(qkv, kcache, vcache, out, group.block_table)
        assert kcache.dtype == qkv.dtype
        page_size = kcache.shape[2]
        win = int(window) if window else 0
        n_decode = batch.num_requests - batch.num_prefill_requests
        split = n_decode > 0 and self.decode_supported(nq, nkv, hd, qkv.dtype)
        tensor_core_prefill = (batch.num_prefill_requests > 0
                               and self.prefill_supported(nq, nkv, hd, qkv.dtype))
        if tensor_core_prefill:
            # Four kernels, the first that takes the sizes: both products on tcgen05 with
            # accumulators in tensor memory, two query tiles per CTA in ping-pong and the
            # probabilities handed on through tensor memory; the same with one query tile per CTA
            # and the probabilities through shared memory; mma.sync fed by TMA; mma.sync fed by
            # cp.async gathers.
            sizes = (ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(page_size))
            row_bytes = hd * 2
            # (the two-tile kernel has half as many CTAs: below one per SM the one-tile kernel,
            # with twice as many, is the faster: 0.5B shape at 2,048 tokens 123 vs 148 TFLOP/s)
            if (self.use_pp_prefill and storage is not None and qkv.shape[1] % 8 == 0
                    and batch.tiles[self.prefill_pp_q_tile].shape[0] * nq >= self.pp_prefill_min_ctas
                    and bool(self.lib.somi_prefill_pp_supported(*sizes))):
                tiles = batch.tiles[self.prefill_pp_q_tile]
                rc = self.lib.somi_paged_attention_prefill_pp(
                    ctypes.c_void_p(self._q_tensor_map(qkv)),
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_pp")
                kernel = "attention_prefill_tcgen05_pingpong"
            elif (self.use_tc_prefill and storage is not None and qkv.shape[1] % 8 == 0
                    and bool(self.lib.somi_prefill_tc_supported(*sizes))):
                tiles = batch.tiles[self.prefill_tc_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tc(
                    ctypes.c_void_p(self._q_tensor_map(qkv)),
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tc")
                kernel = "attention_prefill_tcgen05"
            elif (self.use_tma_prefill and storage is not None
                  and bool(self.lib.somi_prefill_tma_supported(*sizes))):
                tiles = batch.tiles[self.prefill_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tma(
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)), _ptr(qkv),
                    ctypes.c_int(qkv.shape[1]),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tma")
                kernel = "attention_prefill_tma"
            else:
                tiles = batch.tiles[self.prefill_q_tile]
                rc = self.lib.somi_paged_attention_prefill(
                    _ptr(qkv), ctypes.c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill")
                kernel = "attention_prefill_cp_async"
            if trace.active():
                trace.note(kernel, *self._attention_work(batch, 0, batch.num_prefill_requests, nq,
                                                         nkv, hd, qkv.element_size(), win))
        tiles = batch.tiles[self.generic_q_tile]
        n_generic_tiles = 0 if tensor_core_prefill else tiles.shape[0]
        n_generic_decode = 0 if split else n_decode
        if n_generic_tiles + n_generic_decode > 0:
            rc = self.lib.somi_paged_attention_generic(
                _ptr(qkv), _code(qkv), ctypes.c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache),
                _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(n_generic_tiles),
                ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(batch.num_prefill_tokens),
                ctypes.c_int(n_generic_decode), ctypes.c_int(nq), ctypes.c_int(nkv),
                ctypes.c_int(hd), ctypes.c_int(page_size), ctypes.c_float(scale),
                ctypes.c_int(win), _ptr(out), self._stream())
            self._done(rc, "paged_attention")
            if trace.active():
                first = batch.num_prefill_requests if tensor_core_prefill else 0
                last = batch.num_prefill_requests if split else batch.num_requests
                trace.note("attention_generic", *self._attention_work(
                    batch, first, last, nq, nkv, hd, qkv.element_size(), win))
        if split:
            chunk = self.decode_chunk
            max_splits = -(-group.width * page_size // chunk)
            n_o = n_decode * nq * max_splits * hd
            ws = self._scratch(n_o + n_decode * nq * max_splits * 2, qkv.device)
            tma = (self.use_tma_decode and storage is not None and bool(
                self.lib.somi_decode_tma_supported(ctypes.c_int(nq), ctypes.c_int(nkv),
                                                   ctypes.c_int(hd), ctypes.c_int(page_size))))
            if tma:
                row_bytes = hd * 2
                k_row0 = (kcache.data_ptr() - storage.data_ptr()) // row_bytes
                v_row0 = (vcache.data_ptr() - storage.data_ptr()) // row_bytes
                rc = self.lib.somi_paged_attention_decode_tma(
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)), _ptr(qkv),
                    ctypes.c_int(qkv.shape[1]), ctypes.c_int(batch.num_prefill_tokens),
                    ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(n_decode),
                    ctypes.c_longlong(k_row0), ctypes.c_longlong(v_row0),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.ctx_len),
                    ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd),
                    ctypes.c_int(page_size), ctypes.c_float(scale), ctypes.c_int(win),
                    ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(ws.data_ptr() + 4 * n_o),
                    ctypes.c_int(max_splits), _ptr(out), self._stream())
            else:
                rc = self.lib.somi_paged_attention_decode(
                    _ptr(qkv), ctypes.c_int(qkv.shape[1]), ctypes.c_int(batch.num_prefill_tokens),
                    ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(n_decode),
                    _ptr(kcache), _ptr(vcache), _ptr(group.block_table),
                    ctypes.c_int(group.width), _ptr(batch.ctx_len), ctypes.c_int(nq),
                    ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(page_size),
                    ctypes.c_float(scale), ctypes.c_int(win), ctypes.c_void_p(ws.data_ptr()),
                    ctypes.c_void_p(ws.data_ptr() + 4 * n_o), ctypes.c_int(max_splits),
                    _ptr(out), self._stream())
            self._done(rc, "paged_attention_decode")
            if max_splits > 1:
                self.launches += 1
            if trace.active():
                trace.note("attention_decode_tma" if tma else "attention_decode_cp_async",
                           *self._attention_work(batch, batch.num_prefill_requests,
                                                 batch.num_requests, nq, nkv, hd,
                                                 qkv.element_size(), win),
                           detail="with merge" if max_splits > 1 else "")

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
        """out = silu(gate) * up; gate/up are the two halves of `gu`'s rows, or alternate."""
        _check(gu, out)
        rc = self.lib.somi_silu_mul(_ptr(gu), _ptr(out), _code(gu), ctypes.c_longlong(gu.shape[0]),
                                    ctypes.c_int(out.shape[1]), ctypes.c_int(1 if interleaved else 0),
                                    self._stream())
        self._done(rc, "silu_mul")
        if trace.active():
            trace.note("silu_mul", (gu.numel() + out.numel()) * gu.element_size())

    # ------------------------------------------------------- tcgen05 matrix product
    GEMM_BF16, GEMM_F32, GEMM_PARTIAL_F32, GEMM_SWIGLU = 0, 1, 2, 3

    def skinny_splits(self, M: int, N: int, K: int) -> int:
        """How many ranges of K to run side by side: CTAs for about one and a half per SM, at
        least three K blocks each, at most eight (the consumer reads every partial sum: 4 *
        splits * M * N bytes, written and read back), and partial sums that stay below a quarter
        of the weight's own bytes.  Measured with the consumer (norm or rotary kernel) behind
        each product in CUDA graphs, 1 and 8 tokens: more splits than this cost the 0.5B shape's
        down projection 1.2 µs (16 -> 8) and the 7B shape's output projection 0.4 µs (10 -> 8);
        past two CTAs per SM a product takes a third longer."""
        tiles = -(-N // 128)
        k_blocks = -(-K // 64)
        return max(1, min(224 // tiles, k_blocks // 3, K // (16 * M), 8))

    def skinny_supported(self, M: int, N: int, K: int, dtype) -> bool:
        """Whether the tensor-memory kernel takes x[M, K] @ w[N, K]^T (few tokens, bfloat16)."""
        if not (self.use_skinny_gemm and dtype == torch.bfloat16
                and 1 <= M <= self.skinny_max_tokens and K % 8 == 0 and N >= 1):
            return False
        # measured (CUDA graphs of back-to-back products with their consumers, and whole decode
        # steps at batch 32 and 64): above 16 tokens this kernel wins only where a CTA streams a
        # long K range, of a large matrix or of one that is several times as long as it is wide
        # (the 0.5B shape's down projection at 24-64 tokens: 7.8-9.5 µs against the library's
        # 11.4-11.7); short K (few stages per CTA) and small matrices go to the library
        return M <= 16 or (K >= 2048 and (N * K >= (32 << 20) or K >= 4 * N))

    def _gemm_map(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), t.shape[0], t.shape[1], box_rows)
        entry = self._gemm_maps.get(key)
        if entry is None:
            if len(self._gemm_maps) > 8192:
                self._gemm_maps.clear()
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_gemm_tensor_map(ctypes.c_void_p(addr), _ptr(t),
                                                    ctypes.c_longlong(t.shape[0]),
                                                    ctypes.c_longlong(t.shape[1]),
                                                    ctypes.c_int(box_rows))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over a {tuple(t.shape)} matrix (code {rc})")
            entry = (raw, addr)
            self._gemm_maps[key] = entry
        return entry[1]

    def skinny_gemm(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                    mode: int = 0, splits: int = 1, deep_ring: bool = False) -> torch.Tensor:
        """x[M, K] @ w[N, K]^T on tcgen05 tensor cores for M <= 64.

        mode GEMM_BF16 -> bf16 [M, N] (+ bias); GEMM_F32 -> float32 [M, N];
        GEMM_PARTIAL_F32 -> float32 [splits', M, N] partial sums over ranges of K (bias in the
        first); GEMM_SWIGLU -> bf16 [M, N / 2] = silu(even rows) * odd rows of w.
        """
        _check(x, w, bias)
        M, K = x.shape
        N = w.shape[0]
        assert w.shape[1] == K and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        box = 16 if M <= 16 else (32 if M <= 32 else 64)
        if mode == self.GEMM_PARTIAL_F32:
            splits = int(self.lib.somi_skinny_gemm_splits(ctypes.c_int(K), ctypes.c_int(splits)))
            out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        elif mode == self.GEMM_F32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        elif mode == self.GEMM_SWIGLU:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        else:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        # few CTAs: one per SM with the whole shared memory as an 8-stage ring (a CTA's stream
        # is bound by the bytes it keeps in flight); many CTAs: two per SM with 4 stages each
        ctas = -(-N // 128) * (splits if mode == self.GEMM_PARTIAL_F32 else 1)
        deep_ring = deep_ring or ctas <= 148
        rc = self.lib.somi_skinny_gemm(
            ctypes.c_void_p(self._gemm_map(w, 128)), ctypes.c_void_p(self._gemm_map(x, box)),
            ctypes.c_int(box), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_int(splits), ctypes.c_int(mode), _ptr(bias),
            _code(bias) if bias is not None else _F32, _ptr(out),
            ctypes.c_int(1 if deep_ring else 0), self._stream())
        self._done(rc, "skinny_gemm")
        if trace.active():
            trace.note("skinny_gemm", (N * K + M * K) * 2 + out.numel() * out.element_size(),
                       2.0 * M * N * K, detail=f"M={M} N={N} K={K} mode={mode}")
        return out

    def gemm_f32(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """x[M, K] @ w[N, K]^T (+ bias) in float32 FMAs, each output summed over K in ascending
        order (the float32 path's product; the library's is not used there)."""
        _check(x, w, bias)
        M, K = x.shape
        N = w.shape[0]
        if not (x.dtype == w.dtype == torch.float32 and w.shape[1] == K
                and (bias is None or (bias.dtype == torch.float32 and bias.numel() == N))):
            raise KernelError("gemm_f32 takes float32 x[M, K], w[N, K] and bias[N]")
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        rc = self.lib.somi_gemm_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(M),
                                    ctypes.c_int(N), ctypes.c_int(K), self._stream())
        self._done(rc, "gemm_f32")
        if trace.active():
            trace.note("gemm_f32", (N * K + M * K + M * N) * 4, 2.0 * M * N * K, detail=f"M={M} N={N} K={K}")
        return out

    def sample(self, logits, temperature, top_k, top_p, penalty, seed, counter, hist_off,
               hist_tok, out) -> None:
        """seed: int32 view of uint64 pairs [2 * rows]; counter: int32 view of uint32 [rows]."""
        _check(logits, temperature, top_k, top_p, penalty, seed, counter, hist_off, hist_tok, out)
        assert logits.dtype == torch.float32 and out.dtype == torch.int32
        assert seed.data_ptr() % 8 == 0
        rc = self.lib.somi_sample(_ptr(logits), ctypes.c_int(logits.shape[0]),
                                  ctypes.c_int(logits.shape[1]), _ptr(temperature), _ptr(top_k),
                                  _ptr(top_p), _ptr(penalty), _ptr(seed), _ptr(counter),
                                  _ptr(hist_off), _ptr(hist_tok), _ptr(out), self._stream())
        self._done(rc, "sample")
        if trace.active():
            trace.note("sample", logits.numel() * 4)

    def uniform(self, seed: int, counter: int) -> float:
        """The uniform number in [0, 1) that row (seed, counter) draws (host evaluation)."""
        self.lib.somi_sample_uniform.restype = ctypes.c_float
        return float(self.lib.somi_sample_uniform(ctypes.c_ulonglong(seed), ctypes.c_uint(counter)))


_OPS: CudaOps | None = None


def cuda_ops() -> CudaOps:
    """The process-wide kernel table (built and loaded at first use)."""
    global _OPS
    if _OPS is None:
        _OPS = CudaOps()
    return _OPS
