"""The kernel library as the parts see it: one object per precision, bound with ctypes.

``KernelOps("float32")`` loads the exact 32-bit kernels, ``KernelOps("bfloat16")`` the
serving kernels; both offer the same operations on torch tensors.  There is no CPU
implementation behind these names: if the CUDA library cannot be compiled or loaded the
constructor raises, and every call checks that its tensors live on a CUDA device.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_c_int = ctypes.c_int
_c_float = ctypes.c_float
_ptr = ctypes.c_void_p


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class KernelError(RuntimeError):
    pass


class DeviceFailure(KernelError):
    """A kernel gave up a bounded wait: what the device computed since the last check is worthless."""


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _need(t: torch.Tensor, dtype, what: str, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor is not contiguous")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{what}: expected {dims} dimensions, got {tuple(t.shape)}")


class KernelOps:
    """Operations of one precision.  ``act_dtype`` is the dtype of activations between
    kernels (the residual stream, logits and norm weights are float32 in both)."""

    def __init__(self, dtype: str, verbose_build: bool = True):
        if dtype not in ("float32", "bfloat16"):
            raise KernelError(f"unknown dtype {dtype!r} (float32 or bfloat16)")
        self.dtype = dtype
        self.act_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.kind = "f32" if dtype == "float32" else "bf16"
        # The step function hands contexts to the kernels rounded up to this many keys.  The
        # serving kernels derive grids and record strides from that bound, and a step replayed
        # as a CUDA graph keeps what its capture derived: with the bound in steps of 256 a graph
        # serves 256 positions, and a replay launches exactly what an eager step would.
        self.key_granule = 1 if dtype == "float32" else 256
        path = build.ensure_built(self.kind, (), verbose_build)
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
        self.library_path = path
        self.lib.bw_last_error.restype = ctypes.c_char_p
        self.launches = 0  # kernels launched through this object (counted per call)
        self._attn_libs = {}
        self._verbose_build = verbose_build
        self._partials: Optional[torch.Tensor] = None  # scratch of the split products (bfloat16 path)
        self._counters: Optional[torch.Tensor] = None
        self._retired = []
        self._attn_scratch: Optional[torch.Tensor] = None
        self._fns = {}
        self._dev_index: Optional[int] = None
        self._scratch_sizes = {}
        self._kernel_counts = {}
        self._tc_tile_rows = {}
        self.legacy_attention = False  # tests set this to compare the attention kernels bit for bit
        if self.kind == "bf16":
            self.lib.bw_bf16_linear_scratch_floats.restype = ctypes.c_longlong
            self._split_rows = int(self.lib.bw_bf16_linear_split_rows())
        # One word of device memory that every kernel of this object's libraries raises when a
        # bounded wait runs out, and its pinned mirror on the host (filled by failure_poll).
        self._failure_word: Optional[torch.Tensor] = None
        self._failure_host: Optional[torch.Tensor] = None
        if torch.cuda.is_available():
            self._failure_words()  # before any kernel runs: captured graphs keep the word's address

    # -- plumbing ----------------------------------------------------------------------
    def _stream(self):
        # the raw handle of torch's current stream; the private getter skips the Stream object
        # that torch.cuda.current_stream() builds, which costs more than a kernel launch
        if _raw_stream is not None:
            return ctypes.c_void_p(_raw_stream(self._device_index()))
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _device_index(self) -> int:
        if self._dev_index is None:
            self._dev_index = torch.cuda.current_device()
        return self._dev_index

    def _check(self, rc: int, name: str) -> None:
        if rc != 0:
            msg = self.lib.bw_last_error().decode("utf-8", "replace")
            raise KernelError(f"{name} failed ({rc}): {msg}")

    def _call(self, name: str, *args, lib=None, launches: int = 1) -> None:
        fn = self._fns.get(name) if lib is None else None
        if fn is None:
            fn = getattr(lib or self.lib, name)
            fn.restype = _c_int
            if lib is None:
                self._fns[name] = fn
        self._check(fn(*args), name)
        self.launches += launches

    # -- shared kernels ----------------------------------------------------------------
    def embed_rows(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
        """out[r] = table[tokens[r]] widened to float32."""
        n, width = out.shape
        _need(tokens, torch.int32, "embed_rows tokens")
        _need(out, torch.float32, "embed_rows out", 2)
        if table.dtype not in (torch.float32, torch.bfloat16) or table.shape[1] != width:
            raise KernelError("embed_rows: table must be float32 or bfloat16 of the output's width")
        _need(table, table.dtype, "embed_rows table", 2)
        self._call("bw_embed_rows", _p(table), _c_int(int(table.dtype == torch.bfloat16)), _p(tokens), _p(out),
                   _c_int(n), _c_int(width), self._stream())

    def patch_tokens(self, tokens: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, values: torch.Tensor,
                     count: int) -> None:
        """tokens[rows[i]] = values[src[i]] for i < count: tokens that the step before sampled go
        into this step's token list on the device, unread by the host."""
        for t_, what in ((tokens, "tokens"), (rows, "rows"), (src, "src"), (values, "values")):
            _need(t_, torch.int32, "patch_tokens " + what)
        self._call("bw_patch_tokens", _p(tokens), _p(rows), _p(src), _p(values), _c_int(count), self._stream())

    def sample_rows(self, logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                    out_tokens: torch.Tensor) -> None:
        rows, vocab = logits.shape
        _need(logits, torch.float32, "sample_rows logits", 2)
        _need(temperature, torch.float32, "sample_rows temperature")
        _need(uniform, torch.float64, "sample_rows uniform")
        _need(out_tokens, torch.int32, "sample_rows out")
        self._call("bw_sample_rows", _p(logits), _c_int(rows), _c_int(vocab), _p(temperature), _p(uniform),
                   _p(out_tokens), self._stream())

    def fingerprint_rows(self, logits: torch.Tensor, slot: torch.Tensor, state: torch.Tensor) -> None:
        """state[slot[r]] = chained hash of logits row r's raw bits (one row per slot per call)."""
        rows, vocab = logits.shape
        _need(logits, torch.float32, "fingerprint_rows logits", 2)
        _need(slot, torch.int32, "fingerprint_rows slot")
        _need(state, torch.int64, "fingerprint_rows state")
        self._call("bw_fingerprint_rows", _p(logits), _c_int(rows), _c_int(vocab), _p(slot), _p(state),
                   self._stream())

    # -- per-precision kernels ---------------------------------------------------------
    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x and weight float32, out act_dtype."""
        n, width = out.shape
        _need(x, torch.float32, "rmsnorm x", 2)
        _need(weight, torch.float32, "rmsnorm weight", 1)
        _need(out, self.act_dtype, "rmsnorm out", 2)
        if x.shape[1] != width or weight.shape[0] != width:
            raise KernelError("rmsnorm: widths differ")
        if rows is not None:
            _need(rows, torch.int32, "rmsnorm rows")
        self._call(f"bw_{self.kind}_rmsnorm", _p(x), _p(weight), _p(out), _p(rows), _c_int(n), _c_int(width),
                   _c_float(eps), self._stream())

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
               residual: Optional[torch.Tensor] = None, legacy: bool = False) -> None:
        """out = x @ w.T (+ residual).  x [M,K] and w [N,K] in act_dtype; out act_dtype or
        float32; with a float32 residual the sum is formed in 32-bit (out float32, may alias)."""
        m, k = x.shape
        n = w.shape[0]
        _need(x, self.act_dtype, "linear x", 2)
        _need(w, self.act_dtype, "linear w", 2)
        if w.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if residual is not None:
            _need(residual, torch.float32, "linear residual", 2)
            _need(out, torch.float32, "linear out", 2)
            if tuple(residual.shape) != (m, n):
                raise KernelError("linear: residual shape differs from the output's")
        if self.kind == "f32":
            _need(out, torch.float32, "linear out", 2)
            self._call("bw_f32_linear", _p(x), _p(w), _p(out), _p(residual), _c_int(m), _c_int(n), _c_int(k),
                       self._stream())
        else:
            if out.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("linear: out must be float32 or bfloat16")
            _need(out, out.dtype, "linear out", 2)
            partials = counters = None
            if m <= self._split_rows:
                partials, counters = self._linear_scratch(x.device, n, k)
            self._call("bw_bf16_linear", _p(x), _p(w), _p(out), _c_int(int(out.dtype == torch.float32)),
                       _p(residual), _c_int(m), _c_int(n), _c_int(k), _p(partials), _p(counters),
                       _c_int(int(legacy)), self._stream(),
                       launches=1 if legacy else self._linear_kernels(m, n, k, False, partials is not None))

    def fuses_swiglu(self, width: int, intermediate: int) -> bool:
        """Whether ``linear_swiglu`` can take a feed-forward of these sizes (then its gate/up
        weights are to be interleaved with ``interleave_gate_up``)."""
        return self.kind == "bf16" and intermediate % 64 == 0 and width % 8 == 0

    @staticmethod
    def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """Rows in blocks of 64: gate rows 64 b .. 64 b + 63, then the up rows of the same
        indices, so that a 128-row tile of the product holds both halves of 64 outputs."""
        inter, k = gate.shape
        g = gate.reshape(inter // 64, 64, k)
        u = up.reshape(inter // 64, 64, k)
        return torch.stack([g, u], dim=1).reshape(2 * inter, k).contiguous()

    def linear_swiglu(self, x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor) -> None:
        """out[m][i] = silu(x @ gate_i) * (x @ up_i) for interleaved gate/up weights; gate and
        up are rounded to act_dtype before they are combined, as if they had been stored."""
        m, k = x.shape
        n = w_interleaved.shape[0]
        _need(x, self.act_dtype, "linear_swiglu x", 2)
        _need(w_interleaved, self.act_dtype, "linear_swiglu w", 2)
        _need(out, self.act_dtype, "linear_swiglu out", 2)
        if self.kind != "bf16" or n % 128 or k % 8 or tuple(out.shape) != (m, n // 2) or w_interleaved.shape[1] != k:
            raise KernelError("linear_swiglu: unsupported shapes or precision")
        partials = None
        if m <= self._split_rows:
            partials, _ = self._linear_scratch(x.device, n, k)
        self._call("bw_bf16_linear_tc_swiglu", _p(x), _p(w_interleaved), _p(out), _c_int(m), _c_int(n), _c_int(k),
                   _p(partials), self._stream(), launches=self._linear_kernels(m, n, k, True, partials is not None))

    def _linear_kernels(self, m: int, n: int, k: int, swiglu: bool, scratch: bool) -> int:
        """Kernels that a product of this shape launches (2 when it is split along k)."""
        key = (m, n, k, swiglu, scratch)
        c = self._kernel_counts.get(key)
        if c is None:
            c = int(self.lib.bw_bf16_linear_tc_kernels(_c_int(m), _c_int(n), _c_int(k), _c_int(int(swiglu)),
                                                       _c_int(int(scratch))))
            self._kernel_counts[key] = c
        return c

    def _linear_scratch(self, device, n: int, k: int):
        """Scratch of a product that is split along k: chunk sums for up to ``_split_rows``
        rows, and one counter per output tile (zero between launches).  It grows when a
        larger product appears and is otherwise reused by every product of the stream."""
        # sized for the largest batch that may be split, so that the address stays the same
        sizes = self._scratch_sizes.get((n, k))
        if sizes is None:
            sizes = (max(int(self.lib.bw_bf16_linear_scratch_floats(_c_int(r), _c_int(n), _c_int(k)))
                         for r in (64, self._split_rows)), int(self.lib.bw_bf16_linear_counters(_c_int(n))))
            self._scratch_sizes[(n, k)] = sizes
        floats, tiles = sizes
        if floats and (self._partials is None or self._partials.numel() < floats):
            self._retired.append(self._partials)  # a captured graph may still point at the old one
            self._partials = torch.empty(floats, dtype=torch.float32, device=device)
        if self._counters is None or self._counters.numel() < tiles:
            self._retired.append(self._counters)
            self._counters = torch.zeros(max(tiles, 1024), dtype=torch.int32, device=device)
        return self._partials, self._counters

    def force_linear_plan(self, width: int = 0, mode: int = 0) -> None:
        """Tests and measurements: force the tile width of small batches (16 .. 128 in steps of
        16, or 256; 0: chosen from the shape) and the mode (0 chosen, 1 one block walks k,
        2 split along k where possible).  Every combination gives the same bits."""
        if self.kind == "bf16":
            self._kernel_counts.clear()
            self.lib.bw_bf16_linear_tc_force(_c_int(width), _c_int(mode))

    def force_rows_plan(self, tile_cols: int = 0, stages: int = 0) -> None:
        """Tests and measurements of the 32-bit path: force the width of the streaming tile that
        products of up to 16 rows take (16, 32, 64 or 128 columns) and the stages of its ring
        (0: chosen from the shape).  Every combination gives the same bits."""
        if self.kind == "f32":
            self.lib.bw_f32_force_rows_plan(_c_int(tile_cols), _c_int(stages))

    def pair_tiles(self, on: bool) -> bool:
        """Large batches run two thread blocks per 256 x 256 tile of a product (the default) or
        one per 128 x 256 tile; same bits either way.  Returns the previous setting."""
        if self.kind != "bf16":
            return False
        return bool(self.lib.bw_bf16_linear_tc_pair_tiles(_c_int(int(on))))

    def rows_path(self, on: bool) -> bool:
        """Steps of up to 16 rows run their products on the streaming kernel (one kernel per
        product, chunk sums added inside it; the default) or on the tcgen05 kernel like larger
        steps; same bits either way.  Returns the previous setting."""
        if self.kind != "bf16":
            return False
        self._kernel_counts.clear()
        return bool(self.lib.bw_bf16_linear_rows_enable(_c_int(int(on))))

    def stream_attention(self, head_dim: int, mode: int) -> int:
        """How decode steps with head size 64 fetch the cache where TMA boxes fit (pages of 8 keys
        or more that divide 64): 0 never (a thread block per key tile that copies with cp.async),
        1 (the default) the streaming kernel (persistent blocks, TMA rings) for steps of 32 rows
        or more and a block per key tile fed by TMA boxes for fewer, 2 the streaming kernel
        whenever the shape allows.  Same bits every way.  Returns the previous setting."""
        if self.kind != "bf16":
            return 0
        return int(self._attention_lib(head_dim).bw_bf16_attention_stream_mode(_c_int(int(mode))))

    def _failure_words(self):
        if self._failure_word is None:
            dev = torch.device("cuda", self._device_index())
            self._failure_word = torch.zeros(1, dtype=torch.int32, device=dev)
            self._failure_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            for lib in [self.lib] + list(self._attn_libs.values()):
                lib.bw_set_failure_word(_p(self._failure_word))
        return self._failure_word, self._failure_host

    def failure_poll(self) -> None:
        """Enqueue a copy of the failure word to the host on the current stream (four bytes,
        asynchronous).  ``failure_seen`` reads the copy once the stream has been waited for:
        callers that wait for the device anyway (for a step's tokens) learn of a failure
        without a wait of their own."""
        word, host = self._failure_words()
        host.copy_(word, non_blocking=True)

    def failure_seen(self) -> bool:
        """True (once) when the last ``failure_poll`` whose copy has arrived saw the word raised."""
        if self._failure_host is None or int(self._failure_host[0]) == 0:
            return False
        self._failure_host[0] = 0
        self._failure_word.zero_()
        return True

    def device_failure(self) -> bool:
        """True (once) when a kernel gave up a bounded wait since the last call.  This waits
        for the device and reads a word from it; steps use failure_poll / failure_seen."""
        word, _ = self._failure_words()
        bad = bool(int(word.item()))
        if bad:
            word.zero_()
        return bad

    def selftest_bounded_wait(self, polls: int = 4096) -> int:
        """Launch the check kernel of the bounded waits: one warp waits with the kernels' own
        helper for a barrier on which nothing arrives, gives up after ``polls`` polls and
        raises the failure word.  Returns 2 when the wait gave up (as it must), 1 when it
        reported success."""
        self._failure_words()
        out = torch.zeros(1, dtype=torch.int32, device=self._failure_word.device)
        self._call("bw_selftest_bounded_wait", ctypes.c_uint(polls), _p(out), self._stream())
        return int(out.item())

    def attention_tile_rows(self, heads: int, kv_heads: int) -> int:
        """Query rows per attention tile: the bfloat16 kernel stacks the heads of a group
        with the rows, 64 stacked rows per thread block."""
        if self.kind == "f32":
            return 16
        return max(1, 64 // max(1, heads // kv_heads))

    def attention_tile_heights(self, heads: int, kv_heads: int, head_dim: int):
        """The heights of query tiles (rows of one sequence per thread block) that this
        precision's attention kernels want prepared for a step."""
        if self.kind == "f32":
            return [16]
        group = max(1, heads // kv_heads)
        rows = [max(1, 64 // group)]
        if 128 % group == 0:
            rows.append(128 // group)  # the tcgen05 prefill kernel stacks 128 rows per block
        return rows

    def _attention_scratch(self, lib, device, n: int, heads: int, max_keys: int) -> torch.Tensor:
        """Scratch of the split attention: one (output, maximum, sum) record per row, head and
        tile of 64 keys.  Sized for contexts rounded up to 2048 keys so that it seldom grows."""
        lib.bw_bf16_attention_scratch_floats.restype = ctypes.c_longlong
        keys = (max_keys + 2047) // 2048 * 2048
        floats = int(lib.bw_bf16_attention_scratch_floats(_c_int(n), _c_int(heads), _c_int(keys)))
        if self._attn_scratch is None or self._attn_scratch.numel() < floats:
            self._retired.append(self._attn_scratch)  # a captured graph may still point at the old one
            self._attn_scratch = torch.empty(floats, dtype=torch.float32, device=device)
        return self._attn_scratch

    def _attention_lib(self, head_dim: int):
        lib = self._attn_libs.get(head_dim)
        if lib is None:
            path = build.ensure_built("bf16_attn", (f"BW_HEAD_DIM={head_dim}",), self._verbose_build)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the attention library {path}: {e}") from None
            lib.bw_last_error.restype = ctypes.c_char_p
            if self._failure_word is not None:
                lib.bw_set_failure_word(_p(self._failure_word))
            self._attn_libs[head_dim] = lib
        return lib

    def rope_cache(self, qkv: torch.Tensor, pos: torch.Tensor, row_seq: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], block_table: torch.Tensor,
                   kcache: torch.Tensor, vcache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                   write_kv: bool = True) -> None:
        """Rotate q (in place) and k by the table rows of ``pos``; store k and v in the pages
        ``block_table[row_seq[r]][pos[r] // page]``.  kcache / vcache: [pages, kv_heads, page, hd]."""
        n = qkv.shape[0]
        _need(qkv, self.act_dtype, "rope_cache qkv", 2)
        _need(pos, torch.int32, "rope_cache pos")
        _need(row_seq, torch.int32, "rope_cache row_seq")
        _need(block_table, torch.int32, "rope_cache block_table", 2)
        _need(kcache, self.act_dtype, "rope_cache kcache", 4)
        _need(vcache, self.act_dtype, "rope_cache vcache", 4)
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("rope_cache: row width is not (heads + 2 kv_heads) * head_dim")
        if tuple(kcache.shape[1:]) != (kv_heads, kcache.shape[2], head_dim) or kcache.shape != vcache.shape:
            raise KernelError("rope_cache: cache shape is not [pages, kv_heads, page, head_dim]")
        if cos is not None:
            _need(cos, torch.float32, "rope_cache cos", 2)
            _need(sin, torch.float32, "rope_cache sin", 2)
            if cos.shape[1] != head_dim // 2 or cos.shape != sin.shape:
                raise KernelError("rope_cache: table width is not head_dim / 2")
        self._call(f"bw_{self.kind}_rope_cache", _p(qkv), _c_int(qkv.shape[1]), _p(pos), _p(row_seq), _p(cos),
                   _p(sin), _p(block_table), _c_int(block_table.shape[1]), _p(kcache), _p(vcache), _c_int(n),
                   _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(kcache.shape[2]),
                   _c_int(int(write_kv)), self._stream())

    def fuses_rope(self, m: int, width: int, heads: int, kv_heads: int, head_dim: int) -> bool:
        """Whether ``linear_rope_cache`` takes a step of m rows: then the fused q/k/v product
        rotates q and k and stores k and v in the cache itself (steps of up to 16 rows on the
        serving precision)."""
        if self.kind != "bf16":
            return False
        key = ("rope", m, width, heads, kv_heads, head_dim)
        c = self._kernel_counts.get(key)
        if c is None:
            c = int(self.lib.bw_bf16_linear_rows_rope_usable(None, None, _c_int(m), _c_int((heads + 2 * kv_heads) * head_dim),
                                                             _c_int(width), _c_int(heads), _c_int(kv_heads),
                                                             _c_int(head_dim)))
            self._kernel_counts[key] = c
        return bool(c)

    def linear_rope_cache(self, x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, pos: torch.Tensor,
                          row_seq: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                          block_table: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, heads: int,
                          kv_heads: int, head_dim: int, write_kv: bool = True) -> None:
        """``linear(x, w_qkv, qkv)`` followed by ``rope_cache(qkv, ...)`` in one kernel: the
        rotated q lands in qkv's first heads * head_dim columns, the rotated k and v in their
        pages; the k and v columns of qkv are NOT written.  Same bits as the two calls.  Only
        where ``fuses_rope`` says so."""
        m, k = x.shape
        n = w_qkv.shape[0]
        _need(x, self.act_dtype, "linear_rope_cache x", 2)
        _need(w_qkv, self.act_dtype, "linear_rope_cache w", 2)
        _need(qkv, self.act_dtype, "linear_rope_cache qkv", 2)
        _need(pos, torch.int32, "linear_rope_cache pos")
        _need(row_seq, torch.int32, "linear_rope_cache row_seq")
        _need(block_table, torch.int32, "linear_rope_cache block_table", 2)
        _need(kcache, self.act_dtype, "linear_rope_cache kcache", 4)
        _need(vcache, self.act_dtype, "linear_rope_cache vcache", 4)
        if self.kind != "bf16" or w_qkv.shape[1] != k or tuple(qkv.shape) != (m, n) or n != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("linear_rope_cache: shapes do not fit the fused q/k/v projection")
        if tuple(kcache.shape[1:]) != (kv_heads, kcache.shape[2], head_dim) or kcache.shape != vcache.shape:
            raise KernelError("linear_rope_cache: cache shape is not [pages, kv_heads, page, head_dim]")
        if cos is not None:
            _need(cos, torch.float32, "linear_rope_cache cos", 2)
            _need(sin, torch.float32, "linear_rope_cache sin", 2)
            if cos.shape[1] != head_dim // 2 or cos.shape != sin.shape:
                raise KernelError("linear_rope_cache: table width is not head_dim / 2")
        self._call("bw_bf16_linear_rows_rope", _p(x), _p(w_qkv), _p(qkv), _c_int(m), _c_int(n), _c_int(k), _p(pos),
                   _p(row_seq), _p(cos), _p(sin), _p(block_table), _c_int(block_table.shape[1]), _p(kcache), _p(vcache),
                   _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(kcache.shape[2]), _c_int(int(write_kv)),
                   self._stream())

    def attention(self, qkv: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                  block_table: torch.Tensor, row_seq: torch.Tensor, pos: torch.Tensor, out: torch.Tensor,
                  heads: int, kv_heads: int, head_dim: int, window: int, max_keys: int, scale: float,
                  batch=None) -> None:
        """out[r, h] = softmax(q k^T * scale) v over the cached keys lo..pos[r] of row r's
        sequence (lo = max(0, pos - window + 1) when window > 0).  q is read from the first
        heads*head_dim columns of qkv.  ``batch`` carries the step's per-sequence arrays for
        kernels that tile queries by sequence."""
        n = qkv.shape[0]
        _need(qkv, self.act_dtype, "attention qkv", 2)
        _need(out, self.act_dtype, "attention out", 2)
        _need(kcache, self.act_dtype, "attention kcache", 4)
        _need(vcache, self.act_dtype, "attention vcache", 4)
        _need(block_table, torch.int32, "attention block_table", 2)
        _need(row_seq, torch.int32, "attention row_seq")
        _need(pos, torch.int32, "attention pos")
        if out.shape[1] != heads * head_dim or out.shape[0] != n:
            raise KernelError("attention: output shape is not [rows, heads * head_dim]")
        page = kcache.shape[2]
        if self.kind == "f32":
            # prompt portions run as tiles of 16 query rows that share their keys; a step of single
            # rows (a decode step, or a call without the step's arrays) spreads a row's scores over
            # many blocks and needs scratch for them
            tiles = batch.query_tiles(16) if batch is not None and 16 in getattr(batch, "tile_sets", {}) else None
            scratch, floats, launches = None, 0, 1
            if tiles is None or tiles[3] >= n:
                tiles = None
                self.lib.bw_f32_attention_scratch_floats.restype = ctypes.c_longlong
                floats = int(self.lib.bw_f32_attention_scratch_floats(_c_int(n), _c_int(heads), _c_int(max_keys)))
                if self._attn_scratch is None or self._attn_scratch.numel() < floats:
                    self._attn_scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
                scratch, launches = self._attn_scratch, 2
            t_seq, t_row0, t_rows, t_count = tiles if tiles is not None else (None, None, None, 0)
            self._call("bw_f32_attention", _p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                       _c_int(block_table.shape[1]), _p(row_seq), _p(pos), _p(t_seq), _p(t_row0), _p(t_rows),
                       _c_int(t_count), _p(batch.seq_pos0) if tiles is not None else None,
                       _p(batch.seq_row0) if tiles is not None else None, _p(out), _c_int(out.shape[1]), _c_int(n),
                       _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window),
                       _c_int(max_keys), _c_float(scale), _p(scratch), ctypes.c_longlong(floats), self._stream(),
                       launches=launches)
        else:
            if batch is None:
                raise KernelError("attention (bfloat16): the step's sequence arrays are required")
            if head_dim % 16 or not (16 <= head_dim <= 256):
                raise KernelError(f"attention (bfloat16): head size {head_dim} is not a multiple of 16 up to 256")
            lib = self._attention_lib(head_dim)
            t_seq, t_row0, t_rows, t_count = batch.query_tiles(self.attention_tile_rows(heads, kv_heads))
            scratch = None
            split = t_count == n and max_keys > 128  # a decode step: one tile of keys per warp
            if not split and not self.legacy_attention:
                # prefill portions: the tcgen05 kernel, where it takes the shape (same bits)
                shape_key = (heads, kv_heads, head_dim, page, qkv.shape[1])
                rows_tc = self._tc_tile_rows.get(shape_key)
                if rows_tc is None:
                    rows_tc = int(lib.bw_bf16_attention_tc_tile_rows(_c_int(heads), _c_int(kv_heads),
                                                                     _c_int(head_dim), _c_int(page),
                                                                     _c_int(qkv.shape[1])))
                    self._tc_tile_rows[shape_key] = rows_tc
                sets = getattr(batch, "tile_sets", None)
                if rows_tc > 0 and (sets is None or rows_tc in sets) and n > t_count:
                    q_seq, q_row0, q_rows, q_count = batch.query_tiles(rows_tc)
                    fn = lib.bw_bf16_attention_tc
                    fn.restype = _c_int
                    rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _c_int(kcache.shape[0]),
                            _p(block_table), _c_int(block_table.shape[1]), _p(q_seq), _p(q_row0), _p(q_rows),
                            _c_int(q_count), _p(batch.seq_pos0), _p(batch.seq_row0), _p(out), _c_int(out.shape[1]),
                            _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window),
                            _c_float(scale), self._stream())
                    if rc != 0:
                        raise KernelError(f"bw_bf16_attention_tc failed ({rc}): "
                                          + lib.bw_last_error().decode("utf-8", "replace"))
                    self.launches += 1
                    return
            if split:
                scratch = self._attention_scratch(lib, qkv.device, n, heads, max_keys)
                # head size 64: the cache streams through TMA rings, one block per SM (same bits)
                if lib.bw_bf16_attention_stream_usable(_c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page),
                                                       _c_int(qkv.shape[1])):
                    fn = lib.bw_bf16_attention_stream
                    fn.restype = _c_int
                    rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _c_int(kcache.shape[0]),
                            _p(block_table), _c_int(block_table.shape[1]), _p(row_seq), _p(pos), _p(out),
                            _c_int(out.shape[1]), _c_int(n), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                            _c_int(page), _c_int(window), _c_float(scale), _c_int(max_keys), _p(scratch), self._stream())
                    if rc != 0:
                        raise KernelError(f"bw_bf16_attention_stream failed ({rc}): "
                                          + lib.bw_last_error().decode("utf-8", "replace"))
                    self.launches += 2
                    return
            fn = lib.bw_bf16_attention
            fn.restype = _c_int
            rc = fn(_p(qkv), _c_int(qkv.shape[1]), _p(kcache), _p(vcache), _p(block_table),
                    _c_int(block_table.shape[1]), _p(t_seq), _p(t_row0), _p(t_rows), _c_int(t_count),
                    _p(batch.seq_pos0), _p(batch.seq_row0), _p(row_seq), _p(pos), _p(out), _c_int(out.shape[1]), _c_int(n),
                    _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page), _c_int(window), _c_float(scale),
                    _c_int(max_keys), _p(scratch), self._stream())
            if rc != 0:
                raise KernelError(f"bw_bf16_attention failed ({rc}): "
                                  + lib.bw_last_error().decode("utf-8", "replace"))
            self.launches += 2 if split else 1

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        """out = silu(gate) * up for rows laid out [gate | up]."""
        n, inter = out.shape
        _need(gate_up, self.act_dtype, "swiglu gate_up", 2)
        _need(out, self.act_dtype, "swiglu out", 2)
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != n:
            raise KernelError("swiglu: input is not [rows, 2 * intermediate]")
        self._call(f"bw_{self.kind}_swiglu", _p(gate_up), _p(out), _c_int(n), _c_int(inter), self._stream())


_OPS = {}


def get_ops(dtype: str) -> KernelOps:
    """The shared KernelOps of a precision (libraries are loaded once per process)."""
    if dtype not in _OPS:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        _OPS[dtype] = KernelOps(dtype)
    return _OPS[dtype]
