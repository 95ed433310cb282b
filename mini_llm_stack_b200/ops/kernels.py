"""Python faces of the CUDA kernels, and the runtime the parts run on.

Each method checks shapes and types on the host, then calls one exported C
launcher with raw device pointers on torch's current stream.  Nothing here
computes on the CPU and nothing falls back to a library implementation of a
part of the model; the only library call is the plain bfloat16 matrix product
where the own kernel does not apply (the reference multiplies with
``nn.Linear``, i.e. a library GEMM: train/model.py:79-82,130-132,227).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import library

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_LL = ctypes.c_longlong

_ERRORS = {100001: "a size this kernel does not support",
           100002: "the driver refused to encode a tensor map"}


# torch's own fast path to the current stream's handle (a C call without the argument
# handling of torch.cuda.current_stream, which costs several microseconds a launch)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        why = _ERRORS.get(rc)
        if why is None:
            why = f"CUDA error {rc}"
        raise KernelError(f"{what}: {why}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _decl(lib, name, argtypes, restype=ctypes.c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


class SplitParts:
    """A matrix product left as the parts of a cut along K: float32 [parts, M, N].

    Their sum, taken in the order of the slices, is the product.  ``add_rmsnorm``
    adds them up while it reads the residual row anyway, which saves the kernel
    that would do nothing else.  The parts live in one scratch buffer of the
    kernels' owner: they are read (or given up) before the next product that
    wants the buffer, which otherwise takes the ordinary way.
    """

    __slots__ = ("parts", "_ops")

    def __init__(self, parts, ops):
        self.parts = parts
        self._ops = ops

    @property
    def shape(self):
        return self.parts.shape[1:]

    def release(self) -> None:
        if self._ops is not None:
            self._ops._parts_busy = False
            self._ops = None

    def float(self):
        """The product as a float32 tensor of its own."""
        out = self.parts[0].clone()
        for k in range(1, self.parts.shape[0]):
            out += self.parts[k]
        self.release()
        return out

    def clone(self):
        return self.float()

    def to(self, dtype):
        return self.float().to(dtype)


class Ops:
    """The kernels, bound to one device.  Fails at construction without a GPU."""

    def __init__(self, device, act_dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError(
                "this engine runs on a CUDA device only (sm_100a kernels); "
                f"device {device!r} is not one and there is no CPU path")
        self.act_dtype = act_dtype
        self._device_index = (self.device.index if self.device.index is not None
                              else torch.cuda.current_device())
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._libs: list = []                    # every kernel library in use
        self._chained = True                     # what the libraries were last told
        core = self._load("core")
        self._embed = _decl(core, "mls_embed", [_P, _P, _I, _P, _I, _I, _I, _P, _P])
        self._add_rmsnorm = _decl(core, "mls_add_rmsnorm",
                                  [_P, _P, _I, _P, _I, _F, _P, _I, _I, _I, _P, _I, _LL, _P, _P])
        self._gemm_f32 = _decl(core, "mls_gemm_f32", [_P, _P, _P, _I, _I, _I, _P])
        self._rope_store = _decl(core, "mls_rope_store",
                                 [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                                  _LL, _I, _P, _I, _LL, _P, _P])
        self._attention_simt = _decl(core, "mls_attention_simt",
                                     [_P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _I, _LL, _P])
        self._swiglu = _decl(core, "mls_swiglu", [_P, _P, _I, _I, _I, _P])
        self._sample = _decl(core, "mls_sample", [_P, _P, _P, _P, _I, _I, _P, _P])
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._attention_libs: dict = {}
        self._attention_lib_handles: dict = {}
        self._split_ctas_per_sm: dict = {}       # head size -> CTAs of the split kernel an SM holds
        self._attention_fused: dict = {}         # head size -> decode attention that also rotates
        self._tc_rows: dict = {}                 # head size -> rows of a tile of the tcgen05 kernel
        self._scratch: dict = {}
        self._transposed: dict = {}              # id(weight) -> (weight, its transposed view)
        self._gemm = None
        self._tiles_set = False
        self._parts_busy = False
        self.attention_impl = os.environ.get("MLS_B200_ATTENTION", "auto")
        self.gemm_impl = os.environ.get("MLS_B200_GEMM", "auto")
        self.generation = 0          # grows whenever a buffer kernels were given moves
        self.launches = 0            # launches of this package's own kernels
        self.library_launches = 0    # plain matrix products handed to the library

    # ------------------------------------------------------------------ helpers
    def _load(self, name: str, defines: dict | None = None):
        lib = library.load(name, defines)
        lib.mls_set_chained.argtypes = [_I]
        lib.mls_set_chained.restype = None
        lib.mls_set_chained(1 if self._chained else 0)
        self._libs.append(lib)
        return lib

    CHAINED_UP_TO = 256      # tokens of a step whose kernels start under their predecessors

    def begin_step(self, n_tokens: int) -> None:
        """Tell the kernel libraries how to launch this step's kernels: chained
        (each may start, and fetch what no kernel writes, while the one before it
        still runs) pays when kernels are short, plain when they are long."""
        on = n_tokens <= self.CHAINED_UP_TO
        if on != self._chained:
            self._chained = on
            for lib in self._libs:
                lib.mls_set_chained(1 if on else 0)

    def scratch(self, tag: str, n_floats: int):
        """Float32 scratch memory that lives as long as the kernels' owner."""
        buf = self._scratch.get(tag)
        if buf is None or buf.numel() < n_floats:
            buf = torch.empty(max(n_floats, 1 << 16), dtype=torch.float32, device=self.device)
            self._scratch[tag] = buf
            self.generation += 1
        return buf

    def _stream(self):
        """The raw handle of torch's current stream on this device (asked for at every
        launch: a captured step runs on the capture's stream)."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def check_status(self) -> None:
        """Raise if a kernel met a token, position or slot outside its table (waits
        for the device)."""
        self.raise_for_status(int(self.status.item()))

    def raise_for_status(self, code: int) -> None:
        """Raise for a status word already read (``code`` != 0), and clear it on the
        device so that the next step starts clean."""
        if code:
            self.status.zero_()
            what = [n for b, n in ((1, "a token id outside the vocabulary"),
                                   (2, "a position outside the rotary table"),
                                   (4, "a cache slot outside the pool"),
                                   (8, "a bounded wait inside a kernel ran out"),
                                   (16, "shared memory of a kernel was not aligned"))
                    if code & b]
            raise KernelError("a kernel refused its input: " + ("; ".join(what) or
                                                                f"status {code}"))

    # ------------------------------------------------------------------ kernels
    def embed(self, token_ids, table, x, vocab: int) -> None:
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "embed: x must be float32")
        _need(table.shape == (vocab, d) and table.is_contiguous(), "embed: bad table")
        _need(token_ids.dtype == torch.int32 and token_ids.numel() >= t, "embed: bad ids")
        self.launches += 1
        _check(self._embed(_ptr(token_ids), _ptr(table), _code(table.dtype), _ptr(x), t, d,
                           vocab, _ptr(self.status), self._stream()), "embed")

    def _delta_args(self, delta, t: int, d: int, what: str):
        """(pointer, type code, parts, part stride) of a pending residual delta."""
        if delta is None:
            return None, 0, 1, 0
        if isinstance(delta, SplitParts):
            parts = delta.parts
            _need(parts.shape[1:] == (t, d) and parts.is_contiguous()
                  and parts.dtype == torch.float32, f"{what}: bad delta parts")
            return parts.data_ptr(), 0, parts.shape[0], t * d
        _need(delta.shape == (t, d) and delta.is_contiguous(), f"{what}: bad delta")
        return delta.data_ptr(), _code(delta.dtype), 1, 0

    def add_rmsnorm(self, x, delta, weight, eps: float, h) -> None:
        """``x += delta`` (a tensor, ``SplitParts`` or None), ``h = rmsnorm(x) * weight``."""
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be float32")
        _need(h.shape == (t, d) and h.is_contiguous(), "add_rmsnorm: bad output")
        _need(weight.shape == (d,), "add_rmsnorm: bad weight")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "add_rmsnorm")
        self.launches += 1
        _check(self._add_rmsnorm(_ptr(x), dp, dcode, _ptr(weight), _code(weight.dtype),
                                 float(eps), _ptr(h), _code(h.dtype), t, d, None, parts, stride,
                                 _ptr(self.status), self._stream()), "add_rmsnorm")
        if isinstance(delta, SplitParts):
            delta.release()

    def gather_add_rmsnorm(self, x, delta, rows, n_rows: int, weight, eps: float, h) -> None:
        t, d = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "gather_add_rmsnorm: bad x")
        _need(h.shape == (n_rows, d) and h.is_contiguous(), "gather_add_rmsnorm: bad output")
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "gather_add_rmsnorm: rows")
        dp, dcode, parts, stride = self._delta_args(delta, t, d, "gather_add_rmsnorm")
        self.launches += 1
        _check(self._add_rmsnorm(_ptr(x), dp, dcode, _ptr(weight), _code(weight.dtype),
                                 float(eps), _ptr(h), _code(h.dtype), n_rows, d, _ptr(rows),
                                 parts, stride, _ptr(self.status), self._stream()),
               "gather_add_rmsnorm")
        if isinstance(delta, SplitParts):
            delta.release()

    def prepare_weight(self, w):
        """A matrix [out, in] made ready for ``linear`` (contiguous, on device)."""
        return w.contiguous()

    def linear(self, a, w, out) -> None:
        """``out[M, N] = a[M, K] @ w[N, K]^T`` with float32 accumulation."""
        m, k = a.shape
        n = w.shape[0]
        _need(w.shape == (n, k) and out.shape == (m, n), "linear: shapes do not fit")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(),
              "linear: operands must be contiguous")
        if m == 0:
            return
        if w.dtype == torch.float32:
            # a matrix held in 32 bits is multiplied in true 32-bit arithmetic
            a32 = a if a.dtype == torch.float32 else a.float()
            o32 = out if out.dtype == torch.float32 else torch.empty(
                (m, n), dtype=torch.float32, device=out.device)
            self.launches += 1
            _check(self._gemm_f32(_ptr(a32), _ptr(w), _ptr(o32), m, n, k, self._stream()),
                   "gemm_f32")
            if o32 is not out:
                out.copy_(o32)
            return
        _need(w.dtype == torch.bfloat16, f"linear: weight dtype {w.dtype}")
        a16 = a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)
        if self._use_own_gemm(m, n, k):
            self._gemm_bf16(a16, w, out, m, n, k)
            return
        self.library_launches += 1
        held = self._transposed.get(id(w))           # the view costs a microsecond a call
        if held is None or held[0] is not w:
            held = self._transposed[id(w)] = (w, w.t())
        if out.dtype == torch.float32:
            torch.mm(a16, held[1], out_dtype=torch.float32, out=out)
        else:
            torch.mm(a16, held[1], out=out)

    def _use_own_gemm(self, m: int, n: int, k: int) -> bool:
        """The tcgen05 kernel takes rows that are whole 16-byte chunks; the choice
        between it and the library is ``MLS_B200_GEMM`` (tcgen05 | tcgen05-tiles | cublas |
        auto; prompts of more than 128 rows run on pairs of CTAs, with ``tcgen05-tiles``
        on one CTA a tile)."""
        if self.gemm_impl == "cublas" or k % 8 != 0:
            return False
        if self.gemm_impl in ("tcgen05", "tcgen05-tiles"):
            return True
        # auto: a few rows (decoding) go to the tcgen05 kernel, which asks for its
        # first weights while the kernel before it still runs; more rows go to the
        # library (as the reference's nn.Linear does) unless the kernel fuses work
        # (``linear_swiglu``)
        return m <= 64

    def _gemm_splits(self, m: int, n: int, k: int) -> int:
        """Parts along K for the weight-major orientation (M <= 64): the weights are
        read once; every tile x part is a CTA, and two CTAs fit an SM: as many CTAs
        as fit at the same time, at least 256 of K each."""
        tiles = (n + 127) // 128
        kblocks = (k + 63) // 64
        splits = max(1, min(kblocks // 4, (2 * self.sm_count) // tiles))
        per = -(-kblocks // splits)
        return -(-kblocks // per)

    def _gemm_library(self):
        if self._gemm is None:
            lib = self._load("gemm")
            self._gemm = _decl(lib, "mls_gemm_bf16",
                               [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P])
            self._gemm_prompt_scratch = _decl(lib, "mls_gemm_prompt_scratch_floats", [_I, _I, _I],
                                              restype=ctypes.c_longlong)
            self._gemm_lib = lib
        return self._gemm_lib

    def set_gemm_tail_cut(self, mode: str) -> None:
        """Whether a prompt's product cuts the tiles of its last round along K: "never",
        "auto" (where it measured faster; the default) or "always" (wherever every piece
        gets four k-blocks)."""
        _need(mode in ("never", "auto", "always"), f"set_gemm_tail_cut: unknown mode {mode!r}")
        fn = _decl(self._gemm_library(), "mls_gemm_set_tail_cut", [_I], restype=None)
        fn(("never", "auto", "always").index(mode))

    def _gemm_bf16(self, a, w, out, m: int, n: int, k: int, epilogue: int = 0,
                   leave_parts: bool = False):
        """The tcgen05 product.  ``leave_parts``: the K-parts are not added up but
        returned as ``SplitParts`` (the caller has checked that there are several)."""
        self._gemm_library()
        if self.gemm_impl == "tcgen05-tiles" or self._tiles_set:
            # prompts of more than 128 rows on one CTA a tile instead of pairs of CTAs
            self._gemm_lib.mls_gemm_set_prompt_kernel.argtypes = [_I]
            self._gemm_lib.mls_gemm_set_prompt_kernel.restype = None
            self._tiles_set = self.gemm_impl == "tcgen05-tiles"
            self._gemm_lib.mls_gemm_set_prompt_kernel(0 if self._tiles_set else 1)
        swap = 1 if m <= 64 else 0
        splits, partial, sums = 1, None, 0
        if swap:
            splits = self._gemm_splits(m, n, k)
            if splits > 1:
                tag = "gemm_kept_parts" if leave_parts else "gemm_partials"
                partial = self.scratch(tag, splits * m * n)
                sums = 0 if leave_parts else 1
        else:
            # a prompt's product cuts the tiles of its last round along K when that gives
            # every pair of SMs a piece; a second kernel adds the pieces up
            floats = self._gemm_prompt_scratch(m, n, k)
            if floats:
                partial = self.scratch("gemm_tail_parts", floats)
                sums = 1
        _need(not leave_parts or splits > 1, "gemm_bf16: no parts to leave")
        self.launches += 1 + sums
        out_f32 = 1 if (out is not None and out.dtype == torch.float32) else 0
        _check(self._gemm(_ptr(a), _ptr(w), None if leave_parts else _ptr(out), out_f32,
                          m, n, k, swap, splits, epilogue, _ptr(partial), _ptr(self.status),
                          self._stream()), "gemm_bf16")
        if leave_parts:
            self._parts_busy = True
            return SplitParts(partial[:splits * m * n].view(splits, m, n), self)
        return None

    def linear_parts(self, a, w, out):
        """A product for a consumer that can add up K-parts while it reads its input
        anyway (``add_rmsnorm`` for what goes to the residual stream, ``rope_store``
        for q, k and v): returns ``out``, filled, or the product's parts
        (``SplitParts``) with ``out`` untouched."""
        m, k = a.shape
        n = w.shape[0]
        if (0 < m <= 64 and n % 4 == 0 and w.dtype == torch.bfloat16
                and not self._parts_busy
                and w.shape == (n, k) and a.is_contiguous() and w.is_contiguous()
                and self._use_own_gemm(m, n, k) and self._gemm_splits(m, n, k) > 1):
            a16 = a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)
            return self._gemm_bf16(a16, w, None, m, n, k, leave_parts=True)
        self.linear(a, w, out)
        return out

    def can_fuse_swiglu(self, d_model: int, inter: int) -> bool:
        """Whether gate-up projection and SwiGLU can run as one kernel."""
        return (self.act_dtype == torch.bfloat16 and self.gemm_impl != "cublas"
                and inter % 16 == 0 and d_model % 8 == 0)

    @staticmethod
    def interleave_gate_up(w_gate, w_up):
        """Rows [16 gate | 16 up | 16 gate | ...]: the layout ``linear_swiglu`` reads."""
        i, d = w_gate.shape
        both = torch.stack([w_gate.view(i // 16, 16, d), w_up.view(i // 16, 16, d)], dim=1)
        return both.reshape(2 * i, d).contiguous()

    def linear_swiglu(self, a, w_interleaved, out) -> None:
        """``out[M, I] = silu(a @ Wg^T) * (a @ Wu^T)`` in one kernel; the weight holds
        gate and up rows interleaved in blocks of 16 (``interleave_gate_up``)."""
        m, k = a.shape
        n = w_interleaved.shape[0]
        _need(out.shape == (m, n // 2) and a.dtype == torch.bfloat16 and
              w_interleaved.dtype == torch.bfloat16, "linear_swiglu: shapes or types do not fit")
        _need(a.is_contiguous() and w_interleaved.is_contiguous() and out.is_contiguous(),
              "linear_swiglu: operands must be contiguous")
        if m == 0:
            return
        self._gemm_bf16(a, w_interleaved, out, m, n, k, epilogue=1)

    def rope_takes_parts(self, hd: int) -> bool:
        """Whether ``rope_store`` can read its rows from a product's K-parts."""
        return self.act_dtype == torch.bfloat16 and (hd // 2) % 8 == 0

    def rope_store(self, qkv, positions, cos, sin, slot_map, k_pool, v_pool, n_tokens: int,
                   n_heads: int, n_kv: int, hd: int, max_pos: int, writes: bool,
                   parts=None) -> None:
        """Rotate q and k, store rotated k and raw v in the pages, leave rotated q in
        ``qkv``.  With ``parts`` (``SplitParts`` of the projection) the rows are
        read from there instead of from ``qkv``."""
        _need(qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv) * hd,
              "rope_store: bad qkv")
        _need(k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype,
              "rope_store: cache and activations differ in type")
        _need(k_pool.is_contiguous() and v_pool.is_contiguous(), "rope_store: pool layout")
        kvh, pages, block, hd2 = k_pool.shape
        _need(kvh == n_kv and hd2 == hd, "rope_store: pool shape does not fit the heads")
        _need(cos.shape == (max_pos, hd // 2) and cos.dtype == torch.float32,
              "rope_store: bad tables")
        pp, n_parts, stride = None, 0, 0
        if parts is not None:
            _need(self.rope_takes_parts(hd) and qkv.dtype == torch.bfloat16
                  and tuple(parts.shape) == tuple(qkv.shape) and parts.parts.is_contiguous(),
                  "rope_store: these parts cannot be read")
            pp, n_parts = parts.parts.data_ptr(), parts.parts.shape[0]
            stride = qkv.shape[0] * qkv.shape[1]
        self.launches += 1
        _check(self._rope_store(_ptr(qkv), _code(qkv.dtype), _ptr(positions), _ptr(cos),
                                _ptr(sin), _ptr(slot_map), _ptr(k_pool), _ptr(v_pool),
                                n_tokens, n_heads, n_kv, hd, block, max_pos,
                                pages * block, 1 if writes else 0, pp, n_parts, stride,
                                _ptr(self.status), self._stream()), "rope_store")
        if parts is not None:
            parts.release()

    def require_attention(self, hd: int, n_heads: int = 0, n_kv: int = 0) -> None:
        """Make sure attention kernels for this head size exist, or say why not."""
        _need(hd % 16 == 0 and 16 <= hd <= 256,
              f"attention kernels take head sizes 16..256 in steps of 16, not {hd}")
        if self.act_dtype == torch.bfloat16 and hd not in self._attention_libs:
            lib = self._load("attention", {"MLS_HEAD_DIM": int(hd)})
            fn = _decl(lib, "mls_attention_mma",
                       [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I,
                        _P, _P, _LL, _P, _I, _P])
            tc = _decl(lib, "mls_attention_tc",
                       [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _I, _LL, _P, _P])
            fused = _decl(lib, "mls_attention_decode_fused",
                          [_P, _I, _LL, _P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I,
                           _I, _I, _F, _I, _I, _P, _P, _LL, _P, _P])
            self._attention_fused[hd] = fused
            rows_fn = lib.mls_attention_tc_rows
            rows_fn.restype = ctypes.c_int
            self._tc_rows[hd] = int(rows_fn()) or 128
            self._attention_libs[hd] = (fn, tc)
            self._attention_lib_handles[hd] = lib
            per_sm = _decl(lib, "mls_attention_split_ctas_per_sm", [_I])
            tma = self.attention_impl in ("auto", "mma") and hd % 64 == 0
            self._split_ctas_per_sm[hd] = int(per_sm(1 if tma else 0)) or 2

    def set_attention_rows(self, hd: int, rows: int) -> None:
        """Fix the rows a CTA of the tcgen05 attention kernel owns: 256 (two row tiles),
        128 (one, its keys in halves) or 0 (chosen by the step's size; the default)."""
        _need(rows in (0, 128, 256), "set_attention_rows: 0, 128 or 256")
        self.require_attention(hd)
        lib = self._attention_lib_handles[hd]
        fn = _decl(lib, "mls_attention_tc_set_rows", [_I], restype=None)
        fn(rows)

    def attention_facts(self, hd: int) -> dict:
        """What a mixer needs to know of the attention kernels to plan a step's
        launches: ``small_rows`` (requests whose (token, head) rows of one kv head are
        at most this many go to the context-split kernel), ``tile_rows`` and
        ``tc_rows`` (rows of a tile of the mma.sync and of the tcgen05 tile kernel),
        ``split_keys`` (keys of a tile of the split kernel), ``split_slots`` (CTAs of the
        split kernel the GPU runs at a time: as many an SM as the kernel's registers and
        shared memory allow),
        ``cluster_splits`` (up to so many context splits are merged inside the kernel),
        ``tensor_cores`` (False: the one-warp-per-row kernel runs, which needs no plan)."""
        tma = self.attention_impl in ("auto", "mma") and hd % 64 == 0
        return {"small_rows": 16, "tile_rows": 64, "tc_rows": self._tc_rows.get(hd, 128),
                "split_keys": 64,
                "split_slots": self._split_ctas_per_sm.get(hd, 2) * self.sm_count,
                "cluster_slots": 2 * self.sm_count,   # CTAs up to which the splits merge in clusters
                # most context splits that merge inside the split kernel (a merge kernel
                # takes over beyond that)
                "cluster_splits": 8 if tma and os.environ.get(
                    "MLS_B200_CLUSTER_MERGE", "1") != "0" else 0,
                "tensor_cores": self.act_dtype == torch.bfloat16 and self.attention_impl != "simt"}

    def paged_attention(self, qkv, out, cache, step, n_heads: int, n_kv: int, hd: int,
                        scale: float, window: int, plan=None) -> None:
        """Attention of the step's tokens over the pages.  ``plan`` (the mixer's, from
        ``attention_facts``): ``n_tiles`` / ``n_tiles_tc`` / ``n_tiles_tc_wide`` tiles of the
        requests that are not small, ``any_small``, ``n_split`` context splits for the small ones."""
        g = step.groups[cache.group]
        t = step.n_tokens
        _need(out.shape == (t, n_heads * hd) and out.is_contiguous(), "attention: bad out")
        _need(cache.k_pool.dtype == qkv.dtype, "attention: cache and activations differ")
        if qkv.dtype == torch.bfloat16 and self.attention_impl != "simt":
            fns = self._attention_libs.get(hd)
            _need(fns is not None, f"attention kernels for head size {hd} were not required")
            fn, tc = fns
            _need(plan is not None, "attention: the tensor-core kernels need the mixer's plan")
            n_tiles, n_small, n_split, n_tiles_tc = (plan.n_tiles, 1 if plan.any_small else 0,
                                                     plan.n_split, plan.n_tiles_tc)
            if (n_tiles and hd in (64, 128) and g.block_size in (8, 16, 32, 64)
                    and self.attention_impl == "auto"):
                # prompts and portions: the tcgen05 kernel; what is left for the call
                # below are the requests of a few rows
                self.launches += 1
                _check(tc(_ptr(qkv), _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool),
                          _ptr(g.block_table), g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len),
                          step.n_requests, n_heads, n_kv, g.block_size, float(scale), int(window),
                          n_tiles_tc, plan.n_tiles_tc_wide, n_small, cache.k_pool.shape[1],
                          _ptr(self.status), self._stream()), "attention_tc")
                n_tiles = 0
                if not n_small:
                    return
            part_o = part_lse = None
            if n_split > 1:
                units = t * n_heads
                scratch = self.scratch("attention_partials", n_split * units * (hd + 1))
                part_o = scratch[:n_split * units * hd]
                part_lse = scratch[n_split * units * hd:]
            tma = (self.attention_impl != "no_tma" and hd % 64 == 0
                   and g.block_size in (8, 16, 32, 64))
            self.launches += (1 if n_tiles else 0) + (n_small and self._split_launches(
                n_split, tma, step.n_requests * n_kv * n_split))
            _check(fn(_ptr(qkv), _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool),
                      _ptr(g.block_table), g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len),
                      step.n_requests, t, n_heads, n_kv, g.block_size, float(scale), int(window),
                      n_tiles, n_small, n_split, _ptr(part_o), _ptr(part_lse),
                      cache.k_pool.shape[1], _ptr(self.status),
                      0 if self.attention_impl == "no_tma" else 1, self._stream()),
                   "attention_mma")
            return
        self.launches += 1
        _check(self._attention_simt(
            _ptr(qkv), _ptr(out), _code(qkv.dtype), _ptr(cache.k_pool), _ptr(cache.v_pool),
            _ptr(g.block_table), g.max_blocks, _ptr(step.positions), _ptr(step.req_of_token),
            t, n_heads, n_kv, hd, g.block_size, float(scale), int(window),
            cache.k_pool.shape[1], self._stream()), "attention_simt")

    def _split_launches(self, n_split: int, tma: bool, n_ctas: int) -> int:
        """Kernels the context-split attention launches: two to eight splits merge inside
        clusters of the one kernel if all its CTAs are resident at once, else through a
        merge kernel."""
        if n_split == 1:
            return 1
        in_clusters = (tma and n_split <= 8 and n_ctas <= 2 * self.sm_count
                       and os.environ.get("MLS_B200_CLUSTER_MERGE", "1") != "0")
        return 1 if in_clusters else 2

    def can_fuse_rope_attention(self, hd: int, block_size: int) -> bool:
        """Whether a step of single decoded tokens can leave the rotation and the cache
        write to the attention kernel (``attention_decode_fused``)."""
        return (self.act_dtype == torch.bfloat16 and self.attention_impl == "auto"
                and hd % 64 == 0 and block_size in (8, 16, 32, 64)
                and os.environ.get("MLS_B200_FUSED_ROPE", "1") != "0")

    def attention_decode_fused(self, parts, out, cache, step, cos, sin, max_pos: int,
                               n_heads: int, n_kv: int, hd: int, scale: float, window: int,
                               plan) -> None:
        """A step of one token a request: rotate q and k (read as the K-parts of their
        projection), store k and v, attend.  One kernel (and the merge of the context
        splits) instead of ``rope_store`` + ``paged_attention``; the bits are the same."""
        g = step.groups[cache.group]
        t = step.n_tokens
        width = (n_heads + 2 * n_kv) * hd
        _need(step.max_q_len == 1 and t == step.n_requests, "fused attention: single tokens only")
        _need(isinstance(parts, SplitParts) and tuple(parts.shape) == (t, width)
              and parts.parts.is_contiguous(), "fused attention: bad parts")
        _need(out.shape == (t, n_heads * hd) and out.is_contiguous()
              and out.dtype == torch.bfloat16, "fused attention: bad out")
        _need(cache.k_pool.dtype == torch.bfloat16 and cache.k_pool.is_contiguous()
              and cache.v_pool.is_contiguous(), "fused attention: pool layout")
        _need(cos.shape == (max_pos, hd // 2) and cos.dtype == torch.float32, "fused attention: tables")
        fn = self._attention_fused.get(hd)
        _need(fn is not None and plan is not None, "fused attention: kernels were not required")
        n_split = plan.n_split
        part_o = part_lse = None
        if n_split > 1:
            units = t * n_heads
            scratch = self.scratch("attention_partials", n_split * units * (hd + 1))
            part_o = scratch[:n_split * units * hd]
            part_lse = scratch[n_split * units * hd:]
        self.launches += self._split_launches(n_split, True, step.n_requests * n_kv * n_split)
        _check(fn(parts.parts.data_ptr(), parts.parts.shape[0], t * width, _ptr(step.positions),
                  _ptr(cos), _ptr(sin), max_pos, _ptr(g.slot_map), 1 if cache.writes else 0,
                  _ptr(out), _ptr(cache.k_pool), _ptr(cache.v_pool), _ptr(g.block_table),
                  g.max_blocks, _ptr(step.cu_q), _ptr(step.ctx_len), step.n_requests, n_heads,
                  n_kv, g.block_size, float(scale), int(window), n_split, _ptr(part_o),
                  _ptr(part_lse), cache.k_pool.shape[1], _ptr(self.status), self._stream()),
               "attention_decode_fused")
        parts.release()

    def swiglu(self, gu, out) -> None:
        t, inter = out.shape
        _need(gu.shape == (t, 2 * inter) and gu.dtype == out.dtype, "swiglu: shapes")
        _need(gu.is_contiguous() and out.is_contiguous(), "swiglu: layout")
        self.launches += 1
        _check(self._swiglu(_ptr(gu), _ptr(out), _code(out.dtype), t, inter, self._stream()),
               "swiglu")

    def sample(self, logits, temperature, uniform, out) -> None:
        """Tokens for float32 ``logits [n, V]``; rows with temperature <= 0 (or
        ``temperature`` None) take the arg max, lowest index on ties."""
        n, v = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits")
        _need(out.dtype == torch.int32 and out.numel() >= n, "sample: out")
        if temperature is not None:
            _need(temperature.dtype == torch.float32 and uniform.dtype == torch.float32,
                  "sample: temperature and uniform must be float32")
        scratch = None
        if v > 4096:             # chunks of the vocabulary on many SMs, then a pick a row
            scratch = self.scratch("argmax_chunks", 3 * n * ((v + 4095) // 4096))
        self.launches += 2 if scratch is not None else 1
        _check(self._sample(_ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out), n, v,
                            _ptr(scratch), self._stream()), "sample")


class Runtime:
    """Device, element types, kernels and step buffers shared by a model's parts."""

    residual_dtype = torch.float32
    logits_dtype = torch.float32

    def __init__(self, device="cuda:0", dtype: torch.dtype = torch.bfloat16):
        self.device = torch.device(device)
        self.act_dtype = dtype
        self.ops = Ops(self.device, dtype)
        self._buffers: dict = {}
        self._views: dict = {}               # (tag, dtype, shape) -> the view handed out last time

    def buffer(self, tag: str, shape: tuple, dtype: torch.dtype):
        """A step buffer: the same memory for the same tag, grown when needed."""
        shape = tuple(shape)
        view = self._views.get((tag, dtype, shape))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        flat = self._buffers.get(key)
        if flat is None or flat.numel() < n:
            flat = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._buffers[key] = flat
            self.ops.generation += 1       # captured graphs point at the old memory
            for old in [k for k in self._views if k[0] == tag and k[1] == dtype]:
                del self._views[old]
        view = flat[:n].view(shape)
        if len(self._views) > 4096:          # many shapes have come and gone
            self._views.clear()
        self._views[(tag, dtype, shape)] = view
        return view
