"""The engine's kernels as Python functions on torch CUDA tensors.

Every function validates its tensors (device, dtype, contiguity, shapes), then launches a
hand-written kernel from ``iian_b200/csrc`` on the current CUDA stream through ``ctypes``.
Nothing here computes with torch ops; a tensor that is not on a CUDA device is an error, there
is no CPU path.  Large bfloat16 matrix products may go to the library GEMM, as in the reference
(third_party/ggml/src/ggml-cuda/ggml-cuda.cu:1548-1608 calls cuBLAS for batches its own
mat-vec kernels do not cover).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_ERRS = {1: "element types not supported by this kernel", 2: "a size this kernel refuses",
         3: "a pointer or stride is not aligned as the kernel requires", 4: "beyond the kernel's stated maximum",
         5: "the address of a device array inside the library could not be resolved"}


LAUNCHES = [0]        # kernel launches issued by this module (a split attention counts its merge kernel too)
LAUNCHES_BY_ENTRY = {}     # the same by entry point ("attention_tc", "gemm_skinny_fused", ...; "library_gemm" for cuBLAS):
                           # tests read it to see which kernel a step was served by (a replayed graph counts once, at capture)


def _check(code: int, what: str) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        LAUNCHES_BY_ENTRY[what] = LAUNCHES_BY_ENTRY.get(what, 0) + 1
        return
    if code >= 1000:
        raise KernelError(f"{what}: CUDA launch failed with error {code - 1000}")
    raise KernelError(f"{what}: {_ERRS.get(code, f'error {code}')}")


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: Optional[torch.Tensor], what: str, dtype=None) -> int:
    """Pointer of a contiguous CUDA tensor (0 for None)."""
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the engine's kernels run on CUDA only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t.data_ptr()


_PINNED_STREAM = [0]


def _stream() -> int:
    """The CUDA stream the kernels are launched on: torch's current stream, looked up once per forward pass
    (``pin_stream``) rather than once per launch -- the lookup costs more than the launch itself."""
    return _PINNED_STREAM[0] or torch.cuda.current_stream().cuda_stream


class pin_stream:
    """``with pin_stream():`` every launch inside goes to the stream that is current on entry.  Code that
    switches streams inside (the weight prefetcher's side stream) passes its stream explicitly."""

    def __enter__(self):
        self.before = _PINNED_STREAM[0]
        _PINNED_STREAM[0] = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        _PINNED_STREAM[0] = self.before
        return False


_sigs_done = set()


# Programmatic dependent launch (see csrc/common.cuh).  IIAN_PDL names the kernel libraries whose launches get the
# attribute ("gemm_stream,attention_mma"; "1": all, "0": none).  Default: the streaming product alone.  Its CTAs fill
# their ring of shared memory with weights while the kernel before drains, and they cannot crowd that kernel out (a CTA
# takes nearly all of an SM's shared memory, so it only becomes resident where one has left): 3.10 -> 2.91 ms per decode
# step at batch 1, 3.60 -> 3.31 at batch 8.  With the attribute on every kernel of the step the register-bound kernels
# of the chain did lose resources to their successors (4.16 ms at batch 1 when the products were of that kind).
_PDL_ENV = os.environ.get("IIAN_PDL", "gemm_stream")
PDL = _PDL_ENV not in ("0", "false", "off")
_PDL_LIBS = None if _PDL_ENV in ("0", "false", "off", "1", "true", "on") else {n.strip() for n in _PDL_ENV.split(",")}


def pdl_for(lib_name: str) -> bool:
    return PDL and (_PDL_LIBS is None or lib_name in _PDL_LIBS)


_pdl_set = set()


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = _build.load(lib_name)
    if lib_name not in _pdl_set:
        _pdl_set.add(lib_name)
        if hasattr(lib, "iian_set_pdl"):
            lib.iian_set_pdl.argtypes = [c_int]
            lib.iian_set_pdl.restype = None
            lib.iian_set_pdl(1 if pdl_for(lib_name) else 0)
    fn = getattr(lib, fn_name)
    key = (lib_name, fn_name)
    if key not in _sigs_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _sigs_done.add(key)
    return fn


class CudaKernels:
    """The kernel set the product path uses."""

    name = "cuda"

    # ---- libraries a model needs (compiled together on first use) ----------------------
    def prepare(self, dtype: torch.dtype) -> None:
        names = ["elementwise", "rope_kv", "attention_generic", "gemm_simt", "sampling"]
        if dtype == torch.bfloat16:
            names += [n for n in _build.SOURCES if n not in names and n in _build.BF16_SOURCES]
        _build.preload(names)

    # ---- row-wise ------------------------------------------------------------------------
    def embedding(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
        n, h = out.shape
        fn = _fn("elementwise", "iian_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(table, "embedding table"), _code(table, "embedding table"),
                  _cuda(tokens, "tokens", torch.int32), _cuda(out, "embedding out", torch.float32),
                  n, h, table.shape[0], _stream()), "embedding")

    def add_rms_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                     eps: float, out: torch.Tensor) -> None:
        n, h = residual.shape
        if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype):
            raise KernelError(f"add_rms_norm: delta {tuple(delta.shape)} {delta.dtype} does not match "
                              f"residual {tuple(residual.shape)} / out {out.dtype}")
        if out.shape != residual.shape or weight.numel() != h:
            raise KernelError("add_rms_norm: shapes of out / weight do not match the residual")
        fn = _fn("elementwise", "iian_add_rms_norm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(delta, "delta"),
                  _cuda(weight, "norm weight", torch.float32), _cuda(out, "norm out"), _code(out, "norm out"),
                  n, h, eps, _stream()), "add_rms_norm")

    def rms_norm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        n, h = x.shape
        if out.shape != x.shape or out.dtype != x.dtype or weight.numel() != h:
            raise KernelError("rms_norm: out / weight do not match the input")
        fn = _fn("elementwise", "iian_rms_norm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(x, "rms_norm in"), _cuda(weight, "norm weight", torch.float32), _cuda(out, "rms_norm out"),
                  _code(x, "rms_norm in"), n, h, eps, _stream()), "rms_norm")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
        """``interleave`` 0: columns are [gate | up]; 8: groups of 16 columns, 8 gate then 8 up values."""
        n, f2 = gate_up.shape
        if out.shape != (n, f2 // 2) or f2 % 2 or out.dtype != gate_up.dtype:
            raise KernelError("swiglu: out must be [N, F] for gate_up [N, 2F] of the same dtype")
        fn = _fn("elementwise", "iian_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(gate_up, "gate_up"), _cuda(out, "swiglu out"), _code(out, "swiglu out"), n, f2 // 2, interleave,
                  _stream()), "swiglu")

    def gather_rows(self, src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        r, h = out.shape
        if src.shape[1] != h or src.dtype != out.dtype or rows.numel() != r:
            raise KernelError("gather_rows: shapes or dtypes do not match")
        fn = _fn("elementwise", "iian_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(src, "gather src"), _cuda(rows, "rows", torch.int32), _cuda(out, "gather out"),
                  _code(src, "gather src"), r, h, src.shape[0], _stream()), "gather_rows")

    def add_bias(self, x: torch.Tensor, bias: torch.Tensor) -> None:
        n, m = x.shape
        if bias.numel() != m:
            raise KernelError("add_bias: bias length does not match")
        fn = _fn("elementwise", "iian_add_bias", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "add_bias x"), _cuda(bias, "bias", torch.float32), _code(x, "add_bias x"), n, m, _stream()),
               "add_bias")

    # ---- matrix products -----------------------------------------------------------------
    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale=None, residual_norm=None) -> None:
        """out[n, m] = sum_k x[n, k] * w[m, k].  ``row_scale`` (ops.fused.RowScale) and ``residual_norm``
        (ops.fused.ResidualNorm) ask for the fused forms; ``can_fuse_norm`` says whether they are available."""
        n, k = x.shape
        m = w.shape[0]
        if w.shape[1] != k or out.shape != (n, m):
            raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        if n == 0:
            return
        if row_scale is not None or residual_norm is not None:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out, row_scale=row_scale, residual_norm=residual_norm)
            else:
                self.gemm_skinny_fused(x, w, out, 2 if residual_norm is not None else 0, row_scale, residual_norm)
            return
        self._linear_dispatch(x, w, out, n, m, k)

    FUSE_NORM = os.environ.get("IIAN_FUSE_NORM", "1") not in ("0", "false", "off")

    def can_fuse_norm(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """Whether the product of ``x`` with ``w`` can carry a RowScale or a ResidualNorm (the weight-streaming
        kernel's range: up to 8 rows of bfloat16)."""
        n, k = x.shape
        return self.FUSE_NORM and (self._skinny_ok(x, w, n, k) or self._tcgen05_ok(x, w, n, k))

    def can_take_prenormed(self, n_rows: int, w: torch.Tensor, dtype: torch.dtype) -> bool:
        """Whether a product of ``n_rows`` rows with ``w`` can carry a RowScale: the row counts of the weight-streaming
        kernel and of the tcgen05 kernel (the library product between them cannot)."""
        if not self.FUSE_NORM or dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.data_ptr() % 16:
            return False
        k = w.shape[1]
        if n_rows <= self.SKINNY_MAX_ROWS:
            return k % 32 == 0
        return self._tcgen05_rows_ok(n_rows, w.shape[0]) and k % 8 == 0 and not self.LIBRARY_GEMM_ONLY

    def norm_parts(self, w: torch.Tensor, n_rows: int = 1) -> int:
        """Parts in which a ResidualNorm product of ``n_rows`` rows with weight ``w`` leaves the sums of squares."""
        if n_rows > self.SKINNY_MAX_ROWS:
            return -(-w.shape[0] // self.tcgen05_tile_columns(n_rows, w.shape[0]))
        return -(-w.shape[0] // 16)

    def gemm_skinny_fused(self, x, w, out, epilogue: int, row_scale=None, residual_norm=None) -> None:
        n, k = x.shape
        m = w.shape[0]
        if not self._skinny_ok(x, w, n, k):
            raise KernelError("linear: the fused forms need up to 8 rows of bfloat16, K a multiple of 32")
        in_p = in_tiles = 0
        inv_w = eps = 0.0
        if row_scale is not None:
            if row_scale.partials.dtype != torch.float32 or row_scale.partials.shape[0] != n:
                raise KernelError("linear: RowScale partials must be float32 [rows, parts]")
            in_p, in_tiles = _cuda(row_scale.partials, "row-scale partials"), row_scale.partials.shape[1]
            inv_w, eps = 1.0 / row_scale.width, row_scale.eps
        res = nw = out_p = 0
        if residual_norm is not None:
            rn = residual_norm
            if (rn.residual.shape != (n, m) or rn.residual.dtype != torch.float32 or rn.weight.numel() != m
                    or rn.partials.shape != (n, self.norm_parts(w)) or out.dtype != torch.bfloat16):
                raise KernelError("linear: ResidualNorm operands do not fit the product")
            res, nw = _cuda(rn.residual, "residual", torch.float32), _cuda(rn.weight, "norm weight", torch.float32)
            out_p = _cuda(rn.partials, "norm partials", torch.float32)
        if self.prefetcher is not None:
            self.prefetcher.before_product(self)
        if self.STREAM_PRODUCT:
            self._gemm_stream(x, w, out, n, m, k, epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p)
        else:
            fn = _fn("gemm_skinny", "iian_gemm_skinny_fused",
                     [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_float,
                      c_void_p, c_void_p, c_void_p, c_void_p])
            _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"), n, m, k,
                      epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p, _stream()), "gemm_skinny_fused")
        if self.weight_log is not None:
            self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
        if self.prefetcher is not None:
            self.prefetcher.after_product(self)

    # Up to 8 rows: the product whose weights stream through a ring of shared-memory stages filled by bulk asynchronous
    # copies (csrc/gemm_stream.cu) instead of the one that loads them into registers (csrc/gemm_skinny.cu); the results
    # are the same bits.  IIAN_STREAM_PRODUCT=0 goes back to the register form.
    STREAM_PRODUCT = os.environ.get("IIAN_STREAM_PRODUCT", "1") not in ("0", "false", "off")
    STREAM_STAGES = int(os.environ.get("IIAN_STREAM_STAGES", "12"))
    _stream_stages_set = None

    def _gemm_stream(self, x, w, out, n, m, k, epilogue, in_p=0, in_tiles=0, inv_w=0.0, eps=0.0, res=0, nw=0, out_p=0) -> None:
        if self._stream_stages_set != self.STREAM_STAGES:
            fn = _fn("gemm_stream", "iian_gemm_stream_stages", [c_int])
            if fn(self.STREAM_STAGES) != 0:
                raise KernelError("gemm_stream: the ring has 6 or 12 stages")
            type(self)._stream_stages_set = self.STREAM_STAGES
        status = self.tcgen05_status_buffer(x.device).data_ptr()
        CudaKernels._tc_used = True
        fn = _fn("gemm_stream", "iian_gemm_stream",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_float,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"), n, m, k,
                  epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p, status, _stream()), "gemm_stream")

    # rows up to which the weight-streaming kernel is used; above it the library GEMM takes over
    # (measured on B200 at the Qwen3-8B sizes: the streaming kernel wins up to 8 rows, cuBLAS from 16)
    SKINNY_MAX_ROWS = 8

    # Weight prefetch for captured decode graphs (see csrc/prefetch.cu and WeightPrefetcher below)
    weight_log = None          # a list while the order of weight-streaming products is being recorded
    prefetcher = None          # a WeightPrefetcher while a decode graph is being captured

    # rows from which the tcgen05 kernel takes over (below it, and above the streaming kernel's range, the
    # library GEMM is faster: one row tile of 128 leaves most SMs without work)
    TCGEN05_MIN_ROWS = 128
    LIBRARY_GEMM_ONLY = os.environ.get("IIAN_LIBRARY_GEMM", "0") not in ("0", "false", "off")

    # ... and only when the product has many tiles of 256 x 256 (several waves of the 74 pairs of SMs): with few tiles
    # the SMs that work cannot stream the weights fast enough, and with one or two waves the idle tail of the last
    # wave costs more than the fused epilogue saves; the library product (which splits K, and uses TMA multicast in
    # clusters of four) is faster there.  Measured on B200 at the Qwen3-8B sizes, whole prefill steps in ms with the
    # threshold at 0 / 64 / 130 / 400 / all library: 256 tokens 9.4 / 6.5 / - / - / -; 1024 tokens 15.2 / 15.2 / 13.9 /
    # 14.4 / 14.3; 2048 tokens 27.1 / 27.1 / 26.2 / 25.9 / 27.6; 4096 tokens - / - / 54.4 / 52.5 / 52.9.  At 300 the own
    # kernel takes the gate/up product with its SwiGLU epilogue from 1024 rows on (384 tiles) and nothing else of a layer.
    TCGEN05_MIN_TILES = int(os.environ.get("IIAN_TCGEN05_MIN_TILES", "300"))

    def _tcgen05_rows_ok(self, n: int, m: int) -> bool:
        return n >= self.TCGEN05_MIN_ROWS and (-(-n // 256)) * (-(-m // 256)) >= self.TCGEN05_MIN_TILES

    def _tcgen05_ok(self, x, w, n, k) -> bool:
        return (not self.LIBRARY_GEMM_ONLY and self._tcgen05_rows_ok(n, w.shape[0]) and k % 8 == 0
                and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def _skinny_ok(self, x, w, n, k) -> bool:
        return (n <= self.SKINNY_MAX_ROWS and k % 32 == 0 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def can_fuse_swiglu(self, x: torch.Tensor, w: torch.Tensor, interleave: int) -> bool:
        """Whether ``linear_swiglu`` can run for these operands (else: linear, then swiglu)."""
        n, k = x.shape
        return interleave == 8 and w.shape[0] % 16 == 0 and (self._tcgen05_ok(x, w, n, k) or self._skinny_ok(x, w, n, k))

    def linear_swiglu(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale=None) -> None:
        """out[t, f] = silu(x . w_gate_f) * (x . w_up_f) for w with gate and up rows interleaved in groups of 8."""
        n, k = x.shape
        if row_scale is not None:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out, epilogue=1, row_scale=row_scale)
            else:
                self.gemm_skinny_fused(x, w, out, 1, row_scale, None)
            return
        if self._tcgen05_ok(x, w, n, k):
            self.gemm_tcgen05(x, w, out, epilogue=1)
            return
        if self.prefetcher is not None:
            self.prefetcher.before_product(self)
        if self.STREAM_PRODUCT:
            self._gemm_stream(x, w, out, n, w.shape[0], k, 1)
        else:
            self.gemm_skinny(x, w, out, epilogue=1)
        if self.weight_log is not None:
            self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
        if self.prefetcher is not None:
            self.prefetcher.after_product(self)

    def _linear_dispatch(self, x, w, out, n, m, k) -> None:
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out)
                return
            if n <= self.SKINNY_MAX_ROWS and k % 32 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
                if self.prefetcher is not None:
                    self.prefetcher.before_product(self)
                if self.STREAM_PRODUCT:
                    self._gemm_stream(x, w, out, n, m, k, 0)
                else:
                    self.gemm_skinny(x, w, out)
                if self.weight_log is not None:
                    self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
                if self.prefetcher is not None:
                    self.prefetcher.after_product(self)
                return
            if n > self.SKINNY_MAX_ROWS and self._library_gemm(x, w, out):
                return
        self.gemm_simt(x, w, out)

    _library_f32_out = True

    def _library_gemm(self, x, w, out) -> bool:
        """cuBLAS through torch.mm, for large bfloat16 products (as the reference does for large batches)."""
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
            LAUNCHES_BY_ENTRY["library_gemm"] = LAUNCHES_BY_ENTRY.get("library_gemm", 0) + 1
            return True
        if out.dtype == torch.float32 and self._library_f32_out:
            try:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
                LAUNCHES_BY_ENTRY["library_gemm"] = LAUNCHES_BY_ENTRY.get("library_gemm", 0) + 1
                return True
            except (TypeError, RuntimeError):
                type(self)._library_f32_out = False
        return False

    def skinny_ksplit(self, n: int, m: int, k: int) -> int:
        """Into how many CTAs K is cut: matrices with few rows would otherwise leave most of the GPU's
        memory pipeline idle (a row block of 16 is one CTA)."""
        return 1       # measured on B200 at the Qwen3-8B sizes: one CTA per row block is fastest for every shape

    def gemm_skinny(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, cfg: int = 0, ksplit: int = 0,
                    epilogue: int = 0) -> None:
        """``cfg`` picks a tile configuration (rows-per-block tiles * 100 + warps * 10 + unroll); ``ksplit``
        the number of CTAs that share K for one row block; 0: defaults."""
        n, k = x.shape
        m = w.shape[0]
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise KernelError("gemm_skinny: x and w must be bfloat16")
        if ksplit <= 0:
            ksplit = 1 if epilogue else self.skinny_ksplit(n, m, k)
        part = counters = 0
        if ksplit > 1:
            rows = 32 if n > 8 else 16
            blocks = -(-m // rows)
            nt = 1 if n <= 8 else 2 if n <= 16 else 4 if n <= 32 else 8
            part = self.gemm_scratch(x.device, blocks * ksplit * rows * 8 * nt).data_ptr()
            counters = self.gemm_counters(x.device, blocks).data_ptr()
        fn = _fn("gemm_skinny", "iian_gemm_skinny_cfg",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                  n, m, k, cfg, ksplit, part, counters, epilogue, _stream()), "gemm_skinny")

    _gemm_scratch = {}
    _gemm_counters = {}

    def gemm_scratch(self, device, n_floats: int) -> torch.Tensor:
        t = self._gemm_scratch.get(device)
        if t is None or t.numel() < n_floats:
            t = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
            self._gemm_scratch[device] = t
            self._scratch_keep.append(t)
        return t

    def gemm_counters(self, device, n: int) -> torch.Tensor:
        t = self._gemm_counters.get(device)
        if t is None or t.numel() < n:
            t = torch.zeros(max(n, 1 << 14), dtype=torch.int32, device=device)
            self._gemm_counters[device] = t
            self._scratch_keep.append(t)
        return t

    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        n, k = x.shape
        m = w.shape[0]
        fn = _fn("gemm_simt", "iian_gemm_simt",
                 [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "linear x"), _code(x, "linear x"), _cuda(w, "linear w"), _code(w, "linear w"),
                  _cuda(out, "linear out"), _code(out, "linear out"), n, m, k, _stream()), "gemm_simt")

    # ---- tcgen05 + TMA product for many rows ----------------------------------------------------
    _tc_status = {}

    def tcgen05_status_buffer(self, device) -> torch.Tensor:
        t = self._tc_status.get(device)
        if t is None:
            t = torch.zeros(2, dtype=torch.int32, device=device)
            self._tc_status[device] = t
        return t

    _tc_used = False           # a tcgen05 kernel was launched since the status was last read

    def check_device_status(self) -> None:
        """Called where the host has just waited for the device anyway (tokens or logits were read): if a tcgen05
        kernel ran since the last call, read its status words and raise if one gave up on a barrier."""
        if not CudaKernels._tc_used:
            return
        for device in list(self._tc_status):
            self.tcgen05_check(device)

    def tcgen05_check(self, device) -> None:
        """Synchronise and raise if a tcgen05 kernel gave up waiting (its output would be garbage)."""
        CudaKernels._tc_used = False
        t = self._tc_status.get(device)
        if t is None:
            return
        code, where = t.tolist()
        if code != 0:
            t.zero_()
            raise KernelError(f"a kernel gave up waiting on a barrier (wait {code}, iteration {where}); its result is not valid")

    TCGEN05_PAIR = os.environ.get("IIAN_TCGEN05_PAIR", "1") not in ("0", "false", "off")

    @classmethod
    def tcgen05_tile(cls, n_rows: int, n: int) -> int:
        """The tile of the tcgen05 product for ``n_rows`` rows and a weight with ``n`` rows: 128 or 256 columns on one
        SM, or 512: tiles of 256 x 256 on pairs of SMs (from two row tiles on)."""
        wide = n % 256 == 0 or n > 4096
        if wide and cls.TCGEN05_PAIR and n_rows > 128:
            return 512
        return 256 if wide else 128

    @classmethod
    def tcgen05_tile_columns(cls, n_rows: int, n: int) -> int:
        return min(256, cls.tcgen05_tile(n_rows, n))

    def gemm_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, bn: int = 0,
                     row_scale=None, residual_norm=None) -> None:
        """``epilogue`` 0: out[t, n] = x . w; 1: w holds gate and up rows interleaved in groups of 8 and
        out[t, f] = silu(gate_f) * up_f with half as many columns; 2 (with ``residual_norm``): the residual add and
        the next norm's weight ride in the epilogue.  ``row_scale``: rows are multiplied by a folded norm's factor."""
        t_rows, k = x.shape
        n = w.shape[0]
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise KernelError("gemm_tcgen05: x and w must be bfloat16")
        want_cols = n // 2 if epilogue == 1 else n
        if w.shape[1] != k or out.shape != (t_rows, want_cols):
            raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        if bn == 0:
            bn = self.tcgen05_tile(t_rows, n)
        status = self.tcgen05_status_buffer(x.device).data_ptr()
        CudaKernels._tc_used = True
        if row_scale is None and residual_norm is None:
            fn = _fn("gemm_tcgen05", "iian_gemm_tcgen05",
                     [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
            _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                      t_rows, n, k, epilogue, bn, status, _stream()), "gemm_tcgen05")
            return
        in_p = in_tiles = 0
        inv_w = eps = 0.0
        if row_scale is not None:
            if row_scale.partials.dtype != torch.float32 or row_scale.partials.shape[0] != t_rows:
                raise KernelError("linear: RowScale partials must be float32 [rows, parts]")
            in_p, in_tiles = _cuda(row_scale.partials, "row-scale partials"), row_scale.partials.shape[1]
            inv_w, eps = 1.0 / row_scale.width, row_scale.eps
        res = nw = out_p = 0
        if residual_norm is not None:
            rn = residual_norm
            if (rn.residual.shape != (t_rows, n) or rn.residual.dtype != torch.float32 or rn.weight.numel() != n
                    or rn.partials.shape != (t_rows, -(-n // min(bn, 256))) or out.dtype != torch.bfloat16):
                raise KernelError("linear: ResidualNorm operands do not fit the product")
            res, nw = _cuda(rn.residual, "residual", torch.float32), _cuda(rn.weight, "norm weight", torch.float32)
            out_p = _cuda(rn.partials, "norm partials", torch.float32)
            epilogue = 2
        fn = _fn("gemm_tcgen05", "iian_gemm_tcgen05_fused",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                  c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                  t_rows, n, k, epilogue, bn, status, in_p, in_tiles, inv_w, eps, res, nw, out_p, _stream()), "gemm_tcgen05")

    def prefetch_l2(self, ptr: int, nbytes: int, stream: Optional[int] = None) -> None:
        fn = _fn("prefetch", "iian_prefetch_l2", [c_void_p, c_longlong, c_void_p])
        _check(fn(ptr, nbytes, _stream() if stream is None else stream), "prefetch_l2")

    # ---- attention -----------------------------------------------------------------------
    def qk_norm_rope_store(self, qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                           v_cache: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                           inv_freq: Optional[torch.Tensor], rot_dim: int, rope_style: int,
                           positions: torch.Tensor, slots: Optional[torch.Tensor], write_kv: bool,
                           bias: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None) -> None:
        n = qkv.shape[0]
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if qkv.shape[1] != width or q_out.numel() != n * num_heads * head_dim or q_out.dtype != qkv.dtype:
            raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} does not match {num_heads}+2*{num_kv_heads} "
                              f"heads of {head_dim}")
        page_size = num_pages = 0
        if write_kv:
            if k_cache is None or v_cache is None or slots is None:
                raise KernelError("qk_norm_rope_store: a cache and slots are needed to store K and V")
            if k_cache.dtype != qkv.dtype or k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads \
                    or k_cache.shape[3] != head_dim:
                raise KernelError(f"qk_norm_rope_store: cache {tuple(k_cache.shape)} {k_cache.dtype} does not match")
            num_pages, page_size = k_cache.shape[0], k_cache.shape[2]
        if inv_freq is not None and inv_freq.numel() < rot_dim // 2:
            raise KernelError("qk_norm_rope_store: inv_freq is shorter than rot_dim / 2")
        fn = _fn("rope_kv", "iian_qk_norm_rope_store",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
        if table is not None and (inv_freq is None or table.numel() < 2 * n * (rot_dim // 2)):
            raise KernelError("qk_norm_rope_store: the rotary table does not cover these tokens")
        _check(fn(_cuda(qkv, "qkv"), _cuda(bias, "qkv bias", torch.float32), _cuda(q_out, "q out"),
                  _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"),
                  _cuda(q_weight, "q norm weight", torch.float32), _cuda(k_weight, "k norm weight", torch.float32),
                  _cuda(inv_freq, "inv_freq", torch.float32), _cuda(table, "rotary table", torch.float32),
                  _cuda(positions, "positions", torch.int32),
                  _cuda(slots, "slots", torch.int32), _code(qkv, "qkv"), n, num_heads, num_kv_heads, head_dim,
                  rot_dim if inv_freq is not None else 0, rope_style, eps, page_size, num_pages, 1 if write_kv else 0,
                  _stream()), "qk_norm_rope_store")

    def rotary_table(self, inv_freq: torch.Tensor, positions: torch.Tensor, half: int, out: torch.Tensor) -> None:
        """out[t, p] = (cos, sin)(positions[t] * inv_freq[p]), float32 [N, half, 2]."""
        n = positions.shape[0]
        if out.numel() < 2 * n * half or inv_freq.numel() < half:
            raise KernelError("rotary_table: output or inv_freq too small")
        fn = _fn("rope_kv", "iian_rotary_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
        _check(fn(_cuda(inv_freq, "inv_freq", torch.float32), _cuda(positions, "positions", torch.int32),
                  _cuda(out, "rotary table", torch.float32), n, half, _stream()), "rotary_table")

    def paged_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                        meta, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                        window: Optional[int], n_split: Optional[int] = None) -> None:
        """``meta``: an object with ``positions``, ``seq_of_token``, ``block_table`` [S, max_blocks],
        ``ctx_len`` [S] (int32 CUDA tensors) and host-side hints (``num_seqs``, ``max_q_len``, ``max_ctx``,
        ``decode_only``).  ``n_split``: a fixed number of key splits for the decode form (a captured graph's); None:
        chosen per launch."""
        self._attention_dispatch(q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, head_dim, scale, window, n_split)

    # prefill portions on tcgen05 (csrc/attention_tc.cu); IIAN_ATTENTION_TC=0 keeps them on the mma.sync kernel
    ATTENTION_TC = os.environ.get("IIAN_ATTENTION_TC", "1") not in ("0", "false", "off")
    TC_ATTENTION_MIN_ROWS = 64        # rows (tokens x heads per KV head) of the longest portion from which it is used

    def _attention_tc_ok(self, q, k_cache, meta, nh, nkv, hd) -> bool:
        return (self.ATTENTION_TC and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and hd == 128
                and k_cache.shape[2] in (8, 16, 32, 64, 128) and nkv > 0 and nh % nkv == 0
                and meta.max_q_len * (nh // nkv) >= self.TC_ATTENTION_MIN_ROWS)

    def paged_attention_tc(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                           sink: Optional[torch.Tensor] = None) -> None:
        """Prefill attention on tcgen05 + TMA: head size 128, bfloat16, pages of 8 to 128 tokens.  ``sink``: float32 [heads],
        a logit per head that joins the softmax's denominator (needs ``scale`` > 0)."""
        n = q.shape[0]
        if k_cache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("paged_attention_tc: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError("paged_attention_tc: cache / q shapes do not match the head counts")
        status = self.tcgen05_status_buffer(q.device)
        CudaKernels._tc_used = True
        bt = meta.block_table
        if sink is not None and sink.numel() != num_heads:
            raise KernelError("paged_attention_tc: one sink per head")
        fn = _fn("attention_tc", "iian_attention_tc_sink",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, num_heads,
                  num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], scale, window or 0,
                  status.data_ptr(), _cuda(sink, "sink", torch.float32), _stream()), "attention_tc")

    def _attention_dispatch(self, q, k_cache, v_cache, out, meta, nh, nkv, hd, scale, window, n_split=None) -> None:
        if self._attention_tc_ok(q, k_cache, meta, nh, nkv, hd):
            self.paged_attention_tc(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                    scale=scale, window=window)
            return
        if q.dtype == torch.bfloat16 and hd in (64, 128):
            self.paged_attention_mma(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                     scale=scale, window=window, n_split=n_split)
        else:
            self.paged_attention_generic(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                         scale=scale, window=window)

    DECODE_STAGES = int(os.environ.get("IIAN_DECODE_STAGES", "2"))     # shared-memory tiles per CTA of the decode kernel
    _sm_count = {}

    @classmethod
    def sm_count(cls, device=None) -> int:
        """Streaming multiprocessors of ``device`` (the current one by default), asked from the driver once."""
        idx = torch.cuda.current_device() if device is None else torch.device(device).index
        if idx is None:
            idx = torch.cuda.current_device()
        n = cls._sm_count.get(idx)
        if n is None:
            n = cls._sm_count[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
        return n

    @property
    def DECODE_SLOTS(self) -> int:
        """CTAs of the decode kernel with split keys one launch should not exceed: 2.7 per SM (three fit; clusters
        need their CTAs inside one GPC, which leaves some places empty)."""
        return self.DECODE_CTAS_PER_SM_X10 * self.sm_count() // 10

    DECODE_CTAS_PER_SM_X10 = int(round(10 * float(os.environ.get("IIAN_DECODE_CTAS_PER_SM", "2.7"))))
    _stages_set = None

    @staticmethod
    def apply_unsplit_stages() -> None:
        """IIAN_DECODE_UNSPLIT_STAGES=2|3 fixes the tiles per CTA of decode attention with unsplit keys (a measurement
        switch; by default the kernel library chooses by the number of waves of CTAs each form needs)."""
        v = os.environ.get("IIAN_DECODE_UNSPLIT_STAGES")
        if v:
            if _fn("attention_mma", "iian_attention_unsplit_stages", [c_int])(int(v)) != 0:
                raise KernelError("IIAN_DECODE_UNSPLIT_STAGES takes 2 or 3")

    def set_decode_stages(self, stages: int) -> None:
        """2: three CTAs per SM with one tile in flight each; 3: two CTAs with two tiles in flight."""
        fn = _fn("attention_mma", "iian_attention_decode_stages", [c_int])
        code = fn(stages)
        if code != 0:
            raise KernelError("attention: the decode kernel has 2 or 3 stages")
        type(self)._stages_set = stages
        type(self).DECODE_STAGES = stages
        self.apply_unsplit_stages()
    CLUSTER_MERGE = os.environ.get("IIAN_ATTENTION_CLUSTER", "1") not in ("0", "false", "off")
    MAX_SPLITS = int(os.environ.get("IIAN_DECODE_MAX_SPLITS", "32"))
    _scratch = {}
    _scratch_keep = []

    def attention_splits(self, num_seqs: int, num_kv_heads: int, max_ctx: int) -> int:
        """How many parts the keys of a decode step are cut into, so that few long sequences still fill
        the GPU.  Measured on B200 (replayed graphs, 8 KV heads of 128, contexts of 1k to 8k, batches 1 to
        128): all CTAs of a launch should be resident at once (a second wave repeats the whole chain of dependent
        loads: 24.6 us with 8 parts against 14.7 us with 4 at batch 8), which with split keys means up to 2.7 per SM
        (35.0 us with 2 parts against 51.8 us unsplit at batch 20, 21.9 against 30.7 us with 4 against 2 at batch 10;
        but 65 against 53 us at batch 28, where two parts no longer fit), and a CTA should keep at least two key
        tiles.  The parts of a sequence are a power of two and merge inside a thread-block cluster, up to 16 of them
        (more than 8 is a size a kernel has to ask for, and only some 24 such clusters fit the GPU: 13.6 us with 8
        against 22.7 us with 16 parts at batch 3), which saves three trips through L2 (write the parts, count
        arrivals, read them back: one launch at batch 1 and 8k context takes 27.9 us with 8 parts, 18.6 us with 16 in
        a cluster, 25.9 us with 16 and 30.8 us with 32 merged through scratch memory); 32 parts through scratch
        memory are only taken for a single sequence from 32k of context on (48.8 against 52.9 us)."""
        tiles = max(1, (max_ctx + 63) // 64)
        base = max(1, num_seqs * num_kv_heads)
        if os.environ.get("IIAN_DECODE_FORCE_SPLITS"):
            return int(os.environ["IIAN_DECODE_FORCE_SPLITS"])
        n = max(1, min(self.DECODE_SLOTS // base, -(-tiles // 2), self.MAX_SPLITS))
        if n >= 32 and tiles >= 512:
            return n
        if n >= 16:
            return 16 if base * 16 <= 2 * self.sm_count() else 8
        return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1

    def attention_scratch(self, device, n_floats: int) -> torch.Tensor:
        t = self._scratch.get(device)
        if t is None or t.numel() < n_floats:
            t = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
            self._scratch[device] = t
            self._scratch_keep.append(t)        # a captured graph may still point at an older, smaller buffer
        return t

    _counters = {}

    def attention_counters(self, device, n: int) -> torch.Tensor:
        """Zeroed int32 counters for the decode kernel's in-kernel merge (it puts them back to zero)."""
        t = self._counters.get(device)
        if t is None or t.numel() < n:
            t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
            self._counters[device] = t
            self._scratch_keep.append(t)
        return t

    def paged_attention_mma(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                            n_split: Optional[int] = None, small_tiles: Optional[bool] = None,
                            cluster: Optional[bool] = None, sink: Optional[torch.Tensor] = None) -> None:
        """``sink``: float32 [heads], a logit per head that joins the softmax's denominator (needs ``scale`` > 0).
        ``small_tiles``: the decode form (rows of one token, keys split over the warps); ``cluster``: its
        parts merge through the shared memory of a thread-block cluster (2, 4 or 8 parts) instead of scratch
        memory.  None: chosen from the step."""
        n = q.shape[0]
        if k_cache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("paged_attention_mma: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError("paged_attention_mma: cache / q shapes do not match the head counts")
        if self._stages_set != self.DECODE_STAGES:
            self.set_decode_stages(self.DECODE_STAGES)
        decode = meta.max_q_len * (num_heads // num_kv_heads) <= 16
        if small_tiles is None:
            small_tiles = decode
        if n_split is None:
            n_split = self.attention_splits(meta.num_seqs, num_kv_heads, meta.max_ctx) if decode else 1
        if cluster is None:
            cluster = self.CLUSTER_MERGE
        cluster = bool(cluster and small_tiles and n_split in (2, 4, 8, 16))
        part_o = part_lse = counters = 0
        if n_split > 1 and not cluster:
            rows = n * num_heads
            scratch = self.attention_scratch(q.device, rows * n_split * (head_dim + 1))
            part_o = scratch.data_ptr()
            part_lse = part_o + rows * n_split * head_dim * 4
            if small_tiles:
                row_tiles = -(-meta.max_q_len * (num_heads // num_kv_heads) // 16)
                counters = self.attention_counters(q.device, meta.num_seqs * num_kv_heads * row_tiles).data_ptr()
        bt = meta.block_table
        if sink is not None and sink.numel() != num_heads:
            raise KernelError("paged_attention_mma: one sink per head")
        fn = _fn("attention_mma", "iian_attention_mma_sink",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
                  c_void_p])
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  part_o, part_lse, counters, _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, num_heads,
                  num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], scale, window or 0, n_split,
                  (2 if cluster else 1) if small_tiles else 0, self._decode_status(q.device) if small_tiles else None,
                  _cuda(sink, "sink", torch.float32), _stream()), "attention_mma")
        if n_split > 1 and not small_tiles:
            LAUNCHES[0] += 1

    FUSED_DECODE = os.environ.get("IIAN_FUSED_DECODE_ATTENTION", "1") not in ("0", "false", "off")
    # decode attention fetches its K/V tiles by TMA (head size 128, pages of 8 to 64 tokens); IIAN_DECODE_TMA=0: cp.async
    DECODE_TMA = os.environ.get("IIAN_DECODE_TMA", "1") not in ("0", "false", "off")

    # native step function, mixed steps: the decoded tokens' attention runs on the decode kernel on a second stream
    # beside the prefill kernel; IIAN_SPLIT_MIXED=0: one launch of the prefill kernel for all sequences of the step
    SPLIT_MIXED = os.environ.get("IIAN_SPLIT_MIXED", "1") not in ("0", "false", "off")

    def _decode_status(self, device):
        """The status words the decode kernel's TMA form reports to (the ones of the tcgen05 kernels), or None: the
        cp.async form."""
        if not self.DECODE_TMA:
            return None
        CudaKernels._tc_used = True
        return self.tcgen05_status_buffer(device).data_ptr()

    def can_fuse_decode_attention(self, qkv, meta, *, num_heads, num_kv_heads, head_dim, rot_dim, rope_style, bias) -> bool:
        """Whether ``attention_decode_fused`` covers this step: one token per sequence, bfloat16, heads of 64 or
        128, NEOX rotation over the whole head (or none), no projection bias, at most 16 heads per KV head."""
        return (self.FUSED_DECODE and meta.decode_only and meta.num_tokens == meta.num_seqs and qkv.dtype == torch.bfloat16
                and head_dim in (64, 128) and bias is None and rot_dim in (0, head_dim) and (rope_style == 0 or rot_dim == 0)
                and num_kv_heads > 0 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)

    def attention_decode_fused(self, qkv, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                               q_weight, k_weight, eps, table, slots, write_kv: bool,
                               n_split: Optional[int] = None, cluster: Optional[bool] = None) -> None:
        """Per-head RMSNorm, rotation, the write of the new K and V to the cache and attention over the cache in
        one launch, from the Q|K|V projection ``qkv`` [S, (nh + 2 nkv) * hd] of a step with one token per sequence.
        Without ``write_kv`` the projection holds Q only ([S, nh * hd] is not accepted: pass the full width)."""
        s_ = meta.num_seqs
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if qkv.shape != (s_, width) or out.shape != (s_, num_heads * head_dim):
            raise KernelError(f"attention_decode_fused: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not fit {s_} sequences")
        if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention_decode_fused: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
            raise KernelError("attention_decode_fused: cache shape does not match the head counts")
        if table is not None and (table.dtype != torch.float32 or table.numel() != s_ * head_dim):
            raise KernelError("attention_decode_fused: the rotation table must be float32 [S, hd / 2, 2]")
        if self._stages_set != self.DECODE_STAGES:
            self.set_decode_stages(self.DECODE_STAGES)
        if n_split is None:
            n_split = self.attention_splits(s_, num_kv_heads, meta.max_ctx)
        if cluster is None:
            cluster = self.CLUSTER_MERGE
        cluster = bool(cluster and 2 <= n_split <= 16)
        part_o = part_lse = counters = 0
        if n_split > 1 and not cluster:
            rows = s_ * num_heads
            scratch = self.attention_scratch(qkv.device, rows * n_split * (head_dim + 1))
            part_o = scratch.data_ptr()
            part_lse = part_o + rows * n_split * head_dim * 4
            counters = self.attention_counters(qkv.device, s_ * num_kv_heads).data_ptr()
        bt = meta.block_table
        fn = _fn("attention_mma", "iian_attention_decode_fused",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p])
        _check(fn(_cuda(qkv, "qkv"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  part_o, part_lse, counters, _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], s_, num_heads, num_kv_heads, head_dim,
                  k_cache.shape[2], k_cache.shape[0], scale, window or 0, n_split, 1 if cluster else 0,
                  _cuda(q_weight, "q norm weight", torch.float32), _cuda(k_weight, "k norm weight", torch.float32),
                  _cuda(table, "rotation table", torch.float32), _cuda(slots, "slots", torch.int32), eps,
                  1 if write_kv else 0, self._decode_status(qkv.device), _stream()), "attention_decode_fused")

    def paged_attention_generic(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale,
                                window) -> None:
        n = q.shape[0]
        if k_cache.dtype != q.dtype or out.dtype != q.dtype or k_cache.shape != v_cache.shape:
            raise KernelError("paged_attention: q, caches and out must share one dtype and the caches one shape")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError(f"paged_attention: cache {tuple(k_cache.shape)} / q {tuple(q.shape)} do not match "
                              f"{num_heads}/{num_kv_heads} heads of {head_dim}")
        fn = _fn("attention_generic", "iian_paged_attention_generic",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
        bt = meta.block_table
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  _cuda(meta.positions, "positions", torch.int32), _cuda(meta.seq_of_token, "seq_of_token", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _code(q, "q"), n, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
                  scale, window or 0, _stream()), "paged_attention_generic")

    # ---- post-norm layers: gated residual sum + LayerNorm, depth mix, gated activation (csrc/postnorm.cu) ------------
    @staticmethod
    def _rows(t: Optional[torch.Tensor], what: str):
        """(pointer, row stride) of a CUDA matrix whose rows are contiguous (a column slice of a wider matrix is fine)."""
        if t is None:
            return 0, 0
        if not t.is_cuda:
            raise KernelError(f"{what}: tensor is on {t.device}; the engine's kernels run on CUDA only")
        if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
            raise KernelError(f"{what}: expected a matrix with contiguous rows")
        return t.data_ptr(), t.stride(0)

    def gated_add_layer_norm(self, x: torch.Tensor, sub: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                             gate_bias: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                             alpha: float, eps: float, out: Optional[torch.Tensor], out_act: Optional[torch.Tensor]) -> None:
        """``y = LayerNorm(alpha * x + sub * sigmoid(gate + gate_bias)) * weight + bias``; ``out`` float32 and / or
        ``out_act`` in the activation dtype.  ``sub`` and ``gate`` may be column slices; without ``sub`` it is the plain
        norm of ``alpha * x``."""
        n, h = x.shape
        act = out_act if out_act is not None else sub
        act_code = _code(act, "layer norm") if act is not None else F32
        for t, what in ((sub, "sub"), (gate, "gate")):
            if t is not None and t.shape != (n, h):
                raise KernelError(f"gated_add_layer_norm: {what} {tuple(t.shape)} does not match x {tuple(x.shape)}")
        if sub is not None and _code(sub, "sub") != act_code:
            raise KernelError("gated_add_layer_norm: sub and out_act must share the activation dtype")
        sp, ld_sub = self._rows(sub, "sub")
        gp, ld_g = self._rows(gate, "gate")
        fn = _fn("postnorm", "iian_gated_add_layer_norm",
                 [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_float, c_float, c_void_p])
        _check(fn(_cuda(x, "stream", torch.float32), sp, ld_sub, gp, ld_g, _code(gate, "gate") if gate is not None else act_code,
                  _cuda(gate_bias, "gate bias", torch.float32), _cuda(weight, "norm weight", torch.float32),
                  _cuda(bias, "norm bias", torch.float32), _cuda(out, "norm out", torch.float32), _cuda(out_act, "norm out"),
                  act_code, n, h, alpha, eps, _stream()), "gated_add_layer_norm")

    def depth_mix(self, terms, coef: torch.Tensor, rows: Optional[torch.Tensor], last_is_selected: bool,
                  out: Optional[torch.Tensor], out_act: Optional[torch.Tensor]) -> None:
        """``y[r] = sum_j coef[j] * terms[j][row_j(r)]``: float32 streams [*, H]; with ``rows`` every term (but the last, if
        ``last_is_selected``) is read at ``rows[r]``."""
        ref = out if out is not None else out_act
        r, h = ref.shape
        ptrs = (c_void_p * len(terms))(*[_cuda(t, "mix term", torch.float32) for t in terms])
        if coef.numel() != len(terms) or any(t.shape[1] != h for t in terms):
            raise KernelError("depth_mix: one coefficient per term, all terms of the output's width")
        fn = _fn("postnorm", "iian_depth_mix", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                                c_int, c_int, c_void_p])
        _check(fn(ptrs, len(terms), _cuda(coef, "mix coefficients", torch.float32), _cuda(rows, "rows", torch.int32),
                  terms[0].shape[0], 1 if last_is_selected else 0, _cuda(out, "mix out", torch.float32), _cuda(out_act, "mix out"),
                  _code(out_act, "mix out") if out_act is not None else F32, r, h, _stream()), "depth_mix")

    ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}

    def gated_act(self, gate_up: torch.Tensor, out: torch.Tensor, interleave: int, activation: str, limit: float = 0.0) -> None:
        """``out = act(gate) * up`` for rows ``[gate | up]`` (or interleaved in groups of 8); ``gate_up`` may be a column slice.
        ``clamped_swish`` (with ``limit``): ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``g sigmoid(1.702 g) (u + 1)``."""
        n, f2 = gate_up.shape
        if out.shape != (n, f2 // 2) or f2 % 2 or out.dtype != gate_up.dtype:
            raise KernelError("gated_act: out must be [N, F] for gate_up [N, 2F] of the same dtype")
        gp, ld = self._rows(gate_up, "gate_up")
        fn = _fn("postnorm", "iian_gated_act_limit", [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(gp, ld, _cuda(out, "gated_act out"), _code(out, "gated_act out"), n, f2 // 2, interleave,
                  self.ACTIVATIONS[activation], limit, _stream()), "gated_act")

    # ---- attention over a cached latent (csrc/latent_attention.cu) ------------------------------------------------
    def latent_prep(self, qd: torch.Tensor, q_off: int, dkv_off: int, cache_rows: Optional[torch.Tensor], q_cat: torch.Tensor,
                    norm_weight: torch.Tensor, inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                    slots: Optional[torch.Tensor], *, num_heads: int, dim: int, rot: int, rank: int, rot_dims: int,
                    eps: float, queries: Optional[torch.Tensor] = None, style: int = 0) -> None:
        """From the projected rows ``qd`` (queries at column ``q_off``, the down-projected latent and shared key part at
        ``dkv_off``): normalise the latent, rotate the key part, store both at the token's cache cell, and put the
        rotated part of every query head behind the ``rank`` columns of its row of ``q_cat`` [N, H, rank + rot].
        ``inv_freq`` is float64 [rot_dims / 2].  ``queries``: the queries as a matrix of their own [N, heads * (dim + rot)]
        (then ``q_off`` is not used); ``style`` 0 rotates entry i with entry i + rot_dims / 2, 1 entry 2i with entry 2i + 1."""
        n = qd.shape[0]
        width = rank + rot
        if q_cat.shape != (n, num_heads, width) or q_cat.dtype != qd.dtype:
            raise KernelError("latent_prep: q_cat must be [N, heads, rank + rot] in the activation dtype")
        n_cells = 0
        if cache_rows is not None:
            if cache_rows.dtype != qd.dtype or cache_rows.shape[-1] != width:
                raise KernelError(f"latent_prep: cache {tuple(cache_rows.shape)} {cache_rows.dtype} does not match")
            n_cells = cache_rows.numel() // width
        qp, ld = self._rows(qd, "projected rows")
        qm, ld_q = self._rows(queries, "queries")
        if queries is not None and (queries.shape != (n, num_heads * (dim + rot)) or queries.dtype != qd.dtype):
            raise KernelError("latent_prep: queries must be [N, heads * (dim + rot)] in the activation dtype")
        fn = _fn("latent_attention", "iian_latent_prep_split",
                 [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_void_p])
        _check(fn(qp, ld, q_off, dkv_off, qm, ld_q, style, _cuda(cache_rows, "latent cache"), _cuda(q_cat, "q_cat"),
                  _cuda(norm_weight, "latent norm weight", torch.float32), _cuda(inv_freq, "inv_freq", torch.float64),
                  _cuda(positions, "positions", torch.int32), _cuda(slots if cache_rows is not None else None, "slots", torch.int32),
                  _code(qd, "projected rows"), n, num_heads, dim, rot, rank, rot_dims if inv_freq is not None else 0, eps,
                  n_cells, _stream()), "latent_prep")

    HEAD_LINEAR_FAST = os.environ.get("IIAN_HEAD_LINEAR_FAST", "1") not in ("0", "false", "off")

    def head_linear(self, inp: torch.Tensor, in_off: int, in_head_stride: int, w: torch.Tensor, w_head_stride: int, w_in_stride: int,
                    w_out_stride: int, out: torch.Tensor, out_off: int, out_head_stride: int, *, num_heads: int, n_in: int,
                    n_out: int) -> None:
        """Per token and head: ``out[t, h, j] = sum_i inp[t, h, i] * w[h * w_head_stride + i * w_in_stride + j * w_out_stride]``;
        ``inp`` / ``out`` are matrices whose row holds the heads at ``*_off + h * *_head_stride``."""
        n = inp.shape[0]
        ip, ld_in = self._rows(inp, "head_linear in")
        op, ld_out = self._rows(out, "head_linear out")
        es = inp.element_size()
        if out.dtype != inp.dtype:
            raise KernelError("head_linear: in and out must share the activation dtype")
        if n == 0:
            return
        if inp.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.HEAD_LINEAR_FAST:
            # bfloat16: up to 8 tokens a form that reads the weights once; beyond, the library's batched product on
            # strided views (as plain products of that many rows go to the library)
            contiguous, stride = (n_out, w_in_stride) if w_out_stride == 1 else (n_in, w_out_stride)
            if (n <= 8 and (w_in_stride == 1 or w_out_stride == 1) and n_in * 32 + 8192 <= 48 * 1024 and contiguous % 8 == 0
                    and stride % 8 == 0 and w_head_stride % 8 == 0 and w.data_ptr() % 16 == 0):
                fn = _fn("latent_attention", "iian_head_linear_small",
                         [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong, c_int,
                          c_int, c_int, c_int, c_int, c_void_p])
                _check(fn(ip + in_off * es, ld_in, in_head_stride, _cuda(w, "head_linear w"), w_head_stride, w_in_stride,
                          w_out_stride, op + out_off * es, ld_out, out_head_stride, n, num_heads, n_in, n_out, _stream()),
                       "head_linear_small")
                return
            if n > 8:
                a = torch.as_strided(inp, (num_heads, n, n_in), (in_head_stride, ld_in, 1), inp.storage_offset() + in_off)
                b = torch.as_strided(w, (num_heads, n_in, n_out), (w_head_stride, w_in_stride, w_out_stride), w.storage_offset())
                c = torch.as_strided(out, (num_heads, n, n_out), (out_head_stride, ld_out, 1), out.storage_offset() + out_off)
                torch.bmm(a, b, out=c)
                LAUNCHES_BY_ENTRY["library_gemm"] = LAUNCHES_BY_ENTRY.get("library_gemm", 0) + 1
                return
        fn = _fn("latent_attention", "iian_head_linear",
                 [c_void_p, c_longlong, c_int, c_void_p, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(ip + in_off * es, ld_in, in_head_stride, _cuda(w, "head_linear w"), _code(w, "head_linear w"), w_head_stride,
                  w_in_stride, w_out_stride, op + out_off * es, ld_out, out_head_stride, _code(inp, "head_linear in"), n,
                  num_heads, n_in, n_out, _stream()), "head_linear")

    def latent_attention(self, q_cat: torch.Tensor, cache_rows: torch.Tensor, out: torch.Tensor, sink: Optional[torch.Tensor],
                         meta, *, num_heads: int, rank: int, scale: float, window: Optional[int]) -> None:
        """``q_cat`` [N, H, width], ``cache_rows`` [pages, page_size, width] -> ``out`` [N, H, rank]: softmax (with the
        sink in the denominator) over the visible cached rows, weighted sum of their first ``rank`` columns."""
        n, h, width = q_cat.shape
        if h != num_heads or cache_rows.shape[-1] != width or out.shape != (n, h, rank) or cache_rows.dtype != q_cat.dtype \
                or out.dtype != q_cat.dtype:
            raise KernelError(f"latent_attention: q {tuple(q_cat.shape)}, cache {tuple(cache_rows.shape)}, out {tuple(out.shape)} do not fit")
        bt = meta.block_table
        fn = _fn("latent_attention", "iian_latent_attention",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
        _check(fn(_cuda(q_cat, "q_cat"), _cuda(cache_rows, "latent cache"), _cuda(out, "attention out"),
                  _cuda(sink, "sink", torch.float32), _cuda(meta.positions, "positions", torch.int32),
                  _cuda(meta.seq_of_token, "seq_of_token", torch.int32), _cuda(bt, "block table", torch.int32), bt.shape[1],
                  _cuda(meta.ctx_len, "ctx_len", torch.int32), _code(q_cat, "q_cat"), n, h, rank, width, cache_rows.shape[1],
                  cache_rows.shape[0], scale, window or 0, _stream()), "latent_attention")

    # the same on the tensor cores (csrc/latent_attention_mma.cu): bfloat16, rank 64 / 128 / 256 / 512, rot a multiple of 16
    LATENT_MMA = os.environ.get("IIAN_LATENT_MMA", "1") not in ("0", "false", "off")
    # the form for prompts' portions: 1 = tiles of 32 keys in one stage, two CTAs an SM; 0 = tiles of 64 keys in two stages
    LATENT_LARGE_FORM = int(os.environ.get("IIAN_LATENT_LARGE_FORM", "1"))
    # the form for decoded tokens: 0 = two stages, two CTAs an SM; 1 = one stage, three CTAs an SM
    LATENT_SMALL_FORM = int(os.environ.get("IIAN_LATENT_SMALL_FORM", "0"))
    _latent_form_set = None

    def latent_attention_mma_ok(self, q_cat: torch.Tensor, cache_rows: torch.Tensor, rank: int) -> bool:
        if not self.LATENT_MMA or q_cat.dtype != torch.bfloat16 or cache_rows.dtype != torch.bfloat16:
            return False
        fn = _fn("latent_attention_mma", "iian_latent_attention_mma_ok", [c_int, c_int, c_int])
        return fn(rank, q_cat.shape[2], q_cat.shape[1]) == 0

    def latent_attention_parts(self, num_seqs: int, max_q_len: int, num_heads: int, max_ctx: int, window: Optional[int]) -> int:
        """Into how many parts the keys are cut so that a step with few rows still fills the GPU.  Decoded tokens run in
        the kernel's small form (16 rows a CTA, tiles of 32 keys), portions of prompts in the large one (32 rows); of
        either, two CTAs share an SM at the widths of real models; a part keeps at least four tiles."""
        small = max_q_len == 1 or max_q_len * num_heads <= 16
        rows, tile, per_sm, least = (16, 32, 3 if self.LATENT_SMALL_FORM else 2, 4) if small else (32, 32 if self.LATENT_LARGE_FORM else 64, 2 if self.LATENT_LARGE_FORM else 1, 4)
        ctas = max(1, num_seqs * (-(-max_q_len * num_heads // rows)))
        keys = min(max_ctx, window + max_q_len) if window else max_ctx
        tiles = -(-keys // tile) + 1
        return max(1, min(per_sm * self.sm_count() // ctas, tiles // least, 32))

    def latent_attention_mma(self, q_cat: torch.Tensor, cache_rows: torch.Tensor, out: torch.Tensor, sink: Optional[torch.Tensor],
                             meta, *, num_heads: int, rank: int, scale: float, window: Optional[int],
                             parts: Optional[int] = None) -> None:
        n, h, width = q_cat.shape
        if h != num_heads or cache_rows.shape[-1] != width or out.shape != (n, h, rank) or out.dtype != torch.bfloat16:
            raise KernelError(f"latent_attention_mma: q {tuple(q_cat.shape)}, cache {tuple(cache_rows.shape)}, out {tuple(out.shape)} do not fit")
        if parts is None:
            parts = self.latent_attention_parts(meta.num_seqs, meta.max_q_len, h, meta.max_ctx, window)
        if CudaKernels._latent_form_set != (self.LATENT_LARGE_FORM, self.LATENT_SMALL_FORM):
            if _fn("latent_attention_mma", "iian_latent_attention_large_form", [c_int])(self.LATENT_LARGE_FORM) != 0 \
                    or _fn("latent_attention_mma", "iian_latent_attention_small_form", [c_int])(self.LATENT_SMALL_FORM) != 0:
                raise KernelError("IIAN_LATENT_LARGE_FORM and IIAN_LATENT_SMALL_FORM take 0 or 1")
            CudaKernels._latent_form_set = (self.LATENT_LARGE_FORM, self.LATENT_SMALL_FORM)
        part_o = part_ml = 0
        if parts > 1:
            scratch = self.attention_scratch(q_cat.device, n * h * parts * (rank + 2))
            part_o = scratch.data_ptr()
            part_ml = part_o + n * h * parts * rank * 4
        bt = meta.block_table
        fn = _fn("latent_attention_mma", "iian_latent_attention_mma",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
        _check(fn(_cuda(q_cat, "q_cat"), _cuda(cache_rows, "latent cache"), _cuda(out, "attention out"), part_o, part_ml,
                  _cuda(sink, "sink", torch.float32), _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(meta.seq_of_token, "seq_of_token", torch.int32), _cuda(bt, "block table", torch.int32), bt.shape[1],
                  n, meta.num_seqs, meta.max_q_len, h, rank, width, cache_rows.shape[1], cache_rows.shape[0], scale, window or 0,
                  parts, _stream()), "latent_attention_mma")
        if parts > 1:
            LAUNCHES[0] += 1

    # ---- routed experts (csrc/moe.cu) -----------------------------------------------------------------------------
    _moe_tile_rows = None

    def moe_tile_rows(self) -> int:
        if CudaKernels._moe_tile_rows is None:
            lib = _build.load("moe")
            lib.iian_moe_tile_rows.restype = c_int
            CudaKernels._moe_tile_rows = int(lib.iian_moe_tile_rows())
        return CudaKernels._moe_tile_rows

    def moe_max_tiles(self, n_rows: int, num_experts: int, tile_rows: Optional[int] = None) -> int:
        """Upper bound of the row tiles of a grouped product over ``n_rows`` rows sorted by expert."""
        return -(-n_rows // (tile_rows or self.moe_tile_rows())) + num_experts

    # grouped products on tcgen05 (csrc/gemm_tcgen05.cu, row tiles of 128); IIAN_MOE_TCGEN05=0: the general kernel
    MOE_TCGEN05 = os.environ.get("IIAN_MOE_TCGEN05", "1") not in ("0", "false", "off")
    MOE_TC_TILE_ROWS = 128

    def moe_tcgen05_ok(self, dtype: torch.dtype, hidden: int, inter: int, activation: str) -> bool:
        """Whether both grouped products of an expert feed-forward can run on the tcgen05 kernel: bfloat16, rows of 16
        bytes' multiples for TMA, gate and up interleaved in groups of 8 (SiLU rides in the product's epilogue; the clamped
        activation is a pass of its own between the two products)."""
        return (self.MOE_TCGEN05 and not self.LIBRARY_GEMM_ONLY and dtype == torch.bfloat16
                and activation in ("silu", "clamped_swish") and hidden % 8 == 0 and inter % 8 == 0)

    def moe_grouped_gemm_tc(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, tiles: torch.Tensor,
                            gated: bool) -> None:
        """Rows of ``x`` sorted by expert times that expert's block of ``w`` [E, n, K] on tcgen05; ``gated``: the block's
        rows are gate and up interleaved in groups of 8 and ``out`` [M, n / 2] = silu(gate) * up.  The plan's row tiles
        are of 128 rows."""
        m, k = x.shape
        e, n = w.shape[0], w.shape[1]
        if w.shape[2] != k or out.shape != (m, n // 2 if gated else n) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 \
                or out.dtype != torch.bfloat16:
            raise KernelError(f"moe_grouped_gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        bn = 256 if n % 256 == 0 or n > 2048 else 128
        status = self.tcgen05_status_buffer(x.device).data_ptr()
        CudaKernels._tc_used = True
        fn = _fn("gemm_tcgen05", "iian_gemm_tcgen05_grouped",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                  c_void_p])
        _check(fn(_cuda(x, "moe rows"), _cuda(w, "expert weights"), _cuda(out, "moe out"), BF16, m, n, e, k, 1 if gated else 0, bn,
                  status, _cuda(tiles, "tiles", torch.int32), _cuda(offsets, "offsets", torch.int32), (tiles.numel() - 1) // 2,
                  _stream()), "gemm_tcgen05_grouped")

    def moe_route(self, logits: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor) -> None:
        """Router logits (float32, may be a column slice) -> the ``top`` experts of each token by sigmoid score, and the scores."""
        n, e = logits.shape
        if logits.dtype != torch.float32 or ids.shape != (n, top) or weights.shape != (n, top):
            raise KernelError("moe_route: logits float32 [N, E]; ids / weights [N, top]")
        lp, ld = self._rows(logits, "router logits")
        fn = _fn("moe", "iian_moe_route", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
        _check(fn(lp, ld, e, top, _cuda(ids, "expert ids", torch.int32), _cuda(weights, "expert weights", torch.float32), n,
                  _stream()), "moe_route")

    def moe_plan(self, ids: torch.Tensor, num_experts: int, offsets: torch.Tensor, pos: torch.Tensor, tiles: torch.Tensor,
                 tile_rows: Optional[int] = None) -> None:
        m = ids.numel()
        max_tiles = (tiles.numel() - 1) // 2
        if offsets.numel() != num_experts + 1 or pos.numel() != m:
            raise KernelError("moe_plan: offsets [E + 1], pos [M]")
        fn = _fn("moe", "iian_moe_plan", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
        _check(fn(_cuda(ids, "expert ids", torch.int32), m, num_experts, _cuda(offsets, "offsets", torch.int32),
                  _cuda(pos, "pos", torch.int32), _cuda(tiles, "tiles", torch.int32), max_tiles,
                  tile_rows or self.moe_tile_rows(), _stream()), "moe_plan")

    def moe_scatter(self, h: torch.Tensor, pos: torch.Tensor, weights: Optional[torch.Tensor], xs: torch.Tensor, top: int) -> None:
        """Rows of ``h`` to their places among the rows sorted by expert, times ``weights`` (None: as they are)."""
        n, w = h.shape
        if xs.shape != (n * top, w) or xs.dtype != h.dtype:
            raise KernelError("moe_scatter: xs must be [N * top, W] in the dtype of h")
        fn = _fn("moe", "iian_moe_scatter", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(h, "moe in"), _cuda(pos, "pos", torch.int32), _cuda(weights, "expert weights", torch.float32),
                  _cuda(xs, "moe rows"), _code(h, "moe in"), n, w, top, _stream()), "moe_scatter")

    def moe_grouped_gemm(self, x: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor], out: torch.Tensor,
                         offsets: torch.Tensor, tiles: torch.Tensor, activation: str = "silu", limit: float = 0.0) -> None:
        """Rows of ``x`` sorted by expert times that expert's block of ``w`` [E, n_out, K]; with ``w2`` the gated form
        ``act(x . w) * (x . w2)``; with ``w2 is w`` the blocks are [E, 2 n_out, K] and hold both matrices interleaved in
        groups of 8 rows."""
        m, k = x.shape
        n_out = w.shape[1] // 2 if w2 is w else w.shape[1]
        if w.shape[2] != k or out.shape != (m, n_out) or (w2 is not None and w2.shape != w.shape) or out.dtype != x.dtype:
            raise KernelError(f"moe_grouped_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        fn = _fn("moe", "iian_moe_grouped_gemm_act", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(x, "moe rows"), _cuda(w, "expert weights"), _cuda(w2, "expert weights"), _cuda(out, "moe out"),
                  _cuda(offsets, "offsets", torch.int32), _cuda(tiles, "tiles", torch.int32), (tiles.numel() - 1) // 2,
                  _code(x, "moe rows"), _code(w, "expert weights"), n_out, k, self.ACTIVATIONS[activation], limit, _stream()),
               "moe_grouped_gemm")

    def moe_combine(self, ys: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, top: int,
                    weights: Optional[torch.Tensor] = None) -> None:
        """``out[t] = sum_k weights[t, k] * ys[pos[t, k]]`` (``weights`` None: the plain sum), k ascending, in float32."""
        n, w = out.shape
        if ys.shape != (n * top, w) or ys.dtype != out.dtype or (weights is not None and weights.numel() != n * top):
            raise KernelError("moe_combine: ys must be [N * top, W] in the dtype of out")
        fn = _fn("moe", "iian_moe_combine_weighted", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(ys, "moe out rows"), _cuda(pos, "pos", torch.int32), _cuda(weights, "expert weights", torch.float32),
                  _cuda(out, "moe out"), _code(out, "moe out"), n, w, top, _stream()), "moe_combine")

    # ---- a scaled embedding, a second sub-layer output in the norm's sum (csrc/elementwise.cu) -----------------------
    def embedding_scaled(self, table: torch.Tensor, tokens: torch.Tensor, scale: float, out: torch.Tensor) -> None:
        n, h = out.shape
        fn = _fn("elementwise", "iian_embedding_scaled", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(table, "embedding table"), _code(table, "embedding table"), _cuda(tokens, "tokens", torch.int32),
                  _cuda(out, "embedding out", torch.float32), n, h, table.shape[0], scale, _stream()), "embedding_scaled")

    def add2_rms_norm(self, residual: torch.Tensor, delta: torch.Tensor, delta2: torch.Tensor, weight: torch.Tensor, eps: float,
                      out: torch.Tensor) -> None:
        """``residual += delta + delta2`` (the two summed first, all in float32), then ``out = rmsnorm(residual) * weight``."""
        n, h = residual.shape
        for d in (delta, delta2):
            if d.shape != residual.shape or d.dtype != out.dtype:
                raise KernelError("add2_rms_norm: a delta does not match the residual's shape or the output's dtype")
        if out.shape != residual.shape or weight.numel() != h:
            raise KernelError("add2_rms_norm: shapes of out / weight do not match the residual")
        fn = _fn("elementwise", "iian_add2_rms_norm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(delta, "delta"), _cuda(delta2, "delta"),
                  _cuda(weight, "norm weight", torch.float32), _cuda(out, "norm out"), _code(out, "norm out"), n, h, eps, _stream()),
               "add2_rms_norm")

    # ---- gates and the re-injected embedding (csrc/stream_ops.cu) --------------------------------------------------------
    def stream_concat(self, x: torch.Tensor, d1: Optional[torch.Tensor], d2: Optional[torch.Tensor], e: torch.Tensor,
                      out: torch.Tensor) -> None:
        """``out[t] = [x_t + (d1_t + d2_t) ; e_t]`` in the dtype of ``out``; ``x``, ``e`` float32 [N, H], ``out`` [N, 2H]."""
        n, h = x.shape
        if e.shape != x.shape or out.shape != (n, 2 * h) or any(d is not None and (d.shape != x.shape or d.dtype != out.dtype) for d in (d1, d2)):
            raise KernelError("stream_concat: shapes or dtypes do not fit")
        if d1 is None:
            d1, d2 = d2, None
        fn = _fn("stream_ops", "iian_stream_concat", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "stream", torch.float32), _cuda(d1, "delta"), _cuda(d2, "delta"), _cuda(e, "embedding out", torch.float32),
                  _cuda(out, "concat out"), _code(out, "concat out"), n, h, _stream()), "stream_concat")

    def sigmoid_mul(self, x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
        """``out = x * sigmoid(gate)`` element by element; ``gate`` may be a column slice."""
        n, m = x.shape
        if gate.shape != (n, m) or out.shape != (n, m) or gate.dtype != x.dtype or out.dtype != x.dtype:
            raise KernelError("sigmoid_mul: x, gate and out must share shape and dtype")
        gp, ld = self._rows(gate, "gate")
        fn = _fn("stream_ops", "iian_sigmoid_mul", [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "gated x"), gp, ld, _cuda(out, "gated out"), _code(x, "gated x"), n, m, _stream()), "sigmoid_mul")

    def head_norm_gate(self, x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *,
                       num_heads: int, eps: float) -> None:
        """``out[t, h] = x[t, h] / sqrt(mean(x[t, h]^2) + eps) * weight[h] * sigmoid(gate[t, h])``: every head by its own root
        mean square.  ``x`` float32 [N, heads * dv]; ``gate`` (optional, may be a column slice) and ``out`` in one dtype."""
        n, m = x.shape
        if m % num_heads or weight.numel() != m or out.shape != (n, m) or (gate is not None and (gate.shape != (n, m) or gate.dtype != out.dtype)):
            raise KernelError("head_norm_gate: shapes or dtypes do not fit")
        gp, ld = self._rows(gate, "gate")
        fn = _fn("stream_ops", "iian_head_norm_gate", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int,
                                                       c_float, c_void_p])
        _check(fn(_cuda(x, "heads", torch.float32), _cuda(weight, "head norm weight", torch.float32), gp, ld, _cuda(out, "head norm out"),
                  _code(out, "head norm out"), n, num_heads, m // num_heads, eps, _stream()), "head_norm_gate")

    # ---- attention whose values are its keys (csrc/shared_kv.cu), sink and output gate (csrc/attention_generic.cu) ----------
    def projection_norm_rope_store(self, proj: torch.Tensor, q_off: int, k_off: int, q_out: torch.Tensor,
                                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *, num_heads: int,
                                   num_kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                                   eps: float, inv_freq: Optional[torch.Tensor], rot_dim: int, rope_style: int, positions: torch.Tensor,
                                   slots: Optional[torch.Tensor]) -> None:
        """From rows of a stacked product (q at column ``q_off``, k at ``k_off``): RMS norm of q and of k over the whole
        projection, rotation, q into ``q_out`` [N, heads, head_dim], the rotated k into ``k_cache`` and the k as projected into
        ``v_cache`` at the tokens' cells (``slots``; without caches nothing is stored)."""
        n = proj.shape[0]
        pp, ld = self._rows(proj, "projections")
        if q_off + num_heads * head_dim > proj.shape[1] or k_off + num_kv_heads * head_dim > proj.shape[1] \
                or q_out.numel() != n * num_heads * head_dim or q_out.dtype != proj.dtype:
            raise KernelError("projection_norm_rope_store: the projections do not hold these heads")
        page_size, num_pages = 1, 0
        if k_cache is not None:
            if v_cache is None or slots is None or k_cache.dtype != proj.dtype or k_cache.shape != v_cache.shape \
                    or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
                raise KernelError("projection_norm_rope_store: the caches do not match")
            num_pages, page_size = k_cache.shape[0], k_cache.shape[2]
        if rot_dim and (inv_freq is None or inv_freq.dtype != torch.float64 or inv_freq.numel() < rot_dim // 2):
            raise KernelError("projection_norm_rope_store: inv_freq must be float64 [rot_dim / 2]")
        fn = _fn("shared_kv", "iian_projection_norm_rope_store",
                 [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p])
        _check(fn(pp, ld, q_off, k_off, _cuda(q_out, "q out"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"),
                  _cuda(q_weight, "q norm weight", torch.float32), _cuda(k_weight, "k norm weight", torch.float32),
                  _cuda(inv_freq, "inv_freq") if rot_dim else 0, _cuda(positions, "positions", torch.int32),
                  _cuda(slots, "slots", torch.int32) if k_cache is not None else 0, _code(proj, "projections"), n, num_heads,
                  num_kv_heads, head_dim, rot_dim, rope_style, eps, page_size, num_pages, _stream()), "projection_norm_rope_store")

    def paged_attention_sink(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                             sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
        """Paged attention (any sizes, either dtype) whose softmax denominator also holds ``exp(sink[h])`` and whose output is
        multiplied by ``sigmoid(gate)`` (``gate`` [N, heads * head_dim], may be a column slice); both optional."""
        n = q.shape[0]
        if k_cache.dtype != q.dtype or out.dtype != q.dtype or k_cache.shape != v_cache.shape:
            raise KernelError("paged_attention_sink: q, caches and out must share one dtype and the caches one shape")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError("paged_attention_sink: cache / q shapes do not match the head counts")
        if gate is not None and (gate.shape != (n, num_heads * head_dim) or gate.dtype != q.dtype):
            raise KernelError("paged_attention_sink: gate must be [N, heads * head_dim] in the dtype of q")
        if sink is not None and sink.numel() != num_heads:
            raise KernelError("paged_attention_sink: one sink per head")
        gp, ld = self._rows(gate, "gate")
        bt = meta.block_table
        fn = _fn("attention_generic", "iian_paged_attention_sink",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_void_p])
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  _cuda(meta.positions, "positions", torch.int32), _cuda(meta.seq_of_token, "seq_of_token", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _code(q, "q"), n, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
                  scale, window or 0, _cuda(sink, "sink", torch.float32), gp, ld, _stream()), "paged_attention_sink")

    def sink_attention(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window, sink=None,
                       gate=None, plan=None) -> None:
        """Attention with an optional sink and output gate, served by whichever kernel takes these sizes: in bfloat16
        with heads of 64 or 128 the tensor-core kernels (``csrc/attention_tc.cu`` for portions of prompts with heads of 128,
        ``csrc/attention_mma.cu`` otherwise; the gate is then a pass of its own), else
        the general kernel with the gate in its epilogue.  ``plan``: what ``sink_attention_plan`` answered for a captured graph."""
        if self.SINK_ATTENTION_MMA and scale > 0 and self._attention_tc_ok(q, k_cache, meta, num_heads, num_kv_heads, head_dim):
            self.paged_attention_tc(q, k_cache, v_cache, out, meta, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                                    scale=scale, window=window, sink=sink)          # portions of prompts, heads of 128: tcgen05
            if gate is not None:
                self.sigmoid_mul(out, gate, out)
            return
        if self.SINK_ATTENTION_MMA and q.dtype == torch.bfloat16 and head_dim in (64, 128) and scale > 0 and num_heads // num_kv_heads <= 16:
            n_split = plan["n_split"] if plan else None
            if n_split is None and meta.max_q_len * (num_heads // num_kv_heads) <= 16:
                n_split = self.attention_splits(meta.num_seqs, num_kv_heads, min(meta.max_ctx, window) if window else meta.max_ctx)
            self.paged_attention_mma(q, k_cache, v_cache, out, meta, num_heads=num_heads, num_kv_heads=num_kv_heads,
                                     head_dim=head_dim, scale=scale, window=window, n_split=n_split, sink=sink)
            if gate is not None:
                self.sigmoid_mul(out, gate, out)
            return
        self.paged_attention_sink(q, k_cache, v_cache, out, meta, num_heads=num_heads, num_kv_heads=num_kv_heads,
                                  head_dim=head_dim, scale=scale, window=window, sink=sink, gate=gate)

    SINK_ATTENTION_MMA = os.environ.get("IIAN_SINK_ATTENTION_MMA", "1") not in ("0", "false", "off")

    def sink_attention_plan(self, num_seqs: int, num_heads: int, num_kv_heads: int, head_dim: int, max_ctx: int,
                            window: Optional[int], dtype: torch.dtype):
        """The number of key parts of the decode form is part of a captured graph (grid and cluster sizes)."""
        if dtype != torch.bfloat16 or head_dim not in (64, 128) or not self.SINK_ATTENTION_MMA:
            return None
        return {"n_split": self.attention_splits(num_seqs, num_kv_heads, min(max_ctx, window) if window else max_ctx)}

    # ---- the matrix-memory recurrence (csrc/matrix_memory.cu) ------------------------------------------------------------------
    def matrix_memory_scan(self, proj: torch.Tensor, q_off: int, k_off: int, v_off: int, gates: torch.Tensor, gate_bias: torch.Tensor,
                           state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                           dim: int, v_dim: int, columns: int, cap: float, q_scale: float, max_q_len: int = 0) -> None:
        """Walk every sequence's tokens of this step through the recurrence, from and into ``state`` [slots, heads,
        v_dim / columns, block floats] (float32).  ``proj`` rows hold q, k, v at the given column offsets; ``gates`` float32
        [N, 2 heads] the input- and forget-gate pre-activations, ``gate_bias`` [2 heads]; ``out`` float32 [N, heads * v_dim].
        ``max_q_len``: the most tokens a sequence brings (a hint: 1 picks the kernel's form for single tokens; 0: unknown)."""
        n = proj.shape[0]
        pp, ld = self._rows(proj, "projections")
        s = cu_q.numel() - 1
        if gates.shape != (n, 2 * num_heads) or gate_bias.numel() != 2 * num_heads or out.shape != (n, num_heads * v_dim) \
                or state_slots.numel() != s or v_dim % columns:
            raise KernelError("matrix_memory_scan: shapes do not fit")
        if state.dim() != 4 or state.shape[1:] != (num_heads, v_dim // columns, self.matrix_memory_block_floats(dim, columns)):
            raise KernelError(f"matrix_memory_scan: state {tuple(state.shape)} does not match {num_heads} heads of {dim} x {v_dim}")
        fn = _fn("matrix_memory", "iian_matrix_memory_scan",
                 [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
        _check(fn(pp, ld, q_off, k_off, v_off, _cuda(gates, "gates", torch.float32), _cuda(gate_bias, "gate bias", torch.float32),
                  _cuda(state, "state", torch.float32), _cuda(cu_q, "cu_q", torch.int32), _cuda(state_slots, "state slots", torch.int32),
                  _cuda(out, "memory out", torch.float32), _code(proj, "projections"), s, num_heads, dim, v_dim, columns, cap,
                  q_scale, max_q_len, _stream()), "matrix_memory_scan")

    @staticmethod
    def matrix_memory_lanes(dim: int) -> int:
        """Lanes that share one column of the memory in the scan kernel (csrc/matrix_memory.cu: iian_matrix_memory_lanes)."""
        return 8 if dim <= 128 else 16 if dim <= 256 else 32

    @staticmethod
    def matrix_memory_block_floats(dim: int, columns: int) -> int:
        """Floats of one column block of the state: the block's columns, a copy of the normaliser, the running maximum,
        padded to a multiple of 4 (csrc/matrix_memory.cu: iian_matrix_memory_block_floats)."""
        return ((columns + 1) * dim + 1 + 3) // 4 * 4

    # ---- scaled residual sums, a normalised addend, xIELU, a token-indexed factor, the logit cap (csrc/residual_ops.cu) ----
    def scaled_add_rms_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], mult: float, weight: Optional[torch.Tensor],
                            eps: float, out: Optional[torch.Tensor], copy: Optional[torch.Tensor] = None) -> None:
        """``residual += mult * delta`` (float32, in place; nothing without ``delta``); ``out`` (optional) receives
        ``residual / sqrt(mean(residual^2) + eps) * weight``; ``copy`` (optional) the new stream in the activation dtype."""
        n, h = residual.shape
        act = out if out is not None else copy if copy is not None else delta
        if act is None:
            return
        for name, t in (("delta", delta), ("out", out), ("copy", copy)):
            if t is not None and (t.shape != residual.shape or t.dtype != act.dtype):
                raise KernelError(f"scaled_add_rms_norm: {name} {tuple(t.shape)} {t.dtype} does not match the stream {tuple(residual.shape)}")
        if out is not None and (weight is None or weight.numel() != h):
            raise KernelError("scaled_add_rms_norm: the norm's weight does not match the stream")
        fn = _fn("residual_ops", "iian_scaled_add_rms_norm",
                 [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(delta, "delta"), mult, _cuda(weight, "norm weight", torch.float32),
                  _cuda(out, "norm out"), _cuda(copy, "stream copy"), _code(act, "norm out"), n, h, eps, _stream()), "scaled_add_rms_norm")

    def scaled_add_unit_rms(self, residual: torch.Tensor, y: torch.Tensor, mult: float, weight: torch.Tensor, eps: float) -> None:
        """``residual += mult * y / sqrt(mean(y^2) + eps) * weight`` (float32, in place)."""
        n, h = residual.shape
        if y.shape != (n, h) or weight.numel() != h:
            raise KernelError("scaled_add_unit_rms: shapes do not fit")
        fn = _fn("residual_ops", "iian_scaled_add_unit_rms", [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(y, "addend"), mult, _cuda(weight, "norm weight", torch.float32),
                  _code(y, "addend"), n, h, eps, _stream()), "scaled_add_unit_rms")

    def rms_norm_rows(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """``out = x / sqrt(mean(x^2) + eps) * weight`` where ``x`` may be a column slice of a wider matrix."""
        n, h = x.shape
        xp, ld = self._rows(x, "rms_norm_rows in")
        if out.shape != (n, h) or out.dtype != x.dtype or weight.numel() != h:
            raise KernelError("rms_norm_rows: out / weight do not match the input")
        fn = _fn("residual_ops", "iian_rms_norm_rows", [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(xp, ld, _cuda(weight, "norm weight", torch.float32), _cuda(out, "rms_norm_rows out"), _code(x, "rms_norm_rows in"),
                  n, h, eps, _stream()), "rms_norm_rows")

    def gelu_mul_table(self, g: torch.Tensor, table: torch.Tensor, col_off: int, tokens: torch.Tensor, rows: Optional[torch.Tensor],
                       out: torch.Tensor) -> None:
        """``out[r] = gelu_tanh(g[r]) * table[token(r), col_off : col_off + n]``, ``token(r) = tokens[rows[r]]`` (``tokens[r]``
        without ``rows``)."""
        r, n = g.shape
        if out.shape != (r, n) or out.dtype != g.dtype or table.dim() != 2 or col_off < 0 or col_off + n > table.shape[1] \
                or (rows is not None and rows.numel() != r) or (rows is None and tokens.numel() < r):
            raise KernelError("gelu_mul_table: shapes do not fit")
        fn = _fn("residual_ops", "iian_gelu_mul_table",
                 [c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(g, "gate"), _cuda(table, "table"), _code(table, "table"), table.shape[1], col_off, _cuda(tokens, "tokens", torch.int32),
                  _cuda(rows, "rows", torch.int32), _cuda(out, "gated out"), _code(g, "gate"), r, n, table.shape[0], _stream()),
               "gelu_mul_table")

    def xielu(self, x: torch.Tensor, pq: torch.Tensor, out: torch.Tensor) -> None:
        """``z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` with ``pq`` = float32 [p, q]."""
        if out.shape != x.shape or out.dtype != x.dtype or pq.numel() != 2:
            raise KernelError("xielu: shapes or dtypes do not fit")
        fn = _fn("residual_ops", "iian_xielu", [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p])
        _check(fn(_cuda(x, "xielu in"), _cuda(pq, "xielu numbers", torch.float32), _cuda(out, "xielu out"), _code(x, "xielu in"),
                  x.numel(), _stream()), "xielu")

    def tanh_cap(self, x: torch.Tensor, cap: float) -> None:
        """``x <- cap * tanh(x / cap)`` in place (float32)."""
        fn = _fn("residual_ops", "iian_tanh_cap", [c_void_p, c_float, c_longlong, c_void_p])
        _check(fn(_cuda(x, "capped values", torch.float32), cap, x.numel(), _stream()), "tanh_cap")

    # ---- attention inside chunks of positions with a penalty on distance (csrc/chunked_attention.cu) -----------------------
    def kv_store_normed(self, proj: torch.Tensor, k_off: int, v_off: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        slots: torch.Tensor, *, num_kv_heads: int, k_dim: int, v_dim: int, eps: float, norm_values: bool) -> None:
        """Per token: the keys at column ``k_off`` of ``proj`` as they are, the values at ``v_off`` divided by their root mean
        square per head (if ``norm_values``), into the token's cells of ``k_cache`` [pages, kv_heads, page_size, k_dim] and
        ``v_cache`` [.., v_dim]."""
        n = proj.shape[0]
        pp, ld = self._rows(proj, "projections")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != k_dim or v_cache.shape[3] != v_dim or k_cache.shape[:3] != v_cache.shape[:3] \
                or k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype or slots.numel() != n:
            raise KernelError(f"kv_store_normed: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit")
        fn = _fn("chunked_attention", "iian_kv_store_normed",
                 [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong,
                  c_float, c_int, c_void_p])
        _check(fn(pp, ld, k_off, v_off, _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"), _cuda(slots, "slots", torch.int32),
                  _code(proj, "projections"), n, num_kv_heads, k_dim, v_dim, k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2], eps,
                  1 if norm_values else 0, _stream()), "kv_store_normed")

    def chunked_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor, meta, *,
                          num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float, chunk: Optional[int],
                          window: Optional[int], r1: Optional[torch.Tensor], r2: Optional[torch.Tensor],
                          gate: Optional[torch.Tensor], n_split: Optional[int] = None) -> None:
        """``q`` rows of ``heads * k_dim`` (may be a column slice) -> ``out`` [N, heads * v_dim]: softmax of
        ``q . k * scale - r1 ln(1 + r2 (i - j))`` over the keys ``j <= i`` of position ``i``'s chunk (or window), weighted sum
        of the cached values, times ``sigmoid(gate)`` if given (rows of ``heads * v_dim``, may be a column slice).
        In bfloat16 with keys and values of 64 or 128 entries and a positive scale the tensor-core kernels of
        ``csrc/attention_mma.cu`` serve it (mask, penalty and gate inside them); otherwise the general kernel of
        ``csrc/chunked_attention.cu``.  ``n_split``: the key parts of the decode form that a captured graph fixed."""
        n = q.shape[0]
        qp, ld_q = self._rows(q, "queries")
        gp, ld_g = self._rows(gate, "gate")
        if q.shape[1] != num_heads * k_dim or out.shape != (n, num_heads * v_dim) or out.dtype != q.dtype or k_cache.dtype != q.dtype \
                or (gate is not None and (gate.shape != out.shape or gate.dtype != q.dtype)) or (r1 is None) != (r2 is None):
            raise KernelError(f"chunked_attention: q {tuple(q.shape)}, out {tuple(out.shape)} do not fit")
        if self.chunked_attention_mma_ok(q.dtype, num_heads, num_kv_heads, k_dim, v_dim, scale) and ld_q % 8 == 0 \
                and qp % 16 == 0 and (gate is None or (ld_g % 2 == 0 and gp % 4 == 0)):
            self._chunked_attention_mma(qp, ld_q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, k_dim, scale, chunk, window,
                                        r1, r2, gp, ld_g, n, n_split)
            return
        bt = meta.block_table
        fn = _fn("chunked_attention", "iian_chunked_attention",
                 [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p])
        _check(fn(qp, ld_q, _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"), _cuda(out, "attention out"),
                  _cuda(meta.positions, "positions", torch.int32), _cuda(meta.seq_of_token, "seq_of_token", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], _cuda(meta.ctx_len, "ctx_len", torch.int32), _code(q, "queries"),
                  n, num_heads, num_kv_heads, k_dim, v_dim, k_cache.shape[2], k_cache.shape[0], scale, chunk or 0, window or 0,
                  _cuda(r1, "r1", torch.float32), _cuda(r2, "r2", torch.float32), gp, ld_g, _stream()), "chunked_attention")

    CHUNKED_ATTENTION_MMA = os.environ.get("IIAN_CHUNKED_ATTENTION_MMA", "1") not in ("0", "false", "off")

    def chunked_attention_mma_ok(self, dtype, num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float) -> bool:
        return (self.CHUNKED_ATTENTION_MMA and dtype == torch.bfloat16 and k_dim == v_dim and k_dim in (64, 128) and scale > 0
                and num_kv_heads > 0 and num_heads % num_kv_heads == 0)

    def chunked_attention_plan(self, num_seqs: int, num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float,
                               max_ctx: int, chunk: Optional[int], window: Optional[int], dtype: torch.dtype):
        """The number of key parts of the decode form is part of a captured graph (grid and cluster sizes)."""
        if not self.chunked_attention_mma_ok(dtype, num_heads, num_kv_heads, k_dim, v_dim, scale):
            return None
        return {"n_split": self.attention_splits(num_seqs, num_kv_heads, min(max_ctx, chunk or window or max_ctx))}

    def _chunked_attention_mma(self, qp, ld_q, k_cache, v_cache, out, meta, nh, nkv, hd, scale, chunk, window, r1, r2, gp, ld_g,
                               n, n_split, sink=None, keep_first: int = 0, gate_per_head: bool = False) -> None:
        if k_cache.shape[1] != nkv or k_cache.shape[3] != hd or v_cache.shape != k_cache.shape:
            raise KernelError("chunked_attention: cache shapes do not match the head counts")
        bt = meta.block_table
        if self.ATTENTION_TC and hd == 128 and k_cache.shape[2] in (8, 16, 32, 64, 128) and ld_q % 8 == 0 \
                and meta.max_q_len * (nh // nkv) >= self.TC_ATTENTION_MIN_ROWS and (gate_per_head or (gp % 16 == 0 and ld_g % 8 == 0)) \
                and out.data_ptr() % 16 == 0:
            # portions of prompts with heads of 128: tcgen05 (csrc/attention_tc.cu)
            status = self.tcgen05_status_buffer(out.device)
            CudaKernels._tc_used = True
            fn = _fn("attention_tc", "iian_attention_tc_kept",
                     [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_longlong, c_int, c_int, c_void_p])
            _check(fn(qp, ld_q, _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"), _cuda(out, "attention out"),
                      _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                      _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, nh, nkv, hd,
                      k_cache.shape[2], k_cache.shape[0], scale, window or 0, chunk or 0, status.data_ptr(),
                      _cuda(sink, "sink", torch.float32), _cuda(r1, "r1", torch.float32), _cuda(r2, "r2", torch.float32), gp, ld_g,
                      keep_first, 1 if gate_per_head else 0, _stream()), "chunked attention (tcgen05)")
            return
        if self._stages_set != self.DECODE_STAGES:
            self.set_decode_stages(self.DECODE_STAGES)
        small = meta.max_q_len * (nh // nkv) <= 16
        if not small:
            n_split = 1
        elif n_split is None:
            n_split = self.attention_splits(meta.num_seqs, nkv, min(meta.max_ctx, (chunk or window or meta.max_ctx) + keep_first))
        cluster = bool(self.CLUSTER_MERGE and small and n_split in (2, 4, 8, 16))
        part_o = part_lse = counters = 0
        if n_split > 1 and not cluster:
            rows = n * nh
            scratch = self.attention_scratch(out.device, rows * n_split * (hd + 1))
            part_o = scratch.data_ptr()
            part_lse = part_o + rows * n_split * hd * 4
            row_tiles = -(-meta.max_q_len * (nh // nkv) // 16)
            counters = self.attention_counters(out.device, meta.num_seqs * nkv * row_tiles).data_ptr()
        fn = _fn("attention_mma", "iian_attention_mma_kept",
                 [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p])
        _check(fn(qp, ld_q, _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"), _cuda(out, "attention out"),
                  part_o, part_lse, counters, _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, nh, nkv, hd,
                  k_cache.shape[2], k_cache.shape[0], scale, window or 0, chunk or 0, n_split,
                  (2 if cluster else 1) if small else 0, self._decode_status(out.device) if small else None,
                  _cuda(sink, "sink", torch.float32), _cuda(r1, "r1", torch.float32), _cuda(r2, "r2", torch.float32), gp, ld_g,
                  keep_first, 1 if gate_per_head else 0, _stream()), "chunked attention (mma)")

    # ---- a sub-layer output that passes a norm of its own before it joins the stream (csrc/residual_ops.cu) -----------------
    def normed_add_rms_norm(self, residual: torch.Tensor, y: Optional[torch.Tensor], post_weight: Optional[torch.Tensor],
                            post_eps: float, extra: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                            out: Optional[torch.Tensor]) -> None:
        """``residual += y / sqrt(mean(y^2) + post_eps) * post_weight`` (``y`` as it is without ``post_weight``) ``+ extra``
        (float32 rows), all in float32 and in place; ``out`` (optional) receives ``residual / sqrt(mean(residual^2) + eps) *
        weight``.  Each of ``y``, ``extra``, ``out`` may be None."""
        n, h = residual.shape
        act = out if out is not None else y
        if act is None:
            if extra is None:
                return
            act = residual
        for name, t in (("y", y), ("out", out)):
            if t is not None and (t.shape != residual.shape or t.dtype != act.dtype):
                raise KernelError(f"normed_add_rms_norm: {name} {tuple(t.shape)} {t.dtype} does not match the stream {tuple(residual.shape)}")
        if extra is not None and (extra.shape != residual.shape or extra.dtype != torch.float32):
            raise KernelError("normed_add_rms_norm: the second addend must be float32 rows of the stream's shape")
        if (out is not None and (weight is None or weight.numel() != h)) or (post_weight is not None and post_weight.numel() != h):
            raise KernelError("normed_add_rms_norm: a norm's weight does not match the stream")
        fn = _fn("residual_ops", "iian_normed_add_rms_norm",
                 [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(y, "addend"), _cuda(post_weight, "addend norm weight", torch.float32),
                  post_eps, _cuda(extra, "second addend", torch.float32), _cuda(weight, "norm weight", torch.float32),
                  _cuda(out, "norm out"), _code(act, "norm out"), n, h, eps, _stream()), "normed_add_rms_norm")

    def weighted_sum2(self, x: torch.Tensor, a: float, y: torch.Tensor, b: float, out: torch.Tensor) -> None:
        """``out = a x + b y`` element by element (one dtype, one shape)."""
        if x.shape != y.shape or out.shape != x.shape or x.dtype != y.dtype or out.dtype != x.dtype:
            raise KernelError("weighted_sum2: x, y and out must share shape and dtype")
        fn = _fn("stream_ops", "iian_weighted_sum2", [c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_longlong, c_void_p])
        _check(fn(_cuda(x, "x"), a, _cuda(y, "y"), b, _cuda(out, "out"), _code(x, "x"), x.numel(), _stream()), "weighted_sum2")

    def head_norm_gate_act(self, x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *,
                           num_heads: int, eps: float, gate_act: str = "sigmoid") -> None:
        """``head_norm_gate`` with the gate's column passing ``gate_act`` (``sigmoid`` | ``silu``) before it multiplies."""
        n, m = x.shape
        if m % num_heads or weight.numel() != m or out.shape != (n, m) or (gate is not None and (gate.shape != (n, m) or gate.dtype != out.dtype)):
            raise KernelError("head_norm_gate_act: shapes or dtypes do not fit")
        gp, ld = self._rows(gate, "gate")
        fn = _fn("stream_ops", "iian_head_norm_gate_act", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int,
                                                           c_float, c_int, c_void_p])
        _check(fn(_cuda(x, "heads", torch.float32), _cuda(weight, "head norm weight", torch.float32), gp, ld, _cuda(out, "head norm out"),
                  _code(out, "head norm out"), n, num_heads, m // num_heads, eps, {"sigmoid": 0, "silu": 1}[gate_act], _stream()),
               "head_norm_gate_act")

    # ---- rotated attention with a window that keeps the first keys, a sink and a gate per head (csrc/window_attention.cu) ---
    def rotary_table_scaled(self, inv_freq64: torch.Tensor, positions: torch.Tensor, half: int, magnitude: float, out: torch.Tensor) -> None:
        """cos and sin of ``position * inv_freq64`` (product and functions in float64) times ``magnitude`` -> float32 [N, half, 2]."""
        n = positions.shape[0]
        if inv_freq64.dtype != torch.float64 or inv_freq64.numel() < half or out.shape != (n, half, 2) or out.dtype != torch.float32:
            raise KernelError("rotary_table_scaled: frequencies float64 [half], out float32 [N, half, 2]")
        fn = _fn("window_attention", "iian_rotary_table_scaled", [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_double, c_void_p])
        _check(fn(_cuda(inv_freq64, "frequencies"), _cuda(positions, "positions", torch.int32), _cuda(out, "rotary table"), n, half,
                  magnitude, _stream()), "rotary_table_scaled")

    def rotate_unit_store(self, proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor,
                          k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], table: Optional[torch.Tensor],
                          slots: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, rot_dim: int,
                          eps: float, unit_norm: bool) -> None:
        """Per token: rotate the first ``rot_dim`` entries of every head of q and k (entry i with i + rot_dim / 2, angles from
        ``table``), then divide each head by its root mean square (``unit_norm``); q to ``q_out`` [N, heads, k_dim], k and the
        values as projected to the token's cache cells (``k_cache`` None: q only)."""
        n = proj.shape[0]
        pp, ld = self._rows(proj, "projections")
        if q_out.shape != (n, num_heads, k_dim) or q_out.dtype != proj.dtype:
            raise KernelError("rotate_unit_store: q_out must be [N, heads, k_dim] in the projections' dtype")
        if k_cache is not None and (k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != k_dim or v_cache.shape[3] != v_dim
                                    or k_cache.shape[:3] != v_cache.shape[:3] or k_cache.dtype != proj.dtype or slots.numel() != n):
            raise KernelError(f"rotate_unit_store: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit")
        if rot_dim and (table is None or table.shape != (n, rot_dim // 2, 2) or table.dtype != torch.float32):
            raise KernelError("rotate_unit_store: the rotation table must be float32 [N, rot_dim / 2, 2]")
        fn = _fn("window_attention", "iian_rotate_unit_store",
                 [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_longlong, c_float, c_int, c_void_p])
        page = k_cache.shape[2] if k_cache is not None else 1
        cells = k_cache.shape[0] * k_cache.shape[2] if k_cache is not None else 0
        _check(fn(pp, ld, q_off, k_off, v_off, _cuda(q_out, "queries"), _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"),
                  _cuda(table if rot_dim else None, "rotary table"), _cuda(slots, "slots", torch.int32), _code(proj, "projections"), n,
                  num_heads, num_kv_heads if k_cache is not None else 0, k_dim, v_dim, rot_dim, page, cells, eps, 1 if unit_norm else 0,
                  _stream()), "rotate_unit_store")

    WINDOW_ATTENTION_MMA = os.environ.get("IIAN_WINDOW_ATTENTION_MMA", "1") not in ("0", "false", "off")

    def window_attention_mma_ok(self, dtype, num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float) -> bool:
        """Whether the tensor-core kernels of ``csrc/attention_mma.cu`` / ``attention_tc.cu`` serve this attention."""
        return self.WINDOW_ATTENTION_MMA and self.chunked_attention_mma_ok(dtype, num_heads, num_kv_heads, k_dim, v_dim, scale)

    def window_attention_plan(self, num_seqs: int, num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float,
                              max_ctx: int, window: Optional[int], keep_first: int, dtype: torch.dtype):
        if not self.window_attention_mma_ok(dtype, num_heads, num_kv_heads, k_dim, v_dim, scale):
            return None
        return {"n_split": self.attention_splits(num_seqs, num_kv_heads, min(max_ctx, (window or max_ctx) + keep_first))}

    def window_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor, meta, *,
                         num_heads: int, num_kv_heads: int, k_dim: int, v_dim: int, scale: float, window: Optional[int],
                         keep_first: int, sink: Optional[torch.Tensor], gate: Optional[torch.Tensor], gate_per_head: bool,
                         n_split: Optional[int] = None) -> None:
        """``q`` [N, heads * k_dim] -> ``out`` [N, heads * v_dim]: softmax of ``q . k * scale`` over the keys ``j <= i`` with
        ``i - j < window`` or ``j < keep_first``, the denominator also holding ``exp(sink_h)`` if given; weighted sum of the
        cached values, times ``sigmoid(gate)``: one number per head (``gate_per_head``: rows of ``heads`` numbers) or per entry
        (rows of ``heads * v_dim``); the gate may be a column slice.  In bfloat16 with keys and values of 64 or 128 entries
        and a positive scale the tensor-core kernels of ``csrc/attention_mma.cu`` / ``attention_tc.cu`` serve it (kept keys,
        sink and gate inside them); otherwise the general kernel of ``csrc/window_attention.cu``."""
        n = q.shape[0]
        qp, ld_q = self._rows(q, "queries")
        gp, ld_g = self._rows(gate, "gate")
        if q.shape[1] != num_heads * k_dim or out.shape != (n, num_heads * v_dim) or out.dtype != q.dtype or k_cache.dtype != q.dtype \
                or (sink is not None and sink.numel() != num_heads) \
                or (gate is not None and (gate.shape != (n, num_heads if gate_per_head else num_heads * v_dim) or gate.dtype != q.dtype)):
            raise KernelError(f"window_attention: q {tuple(q.shape)}, out {tuple(out.shape)} do not fit")
        if self.window_attention_mma_ok(q.dtype, num_heads, num_kv_heads, k_dim, v_dim, scale) and ld_q % 8 == 0 \
                and qp % 16 == 0 and (gate is None or gate_per_head or (ld_g % 2 == 0 and gp % 4 == 0)):
            self._chunked_attention_mma(qp, ld_q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, k_dim, scale, None, window,
                                        None, None, gp, ld_g, n, n_split, sink=sink, keep_first=keep_first if window else 0,
                                        gate_per_head=gate is not None and gate_per_head)
            return
        bt = meta.block_table
        fn = _fn("window_attention", "iian_window_attention",
                 [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
        _check(fn(qp, ld_q, _cuda(k_cache, "key cache"), _cuda(v_cache, "value cache"), _cuda(out, "attention out"),
                  _cuda(meta.positions, "positions", torch.int32), _cuda(meta.seq_of_token, "seq_of_token", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], _cuda(meta.ctx_len, "ctx_len", torch.int32), _code(q, "queries"),
                  n, num_heads, num_kv_heads, k_dim, v_dim, k_cache.shape[2], k_cache.shape[0], scale, window or 0, keep_first,
                  _cuda(sink, "sink", torch.float32), gp, ld_g, 1 if gate_per_head else 0, _stream()), "window_attention")

    # ---- linear attention with a decay: a matrix state per head (csrc/decay_scan.cu) -----------------------------------------
    def decay_scan(self, proj: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor, cu_q: torch.Tensor,
                   state_slots: torch.Tensor, out: torch.Tensor, *, num_heads: int, dim: int, v_dim: int, activation: Optional[str],
                   q_scale: float, head_decay: Optional[torch.Tensor] = None, z: Optional[torch.Tensor] = None,
                   z_bias: Optional[torch.Tensor] = None, tau: float = 1.0, max_q_len: int = 0) -> None:
        """Walk every sequence's tokens of this step through ``S <- diag(a) S + k v^T``, ``o = S^T q`` from and into ``state``
        [slots, heads, ceil(v_dim / 16), 16, dim rounded up to 4] (float32, column by column in blocks of 16).  ``proj`` rows hold q, k, v at the given column offsets (``activation`` ``silu``:
        all three pass it first); q is multiplied by ``q_scale``.  The decay is ``head_decay`` [heads] (one constant per head)
        or, per token and key channel, ``sigmoid(z + z_bias)^(1 / tau)`` with ``z`` float32 [N, heads * dim] (may be a column
        slice).  ``out`` float32 [N, heads * v_dim]."""
        n = proj.shape[0]
        pp, ld = self._rows(proj, "projections")
        zp, ld_z = self._rows(z, "decay pre-activations")
        s = cu_q.numel() - 1
        if out.shape != (n, num_heads * v_dim) or state_slots.numel() != s or state.dim() != 5 or state.shape[1:] != (num_heads, -(-v_dim // 16), 16, (dim + 3) // 4 * 4) \
                or (head_decay is None) == (z is None) or (head_decay is not None and head_decay.numel() != num_heads) \
                or (z is not None and (z.shape != (n, num_heads * dim) or z.dtype != torch.float32)) \
                or (z_bias is not None and z_bias.numel() != num_heads * dim) or activation not in (None, "silu"):
            raise KernelError("decay_scan: shapes do not fit")
        per_lane = int(os.environ.get("IIAN_DECAY_SCAN_PER_LANE", "0"))
        if per_lane and not getattr(self, "_decay_per_lane_set", False):
            lib = _build.load("decay_scan")
            lib.iian_decay_scan_set_entries_per_lane.argtypes = [c_int]
            lib.iian_decay_scan_set_entries_per_lane.restype = None
            lib.iian_decay_scan_set_entries_per_lane(per_lane)
            self._decay_per_lane_set = True
        fn = _fn("decay_scan", "iian_decay_scan",
                 [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_longlong, c_void_p, c_float, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(pp, ld, q_off, k_off, v_off, 1 if activation == "silu" else 0, q_scale, _cuda(head_decay, "head decays", torch.float32),
                  zp, ld_z, _cuda(z_bias, "decay bias", torch.float32), 1.0 / tau, _cuda(state, "state", torch.float32),
                  _cuda(cu_q, "cu_q", torch.int32), _cuda(state_slots, "state slots", torch.int32), _cuda(out, "scan out", torch.float32),
                  _code(proj, "projections"), s, num_heads, dim, v_dim, state.shape[0], max_q_len, _stream()), "decay_scan")

    # ---- experts weighed by the softmax over the chosen logits; an addend in the experts' sum (csrc/moe.cu) ------------------
    def moe_route_softmax(self, logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor, weights: torch.Tensor) -> None:
        """Router logits (float32, may be a column slice) plus ``bias`` -> the ``top`` experts with the largest values (ties to
        the lower index) and the softmax over those values alone."""
        n, e = logits.shape
        if logits.dtype != torch.float32 or ids.shape != (n, top) or weights.shape != (n, top) or (bias is not None and bias.numel() != e):
            raise KernelError("moe_route_softmax: logits float32 [N, E]; bias [E]; ids / weights [N, top]")
        lp, ld = self._rows(logits, "router logits")
        fn = _fn("moe", "iian_moe_route_softmax", [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
        _check(fn(lp, ld, _cuda(bias, "router bias", torch.float32), e, top, _cuda(ids, "expert ids", torch.int32),
                  _cuda(weights, "expert weights", torch.float32), n, _stream()), "moe_route_softmax")

    def moe_combine_add(self, ys: torch.Tensor, pos: torch.Tensor, out: torch.Tensor, top: int, weights: Optional[torch.Tensor],
                        add: torch.Tensor) -> None:
        """``out[t] = sum_k weights[t, k] * ys[pos[t, k]] + add[t]`` (k ascending, float32); ``add`` may be ``out`` itself."""
        n, w = out.shape
        if ys.shape != (n * top, w) or ys.dtype != out.dtype or add.shape != out.shape or add.dtype != out.dtype \
                or (weights is not None and weights.numel() != n * top):
            raise KernelError("moe_combine_add: ys must be [N * top, W] and add [N, W] in the dtype of out")
        fn = _fn("moe", "iian_moe_combine_add", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(ys, "moe out rows"), _cuda(pos, "pos", torch.int32), _cuda(weights, "expert weights", torch.float32),
                  _cuda(add, "addend"), _cuda(out, "moe out"), _code(out, "moe out"), n, w, top, _stream()), "moe_combine")

    # ---- the delta rule with a decay per key channel (csrc/delta_rule.cu) ---------------------------------------------------
    @staticmethod
    def delta_state_floats(num_heads: int, num_kv_heads: int, dim: int, v_dim: int, taps: int) -> int:
        """Floats of a request's state: S [heads, v_dim, dim], then the convolution's tail [taps - 1, channels]
        (csrc/delta_rule.cu: iian_delta_state_floats)."""
        return num_heads * v_dim * dim + (taps - 1) * (2 * num_kv_heads * dim + num_heads * v_dim)

    def delta_rule(self, proj: torch.Tensor, col_off: int, b_off: int, z: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor,
                   dt_bias: torch.Tensor, state: torch.Tensor, ctx, out: torch.Tensor, *, num_heads: int, num_kv_heads: int, dim: int,
                   v_dim: int) -> None:
        """The recurrence over this step's tokens of every sequence.  ``proj`` rows hold the convolution's inputs q | k | v at
        column ``col_off`` and the write strengths' pre-activations at ``b_off``; ``z`` float32 [N, heads * dim] the decays'
        pre-activations without bias; ``taps`` float32 [channels, taps]; ``state`` float32 [slots, state floats];
        ``out`` float32 [N, heads * v_dim] receives ``S^T q`` per head.  Two launches: per-token preparation, then the scan."""
        n = proj.shape[0]
        h, g, d, v = num_heads, num_kv_heads, dim, v_dim
        channels = 2 * g * d + h * v
        n_taps = taps.shape[1]
        pp, ld = self._rows(proj, "projections")
        s = ctx.cu_q.numel() - 1
        if z.shape != (n, h * d) or taps.shape[0] != channels or a_log.numel() != h or dt_bias.numel() != h * d \
                or out.shape != (n, h * v) or state.dim() != 2 or state.shape[1] != self.delta_state_floats(h, g, d, v, n_taps) \
                or ctx.state_slots.numel() != s:
            raise KernelError("delta_rule: shapes do not fit")
        f32 = torch.float32
        qn = ctx.buf("delta_q", (n, g * d), f32)
        kn = ctx.buf("delta_k", (n, g * d), f32)
        vv = ctx.buf("delta_v", (n, h * v), f32)
        beta = ctx.buf("delta_beta", (n, h), f32)
        decay = ctx.buf("delta_decay", (n, h * d), f32)
        qk = ctx.buf("delta_qk", (n, g), f32)
        code = _code(proj, "projections")
        fn = _fn("delta_rule", "iian_delta_prep",
                 [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_void_p])
        _check(fn(pp, ld, col_off, b_off, code, _cuda(z, "decay pre-activations", f32), _cuda(taps, "taps", f32), n_taps,
                  _cuda(a_log, "A_log", f32), _cuda(dt_bias, "dt_bias", f32), _cuda(state, "state", f32), state.shape[1],
                  _cuda(ctx.seq_of_token, "seq_of_token", torch.int32), _cuda(ctx.cu_q, "cu_q", torch.int32),
                  _cuda(ctx.state_slots, "state slots", torch.int32), qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), beta.data_ptr(),
                  decay.data_ptr(), qk.data_ptr(), n, h, g, d, v, _stream()), "delta_prep")
        fn = _fn("delta_rule", "iian_delta_scan",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int,
                  c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), beta.data_ptr(), decay.data_ptr(), qk.data_ptr(), state.data_ptr(),
                  state.shape[1], pp, ld, col_off, code, n_taps, ctx.cu_q.data_ptr(), ctx.state_slots.data_ptr(),
                  _cuda(out, "delta out", f32), s, h, g, d, v, int(getattr(ctx, "max_q_len", 0) or 0), _stream()), "delta_scan")

    # ---- routing by a table, weights on the experts' outputs (csrc/moe.cu) ------------------------------------------------------
    def moe_table_route(self, tokens: torch.Tensor, rows: Optional[torch.Tensor], table: torch.Tensor, num_experts: int,
                        ids: torch.Tensor, weights: torch.Tensor, weight: float) -> None:
        """``ids[r] = table[tokens[rows[r]]]`` (``rows`` None: every token in order), every weight ``weight``."""
        n, top = ids.shape
        if table.dim() != 2 or table.shape[1] != top or weights.shape != (n, top) or (rows is None and tokens.numel() != n) \
                or (rows is not None and rows.numel() != n):
            raise KernelError("moe_table_route: table [V, top]; ids / weights [N, top]")
        fn = _fn("moe", "iian_moe_table_route", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_int,
                                                 c_int, c_void_p])
        _check(fn(_cuda(tokens, "tokens", torch.int32), _cuda(rows, "rows", torch.int32), _cuda(table, "expert table", torch.int32),
                  table.shape[0], num_experts, top, _cuda(ids, "expert ids", torch.int32), _cuda(weights, "expert weights", torch.float32),
                  weight, n, tokens.numel(), _stream()), "moe_table_route")

    # ---- sampling ------------------------------------------------------------------------
    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        r, v = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("argmax: logits rows must be contiguous")
        if not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("argmax: logits must be float32 on CUDA")
        if v >= 16384 and r <= 65535:      # wide rows: many blocks per row, then a merge
            scratch = self.attention_scratch(logits.device, r * 64 * 2)
            fn = _fn("sampling", "iian_argmax_wide", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p])
            _check(fn(logits.data_ptr(), r, v, logits.stride(0), scratch.data_ptr(), _cuda(out, "argmax out", torch.int32),
                      _stream()), "argmax")
            LAUNCHES[0] += 1
            return
        fn = _fn("sampling", "iian_argmax", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(out, "argmax out", torch.int32), _stream()), "argmax")

    def logit_edits(self, logits: torch.Tensor, ints: torch.Tensor, floats: torch.Tensor, n_allow: int, n_edit: int) -> None:
        """Logits processors on ``logits`` [R, V] float32, in place.  ``ints`` (int32, on the device) holds, one after
        the other, allow_off [R + 1], edit_off [R + 1], allow_ids [n_allow], edit_tok [n_edit]; ``floats`` holds pre,
        mul_pos, mul_neg, post, [n_edit] each."""
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("logit_edits: logits must be float32 on CUDA with contiguous rows")
        if ints.numel() != 2 * (r + 1) + n_allow + n_edit or floats.numel() != 4 * n_edit:
            raise KernelError("logit_edits: the lists do not have the announced lengths")
        ip, fp = _cuda(ints, "edit lists", torch.int32), _cuda(floats, "edit values", torch.float32) if n_edit else 0
        allow_off, edit_off = ip, ip + 4 * (r + 1)
        allow_ids, edit_tok = ip + 8 * (r + 1), ip + 8 * (r + 1) + 4 * n_allow
        fn = _fn("sampling", "iian_logit_edits", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), allow_off, allow_ids, edit_off, edit_tok,
                  fp, fp + 4 * n_edit, fp + 8 * n_edit, fp + 12 * n_edit, _stream()), "logit_edits")

    def logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, want_k: torch.Tensor, kmax: int):
        """Raw log-probabilities of ``tokens`` [R] and of the ``want_k[r]`` most likely tokens of each row (negative:
        the row is skipped): ``(lp [R], top_ids [R, kmax], top_lp [R, kmax])`` on the device."""
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("logprobs: logits must be float32 on CUDA with contiguous rows")
        lp = torch.full((r,), float("-inf"), dtype=torch.float32, device=logits.device)
        ids = torch.full((r, max(kmax, 1)), -1, dtype=torch.int32, device=logits.device)
        lps = torch.full((r, max(kmax, 1)), float("-inf"), dtype=torch.float32, device=logits.device)
        fn = _fn("sampling", "iian_logprobs", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(tokens, "tokens", torch.int32),
                  _cuda(want_k, "want_k", torch.int32), kmax, lp.data_ptr(), ids.data_ptr(), lps.data_ptr(), _stream()), "logprobs")
        return lp, ids, lps

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
               min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("sample: logits must be float32 on CUDA with contiguous rows")
        fn = _fn("sampling", "iian_sample", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(temperature, "temperature", torch.float32),
                  _cuda(top_k, "top_k", torch.int32), _cuda(top_p, "top_p", torch.float32),
                  _cuda(min_p, "min_p", torch.float32), _cuda(uniform, "uniform", torch.float32),
                  _cuda(out, "sample out", torch.int32), _stream()), "sample")


class WeightPrefetcher:
    """Keeps HBM busy between the weight-streaming products of a captured decode step.

    ``weights`` is the order in which the step's products read their weights (recorded on an eager
    run).  Before product ``i`` is launched on the capturing stream, a side stream is forked with an event
    (so it runs beside product ``i``) and prefetches the head of product ``i + 1``'s weights into L2: from the
    end of what was prefetched so far up to ``window`` bytes beyond their start.  Product ``i + 1`` then finds
    its first rounds of loads in L2 and HBM does not idle while it starts up.  ``IIAN_PREFETCH_EARLY=0`` forks
    after product ``i`` instead (the prefetch then runs beside whatever follows it, which only pays where an
    attention kernel follows: 3.55 against 3.48 ms a step at batch 1, 3.72 against 3.67 ms at batch 8).
    The side stream is joined into the main stream before the capture ends.

    Measured on B200 at the Qwen3-8B sizes, batch 8: a window of 8 MB (the head of the next matrix, which
    hides the ramp-up of its product) gains 2.4 % of the step; 24 MB and more lose, because a matrix that
    streams through L2 evicts what was prefetched beyond it.
    """

    def __init__(self, weights, window: int = int(os.environ.get("IIAN_PREFETCH_WINDOW_MB", "8")) << 20):
        self.weights = list(weights)
        self.starts = []
        pos = 0
        for _, nbytes in self.weights:
            self.starts.append(pos)
            pos += nbytes
        self.total = pos
        self.window = window
        self.early = os.environ.get("IIAN_PREFETCH_EARLY", "1") not in ("0", "false", "off")
        self.side = torch.cuda.Stream()
        self.index = 0             # products launched so far
        self.cursor = 0            # bytes of the concatenated weight sequence already asked for
        self.launches = 0

    def before_product(self, kernels) -> None:
        if self.early:
            self._prefetch_head(kernels, self.index + 1)

    def after_product(self, kernels) -> None:
        self.index += 1
        if not self.early:
            self._prefetch_head(kernels, self.index)

    def _prefetch_head(self, kernels, j: int) -> None:
        """Fork the side stream at this point of the main stream and ask for the head of product ``j``'s weights."""
        if j >= len(self.weights):
            return
        begin = max(self.cursor, self.starts[j])
        end = min(self.total, self.starts[j] + self.window)
        if end <= begin:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            while j < len(self.weights) and self.starts[j] < end:
                ptr, nbytes = self.weights[j]
                lo = max(begin, self.starts[j]) - self.starts[j]
                hi = min(end, self.starts[j] + nbytes) - self.starts[j]
                if hi > lo:
                    kernels.prefetch_l2(ptr + lo, hi - lo, stream=self.side.cuda_stream)
                    self.launches += 1
                j += 1
        self.cursor = end

    def join(self) -> None:
        ev = torch.cuda.Event()
        ev.record(self.side)
        torch.cuda.current_stream().wait_event(ev)
