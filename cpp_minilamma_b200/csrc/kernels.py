"""Python face of the kernel library: typed wrappers that check tensors on the host
and launch on the current CUDA stream.

Every function here needs the compiled library and CUDA tensors; there is no other
implementation behind them.  Argument faults raise `KernelError` before any launch.
"""
from __future__ import annotations

import ctypes
from typing import Dict, NamedTuple, Optional

import torch

from ..cache.paged import PAGE  # cache positions per page; the library's MLL_PAGE is checked against it on load
from .build import KernelBuildError, load_library

ABI_VERSION = 33
MAX_TOP_K = 1024


class KernelError(RuntimeError):
    pass


class DeviceKernelError(KernelError):
    """A kernel gave up on the device (a bounded wait ran out, or its shared memory was misplaced): what the
    step computed is not to be used."""


_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        handle = load_library()
        handle.mll_last_error.restype = ctypes.c_char_p
        handle.mll_attn_decode_scratch_floats.restype = ctypes.c_longlong
        if handle.mll_abi_version() != ABI_VERSION:
            raise KernelBuildError(
                f"kernel library reports ABI {handle.mll_abi_version()}, the package expects {ABI_VERSION}; "
                "remove csrc/_build and rebuild")
        if handle.mll_page() != PAGE:
            raise KernelBuildError(f"kernel library built for pages of {handle.mll_page()} positions, the cache uses {PAGE}")
        _lib = handle
    return _lib


def multiprocessor_count() -> int:
    """Multiprocessors of the current CUDA device (the library asks the driver once per device)."""
    return int(lib().mll_multiprocessor_count())


launches = 0  # kernels of this library launched so far (counted per successful call)
calls: Dict[str, int] = {}  # the same, per kind of launch (the name each wrapper gives its kernel)


class KernelTimes:
    """Device time of every launch made through this module while the object is the active timer: a CUDA event
    is recorded on the launching stream before and after each call (`with KernelTimes() as times: ...`;
    `times.totals()` waits for the device and gives {kernel: (calls, milliseconds)})."""

    def __init__(self):
        self.events = []
        self._open = None

    def __enter__(self):
        global _timer
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None

    def begin(self):
        self._open = torch.cuda.Event(enable_timing=True)
        self._open.record()

    def end(self, what: str):
        if self._open is not None:
            done = torch.cuda.Event(enable_timing=True)
            done.record()
            self.events.append((what, self._open, done))
            self._open = None

    def totals(self):
        torch.cuda.synchronize()
        out: Dict[str, list] = {}
        for what, first, last in self.events:
            entry = out.setdefault(what, [0, 0.0])
            entry[0] += 1
            entry[1] += first.elapsed_time(last)
        return {k: (v[0], v[1]) for k, v in out.items()}


_timer: Optional[KernelTimes] = None


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launches
    if _timer is not None:
        _timer.end(what)
    launches += kernels
    calls[what] = calls.get(what, 0) + 1
    if code != 0:
        message = lib().mll_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {message} (code {code})")


def _stream() -> ctypes.c_void_p:
    # every wrapper evaluates this once, among the arguments of its launch: the place where a timer's first event goes
    if _timer is not None:
        _timer.begin()
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (the kernels have no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous, strides {tuple(t.stride())}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got shape {tuple(t.shape)}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype not in _DTYPE_CODE:
        raise KernelError(f"dtype {dtype} not supported by the kernels (float32, bfloat16)")
    return _DTYPE_CODE[dtype]


# --------------------------------------------------------------------------- #
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = scale * float32(table[tokens[t], :]); tokens int32 [T], out float32 [T, D]."""
    _need(tokens, "embedding tokens", torch.int32, 1)
    _need(table, "embedding table", None, 2)
    _need(out, "embedding out", torch.float32, 2)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width:
        raise KernelError(f"embedding: out {tuple(out.shape)} does not fit [{n}, {width}]")
    _check(lib().mll_embedding(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out),
                               ctypes.c_int(n), ctypes.c_int(width), ctypes.c_float(scale), _stream()), "embedding")


def scale_(x: torch.Tensor, factor: float) -> None:
    """x *= factor (float32, in place)."""
    _need(x, "scale x", torch.float32)
    _check(lib().mll_scale(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(factor), _stream()), "scale")


def embedding_pair(tokens, tok_pos, tok_seq, seq_slot, seq_qstart, seq_qlen, prev_token, table, pairs, out,
                   buckets: int, mul_prev: int, mul_cur: int, scale: float) -> None:
    """out[t, :] = scale * table[tokens[t], :] + pairs[row(t), :] (float32 [T, D]), row(t) = (mul_prev * the token
    before + mul_cur * tokens[t]) mod buckets, and `buckets` (the table's last row) at position 0.  The token before
    a step's first one is prev_token[slot] (int32 [slots]), where the step's last token is left for the next step.
    `pairs` None: the scaled rows alone."""
    _need(tokens, "pair embedding tokens", torch.int32, 1)
    _need(table, "pair embedding table", None, 2)
    _need(out, "pair embedding out", torch.float32, 2)
    _need(prev_token, "pair embedding previous tokens", torch.int32, 1)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width:
        raise KernelError(f"pair embedding: out {tuple(out.shape)} does not fit [{n}, {width}]")
    if pairs is not None:
        _need(pairs, "pair embedding pair table", table.dtype, 2)
        if tuple(pairs.shape) != (buckets + 1, width):
            raise KernelError(f"pair embedding: pair table {tuple(pairs.shape)}, expected {(buckets + 1, width)}")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("seq_qstart", seq_qstart),
                    ("seq_qlen", seq_qlen)):
        _need(t, f"pair embedding {name}", torch.int32, 1)
    _check(lib().mll_embedding_pair(_ptr(tokens), _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot), _ptr(seq_qstart),
                                    _ptr(seq_qlen), _ptr(prev_token), _ptr(table), _ptr(pairs), dtype_code(table.dtype),
                                    _ptr(out), ctypes.c_int(n), ctypes.c_int(width), ctypes.c_int(max(buckets, 1)),
                                    ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), ctypes.c_float(scale),
                                    _stream()), "embedding_pair")


ACT_GELU_ERF, ACT_GELU_TANH = 0, 1


def activation(src: torch.Tensor, dst: torch.Tensor, kind: int) -> None:
    """dst = act(src) elementwise, evaluated in float32 (dst may be src): the erf or the tanh form of gelu."""
    _need(src, "activation in")
    _need(dst, "activation out", src.dtype)
    if src.numel() != dst.numel():
        raise KernelError("activation: sizes differ")
    _check(lib().mll_activation(_ptr(src), _ptr(dst), dtype_code(src.dtype), ctypes.c_longlong(src.numel()),
                                ctypes.c_int(kind), _stream()), "activation")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    _need(src, "cast src")
    _need(dst, "cast dst")
    if src.numel() != dst.numel():
        raise KernelError("cast: sizes differ")
    _check(lib().mll_cast(_ptr(src), dtype_code(src.dtype), _ptr(dst), dtype_code(dst.dtype),
                          ctypes.c_longlong(src.numel()), _stream()), "cast")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t, :] += bias (float32 bias, in place)."""
    _need(x, "add_bias x", None, 2)
    _need(bias, "add_bias bias", torch.float32, 1)
    if bias.shape[0] != x.shape[1]:
        raise KernelError("add_bias: bias length differs from the row width")
    _check(lib().mll_add_bias(_ptr(x), _ptr(bias), dtype_code(x.dtype), ctypes.c_int(x.shape[0]),
                              ctypes.c_int(x.shape[1]), _stream()), "add_bias")


def scatter_rows(table: torch.Tensor, staged: torch.Tensor, n_rows: int) -> None:
    """table[staged[r, 0], :] = staged[r, 1:] for r < n_rows: block-table rows that changed on the host.
    table int32 [rows, width]; staged int32, n_rows * (1 + width) values."""
    _need(table, "scatter_rows table", torch.int32, 2)
    _need(staged, "scatter_rows staged", torch.int32)
    if staged.numel() < n_rows * (1 + table.shape[1]):
        raise KernelError("scatter_rows: staged rows shorter than the count says")
    _check(lib().mll_scatter_rows(_ptr(table), _ptr(staged), ctypes.c_int(n_rows), ctypes.c_int(table.shape[1]),
                                  ctypes.c_int(table.shape[0]), _stream()), "scatter_rows")


def gather_int32(dst: torch.Tensor, src: torch.Tensor, index: torch.Tensor, n: int) -> None:
    """dst[i] = src[index[i]] for i < n (int32; an index outside src gives 0): the tokens that a step sampled,
    brought into the order of the next step's rows on the device."""
    for name, t in (("dst", dst), ("src", src), ("index", index)):
        _need(t, f"gather_int32 {name}", torch.int32, 1)
    if dst.shape[0] < n or index.shape[0] < n:
        raise KernelError("gather_int32: dst or index shorter than the count says")
    _check(lib().mll_gather_int32(_ptr(dst), _ptr(src), _ptr(index), ctypes.c_int(n), ctypes.c_int(src.shape[0]),
                                  _stream()), "gather_int32")


EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_RESID = 0, 1, 2, 3
NORM_TILE = 16  # columns per partial sum of squares that the residual epilogue writes


class RowNorm(NamedTuple):
    """Rows that still lack their RMS norm's factor: `sumsq` float32 [rows, stride] holds `partials`
    partial sums of squares per row; the factor is 1 / sqrt(sum / width + eps)."""
    sumsq: torch.Tensor
    partials: int
    eps: float


class ResidualOut(NamedTuple):
    """Where the residual epilogue writes: `resid` float32 [rows, N] (+= result), `next_weight` float32 [N]
    (out = resid * next_weight in bfloat16), `sumsq` float32 [rows, stride >= ceil(N / NORM_TILE)]."""
    resid: torch.Tensor
    next_weight: torch.Tensor
    sumsq: torch.Tensor


def _row_norm_args(row_norm: Optional["RowNorm"], rows: int, what: str):
    if row_norm is None:
        return ctypes.c_void_p(None), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_float(0.0)
    _need(row_norm.sumsq, what + " partial sums", torch.float32, 2)
    if row_norm.sumsq.shape[0] < rows or row_norm.sumsq.shape[1] < row_norm.partials:
        raise KernelError(f"{what}: partial sums {tuple(row_norm.sumsq.shape)} for {rows} rows of {row_norm.partials}")
    return (_ptr(row_norm.sumsq), ctypes.c_int(row_norm.partials), ctypes.c_int(row_norm.sumsq.shape[1]),
            ctypes.c_float(row_norm.eps))


def linear_small_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_small_supported(rows, out_features, in_features, epilogue))


def linear_small(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None,
                 residual: Optional[ResidualOut] = None) -> None:
    """out = x . w^T for at most 64 rows of bfloat16 x [M, K] and bfloat16 w [N, K], read once.

    epilogue EPI_BF16 / EPI_F32: out [M, N] in that dtype (+ float32 bias [N]);
    EPI_SWIGLU: w holds gate and up rows interleaved in blocks of 8, out [M, N / 2] = silu(gate) * up;
    EPI_RESID (at most 16 rows, with `residual`): the result is added to the residual stream, out [M, N]
    is the new stream times the next norm's weight (not yet its factor), with partial sums of squares.
    `row_norm`: x is such an output; the result is multiplied by the rows' factors."""
    _need(x, "linear_small x", torch.bfloat16, 2)
    _need(w, "linear_small w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_small: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_small out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_small: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_small bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_small: bias length differs from the output width")
    if (epilogue == EPI_RESID) != (residual is not None):
        raise KernelError("linear_small: the residual epilogue and its outputs go together")
    resid = next_w = out_sumsq = None
    out_stride = 0
    if residual is not None:
        resid, next_w, out_sumsq = residual
        _need(resid, "linear_small resid", torch.float32, 2)
        _need(next_w, "linear_small next weight", torch.float32, 1)
        _need(out_sumsq, "linear_small sums of squares", torch.float32, 2)
        if tuple(resid.shape) != (rows, n) or next_w.shape[0] != n or out_sumsq.shape[0] < rows:
            raise KernelError(f"linear_small: resid {tuple(resid.shape)}, next weight {tuple(next_w.shape)}, sums "
                              f"{tuple(out_sumsq.shape)} do not fit out {(rows, n)}")
        out_stride = out_sumsq.shape[1]
    _check(lib().mll_linear_small_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                        ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                        *_row_norm_args(row_norm, rows, "linear_small"), _ptr(resid), _ptr(next_w),
                                        _ptr(out_sumsq), ctypes.c_int(out_stride), _stream()), "linear_small")


def linear_tma_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_tma_supported(rows, out_features, in_features, epilogue))


def linear_tma(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
               epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None) -> None:
    """As `linear_small`, with the weights streamed through a TMA + mbarrier pipeline.  Takes
    any N, any K that is a multiple of 8, at most 64 rows."""
    _need(x, "linear_tma x", torch.bfloat16, 2)
    _need(w, "linear_tma w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_tma: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_tma out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_tma: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_tma bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_tma: bias length differs from the output width")
    _check(lib().mll_linear_tma_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                      ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                      *_row_norm_args(row_norm, rows, "linear_tma"), _stream()), "linear_tma")


def linear_tc5_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_tc5_supported(rows, out_features, in_features, epilogue))


def linear_tc5(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
               epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None,
               residual: Optional[ResidualOut] = None) -> None:
    """As `linear_small` (the residual epilogue included, here for up to 64 rows), with the product on the
    fifth-generation tensor cores: tcgen05.mma reads the TMA-filled stages from shared memory and
    accumulates in tensor memory.  Takes any N, any K that is a multiple of 8, at most 64 rows."""
    _need(x, "linear_tc5 x", torch.bfloat16, 2)
    _need(w, "linear_tc5 w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_tc5: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_tc5 out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_tc5: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_tc5 bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_tc5: bias length differs from the output width")
    if (epilogue == EPI_RESID) != (residual is not None):
        raise KernelError("linear_tc5: the residual epilogue and its outputs go together")
    resid = next_w = out_sumsq = None
    out_stride = 0
    if residual is not None:
        resid, next_w, out_sumsq = residual
        _need(resid, "linear_tc5 resid", torch.float32, 2)
        _need(next_w, "linear_tc5 next weight", torch.float32, 1)
        _need(out_sumsq, "linear_tc5 sums of squares", torch.float32, 2)
        if tuple(resid.shape) != (rows, n) or next_w.shape[0] != n or out_sumsq.shape[0] < rows:
            raise KernelError(f"linear_tc5: resid {tuple(resid.shape)}, next weight {tuple(next_w.shape)}, sums "
                              f"{tuple(out_sumsq.shape)} do not fit out {(rows, n)}")
        out_stride = out_sumsq.shape[1]
    _check(lib().mll_linear_tc5_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                      ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                      *_row_norm_args(row_norm, rows, "linear_tc5"), _ptr(resid), _ptr(next_w),
                                      _ptr(out_sumsq), ctypes.c_int(out_stride), _stream()), "linear_tc5")


DEVICE_ERROR_BITS = ("the TMA linear kernel", "the tcgen05 linear kernel", "the tcgen05 prefill attention kernel",
                     "the TMA decode attention kernel")


def take_device_error() -> int:
    """Non-zero when a kernel gave up since the flags were last read (then cleared): bit i stands for
    DEVICE_ERROR_BITS[i]; synchronises.  The sampling kernels read and clear the same flags on the
    device and hand them to `DeviceSampler.collect` in their status word."""
    return int(lib().mll_take_device_error())


def raise_device_error(mask: int) -> None:
    """Set the flags of `mask` from the host, as a kernel that gave up would (for tests of the host side)."""
    _check(lib().mll_raise_device_error(ctypes.c_int(mask)), "raise_device_error", kernels=0)


def device_error_message(mask: int) -> str:
    names = [name for i, name in enumerate(DEVICE_ERROR_BITS) if mask & (1 << i)] or [f"mask {mask}"]
    return ("a bounded wait ran out (or a block's shared memory was misplaced) in " + ", ".join(names)
            + "; the step's results are not valid")


TMA_MAX_ROWS = 8      # rows up to which tall matrices go to the direct kernel, or the TMA + mma.sync kernel (one batch tile of 8 rows)
TC5_TALL_MAX_ROWS = 16  # rows up to which tall matrices go to the tcgen05 kernel (beyond: the library, which shares the
                        # batch tile between the blocks of a cluster)
DIRECT_MAX_ROWS = 16  # rows up to which the other matrices go to the direct kernel
TALL = 16384          # output features from which a matrix counts as tall


def small_linear_kind(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> str:
    """Which of this library's weight-streaming kernels takes the problem: "tc5", "tma", "direct" or "".

    Measured on B200 (CUDA-graph timing) on the shapes of the 8B, 7B and 1B Llama models.  Tall matrices
    (gate/up, lm_head) up to 8 rows: the direct kernel, as it stands since it got its register targets and eight
    warps a block (us at 8 rows, direct / TMA + mma.sync / tcgen05: 8B gate/up + SwiGLU 38.7 / 41.5 / 42.6, lm_head
    154.7 / 159.5 / 161.5; 7B 31.1 / 32.3 / 33.0 and 42.5 / 46.3 / 46.2; 1B 13.3 / 15.2 / 16.1 and 78.3 / 80.4 /
    83.0; the TMA kernel stays for widths the direct kernel does not take); from 9 to 16 rows the tcgen05 kernel
    (8B gate/up 43.0 against 45.3 direct and 54.5 TMA with their second batch tile).  The other projections: the
    direct kernel up to 16 rows (it chooses its variant by rows and tiles).  From 17 rows on the library GEMM: the tcgen05 kernel takes up to 64 rows (32 or 64 batch
    columns per MMA), but inside a CUDA graph the library's kernels are ahead on every shape tried
    (64 rows, us, library / tcgen05: 8B q/k/v 11.8 / 16.2, o 9.9 / 13.1, down 24.9 / 26.5, gate/up 42.8 /
    46.9; 1B q/k/v 5.9 / 9.6, o 5.7 / 9.1, down 13.2 / 14.5, gate/up 13.2 / 19.1), and in a batch-64 step
    the three small products took 60.6 us a layer on it against 46.6 + two norm kernels on the library."""
    if SMALL_LINEAR == "none":
        return ""
    if SMALL_LINEAR != "auto":  # a forced kind (tests, experiments)
        supported = {"tc5": linear_tc5_supported, "tma": linear_tma_supported, "direct": linear_small_supported}
        return SMALL_LINEAR if rows <= 64 and supported[SMALL_LINEAR](rows, out_features, in_features, epilogue) else ""
    if out_features >= TALL:
        if rows <= TMA_MAX_ROWS:  # one batch tile of 8 rows in either kernel
            if linear_small_supported(rows, out_features, in_features, epilogue):
                return "direct"
            if linear_tma_supported(rows, out_features, in_features, epilogue):
                return "tma"
        if rows <= TC5_TALL_MAX_ROWS and linear_tc5_supported(rows, out_features, in_features, epilogue):
            return "tc5"
    if rows <= DIRECT_MAX_ROWS:
        if linear_small_supported(rows, out_features, in_features, epilogue):
            return "direct"
        if linear_tma_supported(rows, out_features, in_features, epilogue):
            return "tma"
    return ""


def small_linear(x, w, bias, out, epilogue: int = EPI_BF16, row_norm: Optional[RowNorm] = None,
                 residual: Optional[ResidualOut] = None) -> bool:
    """Run the product on the kernel that `small_linear_kind` names; False when there is none (then
    nothing ran).  The residual epilogue exists in the direct kernel and in the tcgen05 kernel."""
    kind = small_linear_kind(x.shape[0], w.shape[0], w.shape[1], EPI_BF16 if epilogue == EPI_RESID else epilogue)
    if epilogue == EPI_RESID and kind not in ("direct", "tc5"):
        return False
    if kind == "tc5":
        linear_tc5(x, w, bias, out, epilogue, 0, row_norm, residual)
    elif kind == "tma":
        linear_tma(x, w, bias, out, epilogue, 1 if x.shape[0] > 8 else 0, row_norm)
    elif kind == "direct":
        linear_small(x, w, bias, out, epilogue, 0, row_norm, residual)
    return bool(kind)


def fused_norm_rows(rows: int) -> bool:
    """Whether products over `rows` rows may fold the norms around them in (the residual epilogue
    exists in the kernels that take decode steps' row counts)."""
    return FUSE_NORM and 1 <= rows <= (64 if SMALL_LINEAR == "tc5" else DIRECT_MAX_ROWS)


FUSE_NORM = True  # off: every norm is a kernel of its own


SMALL_LINEAR = "auto"  # "auto", a forced kind ("tc5", "tma", "direct"), or "none" (library GEMM only)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int, row_norm: Optional[RowNorm] = None,
           width: int = 0, bias: Optional[torch.Tensor] = None) -> None:
    """out[t, i] = silu(gate) * up; gate_up [T, 2I] holds halves (block 0) or blocks of `block`.
    `bias` (float32 [2I], in the order of gate_up's columns) is added to gate and up first, in float32.
    `row_norm` (bfloat16, I a multiple of 8): gate_up was computed from rows of `width` columns that lacked their
    norm's factor; gate and up are multiplied by it first."""
    _need(gate_up, "swiglu gate_up", None, 2)
    _need(out, "swiglu out", gate_up.dtype, 2)
    tokens, inter = out.shape
    if gate_up.shape[0] != tokens or gate_up.shape[1] != 2 * inter:
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "swiglu bias", torch.float32, 1)
        if bias.shape[0] != 2 * inter or row_norm is not None:
            raise KernelError("swiglu: the bias has one value per column of gate_up (and no row factors with it)")
    if row_norm is not None:
        if gate_up.dtype != torch.bfloat16 or inter % 8 or block not in (0, 8) or width <= 0:
            raise KernelError("swiglu: rows without their norm's factor need bfloat16, I % 8 == 0 and the rows' width")
        sumsq, partials, stride, eps = _row_norm_args(row_norm, tokens, "swiglu")
        _check(lib().mll_swiglu_rows(_ptr(gate_up), _ptr(out), ctypes.c_int(tokens), ctypes.c_int(inter),
                                     ctypes.c_int(block), sumsq, partials, stride, eps, ctypes.c_int(width), _stream()),
               "swiglu_rows")
        return
    _check(lib().mll_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), ctypes.c_int(tokens),
                            ctypes.c_int(inter), ctypes.c_int(block), _ptr(bias), _stream()), "swiglu")


class DeltaNorm(NamedTuple):
    """What a delta passes on its way into the stream: d = scale1 * delta (+ scale2 * delta2), then, with `weight`
    (float32 [D]), d <- d / sqrt(mean(d^2) + eps) * weight."""
    weight: Optional[torch.Tensor]
    eps: float = 0.0
    scale1: float = 1.0
    scale2: float = 1.0


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, delta2: Optional[torch.Tensor] = None,
                delta_norm: Optional[DeltaNorm] = None) -> None:
    """x += delta (+ delta2) (float32 residual, in place); out = rmsnorm(x) * weight.
    `delta_norm`: the delta is scaled and normalised first (see DeltaNorm), all in float32.

    With `rows` (int32 [n]) only those rows of x are normalised into out [n, D] and x is
    left unchanged.  `delta2`: the output of a second part that read the same norm as `delta`'s.
    out may be float32 whatever the deltas' dtype, and may be x itself."""
    _need(x, "rmsnorm x", torch.float32, 2)
    _need(weight, "rmsnorm weight", torch.float32, 1)
    _need(out, "rmsnorm out", None, 2)
    width = x.shape[1]
    if weight.shape[0] != width or out.shape[1] != width:
        raise KernelError(f"rmsnorm: widths differ: x {width}, weight {weight.shape[0]}, out {out.shape[1]}")
    delta_dtype = out.dtype
    if delta is not None:
        _need(delta, "rmsnorm delta", None, 2)
        delta_dtype = delta.dtype
        if delta.shape != x.shape:
            raise KernelError(f"rmsnorm: delta {tuple(delta.shape)} differs from x {tuple(x.shape)}")
    if delta2 is not None:
        if delta is None:
            raise KernelError("rmsnorm: a second delta without a first")
        _need(delta2, "rmsnorm delta2", delta.dtype, 2)
        if delta2.shape != x.shape:
            raise KernelError(f"rmsnorm: delta2 {tuple(delta2.shape)} differs from x {tuple(x.shape)}")
    if delta_dtype != out.dtype and not (delta_dtype == torch.bfloat16 and out.dtype == torch.float32):
        raise KernelError(f"rmsnorm: delta {delta_dtype} with out {out.dtype}")
    if rows is not None:
        _need(rows, "rmsnorm rows", torch.int32, 1)
        n_rows = rows.shape[0]
    else:
        n_rows = x.shape[0]
    if out.shape[0] != n_rows:
        raise KernelError(f"rmsnorm: out has {out.shape[0]} rows, expected {n_rows}")
    if delta_norm is not None:
        if delta is None:
            raise KernelError("rmsnorm: a norm of the delta without a delta")
        if delta_norm.weight is not None:
            _need(delta_norm.weight, "rmsnorm delta weight", torch.float32, 1)
            if delta_norm.weight.shape[0] != width:
                raise KernelError("rmsnorm: the delta's norm weight differs in width")
        _check(lib().mll_add_normed_rmsnorm(
            _ptr(x), _ptr(delta), _ptr(delta2), ctypes.c_float(delta_norm.scale1), ctypes.c_float(delta_norm.scale2),
            _ptr(delta_norm.weight), ctypes.c_float(delta_norm.eps), _ptr(weight), _ptr(out), _ptr(rows),
            dtype_code(delta_dtype), dtype_code(out.dtype), ctypes.c_int(n_rows), ctypes.c_int(width),
            ctypes.c_float(eps), _stream()), "rmsnorm (normed delta)")
        return
    _check(lib().mll_add2_rmsnorm(_ptr(x), _ptr(delta), _ptr(delta2), _ptr(weight), _ptr(out), _ptr(rows),
                                  dtype_code(delta_dtype), dtype_code(out.dtype), ctypes.c_int(n_rows),
                                  ctypes.c_int(width), ctypes.c_float(eps), _stream()), "rmsnorm")


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                  out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (float32 residual, in place); out = (x - mean) / sqrt(var + eps) * weight + bias, the variance
    being the mean squared deviation.  `rows` as in `add_rmsnorm`."""
    _need(x, "layernorm x", torch.float32, 2)
    _need(weight, "layernorm weight", torch.float32, 1)
    _need(out, "layernorm out", None, 2)
    width = x.shape[1]
    if weight.shape[0] != width or out.shape[1] != width:
        raise KernelError(f"layernorm: widths differ: x {width}, weight {weight.shape[0]}, out {out.shape[1]}")
    if bias is not None:
        _need(bias, "layernorm bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise KernelError(f"layernorm: bias of {bias.shape[0]}, expected {width}")
    delta_dtype = out.dtype
    if delta is not None:
        _need(delta, "layernorm delta", None, 2)
        delta_dtype = delta.dtype
        if delta.shape != x.shape:
            raise KernelError(f"layernorm: delta {tuple(delta.shape)} differs from x {tuple(x.shape)}")
    if delta_dtype != out.dtype and not (delta_dtype == torch.bfloat16 and out.dtype == torch.float32):
        raise KernelError(f"layernorm: delta {delta_dtype} with out {out.dtype}")
    if rows is not None:
        _need(rows, "layernorm rows", torch.int32, 1)
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if out.shape[0] != n_rows:
        raise KernelError(f"layernorm: out has {out.shape[0]} rows, expected {n_rows}")
    _check(lib().mll_add_layernorm(_ptr(x), _ptr(delta), _ptr(weight), _ptr(bias), _ptr(out), _ptr(rows),
                                   dtype_code(delta_dtype), dtype_code(out.dtype), ctypes.c_int(n_rows),
                                   ctypes.c_int(width), ctypes.c_float(eps), _stream()), "layernorm")


def stream_concat(x: torch.Tensor, delta: Optional[torch.Tensor], x0: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [x[t] + delta[t] ; x0[t]] in out's dtype: the float32 stream (with a part's output still to be
    added) beside an earlier state of it."""
    _need(x, "stream_concat x", torch.float32, 2)
    _need(x0, "stream_concat x0", torch.float32, 2)
    _need(out, "stream_concat out", None, 2)
    n, width = x.shape
    if x0.shape != x.shape or tuple(out.shape) != (n, 2 * width):
        raise KernelError(f"stream_concat: x {tuple(x.shape)}, x0 {tuple(x0.shape)}, out {tuple(out.shape)}")
    if delta is not None:
        _need(delta, "stream_concat delta", out.dtype, 2)
        if delta.shape != x.shape:
            raise KernelError("stream_concat: delta differs from x in shape")
    _check(lib().mll_stream_concat(_ptr(x), _ptr(delta), _ptr(x0), _ptr(out), dtype_code(out.dtype), ctypes.c_int(n),
                                   ctypes.c_int(width), _stream()), "stream_concat")


def heads_gate(values: torch.Tensor, gate_rows: torch.Tensor, gate_col: int, out: torch.Tensor, n_heads: int, dv: int,
               per_head: bool, head_major: bool = False) -> None:
    """out[t, h * dv + i] = values(t, h, i) * sigmoid(gate_rows[t, gate_col + (h if per_head else h * dv + i)]).
    values is [T, H * dv], or [H, T, dv] with `head_major`; out [T, H * dv] may be values itself in the first case."""
    _need(values, "heads_gate values", None)
    _need(gate_rows, "heads_gate gate", values.dtype, 2)
    _need(out, "heads_gate out", values.dtype, 2)
    n = out.shape[0]
    if out.shape[1] != n_heads * dv or values.numel() != out.numel() or gate_rows.shape[0] != n:
        raise KernelError(f"heads_gate: values {tuple(values.shape)}, out {tuple(out.shape)} for {n_heads} heads of {dv}")
    if gate_col + (n_heads if per_head else n_heads * dv) > gate_rows.shape[1]:
        raise KernelError("heads_gate: the gate's columns lie outside its rows")
    if head_major and values.data_ptr() == out.data_ptr():
        raise KernelError("heads_gate: a head-major input cannot be gated in place")
    in_t, in_h = (dv, n * dv) if head_major else (n_heads * dv, dv)
    gate = ctypes.c_void_p(gate_rows.data_ptr() + gate_col * gate_rows.element_size())
    _check(lib().mll_heads_gate(_ptr(values), gate, _ptr(out), dtype_code(out.dtype), ctypes.c_int(n),
                                ctypes.c_int(n_heads), ctypes.c_int(dv), ctypes.c_longlong(in_t), ctypes.c_longlong(in_h),
                                ctypes.c_int(gate_rows.shape[1]), ctypes.c_int(int(per_head)), _stream()), "heads_gate")


def apply_row_norm(values: torch.Tensor, row_norm: RowNorm, out: torch.Tensor) -> None:
    """out = values * the rows' norm factors (bfloat16 [T, D]): finishes a norm that the product behind it
    cannot finish itself."""
    _need(values, "apply_row_norm values", torch.bfloat16, 2)
    _need(out, "apply_row_norm out", torch.bfloat16, 2)
    if out.shape != values.shape:
        raise KernelError(f"apply_row_norm: out {tuple(out.shape)} differs from values {tuple(values.shape)}")
    sumsq, partials, stride, eps = _row_norm_args(row_norm, values.shape[0], "apply_row_norm")
    _check(lib().mll_apply_row_norm(_ptr(values), sumsq, partials, stride, eps, _ptr(out),
                                    ctypes.c_int(values.shape[0]), ctypes.c_int(values.shape[1]), _stream()),
           "apply_row_norm")


def rope_cache_write(qkv, bias, cos, sin, tok_pos, tok_seq, seq_slot, block_table, q_out, k_cache, v_cache,
                     n_heads: int, n_kv_heads: int, head_dim: int, interleaved: bool,
                     write_kv: bool = True) -> None:
    """Rotate q and k of qkv [T, (Hq + 2 Hk) d], write q to q_out [T, Hq d] and k, v into the
    paged cache [n_pages, Hk, PAGE, d] at each token's slot and position."""
    _need(qkv, "rope qkv", None, 2)
    _need(q_out, "rope q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot)):
        _need(t, f"rope {name}", torch.int32, 1)
    _need(block_table, "rope block_table", torch.int32, 2)
    if tok_pos.shape[0] < n or tok_seq.shape[0] < n:
        raise KernelError("rope: token metadata shorter than the token count")
    if q_out.shape[0] < n or q_out.shape[1] != n_heads * head_dim:
        raise KernelError(f"rope: q_out {tuple(q_out.shape)} does not fit [{n}, {n_heads * head_dim}]")
    if cos is not None:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope: table {tuple(cos.shape)} does not match head_dim {head_dim}")
    if bias is not None:
        _need(bias, "rope bias", torch.float32, 1)
        if bias.shape[0] != qkv.shape[1]:
            raise KernelError("rope: bias length differs from the qkv width")
    if write_kv:
        _need(k_cache, "rope k_cache", qkv.dtype, 4)
        _need(v_cache, "rope v_cache", qkv.dtype, 4)
        want = (n_kv_heads, PAGE, head_dim)
        if tuple(k_cache.shape[1:]) != want or k_cache.shape != v_cache.shape:
            raise KernelError(f"rope: cache shape {tuple(k_cache.shape)} is not [pages, {want}]")
    _check(lib().mll_rope_cache(_ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(tok_pos), _ptr(tok_seq),
                                _ptr(seq_slot), _ptr(block_table), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                dtype_code(qkv.dtype), ctypes.c_int(n), ctypes.c_int(qkv.shape[1]),
                                ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                ctypes.c_int(block_table.shape[1]), ctypes.c_int(int(interleaved)),
                                ctypes.c_int(int(write_kv)), _stream()), "rope_cache_write")


def _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim):
    _need(q, "attention q", None, 2)
    _need(out, "attention out", q.dtype, 2)
    _need(k_cache, "attention k_cache", q.dtype, 4)
    _need(v_cache, "attention v_cache", q.dtype, 4)
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise KernelError(f"attention: head_dim {head_dim} is not a multiple of 16 in [16, 256]")
    if n_heads % n_kv_heads != 0:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
    if q.shape[1] != n_heads * head_dim or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention: q/out width differs from heads * head_dim")
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache shape {tuple(k_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim}]")


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(lib().mll_attn_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits))


USE_TENSOR_CORE_DECODE = True  # tests switch these off to reach the general kernels at every size
def _check_sink_values(sink_values, n_heads: int) -> None:
    if sink_values is not None:
        _need(sink_values, "attention sink values", torch.float32, 1)
        if sink_values.shape[0] != n_heads:
            raise KernelError(f"attention: {sink_values.shape[0]} sink values for {n_heads} heads")


def attention_decode_takes_window_extras(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether `attention_decode` would run the kernel that knows kept first tokens and capped scores."""
    return bool(USE_TMA_DECODE and USE_TENSOR_CORE_DECODE and dtype == torch.bfloat16
                and lib().mll_attn_decode_tma_supported(dtype_code(dtype), head_dim))


USE_TENSOR_CORE_PREFILL = True
USE_TCGEN05_PREFILL = True      # off: the mma.sync kernel takes the tensor-core prefill


def attention_decode(q, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch, out, n_seqs: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, n_splits: int, window: int,
                     scale: float, counters: Optional[torch.Tensor] = None, order: Optional[torch.Tensor] = None,
                     work: Optional[torch.Tensor] = None, chunk: int = 0, sink: bool = False,
                     sink_values: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: float = 0.0) -> None:
    """One query token per sequence (q row i belongs to sequence i) over the paged cache.
    `keep_first` (with a window) and `softcap`: the TMA-fed kernel only (ask `attention_decode_takes_window_extras`
    first) - keys below `keep_first` stay visible; a score s becomes softcap * tanh(s / softcap) after the scale.
    `sink` (bfloat16 tensor-core kernels only): one more term exp(0) in the softmax's denominator, or
    exp(sink_values[head]) with `sink_values` (float32 [Hq], not scaled).
    `chunk` > 0 (not together with a window): the query sees the keys of its own chunk of that many positions only,
    chunks counted from position 0; the kernels take it as a negative window.
    bfloat16 runs on tensor cores (head sizes 16 .. 256 in steps of 16), float32 on the general kernel.
    `order`: optional int32 permutation of the sequences, longest context first; the TMA-fed kernel starts its
    blocks in that order so that short sequences fill the end of the launch (the others ignore it)."""
    _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim)
    _check_sink_values(sink_values, n_heads)
    sink = bool(sink or sink_values is not None)
    if chunk:
        if chunk < 0 or window:
            raise KernelError("attention decode: a chunk must be positive and comes without a window")
        window = -chunk
    _need(seq_slot, "attention seq_slot", torch.int32, 1)
    _need(seq_ctx, "attention seq_ctx", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if q.shape[0] < n_seqs or out.shape[0] < n_seqs or seq_slot.shape[0] < n_seqs or seq_ctx.shape[0] < n_seqs:
        raise KernelError("attention decode: an input has fewer rows than sequences")
    if n_splits > 1:
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits):
            raise KernelError("attention decode: scratch too small for the split count")
    code = dtype_code(q.dtype)
    if counters is not None:
        _need(counters, "attention counters", torch.int32, 1)
        group = n_heads // n_kv_heads
        if counters.shape[0] < n_seqs * n_kv_heads * ((group + 15) // 16):
            raise KernelError("attention decode: counters shorter than sequences x kv heads x head chunks")
    if q.dtype == torch.bfloat16 and _tma_decode(q, None, None, None, False, False, k_cache, v_cache, seq_slot, seq_ctx,
                                                block_table, scratch, out, n_seqs, n_heads, n_kv_heads, head_dim,
                                                n_splits, window, scale, counters, _order(order, n_seqs), work,
                                                sink=sink, sink_values=sink_values, keep_first=keep_first, softcap=softcap):
        return
    if keep_first or softcap:
        raise KernelError("attention decode: only the TMA-fed kernel keeps first tokens or caps scores")
    if work is not None:
        raise KernelError("attention decode: a work list was given, but the kernel that takes one does not run here")
    if USE_TENSOR_CORE_DECODE and lib().mll_attn_decode_mma_supported(code, head_dim):
        _check(lib().mll_attn_decode_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                         _ptr(block_table), _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs),
                                         ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                         ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits),
                                         ctypes.c_int(window), ctypes.c_float(scale),
                                         _ptr(counters if n_splits > 1 else None), ctypes.c_int(int(sink)),
                                         _ptr(sink_values), _stream()),
               "attention_decode (tensor cores)")
        if n_splits > 1 and counters is None:
            _check(lib().mll_attn_combine(_ptr(scratch), _ptr(out), code, ctypes.c_int(n_seqs), ctypes.c_int(n_heads),
                                          ctypes.c_int(head_dim), ctypes.c_int(n_splits), _stream()),
                   "attention_combine")
        return
    if sink:
        raise KernelError("attention decode: only the tensor-core kernels have a sink")
    _check(lib().mll_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                 _ptr(block_table), _ptr(scratch), _ptr(out), code,
                                 ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
                                 ctypes.c_int(head_dim), ctypes.c_int(block_table.shape[1]),
                                 ctypes.c_int(n_splits), ctypes.c_int(window), ctypes.c_float(scale),
                                 _stream()), "attention_decode", kernels=2 if n_splits > 1 else 1)


USE_FUSED_DECODE = True  # off: rotary encoding and cache write stay a kernel of their own in decode steps
USE_TMA_DECODE = True    # off: the cp.async / mma.sync decode kernel also takes head sizes 64 and 128
USE_CLUSTER_MERGE = True  # off: the TMA decode kernel merges its context splits through global memory and counters


def _order(order, n_seqs: int):
    if order is not None:
        _need(order, "attention order", torch.int32, 1)
        if order.shape[0] < n_seqs:
            raise KernelError("attention decode: the order is shorter than the batch")
    return order


WORK_LIST_MAX_SPLITS = 32  # splits a sequence of a work list can have (the stride of the partial results)


def decode_work_entry(sequence: int, split: int, n_splits: int) -> int:
    """One place of a decode work list: block `split` of the `n_splits` that `sequence` is cut into."""
    return sequence | (split << 16) | (n_splits << 24)


def _work(work, n_seqs: int, n_splits: int):
    if work is not None:
        _need(work, "attention work list", torch.int32, 1)
        if work.shape[0] < n_seqs or work.shape[0] > 65535 or n_seqs > 65535:
            raise KernelError(f"attention decode: a work list of {work.shape[0]} places for {n_seqs} sequences")
        if n_splits > 127:
            raise KernelError("attention decode: a work list takes at most 127 splits a sequence")
    return work


def _tma_decode(q, qkv, cos, sin, interleaved, write_kv, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch, out,
                n_seqs, n_heads, n_kv_heads, head_dim, n_splits, window, scale, counters, order=None, work=None,
                sink: bool = False, sink_values: Optional[torch.Tensor] = None, keep_first: int = 0,
                softcap: float = 0.0) -> bool:
    """Runs the TMA-fed decode kernel when it takes the problem (bfloat16, head_dim 64/128, arrival
    counters whenever the context is split); returns whether it did."""
    if not (USE_TMA_DECODE and USE_TENSOR_CORE_DECODE and lib().mll_attn_decode_tma_supported(dtype_code(out.dtype), head_dim)):
        return False
    if n_splits > 1 and counters is None:
        return False
    work = _work(work, n_seqs, n_splits)
    _check(lib().mll_attn_decode_tma(_ptr(q), _ptr(qkv), ctypes.c_int(qkv.shape[1] if qkv is not None else 0),
                                     _ptr(cos), _ptr(sin), ctypes.c_int(int(interleaved)), ctypes.c_int(int(write_kv)),
                                     _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]), _ptr(seq_slot),
                                     _ptr(seq_ctx), _ptr(block_table), _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs),
                                     ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                     ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits), ctypes.c_int(window),
                                     ctypes.c_float(scale), _ptr(counters if n_splits > 1 else None),
                                     ctypes.c_int(int(USE_CLUSTER_MERGE)), _ptr(order), _ptr(work),
                                     ctypes.c_int(work.shape[0] if work is not None else 0), ctypes.c_int(int(sink)),
                                     _ptr(sink_values), ctypes.c_int(keep_first), ctypes.c_float(softcap), _stream()),
           "attention_decode (TMA, work list)" if work is not None
           else "attention_decode (TMA, cluster merge)" if USE_CLUSTER_MERGE and 2 <= n_splits <= 16
           else "attention_decode (TMA)")
    return True


_cluster_capacity = {}


def attention_decode_cluster_capacity(dtype: torch.dtype, head_dim: int, fused: bool):
    """capacity[s], s = 0 .. 16: how many clusters of s blocks of the TMA decode kernel the device holds at once
    (0: no such cluster), or None when that kernel or its cluster merge is not what runs for this dtype and
    head size.  A launch with more clusters than that runs in two waves; measured on B200 at 8 kv heads of
    128, contexts of 128 .. 2,048: 3 sequences with 12 splits (24 clusters, 21 fit) 14.2 us, with 10 splits
    8.8 us; 4 sequences 9 / 8 splits 14.4 / 9.1 us; 5 sequences 7 / 6 splits 15.1 / 9.9 us."""
    if not (USE_TMA_DECODE and USE_TENSOR_CORE_DECODE and USE_CLUSTER_MERGE and dtype == torch.bfloat16
            and lib().mll_attn_decode_tma_supported(dtype_code(dtype), head_dim)):
        return None
    key = (head_dim, bool(fused))
    if key not in _cluster_capacity:
        _cluster_capacity[key] = (0, 0) + tuple(
            int(lib().mll_attn_decode_tma_resident_clusters(ctypes.c_int(head_dim), ctypes.c_int(int(fused)), ctypes.c_int(s)))
            for s in range(2, 17))
    return _cluster_capacity[key]


def attention_decode_fused_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether a decode step's rotary encoding, cache write and attention can be one launch."""
    return bool(USE_FUSED_DECODE and USE_TENSOR_CORE_DECODE
                and lib().mll_attn_decode_mma_supported(dtype_code(dtype), head_dim))


def attention_decode_fused(qkv, cos, sin, interleaved: bool, write_kv: bool, k_cache, v_cache, seq_slot, seq_ctx,
                           block_table, scratch, out, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
                           n_splits: int, window: int, scale: float, counters: Optional[torch.Tensor] = None,
                           order: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> None:
    """Decode step: row i of qkv [B, (Hq + 2 Hk) d] is sequence i's new token at position seq_ctx[i] - 1.
    Rotates q and k (tables as for rope_cache_write, or None), writes k and v into the paged cache and
    attends over it, in one launch (bfloat16, head sizes 16 .. 256 in steps of 16).
    `work`: int32 list of `decode_work_entry` places (-1: unused) that gives every sequence its own number of
    splits, long ones more than short ones; n_splits is then the most any has (the TMA-fed kernel only)."""
    _need(qkv, "attention qkv", torch.bfloat16, 2)
    _need(out, "attention out", torch.bfloat16, 2)
    _need(k_cache, "attention k_cache", torch.bfloat16, 4)
    _need(v_cache, "attention v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache shape {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim:
        raise KernelError("attention decode (fused): qkv/out width differs from the heads")
    for name, t in (("seq_slot", seq_slot), ("seq_ctx", seq_ctx)):
        _need(t, f"attention {name}", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if min(qkv.shape[0], out.shape[0], seq_slot.shape[0], seq_ctx.shape[0]) < n_seqs:
        raise KernelError("attention decode (fused): an input has fewer rows than sequences")
    if cos is not None:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope: table {tuple(cos.shape)} does not match head_dim {head_dim}")
    if n_splits > 1:
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits):
            raise KernelError("attention decode: scratch too small for the split count")
        if counters is None:
            raise KernelError("attention decode (fused): splits need arrival counters")
        _need(counters, "attention counters", torch.int32, 1)
        if counters.shape[0] < n_seqs * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16):
            raise KernelError("attention decode: counters shorter than sequences x kv heads x head chunks")
    if _tma_decode(None, qkv, cos, sin, interleaved, write_kv, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch,
                   out, n_seqs, n_heads, n_kv_heads, head_dim, n_splits, window, scale, counters, _order(order, n_seqs), work):
        return
    if work is not None:
        raise KernelError("attention decode: a work list was given, but the kernel that takes one does not run here")
    _check(lib().mll_attn_decode_mma_fused(_ptr(qkv), ctypes.c_int(qkv.shape[1]), _ptr(cos), _ptr(sin),
                                           ctypes.c_int(int(interleaved)), ctypes.c_int(int(write_kv)), _ptr(k_cache),
                                           _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx), _ptr(block_table),
                                           _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs), ctypes.c_int(n_heads),
                                           ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                           ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits),
                                           ctypes.c_int(window), ctypes.c_float(scale),
                                           _ptr(counters if n_splits > 1 else None), _stream()),
           "attention_decode (fused)")


PREFILL_TILE = 64  # query rows per entry of the work list that `attention_prefill` takes


def attention_prefill_takes_chunks(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether `attention_prefill` would run the kernel that knows the chunk mask (bfloat16, heads of 64 or 128)."""
    return bool(USE_TENSOR_CORE_PREFILL and USE_TCGEN05_PREFILL and dtype in _DTYPE_CODE
                and lib().mll_attn_prefill_tc5_supported(dtype_code(dtype), head_dim))


def attention_prefill(q, k_cache, v_cache, seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0,
                      block_table, out, n_tiles: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      window: int, scale: float, wide_tiles=None, chunk: int = 0, sink: bool = False,
                      sink_values: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: float = 0.0) -> None:
    """Tiles of up to 64 query tokens of sequences with unequal lengths over the paged cache.
    `wide_tiles`: (sequence, first row) int32 lists of the same rows in tiles of 128, which the tcgen05 kernel
    works on; without them it walks the 64-row list and every other block finds nothing to do.
    `chunk` > 0 (the tcgen05 kernel only; ask `attention_prefill_takes_chunks` first): key j is visible from query i
    only if j // chunk == i // chunk.  `sink` (the same kernel only): one more term exp(0) in the softmax's denominator,
    or exp(sink_values[head]) with `sink_values` (float32 [Hq], not scaled).  `keep_first` (with a window) and
    `softcap` (the same kernel only): keys below `keep_first` stay visible; a score s becomes softcap * tanh(s / softcap)
    after the scale."""
    _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim)
    _check_sink_values(sink_values, n_heads)
    sink = bool(sink or sink_values is not None)
    for name, t in (("seq_slot", seq_slot), ("seq_ctx", seq_ctx), ("seq_qstart", seq_qstart),
                    ("seq_qlen", seq_qlen), ("tile_seq", tile_seq), ("tile_row0", tile_row0)):
        _need(t, f"attention {name}", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if tile_seq.shape[0] < n_tiles or tile_row0.shape[0] < n_tiles:
        raise KernelError("attention prefill: tile lists shorter than the tile count")
    if (USE_TENSOR_CORE_PREFILL and USE_TCGEN05_PREFILL
            and lib().mll_attn_prefill_tc5_supported(dtype_code(q.dtype), head_dim)):
        if wide_tiles is not None:
            tile_seq, tile_row0 = wide_tiles
            _need(tile_seq, "attention wide tile_seq", torch.int32, 1)
            _need(tile_row0, "attention wide tile_row0", torch.int32, 1)
            n_tiles = tile_seq.shape[0]
            if tile_row0.shape[0] != n_tiles:
                raise KernelError("attention prefill: the wide tile lists differ in length")
        _check(lib().mll_attn_prefill_tc5(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                          _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                          _ptr(block_table), _ptr(out), ctypes.c_int(q.shape[0]),
                                          ctypes.c_longlong(k_cache.shape[0]), ctypes.c_int(n_tiles),
                                          ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                          ctypes.c_int(block_table.shape[1]), ctypes.c_int(window), ctypes.c_int(chunk),
                                          ctypes.c_float(scale), ctypes.c_int(int(sink)), _ptr(sink_values),
                                          ctypes.c_int(keep_first), ctypes.c_float(softcap), _stream()),
               "attention_prefill (tcgen05)")
        return
    if chunk or sink or keep_first or softcap:
        raise KernelError("attention prefill: only the tcgen05 kernel masks by chunks, has a sink, keeps first tokens or caps scores")
    if USE_TENSOR_CORE_PREFILL and lib().mll_attn_prefill_mma_supported(dtype_code(q.dtype), head_dim):
        _check(lib().mll_attn_prefill_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                          _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                          _ptr(block_table), _ptr(out), ctypes.c_int(n_tiles), ctypes.c_int(n_heads),
                                          ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                          ctypes.c_int(block_table.shape[1]), ctypes.c_int(window),
                                          ctypes.c_float(scale), _stream()), "attention_prefill (tensor cores)")
        return
    _check(lib().mll_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                  _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                  _ptr(block_table), _ptr(out), dtype_code(q.dtype), ctypes.c_int(n_tiles),
                                  ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                  ctypes.c_int(block_table.shape[1]), ctypes.c_int(window),
                                  ctypes.c_float(scale), _stream()), "attention_prefill")


def argmax(logits: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    """tokens[r] = first index of the maximum of logits[r]; status[r] = 1 if a logit is not finite."""
    _need(logits, "argmax logits", torch.float32, 2)
    _need(tokens, "argmax tokens", torch.int32, 1)
    _need(status, "argmax status", torch.int32, 1)
    n = logits.shape[0]
    if tokens.shape[0] < n or status.shape[0] < n:
        raise KernelError("argmax: outputs shorter than the row count")
    _check(lib().mll_argmax(_ptr(logits), ctypes.c_int(n), ctypes.c_int(logits.shape[1]), _ptr(tokens),
                            _ptr(status), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, request: torch.Tensor,
           step: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    """Temperature (top_k == 0) or top-k sampling with u = f(seed, request[r], step[r])."""
    _need(logits, "sample logits", torch.float32, 2)
    for name, t in (("request", request), ("step", step), ("tokens", tokens), ("status", status)):
        _need(t, f"sample {name}", torch.int32, 1)
        if t.shape[0] < logits.shape[0]:
            raise KernelError(f"sample: {name} shorter than the row count")
    _check(lib().mll_sample(_ptr(logits), ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]),
                            ctypes.c_float(temperature), ctypes.c_int(top_k),
                            ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(request), _ptr(step),
                            _ptr(tokens), _ptr(status), _stream()), "sample")


# --------------------------------------------------------------------------- #
# attention with head sizes of its own for keys and values, chunks, partial rotation
# --------------------------------------------------------------------------- #
def local_attention_prepare(qkv, q_weight, k_weight, cos, sin, tok_pos, tok_seq, seq_slot, block_table, q_out,
                            k_cache, v_cache, n_heads: int, n_kv_heads: int, d: int, dv: int, rot: int,
                            interleaved: bool, eps: float, q_temp=None, v_from_k: bool = False,
                            write_kv: bool = True) -> None:
    """qkv [T, ld] (q heads of d, k heads of d, v heads of dv; `v_from_k`: no v columns - the values are the keys as
    projected, before norm and rotation, and dv == d): q and k each divided by the root mean square of
    their whole projection and multiplied by `q_weight` / `k_weight` (float32; both None: no norm), the first
    `rot` dimensions of every q and k head rotated, q to `q_out` [T, Hq * d], k and v into the cache pages
    ([pages, Hk, PAGE, d] and [pages, Hk, PAGE, dv]).  `q_temp` = (coef, every): q at position p is also
    multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).  `write_kv` False: the rows hold queries only and
    nothing goes to the cache (a layer that reads another layer's keys and values)."""
    _need(qkv, "local attention qkv", None, 2)
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if q_temp and every < 1:
        raise KernelError(f"local attention: a query temperature every {every} positions")
    _need(q_out, "local attention q", qkv.dtype, 2)
    _need(k_cache, "local attention k cache", qkv.dtype, 4)
    _need(v_cache, "local attention v cache", qkv.dtype, 4)
    n = qkv.shape[0]
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, d) or tuple(v_cache.shape[1:]) != (n_kv_heads, PAGE, dv):
        raise KernelError(f"local attention: caches {tuple(k_cache.shape)} / {tuple(v_cache.shape)} do not fit "
                          f"{n_kv_heads} heads of {d} / {dv}")
    if tuple(q_out.shape) != (n, n_heads * d):
        raise KernelError(f"local attention: q out {tuple(q_out.shape)}, expected {(n, n_heads * d)}")
    for name, w, size in (("q", q_weight, n_heads * d), ("k", k_weight, n_kv_heads * d)):
        if w is not None:
            _need(w, f"local attention {name} norm weight", torch.float32, 1)
            if w.shape[0] != size:
                raise KernelError(f"local attention: {name} norm weight of {w.shape[0]}, expected {size}")
    if rot:
        _need(cos, "local attention cos", torch.float32, 2)
        _need(sin, "local attention sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError(f"local attention: rotary table {tuple(cos.shape)} for {rot} rotated dimensions")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot)):
        _need(t, f"local attention {name}", torch.int32, 1)
    _need(block_table, "local attention block table", torch.int32, 2)
    _check(lib().mll_local_attention_prepare(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos if rot else None), _ptr(sin if rot else None),
        _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot), _ptr(block_table), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
        dtype_code(qkv.dtype), ctypes.c_int(n), ctypes.c_int(qkv.shape[1]), ctypes.c_int(n_heads),
        ctypes.c_int(n_kv_heads), ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(rot), ctypes.c_int(int(interleaved)),
        ctypes.c_int(block_table.shape[1]), ctypes.c_float(eps), ctypes.c_float(coef), ctypes.c_int(every),
        ctypes.c_int(int(v_from_k)), ctypes.c_int(int(write_kv)), _stream()),
        "local_attention_prepare")


def _check_local_caches(k_cache, v_cache, n_kv_heads: int, d: int, dv: int, v_in_k: bool) -> None:
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, d):
        raise KernelError(f"local attention: key cache {tuple(k_cache.shape)} does not fit {n_kv_heads} heads of {d}")
    if v_in_k:
        if v_cache.data_ptr() != k_cache.data_ptr() or dv > d:
            raise KernelError("local attention: values inside the keys need the key cache itself and dv <= d")
    elif tuple(v_cache.shape[1:]) != (n_kv_heads, PAGE, dv):
        raise KernelError(f"local attention: value cache {tuple(v_cache.shape)} does not fit {n_kv_heads} heads of {dv}")


def local_attention(q, k_cache, v_cache, tok_pos, tok_seq, seq_slot, block_table, out, n_heads: int, n_kv_heads: int,
                    d: int, dv: int, chunk: int, window: int, scale: float, sink: bool = False,
                    v_in_k: bool = False, sink_values: Optional[torch.Tensor] = None, keep_first: int = 0,
                    softcap: float = 0.0) -> None:
    """out [T, Hq * dv] = softmax(scale * q . k) v over the keys j <= i of the query's own chunk (j // chunk ==
    i // chunk; chunk 0: all) and window (j > i - window; 0: none); the step's own keys are in the cache already.
    `sink`: the softmax's denominator has one more term exp(0), or exp(sink_values[head]) with `sink_values` (float32
    [Hq], not scaled).  `v_in_k`: the values are the leading dv columns of the key rows (v_cache is k_cache).
    `keep_first`: with a window, keys j < keep_first stay visible.  `softcap` > 0: a score s becomes
    softcap * tanh(s / softcap) after the scale."""
    _need(q, "local attention q", None, 2)
    _check_sink_values(sink_values, n_heads)
    _need(out, "local attention out", q.dtype, 2)
    _need(k_cache, "local attention k cache", q.dtype, 4)
    _need(v_cache, "local attention v cache", q.dtype, 4)
    n = q.shape[0]
    if tuple(q.shape) != (n, n_heads * d) or tuple(out.shape) != (n, n_heads * dv):
        raise KernelError(f"local attention: q {tuple(q.shape)} / out {tuple(out.shape)} for {n_heads} heads of {d} / {dv}")
    _check_local_caches(k_cache, v_cache, n_kv_heads, d, dv, v_in_k)
    _check(lib().mll_local_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot), _ptr(block_table),
        _ptr(out), dtype_code(q.dtype), ctypes.c_int(n), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
        ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(chunk), ctypes.c_int(window),
        ctypes.c_int(block_table.shape[1]), ctypes.c_float(scale), ctypes.c_int(int(sink)), _ptr(sink_values),
        ctypes.c_int(int(v_in_k)), ctypes.c_int(keep_first), ctypes.c_float(softcap), _stream()), "local_attention")


USE_TENSOR_CORE_LOCAL = True  # tests switch it off to reach the general kernel in bfloat16 prompt steps


def local_attention_mma_supported(dtype: torch.dtype, d: int, dv: int) -> bool:
    return USE_TENSOR_CORE_LOCAL and dtype == torch.bfloat16 and bool(
        lib().mll_local_attention_mma_supported(dtype_code(dtype), d, dv))


def local_attention_tiles(q, k_cache, v_cache, seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0,
                          block_table, out, n_heads: int, n_kv_heads: int, d: int, dv: int, chunk: int, window: int,
                          scale: float, sink: bool = False, v_in_k: bool = False,
                          sink_values: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: float = 0.0) -> None:
    """`local_attention` for prompt steps in bfloat16 on tensor cores: the work is a list of tiles of up to
    PREFILL_TILE query rows, (sequence, first row among the sequence's new tokens)."""
    _need(q, "local attention q", torch.bfloat16, 2)
    _need(out, "local attention out", torch.bfloat16, 2)
    _need(k_cache, "local attention k cache", torch.bfloat16, 4)
    _need(v_cache, "local attention v cache", torch.bfloat16, 4)
    n = q.shape[0]
    if tuple(q.shape) != (n, n_heads * d) or tuple(out.shape) != (n, n_heads * dv):
        raise KernelError(f"local attention: q {tuple(q.shape)} / out {tuple(out.shape)} for {n_heads} heads of {d} / {dv}")
    _check_local_caches(k_cache, v_cache, n_kv_heads, d, dv, v_in_k)
    for name, t in (("tile_seq", tile_seq), ("tile_row0", tile_row0)):
        _need(t, f"local attention {name}", torch.int32, 1)
    if tile_seq.shape != tile_row0.shape:
        raise KernelError("local attention: the tile lists differ in length")
    _check(lib().mll_local_attention_mma(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx), _ptr(seq_qstart), _ptr(seq_qlen),
        _ptr(tile_seq), _ptr(tile_row0), _ptr(block_table), _ptr(out), ctypes.c_int(tile_seq.shape[0]),
        ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(chunk),
        ctypes.c_int(window), ctypes.c_int(block_table.shape[1]), ctypes.c_float(scale), ctypes.c_int(int(sink)),
        _ptr(sink_values), ctypes.c_int(int(v_in_k)), ctypes.c_int(0), ctypes.c_int(1), _ptr(None),
        ctypes.c_int(keep_first), ctypes.c_float(softcap), _stream()),
        "local_attention_mma (window)" if keep_first or softcap else "local_attention_mma")


def local_attention_heads(q, k_cache, v_cache, seq_slot, seq_ctx, seq_qstart, seq_qlen, block_table, out, n_seqs: int,
                          n_heads: int, n_kv_heads: int, d: int, dv: int, chunk: int, window: int, scale: float,
                          sink: bool = False, v_in_k: bool = False, n_splits: int = 1,
                          scratch: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None,
                          keep_first: int = 0, softcap: float = 0.0) -> None:
    """`local_attention` for steps in which every sequence brings one token, bfloat16, on tensor cores: a block per
    (sequence, kv head) whose rows are the query heads of that kv head's group.  `n_splits` > 1: that many blocks
    along every context and a merge; `scratch` float32 of `local_attention_heads_scratch` floats."""
    if n_splits > 1:
        _need(scratch, "local attention scratch", torch.float32)
        if scratch.numel() < local_attention_heads_scratch(n_seqs, n_heads, dv, n_splits):
            raise KernelError("local attention: scratch too small for the split count")
    _need(q, "local attention q", torch.bfloat16, 2)
    _need(out, "local attention out", torch.bfloat16, 2)
    _need(k_cache, "local attention k cache", torch.bfloat16, 4)
    _need(v_cache, "local attention v cache", torch.bfloat16, 4)
    if tuple(q.shape) != (n_seqs, n_heads * d) or tuple(out.shape) != (n_seqs, n_heads * dv):
        raise KernelError(f"local attention: q {tuple(q.shape)} / out {tuple(out.shape)} for {n_seqs} single tokens")
    _check_local_caches(k_cache, v_cache, n_kv_heads, d, dv, v_in_k)
    _check(lib().mll_local_attention_mma(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx), _ptr(seq_qstart), _ptr(seq_qlen),
        _ptr(seq_slot), _ptr(seq_slot), _ptr(block_table), _ptr(out), ctypes.c_int(n_seqs),
        ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(chunk),
        ctypes.c_int(window), ctypes.c_int(block_table.shape[1]), ctypes.c_float(scale), ctypes.c_int(int(sink)),
        _ptr(sink_values), ctypes.c_int(int(v_in_k)), ctypes.c_int(1), ctypes.c_int(n_splits),
        _ptr(scratch if n_splits > 1 else None), ctypes.c_int(keep_first), ctypes.c_float(softcap), _stream()),
        "local_attention_heads (window)" if keep_first or softcap else "local_attention_heads", kernels=2 if n_splits > 1 else 1)


def local_attention_heads_scratch(n_seqs: int, n_heads: int, dv: int, n_splits: int) -> int:
    return n_seqs * n_heads * n_splits * (dv + 2)


def local_attention_heads_splits(n_seqs: int, blocks_per_seq: int, multiprocessors: int) -> int:
    """Context splits of a single-token step: enough blocks for two a multiprocessor, at most 16 a sequence; a
    function of the batch size alone, so that a captured step keeps its launch."""
    want = -(-2 * max(multiprocessors, 1) // max(n_seqs * blocks_per_seq, 1))
    return max(1, min(16, want))


# --------------------------------------------------------------------------- #
# mixers with a matrix-valued state per sequence and head
# --------------------------------------------------------------------------- #
def retention_prepare(proj, cos, sin, tok_pos, q, k, v, n_heads: int, d: int, dv: int, rot: int, interleaved: bool,
                      k_scale: float) -> None:
    """proj [T, ld] (q heads of d, k heads of d, v heads of dv, ...) -> float32 q, k [T, H, d] with the first `rot`
    dimensions of every head rotated and k * k_scale, v [T, H, dv]."""
    _need(proj, "retention proj", None, 2)
    n = proj.shape[0]
    for name, t, width in (("q", q, n_heads * d), ("k", k, n_heads * d), ("v", v, n_heads * dv)):
        _need(t, f"retention {name}", torch.float32, 2)
        if tuple(t.shape) != (n, width):
            raise KernelError(f"retention prepare: {name} {tuple(t.shape)}, expected {(n, width)}")
    if rot:
        _need(cos, "retention cos", torch.float32, 2)
        _need(sin, "retention sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError(f"retention prepare: rotary table {tuple(cos.shape)} for {rot} rotated dimensions")
    _need(tok_pos, "retention tok_pos", torch.int32, 1)
    _check(lib().mll_retention_prepare(
        _ptr(proj), _ptr(cos if rot else None), _ptr(sin if rot else None), _ptr(tok_pos), _ptr(q), _ptr(k), _ptr(v),
        dtype_code(proj.dtype), ctypes.c_int(n), ctypes.c_int(proj.shape[1]), ctypes.c_int(n_heads), ctypes.c_int(d),
        ctypes.c_int(dv), ctypes.c_int(rot), ctypes.c_int(int(interleaved)), ctypes.c_float(k_scale), _stream()),
        "retention_prepare")


def delta_prepare(proj, rate, conv_w, conv_state, a_log, dt_bias, tok_seq, seq_slot, seq_qstart, q, k, v, g, beta,
                  n_heads: int, n_kv_heads: int, d: int, dv: int, taps: int, unit_eps: float) -> None:
    """The inputs of the gated delta rule from the projections of a step (see csrc/recurrent.cu): proj [T, ld]
    holds q, k (G heads of d), v (H heads of dv) and beta's pre-activation (H); rate float32 [T, >= H * d] the
    decay's; conv_w float32 [C, taps]; conv_state float32 [slots, taps - 1, C]."""
    _need(proj, "delta proj", None, 2)
    _need(rate, "delta rate", torch.float32, 2)
    _need(conv_w, "delta conv weights", torch.float32, 2)
    _need(conv_state, "delta conv state", torch.float32, 3)
    _need(a_log, "delta A_log", torch.float32, 1)
    _need(dt_bias, "delta dt_bias", torch.float32, 1)
    n = proj.shape[0]
    C = 2 * n_kv_heads * d + n_heads * dv
    if tuple(conv_w.shape) != (C, taps) or tuple(conv_state.shape[1:]) != (max(taps - 1, 0), C):
        raise KernelError(f"delta prepare: conv weights {tuple(conv_w.shape)} / state {tuple(conv_state.shape)} "
                          f"for {C} channels of {taps} taps")
    if a_log.shape[0] != n_heads or dt_bias.shape[0] != n_heads * d or rate.shape[0] != n:
        raise KernelError("delta prepare: A_log, dt_bias or rate of the wrong size")
    for name, t, width in (("q", q, n_kv_heads * d), ("k", k, n_kv_heads * d), ("v", v, n_heads * dv),
                           ("g", g, n_heads * d), ("beta", beta, n_heads)):
        _need(t, f"delta {name}", torch.float32, 2)
        if tuple(t.shape) != (n, width):
            raise KernelError(f"delta prepare: {name} {tuple(t.shape)}, expected {(n, width)}")
    _check(lib().mll_delta_prepare(
        _ptr(proj), _ptr(rate), _ptr(conv_w), _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(tok_seq),
        _ptr(seq_slot), _ptr(seq_qstart), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), dtype_code(proj.dtype),
        ctypes.c_int(n), ctypes.c_int(proj.shape[1]), ctypes.c_int(rate.shape[1]), ctypes.c_int(n_heads),
        ctypes.c_int(n_kv_heads), ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(taps), ctypes.c_float(unit_eps),
        _stream()), "delta_prepare")


def conv_state_update(proj, conv_state, seq_slot, seq_qstart, seq_qlen, n_seqs: int, channels: int, taps: int,
                      first_column: int = 0) -> None:
    """conv_state[slot] <- the last taps - 1 rows of (conv_state[slot], this step's rows of
    proj[:, first_column:first_column + channels])."""
    _need(proj, "conv state proj", None, 2)
    _need(conv_state, "conv state", torch.float32, 3)
    if tuple(conv_state.shape[1:]) != (max(taps - 1, 0), channels):
        raise KernelError(f"conv state update: state {tuple(conv_state.shape)} for {channels} channels of {taps} taps")
    _check(lib().mll_conv_state_update(
        _ptr(proj), dtype_code(proj.dtype), ctypes.c_int(first_column), ctypes.c_int(proj.shape[1]), _ptr(conv_state),
        _ptr(seq_slot),
        _ptr(seq_qstart), _ptr(seq_qlen), ctypes.c_int(n_seqs), ctypes.c_int(channels), ctypes.c_int(taps), _stream()),
        "conv_state_update")


def state_scan(q, k, v, g, beta, head_decay, state, out, seq_slot, seq_qstart, seq_qlen, n_seqs: int, n_heads: int,
               n_kv_heads: int, d: int, dv: int, token_decay: Optional[torch.Tensor] = None) -> None:
    """The recurrence S <- decay S + k u^T, o = S^T q over each sequence's tokens of the step, from and to
    state [slots, H, d, dv] (float32).  With g [T, H * d] and beta [T, H]: the gated delta rule
    (u = beta (v - S^T k) after the decay); with g alone: a decay per key channel and u = v; with `token_decay`
    float32 [T, H]: one decay per token and head and u = v; else head_decay float32 [H] and u = v."""
    n = q.shape[0]
    delta = g is not None and beta is not None
    channel = g is not None and beta is None
    per_token = token_decay is not None
    if per_token and (g is not None or beta is not None or head_decay is not None):
        raise KernelError("state scan: a decay per token and head stands alone")
    for name, t, width in (("q", q, n_kv_heads * d), ("k", k, n_kv_heads * d), ("v", v, n_heads * dv),
                           ("out", out, n_heads * dv)):
        _need(t, f"state scan {name}", torch.float32, 2)
        if tuple(t.shape) != (n, width):
            raise KernelError(f"state scan: {name} {tuple(t.shape)}, expected {(n, width)}")
    _need(state, "state scan state", torch.float32, 4)
    if tuple(state.shape[1:]) != (n_heads, d, dv):
        raise KernelError(f"state scan: state {tuple(state.shape)} for {n_heads} heads of {d} x {dv}")
    if delta:
        _need(g, "state scan g", torch.float32, 2)
        _need(beta, "state scan beta", torch.float32, 2)
        if tuple(g.shape) != (n, n_heads * d) or tuple(beta.shape) != (n, n_heads):
            raise KernelError("state scan: g or beta of the wrong size")
    elif channel:
        _need(g, "state scan g", torch.float32, 2)
        if tuple(g.shape) != (n, n_heads * d):
            raise KernelError("state scan: g of the wrong size")
    elif per_token:
        _need(token_decay, "state scan token decay", torch.float32, 2)
        if tuple(token_decay.shape) != (n, n_heads):
            raise KernelError("state scan: one decay per token and head is needed")
        beta = token_decay  # it travels where the delta rule's beta does
    else:
        _need(head_decay, "state scan decay", torch.float32, 1)
        if head_decay.shape[0] != n_heads:
            raise KernelError("state scan: one decay per head is needed")
    _check(lib().mll_state_scan(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(head_decay), _ptr(state), _ptr(out), _ptr(seq_slot),
        _ptr(seq_qstart), _ptr(seq_qlen), ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
        ctypes.c_int(d), ctypes.c_int(dv), ctypes.c_int(1 if delta else (2 if channel else (3 if per_token else 0))),
        _stream()),
        "state_scan (delta rule)" if delta else ("state_scan (channel decay)" if channel else
                                                 ("state_scan (token decay)" if per_token else "state_scan (retention)")))


def ssd_prepare(proj, conv_w, conv_b, conv_state, a_log, dt_bias, tok_seq, seq_slot, seq_qstart, q, k, u, xs, decay,
                n_heads: int, n_groups: int, d: int, dv: int, taps: int) -> None:
    """The inputs of a state-space layer from the projection of a step: a row of proj [T, ld] holds z (H dv), x (H dv),
    B (G d), C (G d) and dt (H).  x, B and C pass a causal convolution over time (conv_w float32 [C, taps], conv_b
    [C], the inputs before the step from conv_state float32 [slots, taps - 1, C]) and silu; dt = softplus(dt +
    dt_bias).  Float32 outputs: q = C and k = B [T, G d], xs = x and u = dt x [T, H dv], decay = exp(-exp(a_log) dt)
    [T, H]."""
    _need(proj, "ssd proj", None, 2)
    n = proj.shape[0]
    inner, gn = n_heads * dv, n_groups * d
    C = inner + 2 * gn
    for name, t, shape in (("conv weights", conv_w, (C, taps)), ("conv bias", conv_b, (C,)), ("A_log", a_log, (n_heads,)),
                           ("dt_bias", dt_bias, (n_heads,)), ("q", q, (n, gn)), ("k", k, (n, gn)), ("u", u, (n, inner)),
                           ("xs", xs, (n, inner)), ("decay", decay, (n, n_heads))):
        _need(t, f"ssd {name}", torch.float32)
        if tuple(t.shape) != shape:
            raise KernelError(f"ssd prepare: {name} {tuple(t.shape)}, expected {shape}")
    _need(conv_state, "ssd conv state", torch.float32, 3)
    if tuple(conv_state.shape[1:]) != (max(taps - 1, 0), C):
        raise KernelError(f"ssd prepare: conv state {tuple(conv_state.shape)} for {C} channels of {taps} taps")
    if proj.shape[1] < 2 * inner + 2 * gn + n_heads:
        raise KernelError(f"ssd prepare: rows of {proj.shape[1]} columns are too short")
    _check(lib().mll_ssd_prepare(
        _ptr(proj), _ptr(conv_w), _ptr(conv_b), _ptr(conv_state), _ptr(a_log), _ptr(dt_bias), _ptr(tok_seq),
        _ptr(seq_slot), _ptr(seq_qstart), _ptr(q), _ptr(k), _ptr(u), _ptr(xs), _ptr(decay), dtype_code(proj.dtype),
        ctypes.c_int(n), ctypes.c_int(proj.shape[1]), ctypes.c_int(n_heads), ctypes.c_int(n_groups), ctypes.c_int(d),
        ctypes.c_int(dv), ctypes.c_int(taps), _stream()), "ssd_prepare")


def gated_group_norm(o, xs, skip, gate, weight, out, dv: int, parts: int, eps: float) -> None:
    """out = y / sqrt(mean(y^2) + eps) * weight over each of `parts` equal pieces of a row, with
    y = (o + skip[head] * xs) * silu(gate[:, :width]); o, xs float32 [T, width], skip float32 [width / dv] (both None:
    no skip), gate [T, >= width] and out [T, width] in the run's dtype, weight float32 [width]."""
    _need(o, "gated group norm o", torch.float32, 2)
    n, width = o.shape
    _need(gate, "gated group norm gate", None, 2)
    _need(out, "gated group norm out", gate.dtype, 2)
    _need(weight, "gated group norm weight", torch.float32, 1)
    if (xs is None) != (skip is None):
        raise KernelError("gated group norm: a skip needs its input and its factors")
    if xs is not None:
        _need(xs, "gated group norm xs", torch.float32, 2)
        _need(skip, "gated group norm skip", torch.float32, 1)
        if tuple(xs.shape) != (n, width) or skip.shape[0] * dv != width:
            raise KernelError("gated group norm: the skip's input or factors of the wrong size")
    if tuple(out.shape) != (n, width) or weight.shape[0] != width or gate.shape[0] != n or gate.shape[1] < width:
        raise KernelError(f"gated group norm: o {tuple(o.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)}")
    if parts < 1 or width % parts:
        raise KernelError(f"gated group norm: {width} columns in {parts} parts")
    _check(lib().mll_gated_group_norm(
        _ptr(o), _ptr(xs), _ptr(skip), _ptr(gate), dtype_code(gate.dtype), ctypes.c_int(gate.shape[1]), _ptr(weight),
        _ptr(out), dtype_code(out.dtype), ctypes.c_int(n), ctypes.c_int(width), ctypes.c_int(dv), ctypes.c_int(parts),
        ctypes.c_float(eps), _stream()), "gated_group_norm")


def channel_decay_prepare(proj, rate, bias, q, k, v, g, n_heads: int, d: int, dv: int, q_scale: float, tau: float) -> None:
    """proj [T, ld] holds q (H * d), k (H * d), v (H * dv) side by side: q * q_scale, k and v to float32, and
    g = sigmoid(rate + bias)^(1 / tau) per key channel (rate float32 [T, >= H * d], bias float32 [H * d] or None)."""
    _need(proj, "channel decay proj", None, 2)
    _need(rate, "channel decay rate", torch.float32, 2)
    n = proj.shape[0]
    for name, t, width in (("q", q, n_heads * d), ("k", k, n_heads * d), ("v", v, n_heads * dv), ("g", g, n_heads * d)):
        _need(t, f"channel decay {name}", torch.float32, 2)
        if tuple(t.shape) != (n, width):
            raise KernelError(f"channel decay: {name} {tuple(t.shape)}, expected {(n, width)}")
    if bias is not None:
        _need(bias, "channel decay bias", torch.float32, 1)
        if bias.shape[0] != n_heads * d:
            raise KernelError("channel decay: one bias per head and key channel is needed")
    if rate.shape[0] != n:
        raise KernelError("channel decay: the rates have other rows than the projections")
    _check(lib().mll_channel_decay_prepare(
        _ptr(proj), _ptr(rate), _ptr(bias), _ptr(q), _ptr(k), _ptr(v), _ptr(g), dtype_code(proj.dtype), ctypes.c_int(n),
        ctypes.c_int(proj.shape[1]), ctypes.c_int(rate.shape[1]), ctypes.c_int(n_heads), ctypes.c_int(d),
        ctypes.c_int(dv), ctypes.c_float(q_scale), ctypes.c_float(tau), _stream()), "channel_decay_prepare")


GATE_SILU, GATE_SIGMOID = 0, 1


def head_norm_gate(o, weight, gate, out, n_heads: int, dv: int, eps: float, act: int, gate_col: int = 0) -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * act(gate[t, h, :]); o float32
    [T, H * dv], weight float32 [dv] or None, gate [T, ld] of which columns gate_col .. gate_col + H * dv are read."""
    _need(o, "head norm o", torch.float32, 2)
    _need(gate, "head norm gate", None, 2)
    _need(out, "head norm out", None, 2)
    n = o.shape[0]
    if (tuple(o.shape) != (n, n_heads * dv) or tuple(out.shape) != (n, n_heads * dv) or gate.shape[0] != n
            or gate_col < 0 or gate_col + n_heads * dv > gate.shape[1]):
        raise KernelError(f"head norm gate: o {tuple(o.shape)}, out {tuple(out.shape)}, gate {tuple(gate.shape)}")
    if weight is not None:
        _need(weight, "head norm weight", torch.float32, 1)
        if weight.shape[0] != dv:
            raise KernelError("head norm gate: the weight has one entry per value channel of a head")
    _check(lib().mll_head_norm_gate(
        _ptr(o), _ptr(weight), ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()),
        dtype_code(gate.dtype), ctypes.c_int(gate.shape[1]), _ptr(out),
        dtype_code(out.dtype), ctypes.c_int(n), ctypes.c_int(n_heads), ctypes.c_int(dv), ctypes.c_float(eps),
        ctypes.c_int(act), _stream()), "head_norm_gate")


# --------------------------------------------------------------------------- #
# attention over a shared low-rank latent
# --------------------------------------------------------------------------- #
def latent_prepare(proj, c_weight, cos, sin, tok_pos, tok_seq, seq_slot, block_table, q_out, kv_cache, n_heads: int,
                   d: int, rot: int, rank: int, interleaved: bool, eps: float) -> None:
    """proj [T, ld]: H heads of (d plain + rot rotated) query columns, then the down projection's rank + rot columns.
    Writes the cache row [c | k_r] of every token (c = the first rank columns divided by their root mean square and
    multiplied by `c_weight`, k_r = the last rot columns rotated by position) into its page of `kv_cache`
    [pages, 1, PAGE, rank + rot], and the rotated part of every head's query into the last rot columns of that head
    in `q_out` [T, H * (rank + rot)]."""
    _need(proj, "latent prepare proj", None, 2)
    _need(q_out, "latent prepare q", proj.dtype, 2)
    _need(kv_cache, "latent prepare cache", proj.dtype, 4)
    _need(c_weight, "latent prepare norm weight", torch.float32, 1)
    n = proj.shape[0]
    if tuple(kv_cache.shape[1:]) != (1, PAGE, rank + rot) or tuple(q_out.shape) != (n, n_heads * (rank + rot)):
        raise KernelError(f"latent prepare: cache {tuple(kv_cache.shape)} / q {tuple(q_out.shape)} for rank {rank} + {rot}")
    if c_weight.shape[0] != rank:
        raise KernelError(f"latent prepare: norm weight of {c_weight.shape[0]}, expected {rank}")
    if rot:
        _need(cos, "latent prepare cos", torch.float32, 2)
        _need(sin, "latent prepare sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError(f"latent prepare: rotary table {tuple(cos.shape)} for {rot} rotated dimensions")
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot)):
        _need(t, f"latent prepare {name}", torch.int32, 1)
    _need(block_table, "latent prepare block table", torch.int32, 2)
    _check(lib().mll_latent_prepare(
        _ptr(proj), _ptr(c_weight), _ptr(cos if rot else None), _ptr(sin if rot else None), _ptr(tok_pos), _ptr(tok_seq),
        _ptr(seq_slot), _ptr(block_table), _ptr(q_out), _ptr(kv_cache), dtype_code(proj.dtype), ctypes.c_int(n),
        ctypes.c_int(proj.shape[1]), ctypes.c_int(n_heads), ctypes.c_int(d), ctypes.c_int(rot), ctypes.c_int(rank),
        ctypes.c_int(int(interleaved)), ctypes.c_int(block_table.shape[1]), ctypes.c_float(eps), _stream()),
        "latent_prepare")


# --------------------------------------------------------------------------- #
# routed feed-forward
# --------------------------------------------------------------------------- #
USE_TENSOR_CORE_MOE = True  # tests switch it off to reach the plain products in bfloat16 prompt steps


class MoePlan(NamedTuple):
    """A step's (token, choice) pairs sorted by expert, all on the device (int32): `order` [pairs] place -> pair,
    `offsets` [E + 1], tiles of up to `rows` places of one expert (`tile_expert`, `tile_row0`, of which the first
    `n_tiles[0]` count; the lists are sized for the most tiles there can be)."""
    order: torch.Tensor
    offsets: torch.Tensor
    tile_expert: torch.Tensor
    tile_row0: torch.Tensor
    n_tiles: torch.Tensor
    rows: int
    mma: bool


MOE_TILE_ROWS_OVERRIDE: Optional[int] = None  # measurements only: 0, 1 or 2 picks the tensor-core tile at every size


def moe_tile_rows(mma: bool, n_pairs: int = 1 << 30, n_experts: int = 1) -> int:
    """Rows of a tile of the routed products: the plain kernels' size, or one of the tensor-core kernels' three - 16
    rows while an expert gets 12 rows or fewer on average (single tokens), 32 rows up to 32 on average, else 128.
    (Measured at 16 experts: at 10.7 rows an expert 16-row tiles are 5 to 18 % faster than 32-row ones, at 16 rows
    an expert - where about half of the experts need a second 16-row tile - 32-row tiles are up to 20 % faster.)"""
    if not mma:
        return int(lib().mll_moe_simt_rows())
    if MOE_TILE_ROWS_OVERRIDE is not None:
        return int(lib().mll_moe_mma_rows(ctypes.c_int(MOE_TILE_ROWS_OVERRIDE)))
    small = 1 if n_pairs <= 12 * n_experts else (2 if n_pairs <= 32 * n_experts else 0)
    return int(lib().mll_moe_mma_rows(ctypes.c_int(small)))


def moe_max_tiles(n_pairs: int, n_experts: int, rows: int) -> int:
    return n_pairs // rows + n_experts


def moe_route(h, w, bias, chosen, weight, top: int, logits: Optional[torch.Tensor] = None, all_scores: bool = False,
              scale: float = 1.0, gate_out: Optional[torch.Tensor] = None, groups=None) -> None:
    """chosen [T, top] (int32) = the experts with the largest z = w h + bias (float32; ties: the lower index),
    weight [T, top] (float32) = softmax over the chosen logits.  `logits`: float32 [T, E] = h w^T when the caller
    has formed the product already (a library product over many tokens).
    `all_scores`: s = softmax(w h) over every expert, the choice goes by s + bias, weight = the chosen s over their
    sum (+ 1e-20), times `scale`.  `groups` = (count, kept): s = sigmoid(w h); the experts are cut into `count` runs of
    consecutive experts of one length, a run is rated by its top two s added up, only experts of the `kept` best-rated runs can be chosen;
    weight as with `all_scores`.  `gate_out` (float32 [T]): w (and logits) have one more row behind the experts';
    the sigmoid of its product with the token goes there."""
    _need(h, "moe route h", None, 2)
    _need(w, "moe route weight", torch.float32, 2)
    _need(chosen, "moe route chosen", torch.int32, 2)
    _need(weight, "moe route weights", torch.float32, 2)
    n, width = h.shape
    rows = w.shape[0]
    experts = rows - (1 if gate_out is not None else 0)
    if gate_out is not None:
        _need(gate_out, "moe route gate", torch.float32, 1)
        if gate_out.shape[0] != n:
            raise KernelError("moe route: one gate per token is needed")
    if w.shape[1] != width or tuple(chosen.shape) != (n, top) or tuple(weight.shape) != (n, top):
        raise KernelError(f"moe route: h {tuple(h.shape)}, w {tuple(w.shape)}, chosen {tuple(chosen.shape)}")
    if bias is not None:
        _need(bias, "moe route bias", torch.float32, 1)
        if bias.shape[0] != experts:
            raise KernelError("moe route: one bias per expert is needed")
    if logits is not None:
        _need(logits, "moe route logits", torch.float32, 2)
        if tuple(logits.shape) != (n, rows):
            raise KernelError(f"moe route: logits {tuple(logits.shape)}, expected {(n, rows)}")
    _check(lib().mll_moe_route(_ptr(h), _ptr(w), _ptr(bias), _ptr(logits), _ptr(chosen), _ptr(weight), dtype_code(h.dtype),
                               ctypes.c_int(n), ctypes.c_int(width), ctypes.c_int(experts), ctypes.c_int(top),
                               ctypes.c_int(2 if groups else int(all_scores)), ctypes.c_float(scale), _ptr(gate_out),
                               ctypes.c_int(int(groups[0]) if groups else 0), ctypes.c_int(int(groups[1]) if groups else 0),
                               _stream()),
           "moe_route")


def moe_sort(chosen, plan: MoePlan, n_experts: int, n_real: Optional[int] = None) -> None:
    """`n_real`: the experts from there on have no matrices (they hand their input on) and get no tiles."""
    n_pairs = chosen.numel()
    need = moe_max_tiles(n_pairs, n_experts, plan.rows)
    if (plan.order.numel() < n_pairs or plan.offsets.numel() < n_experts + 1 or plan.tile_expert.numel() < need
            or plan.tile_row0.numel() < need):
        raise KernelError("moe sort: the plan's arrays are too short")
    _check(lib().mll_moe_sort(_ptr(chosen), _ptr(plan.order), _ptr(plan.offsets), _ptr(plan.tile_expert),
                              _ptr(plan.tile_row0), _ptr(plan.n_tiles), ctypes.c_int(n_pairs), ctypes.c_int(n_experts),
                              ctypes.c_int(plan.rows), ctypes.c_int(n_experts if n_real is None else n_real), _stream()),
           "moe_sort")


def moe_mma_supported(dtype: torch.dtype, width: int, inter: int) -> bool:
    return dtype == torch.bfloat16 and hasattr(lib(), "mll_moe_mma_supported") and bool(
        lib().mll_moe_mma_supported(width, inter))


def _plan_args(plan: MoePlan):
    return (_ptr(plan.order), _ptr(plan.offsets), _ptr(plan.tile_expert), _ptr(plan.tile_row0), _ptr(plan.n_tiles))


EXPERT_SWIGLU, EXPERT_GELU = 0, 1


def moe_gate_up(h, w, act, plan: MoePlan, top: int, form: int = EXPERT_SWIGLU, n_experts: Optional[int] = None) -> None:
    """act[place] = silu(W_gate,e h[token]) * (W_up,e h[token]); w [E, 2 I, D] holds an expert's gate rows, then
    its up rows; act [pairs, I].  form EXPERT_GELU: act[place] = gelu(W_up,e h[token]) (erf form), w [E, I, D].
    `n_experts`: the experts that the plan was sorted for, where more are routed to than have matrices."""
    _need(h, "moe gate_up h", None, 2)
    _need(w, "moe gate_up w", h.dtype, 3)
    _need(act, "moe gate_up act", h.dtype, 2)
    experts, two_inter, width = w.shape
    experts = experts if n_experts is None else n_experts
    inter = two_inter // 2 if form == EXPERT_SWIGLU else two_inter
    n_pairs = h.shape[0] * top
    if h.shape[1] != width or tuple(act.shape) != (n_pairs, inter) or (form == EXPERT_SWIGLU and two_inter != 2 * inter):
        raise KernelError(f"moe gate_up: h {tuple(h.shape)}, w {tuple(w.shape)}, act {tuple(act.shape)}")
    fn = lib().mll_moe_gate_up_mma if plan.mma else lib().mll_moe_gate_up
    args = (_ptr(h), _ptr(w), _ptr(act), *_plan_args(plan))
    tiles = ctypes.c_int(moe_max_tiles(n_pairs, experts, plan.rows))
    if plan.mma:
        _check(fn(*args, tiles, ctypes.c_int(plan.rows), ctypes.c_int(width), ctypes.c_int(inter), ctypes.c_int(top),
                  ctypes.c_int(form), _stream()), "moe_gate_up_mma")
    else:
        _check(fn(*args, dtype_code(h.dtype), tiles, ctypes.c_int(width), ctypes.c_int(inter), ctypes.c_int(top),
                  ctypes.c_int(form), _stream()), "moe_gate_up")


def moe_down(act, w, y, pair_weight, plan: MoePlan, top: int, n_experts: Optional[int] = None) -> None:
    """y[pair] = weight[pair] * W_down,e act[place] (float32 [pairs, D]); w [E, D, I].  `n_experts`: as for
    `moe_gate_up`."""
    _need(act, "moe down act", None, 2)
    _need(w, "moe down w", act.dtype, 3)
    _need(y, "moe down y", torch.float32, 2)
    _need(pair_weight, "moe down weights", torch.float32)
    experts, width, inter = w.shape
    experts = experts if n_experts is None else n_experts
    n_pairs = act.shape[0]
    if act.shape[1] != inter or tuple(y.shape) != (n_pairs, width) or pair_weight.numel() != n_pairs:
        raise KernelError(f"moe down: act {tuple(act.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    fn = lib().mll_moe_down_mma if plan.mma else lib().mll_moe_down
    args = (_ptr(act), _ptr(w), _ptr(y), _ptr(pair_weight), *_plan_args(plan))
    tiles = ctypes.c_int(moe_max_tiles(n_pairs, experts, plan.rows))
    if plan.mma:
        _check(fn(*args, tiles, ctypes.c_int(plan.rows), ctypes.c_int(inter), ctypes.c_int(width), ctypes.c_int(top),
                  _stream()), "moe_down_mma")
    else:
        _check(fn(*args, dtype_code(act.dtype), tiles, ctypes.c_int(inter), ctypes.c_int(width), ctypes.c_int(top),
                  _stream()), "moe_down")


def moe_combine(y, other, out, top: int, chosen=None, pair_weight=None, h=None, n_real: int = 0, other_gate=None) -> None:
    """out[t] = y[t * top] + ... + y[t * top + top - 1] (+ other[t]); y float32 [T * top, D].
    `chosen` (int32 [T, top], with `pair_weight` float32 [T, top], `h` [T, D] of out's dtype and `n_real`): a choice of
    an expert >= n_real adds pair_weight * h[t] instead of its row of y.  `other_gate` (float32 [T]): a factor on
    `other`."""
    _need(y, "moe combine y", torch.float32, 2)
    _need(out, "moe combine out", None, 2)
    n, width = out.shape
    if tuple(y.shape) != (n * top, width):
        raise KernelError(f"moe combine: y {tuple(y.shape)}, out {tuple(out.shape)}, top {top}")
    if other is not None:
        _need(other, "moe combine other", out.dtype, 2)
        if other.shape != out.shape:
            raise KernelError("moe combine: the other part's output differs in shape")
    if chosen is not None:
        _need(chosen, "moe combine chosen", torch.int32, 2)
        _need(pair_weight, "moe combine weights", torch.float32, 2)
        _need(h, "moe combine h", out.dtype, 2)
        if tuple(chosen.shape) != (n, top) or tuple(pair_weight.shape) != (n, top) or h.shape != out.shape:
            raise KernelError("moe combine: chosen, weights or input rows of the wrong shape")
    if other_gate is not None:
        _need(other_gate, "moe combine gate", torch.float32, 1)
        if other_gate.shape[0] != n or other is None:
            raise KernelError("moe combine: one gate per token, on the other part's output")
    _check(lib().mll_moe_combine(_ptr(y), _ptr(other), _ptr(out), dtype_code(out.dtype), ctypes.c_int(n),
                                 ctypes.c_int(width), ctypes.c_int(top), _ptr(chosen), _ptr(pair_weight), _ptr(h),
                                 ctypes.c_int(n_real), _ptr(other_gate), _stream()), "moe_combine")
