"""The kernels as Python functions over torch tensors.

Every function launches hand-written CUDA from `csrc/` on the current stream through
ctypes. There is no CPU path and no library fallback: without a CUDA device, or when a
library cannot be built or loaded, a call raises. A kernel that cannot take a size
refuses it with the message its entry point stored; nothing is retried elsewhere.

Tensors are contiguous; activations and matrices are float32 or bfloat16, biases and
norm weights float32, indices int32, logits float32.
"""

from __future__ import annotations

import ctypes
import re
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_libs: dict[str, ctypes.CDLL] = {}

# Kernel launches made through this module since import (read by the measurement script).
launches = 0


# True when the libraries are the checked build (PAE_BOUNDS=1: see kernels/build.py). The kernels
# then compare every slot, block-table index and page id with the pool before using it; the
# limits are handed to a library whenever they change, which a recorded graph cannot follow, so
# the runner records none in this mode.
bounds_checked = build.BOUNDS
_bounds_set: dict[str, tuple] = {}


class KernelError(RuntimeError):
    pass


def _set_bounds(name: str, pages_of: torch.Tensor | None) -> None:
    """Checked build only: tells library `name` how many pages the pool of `pages_of` has."""
    if not bounds_checked or pages_of is None:
        return
    flag = _error_flag(pages_of.device)
    limits = (int(pages_of.shape[0]), flag.data_ptr())
    if _bounds_set.get(name) != limits:
        lib = _lib(name)
        code = lib.pae_set_bounds(ctypes.c_longlong(limits[0]), c_void_p(limits[1]))
        if code != 0:
            raise KernelError(lib.pae_last_error().decode(errors="replace"))
        _bounds_set[name] = limits


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "paged_attention_engine_b200 runs on a CUDA device only (sm_100a); no device is visible "
            "and there is no CPU path"
        )


_SIGNATURE = re.compile(r"PAE_EXPORT\s+([\w\s\*]+?)\s*\b(pae_\w+)\s*\(([^)]*)\)")


def _ctype_of(declaration: str):
    if "*" in declaration:
        return ctypes.c_char_p if declaration.strip().startswith("const char") and declaration.strip().endswith("*") else c_void_p
    if "long long" in declaration:
        return ctypes.c_longlong
    if "float" in declaration:
        return c_float
    return c_int


def _declare_signatures(lib: ctypes.CDLL, name: str) -> None:
    """Tells ctypes the argument and result types of the family's entry points, read from their
    declarations in the sources (`PAE_EXPORT <type> pae_name(<arguments>)`): a call then takes plain
    Python integers, floats and addresses, which is quicker than wrapping each in a ctypes object,
    and an address is never cut to 32 bits."""
    for source in build.FAMILIES[name]:
        text = (build.CSRC / source).read_text()
        for result, function, arguments in _SIGNATURE.findall(text):
            entry = getattr(lib, function, None)
            if entry is None:
                continue
            arguments = arguments.strip()
            entry.argtypes = [] if arguments in ("", "void") else [
                c_void_p if "*" in a else _ctype_of(a) for a in arguments.split(",")]
            entry.restype = _ctype_of(result)


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        require_cuda()
        path = build.ensure_built([name])[name]
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from exc
        lib.pae_last_error.restype = ctypes.c_char_p
        _declare_signatures(lib, name)
        _libs[name] = lib
    return lib


def preload(names: list[str]) -> None:
    """Builds (in parallel) and loads the given families."""
    require_cuda()
    build.ensure_built([n for n in names if n not in _libs])
    for n in names:
        _lib(n)


def _check(lib: ctypes.CDLL, code: int, count: int = 1) -> None:
    global launches
    launches += count
    if code != 0:
        raise KernelError(lib.pae_last_error().decode(errors="replace") + f" (code {code})")


def _ptr(t: torch.Tensor | None):
    """A tensor's address as an integer (the entry points' pointer arguments are declared)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (asked for at every launch: the quick way when torch has it)."""
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(t: torch.Tensor, what: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} is {t.dtype}, {dtype} is needed")


# ----------------------------------------------------------------------------------- #

class PendingSum:
    """A split-K product whose float32 partial sums [splits, M, N] have not been added up yet.

    `linear` returns one for a step of few tokens. `rms_norm`, `silu_mul` and
    `rotary_qk_cache_write` add the splits up inside their own kernel (bias and residual
    included), which saves a launch; anything else calls `materialized`, which runs the
    stand-alone reduction once and keeps its result in `value`."""

    def __init__(self, partial, bias, residual, out_dtype, activation: int = 0):
        self.partial = partial
        self.bias = bias
        self.residual = residual
        self.dtype = out_dtype
        self.activation = activation      # applied to sum + bias by the stand-alone reduction only
        self.value = None

    @property
    def shape(self):
        return self.partial.shape[1:]

    @property
    def device(self):
        return self.partial.device


class PendingNorm:
    """RMSNorm(x) * weight of a step of few tokens that has not been computed: `rms_norm` returns
    one, and the products that can (`qkv_projection`, `linear_swiglu`, `linear` without bias) apply
    the norm while they stage their operand, which saves the norm's own launch; anything else
    calls `materialized`, which runs the norm's kernel once and keeps its result in `value`."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
        self.x = x
        self.weight = weight
        self.eps = eps
        self.value = None

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


class PendingStreams:
    """Residual streams [tokens, streams * width] whose write x'_t = sum_s mix[s, t] x_s + out[t] y has
    not run: `streams_write` returns one, and the `streams_read_norm` of the next sublayer does
    the write inside its own kernel; anything else calls `materialized`, which runs the write alone."""

    def __init__(self, x, y, mix, out_w, streams: int) -> None:
        self.x, self.y, self.mix, self.out_w, self.streams = x, y, mix, out_w, streams
        self.dtype = torch.float32
        self.value = None

    @property
    def shape(self):
        return (self.x.shape[0], self.streams * self.y.shape[-1])

    @property
    def device(self):
        return self.x.device


class PendingResidual:
    """A float32 residual stream x + mult * post(y) (+ extra) whose sum has not been made: `residual_add`
    returns one, and the norm without statistics that reads the stream next (`dyt_norm`) makes the
    sum inside its own kernel; anything else calls `materialized`, which runs the sum alone. `post`
    is (alpha, weight, bias) of a Dynamic Tanh applied to y first, or None; y may be a product that is
    still in its splits; `extra` is a second stream that joins (or None)."""

    def __init__(self, x, y, post, mult: float, extra=None) -> None:
        self.x, self.y, self.post, self.mult, self.extra = x, y, post, float(mult), extra
        self.dtype = torch.float32
        self.value = None

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device


def materialized(x):
    """The tensor that `x` stands for (x itself unless it is a PendingSum, a PendingNorm, PendingStreams or a PendingResidual)."""
    if isinstance(x, PendingResidual):
        if x.value is None:
            _dyt_step(x, None, None)
        return x.value
    if isinstance(x, PendingNorm):
        if x.value is None:
            x.value = _rms_norm_now(x.x, x.weight, x.eps)
        return x.value
    if isinstance(x, PendingStreams):
        if x.value is None:
            _streams_step(x, None, None, 0.0, None)
        return x.value
    if not isinstance(x, PendingSum):
        return x
    if x.value is None:
        splits, m, n = x.partial.shape
        out = torch.empty((m, n), dtype=x.dtype, device=x.partial.device)
        lib = _lib("gemm_tcgen05")
        _check(lib, lib.pae_reduce_splits(_ptr(out), _ptr(x.partial), _ptr(x.bias), _ptr(x.residual), splits,
                                          m, n, (1 if x.dtype == torch.float32 else 0), x.activation, _stream()))
        x.value = out
    return x.value


def gather_rows(x, rows: torch.Tensor) -> torch.Tensor:
    x = materialized(x)
    _need(x, "gather_rows: x")
    _need(rows, "gather_rows: rows", torch.int32)
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_gather_rows(_ptr(out), _ptr(x), _ptr(rows), (rows.numel()), x.shape[0],
                                    x.shape[1], (_code(x)), _stream()))
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, feedback=None) -> torch.Tensor:
    """Rows of `table` for the token ids. With `feedback` = (last_token, state_slot, seq_index) a
    negative id stands for the token that the request sampled in the step before, read from
    last_token[state_slot[seq_index[t]]] on the device."""
    if feedback is None:
        return gather_rows(table, ids)
    last_token, state_slot, seq_index = feedback
    _need(table, "embedding: table")
    for name, t in (("ids", ids), ("last_token", last_token), ("state_slot", state_slot), ("seq_index", seq_index)):
        _need(t, f"embedding: {name}", torch.int32)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_embedding_feedback(_ptr(out), _ptr(table), _ptr(ids), _ptr(last_token), _ptr(state_slot),
                                           _ptr(seq_index), (ids.numel()), table.shape[0],
                                           table.shape[1], (_code(table)), _stream()))
    return out


def scatter_tokens(last_token, tokens, logit_rows, seq_index, state_slot) -> None:
    """last_token[state_slot[seq_index[logit_rows[r]]]] = tokens[r]: the sampled tokens stay on the
    device where the next step's embedding finds them."""
    for name, t in (("last_token", last_token), ("tokens", tokens), ("logit_rows", logit_rows),
                    ("seq_index", seq_index), ("state_slot", state_slot)):
        _need(t, f"scatter_tokens: {name}", torch.int32)
    lib = _lib("elementwise")
    _check(lib, lib.pae_scatter_tokens(_ptr(last_token), _ptr(tokens), _ptr(logit_rows), _ptr(seq_index),
                                       _ptr(state_slot), (tokens.numel()), _stream()))


def rms_norm(x, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _need(weight, "rms_norm: weight", torch.float32)
    if weight.numel() != x.shape[-1]:
        raise KernelError(f"rms_norm: weight of {weight.numel()} for rows of {x.shape[-1]}")
    if isinstance(x, PendingSum) and x.value is None and not x.activation:
        splits, m, n = x.partial.shape
        value = torch.empty((m, n), dtype=x.dtype, device=x.device)
        normed = torch.empty_like(value)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_rms_norm(_ptr(normed), _ptr(value), _ptr(x.partial), splits, _ptr(x.bias),
                                            _ptr(x.residual), _ptr(weight), m, n, eps,
                                            _DTYPE_CODE[x.dtype], _stream()))
        x.value = value
        return normed
    x = materialized(x)
    _need(x, "rms_norm: x")
    if x.dim() == 2 and _few_tokens(x, x.shape[-1], normed=True):
        return PendingNorm(x, weight, eps)       # the product that follows applies it
    return _rms_norm_now(x, weight, eps)


def _rms_norm_now(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    out = torch.empty_like(x)
    lib = _lib("elementwise")
    rows = x.numel() // x.shape[-1] if x.numel() else 0
    _check(lib, lib.pae_rms_norm(_ptr(out), _ptr(x), _ptr(weight), rows, (x.shape[-1]), eps,
                                 (_code(x)), _stream()))
    return out


# A step of few tokens (decoding) runs a product as one kernel that leaves finished output
# (csrc/gemv_mma.cu: a warp owns 16 weight rows and the whole K, so no partial sums are left for a
# kernel of their own, and the norm before and the rotation, SiLU x up or residual after run
# inside the product) where that is the faster way: where all blocks of that kernel run at once.
# False sends every product to the tcgen05 kernels and their summing kernels (tests compare the
# two); `few_token_products_everywhere` sends every product that the kernels can take at all.
use_few_token_products = True
few_token_products_everywhere = False
FEW_TOKENS_MAX = 24
QKV_KIND, RESIDUAL_KIND, GATE_UP_KIND = 0, 1, 2
# Up to how many tokens a kind of product is faster there than as a tcgen05 product with its summing
# kernel (measured at the 1536-wide sizes, 24 tokens: q|k|v 6.7 against 8.4 us, o 4.9 against 6.5,
# gate|up 14.3 against 16.5; down, whose warps bring the tokens' operand through their rings once
# each, 10.2 against 9.6. A decode step of 24 requests: 1.63 against 1.75 ms; with kernels for 32
# tokens a step of 28 or 32 was no faster, 1.92 against 1.89 and 2.01 against 1.99 ms, and they are not built).
FEW_TOKENS_MAX_QKV = 24
FEW_TOKENS_MAX_RESIDUAL = 24          # while K is short ...
FEW_TOKENS_MAX_RESIDUAL_LONG_K = 16   # ... and from K = 2,048 on
FEW_TOKENS_MAX_GATE_UP = 24


def _few_tokens(x: torch.Tensor, k: int, normed: bool = False, kind: int = GATE_UP_KIND, n: int = 16) -> bool:
    """Whether a product of `kind` over x [tokens, K] with `n` weight rows runs as a few-token
    kernel; `normed`: with the RMSNorm of x folded in (the normed operand has to fit shared memory)."""
    if not (use_few_token_products and use_tensor_cores and x.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= FEW_TOKENS_MAX and x.data_ptr() % 16 == 0):
        return False
    if k < 64 or k % 64:        # not for these kernels: their library is not even built for such a model
        return False
    answer = _lib("gemv_mma").pae_linear_few_tokens_supports(kind, x.shape[0], n, k, 1 if normed else 0)
    if few_token_products_everywhere:
        return answer >= 1
    most = (FEW_TOKENS_MAX_QKV if kind == QKV_KIND else FEW_TOKENS_MAX_GATE_UP if kind == GATE_UP_KIND
            else FEW_TOKENS_MAX_RESIDUAL if k < SWAPPED_LONG_K else FEW_TOKENS_MAX_RESIDUAL_LONG_K)
    return answer == 2 and x.shape[0] <= most


def _norm_of(x):
    """(input tensor, norm weight or None, eps) of an operand that may be a PendingNorm."""
    if isinstance(x, PendingNorm) and x.value is None:
        return x.x, x.weight, x.eps
    return materialized(x), None, 0.0


# The bfloat16 products run on the tcgen05 kernels when the shape allows; set to False to
# send everything to the CUDA-core kernel (tests compare the two).
use_tensor_cores = True
# Whether a split-K product is summed inside the kernel that consumes it (tests compare both).
fuse_split_sums = True
SWAPPED_MAX_TOKENS = 64
# ... and up to this many where K is long (2,048 and more): the swapped product's blocks then
# have enough of K each, and it stays ahead of the many-token kernel with its K shared out in
# planes (128 tokens at the 3584-wide sizes: q|k|v 19.8 against 22.5 us, o 16.3 against 19.2; down of
# the 1536-wide sizes, K = 8960: 14.0 against 16.3; its q|k|v and o, K = 1536: 14.7 and 10.5 against 12.4 and 9.7).
SWAPPED_MAX_TOKENS_LONG_K = 128
SWAPPED_LONG_K = 2048


def _swapped(m: int, k: int) -> bool:
    """Whether a product of m tokens over K takes the swapped split-K kernel."""
    return m <= SWAPPED_MAX_TOKENS or (m <= SWAPPED_MAX_TOKENS_LONG_K and k >= SWAPPED_LONG_K)
# gate|up takes the many-token kernel (SiLU x up in its epilogue, no split of K, tiles of 128 tokens)
# from 33 tokens on: at 64 tokens 16.8 against 21.9 us at the 1536-wide sizes and 52.2 against
# 61.1 us at the 3584-wide ones; at 32 tokens 18.7 against 17.6 and 51.6 against 53.4, below that the
# swapped product and the kernel that adds its two splits are faster.
SWIGLU_SWAPPED_MAX_TOKENS = 32

_error_flags: dict[int, torch.Tensor] = {}


def _error_flag(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    flag = _error_flags.get(index)
    if flag is None:
        with torch.inference_mode(False):      # an ordinary tensor, whoever asks first: it is cleared from anywhere
            flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[index] = flag
    return flag


def error_flag(device) -> torch.Tensor:
    """The device's error word (int32 [1]): 0, or the role code of a wait that gave up. The
    generation path copies it to the host beside the sampled tokens and hands it to
    `raise_for_error_word`, so that a step whose kernel gave up never yields tokens silently."""
    return _error_flag(torch.device(device))


def raise_for_error_word(code: int, device) -> None:
    """Raises (and clears the device's word) when `code`, a copy of the error word, is not 0."""
    if code:
        _error_flag(torch.device(device)).zero_()
        index = torch.device(device).index
        if int(code) >= 100:
            what = {101: "a slot beyond the pool", 102: "a block-table index beyond the table's width",
                    103: "a page id that is negative or beyond the pool"}.get(int(code), "an index out of range")
            raise KernelError(f"a kernel on device {index} met {what} (bounds code {int(code)}); the access was skipped")
        raise KernelError(
            f"a tensor-core kernel on device {index} gave up waiting on an mbarrier (role code {int(code)}; 8: a warp of a "
            "few-token product, others: the roles of a tcgen05 kernel); "
            "its output is not valid"
        )


def check_device_errors() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for index, flag in _error_flags.items():
        raise_for_error_word(int(flag.item()), flag.device)


def _tensor_core_shape(x, weight, residual, out_dtype) -> bool:
    return (
        use_tensor_cores
        and x.dtype == torch.bfloat16
        and weight.dtype == torch.bfloat16
        and x.shape[1] % 8 == 0
        and x.data_ptr() % 16 == 0
        and weight.data_ptr() % 16 == 0
    )


ACTIVATIONS = {None: 0, "gelu_erf": 1, "gelu_tanh": 2, "relu2": 3}


def linear(x, weight, bias=None, residual=None, out_dtype=None, activation: str | None = None) -> torch.Tensor:
    """x [M, K] . weight [N, K]^T (+ bias [N], float32) (+ residual [M, N]) -> [M, N]. `activation`
    ("gelu_erf", "gelu_tanh", "relu2": the square of max(z, 0)) is applied to the product (+ bias), rounded to the output's dtype first,
    before the residual: in the tensor-core product's epilogue or in the sum of its splits, else
    by the activation's own kernel."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"linear: activation '{activation}' (known: gelu_erf, gelu_tanh, relu2)")
    if (activation is None and bias is None and out_dtype in (None, torch.bfloat16) and weight.dtype == torch.bfloat16 and weight.dim() == 2
            and weight.data_ptr() % 16 == 0 and weight.shape[0] <= 65536):
        source, norm_weight, eps = _norm_of(x)
        if (_few_tokens(source, weight.shape[1], norm_weight is not None, RESIDUAL_KIND, weight.shape[0]) and source.dim() == 2 and source.shape[1] == weight.shape[1]
                and source.is_contiguous() and weight.is_contiguous()):
            residual_now = materialized(residual)
            m, n = source.shape[0], weight.shape[0]
            if residual_now is not None:
                _need(residual_now, "linear: residual", torch.bfloat16)
                if tuple(residual_now.shape) != (m, n):
                    raise KernelError(f"linear: residual is {tuple(residual_now.shape)}, the product is [{m}, {n}]")
            out = torch.empty((m, n), dtype=torch.bfloat16, device=source.device)
            lib = _lib("gemv_mma")
            _check(lib, lib.pae_linear_few_tokens(_ptr(out), _ptr(source), _ptr(weight), _ptr(residual_now), _ptr(norm_weight),
                                                  eps, m, n, weight.shape[1], _ptr(_error_flag(source.device)), _stream()))
            return out
    x = materialized(x)
    residual = materialized(residual)
    _need(x, "linear: x")
    _need(weight, "linear: weight")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x is [{m}, {k}], weight is {tuple(weight.shape)}")
    out_dtype = out_dtype or x.dtype
    if bias is not None:
        _need(bias, "linear: bias", torch.float32)
    if residual is not None:
        _need(residual, "linear: residual", out_dtype)
        if tuple(residual.shape) != (m, n):
            raise KernelError(f"linear: residual is {tuple(residual.shape)}, the product is [{m}, {n}]")
    if m == 0:
        return torch.empty((m, n), dtype=out_dtype, device=x.device)
    if _tensor_core_shape(x, weight, residual, out_dtype):
        return _linear_tensor_cores(x, weight, bias, residual, out_dtype, m, n, k, ACTIVATIONS[activation])
    if activation is not None:
        if residual is not None:
            raise KernelError("linear: an activation before a residual needs the tensor-core product")
        return gelu(linear(x, weight, bias, None, out_dtype), activation)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    lib = _lib("gemm_simt")
    _check(lib, lib.pae_linear_simt(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), m, n,
                                    k, (_code(x)), (_code(weight)), _DTYPE_CODE[out_dtype],
                                    _stream()))
    return out


def _linear_tensor_cores(x, weight, bias, residual, out_dtype, m, n, k, activation: int = 0) -> torch.Tensor:
    lib = _lib("gemm_tcgen05")
    flag = _error_flag(x.device)
    out_f32 = (1 if out_dtype == torch.float32 else 0)
    if _swapped(m, k):
        # Few tokens: weight rows fill the MMA's 128 rows, K is split, partial sums are
        # float32 scratch that the reduction (or nothing, for one split) turns into the output.
        splits = lib.pae_linear_swapped_splits(n, k)
        partial = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        _check(lib, lib.pae_linear_tcgen05_swapped(_ptr(partial), _ptr(x), _ptr(weight), m, n, k,
                                                   _ptr(flag), _stream()))
        if splits == 1 and bias is None and residual is None and out_dtype == torch.float32 and not activation:
            return partial[0]
        pending = PendingSum(partial, bias, residual, out_dtype, activation)
        return pending if fuse_split_sums else materialized(pending)
    planes = lib.pae_linear_tcgen05_plane_count(m, n, k)
    if planes > 1:
        # Few output tiles and a long K (a down projection for a few hundred tokens): each
        # tile's K is shared out over several blocks, whose float32 planes are added up later.
        partial = torch.empty((planes, m, n), dtype=torch.float32, device=x.device)
        _check(lib, lib.pae_linear_tcgen05_planes(_ptr(partial), _ptr(x), _ptr(weight), m, n, k,
                                                  planes, _ptr(flag), _stream()))
        pending = PendingSum(partial, bias, residual, out_dtype, activation)
        return pending if fuse_split_sums else materialized(pending)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _check(lib, lib.pae_linear_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), m, n,
                                       k, out_f32, activation, _ptr(flag), _stream()))
    return out


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor, amplitude: float = 1.0) -> torch.Tensor:
    """float32 [tokens, 2 * half]: amplitude * cos(position * inv_freq), then amplitude * sin of the same."""
    _need(positions, "rotary_table: positions", torch.int32)
    _need(inv_freq, "rotary_table: inv_freq", torch.float32)
    half = inv_freq.numel()
    table = torch.empty((positions.numel(), 2 * half), dtype=torch.float32, device=positions.device)
    if amplitude != 1.0:
        lib = _lib("head_prep")
        _check(lib, lib.pae_rotary_table_amplitude(_ptr(table), _ptr(positions), _ptr(inv_freq), positions.numel(), half,
                                                   float(amplitude), _stream()))
        return table
    lib = _lib("elementwise")
    _check(lib, lib.pae_rotary_table(_ptr(table), _ptr(positions), _ptr(inv_freq), (positions.numel()),
                                     half, _stream()))
    return table


def rotary_qk_cache_write(qkv, table, slots, keys, values, num_heads, num_kv_heads, head_dim, page_size) -> torch.Tensor:
    """Rotates q and k of the fused projection's output (in place), writes k and v to their
    pages, and returns the [tokens, (heads + 2 kv_heads) * head_dim] tensor."""
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"rotary_qk_cache_write: qkv rows of {qkv.shape[1]} for {num_heads}+2x{num_kv_heads} heads of {head_dim}")
    tokens = qkv.shape[0]
    if table is not None:
        _need(table, "rotary_qk_cache_write: table", torch.float32)
        if tuple(table.shape) != (tokens, head_dim):
            raise KernelError(f"rotary_qk_cache_write: table is {tuple(table.shape)}, [{tokens}, {head_dim}] is needed")
    if slots is not None:
        _need(slots, "rotary_qk_cache_write: slots", torch.int32)
        _need(keys, "rotary_qk_cache_write: keys", qkv.dtype)
        _need(values, "rotary_qk_cache_write: values", qkv.dtype)
    key_ptr = _ptr(keys if slots is not None else None)
    value_ptr = _ptr(values if slots is not None else None)
    if isinstance(qkv, PendingSum) and qkv.value is None and qkv.residual is None and not qkv.activation:
        splits = qkv.partial.shape[0]
        out = torch.empty((tokens, width), dtype=qkv.dtype, device=qkv.device)
        lib = _lib("fused_decode")
        _set_bounds("fused_decode", keys if slots is not None else None)
        _check(lib, lib.pae_splitk_rotary_cache_write(
            _ptr(out), _ptr(qkv.partial), splits, _ptr(qkv.bias), _ptr(table), _ptr(slots), key_ptr, value_ptr,
            tokens, num_heads, num_kv_heads, head_dim, page_size,
            _DTYPE_CODE[qkv.dtype], _stream()))
        qkv.value = out
        return out
    qkv = materialized(qkv)
    _need(qkv, "rotary_qk_cache_write: qkv")
    lib = _lib("elementwise")
    _set_bounds("elementwise", keys if slots is not None else None)
    _check(lib, lib.pae_rotary_qk_cache_write(
        _ptr(qkv), _ptr(table), _ptr(slots), key_ptr, value_ptr, tokens, num_heads, num_kv_heads,
        head_dim, page_size, (_code(qkv)), _stream()))
    return qkv


# Whether q|k|v of a prompt's portion is finished (bias, rotation, page write) by the product's own epilogue.
fuse_qkv_epilogue = True


def qkv_projection(x, weight, bias, table, slots, keys, values, num_heads, num_kv_heads, head_dim, page_size) -> torch.Tensor:
    """`rotary_qk_cache_write(linear(x, weight, bias), ...)`: q|k|v of the step's tokens, q and k
    rotated, k and v written to their pages. For more than 64 tokens on the tensor-core path it
    is one kernel (the product's epilogue rotates and writes); otherwise the two calls, which
    for few tokens fuse the other way round (the split sum runs inside the rotation kernel)."""
    m, k = x.shape
    n = weight.shape[0]
    source, norm_weight, eps = _norm_of(x)
    if (_few_tokens(source, k, norm_weight is not None, QKV_KIND, n) and weight.dtype == torch.bfloat16 and weight.is_contiguous() and weight.data_ptr() % 16 == 0
            and n == (num_heads + 2 * num_kv_heads) * head_dim and weight.shape[1] == k and head_dim % 16 == 0
            and (slots is None or (keys.dtype == torch.bfloat16 and values.dtype == torch.bfloat16))):
        _need(source, "qkv_projection: x")
        if bias is not None:
            _need(bias, "qkv_projection: bias", torch.float32)
        if table is not None:
            _need(table, "qkv_projection: table", torch.float32)
            if tuple(table.shape) != (m, head_dim):
                raise KernelError(f"qkv_projection: table is {tuple(table.shape)}, [{m}, {head_dim}] is needed")
        if slots is not None:
            _need(slots, "qkv_projection: slots", torch.int32)
            _need(keys, "qkv_projection: keys", torch.bfloat16)
            _need(values, "qkv_projection: values", torch.bfloat16)
        out = torch.empty((m, n), dtype=torch.bfloat16, device=source.device)
        lib = _lib("gemv_mma")
        _set_bounds("gemv_mma", keys if slots is not None else None)
        _check(lib, lib.pae_qkv_few_tokens(
            _ptr(out), _ptr(source), _ptr(weight), _ptr(bias), _ptr(norm_weight), eps, _ptr(table), _ptr(slots),
            _ptr(keys if slots is not None else None), _ptr(values if slots is not None else None), m, num_heads,
            num_kv_heads, head_dim, page_size, k, _ptr(_error_flag(source.device)), _stream()))
        return out
    x = materialized(x)
    if (fuse_qkv_epilogue and not _swapped(m, k) and n >= 256 and n == (num_heads + 2 * num_kv_heads) * head_dim
            and weight.shape[1] == k and not isinstance(x, PendingSum) and _tensor_core_shape(x, weight, None, x.dtype)
            and (slots is None or (keys.dtype == torch.bfloat16 and values.dtype == torch.bfloat16))):
        lib = _lib("gemm_tcgen05")
        # With so few output tiles that K is shared out over blocks, the sum of the planes rotates and writes.
        if lib.pae_linear_rotary_tcgen05_supports(head_dim) and lib.pae_linear_tcgen05_plane_count(m, n, k) == 1:
            _need(x, "qkv_projection: x")
            _need(weight, "qkv_projection: weight")
            if bias is not None:
                _need(bias, "qkv_projection: bias", torch.float32)
                if bias.numel() != n:
                    raise KernelError(f"qkv_projection: bias of {bias.numel()} for {n} columns")
            if table is not None:
                _need(table, "qkv_projection: table", torch.float32)
                if tuple(table.shape) != (m, head_dim):
                    raise KernelError(f"qkv_projection: table is {tuple(table.shape)}, [{m}, {head_dim}] is needed")
            if slots is not None:
                _need(slots, "qkv_projection: slots", torch.int32)
                _need(keys, "qkv_projection: keys", torch.bfloat16)
                _need(values, "qkv_projection: values", torch.bfloat16)
            out = torch.empty((m, n), dtype=x.dtype, device=x.device)
            _set_bounds("gemm_tcgen05", keys if slots is not None else None)
            _check(lib, lib.pae_linear_rotary_tcgen05(
                _ptr(out), _ptr(x), _ptr(weight), _ptr(bias), _ptr(table), _ptr(slots),
                _ptr(keys if slots is not None else None), _ptr(values if slots is not None else None), m,
                num_heads, num_kv_heads, head_dim, page_size, k,
                _ptr(_error_flag(x.device)), _stream()))
            return out
    return rotary_qk_cache_write(linear(x, weight, bias), table, slots, keys, values, num_heads, num_kv_heads, head_dim,
                                 page_size)


def decode_slicing(seqs: int, kv_heads: int, max_kv_len: int, most: int | None = None, wave_blocks: int = 444,
                   slices_per_block: int = 4) -> tuple[int, int]:
    """(keys per slice, slices) for the decode kernel. A block is `slices_per_block` slices of
    one (request, kv head) pair, and `wave_blocks` blocks run at one time: as many slices as
    keep all blocks in that one wave (a second, partly filled wave costs as much as a full
    one), at most `most`, each of at least 32 keys in steps of 16. A warp walks its slice one
    trip to memory after the other, so short slices are what makes few requests fast: up to 96
    for contexts of up to 6,144 keys (batch 1 at context 4,096: 0.940 -> 0.915 ms a step, batch 8:
    1.032 -> 1.024), beyond that up to 192 of at least 64 keys (batch 1 at context 32,768: 1.72 ms
    with 64 slices, 1.43 with 96, 1.24 with 192, 1.21 with 256, 1.25 with 384; batch 4 at 16,384:
    1.33, 1.20, 1.21; eight requests and more fill the wave with fewer slices anyway). The merge
    holds 96 slices' partial outputs in registers and walks the rest one by one."""
    if most is None:
        most = 96 if max_kv_len <= 96 * 64 else min(192, max_kv_len // 64)
    pairs = max(1, seqs * kv_heads)
    blocks_per_pair = max(1, wave_blocks // pairs)
    wanted = max(1, min(most, slices_per_block * blocks_per_pair))
    slice_keys = max(32, -(-(-(-max_kv_len // wanted)) // 16) * 16)
    while -(-(max_kv_len + 15) // slice_keys) > wanted:
        slice_keys += 16
    return slice_keys, -(-(max_kv_len + 15) // slice_keys)


use_tcgen05_attention = True
TCGEN05_ATTENTION_MIN_TOKENS = 64


def _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles, num_heads,
                      num_kv_heads, head_dim, page_size, max_kv_len, scale, window) -> None:
    """The requests that bring one token: sliced over their keys, then merged."""
    count = seqs if singles < 0 else singles
    wave = lib.pae_decode_blocks_per_wave(head_dim)
    slice_keys, max_slices = decode_slicing(count, num_kv_heads, max_kv_len, wave_blocks=wave,
                                            slices_per_block=lib.pae_decode_slices_per_block())
    floats = lib.pae_decode_scratch_floats(seqs, num_heads, head_dim, max_slices)
    scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
    launches = 2
    _set_bounds("attention_mma", keys)
    _check(lib, lib.pae_paged_attention_decode(
        _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1],
        _ptr(q_start), _ptr(kv_len), seqs, num_heads, num_kv_heads, head_dim,
        page_size, scale, window, slice_keys, max_slices,
        _ptr(scratch), _stream()), launches)


def paged_attention(qkv, keys, values, block_table, q_start, q_pos0, kv_len, num_heads, num_kv_heads, head_dim,
                    page_size, max_q_len, max_kv_len, scale, window, num_single=None, form: int = 0,
                    info: dict | None = None, multi_index: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's pages. `num_single` is the number
    of requests that bring exactly one token when the caller knows it (it decides which kernels
    are launched; None launches whatever may be needed). `multi_index` (int32, device) lists the
    requests that bring more than one token when some do and some do not: the portion kernels
    then launch blocks for those only (a step of 64 decoding requests and one prompt portion
    otherwise launches 65 requests' worth of blocks, 64 of which return at once but not for free). `form` 0 lets the tcgen05 attention pick
    its kernel by the size of the launch (two blocks of 64-key tiles per SM when there are that
    many blocks, else one block of 128-key tiles, its keys shared out over a cluster when the
    blocks are few); 1, 2, 4, 8, 16 name the kernel (tests). `info`, when given, receives which
    kernel ran ("kernel") and, for tcgen05, the blocks per query tile ("cluster": 0 is the
    paired kernel)."""
    qkv = materialized(qkv)
    _need(qkv, "paged_attention: qkv")
    _need(keys, "paged_attention: keys", qkv.dtype)
    _need(values, "paged_attention: values", qkv.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_pos0", q_pos0), ("kv_len", kv_len)):
        _need(t, f"paged_attention: {name}", torch.int32)
    tokens = qkv.shape[0]
    seqs = kv_len.numel()
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if qkv.dtype == torch.bfloat16 and use_tensor_cores:
        lib = _lib("attention_mma")
        mma_ok = bool(lib.pae_attention_mma_supports(num_heads, num_kv_heads, head_dim, page_size))
        singles = num_single if num_single is not None else (seqs if max_q_len == 1 else -1)
        # The requests that bring more than one token, when the caller lists them and the decode kernel takes the others.
        listed = multi_index if (multi_index is not None and mma_ok and singles > 0) else None
        if listed is not None:
            _need(listed, "paged_attention: multi_index", torch.int32)
            if listed.numel() != seqs - singles:
                raise KernelError(f"paged_attention: {listed.numel()} requests listed, {seqs - singles} bring more than one token")
        # Portions of 64 tokens and more: both products on tcgen05, one thread per query row.
        if use_tcgen05_attention and max_q_len >= TCGEN05_ATTENTION_MIN_TOKENS:
            tc5 = _lib("attention_tcgen05")
            if tc5.pae_attention_tcgen05_supports(num_heads, num_kv_heads, head_dim, page_size):
                decode_after = mma_ok and singles != 0
                chosen = c_int(-1)
                _set_bounds("attention_tcgen05", keys)
                _check(tc5, tc5.pae_paged_attention_prefill_tcgen05(
                    _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), ctypes.c_longlong(keys.shape[0]), _ptr(block_table),
                    block_table.shape[1], _ptr(q_start), _ptr(q_pos0), _ptr(kv_len), tokens, seqs,
                    max_q_len, max_kv_len, num_heads, num_kv_heads, head_dim, page_size,
                    scale, window, (1 if decode_after else 0), singles, form,
                    ctypes.byref(chosen), _ptr(listed), (listed.numel() if listed is not None else 0),
                    _ptr(_error_flag(qkv.device)), _stream()))
                if info is not None:
                    info.update(kernel="tcgen05", cluster=chosen.value)
                if decode_after:
                    _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles,
                                      num_heads, num_kv_heads, head_dim, page_size, max_kv_len, scale, window)
                return out
        if mma_ok:
            if info is not None:
                info.update(kernel="mma")
            if max_q_len > 1:
                _set_bounds("attention_mma", keys)
                _check(lib, lib.pae_paged_attention_prefill(
                    _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1],
                    _ptr(q_start), _ptr(q_pos0), _ptr(kv_len), seqs, max_q_len, num_heads,
                    num_kv_heads, head_dim, page_size, scale, window,
                    1, _ptr(listed), (listed.numel() if listed is not None else 0), _stream()))
            if singles != 0:
                _decode_attention(lib, out, qkv, keys, values, block_table, q_start, kv_len, seqs, singles, num_heads,
                                  num_kv_heads, head_dim, page_size, max_kv_len, scale, window)
            return out
    if info is not None:
        info.update(kernel="simt")
    lib = _lib("attention_simt")
    _set_bounds("attention_simt", keys)
    _check(lib, lib.pae_paged_attention_simt(
        _ptr(out), _ptr(qkv), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1], _ptr(q_start),
        _ptr(q_pos0), _ptr(kv_len), seqs, max_q_len, num_heads, num_kv_heads,
        head_dim, page_size, scale, window, (_code(qkv)), _stream()))
    return out


def silu_mul(gate_up, block: int = 0) -> torch.Tensor:
    """silu(gate) * up of a [tokens, 2 I] product. block 0: gate is columns [0, I) and up [I, 2 I);
    block b: b gate columns, then their b up columns, and so on (`linear_swiglu`'s weight layout)."""
    tokens, two_i = gate_up.shape
    if two_i % 2 or (block and two_i % (2 * block)):
        raise KernelError(f"silu_mul: rows of {two_i} do not split into gate and up (blocks of {block})")
    if (isinstance(gate_up, PendingSum) and gate_up.value is None and gate_up.bias is None and gate_up.residual is None
            and not gate_up.activation):
        splits = gate_up.partial.shape[0]
        out = torch.empty((tokens, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_silu_mul(_ptr(out), _ptr(gate_up.partial), splits, tokens,
                                            (two_i // 2), block, _DTYPE_CODE[gate_up.dtype], _stream()))
        return out
    gate_up = materialized(gate_up)
    _need(gate_up, "silu_mul: gate_up")
    out = torch.empty((tokens, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    lib = _lib("elementwise")
    _check(lib, lib.pae_silu_mul(_ptr(out), _ptr(gate_up), tokens, (two_i // 2), block,
                                 (_code(gate_up)), _stream()))
    return out


SWIGLU_BLOCK = 16


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor | None:
    """[2 I, K] with 16 gate rows, their 16 up rows, and so on: the weight layout of
    `linear_swiglu`, in which a product's tile holds gate and up of the same columns. None
    when I is not a multiple of 16."""
    inter, k = gate.shape
    if inter % SWIGLU_BLOCK:
        return None
    both = torch.stack((gate.view(inter // SWIGLU_BLOCK, SWIGLU_BLOCK, k), up.view(inter // SWIGLU_BLOCK, SWIGLU_BLOCK, k)), dim=1)
    return both.reshape(2 * inter, k).contiguous()


def linear_swiglu(x, weight) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) -> [M, I] for a weight from `interleave_gate_up`. With many
    tokens the activation runs in the product's epilogue; with few, in the kernel that sums the
    splits; otherwise as a kernel of its own. Gate and up are rounded to the engine dtype first in
    every one of them, so all give the same bits."""
    source, norm_weight, eps = _norm_of(x)
    if (_few_tokens(source, weight.shape[1], norm_weight is not None, GATE_UP_KIND, weight.shape[0]) and weight.dtype == torch.bfloat16 and weight.is_contiguous()
            and weight.data_ptr() % 16 == 0 and weight.shape[0] % 32 == 0 and source.shape[1] == weight.shape[1]):
        _need(source, "linear_swiglu: x")
        out = torch.empty((source.shape[0], weight.shape[0] // 2), dtype=torch.bfloat16, device=source.device)
        lib = _lib("gemv_mma")
        _check(lib, lib.pae_linear_swiglu_few_tokens(_ptr(out), _ptr(source), _ptr(weight), _ptr(norm_weight), eps,
                                                     source.shape[0], weight.shape[0], weight.shape[1],
                                                     _ptr(_error_flag(source.device)), _stream()))
        return out
    x = materialized(x)
    m, k = x.shape
    n = weight.shape[0]
    if (m > SWIGLU_SWAPPED_MAX_TOKENS and n >= 256 and n % 32 == 0 and _tensor_core_shape(x, weight, None, x.dtype)
            and weight.shape[1] == k):
        _need(x, "linear_swiglu: x")
        _need(weight, "linear_swiglu: weight")
        out = torch.empty((m, n // 2), dtype=x.dtype, device=x.device)
        lib = _lib("gemm_tcgen05")
        _check(lib, lib.pae_linear_swiglu_tcgen05(_ptr(out), _ptr(x), _ptr(weight), m, n, k,
                                                  _ptr(_error_flag(x.device)), _stream()))
        return out
    return silu_mul(linear(x, weight), SWIGLU_BLOCK)


def sample(logits, temperature, seed_lo, seed_hi, request_key, output_index, keep=None) -> torch.Tensor:
    """int32 [rows]: argmax where temperature is 0, else the Gumbel-max draw of the row's counters.
    `keep` = (last_token, logit_rows, seq_index, state_slot): the kernel that picks a row's token
    also does what `scatter_tokens` would (one launch fewer in a step)."""
    _need(logits, "sample: logits", torch.float32)
    _need(temperature, "sample: temperature", torch.float32)
    for name, t in (("seed_lo", seed_lo), ("seed_hi", seed_hi), ("request_key", request_key), ("output_index", output_index)):
        _need(t, f"sample: {name}", torch.int32)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    words = lib.pae_sample_scratch_words(rows, vocab)
    scratch = torch.empty(words, dtype=torch.int32, device=logits.device) if words else None
    kept = (None, None, None, None)
    if keep is not None:
        kept = keep
        for name, t in zip(("last_token", "logit_rows", "seq_index", "state_slot"), kept):
            _need(t, f"sample: {name}", torch.int32)
        if kept[1].numel() != rows:
            raise KernelError(f"sample: {rows} rows of logits, {kept[1].numel()} wanted places")
    _check(lib, lib.pae_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(seed_lo), _ptr(seed_hi),
                               _ptr(request_key), _ptr(output_index), rows, vocab, _ptr(scratch),
                               _ptr(kept[0]), _ptr(kept[1]), _ptr(kept[2]), _ptr(kept[3]),
                               _stream()), 2 if words else 1)
    return out


# ----------------------------------------------------------------------------------- #
# Kernels of decoders with a float32 residual stream, short convolutions, a scored
# attention rule and recurrent state (csrc/norm_act.cu, short_conv.cu, attention_scored.cu,
# delta_rule.cu). Each takes the engine's element type where it reads or writes
# activations and float32 where the arithmetic is float32 by design.
# ----------------------------------------------------------------------------------- #

def embedding_positions(ids, positions, table, position_table, feedback=None, position_scale: float = 1.0) -> torch.Tensor:
    """float32 [tokens, width]: table[id] + position_scale * position_table[position]. `feedback`
    as in `embedding`."""
    _need(table, "embedding_positions: table")
    _need(position_table, "embedding_positions: position table", table.dtype)
    _need(ids, "embedding_positions: ids", torch.int32)
    _need(positions, "embedding_positions: positions", torch.int32)
    if position_table.shape[1] != table.shape[1]:
        raise KernelError(f"embedding_positions: rows of {table.shape[1]} and of {position_table.shape[1]}")
    last_token, state_slot, seq_index = feedback if feedback is not None else (None, None, None)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    lib = _lib("norm_act")
    _check(lib, lib.pae_embedding_positions(_ptr(out), _ptr(table), _ptr(position_table), _ptr(ids), _ptr(positions),
                                            _ptr(last_token), _ptr(state_slot), _ptr(seq_index), ids.numel(),
                                            table.shape[0], position_table.shape[0], table.shape[1], position_scale, 1.0,
                                            _code(table), _stream()))
    return out


def embedding_scaled(ids, table, scale: float, feedback=None) -> torch.Tensor:
    """float32 [tokens, width]: scale * table[id]. `feedback` as in `embedding`."""
    _need(table, "embedding_scaled: table")
    _need(ids, "embedding_scaled: ids", torch.int32)
    last_token, state_slot, seq_index = feedback if feedback is not None else (None, None, None)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    lib = _lib("norm_act")
    _check(lib, lib.pae_embedding_positions(_ptr(out), _ptr(table), None, _ptr(ids), None, _ptr(last_token), _ptr(state_slot),
                                            _ptr(seq_index), ids.numel(), table.shape[0], 0, table.shape[1], 0.0, float(scale),
                                            _code(table), _stream()))
    return out


def rms_norm_cast(x, weight: torch.Tensor, eps: float, out_dtype=None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis; x float32 or the engine's dtype, the
    result in `out_dtype` (x's when None)."""
    _need(weight, "rms_norm_cast: weight", torch.float32)
    if (isinstance(x, PendingSum) and x.value is None and not x.activation and x.dtype == torch.float32 and fuse_split_sums
            and weight.numel() == x.shape[-1]):
        # the sum of a split product (+ bias + residual) and the norm of the result as one kernel
        splits, m, n = x.partial.shape
        value = torch.empty((m, n), dtype=torch.float32, device=x.device)
        normed = torch.empty((m, n), dtype=out_dtype or torch.float32, device=x.device)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_rms_norm_cast(_ptr(normed), _ptr(value), _ptr(x.partial), splits, _ptr(x.bias), _ptr(x.residual),
                                                 _ptr(weight), m, n, eps, _code(normed), _stream()))
        x.value = value
        return normed
    x = materialized(x)
    _need(x, "rms_norm_cast: x")
    width = x.shape[-1]
    if weight.numel() != width:
        raise KernelError(f"rms_norm_cast: weight of {weight.numel()} for rows of {width}")
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    rows = x.numel() // width if x.numel() else 0
    lib = _lib("norm_act")
    _check(lib, lib.pae_rms_norm_cast(_ptr(out), _ptr(x), _ptr(weight), rows, width, eps, _code(x), _code(out), _stream()))
    return out


def rms_norm_columns(x, offset: int, width: int, weight: torch.Tensor, eps: float, out_dtype) -> torch.Tensor:
    """The RMS norm, times `weight`, of columns [offset, offset + width) of float32 rows, in `out_dtype`
    [rows, width]: a part of a fused projection that is normed on its own (a latent)."""
    x = materialized(x)
    _need(x, "rms_norm_columns: x", torch.float32)
    _need(weight, "rms_norm_columns: weight", torch.float32)
    if weight.numel() != width:
        raise KernelError(f"rms_norm_columns: weight of {weight.numel()} for {width} columns")
    out = torch.empty((x.shape[0], width), dtype=out_dtype, device=x.device)
    lib = _lib("norm_act")
    _check(lib, lib.pae_rms_norm_columns(_ptr(out), _ptr(x), x.shape[1], offset, _ptr(weight), x.shape[0], width, float(eps),
                                         _DTYPE_CODE[out_dtype], _stream()))
    return out


def clamped_glu(gate_up, limit: float, alpha: float, out_dtype=None) -> torch.Tensor:
    """g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), for
    rows [tokens, 2 I] that hold the gate in columns [0, I) and the up projection in [I, 2 I)."""
    if (isinstance(gate_up, PendingSum) and gate_up.value is None and gate_up.residual is None and not gate_up.activation
            and fuse_split_sums and gate_up.shape[1] % 2 == 0 and out_dtype is not None):
        splits, tokens, two_i = gate_up.partial.shape
        out = torch.empty((tokens, two_i // 2), dtype=out_dtype, device=gate_up.device)
        lib = _lib("fused_decode")
        _check(lib, lib.pae_splitk_clamped_glu(_ptr(out), _ptr(gate_up.partial), splits, _ptr(gate_up.bias), tokens, two_i // 2,
                                               float(limit), float(alpha), _code(out), _stream()))
        return out
    gate_up = materialized(gate_up)
    _need(gate_up, "clamped_glu: gate_up")
    tokens, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"clamped_glu: rows of {two_i} do not split into gate and up")
    out = torch.empty((tokens, two_i // 2), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    lib = _lib("norm_act")
    _check(lib, lib.pae_clamped_glu(_ptr(out), _ptr(gate_up), tokens, two_i // 2, float(limit), float(alpha), _code(gate_up),
                                    _code(out), _stream()))
    return out


def softcap(logits, cap: float) -> torch.Tensor:
    """cap * tanh(logits / cap), float32, in place."""
    logits = materialized(logits)
    _need(logits, "softcap: logits", torch.float32)
    lib = _lib("norm_act")
    _check(lib, lib.pae_softcap(_ptr(logits), logits.numel(), float(cap), _stream()))
    return logits


def head_prep(proj, *, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, q_dim: int, k_dim: int, value_dim: int,
              q_norm, k_norm, q_span: int, k_span: int, eps: float, table, interleaved: bool, q_rot0: int, k_rot0: int,
              slots, keys, values, page_size: int, out_dtype, whole: bool = False) -> torch.Tensor:
    """From a fused projection [tokens, ld] to attention's operands (csrc/head_prep.cu): every
    query head (q_dim channels at q_off) and key head (k_dim channels at k_off) is RMS-normed over
    its first q_span / k_span channels with the weight q_norm / k_norm (None: not normed; `whole`:
    ONE norm over all query heads of the token and one over all key heads, the weights as long as
    those projections), the span
    of `table.shape[1]` channels from q_rot0 / k_rot0 is rotated by the table (pairs (i, i + half),
    or (2i, 2i + 1) when `interleaved`), the queries are returned as [tokens, heads * q_dim] in
    `out_dtype`, and keys and values (value_dim channels at v_off; `values` None: none) are written
    to their pages at `slots` (None: nothing is written and kv_heads is ignored)."""
    proj = materialized(proj)
    _need(proj, "head_prep: projection")
    tokens, ld = proj.shape
    writes = slots is not None and kv_heads > 0
    need = max(q_off + heads * q_dim, (k_off + kv_heads * k_dim) if writes else 0,
               (v_off + kv_heads * value_dim) if writes and values is not None else 0)
    if need > ld:
        raise KernelError(f"head_prep: columns up to {need} of rows of {ld}")
    for name, t, n in (("q_norm", q_norm, q_span * (heads if whole else 1)), ("k_norm", k_norm, k_span * (kv_heads if whole else 1))):
        if t is not None and n > 0:
            _need(t, f"head_prep: {name}", torch.float32)
            if t.numel() != n:
                raise KernelError(f"head_prep: {name} has {t.numel()} numbers, {n} are needed")
    dims = 0
    if table is not None:
        _need(table, "head_prep: table", torch.float32)
        if table.shape[0] != tokens:
            raise KernelError(f"head_prep: a table of {table.shape[0]} rows for {tokens} tokens")
        dims = int(table.shape[1])
    if writes:
        _need(slots, "head_prep: slots", torch.int32)
        _need(keys, "head_prep: keys", out_dtype)
        if values is not None:
            _need(values, "head_prep: values", out_dtype)
    q = torch.empty((tokens, heads * q_dim), dtype=out_dtype, device=proj.device)
    lib = _lib("head_prep")
    _set_bounds("head_prep", keys if writes else None)
    _check(lib, lib.pae_head_prep(
        _ptr(q), _ptr(keys if writes else None), _ptr(values if writes else None), _ptr(proj), ld, q_off, k_off, v_off, tokens,
        heads, kv_heads if writes else 0, q_dim, k_dim, value_dim if values is not None else 0, _ptr(q_norm), q_span,
        _ptr(k_norm), k_span, float(eps), _ptr(table), dims, 1 if interleaved else 0, q_rot0, k_rot0,
        _ptr(slots if writes else None), page_size, 1 if whole else 0, _code(proj), _DTYPE_CODE[out_dtype], _stream()))
    return q


def sigmoid_gate(x, gate_proj, gate_off: int, group: int = 1) -> torch.Tensor:
    """x * sigmoid(gate_proj[:, gate_off : gate_off + x.shape[1] / group]): a gate column for every
    `group` neighbouring channels of x (1: a gate per channel; a head's size: a gate per head)."""
    x = materialized(x)
    gate_proj = materialized(gate_proj)
    _need(x, "sigmoid_gate: x")
    _need(gate_proj, "sigmoid_gate: gate")
    if gate_proj.shape[0] != x.shape[0]:
        raise KernelError(f"sigmoid_gate: {x.shape[0]} rows and {gate_proj.shape[0]} rows of gates")
    out = torch.empty_like(x)
    lib = _lib("head_prep")
    if group < 1 or x.shape[1] % group:
        raise KernelError(f"sigmoid_gate: rows of {x.shape[1]} channels do not split into groups of {group}")
    _check(lib, lib.pae_sigmoid_gate(_ptr(out), _ptr(x), _ptr(gate_proj), x.shape[0], x.shape[1], gate_proj.shape[1], gate_off,
                                     group, _code(x), _code(gate_proj), _stream()))
    return out


def linear_heads(x, weight, heads: int, in_stride: int, tail: int = 0) -> torch.Tensor:
    """One product per head (csrc/linear_heads.cu): x [tokens, heads * in_stride], of which a head's
    first K channels are the operand and the next `tail` pass through; weight [heads, N, K] ->
    [tokens, heads * (N + tail)]."""
    x = materialized(x)
    _need(x, "linear_heads: x")
    _need(weight, "linear_heads: weight", x.dtype)
    if weight.dim() != 3 or weight.shape[0] != heads:
        raise KernelError(f"linear_heads: weight is {tuple(weight.shape)} for {heads} heads")
    n, k = int(weight.shape[1]), int(weight.shape[2])
    if x.shape[1] != heads * in_stride or k + tail > in_stride:
        raise KernelError(f"linear_heads: rows of {x.shape[1]} for {heads} heads of {k} + {tail} channels at a stride of {in_stride}")
    out = torch.empty((x.shape[0], heads * (n + tail)), dtype=x.dtype, device=x.device)
    lib = _lib("linear_heads")
    _check(lib, lib.pae_linear_heads(_ptr(out), _ptr(x), _ptr(weight), x.shape[0], heads, n, k, tail, x.shape[1], in_stride,
                                     out.shape[1], n + tail, _code(x), _stream()))
    return out


def matrix_memory(proj, offsets, i_bias, f_bias, norm_weight, state, q_start, state_slot, num_seqs: int, num_heads: int,
                  head_dim: int, value_dim: int, gate_cap: float, q_scale: float, norm_eps: float, out_dtype) -> torch.Tensor:
    """The matrix memory (mLSTM) over the step's tokens, from and into the per-request state (float32
    [slots, heads, head_dim * (value_dim + 1) + 1]): see csrc/matrix_memory.cu. `proj` float32
    [tokens, ld] holds q, k, v, the output gate's and the two gates' projections at `offsets` =
    (q, k, v, g, i, f). Returns rms_norm_per_head(o) * norm_weight * sigmoid(g) as [tokens, heads *
    value_dim] in `out_dtype`."""
    proj = materialized(proj)
    _need(proj, "matrix_memory: projections", torch.float32)
    _need(state, "matrix_memory: state", torch.float32)
    for name, t, n in (("i bias", i_bias, num_heads), ("f bias", f_bias, num_heads), ("norm weight", norm_weight, num_heads * value_dim)):
        _need(t, f"matrix_memory: {name}", torch.float32)
        if t.numel() != n:
            raise KernelError(f"matrix_memory: {name} has {t.numel()} numbers, {n} are needed")
    _need(q_start, "matrix_memory: q_start", torch.int32)
    _need(state_slot, "matrix_memory: state_slot", torch.int32)
    tokens, ld = proj.shape
    lib = _lib("matrix_memory")
    per_head = lib.pae_matrix_memory_state_floats(head_dim, value_dim)
    if tuple(state.shape[1:]) != (num_heads, per_head):
        raise KernelError(f"matrix_memory: state rows are {tuple(state.shape[1:])}, ({num_heads}, {per_head}) is needed")
    q_off, k_off, v_off, g_off, i_off, f_off = offsets
    for off, width in ((q_off, num_heads * head_dim), (k_off, num_heads * head_dim), (v_off, num_heads * value_dim),
                       (g_off, num_heads * value_dim), (i_off, num_heads), (f_off, num_heads)):
        if off < 0 or off + width > ld:
            raise KernelError(f"matrix_memory: columns {off}..{off + width} of rows of {ld}")
    # Few (request, head) pairs leave SMs idle: a head's value columns are shared out over blocks
    # (a column's recurrence needs no other column), each at least a warp wide.
    splits, most, sms = 1, lib.pae_matrix_memory_max_splits(value_dim), _sm_count(proj.device)
    while num_seqs * num_heads * splits < sms and splits * 2 <= most:
        splits *= 2
    o = torch.empty((tokens, num_heads * value_dim), dtype=torch.float32, device=proj.device)
    carry = torch.empty(num_seqs * num_heads * (head_dim + 1), dtype=torch.float32, device=proj.device)
    _check(lib, lib.pae_matrix_memory_scan(_ptr(o), _ptr(state), _ptr(carry), _ptr(proj), ld, q_off, k_off, v_off, i_off, f_off,
                                           _ptr(i_bias), _ptr(f_bias), _ptr(q_start), _ptr(state_slot), num_seqs, num_heads,
                                           head_dim, value_dim, splits, float(gate_cap), float(q_scale), _stream()), 2)
    out = torch.empty((tokens, num_heads * value_dim), dtype=out_dtype, device=proj.device)
    _check(lib, lib.pae_matrix_memory_output(_ptr(out), _ptr(o), _ptr(proj), ld, g_off, _ptr(norm_weight), tokens, num_heads,
                                             value_dim, float(norm_eps), _DTYPE_CODE[out_dtype], _stream()))
    return out


def layer_norm(x, weight: torch.Tensor, bias: torch.Tensor | None, eps: float, out_dtype=None) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight + bias over the last axis; x float32 or the engine's
    dtype, the result in `out_dtype` (x's when None)."""
    x = materialized(x)
    _need(x, "layer_norm: x")
    _need(weight, "layer_norm: weight", torch.float32)
    if bias is not None:
        _need(bias, "layer_norm: bias", torch.float32)
    width = x.shape[-1]
    if weight.numel() != width or (bias is not None and bias.numel() != width):
        raise KernelError(f"layer_norm: weight of {weight.numel()} for rows of {width}")
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    rows = x.numel() // width if x.numel() else 0
    lib = _lib("norm_act")
    _check(lib, lib.pae_layer_norm(_ptr(out), _ptr(x), _ptr(weight), _ptr(bias), rows, width, eps, _code(x), _code(out), _stream()))
    return out


GELU_KINDS = {"gelu_erf": 0, "gelu_tanh": 1, "relu2": 2}


def gelu(x, kind: str = "gelu_erf") -> torch.Tensor:
    x = materialized(x)
    _need(x, "gelu: x")
    if kind not in GELU_KINDS:
        raise KernelError(f"gelu: kind '{kind}' (known: {', '.join(GELU_KINDS)})")
    out = torch.empty_like(x)
    lib = _lib("norm_act")
    _check(lib, lib.pae_gelu(_ptr(out), _ptr(x), x.numel(), GELU_KINDS[kind], _code(x), _stream()))
    return out


def conv_heads_cache_write(proj, taps_weight, state, positions, seq_index, q_start, q_pos0, state_slot, slots, keys,
                           values, num_heads, num_kv_heads, head_dim, value_dim, page_size, normalize: bool, eps: float,
                           out_dtype) -> torch.Tensor:
    """The short causal convolution of a float32 q|k|v projection [tokens, channels] (taps_weight
    float32 [channels, taps] or None; state float32 [slots, taps - 1, channels] holds every
    request's last projected rows and is brought up to date), unit RMS per q and k head when
    `normalize`, k and v written to their pages at `slots`. Returns q [tokens, heads * head_dim]
    in `out_dtype`."""
    proj = materialized(proj)
    _need(proj, "conv_heads_cache_write: projection", torch.float32)
    channels = (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim
    tokens = proj.shape[0]
    if proj.shape[1] != channels:
        raise KernelError(f"conv_heads_cache_write: rows of {proj.shape[1]} for {channels} channels")
    taps = 1
    if taps_weight is not None:
        _need(taps_weight, "conv_heads_cache_write: taps", torch.float32)
        if taps_weight.dim() != 2 or taps_weight.shape[0] != channels:
            raise KernelError(f"conv_heads_cache_write: taps are {tuple(taps_weight.shape)} for {channels} channels")
        taps = int(taps_weight.shape[1])
    if taps > 1:
        _need(state, "conv_heads_cache_write: state", torch.float32)
        if tuple(state.shape[1:]) != (taps - 1, channels):
            raise KernelError(f"conv_heads_cache_write: state rows are {tuple(state.shape[1:])}, ({taps - 1}, {channels}) is needed")
    for name, t in (("positions", positions), ("seq_index", seq_index), ("q_start", q_start), ("q_pos0", q_pos0),
                    ("state_slot", state_slot)):
        _need(t, f"conv_heads_cache_write: {name}", torch.int32)
    if slots is not None:
        _need(slots, "conv_heads_cache_write: slots", torch.int32)
        _need(keys, "conv_heads_cache_write: keys", out_dtype)
        _need(values, "conv_heads_cache_write: values", out_dtype)
    q = torch.empty((tokens, num_heads * head_dim), dtype=out_dtype, device=proj.device)
    lib = _lib("short_conv")
    _set_bounds("short_conv", keys if slots is not None else None)
    _check(lib, lib.pae_conv_heads_cache_write(
        _ptr(q), _ptr(keys if slots is not None else None), _ptr(values if slots is not None else None), _ptr(proj),
        _ptr(taps_weight), _ptr(state if taps > 1 else None), _ptr(positions), _ptr(seq_index), _ptr(q_start), _ptr(q_pos0),
        _ptr(state_slot), _ptr(slots), tokens, taps, num_heads, num_kv_heads, head_dim, value_dim, page_size,
        1 if normalize else 0, eps, _DTYPE_CODE[out_dtype], _stream()))
    if taps > 1:
        _check(lib, lib.pae_conv_state_update(_ptr(state), _ptr(proj), _ptr(q_start), _ptr(q_pos0), _ptr(state_slot),
                                              state_slot.numel(), taps, channels, _stream()))
    return q


def paged_attention_scored(q, keys, values, block_table, q_start, q_pos0, kv_len, num_heads, num_kv_heads, head_dim,
                           value_dim, page_size, max_q_len, scale, softcap=0.0, temp=None, r1=None, r2=None, sink=None,
                           window: int = 0, keep_first: int = 0, form: str | None = None, max_kv_len: int | None = None,
                           num_single: int | None = None) -> torch.Tensor:
    """Attention of every token of the step over its request's pages under a score rule:
    (q . k) * scale * temp[h], capped by softcap * tanh(. / softcap), minus r1[h] * log(1 + r2[h] *
    distance), a window that keeps the first `keep_first` keys, and a sink logit per head in the
    softmax's denominator. temp, r1, r2, sink are float32 [heads] or None. -> [tokens, heads * value_dim].
    bfloat16 with head sizes of 32, 64 or 128 runs on tensor cores (csrc/attention_scored_mma.cu), everything
    else, and everything when `form` is "simt", on the CUDA cores (csrc/attention_scored.cu). `max_kv_len` (the
    longest context of the step) and `num_single` (how many requests bring one token) let the tensor-core
    kernel share a single token's keys out over several blocks."""
    q = materialized(q)
    _need(q, "paged_attention_scored: q")
    _need(keys, "paged_attention_scored: keys", q.dtype)
    _need(values, "paged_attention_scored: values", q.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_pos0", q_pos0), ("kv_len", kv_len)):
        _need(t, f"paged_attention_scored: {name}", torch.int32)
    for name, t in (("temp", temp), ("r1", r1), ("r2", r2), ("sink", sink)):
        if t is not None:
            _need(t, f"paged_attention_scored: {name}", torch.float32)
            if t.numel() != num_heads:
                raise KernelError(f"paged_attention_scored: {name} has {t.numel()} numbers for {num_heads} heads")
    tokens = q.shape[0]
    if q.shape[1] != num_heads * head_dim:
        raise KernelError(f"paged_attention_scored: q rows of {q.shape[1]} for {num_heads} heads of {head_dim}")
    out = torch.empty((tokens, num_heads * value_dim), dtype=q.dtype, device=q.device)
    in_keys = values.data_ptr() == keys.data_ptr()        # a key row's leading channels are its value
    if (in_keys and q.dtype == torch.bfloat16 and use_tensor_cores and form != "simt" and num_kv_heads == 1 and not keep_first
            and not softcap and temp is None and r1 is None and sink is None):
        # Many heads over one latent key/value head, causal or windowed (csrc/attention_latent_mma.cu). A request that brings one
        # token is blocks of up to 32 heads; its keys are shared out (two tiles of 64 a block at least) until the launch fills the GPU once.
        lib = _lib("attention_latent_mma")
        if lib.pae_attention_latent_mma_supports(head_dim, value_dim):
            _set_bounds("attention_latent_mma", keys)
            seqs = kv_len.numel()
            splits, scratch = 1, None
            if num_single is None or num_single > 0:
                groups = -(-num_heads // 32)
                reach = min(max_kv_len or 0, window + 63) if window else (max_kv_len or 0)       # a window's keys and the tile they start in
                splits = max(1, min(-(-reach // 128), _sm_count(q.device) // max(1, seqs * groups)))
                scratch = torch.empty(seqs * num_heads * splits * (value_dim + 2), dtype=torch.float32, device=q.device)
            _check(lib, lib.pae_paged_attention_latent_mma(
                _ptr(out), _ptr(q), _ptr(keys), _ptr(block_table), block_table.shape[1], _ptr(q_start), _ptr(q_pos0), _ptr(kv_len),
                seqs, max_q_len, num_heads, head_dim, value_dim, page_size, scale, int(window or 0), splits, _ptr(scratch), _stream()),
                2 if scratch is not None else 1)
            return out
    if (q.dtype == torch.bfloat16 and use_tensor_cores and head_dim in (32, 64, 128) and value_dim in (32, 64, 128)
            and form != "simt" and not in_keys):
        lib = _lib("attention_scored_mma")
        _set_bounds("attention_scored_mma", keys)
        # A request that brings one token is one row of one block per head: its keys are shared out
        # over blocks until the launch fills the GPU about twice (64 keys a tile, at least one tile each;
        # with four times as many blocks a step was slower: 0.63 against 0.60 ms at batch 8, 1.78 against 1.60 at 64).
        seqs = kv_len.numel()
        reach = min(max_kv_len, window + keep_first) if window and max_kv_len else (max_kv_len or 0)
        splits, scratch = 1, None
        if (num_single is None or num_single > 0) and num_heads // num_kv_heads <= 64:
            splits = max(1, min(-(-reach // 64), (6 * _sm_count(q.device)) // max(1, seqs * num_kv_heads)))
            scratch = torch.empty(seqs * num_heads * splits * (value_dim + 2), dtype=torch.float32, device=q.device)
        _check(lib, lib.pae_paged_attention_scored_mma(
            _ptr(out), _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1], _ptr(q_start),
            _ptr(q_pos0), _ptr(kv_len), kv_len.numel(), max_q_len, num_heads, num_kv_heads, head_dim, value_dim, page_size,
            scale, float(softcap or 0.0), _ptr(temp), _ptr(r1), _ptr(r2), _ptr(sink), int(window), int(keep_first),
            splits, _ptr(scratch), _stream()), 2 if scratch is not None else 1)
        return out
    lib = _lib("attention_scored")
    _set_bounds("attention_scored", keys)
    _check(lib, lib.pae_paged_attention_scored(
        _ptr(out), _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), block_table.shape[1], _ptr(q_start), _ptr(q_pos0),
        _ptr(kv_len), kv_len.numel(), max_q_len, num_heads, num_kv_heads, head_dim, value_dim, page_size, scale,
        float(softcap or 0.0), _ptr(temp), _ptr(r1), _ptr(r2), _ptr(sink), int(window), int(keep_first), _code(q), _stream()))
    return out


def tanh_columns(x, offset: int, width: int, out_dtype) -> torch.Tensor:
    """tanh of columns [offset, offset + width) of float32 rows, in `out_dtype`."""
    x = materialized(x)
    _need(x, "tanh_columns: x", torch.float32)
    if offset < 0 or offset + width > x.shape[1]:
        raise KernelError(f"tanh_columns: columns {offset}..{offset + width} of rows of {x.shape[1]}")
    out = torch.empty((x.shape[0], width), dtype=out_dtype, device=x.device)
    lib = _lib("delta_rule")
    _check(lib, lib.pae_tanh_columns(_ptr(out), _ptr(x), x.shape[0], x.shape[1], offset, width, _DTYPE_CODE[out_dtype], _stream()))
    return out


_SM_COUNT: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNT[index]


def delta_rule(proj, offsets, w_pre, w0, a_bias, gate_offset, norm_weight, state, q_start, state_slot, num_seqs, num_heads,
               head_dim, decay_scale: float, key_eps: float, norm_eps: float, out_dtype) -> torch.Tensor:
    """The generalized delta rule over the step's tokens, from and into the per-request state
    (float32 [slots, heads, head_dim, head_dim]): see csrc/delta_rule.cu. `proj` float32 [tokens, ld]
    holds r, k, v, the removal rate's and the gate's projections at `offsets` = (r, k, v, a) and
    `gate_offset`; `w_pre` float32 [tokens, heads * head_dim] the decay's. Returns
    rms_norm_per_head(o) * norm_weight * sigmoid(gate) as [tokens, heads * head_dim] in `out_dtype`."""
    proj = materialized(proj)
    w_pre = materialized(w_pre)
    _need(proj, "delta_rule: projections", torch.float32)
    _need(w_pre, "delta_rule: decay projection", torch.float32)
    _need(state, "delta_rule: state", torch.float32)
    for name, t in (("w0", w0), ("a_bias", a_bias), ("norm weight", norm_weight)):
        _need(t, f"delta_rule: {name}", torch.float32)
        if t.numel() != num_heads * head_dim:
            raise KernelError(f"delta_rule: {name} has {t.numel()} numbers for {num_heads} heads of {head_dim}")
    _need(q_start, "delta_rule: q_start", torch.int32)
    _need(state_slot, "delta_rule: state_slot", torch.int32)
    tokens, ld = proj.shape
    width = num_heads * head_dim
    if tuple(w_pre.shape) != (tokens, width):
        raise KernelError(f"delta_rule: the decay projection is {tuple(w_pre.shape)}, [{tokens}, {width}] is needed")
    if tuple(state.shape[1:]) != (num_heads, head_dim, head_dim):
        raise KernelError(f"delta_rule: state rows are {tuple(state.shape[1:])}")
    for off in (*offsets, gate_offset):
        if off < 0 or off + width > ld:
            raise KernelError(f"delta_rule: columns {off}..{off + width} of rows of {ld}")
    lib = _lib("delta_rule")
    per_column = c_int(0)
    if lib.pae_delta_rule_layout(head_dim, ctypes.byref(per_column)) == 0:
        raise KernelError(f"delta_rule: head size {head_dim} is not supported (1 to 256)")
    # Few (request, head) pairs leave SMs idle: a head's value channels are shared out over blocks
    # (the recurrence of a value channel needs no other), at least a warp's worth of threads each.
    splits, sms = lib.pae_delta_rule_min_splits(head_dim), _sm_count(proj.device)
    while (num_seqs * num_heads * splits < 2 * sms and head_dim % (2 * splits) == 0
           and (head_dim // (2 * splits)) * per_column.value >= 128):
        splits *= 2
    o = torch.empty((tokens, width), dtype=torch.float32, device=proj.device)
    prepared = torch.empty(lib.pae_delta_rule_scratch_floats(tokens, num_heads, head_dim), dtype=torch.float32, device=proj.device)
    _check(lib, lib.pae_delta_rule_scan(_ptr(o), _ptr(state), _ptr(prepared), _ptr(proj), ld, offsets[0], offsets[1],
                                        offsets[2], offsets[3], _ptr(w_pre), _ptr(w0), _ptr(a_bias), _ptr(q_start),
                                        _ptr(state_slot), tokens, num_seqs, num_heads, head_dim, splits, decay_scale, key_eps,
                                        _stream()), 2)
    out = torch.empty((tokens, width), dtype=out_dtype, device=proj.device)
    _check(lib, lib.pae_delta_rule_output(_ptr(out), _ptr(o), proj.data_ptr() + 4 * gate_offset, ld, _ptr(norm_weight), tokens,
                                          num_heads, head_dim, norm_eps, _DTYPE_CODE[out_dtype], _stream()))
    return out


# ----------------------------------------------------------------------------------- #
# Norms without statistics around both sides of a sublayer (csrc/dyt.cu)

def _dyt_step(pending, next_norm, out_dtype):
    """Runs the sum of a PendingResidual (or, for a plain tensor, nothing) and, with `next_norm` =
    (alpha, weight, bias), the Dynamic Tanh of the result in `out_dtype`: one kernel. Keeps the new
    stream in `pending.value` and returns the normed rows or None."""
    if isinstance(pending, PendingResidual):
        x, y, post, mult, extra = materialized(pending.x), pending.y, pending.post, pending.mult, materialized(pending.extra)
    else:
        x, y, post, mult, extra = pending, None, None, 0.0, None
    _need(x, "dyt: the stream", torch.float32)
    tokens, width = x.shape
    planes = 1
    if y is not None:
        y, planes = _sublayer_output(y)
        if tuple(y.shape[-2:]) != (tokens, width):
            raise KernelError(f"dyt: a sublayer's output {tuple(y.shape)} for a stream {tuple(x.shape)}")
    if extra is not None:
        _need(extra, "dyt: the joining stream", torch.float32)
        if tuple(extra.shape) != (tokens, width):
            raise KernelError(f"dyt: a joining stream {tuple(extra.shape)} for a stream {tuple(x.shape)}")
    for name, norm in (("the norm after the sublayer", post), ("the next norm", next_norm)):
        if norm is not None:
            alpha, weight, bias = norm
            _need(alpha, f"dyt: alpha of {name}", torch.float32)
            _need(weight, f"dyt: weight of {name}", torch.float32)
            if weight.numel() != width or alpha.numel() != 1 or (bias is not None and bias.numel() != width):
                raise KernelError(f"dyt: {name} has {weight.numel()} weights for rows of {width}")
            if bias is not None:
                _need(bias, f"dyt: bias of {name}", torch.float32)
    writes = y is not None or extra is not None
    x_new = torch.empty_like(x) if writes else None
    normed = torch.empty((tokens, width), dtype=out_dtype, device=x.device) if next_norm is not None else None
    post = post or (None, None, None)
    nxt = next_norm or (None, None, None)
    if writes or normed is not None:
        lib = _lib("dyt")
        _check(lib, lib.pae_dyt_step(_ptr(x_new), _ptr(normed), _ptr(x), _ptr(y), planes, _ptr(extra), _ptr(post[0]), _ptr(post[1]),
                                     _ptr(post[2]), float(mult), _ptr(nxt[0]), _ptr(nxt[1]), _ptr(nxt[2]), tokens, width,
                                     _DTYPE_CODE[out_dtype] if out_dtype is not None else 0, _stream()))
    if isinstance(pending, PendingResidual):
        pending.value = x_new if writes else x
    return normed


def dyt_norm(x, alpha, weight, bias, out_dtype) -> torch.Tensor:
    """tanh(alpha * x) * weight + bias in `out_dtype`: x float32 [tokens, width], or a residual sum
    that is still pending, which this kernel makes on the way (`materialized(x)` then has it)."""
    if isinstance(x, PendingResidual) and x.value is None:
        return _dyt_step(x, (alpha, weight, bias), out_dtype)
    x = materialized(x)
    if x.dtype != torch.float32:
        raise KernelError(f"dyt_norm: the stream is {x.dtype}, float32 is needed")
    return _dyt_step(x, (alpha, weight, bias), out_dtype)


def residual_add(x, y, mult: float = 1.0, post=None):
    """The stream x + mult * post(y), float32, pending: `post` = (alpha, weight, bias) of a Dynamic Tanh
    over y, or None. The next `dyt_norm` makes the sum in its own kernel."""
    return PendingResidual(x, y, post, mult)


def join_stream(x, extra):
    """The stream x + extra (both float32 [tokens, width]), pending; a pending residual sum takes
    `extra` along in its own kernel."""
    if isinstance(x, PendingResidual) and x.value is None and x.extra is None:
        x.extra = extra
        return x
    return PendingResidual(materialized(x), None, None, 0.0, extra)


# ----------------------------------------------------------------------------------- #
# Hyper-connections (csrc/streams.cu) and routed experts (csrc/routing.cu)

def _sublayer_output(y):
    """(float32 planes [splits, tokens, width], splits) of a sublayer's output that is a tensor or a
    split product without bias, residual or activation."""
    if (isinstance(y, PendingSum) and y.value is None and y.bias is None and y.residual is None and not y.activation
            and y.dtype == torch.float32 and fuse_split_sums):
        return y.partial, int(y.partial.shape[0])
    y = materialized(y)
    _need(y, "streams: the sublayer's output", torch.float32)
    return y, 1


def _streams_launch(x, src_streams: int, streams: int, width: int, y, splits: int, mix, out_w, in_w, norm_w, eps: float, out_dtype):
    tokens = x.shape[0]
    x_new = torch.empty((tokens, streams * width), dtype=torch.float32, device=x.device) if y is not None else None
    normed = torch.empty((tokens, width), dtype=out_dtype, device=x.device) if norm_w is not None else None
    lib = _lib("streams")
    _check(lib, lib.pae_streams_step(_ptr(x_new), _ptr(normed), _ptr(x), src_streams, _ptr(y), splits, _ptr(mix), _ptr(out_w),
                                     _ptr(in_w), _ptr(norm_w), tokens, streams, width, float(eps),
                                     _DTYPE_CODE[out_dtype] if out_dtype is not None else 0, _stream()))
    return x_new, normed


def _streams_step(pending, in_w, norm_w, eps: float, out_dtype):
    """Runs the write of a PendingStreams and, with a norm weight, the read of what it wrote (one
    kernel); keeps the written streams in `pending.value` and returns the normed rows or None."""
    x = materialized(pending.x)
    _need(x, "streams: x", torch.float32)
    y, splits = _sublayer_output(pending.y)
    width, streams = int(y.shape[-1]), pending.streams
    if x.shape[1] not in (width, streams * width):
        raise KernelError(f"streams: rows of {x.shape[1]} for {streams} streams of {width}")
    for name, t, n in (("mix", pending.mix, streams * streams), ("out", pending.out_w, streams)):
        _need(t, f"streams: {name}", torch.float32)
        if t.numel() != n:
            raise KernelError(f"streams: {name} has {t.numel()} numbers, {n} are needed")
    pending.value, normed = _streams_launch(x, x.shape[1] // width, streams, width, y, splits, pending.mix, pending.out_w,
                                            in_w, norm_w, eps, out_dtype)
    return normed


def streams_write(x, y, mix: torch.Tensor, out_w: torch.Tensor, streams: int):
    """The streams after a sublayer: x'_t = sum_s mix[s, t] x_s + out_w[t] y, float32 [tokens, streams *
    width]; x is [tokens, streams * width], or [tokens, width] for streams that are all equal. The
    result is pending: the read that follows runs the write in its own kernel."""
    return PendingStreams(x, y, mix, out_w, streams)


def streams_read_norm(x, in_w, norm_w: torch.Tensor, eps: float, streams: int, out_dtype) -> torch.Tensor:
    """RMS norm of u = sum_s in_w[s] x_s (in_w None: the plain sum) times norm_w, in `out_dtype`; x
    float32 [tokens, streams * width] or [tokens, width] (equal streams), or a pending write."""
    _need(norm_w, "streams_read_norm: norm weight", torch.float32)
    if in_w is not None:
        _need(in_w, "streams_read_norm: read weights", torch.float32)
        if in_w.numel() != streams:
            raise KernelError(f"streams_read_norm: {in_w.numel()} read weights for {streams} streams")
    if isinstance(x, PendingStreams) and x.value is None:
        if x.streams != streams or x.y.shape[-1] != norm_w.numel():
            raise KernelError("streams_read_norm: the pending write has other streams than the read")
        return _streams_step(x, in_w, norm_w, eps, out_dtype)
    x = materialized(x)
    _need(x, "streams_read_norm: x", torch.float32)
    width = norm_w.numel()
    if x.shape[1] not in (width, streams * width):
        raise KernelError(f"streams_read_norm: rows of {x.shape[1]} for {streams} streams of {width}")
    return _streams_launch(x, x.shape[1] // width, streams, width, None, 0, None, None, in_w, norm_w, eps, out_dtype)[1]


def route(logits, correction, top: int, groups: int = 0, keep: int = 0, score: str = "softmax", eps: float = 0.0,
          scale: float = 1.0, dense: bool = True, normalize: bool = True, experts: int | None = None):
    """Chooses `top` experts per token from float32 router logits [tokens, experts] (csrc/routing.cu):
    scores softmax (or sigmoid) of the logits, the choice by score + correction among the experts of
    the `keep` best of `groups` groups (0: all experts), weights score / (sum of the chosen + eps) *
    scale (`normalize` False: score * scale, the chosen scores as they are). `experts` (default: every
    column): the router's outputs are the first `experts` columns of wider rows, whose other columns
    (a gate that the same product computes) are not looked at. -> (chosen int32 [tokens, top], weights
    float32 [tokens, top], dense float32 [tokens, experts] with the weights at the chosen experts'
    columns and 0 elsewhere, or None when `dense` is False)."""
    logits, splits = _sublayer_output(logits)         # a split product's planes are added by the kernel itself
    _need(logits, "route: logits", torch.float32)
    tokens, ld = logits.shape[-2:]
    total = ld if experts is None else int(experts)
    if total > ld:
        raise KernelError(f"route: {total} experts in rows of {ld}")
    if correction is not None:
        _need(correction, "route: correction", torch.float32)
        if correction.numel() != total:
            raise KernelError(f"route: a correction of {correction.numel()} numbers for {total} experts")
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"route: score '{score}' (softmax, sigmoid)")
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    dense = torch.empty((tokens, total), dtype=torch.float32, device=logits.device) if dense else None
    lib = _lib("routing")
    _check(lib, lib.pae_route(_ptr(chosen), _ptr(weights), _ptr(dense), _ptr(logits), splits, ld, _ptr(correction), tokens, total, top,
                              groups, keep, 1 if score == "sigmoid" else 0, 1 if normalize else 0, float(eps), float(scale), _stream()))
    return chosen, weights, dense


EXPERT_TILE = 128
# Up to this many pairs one block sorts them (one launch); beyond, a memset and three kernels.
EXPERT_FEW_PAIRS = 2048


class ExpertPlan:
    """The (token, expert) pairs of a step sorted by expert: `staged` [max_tiles * tile, width] holds
    the tokens' inputs in rows grouped by expert and padded to whole tiles, `tiles` int32 [max_tiles +
    1, 2] each tile's expert (negative: unused) and how many of its rows are pairs, and in its last
    entry how many tiles are in use, `rows` int32 [tokens, top] each pair's row (negative: an expert
    without tensors)."""

    def __init__(self, staged, tiles, rows, experts: int) -> None:
        self.staged, self.tiles, self.rows, self.experts = staged, tiles, rows, experts
        self.max_tiles = tiles.shape[0] - 1


def expert_plan(x, chosen, experts: int, input_weights=None) -> ExpertPlan:
    """Sorts the pairs of `chosen` int32 [tokens, top] by expert and copies every pair's input row
    of x [tokens, width] into the staging matrix (csrc/routing.cu). Experts from `experts` on have no
    tensors and get no rows. `input_weights` float32 [tokens, top]: a pair's row is its weight times
    the token's input (float32 product, rounded once), for experts that are weighted on their input.
    Every shape depends on (tokens, top, experts) alone, so a replayed step keeps its buffers."""
    x = materialized(x)
    _need(x, "expert_plan: x")
    _need(chosen, "expert_plan: chosen", torch.int32)
    tokens, top = chosen.shape
    if input_weights is not None:
        _need(input_weights, "expert_plan: input weights", torch.float32)
        if tuple(input_weights.shape) != (tokens, top):
            raise KernelError(f"expert_plan: weights {tuple(input_weights.shape)} for {tokens} x {top} pairs")
    lib = _lib("routing")
    max_tiles = lib.pae_expert_max_tiles(tokens * top, experts, EXPERT_TILE)
    staged = torch.empty((max_tiles * EXPERT_TILE, x.shape[1]), dtype=x.dtype, device=x.device)
    tiles = torch.empty((max_tiles + 1, 2), dtype=torch.int32, device=x.device)
    rows = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    scratch = torch.empty((2 * experts + tokens * top,), dtype=torch.int32, device=x.device)
    _check(lib, lib.pae_expert_plan(_ptr(scratch), _ptr(tiles), _ptr(rows), _ptr(staged), _ptr(x), _ptr(chosen), _ptr(input_weights), tokens, top,
                                    experts, EXPERT_TILE, max_tiles, x.shape[1], _code(x), _stream()),
           1 if tokens * top <= EXPERT_FEW_PAIRS else 4)
    return ExpertPlan(staged, tiles, rows, experts)


def linear_grouped(x, weight, plan: ExpertPlan, out_dtype=None, activation: str | None = None, swiglu_block: int | None = None) -> torch.Tensor:
    """out[row] = act(x[row] . weight[g(row)]^T) for the rows of the plan's tiles: x [max_tiles *
    tile, K] sorted by expert, weight [experts, N, K]. Rows that are no pair keep what the fresh
    output held (or hold anything). The tcgen05 kernel walks the tiles as it walks a plain product's (bfloat16, K a
    multiple of 8); everything else, float32 above all, takes the CUDA-core kernel. `swiglu_block`
    (0: an expert's rows [0, N/2) are its gate and [N/2, N) its up projection; 16: blocks of 16 gate
    rows and their 16 up rows, the layout of `interleave_gate_up`): the result is silu(gate) * up,
    [rows, N / 2] in x's dtype, in the tcgen05 product's epilogue for blocks of 16, else by `silu_mul`."""
    _need(x, "linear_grouped: x")
    _need(weight, "linear_grouped: weight", x.dtype)
    experts, n, k = weight.shape
    if x.shape[1] != k or experts != plan.experts or x.shape[0] != plan.max_tiles * EXPERT_TILE:
        raise KernelError(f"linear_grouped: x {tuple(x.shape)}, weight {tuple(weight.shape)}, {plan.max_tiles} tiles of {plan.experts} experts")
    if swiglu_block is not None:
        if activation is not None or out_dtype not in (None, x.dtype):
            raise KernelError("linear_grouped: SiLU x up leaves the operands' dtype and takes no other activation")
        if swiglu_block == SWIGLU_BLOCK and n % 32 == 0 and _tensor_core_shape(x, weight, None, x.dtype):
            out = torch.empty((x.shape[0], n // 2), dtype=x.dtype, device=x.device)
            lib = _lib("gemm_tcgen05")
            _check(lib, lib.pae_linear_grouped_swiglu_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(plan.tiles), plan.max_tiles, experts,
                                                              n, k, _ptr(_error_flag(x.device)), _stream()))
            return out
        return silu_mul(linear_grouped(x, weight, plan), swiglu_block)
    out_dtype = out_dtype or x.dtype
    out = torch.empty((x.shape[0], n), dtype=out_dtype, device=x.device)
    max_tiles = plan.max_tiles
    if _tensor_core_shape(x, weight, None, out_dtype):
        lib = _lib("gemm_tcgen05")
        _check(lib, lib.pae_linear_grouped_tcgen05(_ptr(out), _ptr(x), _ptr(weight), _ptr(plan.tiles), max_tiles, experts, n, k,
                                                   1 if out_dtype == torch.float32 else 0, ACTIVATIONS[activation],
                                                   _ptr(_error_flag(x.device)), _stream()))
        return out
    lib = _lib("gemm_simt")
    _check(lib, lib.pae_linear_grouped_simt(_ptr(out), _ptr(x), _ptr(weight), _ptr(plan.tiles), max_tiles, EXPERT_TILE, n, k,
                                            _code(x), _DTYPE_CODE[out_dtype], ACTIVATIONS[activation], _stream()))
    return out


def expert_combine(y, plan: ExpertPlan, weights, x, base=None, base_gate=None) -> torch.Tensor:
    """float32 out[t] = (base[t]) + sum over the token's chosen experts, in the order of the choice, of
    weights[t, k] * (y[rows[t, k]] for an expert with tensors, x[t] for one that returns its input).
    y float32 [rows, width] (or None when no expert has tensors), x [tokens, width], base float32.
    `weights` None: every weight is 1 (experts that were weighted on their input). `base_gate` =
    (float32 rows [tokens, ld], column): base[t] is multiplied by the sigmoid of that column first."""
    x = materialized(x)
    planes = 1
    if base is not None:
        base, planes = _sublayer_output(base)
    _need(x, "expert_combine: x")
    gate, gate_planes, gate_ld, gate_col = None, 1, 0, 0
    if base_gate is not None:
        gate_col = int(base_gate[1])
        gate, gate_planes = _sublayer_output(base_gate[0])        # a split product's planes are added by the kernel itself
        gate_ld = int(gate.shape[-1])
        if base is None or gate.shape[-2] != x.shape[0] or not 0 <= gate_col < gate_ld:
            raise KernelError(f"expert_combine: a gate {tuple(gate.shape)}, column {gate_col}, for {x.shape[0]} tokens' base")
    if weights is None:
        top = int(plan.rows.shape[1])
    else:
        _need(weights, "expert_combine: weights", torch.float32)
        top = int(weights.shape[1])
    if y is not None:
        _need(y, "expert_combine: y", torch.float32)
    if base is not None:
        _need(base, "expert_combine: base", torch.float32)
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    lib = _lib("routing")
    _check(lib, lib.pae_expert_combine(_ptr(out), _ptr(y), _ptr(plan.rows), _ptr(weights), _ptr(x), _ptr(base), planes, _ptr(gate), gate_planes,
                                       gate_ld, gate_col, x.shape[0], top, x.shape[1], _code(x), _stream()))
    return out

