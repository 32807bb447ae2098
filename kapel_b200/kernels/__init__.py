"""Tensor-level entry points of the CUDA library (`kapel_b200/csrc`).

Every function here checks devices, dtypes, shapes and contiguity, then calls one C launcher
on torch's current stream. There is no other implementation behind them: without the built
library, or without a CUDA device, they raise. Tensors are torch tensors only as owners of
device memory; no torch operator computes anything on this path.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

_lib = None
_lock = threading.Lock()

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

ACT_CODES = {"gelu_tanh": 0, "silu": 1}

# Which kernel multiplies more than 64 rows of bfloat16: "tcgen05" (TMA, TMEM, tcgen05.mma; the
# library picks between one block a tile and persistent pairs of blocks, "single" and "pair" force
# one) or "mma" (the warp-level mma.sync tile kernel, kept as the yardstick the tcgen05 kernels are
# measured against).
import os as _os

GEMM_LARGE = _os.environ.get("KAPEL_B200_GEMM_LARGE", "tcgen05")
# Which kernel multiplies up to 64 rows of bfloat16: "skinny" (tcgen05 with the operands swapped: the
# weights stream through shared memory by TMA) or "stream" (the mma.sync kernels that read the weights
# straight into registers).
GEMM_SMALL = _os.environ.get("KAPEL_B200_GEMM_SMALL", "skinny")
# Which kernel runs attention over prompt portions where both apply: "tcgen05" (products by
# tcgen05.mma, scores and probabilities in tensor memory) or "mma" (the mma.sync flash kernel, which
# also takes what the first does not: no soft cap, other head sizes).
ATTENTION_PROMPT = _os.environ.get("KAPEL_B200_ATTENTION_PROMPT", "tcgen05")
# Whether the tcgen05 prompt attention runs on pairs of blocks (tcgen05.mma.cta_group::2, 256 rows to one
# tile of 128 keys and values): 0 never, 1 at both head sizes that have such a kernel (128 and 256), 2 (the
# default) where it measured faster than single blocks (256).
ATTENTION_PAIRS = int(_os.environ.get("KAPEL_B200_ATTENTION_PAIRS", "2"))
# Whether the kernels of a decode step are launched as programmatic dependents of one another, so
# that a kernel sets up (and asks for its first weights) while the one before it finishes.
PDL = _os.environ.get("KAPEL_B200_PDL", "1") == "1"


class KernelError(RuntimeError):
    """A launcher refused its arguments or a launch failed; the message is the library's."""


def library():
    """The loaded library; builds it at the first call if it is missing or stale."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import ensure_built

                path = ensure_built()
                lib = ctypes.CDLL(str(path))
                lib.kb_last_error.restype = ctypes.c_char_p
                for name in ("kb_gemm_bf16_scratch_floats", "kb_paged_attention_scratch_floats", "kb_attention_mma_scratch_floats", "kb_sample_scratch_floats",
                             "kb_mlstm_state_floats", "kb_delta_state_floats", "kb_delta_scratch_floats", "kb_pooled_attention_scratch_floats",
                             "kb_pooled_attention_mma_scratch_floats", "kb_pooled_attention_mma_kept_floats", "kb_decay_scan_scratch_floats"):
                    getattr(lib, name).restype = ctypes.c_longlong
                lib.kb_launch_count.restype = ctypes.c_ulonglong
                lib.kb_set_pdl(1 if PDL else 0)
                if _os.environ.get("KAPEL_B200_DELTA_COLUMNS"):      # 1, 2 or 4 columns a warp in the delta scan instead of the launcher's choice
                    lib.kb_delta_columns_per_warp(int(_os.environ["KAPEL_B200_DELTA_COLUMNS"]))
                _lib = lib
    return _lib


def check_async_errors() -> None:
    """Raises if a bounded wait inside a kernel (on an mbarrier: a TMA copy or a tensor-core
    commit that never arrived) ran out since the last check. Synchronises the device."""
    lib = library()
    bad = []
    if lib.kb_attention_error() != 0:
        bad.append("paged attention (a bulk copy into shared memory never completed)")
    if lib.kb_tcgen05_error() != 0:
        bad.append("tcgen05 product (a TMA load or an MMA commit never arrived)")
    if lib.kb_attention_tc_error() != 0:
        bad.append("tcgen05 attention (a TMA load, an MMA commit or a softmax warp never arrived)")
    if lib.kb_rope_error() != 0:
        bad.append("rotate and append (a bulk copy of partial sums into shared memory never completed)")
    if lib.kb_norm_error() != 0:
        bad.append("add-and-norm (a bulk copy of partial sums into shared memory never completed)")
    if bad:
        raise KernelError("a wait inside a kernel gave up after its time limit: " + "; ".join(bad))


def wait_probe(limit_clocks: int = 2_000_000) -> None:
    """Launches one small block whose bounded wait (the products' own) runs out after
    `limit_clocks` because nothing ever arrives at its barrier. For testing that the flag reaches
    `check_async_errors` and that the device goes on working afterwards."""
    _check(library().kb_wait_probe(ctypes.c_longlong(int(limit_clocks)), _stream()))


def launch_count() -> int:
    """Kernels launched (or recorded under a graph capture) by this library so far."""
    return int(library().kb_launch_count())


def library_path() -> str:
    library()
    from ..csrc.build import ensure_built

    return str(ensure_built(verbose=False))


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().kb_last_error().decode("utf-8", "replace"))


# torch's current stream as a raw handle. The public route (torch.cuda.current_stream) builds a
# Stream object and resolves the device each time, about 15 us a call, once a kernel: more host
# time than everything else a launch does. torch's own C entry points give the same handle in
# well under a microsecond; without them the public route stands.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _dt(t: torch.Tensor, what: str) -> int:
    if t.dtype not in _CODES:
        raise KernelError(f"{what}: dtype {t.dtype} is not float32 or bfloat16")
    return _CODES[t.dtype]


def _need(t: torch.Tensor, what: str, dtype=None, shape=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        if len(shape) != t.dim() or any(s is not None and s != a for s, a in zip(shape, t.shape)):
            raise KernelError(f"{what}: shape {tuple(t.shape)}, expected {tuple(shape)}")
    return t


def _f(x: float) -> ctypes.c_float:
    return ctypes.c_float(float(x))


# With KAPEL_B200_POISON=1 every buffer a kernel is about to write (outputs, scratch, split-K partial
# sums) is first filled with NaN, so that a kernel which reads what nobody wrote, or leaves part
# of its output unwritten, shows in the logits instead of passing on whatever the allocator left
# there. Kapel's debugging switch of the same kind is `poison_buffers` (crates/kapel-cuda/src/device.rs:1019).
POISON = _os.environ.get("KAPEL_B200_POISON", "0") == "1"


def set_poison(on: bool) -> None:
    global POISON
    POISON = bool(on)


_fail_allocation_in = 0


def fail_allocation_in(calls: int) -> None:
    """Failure injection on the host, for tests: the `calls`-th buffer asked for from now on is
    refused with torch's out-of-memory error, as if the device had no room (0 turns it off)."""
    global _fail_allocation_in
    _fail_allocation_in = int(calls)


def _fresh(shape, dtype, device) -> torch.Tensor:
    """A new buffer for a kernel to write; NaN all over in the poisoning mode."""
    global _fail_allocation_in
    if _fail_allocation_in > 0:
        _fail_allocation_in -= 1
        if _fail_allocation_in == 0:
            raise torch.OutOfMemoryError(f"injected: no room for a buffer of shape {tuple(shape)}")
    t = torch.empty(tuple(shape), dtype=dtype, device=device)
    if POISON and dtype in _CODES and t.numel():
        _check(library().kb_poison(_ptr(t), _CODES[dtype], ctypes.c_longlong(t.numel()), _stream()))
    return t


def fill_rows(table: torch.Tensor, rows: torch.Tensor, value: float = 0.0) -> None:
    """table[rows[i]] = value for a float32 table [n, ...] and int32 row numbers on the device."""
    _need(table, "fill_rows table", torch.float32)
    _need(rows, "fill_rows rows", torch.int32)
    if table.dim() < 1 or table.shape[0] == 0 or rows.numel() == 0:
        return
    width = table.numel() // table.shape[0]
    _check(library().kb_fill_rows_f32(_ptr(table), _ptr(rows), int(rows.numel()), ctypes.c_longlong(width), int(table.shape[0]),
                                      _f(value), _stream()))


class SplitSum:
    """A product that is still a stack of split-K partial sums: `partials` is float32
    [splits, rows, cols] and the value is their sum over the first dimension. The kernels that
    read a product next (the norm with the residual sum, the gated unit, the rotation) add the
    slices up on the way in, so the sum is never written out and read back; `finish` does it
    for anything else."""

    __slots__ = ("partials",)

    def __init__(self, partials: torch.Tensor):
        self.partials = partials

    @property
    def shape(self):
        return tuple(self.partials.shape[1:])

    @property
    def splits(self) -> int:
        return int(self.partials.shape[0])

    @property
    def device(self):
        return self.partials.device


def _src(x, what: str):
    """(tensor to read, dtype code, slices, elements between slices) of a tensor or a SplitSum."""
    if isinstance(x, SplitSum):
        t = _need(x.partials, what, torch.float32)
        return t, F32, x.splits, t.shape[1] * t.shape[2]
    _need(x, what)
    return x, _dt(x, what), 1, 0


def finish(x, dtype: torch.dtype) -> torch.Tensor:
    """A SplitSum added up into a tensor of `dtype`; a tensor as it is (cast if need be)."""
    if isinstance(x, SplitSum):
        _need(x.partials, "finish partials", torch.float32)
        out = _fresh(x.shape, dtype, x.device)
        _check(library().kb_splitk_reduce(_ptr(out), _dt(out, "finish output"), _ptr(x.partials),
                                          ctypes.c_longlong(out.numel()), x.splits, _stream()))
        return out
    return x if x.dtype == dtype else cast(x, dtype)


# ------------------------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None,
          pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = table[ids[r]] * scale in float32; with `pos_table` [max positions, width] (the
    table's dtype) and the rows' `positions`, plus pos_table[positions[r]] (not scaled)."""
    _need(table, "embed table")
    _need(ids, "embed ids", torch.int32)
    vocab, width = table.shape
    rows = ids.numel()
    most = 0
    if pos_table is not None:
        _need(pos_table, "embed positions' table", table.dtype)
        if pos_table.dim() != 2 or pos_table.shape[1] != width:
            raise KernelError(f"embed: a table of positions {tuple(pos_table.shape)} beside rows of {width}")
        _need(positions, "embed positions", torch.int32, (rows,))
        most = int(pos_table.shape[0])
    if out is None:
        out = _fresh((rows, width), torch.float32, table.device)
    _need(out, "embed out", torch.float32, (rows, width))
    _check(library().kb_embed(_ptr(out), _ptr(table), _dt(table, "embed table"), _ptr(ids), rows, width, vocab, _f(scale),
                              _ptr(pos_table), _ptr(positions if pos_table is not None else None), most, _stream()))
    return out


def rope_table_freqs(positions: torch.Tensor, freqs: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """[rows, pairs, 2] float32 of (cos, sin) * magnitude of position * freqs[pair]; `freqs` is float64
    on the device (frequencies that a scaling rule has already changed); angles in float64."""
    _need(positions, "rope positions", torch.int32)
    _need(freqs, "rope frequencies", torch.float64)
    rows, half = positions.numel(), freqs.numel()
    out = _fresh((rows, half, 2), torch.float32, positions.device)
    _check(library().kb_rope_table_freqs(_ptr(out), _ptr(positions), rows, int(half), _ptr(freqs), ctypes.c_double(float(magnitude)), _stream()))
    return out


PLAIN_ACT_CODES = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def act(x, activation: str, out_dtype: torch.dtype) -> torch.Tensor:
    """activation(x) element by element for a product (a tensor or a SplitSum): "relu2" (the square
    of relu), "gelu_tanh" or "silu"."""
    src, in_dt, splits, stride = _src(x, "act input")
    if activation not in PLAIN_ACT_CODES:
        raise KernelError(f"act: activation {activation!r} is not known ({sorted(PLAIN_ACT_CODES)})")
    out = _fresh(x.shape, out_dtype, src.device)
    _check(library().kb_act(_ptr(out), _dt(out, "act output"), _ptr(src), in_dt, splits, ctypes.c_longlong(stride),
                            ctypes.c_longlong(out.numel()), PLAIN_ACT_CODES[activation], _stream()))
    return out


def rope_table(positions: torch.Tensor, rotary: int, theta: float, divisor: float = 1.0) -> torch.Tensor:
    """[rows, rotary/2, 2] float32 of (cos, sin); angles in float64 on the device. Every frequency
    theta^(-2j/rotary) is divided by `divisor` (1: the plain rotation)."""
    _need(positions, "rope positions", torch.int32)
    rows = positions.numel()
    out = _fresh((rows, rotary // 2, 2), torch.float32, positions.device)
    _check(library().kb_rope_table(_ptr(out), _ptr(positions), rows, int(rotary), ctypes.c_double(float(theta)), ctypes.c_double(float(divisor)),
                                  _stream()))
    return out


def rope_append(qkv, cos_sin, lines, k_table, v_table, hq: int, hkv: int, d: int, rotary: int, write_kv: bool = True,
                out_dtype: Optional[torch.dtype] = None):
    """Rotates the q and k heads of the stacked product `qkv` [rows, (hq + 2 hkv) d] (a tensor or a
    SplitSum), returns q [rows, hq, d], and writes k and v at each row's line (page * page_size +
    offset) of the tables [pages, hkv, page_size, d]."""
    src, in_dt, splits, stride = _src(qkv, "rope_append qkv")
    rows = qkv.shape[0]
    if tuple(qkv.shape) != (rows, (hq + 2 * hkv) * d):
        raise KernelError(f"rope_append: qkv {tuple(qkv.shape)}, expected {(rows, (hq + 2 * hkv) * d)}")
    out_dtype = out_dtype or (src.dtype if not isinstance(qkv, SplitSum) else k_table.dtype)
    if rotary:
        _need(cos_sin, "rope_append cos_sin", torch.float32, (rows, rotary // 2, 2))
    q = _fresh((rows, hq, d), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "rope_append lines", torch.int32, (rows,))
        _need(k_table, "rope_append k table", out_dtype)
        _need(v_table, "rope_append v table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d or v_table.shape != k_table.shape:
            raise KernelError(f"rope_append: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, {hkv}, page_size, {d}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(
        library().kb_rope_append(
            _ptr(src), in_dt, splits, ctypes.c_longlong(stride), _ptr(cos_sin if rotary else None),
            _ptr(lines if write_kv else None), _ptr(q), _ptr(k_table if write_kv else None), _ptr(v_table if write_kv else None),
            _dt(q, "rope_append output"), rows, hq, hkv, d, int(rotary), int(bool(write_kv)), ctypes.c_longlong(table_lines), int(page_size), _stream(),
        )
    )
    return q


def glu(x, activation: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(x[:, :n]) * x[:, n:] for a stacked gate|up product (a tensor or a SplitSum)."""
    src, in_dt, splits, stride = _src(x, "glu input")
    if activation not in ACT_CODES:
        raise KernelError(f"glu: activation {activation!r} is not known")
    rows, two_n = x.shape
    n = two_n // 2
    out_dtype = out_dtype or (src.dtype if not isinstance(x, SplitSum) else torch.bfloat16)
    out = _fresh((rows, n), out_dtype, src.device)
    _check(library().kb_glu(_ptr(out), _dt(out, "glu output"), _ptr(src), in_dt, splits, ctypes.c_longlong(stride),
                            ctypes.c_longlong(rows), n, ACT_CODES[activation], _stream()))
    return out


def glu_clamped(x, limit: float, alpha: float, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """g' sigmoid(alpha g') (u' + 1) for a stacked gate|up product (a tensor or a SplitSum), with
    g' = min(gate, limit) and u' = clamp(up, -limit, limit)."""
    src, in_dt, splits, stride = _src(x, "glu_clamped input")
    rows, two_n = x.shape
    n = two_n // 2
    out_dtype = out_dtype or (src.dtype if not isinstance(x, SplitSum) else torch.bfloat16)
    out = _fresh((rows, n), out_dtype, src.device)
    _check(library().kb_glu_clamped(_ptr(out), _dt(out, "glu_clamped output"), _ptr(src), in_dt, splits, ctypes.c_longlong(stride),
                                    ctypes.c_longlong(rows), n, _f(limit), _f(alpha), _stream()))
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need(x, "cast input")
    out = _fresh(x.shape, dtype, x.device)
    _check(library().kb_cast(_ptr(out), _dt(out, "cast output"), _ptr(x), _dt(x, "cast input"), ctypes.c_longlong(x.numel()), _stream()))
    return out


def pad_cols(x: torch.Tensor, wide: int) -> torch.Tensor:
    """x [rows, width] (bfloat16) with zero columns up to `wide`."""
    _need(x, "pad_cols input", torch.bfloat16)
    rows, width = x.shape
    out = _fresh((rows, int(wide)), torch.bfloat16, x.device)
    _check(library().kb_pad_cols_bf16(_ptr(out), _ptr(x), ctypes.c_longlong(rows), int(width), int(wide), _stream()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _need(x, "gather_rows input", torch.float32)
    _need(rows, "gather_rows rows", torch.int32)
    n, width = rows.numel(), x.shape[1]
    out = _fresh((n, width), torch.float32, x.device)
    _check(library().kb_gather_rows_f32(_ptr(out), _ptr(x), _ptr(rows), n, width, x.shape[0], _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype) -> torch.Tensor:
    _need(x, "rmsnorm input")
    rows, width = x.shape
    _need(weight, "rmsnorm weight", shape=(width,))
    y = _fresh((rows, width), out_dtype, x.device)
    _check(
        library().kb_rmsnorm(_ptr(y), _dt(y, "rmsnorm output"), _ptr(x), _dt(x, "rmsnorm input"), _ptr(weight),
                             _dt(weight, "rmsnorm weight"), rows, width, _f(eps), _f(offset), _stream())
    )
    return y


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype) -> torch.Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * (offset + weight) over each row, in 32-bit."""
    _need(x, "layernorm input")
    rows, width = x.shape
    _need(weight, "layernorm weight", shape=(width,))
    y = _fresh((rows, width), out_dtype, x.device)
    _check(
        library().kb_layernorm(_ptr(y), _dt(y, "layernorm output"), _ptr(x), _dt(x, "layernorm input"), _ptr(weight),
                               _dt(weight, "layernorm weight"), rows, width, _f(eps), _f(offset), _stream())
    )
    return y


def concat2(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[rows, 2 width]: the float32 rows of `a` and of `b` side by side, in `out_dtype`."""
    _need(a, "concat2 first", torch.float32)
    _need(b, "concat2 second", torch.float32, tuple(a.shape))
    rows, width = a.shape
    out = _fresh((rows, 2 * width), out_dtype, a.device)
    _check(library().kb_concat2(_ptr(out), _CODES[out_dtype], _ptr(a), _ptr(b), ctypes.c_longlong(rows), int(width), _stream()))
    return out


def add_rmsnorm(residual, branch, post, nxt, out_dtype, copy_out: bool = False):
    """residual += norm_post(branch) (post = (weight, eps, offset) or None: plain add); returns
    norm_next(residual) when nxt = (weight, eps, offset) is given; without it, None, or with
    `copy_out` the new residual itself in `out_dtype` (what a reader of the residual takes next).
    A fourth value True in either tuple makes that norm take the row's mean off first (a layer
    norm with a weight and no bias). In place on residual. `branch` is a tensor or a SplitSum."""
    rows, width = residual.shape
    _need(residual, "add_rmsnorm residual", torch.float32)
    src, b_dt, splits, stride = _src(branch, "add_rmsnorm branch")
    if tuple(branch.shape) != (rows, width):
        raise KernelError(f"add_rmsnorm: branch {tuple(branch.shape)} against residual {(rows, width)}")
    w_post, eps_post, off_post = post[:3] if post is not None else (None, 0.0, 0.0)
    w_next, eps_next, off_next = nxt[:3] if nxt is not None else (None, 0.0, 0.0)
    center_post = bool(post is not None and len(post) > 3 and post[3])
    center_next = bool(nxt is not None and len(nxt) > 3 and nxt[3])
    ws = [w for w in (w_post, w_next) if w is not None]
    for w in ws:
        _need(w, "add_rmsnorm weight", shape=(width,))
    if len({w.dtype for w in ws}) > 1:
        raise KernelError("add_rmsnorm: the two norms' weights differ in dtype; call the norms one by one")
    w_dt = _dt(ws[0], "add_rmsnorm weight") if ws else F32
    h = _fresh((rows, width), out_dtype, residual.device) if (w_next is not None or copy_out) else None
    if center_post or center_next:
        _check(
            library().kb_add_norm(_ptr(residual), _ptr(src), b_dt, splits, ctypes.c_longlong(stride), _ptr(w_post), _f(eps_post),
                                  _f(off_post), int(center_post), _ptr(w_next), _f(eps_next), _f(off_next), int(center_next),
                                  _ptr(h), _CODES[out_dtype], w_dt, rows, width, _stream())
        )
        return h
    _check(
        library().kb_add_rmsnorm(_ptr(residual), _ptr(src), b_dt, splits, ctypes.c_longlong(stride), _ptr(w_post), _f(eps_post),
                                 _f(off_post), _ptr(w_next), _f(eps_next), _f(off_next), _ptr(h), _CODES[out_dtype], w_dt,
                                 rows, width, _stream())
    )
    return h


# Up to 64 rows, and up to SKINNY_ROWS where the kernels for many rows would have few tiles, a
# product streams the weights once through many blocks that split K (the "few-rows" kernels, whose
# MMA takes the rows as its N, up to 256). With one or two row tiles and a narrow weight the kernels
# for many rows leave most multiprocessors idle: the way down of Gemma 2 2B at 128 rows took 50 us by
# 9 blocks against 15 us, o 17 against 7; a wide weight has tiles enough (gate|up: 22 us either way).
SKINNY_ROWS = int(_os.environ.get("KAPEL_B200_SKINNY_ROWS", "256"))
SKINNY_TILES = 24          # tiles of 128 x 256 below which the few-rows kernel is taken beyond 64 rows


def few_rows_product(m: int, n: int) -> bool:
    """Whether a product of m rows by a weight of n rows goes to the few-rows kernels."""
    if m <= 0:
        return False
    if m <= 64:
        return True
    return m <= SKINNY_ROWS and -(-m // 128) * -(-n // 256) <= SKINNY_TILES


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, softcap: Optional[float] = None,
         keep_split: bool = False):
    """a [m, k] . w [n, k]^T -> [m, n]; float32 x float32 in true 32-bit, bfloat16 x bfloat16 on
    tensor cores with 32-bit sums. `softcap` c applies c * tanh(x / c) to the result. With
    `keep_split`, a product that the kernel splits over K comes back as a SplitSum (its partial
    sums, not yet added up) for a kernel that adds them on the way in."""
    _need(a, "gemm input")
    _need(w, "gemm weight")
    m, k = a.shape
    n, k2 = w.shape
    if k != k2:
        raise KernelError(f"gemm: input [{m}, {k}] against weight [{n}, {k2}]")
    if a.dtype != w.dtype:
        raise KernelError(f"gemm: input {a.dtype} against weight {w.dtype}")
    epi, cap = (1, softcap) if softcap is not None else (0, 0.0)
    lib = library()
    if a.dtype == torch.float32:
        out = _fresh((m, n), torch.float32, a.device)
        _check(lib.kb_gemm_f32(_ptr(out), _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _stream()))
        if out_dtype is not None and out_dtype != torch.float32:
            out = cast(out, out_dtype)
        return out
    out_dtype = out_dtype or torch.bfloat16
    if few_rows_product(m, n) and GEMM_SMALL == "skinny":
        splits = int(lib.kb_gemm_skinny_splits_for(m, n, k))
        if splits == 1:
            out = _fresh((m, n), out_dtype, a.device)
            _check(lib.kb_gemm_skinny(_ptr(out), _dt(out, "gemm output"), None, _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _stream()))
            return out
        if softcap is None:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_skinny(None, 0, _ptr(partials), _ptr(a), _ptr(w), m, n, k, 0, _f(0.0), _stream()))
            split_sum = SplitSum(partials)
            return split_sum if keep_split else finish(split_sum, out_dtype)
        # a soft cap over partial sums: the streaming kernels' reduction applies it
    if keep_split and softcap is None and 0 < m <= 16:
        splits = int(lib.kb_gemm_bf16_row16_splits(n, k))
        if splits > 1:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_bf16_partial(_ptr(partials), _ptr(a), _ptr(w), m, n, k, _stream()))
            return SplitSum(partials)
    if keep_split and softcap is None and m > 64 and GEMM_LARGE == "tcgen05":
        # a few hundred rows by a narrow weight: few tiles, each walking all of K; cut over K instead
        splits = int(lib.kb_gemm_tcgen05_splits(m, n, k))
        if splits > 1:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_tcgen05_split(_ptr(partials), _ptr(a), _ptr(w), m, n, k, _stream()))
            return SplitSum(partials)
    out = _fresh((m, n), out_dtype, a.device)
    if m > 64 and GEMM_LARGE in _TCGEN05_KERNELS:
        _check(lib.kb_gemm_tcgen05(_ptr(out), _dt(out, "gemm output"), _ptr(a), _ptr(w), m, n, k, epi, _f(cap),
                                   _TCGEN05_KERNELS[GEMM_LARGE], _stream()))
        return out
    need = lib.kb_gemm_bf16_scratch_floats(m, n, k)
    scratch = _fresh((need,), torch.float32, a.device) if need else None
    _check(lib.kb_gemm_bf16(_ptr(out), _dt(out, "gemm output"), _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _ptr(scratch), _stream()))
    return out


_TCGEN05_KERNELS = {"tcgen05": 0, "single": 1, "pair": 2}       # the kernel chooses; one block a tile; persistent pairs


def gemm_glu_fused(a: torch.Tensor, w: torch.Tensor, act: str) -> Optional[torch.Tensor]:
    """act(a . gate^T) * (a . up^T) for a stacked gate|up weight w [2 n, k], in one kernel whose
    epilogue applies the gated unit to the 32-bit sums; None where no such kernel applies
    (32-bit operands, the mma.sync yardsticks selected) and the caller multiplies and gates in two steps."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] == 0:
        return None
    few = a.shape[0] <= 64
    if (few and GEMM_SMALL != "skinny") or (not few and GEMM_LARGE not in ("tcgen05", "pair")):
        return None
    if act not in ACT_CODES:
        raise KernelError(f"gemm_glu: activation {act!r} is not known")
    _need(a, "gemm input")
    _need(w, "gemm weight")
    m, k = a.shape
    n2, k2 = w.shape
    if k != k2 or n2 % 2:
        raise KernelError(f"gemm_glu: input [{m}, {k}] against stacked weight [{n2}, {k2}]")
    out = _fresh((m, n2 // 2), torch.bfloat16, a.device)
    if few:
        _check(library().kb_gemm_skinny_glu(_ptr(out), _ptr(a), _ptr(w), m, n2 // 2, k, ACT_CODES[act], _stream()))
        return out
    _check(library().kb_gemm_tcgen05_glu(_ptr(out), _ptr(a), _ptr(w), m, n2 // 2, k, ACT_CODES[act], _stream()))
    return out


_ATT_CHUNK = None


def attention_chunk() -> int:
    global _ATT_CHUNK
    if _ATT_CHUNK is None:
        _ATT_CHUNK = int(library().kb_attention_chunk())
    return _ATT_CHUNK


def paged_attention_rows(q, k_table, v_table, block_table, row_entry, row_count, page_size: int, window: Optional[int],
                         scale: float, softcap: Optional[float], slots: int, keep_first: int = 0,
                         sinks: Optional[torch.Tensor] = None, value_dim: Optional[int] = None, block: int = 0) -> torch.Tensor:
    """Attention of each query row over its sequence's pages; with `block` > 0 a row at position i sees
    only the keys from floor(i / block) * block on (`slots` as for a window of `block` positions); `slots` is the largest number of
    key chunks (of `attention_chunk()` positions, cut at absolute multiples) any row touches, plus,
    with a window and `keep_first` > 0, the chunks of the first `keep_first` keys, which stay
    visible below the window (`attention_keep_slots`). The values' size is the v table's last, or
    `value_dim`: the first that many components of each of the v table's lines (the v table may then be
    the k table itself). `sinks` [hq] float32: e^sink joins each row's denominator (no key, no value)."""
    rows, hq, d = q.shape
    _need(q, "attention q")
    _need(k_table, "attention k table", q.dtype)
    _need(v_table, "attention v table", q.dtype)
    if k_table.dim() != 4 or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.dim() != 4 or v_table.shape[:3] != k_table.shape[:3]:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, kv_heads, {page_size}, {d}]")
    n_pages, hkv, v_stride = k_table.shape[0], k_table.shape[1], v_table.shape[3]
    dv = int(value_dim) if value_dim is not None else v_stride
    if not 0 < dv <= v_stride:
        raise KernelError(f"attention: values of {dv} in lines of {v_stride}")
    if sinks is not None:
        _need(sinks, "attention sinks", torch.float32, (hq,))
    _need(block_table, "attention block table", torch.int32)
    _need(row_entry, "attention row_entry", torch.int32, (rows,))
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh((rows, hq, dv), q.dtype, q.device)
    lib = library()
    need = lib.kb_paged_attention_scratch_floats(rows, hq, dv, int(slots))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    _check(
        lib.kb_paged_attention_rows_blocked(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _dt(q, "attention q"), _ptr(block_table),
                                    _ptr(row_entry), _ptr(row_count), rows, hq, hkv, d, int(dv), int(page_size), int(block_table.shape[1]),
                                    int(n_pages), int(window or 0), int(keep_first or 0), int(slots), _f(scale), _f(softcap or 0.0),
                                    _ptr(scratch), int(v_stride), _ptr(sinks), int(block or 0), _stream())
    )
    return out


def latent_attention_mma_takes(dtype, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel for attention over lines that are key and value at once takes
    these sizes (else the row-wise kernel does)."""
    return dtype == torch.bfloat16 and bool(library().kb_latent_attention_mma_takes(int(d), int(dv)))


# A prompt's slots of the latent attention kernel hold this many of the row-wise kernel's chunks.
LATENT_PROMPT_CHUNKS = max(1, int(_os.environ.get("KAPEL_B200_LATENT_PROMPT_CHUNKS", "8")))


def latent_attention_mma(q, table, block_table, row_count, ranges, entries: int, longest: int, page_size: int, scale: float,
                         slots: int, sinks: Optional[torch.Tensor], value_dim: int) -> torch.Tensor:
    """Attention of every query head [rows, hq, d] over the lines of `table` [pages, 1, page_size, d],
    whose first `value_dim` components are the values, on tensor cores (bfloat16). `ranges` =
    (start, end) of each request's rows on the device, `longest` the most rows a request brings;
    `slots` as for `paged_attention_rows` without a window (chunks of `attention_chunk()` keys): a pass
    of single tokens is cut that way, a pass with prompt portions into slots eight times as long
    (fewer partial sums to write and merge; it has tiles enough). `sinks` [hq] float32 or None."""
    rows, hq, d = q.shape
    _need(q, "latent attention q", torch.bfloat16)
    _need(table, "latent attention table", torch.bfloat16)
    if table.dim() != 4 or table.shape[1] != 1 or table.shape[2] != page_size or table.shape[3] != d:
        raise KernelError(f"latent attention: a table of {tuple(table.shape)} is not [pages, 1, {page_size}, {d}]")
    _need(block_table, "latent attention block table", torch.int32)
    _need(row_count, "latent attention row_count", torch.int32, (rows,))
    start, end = ranges
    _need(start, "latent attention entry starts", torch.int32)
    _need(end, "latent attention entry ends", torch.int32)
    if min(start.numel(), end.numel()) < entries or block_table.shape[0] < entries:
        raise KernelError(f"latent attention: {entries} requests but ranges or block tables for fewer")
    if sinks is not None:
        _need(sinks, "latent attention sinks", torch.float32, (hq,))
    dv = int(value_dim)
    out = _fresh((rows, hq, dv), torch.bfloat16, q.device)
    lib = library()
    chunk = attention_chunk()
    if longest > 1:         # measured at 2,048 tokens, 16 heads, lines of 576: 4.91, 4.68, 4.52, 4.43 ms a four-layer prefill with 1, 2, 4, 8
        chunk, slots = chunk * LATENT_PROMPT_CHUNKS, -(-int(slots) // LATENT_PROMPT_CHUNKS)
    need = lib.kb_paged_attention_scratch_floats(rows, hq, dv, int(slots))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    _check(lib.kb_latent_attention_mma(_ptr(out), _ptr(q), _ptr(table), _ptr(block_table), _ptr(row_count), _ptr(start), _ptr(end),
                                       int(entries), int(longest), rows, hq, d, dv, int(page_size), int(block_table.shape[1]),
                                       int(table.shape[0]), int(slots), int(chunk), _f(scale), _ptr(scratch), _ptr(sinks), _stream()))
    return out


def attention_keep_slots(window: Optional[int], keep_first: int) -> int:
    """Chunk slots the row-wise kernel spends on the kept first keys of a windowed layer."""
    return -(-int(keep_first) // attention_chunk()) if (window and keep_first) else 0


def attention_mma_rows(decode: bool) -> int:
    """Rows (token, query head of one kv head's group) a tile of the tensor-core kernel holds."""
    return int(library().kb_attention_mma_rows(int(bool(decode))))


def prompt_pairs(rows: int, longest: int) -> int:
    """The pairs setting for a pass of `rows` query rows whose longest request sees `longest` keys:
    ATTENTION_PAIRS, except that a small pass runs on single blocks (setting 0) where pairs would be
    the default only for head size 256: a pair's launch costs a few microseconds more than it saves
    until there are some hundreds of keys to walk (128 tokens at Gemma 2 2B sizes: 13.4 us on single
    blocks, 17.2 us on pairs; 2,048 tokens: 55 against 42)."""
    if ATTENTION_PAIRS == 2 and rows < 768 and longest < 2048:
        return 0
    return ATTENTION_PAIRS


def attention_tile_rows(decode: bool, prompt_kernel: str = "mma", d: int = 0, pairs: Optional[int] = None) -> int:
    """Rows a tile holds for the kernel that will run: the decode kernel's, the mma.sync prompt
    kernel's, or the tcgen05 prompt kernel's (twice as many where pairs of blocks run it)."""
    if not decode and prompt_kernel == "tcgen05":
        return int(library().kb_attention_tc_rows(int(d), int(ATTENTION_PAIRS if pairs is None else pairs)))
    return attention_mma_rows(decode)


def attention_mma_takes(dtype, d: int, heads_per_kv: int) -> bool:
    """Whether the tensor-core kernel takes these sizes (else the row-wise kernel does)."""
    return dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and heads_per_kv <= 16


def attention_prompt_kernel(hq: int, hkv: int, d: int, page_size: int, softcap: Optional[float]) -> str:
    """Which kernel `paged_attention_mma` runs for prompt portions of these sizes: "tcgen05" or "mma"."""
    if ATTENTION_PROMPT == "tcgen05" and library().kb_attention_tc_takes(int(hq), int(hkv), int(d), int(page_size), _f(softcap or 0.0)):
        return "tcgen05"
    return "mma"


# KAPEL_B200_DECODE_FUSED=0: the rotation and the cache's newest line stay a kernel of their own
# ahead of the decode attention (the yardstick of the kernel that takes both over). Measured at
# Gemma 2 2B sizes with 6,144 tokens of history, both ways in one call: +2 % at one request, +6 % at 8,
# +4 % at 64. DECODE_FUSED_ROWS is the number of requests from which it is used.
DECODE_FUSED = _os.environ.get("KAPEL_B200_DECODE_FUSED", "1") != "0"
DECODE_FUSED_ROWS = int(_os.environ.get("KAPEL_B200_DECODE_FUSED_ROWS", "1"))


def attention_decode_fused_takes(qkv, hq: int, hkv: int, d: int, rotary: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether `paged_attention_decode_fused` takes this stacked product: float32 split sums on the
    bfloat16 path, the whole head rotated, sizes the kernel is built for."""
    if not DECODE_FUSED or not isinstance(qkv, SplitSum) or dtype != torch.bfloat16 or rotary != d:
        return False
    if qkv.shape[0] < DECODE_FUSED_ROWS:
        return False
    return bool(library().kb_attention_decode_fused_takes(int(hq), int(hkv), int(d), int(page_size), qkv.splits))


def paged_attention_decode_fused(qkv: "SplitSum", cos_sin, lines, k_table, v_table, block_table, row_count, hq: int, hkv: int,
                                 d: int, write_kv: bool, page_size: int, window: Optional[int], scale: float,
                                 softcap: Optional[float], split: int, slots: int) -> torch.Tensor:
    """A decode step in which every request brings one token (row r is request r), straight from
    the stacked q|k|v product's partial sums: the attention kernel adds up the slices of its row's
    query heads, rotates them, and where a block's keys end with the row's own position it does the
    same for the key and the value, writes them to the cache at `lines[row]` (with `write_kv`) and
    uses them. The result is `rope_append` followed by `paged_attention_mma(decode, relative)`, bit
    for bit, one kernel and one wait between kernels fewer."""
    parts = qkv.partials
    _need(parts, "attention qkv slices", torch.float32)
    splits, rows, width = parts.shape
    if width != (hq + 2 * hkv) * d:
        raise KernelError(f"attention: qkv slices {tuple(parts.shape)}, expected a width of {(hq + 2 * hkv) * d}")
    _need(cos_sin, "attention cos_sin", torch.float32, (rows, d // 2, 2))
    _need(lines, "attention lines", torch.int32, (rows,))
    _need(k_table, "attention k table", torch.bfloat16)
    _need(v_table, "attention v table", torch.bfloat16)
    if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.shape != k_table.shape:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} are not [pages, {hkv}, {page_size}, {d}]")
    _need(block_table, "attention block table", torch.int32)
    if block_table.dim() != 2 or block_table.shape[0] < rows:
        raise KernelError(f"attention: a block table of {tuple(block_table.shape)} for {rows} requests")
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh((rows, hq, d), torch.bfloat16, parts.device)
    lib = library()
    need = lib.kb_attention_mma_scratch_floats(rows, hq, d, int(slots))
    scratch = _fresh((need,), torch.float32, parts.device) if need else None
    n_pages = k_table.shape[0]
    _check(
        lib.kb_attention_decode_fused(
            _ptr(out), _ptr(parts), int(splits), ctypes.c_longlong(rows * width), _ptr(cos_sin), _ptr(lines), _ptr(k_table),
            _ptr(v_table), int(bool(write_kv)), ctypes.c_longlong(n_pages * page_size), _ptr(block_table), _ptr(row_count), rows,
            hq, hkv, d, int(page_size), int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots),
            _f(scale), _f(softcap or 0.0), _ptr(scratch), _stream(),
        )
    )
    return out


def paged_attention_mma(q, k_table, v_table, block_table, row_count, tiles, page_size: int, window: Optional[int],
                        scale: float, softcap: Optional[float], decode: int, split: int, slots: int,
                        relative: bool = False, pairs: Optional[int] = None, keep_first: int = 0, block: int = 0,
                        sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention over the paged cache on tensor cores (bfloat16). `tiles` = (tile_entry, tile_row0,
    tile_nq) int32 device tensors: each tile is up to `attention_mma_rows(decode) // group` tokens of
    one request at consecutive positions. `decode` is 0 for prompt portions, else the most rows
    (tokens x query heads of a kv head) any tile holds, at most 16. `split` > 0 cuts the keys at
    absolute multiples of it over `slots` blocks (slots >= ceil(longest count / split)). With
    `relative` (decode mode, every tile one token) the multiples are counted from each row's first
    visible key, so a windowed row needs ceil(window / split) slots however long its history. With a
    window, `keep_first` keys from position 0 stay visible below it (prompt portions in one slot only).
    With `block` > 0 a row at position i sees only the keys from floor(i / block) * block on, and with
    `sinks` [hq] float32 e^sink joins each row's denominator (both: prompt portions in one slot only)."""
    rows, hq, d = q.shape
    if sinks is not None:
        _need(sinks, "attention sinks", torch.float32, (hq,))
    _need(q, "attention q", torch.bfloat16)
    _need(k_table, "attention k table", torch.bfloat16)
    _need(v_table, "attention v table", torch.bfloat16)
    if k_table.dim() != 4 or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.shape != k_table.shape:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} are not [pages, kv_heads, {page_size}, {d}]")
    n_pages, hkv = k_table.shape[0], k_table.shape[1]
    tile_entry, tile_row0, tile_nq = tiles
    n_tiles = tile_entry.numel()
    for t in tiles:
        _need(t, "attention tiles", torch.int32, (n_tiles,))
    _need(block_table, "attention block table", torch.int32)
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh(q.shape, q.dtype, q.device)
    lib = library()
    need = lib.kb_attention_mma_scratch_floats(rows, hq, d, int(slots))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    if not decode and not keep_first and not block and sinks is None and attention_prompt_kernel(hq, hkv, d, page_size, softcap) == "tcgen05":
        _check(
            lib.kb_attention_tc(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _ptr(block_table), _ptr(row_count),
                                _ptr(tile_entry), _ptr(tile_row0), _ptr(tile_nq), n_tiles, rows, hq, hkv, d, int(page_size),
                                int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots), _f(scale),
                                _f(softcap or 0.0), _ptr(scratch), int(ATTENTION_PAIRS if pairs is None else pairs), _stream())
        )
        if slots > 1:
            _check(lib.kb_attention_mma_combine(_ptr(out), _ptr(row_count), _ptr(scratch), rows, hq, d, int(window or 0), int(split),
                                                int(slots), _stream()))
        return out
    _check(
        lib.kb_attention_mma_masked(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _ptr(block_table), _ptr(row_count),
                                    _ptr(tile_entry), _ptr(tile_row0), _ptr(tile_nq), n_tiles, rows, hq, hkv, d, int(page_size),
                                    int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots), _f(scale),
                                    _f(softcap or 0.0), int(decode), int(bool(relative) and bool(decode)), int(keep_first or 0),
                                    _ptr(scratch), int(block or 0), _ptr(sinks), _stream())
    )
    return out


# ------------------------------------------------------------------------------------------
# Mixers whose roles share one stacked product: a role is a run of columns of each row.
GATE_ACTS = {"sigmoid": 0, "silu": 1, "none": 2}        # "none": the gate is not read


def _stacked(x, what: str):
    """(tensor, dtype code, slices, stride, rows, row width) of a stacked product (a tensor or a SplitSum)."""
    src, dt, splits, stride = _src(x, what)
    rows, width = x.shape
    return src, dt, splits, stride, int(rows), int(width)


def proj_norm_append(stacked, q_off: int, k_off: int, v_off: int, q_norm, k_norm, lines, k_table, v_table, hq: int, hkv: int,
                     d: int, dv: int, write_kv: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """q [rows, hq, d] from the columns q_off.. of `stacked`, normed over the whole projection when
    `q_norm` = (weight [hq d], eps, offset) is given; the keys (normed by `k_norm` likewise) and the
    values written at each row's line of the tables [pages, hkv, page_size, d] and [.., dv]."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "proj_norm_append input")
    wq, eq, oq = q_norm if q_norm is not None else (None, 0.0, 0.0)
    wk, ek, ok = k_norm if k_norm is not None else (None, 0.0, 0.0)
    ws = [w for w in (wq, wk) if w is not None]
    if len({w.dtype for w in ws}) > 1:
        raise KernelError("proj_norm_append: the two norms' weights differ in dtype")
    if wq is not None:
        _need(wq, "proj_norm_append q norm", shape=(hq * d,))
    if wk is not None:
        _need(wk, "proj_norm_append k norm", shape=(hkv * d,))
    w_dt = _dt(ws[0], "proj_norm_append norm") if ws else F32
    q = _fresh((rows, hq, d), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "proj_norm_append lines", torch.int32, (rows,))
        _need(k_table, "proj_norm_append k table", out_dtype)
        _need(v_table, "proj_norm_append v table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d or v_table.dim() != 4 or \
                tuple(v_table.shape) != (*k_table.shape[:3], dv):
            raise KernelError(f"proj_norm_append: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, {hkv}, page_size, {d} / {dv}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(library().kb_proj_norm_append(
        _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(k_off), int(v_off), _ptr(wq), _f(eq), _f(oq),
        _ptr(wk), _f(ek), _f(ok), w_dt, _ptr(lines if write_kv else None), _ptr(q), _ptr(k_table if write_kv else None),
        _ptr(v_table if write_kv else None), _CODES[out_dtype], rows, hq, hkv, d, dv, int(bool(write_kv)),
        ctypes.c_longlong(table_lines), int(page_size), _stream()))
    return q


def head_gate(y: torch.Tensor, stacked, g_off: int, weight: Optional[torch.Tensor], unit: bool, eps: float,
              out_dtype: torch.dtype, pad_to: int = 0, gate_act: str = "sigmoid") -> torch.Tensor:
    """y [rows, heads, e] times sigmoid (or, with `gate_act` "silu", silu) of the columns g_off.. of
    `stacked`; with `unit` each head is first divided by its root mean square (eps inside the
    root); `weight` [heads e] multiplies too.
    The result is [rows, heads e], or [rows, pad_to] with zeros behind the heads."""
    if gate_act not in GATE_ACTS:
        raise KernelError(f"head_gate: gate activation {gate_act!r} is not known ({sorted(GATE_ACTS)})")
    _need(y, "head_gate input")
    rows, heads, e = y.shape
    src, dt, splits, stride, g_rows, width = _stacked(stacked, "head_gate gate")
    if g_rows != rows:
        raise KernelError(f"head_gate: {rows} rows against a gate of {g_rows}")
    if weight is not None:
        _need(weight, "head_gate weight", shape=(heads * e,))
    out_width = max(int(pad_to), heads * e)
    out = _fresh((rows, out_width), out_dtype, y.device)
    _check(library().kb_head_gate(
        _ptr(out), _CODES[out_dtype], _ptr(y), _dt(y, "head_gate input"), _ptr(src), dt, splits, ctypes.c_longlong(stride), width,
        int(g_off), _ptr(weight), _dt(weight, "head_gate weight") if weight is not None else F32, int(bool(unit)), _f(eps),
        ctypes.c_longlong(rows), heads, e, out_width, GATE_ACTS[gate_act], _stream()))
    return out


def head_norm_rope_append(stacked, q_off: int, k_off: int, v_off: int, q_norm, k_norm, cos_sin, rotary: int, lines, k_table, v_table,
                          hq: int, hkv: int, d: int, dv: int, write_kv: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """q [rows, hq, d] from the columns q_off.. of `stacked`: every head RMS-normed when `q_norm` =
    (weight [d], eps, offset) is given (one weight for all heads), then its first `rotary` components
    turned by `cos_sin` [rows, rotary/2, 2]; the keys likewise (`k_norm`) and the values as they are,
    written at each row's line of the tables [pages, hkv, page_size, d] and [.., dv]."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "head_norm_rope_append input")
    wq, eq, oq = q_norm[:3] if q_norm is not None else (None, 0.0, 0.0)
    wk, ek, ok = k_norm[:3] if k_norm is not None else (None, 0.0, 0.0)
    ws = [w for w in (wq, wk) if w is not None]
    if len({w.dtype for w in ws}) > 1:
        raise KernelError("head_norm_rope_append: the two norms' weights differ in dtype")
    for w in ws:
        _need(w, "head_norm_rope_append norm", shape=(d,))
    w_dt = _dt(ws[0], "head_norm_rope_append norm") if ws else F32
    if rotary:
        _need(cos_sin, "head_norm_rope_append cos_sin", torch.float32, (rows, rotary // 2, 2))
    q = _fresh((rows, hq, d), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "head_norm_rope_append lines", torch.int32, (rows,))
        _need(k_table, "head_norm_rope_append k table", out_dtype)
        _need(v_table, "head_norm_rope_append v table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d or v_table.dim() != 4 or \
                tuple(v_table.shape) != (*k_table.shape[:3], dv):
            raise KernelError(f"head_norm_rope_append: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, {hkv}, page_size, {d} / {dv}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(library().kb_head_norm_rope_append(
        _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(k_off), int(v_off), _ptr(wq), _f(eq), _f(oq),
        _ptr(wk), _f(ek), _f(ok), w_dt, _ptr(cos_sin if rotary else None), int(rotary), _ptr(lines if write_kv else None), _ptr(q),
        _ptr(k_table if write_kv else None), _ptr(v_table if write_kv else None), _CODES[out_dtype], rows, hq, hkv, d, dv,
        int(bool(write_kv)), ctypes.c_longlong(table_lines), int(page_size), _stream()))
    return q


def latent_append(stacked, q_off: int, kv_off: int, q_rank: int, kv_rank: int, rot: int, q_weight, kv_weight, eps: float, cos_sin,
                  lines, k_table, write_kv: bool, out_dtype: torch.dtype, pad_to: int = 0) -> torch.Tensor:
    """For attention through latents. Returns the query latent [rows, max(q_rank, pad_to)] (zeros
    behind it): the columns q_off.. of `stacked`, RMS-normed with `q_weight`. The columns kv_off..
    hold the key/value latent (kv_rank, RMS-normed with `kv_weight`) and the row's one rotated key
    part (rot, turned by `cos_sin`); both are written, side by side, as the row's line of the table
    [pages, 1, page_size, kv_rank + rot]."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "latent_append input")
    _need(q_weight, "latent_append query norm", shape=(q_rank,))
    _need(kv_weight, "latent_append key/value norm", q_weight.dtype, (kv_rank,))
    if rot:
        _need(cos_sin, "latent_append cos_sin", torch.float32, (rows, rot // 2, 2))
    cq_width = max(int(pad_to), q_rank)
    cq = _fresh((rows, cq_width), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "latent_append lines", torch.int32, (rows,))
        _need(k_table, "latent_append table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != 1 or k_table.shape[3] != kv_rank + rot:
            raise KernelError(f"latent_append: a table of {tuple(k_table.shape)} is not [pages, 1, page_size, {kv_rank + rot}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(library().kb_latent_append(
        _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(kv_off), int(q_rank), int(kv_rank), int(rot),
        _ptr(q_weight), _ptr(kv_weight), _dt(q_weight, "latent_append norm"), _f(eps), _ptr(cos_sin if rot else None),
        _ptr(lines if write_kv else None), _ptr(cq), cq_width, _ptr(k_table if write_kv else None), _CODES[out_dtype], rows,
        int(bool(write_kv)), ctypes.c_longlong(table_lines), int(page_size), _stream()))
    return cq


def head_linear(x, heads: int, x_head: int, x_off: int, m: torch.Tensor, y_head: Optional[int] = None, tail_off: int = 0,
                tail: int = 0, cos_sin=None, gate=None, g_off: int = 0, pad_to: int = 0, transposed: bool = False) -> torch.Tensor:
    """y[r, h, :n_out] = x[r, h, x_off : x_off + n_in] . m[h] for `m` [heads, n_in, n_out] (its dtype is
    the output's); `x` [rows, heads * x_head] is a tensor or a SplitSum. With `tail`, the components
    x[r, h, tail_off : tail_off + tail] follow the product in y, turned by `cos_sin` [rows, tail/2, 2].
    With `gate` (a float32 stacked product, tensor or SplitSum) the result is multiplied by the sigmoid
    of its columns g_off + h * n_out ... The result is [rows, heads * y_head] (y_head defaults to
    n_out + tail), or [rows, pad_to] with zeros behind the heads. With `transposed`, `m` is bfloat16
    [heads, n_out, n_in] and the product runs on tensor cores."""
    src, x_dt, splits, stride, rows, x_row = _stacked(x, "head_linear input")
    _need(m, "head_linear matrices", torch.bfloat16 if transposed else None)
    if m.dim() != 3 or m.shape[0] != heads:
        raise KernelError(f"head_linear: matrices of {tuple(m.shape)} for {heads} heads")
    n_in, n_out = (int(m.shape[2]), int(m.shape[1])) if transposed else (int(m.shape[1]), int(m.shape[2]))
    y_head = int(y_head) if y_head is not None else n_out + int(tail)
    y_row = max(int(pad_to), heads * y_head)
    if tail:
        _need(cos_sin, "head_linear cos_sin", torch.float32, (rows, tail // 2, 2))
    g_src, g_splits, g_stride, g_row = None, 1, 0, 0
    if gate is not None:
        g_src, g_dt, g_splits, g_stride, g_rows, g_row = _stacked(gate, "head_linear gate")
        if g_dt != F32 or g_rows != rows:
            raise KernelError("head_linear: the gate must be a float32 product of as many rows")
    y = _fresh((rows, y_row), m.dtype, src.device)
    if transposed:
        _check(library().kb_head_linear_mma(
            _ptr(y), y_row, y_head, _ptr(src), x_dt, splits, ctypes.c_longlong(stride), x_row, int(x_head), int(x_off), _ptr(m), n_in, n_out,
            rows, int(heads), int(tail_off), int(tail), _ptr(cos_sin if tail else None), _ptr(g_src), int(g_splits),
            ctypes.c_longlong(g_stride), int(g_row), int(g_off), _stream()))
        return y
    _check(library().kb_head_linear(
        _ptr(y), _dt(m, "head_linear matrices"), y_row, y_head, _ptr(src), x_dt, splits, ctypes.c_longlong(stride), x_row, int(x_head),
        int(x_off), _ptr(m), n_in, n_out, rows, int(heads), int(tail_off), int(tail), _ptr(cos_sin if tail else None), _ptr(g_src),
        int(g_splits), ctypes.c_longlong(g_stride), int(g_row), int(g_off), _stream()))
    return y


def delta_state_floats(heads: int, kv_heads: int, d: int, e: int, taps: int) -> int:
    """Floats a request keeps between steps in a gated-delta-rule layer: the last taps - 1 inputs of
    every convolved channel (queries, keys, values), then every head's memory [e, d]. Plain
    arithmetic (a cache is sized without the CUDA library); `delta_scan` checks it against the library's."""
    return (taps - 1) * (2 * kv_heads * d + heads * e) + heads * d * e


def delta_columns_per_warp(n: int = 0) -> None:
    """How many columns of a head's memory a warp of the delta scan holds: 1, 2 or 4, or 0 for the
    launcher's own choice by the warps a step has (for tests and measurements)."""
    library().kb_delta_columns_per_warp(int(n))


def delta_scan(stacked, q_off: int, k_off: int, v_off: int, b_off: int, a_off: int, conv: torch.Tensor, a_log: torch.Tensor,
               dt_bias: torch.Tensor, state: torch.Tensor, row_entry: torch.Tensor, ranges, slots, entries: int, heads: int,
               kv_heads: int, d: int, e: int, taps: int, q_scale: float, unit_eps: float) -> torch.Tensor:
    """The gated delta rule's read-out [rows, heads, e] (float32, not yet normed) over the rows of a
    step, request by request in row order, from and into `state` [slots, state floats]. `conv`
    [2 kv_heads d + heads e, taps] float32: the short convolutions' filters, the queries' channels
    first, then the keys', then the values'."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "delta input")
    channels = 2 * kv_heads * d + heads * e
    _need(conv, "delta convolution filters", torch.float32, (channels, taps))
    _need(a_log, "delta decay rates", torch.float32, (heads,))
    _need(dt_bias, "delta step biases", torch.float32, (heads,))
    _need(state, "delta state", torch.float32)
    per = delta_state_floats(heads, kv_heads, d, e, taps)
    lib = library()
    if state.dim() != 2 or state.shape[1] != per or int(lib.kb_delta_state_floats(heads, kv_heads, d, e, taps)) != per:
        raise KernelError(f"delta: a state table of {tuple(state.shape)}, expected [slots, {per}]")
    start, end = ranges
    _need(start, "delta entry starts", torch.int32)
    _need(end, "delta entry ends", torch.int32)
    _need(slots, "delta slots", torch.int32)
    _need(row_entry, "delta row_entry", torch.int32, (rows,))
    if min(start.numel(), end.numel(), slots.numel()) < entries:
        raise KernelError(f"delta: {entries} requests but ranges or slots for fewer")
    out = _fresh((rows, heads, e), torch.float32, src.device)
    scratch = _fresh((max(1, int(lib.kb_delta_scratch_floats(rows, heads, kv_heads, d, e))),), torch.float32, src.device)
    _check(lib.kb_delta_scan(
        _ptr(out), _ptr(scratch), _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(k_off), int(v_off),
        int(b_off), int(a_off), _ptr(conv), _ptr(a_log), _ptr(dt_bias), _ptr(state), int(state.shape[0]), ctypes.c_longlong(per),
        _ptr(row_entry), _ptr(start), _ptr(end), _ptr(slots), int(entries), rows, heads, kv_heads, d, e, int(taps), _f(q_scale),
        _f(unit_eps), _stream()))
    return out


def _ranges(ranges, slots, entries: int, what: str):
    start, end = ranges
    _need(start, f"{what} entry starts", torch.int32)
    _need(end, f"{what} entry ends", torch.int32)
    _need(slots, f"{what} slots", torch.int32)
    if min(start.numel(), end.numel(), slots.numel()) < entries:
        raise KernelError(f"{what}: {entries} requests but ranges or slots for fewer")
    return start, end


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, row_entry, ranges, slots, entries: int, keep: bool = True,
                pad_to: int = 0) -> torch.Tensor:
    """y[r] = h[r] + (h[r-1] - h[r]) * mu, channel by channel, for h [rows, width]; the row before a
    request's first row of the step is its slot's line of `state` [slots, width] (float32), and with
    `keep` that line then becomes the request's last h of the step. The result's rows may be wider
    (`pad_to`, zeros behind)."""
    _need(h, "token_shift input")
    rows, width = h.shape
    _need(mu, "token_shift weights", torch.float32, (width,))
    _need(state, "token_shift state", torch.float32)
    if state.dim() != 2 or state.shape[1] != width:
        raise KernelError(f"token_shift: a state table of {tuple(state.shape)}, expected [slots, {width}]")
    _need(row_entry, "token_shift row_entry", torch.int32, (rows,))
    start, end = _ranges(ranges, slots, entries, "token_shift")
    out_width = max(int(pad_to), width)
    out = _fresh((rows, out_width), h.dtype, h.device)
    _check(library().kb_token_shift(_ptr(out), _ptr(h), _dt(h, "token_shift input"), _ptr(mu), _ptr(state), _ptr(row_entry), _ptr(start),
                                    _ptr(end), _ptr(slots), int(entries), int(state.shape[0]), rows, width, out_width, int(bool(keep)),
                                    _stream()))
    return out


def conv_state_floats(hq: int, hkv: int, d: int, taps: int) -> int:
    """Floats a request keeps between steps for the short convolutions on queries and keys: the last
    taps - 1 inputs of every channel (one float that nobody reads where a filter has one weight, so that
    the state table has a line a request all the same)."""
    return max(1, (taps - 1) * (hq + hkv) * d)


def conv_append(stacked, q_off: int, k_off: int, bias: Optional[torch.Tensor], conv: torch.Tensor, state: torch.Tensor, row_entry,
                ranges, slots, entries: int, lines, k_table, hq: int, hkv: int, d: int, taps: int, write_kv: bool,
                out_dtype: torch.dtype, pad_to: int = 0) -> torch.Tensor:
    """Queries [rows, hq d] (or `pad_to` wide, zeros behind) and keys through a short causal convolution
    over time, one filter a channel (`conv` [(hq + hkv) d, taps] float32, the last weight for the row
    itself), after `bias` [(hq + hkv) d]; the keys are written at each row's line of `k_table`
    [pages, hkv, page_size, d]. `state` [slots, (taps - 1) (hq + hkv) d] holds every request's last inputs."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "conv_append input")
    channels = (hq + hkv) * d
    _need(conv, "conv_append filters", torch.float32, (channels, taps))
    if bias is not None:
        _need(bias, "conv_append bias", torch.float32, (channels,))
    _need(state, "conv_append state", torch.float32)
    if state.dim() != 2 or state.shape[1] != conv_state_floats(hq, hkv, d, taps):
        raise KernelError(f"conv_append: a state table of {tuple(state.shape)}, expected [slots, {conv_state_floats(hq, hkv, d, taps)}]")
    _need(row_entry, "conv_append row_entry", torch.int32, (rows,))
    start, end = _ranges(ranges, slots, entries, "conv_append")
    q_width = max(int(pad_to), hq * d)
    q = _fresh((rows, q_width), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "conv_append lines", torch.int32, (rows,))
        _need(k_table, "conv_append table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d:
            raise KernelError(f"conv_append: a table of {tuple(k_table.shape)} is not [pages, {hkv}, page_size, {d}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(library().kb_conv_append(
        _ptr(q), q_width, _ptr(k_table if write_kv else None), _CODES[out_dtype], _ptr(src), dt, splits, ctypes.c_longlong(stride), width,
        int(q_off), int(k_off), _ptr(bias), _ptr(conv), _ptr(state), int(state.shape[0]), _ptr(row_entry), _ptr(start), _ptr(end),
        _ptr(slots), _ptr(lines if write_kv else None), int(entries), rows, int(hq), int(hkv), int(d), int(taps), int(bool(write_kv)),
        ctypes.c_longlong(table_lines), int(page_size), _stream()))
    return q


def decay_scan_columns(n: int = 0) -> None:
    """How many columns of a head's memory a warp of the decay scan holds: 1, 2 or 4, or 0 for the
    launcher's own choice by the warps a step has (for tests and measurements)."""
    library().kb_decay_scan_columns(int(n))


def gdelta_scan(stacked, r_off: int, k_off: int, v_off: int, a_off: int, w1_off: int, w2: torch.Tensor, w0: torch.Tensor,
                a_bias: torch.Tensor, decay_scale: float, unit_eps: float, state: torch.Tensor, ranges, slots, entries: int,
                heads: int, d: int) -> torch.Tensor:
    """The generalized delta rule's read-out [rows, heads, d] (float32, not yet normed) over the rows of a
    step, request by request in row order, from and into `state` [slots, heads, d, d]. Per head, with the
    decay w = exp(-decay_scale sigmoid(w2 tanh(w1 h) + w0)), the removal rate a = sigmoid(a h + a_bias) and
    the unit key u = k / sqrt(sum k^2 + unit_eps): S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r. `w2` is
    the net's second layer turned, [hidden, heads d] (neighbouring threads read neighbouring weights). The
    columns r_off, k_off, v_off, a_off (heads d each) and w1_off (the small net's hidden layer, before
    its tanh) of `stacked` hold the projections."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "gdelta input")
    n = heads * d
    _need(w2, "gdelta decay weights", torch.float32)
    if w2.dim() != 2 or w2.shape[1] != n:
        raise KernelError(f"gdelta: decay weights of {tuple(w2.shape)}, expected [hidden, {n}] (the net's second layer, turned)")
    lora = int(w2.shape[0])
    _need(w0, "gdelta decay bias", torch.float32, (n,))
    _need(a_bias, "gdelta removal bias", torch.float32, (n,))
    _need(state, "gdelta state", torch.float32)
    if state.dim() != 2 or state.shape[1] != n * d:
        raise KernelError(f"gdelta: a state table of {tuple(state.shape)}, expected [slots, {n * d}]")
    start, end = _ranges(ranges, slots, entries, "gdelta")
    lib = library()
    out = _fresh((rows, heads, d), torch.float32, src.device)
    scratch = _fresh((max(1, int(lib.kb_decay_scan_scratch_floats(rows, heads, d, d, 1))),), torch.float32, src.device)
    _check(lib.kb_gdelta_scan(
        _ptr(out), _ptr(scratch), _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(r_off), int(k_off), int(v_off), int(a_off),
        int(w1_off), lora, _ptr(w2), _ptr(w0), _ptr(a_bias), _f(decay_scale), _f(unit_eps), _ptr(state), int(state.shape[0]),
        _ptr(start), _ptr(end), _ptr(slots), int(entries), rows, int(heads), int(d), _stream()))
    return out


def gate_scan(stacked, q_off: int, f_off: int, v_off: int, f_bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor, ranges,
              slots, entries: int, heads: int, d: int, e: int) -> torch.Tensor:
    """The read-out [rows, heads, e] (float32, not yet normed) of a matrix memory with tied gates (the
    input gate is one minus the forget gate): q = silu(.), f = lower + (1 - lower) sigmoid(. + f_bias) per head and
    channel; S <- diag(f) S + (1 - f) v^T, o = S^T q; `state` [slots, heads e d]."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "gate_scan input")
    _need(f_bias, "gate_scan gate bias", torch.float32, (heads * d,))
    _need(lower, "gate_scan lower bounds", torch.float32, (heads * d,))
    _need(state, "gate_scan state", torch.float32)
    if state.dim() != 2 or state.shape[1] != heads * d * e:
        raise KernelError(f"gate_scan: a state table of {tuple(state.shape)}, expected [slots, {heads * d * e}]")
    start, end = _ranges(ranges, slots, entries, "gate_scan")
    lib = library()
    out = _fresh((rows, heads, e), torch.float32, src.device)
    scratch = _fresh((max(1, int(lib.kb_decay_scan_scratch_floats(rows, heads, d, e, 0))),), torch.float32, src.device)
    _check(lib.kb_gate_scan(
        _ptr(out), _ptr(scratch), _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(f_off), int(v_off),
        _ptr(f_bias), _ptr(lower), _ptr(state), int(state.shape[0]), _ptr(start), _ptr(end), _ptr(slots), int(entries), rows,
        int(heads), int(d), int(e), _stream()))
    return out


def weighted_sum2(a, va: torch.Tensor, b=None, vb: Optional[torch.Tensor] = None, vc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a * va + b * vb + vc in float32 for branches [rows, width] (tensors or SplitSums) with a weight a
    channel each (float32 [width]); `b` and `vc` may be absent."""
    a_src, a_dt, a_splits, a_stride = _src(a, "weighted_sum2 first branch")
    rows, width = a.shape
    _need(va, "weighted_sum2 first weights", torch.float32, (width,))
    b_src, b_dt, b_splits, b_stride = None, F32, 1, 0
    if b is not None:
        if tuple(b.shape) != (rows, width):
            raise KernelError(f"weighted_sum2: branches of {tuple(a.shape)} and {tuple(b.shape)}")
        b_src, b_dt, b_splits, b_stride = _src(b, "weighted_sum2 second branch")
        _need(vb, "weighted_sum2 second weights", torch.float32, (width,))
    if vc is not None:
        _need(vc, "weighted_sum2 offsets", torch.float32, (width,))
    out = _fresh((rows, width), torch.float32, a_src.device)
    _check(library().kb_weighted_sum2(_ptr(out), _ptr(a_src), a_dt, a_splits, ctypes.c_longlong(a_stride), _ptr(va), _ptr(b_src), b_dt,
                                      b_splits, ctypes.c_longlong(b_stride), _ptr(vb if b is not None else None), _ptr(vc),
                                      ctypes.c_longlong(rows), int(width), _stream()))
    return out


def entry_ranges(row_entry: torch.Tensor, entries: int):
    """(start, end) int32 [entries]: rows [start[e], end[e]) are request e's in this step."""
    _need(row_entry, "entry_ranges row_entry", torch.int32)
    both = _fresh((2, max(int(entries), 1)), torch.int32, row_entry.device)
    _check(library().kb_entry_ranges(_ptr(both[0]), _ptr(both[1]), _ptr(row_entry), int(row_entry.numel()), int(entries), _stream()))
    return both[0], both[1]


MLSTM_SLICE = 4           # value components a block of the scan kernel holds (the kernel file's MV)
MLSTM_SHARE = 32          # threads that share a value component (its MJ)


def mlstm_state_floats(d: int, e: int) -> int:
    """Floats a head keeps between steps: for every slice of value components the scan kernel cuts
    a head into, the memory's rows in the order of the threads that hold them and a copy of the
    normaliser [d]; then the running maximum, once. Plain arithmetic (a cache is sized without the CUDA
    library); `mlstm_scan` checks it against the library's."""
    return -(-e // MLSTM_SLICE) * (-(-d // MLSTM_SHARE) * MLSTM_SLICE * MLSTM_SHARE + d) + 1


def mlstm_scan(stacked, q_off: int, k_off: int, v_off: int, i_off: int, f_off: int, bias_i, bias_f, state, ranges, slots,
               entries: int, heads: int, d: int, e: int, cap: float, q_scale: float, floor: float) -> torch.Tensor:
    """The matrix memory's read-out [rows, heads, e] (float32, not yet normed) over the rows of a
    step, request by request in row order, from and into `state` [slots, heads, state floats]."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "mlstm input")
    _need(bias_i, "mlstm input-gate bias", torch.float32, (heads,))
    _need(bias_f, "mlstm forget-gate bias", torch.float32, (heads,))
    _need(state, "mlstm state", torch.float32)
    per_head = mlstm_state_floats(d, e)
    if state.dim() != 3 or state.shape[1] != heads or state.shape[2] != per_head:
        raise KernelError(f"mlstm: a state table of {tuple(state.shape)}, expected [slots, {heads}, {per_head}]")
    if int(library().kb_mlstm_state_floats(d, e)) != per_head:
        raise KernelError("mlstm: the library cuts a head's state differently from the cache")
    start, end = ranges
    _need(start, "mlstm entry starts", torch.int32)
    _need(end, "mlstm entry ends", torch.int32)
    _need(slots, "mlstm slots", torch.int32)
    if min(start.numel(), end.numel(), slots.numel()) < entries:
        raise KernelError(f"mlstm: {entries} requests but ranges or slots for fewer")
    out = _fresh((rows, heads, e), torch.float32, src.device)
    factors = _fresh((rows, heads, 3), torch.float32, src.device)        # the gates' kernel leaves every row's three factors here
    _check(library().kb_mlstm_scan(
        _ptr(out), _ptr(factors), _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(k_off), int(v_off), int(i_off), int(f_off),
        _ptr(bias_i), _ptr(bias_f), _ptr(state), int(state.shape[0]), _ptr(start), _ptr(end), _ptr(slots), int(entries), rows,
        heads, d, e, _f(cap), _f(q_scale), _f(floor), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Attention over a window plus pooled blocks, with the heads' weights mixed.
def proj_rope_append(stacked, q_off: int, k_off: int, v_off: int, biases, q_norm, k_norm, cos_sin, rotary: int, neighbours: bool,
                     v_other: Optional[torch.Tensor], v_weight: Optional[torch.Tensor], keep_values: bool, lines, k_table, v_table,
                     hq: int, hkv: int, d: int, dv: int, write_kv: bool, out_dtype: torch.dtype):
    """q [rows, hq, d] from the columns q_off.. of `stacked` (a tensor or a SplitSum): plus the bias
    `biases[0]`, normed over the whole projection when `q_norm` = (weight [hq d], eps, offset) is given,
    the first `rotary` components of every head turned by `cos_sin` [rows, rotary/2, 2] (pairs
    (i, i + rotary/2), or (2i, 2i+1) with `neighbours`). Keys likewise (`biases[1]`, `k_norm`) and written
    at each row's line of the table [pages, hkv, page_size, d]. Values: plus `biases[2]`; with `v_other`
    [rows, hkv dv] float32 and `v_weight` (one value l on the device) v <- (1 - l) v + l v_other; written
    to the table [.., dv]. Returns (q, the values before that mix as float32 [rows, hkv dv] if
    `keep_values`, else None). Biases and norm weights share a dtype."""
    src, dt, splits, stride, rows, width = _stacked(stacked, "proj_rope_append input")
    bq, bk, bv = biases if biases is not None else (None, None, None)
    wq, eq, oq = q_norm if q_norm is not None else (None, 0.0, 0.0)
    wk, ek, ok = k_norm if k_norm is not None else (None, 0.0, 0.0)
    small = [t for t in (bq, bk, bv, wq, wk, v_weight) if t is not None]
    if len({t.dtype for t in small}) > 1:
        raise KernelError("proj_rope_append: biases, norm weights and the values' weight differ in dtype")
    for t, n, what in ((bq, hq * d, "q bias"), (bk, hkv * d, "k bias"), (bv, hkv * dv, "v bias"), (wq, hq * d, "q norm"), (wk, hkv * d, "k norm")):
        if t is not None:
            _need(t, f"proj_rope_append {what}", shape=(n,))
    w_dt = _dt(small[0], "proj_rope_append weights") if small else F32
    if rotary:
        _need(cos_sin, "proj_rope_append rotation table", torch.float32, (rows, rotary // 2, 2))
    if (v_other is None) != (v_weight is None):
        raise KernelError("proj_rope_append: other values and their weight come together")
    if v_other is not None:
        _need(v_other, "proj_rope_append other values", torch.float32, (rows, hkv * dv))
        if v_weight.numel() != 1:
            raise KernelError(f"proj_rope_append: the values' weight has {v_weight.numel()} values")
    q = _fresh((rows, hq, d), out_dtype, src.device)
    kept = _fresh((rows, hkv * dv), torch.float32, src.device) if keep_values else None
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "proj_rope_append lines", torch.int32, (rows,))
        _need(k_table, "proj_rope_append k table", out_dtype)
        _need(v_table, "proj_rope_append v table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d or v_table.dim() != 4 or \
                tuple(v_table.shape) != (*k_table.shape[:3], dv):
            raise KernelError(f"proj_rope_append: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, {hkv}, page_size, {d} / {dv}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(library().kb_proj_rope_append(
        _ptr(src), dt, splits, ctypes.c_longlong(stride), width, int(q_off), int(k_off), int(v_off), _ptr(bq), _ptr(bk), _ptr(bv),
        _ptr(wq), _f(eq), _f(oq), _ptr(wk), _f(ek), _f(ok), w_dt, _ptr(cos_sin if rotary else None), int(rotary), int(bool(neighbours)),
        _ptr(v_other), _ptr(v_weight), _ptr(kept), _ptr(lines if write_kv else None), _ptr(q), _ptr(k_table if write_kv else None),
        _ptr(v_table if write_kv else None), _CODES[out_dtype], rows, hq, hkv, d, dv, int(bool(write_kv)),
        ctypes.c_longlong(table_lines), int(page_size), _stream()))
    return q, kept


def pool_blocks(k_table, v_table, block_table, row_entry, positions, lines, slots, pooled: torch.Tensor, pool: int) -> None:
    """For every row whose position ends a block of `pool` positions: the means of the block's keys and
    of its values, read back from the cache, into pooled[slot of the row's request, block] (`pooled` is
    float32 [slots, blocks, kv_heads, d + dv])."""
    _need(k_table, "pool_blocks k table")
    _need(v_table, "pool_blocks v table", k_table.dtype)
    _need(pooled, "pool_blocks means", torch.float32)
    n_pages, hkv, page_size, d = k_table.shape
    dv = v_table.shape[3]
    if pooled.dim() != 4 or pooled.shape[2] != hkv or pooled.shape[3] != d + dv:
        raise KernelError(f"pool_blocks: means {tuple(pooled.shape)} are not [slots, blocks, {hkv}, {d + dv}]")
    rows = positions.numel()
    for t, what in ((row_entry, "row_entry"), (positions, "positions"), (lines, "lines")):
        _need(t, f"pool_blocks {what}", torch.int32, (rows,))
    _need(slots, "pool_blocks slots", torch.int32)
    _need(block_table, "pool_blocks block table", torch.int32)
    _check(library().kb_pool_blocks(
        _ptr(k_table), _ptr(v_table), _dt(k_table, "pool_blocks k table"), _ptr(block_table), int(block_table.shape[1]), int(n_pages),
        _ptr(row_entry), _ptr(positions), _ptr(lines), _ptr(slots), _ptr(pooled), ctypes.c_longlong(pooled.stride(0)), int(pooled.shape[0]),
        int(pooled.shape[1]), int(pool), rows, int(hkv), int(d), int(dv), int(page_size), _stream()))


_POOLED_CHUNK = None


def pooled_attention_chunk() -> int:
    """Keys a step of the kernel below: slices of the keys are multiples of it."""
    global _POOLED_CHUNK
    if _POOLED_CHUNK is None:
        _POOLED_CHUNK = int(library().kb_pooled_attention_chunk())
    return _POOLED_CHUNK


POOLED_KEPT_BYTES = int(_os.environ.get("KAPEL_B200_POOLED_KEPT_BYTES", str(4 << 30)))


def pooled_attention_tile_rows() -> int:
    """Tokens a tile of the tensor-core kernel of `pooled_attention`."""
    return int(library().kb_pooled_attention_mma_tile_rows())


def pooled_attention_tiled(hq: int, hkv: int, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel of `pooled_attention` takes these sizes (bfloat16 rows in tiles)."""
    return bool(library().kb_pooled_attention_mma_takes(int(hq), int(hkv), int(d), int(dv)))


def pooled_attention(q, k_table, v_table, pooled: Optional[torch.Tensor], block_table, row_entry, row_count, slots, talk, temp,
                     page_size: int, window: Optional[int], pool: int, scale: float, splits: int = 1, split_keys: int = 0,
                     tiles=None, longest: Optional[int] = None) -> torch.Tensor:
    """Attention of each query row [rows, hq, d] over the last `window` tokens of its sequence (all with
    `window` None) and the pooled blocks of `pool` positions that lie wholly below the window (their mean
    keys and values in `pooled` [slots, blocks, hkv, d + dv], float32), in one softmax; score = q.k * scale
    * temp[h]; then the heads' weights are mixed by `talk` [hq, hq] (float32; None: no mix) ahead of the
    values. With `splits` > 1 the keys are cut into that many slices of `split_keys` across blocks.
    With `tiles` ((tile_entry, tile_row0, tile_nq) on the device: each request's rows in runs of at most
    `pooled_attention_tile_rows()`) bfloat16 rows of sizes that `pooled_attention_tiled` names go to the
    tensor-core kernel, which walks a tile's keys for all heads together; `longest` is the most positions any row
    has seen (read back from `row_count` if not given)."""
    rows, hq, d = q.shape
    _need(q, "pooled attention q")
    _need(k_table, "pooled attention k table", q.dtype)
    _need(v_table, "pooled attention v table", q.dtype)
    if k_table.dim() != 4 or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.dim() != 4 or v_table.shape[:3] != k_table.shape[:3]:
        raise KernelError(f"pooled attention: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, kv_heads, {page_size}, {d}]")
    n_pages, hkv, dv = k_table.shape[0], k_table.shape[1], v_table.shape[3]
    n_slots = max_blocks = 0
    stride = 0
    if pool:
        _need(pooled, "pooled attention means", torch.float32)
        if pooled.dim() != 4 or pooled.shape[2] != hkv or pooled.shape[3] != d + dv:
            raise KernelError(f"pooled attention: means {tuple(pooled.shape)} are not [slots, blocks, {hkv}, {d + dv}]")
        n_slots, max_blocks, stride = int(pooled.shape[0]), int(pooled.shape[1]), int(pooled.stride(0))
    if talk is not None:
        _need(talk, "pooled attention head mix", torch.float32, (hq, hq))
    if temp is not None:
        _need(temp, "pooled attention head temperatures", torch.float32, (hq,))
    _need(block_table, "pooled attention block table", torch.int32)
    _need(row_entry, "pooled attention row_entry", torch.int32, (rows,))
    _need(row_count, "pooled attention row_count", torch.int32, (rows,))
    _need(slots, "pooled attention slots", torch.int32)
    out = _fresh((rows, hq, dv), q.dtype, q.device)
    lib = library()
    if tiles is not None and q.dtype == torch.bfloat16 and pooled_attention_tiled(hq, int(hkv), d, int(dv)):
        tile_entry, tile_row0, tile_nq = tiles
        n_tiles = int(tile_entry.shape[0])
        for name, t in (("tile_entry", tile_entry), ("tile_row0", tile_row0), ("tile_nq", tile_nq)):
            _need(t, f"pooled attention {name}", torch.int32, (n_tiles,))
        scratch = _fresh((lib.kb_pooled_attention_mma_scratch_floats(rows, hq),), torch.float32, q.device)
        # The first launch keeps its scores for the second where that costs at most POOLED_KEPT_BYTES of scratch memory.
        if longest is None:
            longest = int(row_count.max())
        n_kept = int(lib.kb_pooled_attention_mma_kept_floats(n_tiles, hq, int(hkv), d, int(dv), int(window or 0), int(pool or 0), max_blocks, int(longest)))
        kept = _fresh((n_kept,), torch.float32, q.device) if 0 < n_kept * 4 <= POOLED_KEPT_BYTES else None
        _check(lib.kb_pooled_attention_mma(
            _ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _ptr(pooled if pool else None), ctypes.c_longlong(stride), n_slots, max_blocks,
            _ptr(block_table), _ptr(row_count), _ptr(tile_entry), _ptr(tile_row0), _ptr(tile_nq), n_tiles, _ptr(slots), _ptr(talk), _ptr(temp),
            rows, hq, int(hkv), d, int(dv), int(page_size), int(block_table.shape[1]), int(n_pages), int(window or 0), int(pool or 0), _f(scale),
            _ptr(scratch), _ptr(kept), int(longest), _stream()))
        return out
    need = lib.kb_pooled_attention_scratch_floats(rows, hq, int(dv), int(splits), int(split_keys))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    _check(lib.kb_pooled_attention(
        _ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _dt(q, "pooled attention q"), _ptr(pooled if pool else None),
        ctypes.c_longlong(stride), n_slots, max_blocks, _ptr(block_table), _ptr(row_entry), _ptr(row_count), _ptr(slots), _ptr(talk),
        _ptr(temp), rows, hq, int(hkv), d, int(dv), int(page_size), int(block_table.shape[1]), int(n_pages), int(window or 0), int(pool or 0),
        _f(scale), int(splits), int(split_keys), _ptr(scratch), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Mixture of experts.
MOE_ACT_CODES = {"none": 0, "relu2": 1, "gelu_tanh": 2, "silu": 3}
# How the router's logits z become scores: sigmoid(z); the softmax over all experts; or "softmax_chosen":
# z itself chooses and the chosen experts are weighted by the softmax over their logits alone.
ROUTE_SCORING = {"sigmoid": 0, "softmax": 1, "softmax_chosen": 2}


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep_groups: int,
              group_top: int, scoring: str, renormalize: bool):
    """(experts int32 [rows, top], weights float32 [rows, top]) of each row of h [rows, width];
    the router [experts, width] and the correction [experts] are float32."""
    _need(h, "moe_route input")
    rows, width = h.shape
    _need(router, "moe_route router", torch.float32)
    n_experts = router.shape[0]
    if router.shape[1] != width:
        raise KernelError(f"moe_route: router {tuple(router.shape)} against rows of {width}")
    if correction is not None:
        _need(correction, "moe_route correction", torch.float32, (n_experts,))
    if scoring not in ROUTE_SCORING:
        raise KernelError(f"moe_route: scoring {scoring!r} is not known ({sorted(ROUTE_SCORING)})")
    experts = _fresh((rows, top), torch.int32, h.device)
    weights = _fresh((rows, top), torch.float32, h.device)
    _check(library().kb_moe_route(_ptr(experts), _ptr(weights), _ptr(h), _dt(h, "moe_route input"), _ptr(router), _ptr(correction),
                                  rows, width, n_experts, int(top), int(groups), int(keep_groups), int(group_top),
                                  ROUTE_SCORING[scoring], int(bool(renormalize)), _stream()))
    return experts, weights


class ExpertLists:
    """The (token, k) pairs of a step listed by expert, and the row tiles of the grouped products."""

    __slots__ = ("order", "offsets", "tiles", "tile_cap", "tile_rows", "pairs", "top")


def moe_sort(experts: torch.Tensor, n_experts: int, dtype: torch.dtype = torch.float32) -> ExpertLists:
    """Lists the pairs of `experts` [rows, top] by expert; `dtype` is the grouped products' (it and the
    rows an expert gets on average decide how many rows a tile of those products has)."""
    _need(experts, "moe_sort experts", torch.int32)
    rows, top = experts.shape
    pairs = rows * top
    lists = ExpertLists()
    lists.pairs, lists.top = pairs, top
    lists.tile_rows = int(library().kb_moe_tile_rows(_CODES[dtype], ctypes.c_longlong(pairs // max(n_experts, 1))))
    # every expert's list ends with at most one tile that is not full
    lists.tile_cap = pairs // lists.tile_rows + min(n_experts, pairs)
    buf = _fresh((n_experts + 1 + pairs + 3 * max(lists.tile_cap, 1) + 1,), torch.int32, experts.device)
    at = n_experts + 1
    lists.offsets, lists.order = buf[:at], buf[at : at + pairs]
    at += pairs
    cap = max(lists.tile_cap, 1)
    lists.tiles = (buf[at : at + cap], buf[at + cap : at + 2 * cap], buf[at + 2 * cap : at + 3 * cap], buf[at + 3 * cap :])
    _check(library().kb_moe_sort(_ptr(experts), pairs, int(n_experts), _ptr(lists.offsets), _ptr(lists.order), _ptr(lists.tiles[0]),
                                 _ptr(lists.tiles[1]), _ptr(lists.tiles[2]), _ptr(lists.tiles[3]), int(lists.tile_cap),
                                 int(lists.tile_rows), _stream()))
    return lists


def moe_grouped(a: torch.Tensor, w: torch.Tensor, lists: ExpertLists, act: str, a_by_token: bool, out_by_pair: bool,
                out_dtype: torch.dtype) -> torch.Tensor:
    """out [pairs, n]: act(a[row] . w[expert]^T) for every (token, k) pair, by expert. `a` rows are
    taken by the pair's token (`a_by_token`) or by its place in the expert lists; the result's rows
    are placed by pair number (`out_by_pair`) or by that place. w is [experts, n, k]."""
    _need(a, "moe_grouped input")
    _need(w, "moe_grouped weights", a.dtype)
    if w.dim() != 3 or w.shape[2] != a.shape[1]:
        raise KernelError(f"moe_grouped: weights {tuple(w.shape)} against rows of {a.shape[1]}")
    if act not in MOE_ACT_CODES:
        raise KernelError(f"moe_grouped: activation {act!r} is not known")
    n, k = int(w.shape[1]), int(w.shape[2])
    out = _fresh((lists.pairs, n), out_dtype, a.device)
    t = lists.tiles
    _check(library().kb_moe_grouped(_ptr(out), _CODES[out_dtype], _ptr(a), _ptr(w), _dt(a, "moe_grouped input"), _ptr(lists.order),
                                    _ptr(t[0]), _ptr(t[1]), _ptr(t[2]), _ptr(t[3]), int(lists.tile_cap), int(lists.tile_rows), n, k, int(lists.top),
                                    MOE_ACT_CODES[act], int(bool(a_by_token)), int(bool(out_by_pair)), _stream()))
    return out


def moe_combine(y: torch.Tensor, weights: torch.Tensor, out_dtype: torch.dtype, also=None) -> torch.Tensor:
    """out[token] = sum over k, in order, of weights[token, k] * y[token * top + k], plus `also`[token]
    where given (a tensor or a SplitSum [tokens, width]: the output of an expert that every token uses)."""
    _need(y, "moe_combine input", torch.float32)
    _need(weights, "moe_combine weights", torch.float32)
    rows, top = weights.shape
    width = y.shape[1]
    if y.shape[0] != rows * top:
        raise KernelError(f"moe_combine: {y.shape[0]} rows for {rows} tokens of {top} experts")
    a_src, a_dt, a_splits, a_stride = (None, F32, 1, 0)
    if also is not None:
        a_src, a_dt, a_splits, a_stride = _src(also, "moe_combine addend")
        if tuple(also.shape) != (rows, width):
            raise KernelError(f"moe_combine: an addend {tuple(also.shape)} beside a sum of {(rows, width)}")
    out = _fresh((rows, width), out_dtype, y.device)
    _check(library().kb_moe_combine(_ptr(out), _CODES[out_dtype], _ptr(y), _ptr(weights), ctypes.c_longlong(rows), int(width), int(top),
                                    _ptr(a_src), a_dt, int(a_splits), ctypes.c_longlong(a_stride), _stream()))
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None, uniform: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token a row: the first largest logit where temperature <= 0 (or none is given), else
    a draw with the row's uniform number."""
    _need(logits, "sample logits", torch.float32)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "sample temperature", torch.float32, (rows,))
        _need(uniform, "sample uniform", torch.float32, (rows,))
    out = _fresh((rows,), torch.int32, logits.device)
    lib = library()
    need = int(lib.kb_sample_scratch_floats(rows, vocab))
    scratch = _fresh((need,), torch.float32, logits.device) if need else None
    _check(lib.kb_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(uniform), rows, vocab, _ptr(scratch), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Timing by kernel name, in the manner of Kapel's `Timed<B>` wrapper backend
# (crates/kapel-cli/examples/profile.rs:17-56): every entry point above is bracketed by CUDA
# events and its device time added up under its name and its largest argument's shape.
_TIMED = ("embed", "rope_table", "rope_append", "glu", "cast", "gather_rows", "rmsnorm", "add_rmsnorm", "gemm",
          "paged_attention_rows", "paged_attention_mma", "sample", "proj_norm_append", "head_gate", "mlstm_scan", "moe_route",
          "moe_sort", "moe_grouped", "moe_combine", "gemm_glu_fused", "paged_attention_decode_fused", "layernorm", "concat2",
          "head_norm_rope_append", "latent_append", "head_linear", "delta_scan", "latent_attention_mma", "proj_rope_append",
          "pool_blocks", "pooled_attention", "act", "token_shift", "conv_append", "gdelta_scan", "gate_scan", "weighted_sum2",
          "glu_clamped")
_timing = None
_originals = {}


def enable_timing() -> None:
    """Wraps the entry points with CUDA-event timers (each call then synchronises: for
    measuring where a step's time goes, never while timing the step itself, and not with
    recorded steps)."""
    global _timing
    if _timing is not None:
        return
    _timing = {}
    g = globals()
    for name in _TIMED:
        fn = g[name]
        _originals[name] = fn

        def timed(*args, __fn=fn, __name=name, **kw):
            shape = max((tuple(a.shape) for a in args if isinstance(a, torch.Tensor)), key=lambda s: int(torch.Size(s).numel()), default=())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = __fn(*args, **kw)
            b.record()
            b.synchronize()
            rec = _timing.setdefault((__name, shape), [0, 0.0])
            rec[0] += 1
            rec[1] += a.elapsed_time(b)
            return out

        g[name] = timed


def disable_timing() -> None:
    global _timing
    for name, fn in _originals.items():
        globals()[name] = fn
    _originals.clear()
    _timing = None


def timing_report(reset: bool = True):
    """[(name, shape, calls, total ms)] sorted by total time."""
    rows = sorted(((n, s, c, ms) for (n, s), (c, ms) in (_timing or {}).items()), key=lambda r: -r[3])
    if reset and _timing is not None:
        _timing.clear()
    return rows
