"""The kernels as Python functions over CUDA tensors.

This module loads the compiled library (building it at the first call) and
checks every argument before handing raw pointers to it.  There is no CPU
fallback and no library model code behind these functions: without a GPU, or
when the library cannot be built or loaded, they raise.

Conventions: the residual stream and every matrix product's output are
float32.  A product's output is a stack ``[S, n, m]`` of S partial sums whose
sum over S is the result (S = 1 unless the product was split over k); the
kernels that consume a product add the partial sums in the order 0 .. S-1.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import torch

from . import build

PAGE = 64  # positions per cache page; common.cuh has the same number

_DT = {torch.float32: 0, torch.bfloat16: 1}
_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    pass


_C_TYPES = {"int": ctypes.c_int, "int32_t": ctypes.c_int32, "unsigned": ctypes.c_uint,
            "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
            "float": ctypes.c_float, "double": ctypes.c_double, "size_t": ctypes.c_size_t,
            "cudaStream_t": ctypes.c_void_p}


def _c_type(decl: str, with_name: bool):
    """The ctypes type of a parameter (or return type) as kernels.h writes it."""
    decl = decl.strip()
    if "*" in decl:
        return ctypes.c_void_p
    words = [w for w in decl.split() if w != "const"]     # also folds runs of blanks
    if with_name:
        words = words[:-1]
    return _C_TYPES[" ".join(words)]


def declare(library: ctypes.CDLL, header: str) -> int:
    """Gives every function that ``header`` (the text of kernels.h) declares its
    argument and return types, so that a call converts plain Python numbers (and
    None for a null pointer) by the declared type instead of guessing it from each
    argument: a wrong guess would pass a 64-bit size as 32 bits.  Returns how many
    functions were declared; one that the header has and the library lacks, or a
    type the table above does not know, raises."""
    import re
    text = re.sub(r"//[^\n]*", "", header)
    count = 0
    for ret, name, params in re.findall(
            r"\b((?:unsigned\s+)?(?:long\s+long|int|float|double))\s+(jb_\w+)\s*\(([^)]*)\)\s*;", text):
        fn = getattr(library, name)
        params = params.strip()
        fn.argtypes = [] if params in ("", "void") else [_c_type(p, True)
                                                         for p in params.split(",")]
        fn.restype = _c_type(ret, False)
        count += 1
    return count


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build.library_path()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"janas_b200: cannot load {path}: {e}") from None
                import os
                with open(os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                       "kernels.h")) as f:
                    declare(loaded, f.read())
                _lib = loaded
    return _lib


def loaded_library_path() -> Optional[str]:
    return _lib._name if _lib is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked on every launch, so by the short
    way when this PyTorch has it (the Stream object costs several microseconds)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    """A tensor's address for a pointer argument (None: a null pointer)."""
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    """A contiguous CUDA tensor of the given dtype (one, or a tuple of allowed ones)
    and shape (None: any size there).  Called several times per launch, so written
    for speed: dtypes are compared by identity, sizes in a plain loop."""
    try:
        ok = t.is_cuda
    except AttributeError:
        ok = False
    if not ok:
        raise KernelError(f"{name}: a CUDA tensor is needed (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None:
        td = t.dtype
        if td is not dtype and (dtype.__class__ is torch.dtype or td not in dtype):
            raise KernelError(f"{name}: dtype {td}, expected {dtype}")
    if shape is not None:
        ts = t.shape
        bad = len(shape) != len(ts)
        if not bad:
            for s, d in zip(shape, ts):
                if s is not None and s != d:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(ts)}, expected {tuple(shape)}")


# how many of the library's kernels have been launched (for measurements)
COUNTERS = {"launches": 0}


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code == 0:
        COUNTERS["launches"] += kernels
        return
    if code == -1:
        raise KernelError(f"{what}: the kernel does not take these sizes or types")
    raise KernelError(f"{what}: the launch failed (code {code})")


_FLOATS = (torch.float32, torch.bfloat16)


def stack(t: torch.Tensor) -> torch.Tensor:
    """A product's output as a stack of partial sums: [n, m] -> [1, n, m]."""
    return t if t.dim() == 3 else t.unsqueeze(0)


# ------------------------------------------------------------------ row-wise
def embed(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[j, :] = table[tokens[j], :] as float32."""
    _need(table, "embedding table", _FLOATS)
    _need(tokens, "tokens", torch.int32)
    n, dm = tokens.numel(), table.shape[1]
    x = torch.empty((n, dm), dtype=torch.float32, device=table.device)
    _check(lib().jb_embed(_p(table), _DT[table.dtype], _p(tokens), _p(x), n, dm, _stream()),
           "embed")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the rows of x (float32 [n, dm]).

    With ``delta`` (a stack [S, n, dm] of float32 partial sums) x is first
    updated in place, x += delta[0] + ... + delta[S-1].  With ``rows`` (int32
    indices) only those rows are normalized and returned, in that order."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    _need(weight, "norm weight", _FLOATS, (dm,))
    S, stride = 0, 0
    if delta is not None:
        delta = stack(delta)
        _need(delta, "delta", torch.float32, (None, n, dm))
        S, stride = delta.shape[0], n * dm
        if rows is not None:
            raise KernelError("rmsnorm: delta and rows cannot be combined")
    n_out = n
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    out = torch.empty((n_out, dm), dtype=out_dtype, device=x.device)
    _check(lib().jb_rmsnorm(_p(x), _p(delta), S, int(stride), _p(rows),
                            _p(weight), _DT[weight.dtype], _p(out), _DT[out_dtype], n_out, dm,
                            float(eps), _stream()), "rmsnorm")
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta[0] + ... + delta[S-1] in place (float32)."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    delta = stack(delta)
    _need(delta, "delta", torch.float32, (None, n, dm))
    _check(lib().jb_rmsnorm(_p(x), _p(delta), delta.shape[0], int(n * dm),
                            _p(None), _p(None), 0, _p(None), 0, n, dm, float(0.0),
                            _stream()), "add")
    return x


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """SiLU(gate) * up for a stack [S, n, 2 ff] whose columns are [gate | up]."""
    gate_up = stack(gate_up)
    _need(gate_up, "gate_up", torch.float32, (None, None, None))
    S, n, two_ff = gate_up.shape
    if two_ff % 2:
        raise KernelError("swiglu: the gate_up width must be even")
    ff = two_ff // 2
    out = torch.empty((n, ff), dtype=out_dtype, device=gate_up.device)
    _check(lib().jb_swiglu(_p(gate_up), S, int(n * two_ff), _p(out),
                           _DT[out_dtype], n, ff, _stream()), "swiglu")
    return out


# ------------------------------------------------------------------ position
def rope_table(inv_freq: torch.Tensor, n_pos: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of (float)p * inv_freq[i] for p < n_pos: two [n_pos, half]."""
    _need(inv_freq, "inv_freq", torch.float32)
    half = inv_freq.numel()
    cs = torch.empty((n_pos, half), dtype=torch.float32, device=inv_freq.device)
    sn = torch.empty_like(cs)
    _check(lib().jb_rope_table(_p(cs), _p(sn), _p(inv_freq), n_pos, half, _stream()),
           "rope_table")
    return cs, sn


def qk_norm_rope_append(qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                        row_pos: torch.Tensor, row_seq: torch.Tensor,
                        block_table: torch.Tensor, k_cache: Optional[torch.Tensor],
                        v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                        head_dim: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Per-head RMSNorm of q and k (when weights are given), NeoX rotation by
    the rows' positions (when tables are given), K and V appended to the cache
    pages (when caches are given).  Returns q [n, heads, head_dim].

    qkv: stack [S, n, (heads + 2 kv_heads) head_dim] float32, columns
    [q | k | v].  k_cache, v_cache: [pages, kv_heads, PAGE, head_dim]."""
    qkv = stack(qkv)
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv, "qkv", torch.float32, (None, None, width))
    S, n, _ = qkv.shape
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    w_dt = 0
    if q_weight is not None:
        _need(q_weight, "q_norm weight", _FLOATS, (head_dim,))
        _need(k_weight, "k_norm weight", q_weight.dtype, (head_dim,))
        w_dt = _DT[q_weight.dtype]
    rot_half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32, (None, head_dim // 2))
        _need(sin, "sin", torch.float32, tuple(cos.shape))
        rot_half = head_dim // 2
    if k_cache is not None:
        _need(k_cache, "k_cache", out_dtype, (None, num_kv_heads, PAGE, head_dim))
        _need(v_cache, "v_cache", out_dtype, tuple(k_cache.shape))
    q = torch.empty((n, num_heads, head_dim), dtype=out_dtype, device=qkv.device)
    _check(lib().jb_qk_norm_rope_append(
        _p(qkv), S, int(n * width), _p(q_weight), _p(k_weight), w_dt,
        float(eps), _p(cos), _p(sin), rot_half, _p(row_pos), _p(row_seq),
        _p(block_table), block_table.shape[1], _p(q), _p(k_cache), _p(v_cache), _DT[out_dtype],
        n, num_heads, num_kv_heads, head_dim, _stream()), "qk_norm_rope_append")
    return q


# ----------------------------------------------------------------- attention
def embed_pos(table: torch.Tensor, pos_table: torch.Tensor, tokens: torch.Tensor,
              row_pos: torch.Tensor) -> torch.Tensor:
    """x[j] = table[tokens[j]] + pos_table[row_pos[j]] as float32 [n, dm]."""
    _need(table, "table", _FLOATS, (None, None))
    dm = table.shape[1]
    _need(pos_table, "pos_table", _FLOATS, (None, dm))
    n = tokens.shape[0]
    _need(tokens, "tokens", torch.int32, (n,))
    _need(row_pos, "row_pos", torch.int32, (n,))
    x = torch.empty((n, dm), dtype=torch.float32, device=table.device)
    _check(lib().jb_embed_pos(_p(table), _DT[table.dtype], _p(pos_table), _DT[pos_table.dtype],
                              _p(tokens), _p(row_pos), _p(x), n, dm, _stream()), "embed_pos")
    return x


def dyt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor,
        out_dtype: torch.dtype, delta: Optional[torch.Tensor] = None,
        rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dynamic Tanh: tanh(alpha x) weight + bias on the rows of x (float32 [n, dm]);
    with ``delta`` (a stack of partial sums) x += sum(delta) first, in place; with
    ``rows`` only those rows.  weight, bias [dm] and alpha [] or [1]: float32."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    _need(weight, "weight", torch.float32, (dm,))
    _need(bias, "bias", torch.float32, (dm,))
    _need(alpha, "alpha", torch.float32)
    S, stride = 0, 0
    if delta is not None:
        delta = stack(delta)
        _need(delta, "delta", torch.float32, (None, n, dm))
        S, stride = delta.shape[0], n * dm
    n_out = n
    if rows is not None:
        _need(rows, "rows", torch.int32, (None,))
        n_out = rows.shape[0]
    out = torch.empty((n_out, dm), dtype=out_dtype, device=x.device)
    _check(lib().jb_dyt(_p(x), _p(delta), S, stride, _p(rows), _p(weight), _p(bias), _p(alpha),
                        _p(out), _DT[out_dtype], n_out, dm, _stream()), "dyt")
    return out


def gate_mul(y: torch.Tensor, y_bias: Optional[torch.Tensor], g: torch.Tensor,
             g_bias: Optional[torch.Tensor], g_col0: int = 0) -> torch.Tensor:
    """(sum y + y_bias) * sigmoid(sum g + g_bias) as float32 [n, dm]; y, g: stacks of
    partial sums; g's rows may be wider than dm (the gate starts at column g_col0)."""
    y, g = stack(y), stack(g)
    _need(y, "y", torch.float32, (None, None, None))
    Sy, n, dm = y.shape
    _need(g, "g", torch.float32, (None, n, None))
    out = torch.empty((n, dm), dtype=torch.float32, device=y.device)
    _check(lib().jb_gate_mul(_p(y), Sy, n * dm, _p(y_bias), _p(g), g.shape[0], n * g.shape[2],
                             g.shape[2], g_col0, _p(g_bias), _p(out), n, dm, _stream()), "gate_mul")
    return out


def gated_dyt_residual(x: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor],
                       g: torch.Tensor, g_bias: Optional[torch.Tensor], post, nxt=None,
                       out_dtype: torch.dtype = torch.float32) -> Optional[torch.Tensor]:
    """x += dyt_post(gate_mul(y, g)) in place; with ``nxt`` also returns dyt_nxt(x).
    post, nxt: (weight, bias, alpha) float32 tensors."""
    y, g = stack(y), stack(g)
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    _need(y, "y", torch.float32, (None, n, dm))
    _need(g, "g", torch.float32, (None, n, None))
    out = torch.empty((n, dm), dtype=out_dtype, device=x.device) if nxt is not None else None
    nw, nb, na = nxt if nxt is not None else (None, None, None)
    _check(lib().jb_gated_dyt_residual(_p(x), _p(y), y.shape[0], n * dm, _p(y_bias), _p(g),
                                       g.shape[0], n * g.shape[2], g.shape[2], 0, _p(g_bias),
                                       _p(post[0]), _p(post[1]), _p(post[2]), _p(nw), _p(nb),
                                       _p(na), _p(out), _DT[out_dtype], n, dm,
                                       1 if out_dtype == torch.bfloat16 else 0, _stream()),
           "gated_dyt_residual")
    return out


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float,
             out_dtype: torch.dtype) -> torch.Tensor:
    """c0 n(z) + c1 n(z^2) + c2 n(z^3) + c3 per row, n(u) = u / sqrt(mean(u^2) + eps);
    z: a stack of partial sums [S, n, ff]; coef: float32 [4]."""
    z = stack(z)
    _need(z, "z", torch.float32, (None, None, None))
    S, n, ff = z.shape
    _need(coef, "coef", torch.float32, (4,))
    out = torch.empty((n, ff), dtype=out_dtype, device=z.device)
    _check(lib().jb_polynorm(_p(z), S, n * ff, ff, _p(coef), float(eps), _p(out), _DT[out_dtype],
                             n, ff, _stream()), "polynorm")
    return out


def qkv_bias_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], row_pos: torch.Tensor,
                    row_seq: torch.Tensor, block_table: torch.Tensor,
                    k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                    num_heads: int, head_dim: int, out_dtype: torch.dtype,
                    q_temp_coef: float = 0.0, q_temp_every: int = 0) -> torch.Tensor:
    """The fused [q | k | v] product's sums plus its bias: returns q [n, heads, hd] in
    out_dtype and writes K and V to the cache pages at the rows' positions; with no
    caches the product holds q alone.  With q_temp_every > 0 the queries of a row at
    position p are multiplied by 1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1)."""
    qkv = stack(qkv)
    _need(qkv, "qkv", torch.float32, (None, None, None))
    S, n, width = qkv.shape
    append = k_cache is not None
    nkv = k_cache.shape[1] if append else 0
    vd = v_cache.shape[3] if append else 0
    q = torch.empty((n, num_heads, head_dim), dtype=out_dtype, device=qkv.device)
    _check(lib().jb_qkv_bias_append_temp(_p(qkv), S, n * width, width, _p(bias), _p(row_pos),
                                         _p(row_seq), _p(block_table), block_table.shape[1], _p(q),
                                         _p(k_cache), _p(v_cache), _DT[out_dtype], n, num_heads, nkv,
                                         head_dim, vd, 1 if append else 0, float(q_temp_coef),
                                         int(q_temp_every), _stream()), "qkv_bias_append")
    return q


def layernorm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
              eps: float, out_dtype: torch.dtype, a: Optional[torch.Tensor] = None,
              b: Optional[torch.Tensor] = None, mult: float = 1.0,
              rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Layer norm with weight and bias of the rows of x (float32 [n, dm]).  With ``a``
    (and ``b``), stacks of partial sums [S, n, dm], x += mult * (sum a + sum b) happens
    first, in place.  ``rows``: only those rows (no add then).  ``weight`` None: the add
    alone, nothing is returned."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    sa = sb = None
    if a is not None:
        sa = stack(a)
        _need(sa, "a", torch.float32, (None, n, dm))
    if b is not None:
        sb = stack(b)
        _need(sb, "b", torch.float32, (None, n, dm))
    n_out = n if rows is None else rows.numel()
    out = None
    if weight is not None:
        _need(weight, "weight", torch.float32, (dm,))
        out = torch.empty((n_out, dm), dtype=out_dtype, device=x.device)
    _check(lib().jb_layernorm(_p(x), _p(sa), 0 if sa is None else sa.shape[0], n * dm, _p(sb),
                              0 if sb is None else sb.shape[0], n * dm, float(mult), _p(rows),
                              _p(weight), _p(bias), _p(out), _DT[out_dtype], n_out, dm, float(eps),
                              _stream()), "layernorm")
    return out


ACTIVATIONS = {"relu2": 0, "relu": 1, "gelu_tanh": 2}


def activation(z: torch.Tensor, kind: str, out_dtype: torch.dtype, ff: Optional[int] = None) -> torch.Tensor:
    """act(sum of the partial sums z [S, n, width]) over the first ff columns."""
    z = stack(z)
    _need(z, "z", torch.float32, (None, None, None))
    S, n, width = z.shape
    ff = width if ff is None else ff
    out = torch.empty((n, ff), dtype=out_dtype, device=z.device)
    _check(lib().jb_activation(_p(z), S, n * width, width, ACTIVATIONS[kind], _p(out), _DT[out_dtype],
                               n, ff, _stream()), "activation")
    return out


def attention_kept_chunks(window: int, keep_first: int) -> int:
    """Chunks that the kept first positions of a windowed mixer add to a row's range."""
    return int(lib().jb_attention_kept_chunks(int(window), int(keep_first)))


def norm_residual_(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                   y_bias: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                   skip: Optional[torch.Tensor] = None, skip_coef: Optional[torch.Tensor] = None,
                   rms: bool = False, few_rows: bool = False) -> torch.Tensor:
    """x += norm(sum y + y_bias + skip_coef[:, None] * skip) * weight (+ bias), in place: a
    layer norm (``rms``: an RMS norm) on a sublayer's result alone.  y: [S, n, dm] float32
    partial sums; skip: [n, dm] float32 or bfloat16 with skip_coef float32 [n]."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    y = stack(y)
    _need(y, "y", torch.float32, (None, n, dm))
    _need(weight, "weight", torch.float32, (dm,))
    if skip is not None:
        _need(skip, "skip", _FLOATS, (n, dm))
        _need(skip_coef, "skip_coef", torch.float32, (n,))
    _check(lib().jb_norm_residual(_p(x), _p(y), y.shape[0], n * dm, _p(y_bias), _p(skip),
                                  0 if skip is None else _DT[skip.dtype], _p(skip_coef), 1, _p(weight),
                                  _p(bias), n, dm, float(eps), 1 if rms else 0, 1 if few_rows else 0,
                                  _stream()), "norm_residual")
    return x


def short_conv(x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], row_pos: torch.Tensor,
               row_seq: torch.Tensor, seq_slot: torch.Tensor, out_dtype: torch.dtype,
               write_h: bool = True, write_state: bool = True) -> Optional[torch.Tensor]:
    """h = x + a causal convolution over time on every channel.  x: float32 [n, dm]; w: float32
    [dm, taps]; state: float32 [slots, taps - 1, dm] (None with one tap), the last inputs of
    every slot's sequence, read for positions before the step's rows and written for the
    step's last ones.  Both in one call only where every sequence starts at position 0 or
    brings one row."""
    _need(x, "x", torch.float32, (None, None))
    n, dm = x.shape
    _need(w, "w", torch.float32, (dm, None))
    taps = w.shape[1]
    if taps > 1:
        _need(state, "state", torch.float32, (None, taps - 1, dm))
    out = torch.empty((n, dm), dtype=out_dtype, device=x.device) if write_h else None
    what = (1 if write_h else 0) | (2 if write_state and taps > 1 else 0)
    _check(lib().jb_short_conv(_p(x), _p(w), _p(state), (taps - 1) * dm, _p(row_pos), _p(row_seq),
                               _p(seq_slot), _p(out), _DT[out_dtype], n, dm, taps, what, _stream()),
           "short_conv")
    return out


def mingru(P: torch.Tensor, width: int, bias: Optional[torch.Tensor], state: torch.Tensor,
           row_seq: torch.Tensor, seq_slot: torch.Tensor, out_dtype: torch.dtype,
           every_row_starts: bool = False, col0: int = 0) -> torch.Tensor:
    """The minGRU's recurrence over the rows from the sums P [S, n, ld] of [z | x | g] (from
    column col0 on, ``width`` each; bias float32 [3 width] or None): S * silu(g) as
    [n, width].  state: float32 [slots, width], read and left updated."""
    P = stack(P)
    _need(P, "P", torch.float32, (None, None, None))
    S, n, ld = P.shape
    _need(state, "state", torch.float32, (None, width))
    if bias is not None:
        _need(bias, "bias", torch.float32, (3 * width,))
    n_seqs = seq_slot.numel()
    L = lib()
    need = int(L.jb_mingru_scratch(n, n_seqs, width, 1 if every_row_starts else 0))
    scratch = _scratch(P.device, need) if need > 0 else None
    out = torch.empty((n, width), dtype=out_dtype, device=P.device)
    _check(L.jb_mingru(_p(P), S, n * ld, ld, col0, _p(bias), _p(state), _p(row_seq), _p(seq_slot),
                       _p(scratch), _p(out), _DT[out_dtype], n, n_seqs, width,
                       1 if every_row_starts else 0, _stream()), "mingru", 3 if need > 0 else 1)
    return out


def moe_route(P: torch.Tensor, col0: int, outputs: int, correction: Optional[torch.Tensor], groups: int,
              keep: int, top: int, first_identity: int, scale: float, sigmoid_scores: bool = False,
              group_best: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """The router of a routed feed-forward over the logits in columns col0 .. col0 + outputs - 1
    of the sums P [S, n, ld]: (weights [n, outputs], 0 for outputs not chosen; the summed
    weight of the chosen outputs from first_identity on, [n]).  sigmoid_scores: each score is
    the sigmoid of its logit instead of a softmax over all; group_best: a group's score is the
    sum of that many of its largest choice scores."""
    P = stack(P)
    _need(P, "P", torch.float32, (None, None, None))
    S, n, ld = P.shape
    if correction is not None:
        _need(correction, "correction", torch.float32, (outputs,))
    weights = torch.empty((n, outputs), dtype=torch.float32, device=P.device)
    skip = torch.empty((n,), dtype=torch.float32, device=P.device)
    _check(lib().jb_moe_route(_p(P), S, n * ld, ld, col0, _p(correction), _p(weights), _p(skip), n, outputs,
                              groups, keep, top, first_identity, float(scale), 1 if sigmoid_scores else 0,
                              group_best, _stream()), "moe_route")
    return weights, skip


def gated_weighted(z: torch.Tensor, weights: torch.Tensor, n_experts: int, ff: int, kind: str,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """act(gate) * up * weights[row, expert] for experts whose sums lie [gate (ff) | up (ff)] one
    after the other in z [S, n, ld]: [n, n_experts * ff]."""
    z = stack(z)
    _need(z, "z", torch.float32, (None, None, None))
    S, n, ld = z.shape
    _need(weights, "weights", torch.float32, (n, None))
    out = torch.empty((n, n_experts * ff), dtype=out_dtype, device=z.device)
    kinds = {"relu2": 0, "relu": 1, "gelu_tanh": 2, "silu": 3}
    _check(lib().jb_gated_weighted(_p(z), S, n * ld, ld, _p(weights), weights.shape[1], n_experts, ff,
                                   kinds[kind], _p(out), _DT[out_dtype], n, _stream()), "gated_weighted")
    return out


def causal_conv(u: torch.Tensor, col0: int, C: int, w: torch.Tensor, bias: Optional[torch.Tensor],
                state: Optional[torch.Tensor], row_pos: torch.Tensor, row_seq: torch.Tensor,
                seq_slot: torch.Tensor, silu: bool, out_dtype: torch.dtype, write_out: bool = True,
                write_state: bool = True, slot_stride: Optional[int] = None) -> Optional[torch.Tensor]:
    """A causal convolution over time on columns col0 .. col0 + C - 1 of the sums u [S, n, ld],
    without the input added: act(bias + sum_j w[:, j] u_{t - taps + 1 + j}); w float32 [C, taps];
    state: float32, per slot a ring [taps - 1, C] of the last inputs (slot_stride floats apart)."""
    u = stack(u)
    _need(u, "u", torch.float32, (None, None, None))
    S, n, ld = u.shape
    _need(w, "w", torch.float32, (C, None))
    taps = w.shape[1]
    out = torch.empty((n, C), dtype=out_dtype, device=u.device) if write_out else None
    what = (1 if write_out else 0) | (2 if write_state and taps > 1 else 0)
    stride = slot_stride if slot_stride is not None else (taps - 1) * C
    _check(lib().jb_causal_conv(_p(u), S, n * ld, ld, col0, _p(w), _p(bias), _p(state), stride, _p(row_pos),
                                _p(row_seq), _p(seq_slot), _p(out), _DT[out_dtype], C, n, C, taps,
                                1 if silu else 0, what, _stream()), "causal_conv")
    return out


def matrix_state_scan(src: torch.Tensor, H: int, G: int, N: int, P: int, val_col0: int, key_col0: int,
                      qry_col0: int, state: torch.Tensor, row_seq: torch.Tensor, seq_slot: torch.Tensor,
                      n_seqs: int, every_row_starts: bool = False, silu: bool = False,
                      dt: Optional[torch.Tensor] = None, dt_col0: int = 0,
                      dt_bias: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None,
                      skip: Optional[torch.Tensor] = None, decay: Optional[torch.Tensor] = None,
                      slot_stride: Optional[int] = None, max_len: int = 0) -> torch.Tensor:
    """S_t = a_t S_{t-1} + b_t k_t v_t^T, y_t = S_t^T q_t + d v_t per head over the rows of each
    sequence; src [S, n, ld] holds v (H P columns), k and q (G N columns each).  With dt (sums
    with H columns from dt_col0): a = exp(-exp(a_log) softplus(dt + dt_bias)), b = the softplus,
    d = skip; otherwise a = decay, b = 1, d = 0.  state: float32 [slots, H, N, P].  y: [n, H P].
    max_len: the most rows one sequence brings; from twice ``jb_matrix_state_piece()`` rows on the
    sequences are cut into pieces that run side by side."""
    src = stack(src)
    _need(src, "src", torch.float32, (None, None, None))
    S, n, ld = src.shape
    dS = dn = dld = 0
    if dt is not None:
        dt = stack(dt)
        _need(dt, "dt", torch.float32, (None, n, None))
        dS, dn, dld = dt.shape
    y = torch.empty((n, H * P), dtype=torch.float32, device=src.device)
    stride = slot_stride if slot_stride is not None else H * N * P
    need = 0 if every_row_starts else lib().jb_matrix_state_scratch(n_seqs, max_len, H, N, P)
    scratch = torch.empty((need,), dtype=torch.float32, device=src.device) if need > 0 else None
    _check(lib().jb_matrix_state_scan(_p(src), S, n * ld, ld, val_col0, key_col0, qry_col0, 1 if silu else 0,
                                      _p(dt), dS, dn * dld, dld, dt_col0, _p(dt_bias), _p(a_log), _p(skip),
                                      _p(decay), _p(state), stride, _p(row_seq), _p(seq_slot), _p(y), n, n_seqs,
                                      H, G, N, P, 1 if every_row_starts else 0, _p(scratch), max_len, _stream()),
           "matrix_state_scan", 3 if need > 0 else 1)
    return y


def gated_part_norm(y: torch.Tensor, parts: int, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
                    pre: Optional[torch.Tensor] = None, pre_col0: int = 0,
                    post: Optional[torch.Tensor] = None, post_col0: int = 0, few_rows: bool = False) -> torch.Tensor:
    """rms(y * silu(pre)) in ``parts`` equal parts of each row, times w, times sigmoid(post)."""
    _need(y, "y", torch.float32, (None, None))
    n, width = y.shape
    _need(w, "w", torch.float32, (width,))
    pre = None if pre is None else stack(pre)
    post = None if post is None else stack(post)
    out = torch.empty((n, width), dtype=out_dtype, device=y.device)
    a = (0, 0, 0) if pre is None else (pre.shape[0], n * pre.shape[2], pre.shape[2])
    b = (0, 0, 0) if post is None else (post.shape[0], n * post.shape[2], post.shape[2])
    _check(lib().jb_gated_part_norm(_p(y), _p(pre), a[0], a[1], a[2], pre_col0, _p(post), b[0], b[1], b[2],
                                    post_col0, _p(w), float(eps), _p(out), _DT[out_dtype], n, width, parts,
                                    1 if few_rows else 0, _stream()), "gated_part_norm")
    return out


def pair_combine(L: torch.Tensor, R: torch.Tensor, wl: Optional[torch.Tensor], wr: Optional[torch.Tensor],
                 sl: float, sr: float, eps: float, few_rows: bool = False) -> torch.Tensor:
    """sl * sum(L) + sr * sum(R), or with weights sl * rms(sum L) wl + sr * rms(sum R) wr."""
    L, R = stack(L), stack(R)
    _need(L, "L", torch.float32, (None, None, None))
    _need(R, "R", torch.float32, (None, L.shape[1], L.shape[2]))
    n, m = L.shape[1], L.shape[2]
    out = torch.empty((n, m), dtype=torch.float32, device=L.device)
    _check(lib().jb_pair_combine(_p(L), L.shape[0], n * m, _p(R), R.shape[0], n * m, _p(wl), _p(wr), float(sl),
                                 float(sr), float(eps), _p(out), n, m, 1 if few_rows else 0, _stream()),
           "pair_combine")
    return out


def token_gate(P: torch.Tensor, table: torch.Tensor, col0: int, dim: int, tokens: torch.Tensor,
               out_dtype: torch.dtype) -> torch.Tensor:
    """gelu_tanh(sum P) * table[tokens[row], col0 .. col0 + dim - 1] as [n, dim]."""
    P = stack(P)
    _need(P, "P", torch.float32, (None, None, None))
    S, n, ld = P.shape
    _need(table, "table", _FLOATS, (None, None))
    out = torch.empty((n, dim), dtype=out_dtype, device=P.device)
    _check(lib().jb_token_gate(_p(P), S, n * ld, ld, _p(table), _DT[table.dtype], table.shape[1], col0,
                               _p(tokens), _p(out), _DT[out_dtype], n, dim, _stream()), "token_gate")
    return out


def activation_weighted(z: torch.Tensor, width: int, weights: torch.Tensor, n_experts: int, ff: int,
                        kind: str, out_dtype: torch.dtype) -> torch.Tensor:
    """act(sum z) * weights[row, column // ff] over the first n_experts * ff columns of z
    [S, n, ld], act alone over the rest up to ``width``."""
    z = stack(z)
    _need(z, "z", torch.float32, (None, None, None))
    S, n, ld = z.shape
    _need(weights, "weights", torch.float32, (n, None))
    out = torch.empty((n, width), dtype=out_dtype, device=z.device)
    _check(lib().jb_activation_weighted(_p(z), S, n * ld, ld, _p(weights), weights.shape[1], n_experts, ff,
                                        ACTIVATIONS[kind], _p(out), _DT[out_dtype], n, width, _stream()),
           "activation_weighted")
    return out


def qkv_prepare_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                       k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                       sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_seq: torch.Tensor,
                       block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       num_heads: int, pairs: bool = False, unit_norm: bool = False) -> torch.Tensor:
    """pairs: the rotation turns neighbours (2i, 2i + 1); unit_norm: q and k heads are divided by
    their root mean square after the rotation.
    q, k, v out of the sums of one product [S, n, ld] = [q | k | v | ...]: the bias, an RMS
    norm per head on q and k (weights float32 [hd] or None), a rotation of the first
    2 * cos.shape[1] values of each head (value i with value i + cos.shape[1]), K and V
    into the cache pages at the rows' positions.  Returns q [n, heads, hd] in the cache's type."""
    qkv = stack(qkv)
    _need(qkv, "qkv", torch.float32, (None, None, None))
    S, n, ld = qkv.shape
    _need(k_cache, "k_cache", _FLOATS, (None, None, PAGE, None))
    nkv, hd = k_cache.shape[1], k_cache.shape[3]
    _need(v_cache, "v_cache", k_cache.dtype, (k_cache.shape[0], nkv, PAGE, None))
    vd = v_cache.shape[3]
    rot_half = 0 if cos is None else cos.shape[1]
    if cos is not None:
        _need(cos, "cos", torch.float32, (None, rot_half))
        _need(sin, "sin", torch.float32, (cos.shape[0], rot_half))
    q = torch.empty((n, num_heads, hd), dtype=k_cache.dtype, device=qkv.device)
    _check(lib().jb_qkv_prepare_append(_p(qkv), S, n * ld, ld, _p(bias), _p(q_weight), _p(k_weight),
                                       float(eps), _p(cos), _p(sin), rot_half, _p(row_pos), _p(row_seq),
                                       _p(block_table), block_table.shape[1], _p(q), _p(k_cache),
                                       _p(v_cache), _DT[k_cache.dtype], n, num_heads, nkv, hd, vd,
                                       (1 if pairs else 0) | (2 if unit_norm else 0), _stream()),
           "qkv_prepare_append")
    return q


def latent_down(P: torch.Tensor, q_rank: int, wq: Optional[torch.Tensor], kv_rank: int,
                wkv: torch.Tensor, rot_dim: int, cos: Optional[torch.Tensor],
                sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_seq: torch.Tensor,
                block_table: torch.Tensor, k_cache: torch.Tensor, eps: float) -> torch.Tensor:
    """P: sums [S, n, >= q_rank + kv_rank + rot_dim], columns [query latent | latent |
    shared key part].  Returns the RMS-normed query latent [n, q_rank] in the cache's
    dtype and writes [RMS-normed latent | rotated key part] to the cache rows
    (k_cache [pages, 1, PAGE, kv_rank + rot_dim]) at the rows' positions."""
    P = stack(P)
    _need(P, "P", torch.float32, (None, None, None))
    S, n, ld = P.shape
    _need(k_cache, "k_cache", _FLOATS, (None, 1, PAGE, kv_rank + rot_dim))
    rot_half = 0 if cos is None else cos.shape[1]
    cq = torch.empty((n, q_rank), dtype=k_cache.dtype, device=P.device)
    _check(lib().jb_latent_down(_p(P), S, n * ld, ld, 0, q_rank, _p(wq), q_rank, kv_rank, _p(wkv),
                                rot_dim, _p(cos), _p(sin), rot_half, _p(row_pos), _p(row_seq),
                                _p(block_table), block_table.shape[1], _p(cq), _p(k_cache),
                                _DT[k_cache.dtype], n, float(eps), _stream()), "latent_down")
    return cq


def latent_queries(Q: torch.Tensor, w_ukT: torch.Tensor, num_heads: int, D: int, R: int, C: int,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], row_pos: torch.Tensor,
                   dtype: torch.dtype) -> torch.Tensor:
    """Q: the query product's sums [S, n, heads (D + R)]; w_ukT [heads C, D]: per head
    the key matrix, transposed.  Returns the latent queries [n, heads, C + R]: per head
    [Wuk_head^T q_plain | rotated q_rot]."""
    Q = stack(Q)
    _need(Q, "Q", torch.float32, (None, None, num_heads * (D + R)))
    S, n, _ = Q.shape
    rot_half = 0 if cos is None else cos.shape[1]
    q_plain = torch.empty((num_heads, n, D), dtype=dtype, device=Q.device)
    q_lat = torch.empty((n, num_heads, C + R), dtype=dtype, device=Q.device)
    L = lib()
    _check(L.jb_latent_q_split(_p(Q), S, Q.shape[1] * Q.shape[2], num_heads, D, R, C, _p(cos), _p(sin),
                               rot_half, _p(row_pos), _p(q_plain), _p(q_lat), _DT[dtype], n, _stream()),
           "latent_q_split")
    A = torch.stack([stack(linear(q_plain[h], w_ukT[h * C:(h + 1) * C], force_simt=True))
                     for h in range(num_heads)])
    _check(L.jb_latent_q_join(_p(A.contiguous()), A.shape[1], num_heads, C, R, _p(q_lat), _DT[dtype], n,
                              _stream()), "latent_q_join")
    return q_lat


def heads_gate(A: torch.Tensor, g: Optional[torch.Tensor], g_col0: int,
               out_dtype: torch.dtype) -> torch.Tensor:
    """A: per-head sums [heads, S, n, Dv]; g: a gate's sums [Sg, n, width] whose columns
    g_col0.. are the gate (or None).  Returns [n, heads Dv] = concat(sum A) * sigmoid(sum g)."""
    _need(A, "A", torch.float32, (None, None, None, None))
    H, S, n, Dv = A.shape
    sg = None
    if g is not None:
        sg = stack(g)
        _need(sg, "g", torch.float32, (None, n, None))
    out = torch.empty((n, H * Dv), dtype=out_dtype, device=A.device)
    _check(lib().jb_heads_gate(_p(A), S, H, Dv, _p(sg), 0 if sg is None else sg.shape[0],
                               0 if sg is None else n * sg.shape[2], 0 if sg is None else sg.shape[2],
                               g_col0, _p(out), _DT[out_dtype], n, _stream()), "heads_gate")
    return out


def transpose_heads(w: torch.Tensor, num_heads: int) -> torch.Tensor:
    """w [heads D, C] -> [heads C, D]: every head's block transposed."""
    _need(w, "w", _FLOATS, (None, None))
    D, C = w.shape[0] // num_heads, w.shape[1]
    out = torch.empty((num_heads * C, D), dtype=w.dtype, device=w.device)
    _check(lib().jb_transpose_heads(_p(w), _p(out), _DT[w.dtype], num_heads, D, C, _stream()),
           "transpose_heads")
    return out


def attention_chunk() -> int:
    return int(lib().jb_attention_chunk())


_ATT_SCRATCH_BYTES = 256 << 20
_att_scratch: dict = {}


def _scratch(device: torch.device, floats: int) -> torch.Tensor:
    buf = _att_scratch.get(device)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        _att_scratch[device] = buf
    return buf


def attention_block_positions(num_heads: int, num_kv_heads: int) -> int:
    """Positions of one sequence that a block of the tensor-core prefill kernel holds."""
    return int(lib().jb_attn_tc_block_positions(num_heads, num_kv_heads))


def attention_blocks(seq_row0, seq_pos0, seq_len, positions_per_block: int,
                     device: torch.device) -> torch.Tensor:
    """The blocks a prefill step is cut into for the tensor-core kernel: int32
    [blocks, 4] = first row, positions, the first row's position, sequence."""
    import numpy as np
    rows = []
    for i, (r0, p0, n) in enumerate(zip(seq_row0, seq_pos0, seq_len)):
        for a in range(0, int(n), positions_per_block):
            rows.append((int(r0) + a, min(positions_per_block, int(n) - a), int(p0) + a, i))
    # the runs that end latest see the most keys and take longest: they start first
    rows.sort(key=lambda b: -(b[2] + b[1]))
    return torch.from_numpy(np.asarray(rows, dtype=np.int32).reshape(-1, 4)).to(device)


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              row_pos: torch.Tensor, row_seq: torch.Tensor, block_table: torch.Tensor,
              window: int, scale: float, max_chunks: int, blocks: Optional[torch.Tensor] = None,
              decode: bool = False, force_simt: bool = False,
              head_scale: Optional[torch.Tensor] = None,
              sink: Optional[torch.Tensor] = None, softcap: float = 0.0,
              slopes: Optional[torch.Tensor] = None, value_dim: int = 0,
              head_major: bool = False, keep_first: int = 0,
              score_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal GQA attention of every row over its sequence's cache pages.

    ``keep_first`` > 0 (with a window): positions below it stay visible to every later
    row beside the window; ``max_chunks`` then counts their chunks too
    (``attention_kept_chunks``).  ``score_bias`` (float32 [heads]): the weight of a visible
    key is sigmoid(score + score_bias[head]), not normalized over the keys (no softmax).

    ``softcap`` > 0: a score s becomes softcap * tanh(s / softcap); ``slopes`` (float32
    [heads]): slopes[h] * (the row's position - the key's) is taken off the score, after
    the cap.  ``value_dim`` > 0 with ``v_cache is None``: the values are the first
    value_dim entries of the keys' rows.  ``head_major``: the result is [heads, n, vd].

    q: [n, heads, hd]; caches [pages, kv_heads, PAGE, hd] of q's dtype.  Row r
    is at position row_pos[r] of sequence row_seq[r], whose pages are
    block_table[row_seq[r]]; it sees positions max(0, pos + 1 - window) .. pos
    (all of 0 .. pos when window is 0).  max_chunks: the most chunks of
    ``attention_chunk()`` positions that any row's range touches.

    bfloat16 heads of 64 or 128 values run on the tensor cores when the caller
    says how the rows are arranged: ``decode=True`` (every row is the one new
    token of its sequence) or ``blocks`` (from ``attention_blocks``: runs of
    consecutive positions of one sequence).  Everything else, and float32, runs on
    the plain kernel.

    The values may have a head size of their own (v_cache [pages, kv_heads, PAGE,
    vd]; the result is then [n, heads, vd]).  ``head_scale`` (float32 [heads]) is a
    factor per head on the scores; ``sink`` (float32 [heads]) adds exp(sink) once to
    each softmax's denominator, with no value."""
    _need(q, "q", _FLOATS, (None, None, None))
    n, nh, hd = q.shape
    _need(k_cache, "k_cache", q.dtype, (None, None, PAGE, hd))
    nkv = k_cache.shape[1]
    v_ld = 0
    if v_cache is None:
        if not 0 < value_dim <= hd:
            raise KernelError("attention: values inside the keys' rows need 0 < value_dim <= head size")
        v_cache, vd, v_ld = k_cache, value_dim, hd
    else:
        _need(v_cache, "v_cache", q.dtype, (k_cache.shape[0], nkv, PAGE, None))
        vd = v_cache.shape[3]
    if slopes is not None:
        _need(slopes, "slopes", torch.float32, (nh,))
    if head_scale is not None:
        _need(head_scale, "head_scale", torch.float32, (nh,))
    if sink is not None:
        _need(sink, "sink", torch.float32, (nh,))
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    out = torch.empty((nh, n, vd) if head_major else (n, nh, vd), dtype=q.dtype, device=q.device)
    L = lib()
    if score_bias is not None:
        _need(score_bias, "score_bias", torch.float32, (nh,))
    tc = (not force_simt and vd == hd and q.dtype == torch.bfloat16
          and v_ld == 0 and not head_major
          and (decode or blocks is not None) and bool(L.jb_attn_tc_ok(nh, nkv, hd))
          and (decode or head_scale is None or bool((head_scale > 0).all())))
    # kept first tokens and sigmoid weights: the prefill kernel has them for all its sizes, of
    # the decode kernels the one that runs over several chunks
    if tc and (keep_first or score_bias is not None):
        if decode and not L.jb_attn_tc_decode_runs(nh, nkv, hd):
            tc = False
        if score_bias is not None and (head_scale is not None or sink is not None or softcap
                                       or slopes is not None):
            tc = False
    if tc and not decode:
        _need(blocks, "blocks", torch.int32, (None, 4))
        _check(L.jb_attn_tc_prefill_gen(_p(q), _p(k_cache), _p(v_cache),
                                        int(k_cache.shape[0]), _p(blocks),
                                        blocks.shape[0], _p(block_table), block_table.shape[1],
                                        _p(out), n, nh, nkv, hd, window, float(scale),
                                        _p(head_scale), _p(sink), float(softcap), _p(slopes),
                                        int(keep_first), _p(score_bias), _stream()),
               "attention (tcgen05, prefill)")
        return out
    kc = int(L.jb_attention_kept_chunks(window, int(keep_first)))
    if tc:
        # CTAs per (token, KV head): each runs over per_cta chunks and leaves one partial;
        # the kept first tokens' chunks are a CTA and a partial each, before the others
        win = max(max_chunks - kc, 1)
        if L.jb_attn_tc_decode_runs(nh, nkv, hd):
            parts = _decode_parts(min(n, 4096) * nkv, win, 2 * _sm_count(q.device))
        else:
            parts = win
        per_cta = (win + parts - 1) // parts
        parts = kc + (win + per_cta - 1) // per_cta
    else:
        parts, per_cta = max_chunks, 1
    per_row = int(L.jb_attention_scratch(1, nh, vd, parts))
    rows_per_call = max(1, min(n, (_ATT_SCRATCH_BYTES // 4) // max(per_row, 1)))
    scratch = _scratch(q.device, per_row * rows_per_call)
    for row0 in range(0, n, rows_per_call):
        cnt = min(rows_per_call, n - row0)
        if tc:
            _check(L.jb_attn_tc_decode_gen(_p(q), _p(k_cache), _p(v_cache),
                                           int(k_cache.shape[0]), _p(row_pos),
                                           _p(row_seq), _p(block_table), block_table.shape[1],
                                           _p(scratch), n, row0, cnt, nh, nkv, hd, window,
                                           float(scale), _p(head_scale), float(softcap),
                                           _p(slopes), int(keep_first), _p(score_bias),
                                           max(max_chunks, kc + 1), per_cta, _stream()),
                   "attention (tcgen05, decode)")
            _check(L.jb_attention_merge_gen(_p(scratch), _p(row_pos), _p(out), _DT[q.dtype], row0,
                                            cnt, nh, hd, window, parts, per_cta, _p(sink),
                                            int(keep_first), 1 if score_bias is not None else 0,
                                            _stream()), "attention merge")
        else:
            _check(L.jb_attention_gen(_p(q), _p(k_cache), _p(v_cache), _DT[q.dtype], _p(row_pos),
                                      _p(row_seq), _p(block_table), block_table.shape[1],
                                      _p(scratch), _p(out), row0, cnt, nh, nkv, hd, vd, window,
                                      float(scale), _p(head_scale), _p(sink), max_chunks, v_ld,
                                      float(softcap), _p(slopes), n if head_major else 0,
                                      int(keep_first), _p(score_bias), _stream()), "attention", kernels=2)
    return out


def attention_decode_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor],
                         k_weight: Optional[torch.Tensor], eps: float,
                         cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                         k_cache: torch.Tensor, v_cache: torch.Tensor, append: bool,
                         row_pos: torch.Tensor, row_seq: torch.Tensor, block_table: torch.Tensor,
                         window: int, scale: float, max_chunks: int,
                         num_heads: int) -> Optional[torch.Tensor]:
    """``qk_norm_rope_append`` and ``attention(decode=True)`` in one kernel: the
    attention's CTAs make q, and the one that holds the new position's chunk makes
    that position's key and value and writes them to the cache (``append``), from
    the q,k,v product's partial sums ``qkv`` [S, n, (heads + 2 kv_heads) 128].
    Returns the attention's output [n, heads, 128] in bfloat16, or None where the
    kernel does not take these sizes and types (bfloat16 caches, heads of 128
    values in groups of at most 16): the caller then goes the two-kernel way."""
    L = lib()
    if k_cache.dtype != torch.bfloat16 or k_cache.dim() != 4:
        return None
    nkv, hd = k_cache.shape[1], k_cache.shape[3]
    if not L.jb_attn_tc_decode_runs(num_heads, nkv, hd):
        return None
    qkv = stack(qkv)
    width = (num_heads + 2 * nkv) * hd
    _need(qkv, "qkv", torch.float32, (None, None, width))
    S, n, _ = qkv.shape
    _need(k_cache, "k_cache", torch.bfloat16, (None, nkv, PAGE, hd))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(row_pos, "row_pos", torch.int32, (n,))
    _need(row_seq, "row_seq", torch.int32, (n,))
    _need(block_table, "block_table", torch.int32, (None, None))
    w_dt = 0
    if q_weight is not None:
        _need(q_weight, "q_norm weight", _FLOATS, (hd,))
        _need(k_weight, "k_norm weight", q_weight.dtype, (hd,))
        w_dt = _DT[q_weight.dtype]
    if cos is not None:
        _need(cos, "cos", torch.float32, (None, hd // 2))
        _need(sin, "sin", torch.float32, tuple(cos.shape))
    parts = _decode_parts(min(n, 4096) * nkv, max_chunks, 2 * _sm_count(qkv.device))
    per_cta = (max_chunks + parts - 1) // parts
    parts = (max_chunks + per_cta - 1) // per_cta
    per_row = int(L.jb_attention_scratch(1, num_heads, hd, parts))
    rows_per_call = max(1, min(n, (_ATT_SCRATCH_BYTES // 4) // max(per_row, 1)))
    scratch = _scratch(qkv.device, per_row * rows_per_call)
    out = torch.empty((n, num_heads, hd), dtype=torch.bfloat16, device=qkv.device)
    for row0 in range(0, n, rows_per_call):
        cnt = min(rows_per_call, n - row0)
        code = L.jb_attn_tc_decode_qkv(
            _p(qkv), S, int(n * width), _p(q_weight), _p(k_weight), w_dt,
            float(eps), _p(cos), _p(sin), _p(k_cache), _p(v_cache), int(bool(append)),
            int(k_cache.shape[0]), _p(row_pos), _p(row_seq), _p(block_table),
            block_table.shape[1], _p(scratch), n, row0, cnt, num_heads, nkv, hd, window,
            float(scale), max_chunks, per_cta, _stream())
        if code == -1 and row0 == 0:
            return None             # an address the kernel's 16-byte loads cannot take
        _check(code, "attention (tcgen05, decode, from the product's sums)")
        _check(L.jb_attention_merge(_p(scratch), _p(row_pos), _p(out), _DT[out.dtype], row0, cnt,
                                    num_heads, hd, window, parts, per_cta, _stream()),
               "attention merge")
    return out


_SM_COUNT = {}


def _sm_count(device: torch.device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def _decode_parts(pairs: int, chunks: int, places: int) -> int:
    """Into how many CTAs the chunks of one (token, KV head) pair are cut.  A CTA
    costs about three chunks' time to set up, and CTAs beyond the device's places
    (two per SM) come in waves: the cut that finishes first by that estimate."""
    sms = places
    best, best_t = 1, None
    for parts in range(1, chunks + 1):
        per_cta = -(-chunks // parts)
        waves = -(-(pairs * -(-chunks // per_cta)) // sms)
        t = waves * (3.0 + per_cta)
        if best_t is None or t < best_t:
            best, best_t = parts, t
    return best


def attn_tc_error() -> int:
    """0, or which bounded wait of a tensor-core attention kernel ran out since
    the last call.  Synchronizes the device."""
    return int(lib().jb_attn_tc_error())


# ------------------------------------------------------------------ products
def _tensor_core_ok(a: torch.Tensor, weight: torch.Tensor) -> bool:
    """What jb_gemm_tc_ok asks (bfloat16 rows of a multiple of 8 values, 16-byte
    aligned bases), asked here: it is on the path of every product."""
    if a.dtype is not torch.bfloat16 or weight.dtype is not torch.bfloat16:
        return False
    k = a.shape[1]
    return (a.shape[0] > 0 and weight.shape[0] > 0 and k >= 8 and k % 8 == 0
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


_SPLITS: dict = {}


def _splits(n: int, m: int, k: int, device=None) -> int:
    """jb_gemm_tc_splits, remembered per shape and device (it depends on nothing
    else but the device's SM count)."""
    key = (n, m, k, device)
    s = _SPLITS.get(key)
    if s is None:
        if len(_SPLITS) > 4096:
            _SPLITS.clear()
        s = _SPLITS[key] = int(lib().jb_gemm_tc_splits(n, m, k))
    return s


def linear(a: torch.Tensor, weight: torch.Tensor, force_simt: bool = False,
           whole: bool = False, splits: Optional[int] = None) -> torch.Tensor:
    """a [n, k] . weight[m, k]^T as a stack [S, n, m] of float32 partial sums.

    bfloat16 operands whose rows are a multiple of 8 long go to the tensor-core
    kernel (which may cut k into S parts); everything else (float32 on either
    side, other row lengths) goes to the plain multiply-add kernel, S = 1.
    ``whole=True`` asks for S = 1 in every case (the result itself, not parts).

    The tensor-core kernel starts fetching ``weight`` before the kernel launched
    just before it has finished; weights must therefore not be the output of that
    kernel (model weights never are)."""
    _need(a, "activations", _FLOATS, (None, None))
    _need(weight, "weight", _FLOATS, (None, a.shape[1]))
    n, k = a.shape
    m = weight.shape[0]
    L = lib()
    if not force_simt and n > 0 and _tensor_core_ok(a, weight):
        S = 1 if whole else int(splits or _splits(n, m, k, a.device.index))
        out = torch.empty((S, n, m), dtype=torch.float32, device=a.device)
        _check(L.jb_gemm_tc(_p(a), _p(weight), _p(out), n, m, k, S, _stream()), "linear (tcgen05)")
        return out
    out = torch.empty((1, n, m), dtype=torch.float32, device=a.device)
    need = int(L.jb_gemm_simt_scratch(n, m, k))
    scratch = torch.empty((need,), dtype=torch.float32, device=a.device) if need else None
    _check(L.jb_gemm_simt(_p(a), _DT[a.dtype], _p(weight), _DT[weight.dtype], _p(out), n, m,
                          k, _p(scratch), _stream()), "linear", kernels=2 if need else 1)
    return out


def linear_heads(a: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """One product per head in one launch of the tensor-core kernel: a [H, n, k] . weight
    [H m, k]^T, head h with rows h m .. of the weight.  Returns float32 [H, S, n, m].
    bfloat16 operands whose rows are a multiple of 8 long only."""
    _need(a, "activations", torch.bfloat16, (None, None, None))
    H, n, k = a.shape
    _need(weight, "weight", torch.bfloat16, (None, k))
    if weight.shape[0] % H or k % 8:
        raise KernelError("linear_heads: the weight's rows are no multiple of the heads, or k of 8")
    m = weight.shape[0] // H
    S = _splits(n, m, k, a.device.index)
    out = torch.empty((H, S, n, m), dtype=torch.float32, device=a.device)
    _check(lib().jb_gemm_tc_heads(_p(a), _p(weight), _p(out), n, m, k, S, H, _stream()),
           "linear_heads (tcgen05)")
    return out


def linear_swiglu(a: torch.Tensor, gate_up: torch.Tensor) -> Optional[torch.Tensor]:
    """SiLU(a . gate^T) * (a . up^T) in one tensor-core kernel, for bfloat16
    a [n, k] and gate_up [2 ff, k] (rows [gate | up]); returns bfloat16 [n, ff],
    or None when the kernel does not take the operands."""
    _need(a, "activations", _FLOATS, (None, None))
    _need(gate_up, "gate_up weight", _FLOATS, (None, a.shape[1]))
    if gate_up.shape[0] % 2 or a.shape[0] == 0 or not _tensor_core_ok(a, gate_up):
        return None
    n, k = a.shape
    ff = gate_up.shape[0] // 2
    out = torch.empty((n, ff), dtype=torch.bfloat16, device=a.device)
    _check(lib().jb_gemm_tc_swiglu(_p(a), _p(gate_up), _p(out), n, ff, k, _stream()),
           "linear_swiglu (tcgen05)")
    return out


def linear_parts(n: int, m: int, k: int) -> int:
    """Into how many parts of k the tensor-core product of n rows with a weight
    [m, k] is cut when the caller leaves it open (see ``linear``)."""
    return _splits(n, m, k)


def gemm_tc_error() -> int:
    """0, or which bounded wait of a tensor-core product ran out since the last
    call (the product's output is then not valid).  Synchronizes the device."""
    return int(lib().jb_gemm_tc_error())


# ------------------------------------------------------------------ sampling
def sample(logits: torch.Tensor, out: Optional[torch.Tensor] = None,
           row_slot: Optional[torch.Tensor] = None,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
           rng: Optional[torch.Tensor] = None, big_keys: Optional[torch.Tensor] = None,
           big_probs: Optional[torch.Tensor] = None,
           forced: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of logits [rows, V] (float32).

    Without ``temperature`` every row takes the first index of its maximum.
    Otherwise the settings (float32 / int32 arrays) and ``rng`` (int64 array,
    the splitmix64 states) are indexed by row_slot[row]; a row whose
    temperature is 0 is still greedy and leaves its state alone."""
    _need(logits, "logits", torch.float32, (None, None))
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (rows,))
    for t, name, dt in ((row_slot, "row_slot", torch.int32), (temperature, "temperature",
                        torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (rng, "rng", torch.int64), (forced, "forced", torch.int32)):
        if t is not None:
            _need(t, name, dt)
    big_cap = 0
    if big_keys is not None:
        _need(big_keys, "big_keys", torch.int64, (None, None))
        _need(big_probs, "big_probs", torch.float32, tuple(big_keys.shape))
        if big_keys.shape[0] < rows:
            raise KernelError("sample: scratch for fewer rows than logits")
        big_cap = big_keys.shape[1]
    if temperature is not None and rng is None:
        raise KernelError("sample: temperature needs the random states")
    L = lib()
    chunk_keys = torch.empty((int(L.jb_sample_scratch(rows, V)),), dtype=torch.int64,
                             device=logits.device)
    launches = int(L.jb_sample_launches(V, int(big_cap), int(temperature is not None)))
    _check(L.jb_sample(_p(logits), rows, V, _p(row_slot), _p(temperature), _p(top_k),
                       _p(top_p), _p(min_p), _p(rng), _p(big_keys), _p(big_probs),
                       int(big_cap), _p(chunk_keys), _p(out), _p(forced), _stream()),
           "sample", kernels=launches)
    return out


def sample_small_cap() -> int:
    return int(lib().jb_sample_small_cap())
