"""Python face of the CUDA kernels: argument checks, then one C call per kernel.

Every function launches on torch's current CUDA stream and returns without
synchronising.  Tensors must live on the GPU and be contiguous; a wrong dtype,
shape or device raises before anything is launched.  There is no CPU path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build, tuning

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

CORE_SOURCES = ["elementwise.cu", "rope_kv.cu", "gemm_f32.cu", "gemm_small_m.cu", "attention_generic.cu",
                "sampling.cu", "norm_exact.cu", "gated_activation.cu", "qkv_store.cu", "gla_scan.cu", "moe.cu",
                "short_conv.cu", "rotary_freq.cu"]
SMALL_M_MAX_ROWS = min(16, tuning.SMALL_M_MAX_ROWS)      # the kernel takes 16 at most

_core = None


class KernelError(RuntimeError):
    pass


def core():
    global _core
    if _core is None:
        _core = build.load("qil_core", CORE_SOURCES)
    return _core


def dtype_code(dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


_post_step_checks: list = []


def register_post_step_check(check) -> None:
    """``check()`` raises if a kernel reported a fault of its own since the last call.  A kernel whose
    waits are bounded reports through an error word; its module registers the reader of that word here
    when its library is first loaded, and the step function's owner calls them after steps."""
    if check not in _post_step_checks:
        _post_step_checks.append(check)


def run_post_step_checks(wait=True) -> None:
    for check in _post_step_checks:
        check(wait)


class ErrorWord:
    """An int32 on the device that kernels with bounded waits set when a wait runs out, and its reader.

    ``check(wait=True)`` reads the word if a kernel that may set it was launched since the last check
    (``mark``); that waits for the device.  ``check(wait=False)`` never waits: it queues a copy of the
    word to pinned memory behind the work queued so far and reports what an earlier such copy
    brought, so a fault is reported a step or two late but the host never stalls a stream it is
    running ahead of.  The word stays set until it has been reported.
    """

    def __init__(self, describe):
        self._describe = describe
        self._word = self._host = self._event = None
        self._launched = self._copy_queued = False

    def tensor(self, device):
        if self._word is None:
            self._word = torch.zeros(1, dtype=torch.int32, device=device)
            self._host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
            self._event = torch.cuda.Event()
        return self._word

    def mark(self) -> None:
        self._launched = True

    def check(self, wait=True) -> None:
        if self._word is None:
            return
        code = 0
        if self._copy_queued and (wait or self._event.query()):
            self._event.synchronize()
            self._copy_queued = False
            code = int(self._host[0])
        if self._launched:
            self._launched = False
            if wait:
                code = code or int(self._word.item())
            else:
                self._host.copy_(self._word, non_blocking=True)
                self._event.record()
                self._copy_queued = True
        if code:
            self._word.zero_()
            self._copy_queued = False
            raise KernelError(self._describe(code))


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module since import (graph replays are counted by their owner)."""
    return _launches


def _check(lib, code, what, kernels=1):
    global _launches
    if code != 0:
        raise KernelError(f"{what}: {lib.qil_last_error().decode()} (code {code})")
    _launches += kernels


def _p(tensor):
    return c_void_p(tensor.data_ptr()) if tensor is not None else c_void_p(0)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(tensor, name, dtype=None, ndim=None):
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if ndim is not None and tensor.ndim != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got {tuple(tensor.shape)}")


def embed_gather(table, ids, out, scale=1.0):
    """out[r] = table[ids[r]] * scale cast to out's dtype (a float32 product, one rounding).  table [V,H]; ids int32
    [N]; out [N,H]."""
    _need(table, "table", ndim=2); _need(ids, "ids", torch.int32, 1); _need(out, "out", ndim=2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError(f"embed_gather: out {tuple(out.shape)} for ids {tuple(ids.shape)} table {tuple(table.shape)}")
    lib = core()
    _check(lib, lib.qil_embed_gather(_p(table), c_int(dtype_code(table.dtype)), _p(ids), _p(out),
                                     c_int(dtype_code(out.dtype)), c_int(ids.shape[0]), c_int(table.shape[1]),
                                     c_int(table.shape[0]), c_float(scale), _stream()), "embed_gather")
    return out


def fill_normal(out, seed, std, mean=0.0):
    """out[i] = mean + std * z(seed, i), z close to N(0, 1) from a counter hash (the same bits as
    ``weights.random_init.normal_values`` gives on the host)."""
    _need(out, "out")
    lib = core()
    _check(lib, lib.qil_fill_normal(_p(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
                                    ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), c_float(std), c_float(mean),
                                    _stream()), "fill_normal")
    return out


def rmsnorm(x, weight, eps, out=None, rows=None):
    """RMSNorm over the last dimension; with ``rows`` (int32) only those rows, in that order."""
    _need(x, "x", ndim=2); _need(weight, "weight", ndim=1)
    width = x.shape[1]
    if weight.shape[0] != width:
        raise KernelError(f"rmsnorm: weight of {weight.shape[0]} for width {width}")
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    if out is None:
        out = torch.empty((n_rows, width), dtype=x.dtype, device=x.device)
    _need(out, "out", x.dtype, 2)
    if out.shape != (n_rows, width):
        raise KernelError("rmsnorm: out has the wrong shape")
    lib = core()
    _check(lib, lib.qil_rmsnorm(_p(x), _p(weight), _p(rows), _p(out), c_int(n_rows), c_int(width),
                                c_float(eps), c_int(dtype_code(x.dtype)), c_int(dtype_code(weight.dtype)),
                                _stream()), "rmsnorm")
    return out


def silu_mul(gate_up, out=None, pairs8=False):
    """out = silu(gate) * up.  gate_up holds the gate columns then the up columns, or with
    ``pairs8`` groups of 16 columns: 8 gate columns followed by their 8 up columns."""
    _need(gate_up, "gate_up", ndim=2)
    if gate_up.shape[1] % 2:
        raise KernelError("silu_mul: the input's width must be even (gate columns then up columns)")
    width = gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((gate_up.shape[0], width), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype, 2)
    lib = core()
    _check(lib, lib.qil_silu_mul(_p(gate_up), _p(out), c_int(gate_up.shape[0]), c_int(width),
                                 c_int(dtype_code(gate_up.dtype)), c_int(1 if pairs8 else 0), _stream()), "silu_mul")
    return out


def small_m_ok(a, weight) -> bool:
    """Should ``gemm_small_m`` take this product?  bfloat16, at most 16 rows, K a multiple of 8.

    With 9 to 16 rows the kernel keeps three stages in flight instead of four; on a matrix as large
    as a vocabulary head (measured at 151936 x 4096: 274 us against the library's 211 us) that
    costs more than its epilogues save, so those go to the library.
    """
    if a.shape[0] > 8 and weight.shape[0] * weight.shape[1] >= tuning.SMALL_M_LIBRARY_ELEMENTS:
        return False
    return (a.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and a.shape[0] <= SMALL_M_MAX_ROWS
            and weight.shape[1] % 8 == 0 and a.is_contiguous())


def gemm_small_m(a, weight, bias=None, residual=None, out=None, out_float32=False, silu_pairs=False,
                 norm_weight=None, norm_eps=0.0, rows_per_block=None, col_scale=None, activation=None):
    """out = a @ weight.T (+ bias) (+ residual) for a decode step's few rows, streaming the weight once.

    a bfloat16 [M <= 16, K]; weight bfloat16 [N, K].  ``out_float32`` returns float32 (the LM head).
    ``silu_pairs``: weight rows are groups of [8 gate, 8 up]; returns silu(gate) * up, bfloat16 [M, N/2].
    ``residual`` may be ``out`` itself.  With ``norm_weight`` (bfloat16 [K]) the kernel first applies
    RMSNorm(a; norm_weight, norm_eps): the product of the normed rows, with no pass of its own over them.
    ``rows_per_block``: 16 or 32 output features a block (32 wants N a multiple of 32); None leaves it to the
    measured rule in ``tuning``.  The two forms add a product's terms in different orders.
    ``col_scale`` float32 [N]: out = (a @ weight.T + bias) * col_scale + residual.
    ``activation``: one of ``PLAIN_ACTIVATIONS`` on the product's bfloat16-rounded value (no residual, no scale).
    """
    _need(a, "a", torch.bfloat16, 2); _need(weight, "weight", torch.bfloat16, 2)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"gemm_small_m: a {tuple(a.shape)} against weight {tuple(weight.shape)}")
    out_shape = (m, n // 2) if silu_pairs else (m, n)
    out_dtype = torch.float32 if out_float32 else torch.bfloat16
    if bias is not None:
        _need(bias, "bias", torch.bfloat16, 1)
    if residual is not None:
        _need(residual, "residual", out_dtype, 2)          # a float32 output adds a float32 residual
        if residual.shape != out_shape:
            raise KernelError("gemm_small_m: residual has the wrong shape")
    if out is None:
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
    _need(out, "out", out_dtype, 2)
    if out.shape != out_shape:
        raise KernelError("gemm_small_m: out has the wrong shape")
    if norm_weight is not None:
        _need(norm_weight, "norm_weight", torch.bfloat16, 1)
        if norm_weight.shape[0] != k:
            raise KernelError("gemm_small_m: the norm weight must have one value per input feature")
    if col_scale is not None:
        _need(col_scale, "col_scale", torch.float32, 1)
        if col_scale.shape[0] != n or silu_pairs:
            raise KernelError("gemm_small_m: one output scale per feature, and none with silu_pairs")
    if activation is not None and (activation not in PLAIN_ACTIVATIONS or out_float32 or residual is not None
                                   or col_scale is not None or silu_pairs):
        raise KernelError("gemm_small_m: an activation goes with a plain bfloat16 output")
    if rows_per_block is None:
        wide = (n % 32 == 0 and n // 32 >= tuning.SMALL_M_WIDE_MIN_BLOCKS
                and (m > 8 or n * k < tuning.SMALL_M_WIDE_MAX_ELEMENTS))
        rows_per_block = 32 if wide else 16
    lib = core()
    _check(lib, lib.qil_gemm_small_m(_p(a), _p(weight), _p(bias), _p(residual), _p(out), _p(norm_weight),
                                     c_float(float(norm_eps)), c_int(m), c_int(n), c_int(k),
                                     c_int(1 if out_float32 else 0), c_int(1 if silu_pairs else 0),
                                     c_int(rows_per_block), _p(col_scale),
                                     c_int(ACTIVATIONS[activation] if activation is not None else -1), _stream()),
           "gemm_small_m")
    return out


def feed_tokens(token_ids, pairs, count, source):
    """token_ids[pairs[2i]] = source[pairs[2i + 1]] for i < count, on the stream (all int32, on the device):
    fills the places of tokens that the previous step sampled and the host has not read yet."""
    _need(token_ids, "token_ids", torch.int32, 1); _need(pairs, "pairs", torch.int32, 1)
    _need(source, "source", torch.int32, 1)
    if pairs.shape[0] < 2 * count:
        raise KernelError("feed_tokens: fewer pairs than count")
    lib = core()
    _check(lib, lib.qil_feed_tokens(_p(token_ids), _p(pairs), c_int(count), _p(source), c_int(source.shape[0]),
                                    c_int(token_ids.shape[0]), _stream()), "feed_tokens")


def add_inplace(x, y):
    _need(x, "x"); _need(y, "y", x.dtype)
    if x.shape != y.shape:
        raise KernelError("add_inplace: shapes differ")
    lib = core()
    _check(lib, lib.qil_add_inplace(_p(x), _p(y), c_longlong(x.numel()), c_int(dtype_code(x.dtype)), _stream()),
           "add_inplace")
    return x


def cast(src, dtype, out=None):
    _need(src, "src")
    if out is None:
        out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _need(out, "out", dtype)
    lib = core()
    _check(lib, lib.qil_cast(_p(src), c_int(dtype_code(src.dtype)), _p(out), c_int(dtype_code(dtype)),
                             c_longlong(src.numel()), _stream()), "cast")
    return out


def gemm_f32(a, weight, bias=None, residual=None, out=None, col_scale=None):
    """out = (a @ weight.T (+ bias)) (* col_scale) (+ residual), float32 accumulation on the CUDA cores.

    a [M,K] and out [M,N] share a dtype; weight [N,K] and bias [N] share another.
    ``residual`` may be ``out`` itself.  ``col_scale`` float32 [N]: a scale per output feature.
    """
    _need(a, "a", ndim=2); _need(weight, "weight", ndim=2)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"gemm_f32: a {tuple(a.shape)} against weight {tuple(weight.shape)}")
    if bias is not None:
        _need(bias, "bias", weight.dtype, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm_f32: bias has the wrong length")
    if out is None:
        out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    _need(out, "out", a.dtype, 2)
    if out.shape != (m, n):
        raise KernelError("gemm_f32: out has the wrong shape")
    if residual is not None:
        _need(residual, "residual", a.dtype, 2)
        if residual.shape != (m, n):
            raise KernelError("gemm_f32: residual has the wrong shape")
    if col_scale is not None:
        _need(col_scale, "col_scale", torch.float32, 1)
        if col_scale.shape[0] != n:
            raise KernelError("gemm_f32: col_scale has the wrong length")
    lib = core()
    _check(lib, lib.qil_gemm_f32(_p(a), c_int(k), _p(weight), _p(bias), _p(residual), _p(out), c_int(m), c_int(n),
                                 c_int(k), c_int(dtype_code(a.dtype)), c_int(dtype_code(weight.dtype)), _p(col_scale),
                                 _stream()),
           "gemm_f32")
    return out


def qk_norm_rope_store(qkv, q_out, kv_cache, q_norm_w, k_norm_w, eps, rope_table, rotary_dim,
                       positions, token_row, block_table, n_q_heads, n_kv_heads, head_dim, page_size):
    """Norm and rotate q and k heads of ``qkv``, write q to ``q_out`` and k, v into ``kv_cache``.

    qkv [N, (Hq + 2*Hkv) * D]; q_out [N, Hq*D]; kv_cache [pages, 2, Hkv, P, D] (one layer);
    rope_table float32 [positions, rotary_dim] or None; block_table int32 [rows, max_pages].
    With n_kv_heads == 0 only queries are processed (a layer that reads another layer's cache).
    """
    _need(qkv, "qkv", ndim=2); _need(q_out, "q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * head_dim or q_out.shape != (n, n_q_heads * head_dim):
        raise KernelError("qk_norm_rope_store: qkv/q_out shapes do not match the head counts")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    num_pages = 0
    if n_kv_heads:
        _need(kv_cache, "kv_cache", qkv.dtype, 5); _need(block_table, "block_table", torch.int32, 2)
        if tuple(kv_cache.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise KernelError(f"qk_norm_rope_store: cache layout {tuple(kv_cache.shape)}")
        num_pages = kv_cache.shape[0]
    norm_code = F32
    if q_norm_w is not None:
        _need(q_norm_w, "q_norm_w", ndim=1); _need(k_norm_w, "k_norm_w", q_norm_w.dtype, 1)
        if q_norm_w.shape[0] != head_dim or k_norm_w.shape[0] != head_dim:
            raise KernelError("qk_norm_rope_store: norm weights must have head_dim elements")
        norm_code = dtype_code(q_norm_w.dtype)
    table_rows = 0
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32, 2)
        if rope_table.shape[1] != rotary_dim:
            raise KernelError("qk_norm_rope_store: rope table width must equal rotary_dim")
        table_rows = rope_table.shape[0]
    lib = core()
    _check(lib, lib.qil_qk_norm_rope_store(
        _p(qkv), _p(q_out), _p(kv_cache if n_kv_heads else None), _p(q_norm_w), _p(k_norm_w), c_int(norm_code),
        c_float(eps), _p(rope_table), c_int(rotary_dim if rope_table is not None else 0), c_int(table_rows),
        _p(positions), _p(token_row), _p(block_table if n_kv_heads else None),
        c_int(block_table.shape[1] if n_kv_heads else 0), c_int(n), c_int(n_q_heads), c_int(n_kv_heads),
        c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(dtype_code(qkv.dtype)), _stream()),
        "qk_norm_rope_store")
    return q_out


def check_pages(kv_cache, dtype, n_kv_heads, page_size, head_dim, v_dim, what, shared_rows=False):
    """One layer's pages: [pages, 2, kv_heads, page_size, head_dim] when keys and values have one size,
    else [pages, kv_heads * page_size * (head_dim + v_dim)] (a page's key rows, then its value rows); with
    ``shared_rows`` [pages, 1, kv_heads, page_size, head_dim] (the value is the key's first v_dim columns)."""
    _need(kv_cache, "kv_cache", dtype)
    if shared_rows:
        if tuple(kv_cache.shape[1:]) != (1, n_kv_heads, page_size, head_dim) or not 0 < v_dim <= head_dim:
            raise KernelError(f"{what}: cache layout {tuple(kv_cache.shape)} for {n_kv_heads} shared rows of {head_dim} "
                              f"(values of {v_dim}), pages of {page_size}")
        return
    equal = tuple(kv_cache.shape[1:]) == (2, n_kv_heads, page_size, head_dim) and v_dim == head_dim
    flat = kv_cache.ndim == 2 and kv_cache.shape[1] == n_kv_heads * page_size * (head_dim + v_dim)
    if not (equal or flat):
        raise KernelError(f"{what}: cache layout {tuple(kv_cache.shape)} for {n_kv_heads} heads of {head_dim}/{v_dim}, "
                          f"pages of {page_size}")


def attention_generic(q, kv_cache, out, positions, token_row, block_table, n_q_heads, n_kv_heads,
                      head_dim, page_size, window, scale, v_dim=None, slopes=None, softcap=0.0, distance_bias=None,
                      chunk=0, sink=False, sink_logits=None, shared_rows=False):
    """Causal GQA attention of every token over its request's pages (CUDA cores, float32 math).

    ``v_dim``: the size of a value head when it differs from ``head_dim`` (out is then [N, Hq * v_dim]).
    ``shared_rows``: a page holds one row per position, the key; its first ``v_dim`` columns are the value.
    ``slopes`` float32 [Hq]: score = q.k * scale - slopes[h] * (query position - key position).
    ``softcap``: score <- softcap * tanh(score / softcap) before any bias.  ``distance_bias`` float32
    [Hq, distances]: added by distance, the last entry for every distance beyond.  ``chunk``: a position sees
    only the keys of its own chunk of that many positions.  ``sink``: one is added to the softmax's denominator;
    ``sink_logits`` float32 [Hq]: exp(sink_logits[h]) is added instead (a learned score per head, not scaled)."""
    v_dim = head_dim if v_dim is None else int(v_dim)
    _need(q, "q", ndim=2); _need(out, "out", q.dtype, 2)
    check_pages(kv_cache, q.dtype, n_kv_heads, page_size, head_dim, v_dim, "attention_generic", shared_rows)
    n = q.shape[0]
    if q.shape[1] != n_q_heads * head_dim or out.shape != (n, n_q_heads * v_dim):
        raise KernelError("attention_generic: q/out shapes do not match the head counts")
    if slopes is not None:
        _need(slopes, "slopes", torch.float32, 1)
        if slopes.shape[0] != n_q_heads:
            raise KernelError("attention_generic: one slope per query head")
    if distance_bias is not None:
        _need(distance_bias, "distance_bias", torch.float32, 2)
        if distance_bias.shape[0] != n_q_heads or distance_bias.shape[1] < 1:
            raise KernelError("attention_generic: the distance table is [query heads, distances]")
    if sink_logits is not None:
        _need(sink_logits, "sink_logits", torch.float32, 1)
        if sink_logits.shape[0] != n_q_heads:
            raise KernelError("attention_generic: one sink score per query head")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    lib = core()
    _check(lib, lib.qil_attention_generic(
        _p(q), _p(kv_cache), _p(out), _p(positions), _p(token_row), _p(block_table), c_int(block_table.shape[1]),
        c_int(n), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(v_dim), c_int(page_size),
        c_int(kv_cache.shape[0]), c_int(window), c_float(scale), _p(slopes), c_float(softcap), _p(distance_bias),
        c_int(distance_bias.shape[1] if distance_bias is not None else 0), c_int(chunk), c_int(1 if sink else 0),
        _p(sink_logits), c_int(1 if shared_rows else 0), c_int(dtype_code(q.dtype)), _stream()),
        "attention_generic")
    return out


def rmsnorm_exact(x, weight, eps, offset=0.0, out_dtype=None, rows=None, out=None, columns=None):
    """y = x / sqrt(mean(x^2) + eps) * (offset + weight) with float32 arithmetic and one rounding.
    ``x`` float32 or bfloat16 [N, width]; the result has ``out_dtype`` (default: x's).  ``columns`` = (first, width):
    the norm is over that column range of ``x`` alone (a piece of a stacked projection)."""
    _need(x, "x", ndim=2); _need(weight, "weight", ndim=1)
    ld = x.shape[1]
    first, width = (0, ld) if columns is None else (int(columns[0]), int(columns[1]))
    if first < 0 or width <= 0 or first + width > ld:
        raise KernelError(f"rmsnorm_exact: columns {first} .. {first + width} of {ld}")
    if weight.shape[0] != width:
        raise KernelError(f"rmsnorm_exact: weight of {weight.shape[0]} for width {width}")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, width), dtype=out_dtype or x.dtype, device=x.device)
    _need(out, "out", ndim=2)
    if out.shape != (n_rows, width):
        raise KernelError("rmsnorm_exact: out has the wrong shape")
    lib = core()
    _check(lib, lib.qil_rmsnorm_exact(c_void_p(x.data_ptr() + first * x.element_size()), c_int(dtype_code(x.dtype)),
                                      _p(weight), c_int(dtype_code(weight.dtype)),
                                      _p(rows), _p(out), c_int(dtype_code(out.dtype)), c_int(n_rows), c_int(width),
                                      c_float(eps), c_float(offset), c_longlong(ld), _stream()), "rmsnorm_exact")
    return out


def layernorm_exact(x, weight, bias, eps, out_dtype=None, rows=None, out=None):
    """y = (x - mean) / sqrt(var + eps) * weight + bias with float32 arithmetic and one rounding; var is the mean
    of the squared deviations.  ``x`` float32 or bfloat16 [N, width]; the result has ``out_dtype`` (default: x's).
    ``bias`` None: a layer norm without one."""
    _need(x, "x", ndim=2); _need(weight, "weight", ndim=1)
    width = x.shape[1]
    if bias is not None:
        _need(bias, "bias", weight.dtype, 1)
    if weight.shape[0] != width or (bias is not None and bias.shape[0] != width):
        raise KernelError(f"layernorm_exact: weight of {weight.shape[0]} (or the bias) for width {width}")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    n_rows = x.shape[0] if rows is None else rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, width), dtype=out_dtype or x.dtype, device=x.device)
    _need(out, "out", ndim=2)
    if out.shape != (n_rows, width):
        raise KernelError("layernorm_exact: out has the wrong shape")
    lib = core()
    _check(lib, lib.qil_layernorm_exact(_p(x), c_int(dtype_code(x.dtype)), _p(weight), _p(bias),
                                        c_int(dtype_code(weight.dtype)), _p(rows), _p(out), c_int(dtype_code(out.dtype)),
                                        c_int(n_rows), c_int(width), c_float(eps), _stream()), "layernorm_exact")
    return out


def rms_scale_add(x, y, weight, eps):
    """x += y / sqrt(mean(y^2) + eps) * weight, row by row, float32 arithmetic: a branch normed by its own root
    mean square joins the stream ``x`` (float32 or bfloat16 [N, width]) in place."""
    _need(x, "x", ndim=2); _need(y, "y", ndim=2); _need(weight, "weight", ndim=1)
    if y.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError("rms_scale_add: shapes differ")
    lib = core()
    _check(lib, lib.qil_rms_scale_add(_p(x), c_int(dtype_code(x.dtype)), _p(y), c_int(dtype_code(y.dtype)), _p(weight),
                                      c_int(dtype_code(weight.dtype)), c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps),
                                      _stream()), "rms_scale_add")
    return x


def scaled_add(x, y, scale):
    """x[r, c] += scale[c] * y[r, c] in place (float32 arithmetic); ``scale`` float32 [width]."""
    _need(x, "x", ndim=2); _need(y, "y", ndim=2); _need(scale, "scale", torch.float32, 1)
    if y.shape != x.shape or scale.shape[0] != x.shape[1]:
        raise KernelError("scaled_add: shapes differ")
    lib = core()
    _check(lib, lib.qil_scaled_add(_p(x), c_int(dtype_code(x.dtype)), _p(y), c_int(dtype_code(y.dtype)), _p(scale),
                                   c_int(x.shape[0]), c_int(x.shape[1]), _stream()), "scaled_add")
    return x


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2, "relu2": 3}
PLAIN_ACTIVATIONS = ("silu", "gelu_tanh", "relu2")      # those that need no gate


def activation(z, kind, *, table=None, ids=None, first_col=0, out=None):
    """out = act(z) for ``kind`` in ``PLAIN_ACTIVATIONS`` (``relu2``: max(z, 0)^2); with ``table`` [rows, columns]
    and ``ids`` int32 [N]: out[r, c] = act(z[r, c]) * table[ids[r], first_col + c].  ``out`` may be ``z``."""
    _need(z, "z", ndim=2)
    if kind not in PLAIN_ACTIVATIONS:
        raise KernelError(f"activation: unknown kind {kind!r} (known: {PLAIN_ACTIVATIONS})")
    if out is None:
        out = torch.empty_like(z)
    _need(out, "out", z.dtype, 2)
    if table is not None:
        _need(table, "table", ndim=2); _need(ids, "ids", torch.int32, 1)
        if ids.shape[0] != z.shape[0] or first_col < 0 or first_col + z.shape[1] > table.shape[1]:
            raise KernelError("activation: the table's columns or the ids do not fit the rows")
    lib = core()
    _check(lib, lib.qil_activation(_p(z), _p(out), c_int(z.shape[0]), c_int(z.shape[1]), c_int(dtype_code(z.dtype)),
                                   c_int(ACTIVATIONS[kind]), _p(table),
                                   c_int(dtype_code(table.dtype) if table is not None else 0), _p(ids),
                                   c_int(table.shape[1] if table is not None else 0), c_int(first_col),
                                   c_int(table.shape[0] if table is not None else 0), _stream()), "activation")
    return out


def short_conv_store(u, taps_weight, state, q_out, kv_cache, positions, token_row, block_table, seg_row, seg_start,
                     seg_len, n_segments, n_q_heads, n_kv_heads, head_dim, v_dim, page_size):
    """A short causal convolution over time on every channel of ``u`` [N, Hq*d + Hkv*d + Hkv*e] (the stacked q/k/v
    projection), queries to ``q_out``, keys and values into the pages.  ``taps_weight`` [taps, channels];
    ``state`` float32 [slots, taps - 1, channels]: the last rows of ``u`` that each request has seen, read for
    the positions before a step's first token and moved on.  Segments are the step's (int32 device arrays)."""
    _need(u, "u", ndim=2); _need(q_out, "q_out", u.dtype, 2); _need(taps_weight, "taps_weight", ndim=2)
    n, channels = u.shape
    taps = taps_weight.shape[0]
    if channels != n_q_heads * head_dim + n_kv_heads * (head_dim + v_dim) or q_out.shape != (n, n_q_heads * head_dim) \
            or taps_weight.shape[1] != channels:
        raise KernelError("short_conv_store: shapes do not match the head counts")
    _need(state, "state", torch.float32, 3)
    if tuple(state.shape[1:]) != (taps - 1, channels):
        raise KernelError(f"short_conv_store: state {tuple(state.shape)} for {taps} taps and {channels} channels")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    num_pages = 0
    if n_kv_heads:
        check_pages(kv_cache, u.dtype, n_kv_heads, page_size, head_dim, v_dim, "short_conv_store")
        _need(block_table, "block_table", torch.int32, 2)
        num_pages = kv_cache.shape[0]
    lib = core()
    _check(lib, lib.qil_short_conv_store(
        _p(u), _p(taps_weight), _p(state), _p(q_out), _p(kv_cache if n_kv_heads else None), _p(positions),
        _p(token_row), _p(block_table if n_kv_heads else None), c_int(block_table.shape[1] if n_kv_heads else 0),
        c_int(n), c_int(taps), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(v_dim), c_int(page_size),
        c_int(num_pages), c_int(dtype_code(u.dtype)), c_int(dtype_code(taps_weight.dtype)), _stream()),
        "short_conv_store")
    if taps > 1 and n_segments < n:      # some request brought more than one token: its state moves on here
        for t in (seg_row, seg_start, seg_len):
            _need(t, "segments", torch.int32, 1)
        _check(lib, lib.qil_short_conv_state(_p(u), _p(state), _p(seg_row), _p(seg_start), _p(seg_len), c_int(n_segments),
                                             c_int(taps), c_int(channels), c_int(dtype_code(u.dtype)), _stream()),
               "short_conv_state")
    return q_out


def gated_activation(gate_up, kind, *, limit=0.0, alpha=1.0, pairs8=False, out=None):
    """out = act(gate) * f(up) for rows of [gate columns, up columns]: ``kind`` is ``silu``, ``gelu_tanh``, or
    ``clamped_swish``: min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    _need(gate_up, "gate_up", ndim=2)
    if gate_up.shape[1] % 2:
        raise KernelError("gated_activation: the input's width must be even (gate columns then up columns)")
    if kind not in ACTIVATIONS:
        raise KernelError(f"gated_activation: unknown kind {kind!r} (known: {sorted(ACTIVATIONS)})")
    width = gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((gate_up.shape[0], width), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype, 2)
    lib = core()
    _check(lib, lib.qil_gated_activation(_p(gate_up), _p(out), c_int(gate_up.shape[0]), c_int(width),
                                         c_int(dtype_code(gate_up.dtype)), c_int(1 if pairs8 else 0),
                                         c_int(ACTIVATIONS[kind]), c_float(limit), c_float(alpha), _stream()),
           "gated_activation")
    return out


def qkv_store(qkv, q_out, kv_cache, positions, token_row, block_table, n_q_heads, n_kv_heads, head_dim, v_dim,
              page_size, temp_coef=0.0, temp_every=0):
    """Copy the queries of ``qkv`` [N, Hq*d + Hkv*d + Hkv*e] to ``q_out`` (times 1 + coef * ln(floor((p + 1) /
    every) + 1) at position p when ``temp_coef`` is set) and write keys and values into the pages.
    With n_kv_heads == 0 ``qkv`` holds queries only."""
    _need(qkv, "qkv", ndim=2); _need(q_out, "q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != n_q_heads * head_dim + n_kv_heads * (head_dim + v_dim) or q_out.shape != (n, n_q_heads * head_dim):
        raise KernelError("qkv_store: qkv/q_out shapes do not match the head counts")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    num_pages = 0
    if n_kv_heads:
        check_pages(kv_cache, qkv.dtype, n_kv_heads, page_size, head_dim, v_dim, "qkv_store")
        _need(block_table, "block_table", torch.int32, 2)
        num_pages = kv_cache.shape[0]
    lib = core()
    _check(lib, lib.qil_qkv_store(
        _p(qkv), _p(q_out), _p(kv_cache if n_kv_heads else None), _p(positions), _p(token_row),
        _p(block_table if n_kv_heads else None), c_int(block_table.shape[1] if n_kv_heads else 0), c_int(n),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(v_dim), c_int(page_size), c_int(num_pages),
        c_float(temp_coef), c_int(temp_every), c_int(dtype_code(qkv.dtype)), _stream()), "qkv_store")
    return q_out


def gla_scan_needs_scratch(d, e) -> bool:
    code = core().qil_gla_scan_needs_scratch(c_int(d), c_int(e))
    if code < 0:
        raise KernelError(f"gla_scan: {d} key channels per head are too many")
    return bool(code)


GLA_WHOLE, GLA_OWN_STATE, GLA_FROM_STATE = 0, 1, 2


def gla_decay(projected, low_column, a2, a2_bias, tau, out=None):
    """alpha float32 [N, channels] = sigmoid(a2 low + a2_bias)^(1/tau), ``low`` being the a2.shape[1] columns of
    ``projected`` from ``low_column`` on: the decay of every key channel at every token, in float32."""
    _need(projected, "projected", ndim=2); _need(a2, "a2", ndim=2); _need(a2_bias, "a2_bias", a2.dtype, 1)
    n, ld = projected.shape
    channels, rank = a2.shape
    if a2_bias.shape[0] != channels or low_column + rank > ld or not tau > 0:
        raise KernelError("gla_decay: shapes do not fit together")
    if out is None:
        out = torch.empty((n, channels), dtype=torch.float32, device=projected.device)
    _need(out, "out", torch.float32, 2)
    lib = core()
    _check(lib, lib.qil_gla_decay(c_void_p(projected.data_ptr() + low_column * projected.element_size()), c_int(ld),
                                  _p(a2), _p(a2_bias), c_int(rank), c_float(tau), c_int(n), c_int(channels), _p(out),
                                  c_int(dtype_code(projected.dtype)), c_int(dtype_code(a2.dtype)), _stream()), "gla_decay")
    return out


def gla_scan(projected, columns, alpha, q_scale, norm_weight, eps, state, seg_start, seg_len, seg_row,
             n_segments, n_heads, d, e, out, scratch=None, mode=GLA_WHOLE, decay_product=None, head_decay=None,
             silu_inputs=False, raw_only=False):
    """Gated linear attention over segments of a step (see csrc/gla_scan.cu for the equations).

    ``projected`` [N, width]: the stacked projection; ``columns`` = (q, k, v, g) first columns in it
    (q, k: n_heads * d wide; v, g: n_heads * e).  ``alpha`` float32 [N, n_heads * d]: the decays
    (``gla_decay``).  ``state`` float32 [slots, n_heads, d, e] is read and written at the rows ``seg_row`` names.
    ``out`` [N, n_heads * e].  ``scratch``: float32 [N, n_heads * e], needed when ``gla_scan_needs_scratch``: the
    outputs then go there un-normed and ``gla_norm_gate`` finishes them.  ``mode``: GLA_WHOLE; GLA_OWN_STATE scans
    from zero and writes only the segment's own state to ``state[seg_row]`` and the product of its decays to
    ``decay_product`` [slots, n_heads, d]; GLA_FROM_STATE reads ``state[seg_row]``, writes the outputs and leaves
    the state.

    ``head_decay`` float32 [n_heads] (with ``alpha`` None): one fixed decay per head instead of a decay per token and
    key channel.  ``silu_inputs``: silu on q, k and v as they are read.  ``raw_only``: the un-normed outputs go to
    ``scratch`` whatever the sizes and nothing is normed or gated here (``out`` and ``norm_weight`` may be None)."""
    _need(projected, "projected", ndim=2)
    if not raw_only:
        _need(out, "out", projected.dtype, 2); _need(norm_weight, "norm_weight", ndim=1)
    elif scratch is None and mode != GLA_OWN_STATE:
        raise KernelError("gla_scan: raw outputs need the scratch buffer")
    if (alpha is None) == (head_decay is None):
        raise KernelError("gla_scan: give the decays per token or one per head")
    if alpha is not None:
        _need(alpha, "alpha", torch.float32, 2)
    else:
        _need(head_decay, "head_decay", torch.float32, 1)
        if head_decay.shape[0] != n_heads:
            raise KernelError("gla_scan: one decay per head")
    _need(state, "state", torch.float32, 4)
    n, ld = projected.shape
    q_at, k_at, v_at, g_at = (int(c) for c in columns[:4])
    if ((alpha is not None and alpha.shape != (n, n_heads * d)) or tuple(state.shape[1:]) != (n_heads, d, e)
            or (not raw_only and (norm_weight.shape[0] != e or out.shape != (n, n_heads * e)))):
        raise KernelError("gla_scan: shapes do not match the head counts")
    if max(q_at + n_heads * d, k_at + n_heads * d, v_at + n_heads * e, g_at + n_heads * e) > ld:
        raise KernelError("gla_scan: a column range lies outside the projection")
    for t in (seg_start, seg_len, seg_row):
        _need(t, "segments", torch.int32, 1)
        if t.shape[0] < n_segments:
            raise KernelError("gla_scan: fewer segment entries than segments")
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < n * n_heads * e:
            raise KernelError("gla_scan: the scratch buffer is too small")
    if mode == GLA_OWN_STATE:
        _need(decay_product, "decay_product", torch.float32, 3)
        if decay_product.shape != (state.shape[0], n_heads, d):
            raise KernelError("gla_scan: decay_product must be [states, heads, d]")
    size = projected.element_size()
    base = projected.data_ptr()
    lib = core()
    _check(lib, lib.qil_gla_scan(
        c_void_p(base + q_at * size), c_void_p(base + k_at * size), c_void_p(base + v_at * size),
        c_void_p(base + g_at * size), _p(alpha), _p(head_decay), c_int(1 if silu_inputs else 0),
        c_int(1 if raw_only else 0), c_int(ld), c_float(q_scale), _p(norm_weight), c_float(eps), _p(state),
        _p(seg_start), _p(seg_len), _p(seg_row), c_int(n_segments), c_int(n), c_int(n_heads), c_int(d), c_int(e),
        _p(scratch), _p(out), c_int(mode), _p(decay_product), c_int(dtype_code(projected.dtype)),
        c_int(dtype_code(norm_weight.dtype) if norm_weight is not None else F32), _stream()), "gla_scan")
    return out


def gla_carry(chunk_state, decay_product, slots, carry, n_carries):
    """Walk the chunks of long segments in order: ``chunk_state`` [chunks, heads, d, e] holds every chunk's own
    state and receives its incoming one; the state after a segment's last chunk goes to its slot.
    ``carry`` int32 [n_carries * 3] = (slot, first chunk, chunks)."""
    _need(chunk_state, "chunk_state", torch.float32, 4); _need(decay_product, "decay_product", torch.float32, 3)
    _need(slots, "slots", torch.float32, 4); _need(carry, "carry", torch.int32, 1)
    if tuple(slots.shape[1:]) != tuple(chunk_state.shape[1:]) or decay_product.shape != chunk_state.shape[:3] \
            or carry.shape[0] < 3 * n_carries:
        raise KernelError("gla_carry: shapes do not fit together")
    lib = core()
    _check(lib, lib.qil_gla_carry(_p(chunk_state), _p(decay_product), _p(slots), _p(carry), c_int(n_carries),
                                  c_int(chunk_state.shape[1]), c_int(chunk_state.shape[2]), c_int(chunk_state.shape[3]),
                                  _stream()), "gla_carry")


def gla_norm_gate(scratch, projected, gate_column, norm_weight, eps, n_heads, e, out):
    """out = rmsnorm over each head's e values of ``scratch`` (weight ``norm_weight``) * silu(gate), the gate
    being the columns of ``projected`` from ``gate_column`` on."""
    _need(scratch, "scratch", torch.float32); _need(projected, "projected", ndim=2); _need(out, "out", projected.dtype, 2)
    n = projected.shape[0]
    if out.shape != (n, n_heads * e) or scratch.numel() < n * n_heads * e or gate_column + n_heads * e > projected.shape[1]:
        raise KernelError("gla_norm_gate: shapes do not fit together")
    lib = core()
    _check(lib, lib.qil_gla_norm_gate(_p(scratch), c_void_p(projected.data_ptr() + gate_column * projected.element_size()),
                                      c_int(projected.shape[1]), _p(norm_weight), c_float(eps), c_int(n), c_int(n_heads),
                                      c_int(e), _p(out), c_int(dtype_code(projected.dtype)),
                                      c_int(dtype_code(norm_weight.dtype)), _stream()), "gla_norm_gate")
    return out


def lin_norm_gate_whole(scratch, projected, gate_column, norm_weight, eps, out):
    """out [N, width] = ``scratch`` (float32 [N, width]) / sqrt(mean(scratch^2) + eps) * norm_weight * sigmoid(gate): one
    norm over a token's whole row (all heads together); the gate is the ``width`` columns of ``projected`` from
    ``gate_column`` on."""
    _need(scratch, "scratch", torch.float32); _need(projected, "projected", ndim=2); _need(out, "out", projected.dtype, 2)
    _need(norm_weight, "norm_weight", ndim=1)
    n, width = out.shape
    if projected.shape[0] != n or scratch.numel() < n * width or gate_column + width > projected.shape[1] \
            or norm_weight.shape[0] != width:
        raise KernelError("lin_norm_gate_whole: shapes do not fit together")
    lib = core()
    _check(lib, lib.qil_lin_norm_gate_whole(_p(scratch), c_void_p(projected.data_ptr() + gate_column * projected.element_size()),
                                            c_int(projected.shape[1]), _p(norm_weight), c_float(eps), c_int(n), c_int(width),
                                            _p(out), c_int(dtype_code(projected.dtype)),
                                            c_int(dtype_code(norm_weight.dtype)), _stream()), "lin_norm_gate_whole")
    return out


def rms_join(x, a, weight, eps, mult=1.0, *, b=None, weight_a=None, weight_b=None, pre=0.5, rows=None):
    """x += mult * a / sqrt(mean(a^2) + eps) * weight, row by row in float32: a branch joins the stream ``x`` (float32
    or bfloat16 [N, width], updated in place) through a norm on the branch.  With a second branch ``b``:
    y = pre * (rms(a) * weight_a + rms(b) * weight_b), x += mult * rms(y) * weight.  ``rows``: bfloat16 [N, width] that
    receives the stream's new values rounded (what the next product reads, without a cast of its own)."""
    if rows is not None:
        _need(rows, "rows", torch.bfloat16, 2)
        if rows.shape != x.shape:
            raise KernelError("rms_join: the rounded copy has another shape")
    _need(x, "x", ndim=2); _need(a, "a", ndim=2); _need(weight, "weight", ndim=1)
    if a.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError("rms_join: shapes differ")
    if b is not None:
        _need(b, "b", a.dtype, 2); _need(weight_a, "weight_a", weight.dtype, 1); _need(weight_b, "weight_b", weight.dtype, 1)
        if b.shape != x.shape or weight_a.shape != weight.shape or weight_b.shape != weight.shape:
            raise KernelError("rms_join: the second branch or its weights have another shape")
    lib = core()
    _check(lib, lib.qil_rms_join(_p(x), c_int(dtype_code(x.dtype)), _p(a), _p(weight_a), _p(b), _p(weight_b),
                                 c_int(dtype_code(a.dtype)), _p(weight), c_int(dtype_code(weight.dtype)), c_int(x.shape[0]),
                                 c_int(x.shape[1]), c_float(eps), c_float(pre), c_float(mult), _p(rows), _stream()),
           "rms_join")
    return x


def softcap_inplace(x, cap):
    """x <- cap * tanh(x / cap) for float32 ``x`` (logits)."""
    _need(x, "x", torch.float32)
    lib = core()
    _check(lib, lib.qil_softcap_inplace(_p(x), c_longlong(x.numel()), c_float(cap), _stream()), "softcap_inplace")
    return x


NORM_KINDS = {"rms": 0, "layer": 1}     # root mean square; mean taken off first (a layer norm without a bias)


def norm_join(x, branch, weight, eps, kind="rms", *, next_weight=None, next_eps=None, next_kind=None, rows=None):
    """x += norm(branch) * weight row by row in float32 (``kind``: ``"rms"`` or ``"layer"``, the layer norm without a
    bias): a float32 branch joins the stream ``x`` (float32 or bfloat16 [N, width], updated in place) through a norm
    on the branch.  ``rows`` [N, width] (bfloat16 or float32) receives what the next sublayer reads: with
    ``next_weight`` the norm of the new stream (``next_kind``, ``next_eps``; the defaults are this norm's), without it
    the new stream rounded."""
    _need(x, "x", ndim=2); _need(branch, "branch", torch.float32, 2); _need(weight, "weight", ndim=1)
    if branch.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError("norm_join: shapes differ")
    if kind not in NORM_KINDS or (next_kind or kind) not in NORM_KINDS:
        raise KernelError(f"norm_join: a norm is one of {sorted(NORM_KINDS)}")
    if rows is not None:
        _need(rows, "rows", ndim=2)
        if rows.shape != x.shape:
            raise KernelError("norm_join: the next sublayer's rows have another shape")
    if next_weight is not None:
        _need(next_weight, "next_weight", weight.dtype, 1)
        if rows is None or next_weight.shape != weight.shape:
            raise KernelError("norm_join: the next norm needs rows to write and a weight of the same size")
    lib = core()
    _check(lib, lib.qil_norm_join(_p(x), c_int(dtype_code(x.dtype)), _p(branch), _p(weight), c_int(dtype_code(weight.dtype)),
                                  c_int(x.shape[0]), c_int(x.shape[1]), c_float(eps), c_int(NORM_KINDS[kind]),
                                  _p(next_weight), c_float(eps if next_eps is None else next_eps),
                                  c_int(NORM_KINDS[next_kind or kind]), _p(rows),
                                  c_int(dtype_code(rows.dtype) if rows is not None else 0), _stream()), "norm_join")
    return x


def scale_inplace(x, factor):
    """x *= factor for float32 ``x`` (logits)."""
    _need(x, "x", torch.float32)
    lib = core()
    _check(lib, lib.qil_scale_inplace(_p(x), c_longlong(x.numel()), c_float(factor), _stream()), "scale_inplace")
    return x


ROTARY_HALVES, ROTARY_INTERLEAVED = 0, 1     # which dimensions pair up: i with i + dims / 2, or 2 i with 2 i + 1


def _check_rotation(freq, rot_dims, layout, most, what):
    if rot_dims:
        _need(freq, "freq", torch.float32, 1)
        if freq.shape[0] != rot_dims // 2:
            raise KernelError(f"{what}: one frequency per rotated pair")
    if rot_dims % 2 or not 0 <= rot_dims <= most or layout not in (ROTARY_HALVES, ROTARY_INTERLEAVED):
        raise KernelError(f"{what}: {rot_dims} rotated dimensions of {most}, layout {layout}")


def qk_rotate_store(proj, columns, q_out, kv_cache, q_norm_w, k_norm_w, eps, freq, rot_dims, layout, positions,
                    token_row, block_table, n_q_heads, n_kv_heads, head_dim, v_dim, page_size, per_head=False):
    """The tail of a q/k/v projection with rotation from frequencies (float32 angles position * freq[i]).

    ``proj`` [N, width] holds q, k, v from the columns ``columns`` = (q, k, v) on.  With ``q_norm_w`` [Hq * d] and
    ``k_norm_w`` [Hkv * d], q and k are first divided by their root mean square over the whole projection (all heads
    at once) and multiplied by the weight; with ``per_head`` every head is normed by itself over its d dimensions and
    the weights are [d], one for all query heads and one for all key heads.  The values are copied as projected from
    column v on: giving the keys' column there stores the keys as projected, before norm and rotation, as values.
    Then the first ``rot_dims`` dimensions of every head are rotated
    (``layout``: ``ROTARY_HALVES`` or ``ROTARY_INTERLEAVED``); queries go to ``q_out`` [N, Hq * d], keys and values
    into the pages."""
    _need(proj, "proj", ndim=2); _need(q_out, "q_out", proj.dtype, 2)
    n, ld = proj.shape
    q_at, k_at, v_at = (int(c) for c in columns)
    if q_out.shape != (n, n_q_heads * head_dim) or max(q_at + n_q_heads * head_dim, k_at + n_kv_heads * head_dim,
                                                       v_at + n_kv_heads * v_dim) > ld:
        raise KernelError("qk_rotate_store: shapes do not match the head counts")
    _check_rotation(freq, rot_dims, layout, head_dim, "qk_rotate_store")
    norm_code = F32
    if q_norm_w is not None:
        _need(q_norm_w, "q_norm_w", ndim=1)
        if n_kv_heads:
            _need(k_norm_w, "k_norm_w", q_norm_w.dtype, 1)
        if per_head:
            if q_norm_w.shape[0] != head_dim or (n_kv_heads and k_norm_w.shape[0] != head_dim):
                raise KernelError("qk_rotate_store: a per-head norm has one weight per dimension of a head")
        elif q_norm_w.shape[0] != n_q_heads * head_dim or (n_kv_heads and k_norm_w.shape[0] != n_kv_heads * head_dim):
            raise KernelError("qk_rotate_store: the norm weights cover the whole projections")
        norm_code = dtype_code(q_norm_w.dtype)
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    num_pages = 0
    if n_kv_heads:          # none: a layer that reads pages another layer wrote
        check_pages(kv_cache, proj.dtype, n_kv_heads, page_size, head_dim, v_dim, "qk_rotate_store")
        _need(block_table, "block_table", torch.int32, 2)
        num_pages = kv_cache.shape[0]
    lib = core()
    _check(lib, lib.qil_qk_rotate_store(
        _p(proj), c_int(ld), c_int(q_at), c_int(k_at), c_int(v_at), _p(q_out), _p(kv_cache if n_kv_heads else None),
        _p(q_norm_w), _p(k_norm_w), c_int(norm_code), c_float(eps), _p(freq), c_int(rot_dims), c_int(layout),
        _p(positions), _p(token_row), _p(block_table if n_kv_heads else None),
        c_int(block_table.shape[1] if n_kv_heads else 0), c_int(n), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim),
        c_int(v_dim), c_int(page_size), c_int(num_pages), c_int(dtype_code(proj.dtype)), c_int(1 if per_head else 0),
        _stream()), "qk_rotate_store")
    return q_out


def latent_prepare(proj, q_column, kv_column, q_att, kv_cache, norm_w, eps, freq, rot_dims, layout, positions, token_row,
                   block_table, n_heads, plain_dim, rot_dim, latent_dim, value_width, page_size, query_latent=None):
    """The tail of a latent attention's projection.  ``proj`` [N, width] holds the queries [H][plain_dim, rot_dim]
    from ``q_column`` on and one row [latent_dim, rot_dim] per token from ``kv_column`` on.  The latent is normed
    (root mean square, ``norm_w``), the shared key part and the queries' rotated parts are rotated; the token's page
    row becomes key [latent, rotated part] and value [latent, zeros up to ``value_width``] (``value_width`` 0: pages
    of shared rows, which hold the key alone); the rotated query parts go to the last rot_dim columns of every
    head's row of ``q_att`` [N, H * (latent_dim + rot_dim)].  ``query_latent`` = (column, weight, out): the queries'
    own latent, ``len(weight)`` columns of ``proj`` from ``column`` on, is normed the same way (``eps``, a weight of
    ``norm_w``'s dtype) into ``out`` [N, len(weight)]."""
    _need(proj, "proj", ndim=2); _need(q_att, "q_att", proj.dtype, 2); _need(norm_w, "norm_w", ndim=1)
    n, ld = proj.shape
    qn_col, qn_width, qn_w, qn_out = 0, 0, None, None
    if query_latent is not None:
        qn_col, qn_w, qn_out = query_latent
        _need(qn_w, "query latent's weight", norm_w.dtype, 1); _need(qn_out, "query latent's rows", proj.dtype, 2)
        qn_col, qn_width = int(qn_col), qn_w.shape[0]
        if qn_out.shape != (n, qn_width) or qn_col < 0 or qn_col + qn_width > ld:
            raise KernelError("latent_prepare: the queries' latent does not fit the projection")
    width = latent_dim + rot_dim
    if q_att.shape != (n, n_heads * width) or norm_w.shape[0] != latent_dim or kv_column + width > ld \
            or (rot_dim > 0 and q_column + n_heads * (plain_dim + rot_dim) > ld):      # without a rotated part q is not read
        raise KernelError("latent_prepare: shapes do not fit together")
    _check_rotation(freq, rot_dims, layout, rot_dim, "latent_prepare")
    _need(positions, "positions", torch.int32, 1); _need(token_row, "token_row", torch.int32, 1)
    check_pages(kv_cache, proj.dtype, 1, page_size, width, value_width or latent_dim, "latent_prepare", value_width == 0)
    _need(block_table, "block_table", torch.int32, 2)
    lib = core()
    _check(lib, lib.qil_latent_prepare(
        _p(proj), c_int(ld), c_int(q_column), c_int(kv_column), _p(q_att), _p(kv_cache), _p(norm_w),
        c_int(dtype_code(norm_w.dtype)), c_float(eps), _p(freq), c_int(rot_dims), c_int(layout), _p(positions),
        _p(token_row), _p(block_table), c_int(block_table.shape[1]), c_int(n), c_int(n_heads), c_int(plain_dim),
        c_int(rot_dim), c_int(latent_dim), c_int(value_width), c_int(page_size), c_int(kv_cache.shape[0]),
        c_int(dtype_code(proj.dtype)), c_int(qn_col), c_int(qn_width), _p(qn_w), _p(qn_out), _stream()), "latent_prepare")
    return q_att


def head_product(x, x_column, x_head_stride, weight, y, y_column, y_head_stride, *, gate=None, gate_column=0,
                 gate_each=False):
    """y[n, y_column + h * y_head_stride + j] = sum_i weight[h, j, i] * x[n, x_column + h * x_head_stride + i], times
    sigmoid(gate[n, gate_column + h]) when ``gate`` is given: one small product per head over column ranges of the
    row-major buffers ``x`` and ``y`` (float32 sums).  ``weight`` [H, out, in].  ``gate_each``: a gate per output,
    sigmoid(gate[n, gate_column + h * out + j]), instead of one per head."""
    _need(x, "x", ndim=2); _need(y, "y", x.dtype, 2); _need(weight, "weight", ndim=3)
    heads, n_out, n_in = weight.shape
    n = x.shape[0]
    if y.shape[0] != n or x_column + (heads - 1) * x_head_stride + n_in > x.shape[1] \
            or y_column + (heads - 1) * y_head_stride + n_out > y.shape[1]:
        raise KernelError("head_product: a column range lies outside its buffer")
    gate_ptr, gate_row = c_void_p(0), 0
    if gate is not None:
        _need(gate, "gate", x.dtype, 2)
        if gate.shape[0] != n or gate_column + heads * (n_out if gate_each else 1) > gate.shape[1]:
            raise KernelError("head_product: the gate's columns lie outside its buffer")
        gate_ptr, gate_row = c_void_p(gate.data_ptr() + gate_column * gate.element_size()), gate.shape[1]
    size = x.element_size()
    lib = core()
    _check(lib, lib.qil_head_product(
        c_void_p(x.data_ptr() + x_column * size), c_longlong(x.shape[1]), c_int(x_head_stride), _p(weight),
        c_void_p(y.data_ptr() + y_column * size), c_longlong(y.shape[1]), c_int(y_head_stride), gate_ptr,
        c_longlong(gate_row), c_int(n), c_int(heads), c_int(n_in), c_int(n_out), c_int(dtype_code(x.dtype)),
        c_int(dtype_code(weight.dtype)), c_int(1 if gate_each else 0), _stream()), "head_product")
    return y


def head_gate(y, width, gate, gate_column):
    """y[n, h * width + j] *= sigmoid(gate[n, gate_column + h]) in place: a gate per token and head on rows laid out
    head by head (float32 arithmetic, one rounding)."""
    _need(y, "y", ndim=2); _need(gate, "gate", y.dtype, 2)
    n = y.shape[0]
    if width <= 0 or y.shape[1] % width or gate.shape[0] != n or gate_column + y.shape[1] // width > gate.shape[1]:
        raise KernelError("head_gate: the gate's columns do not match the heads")
    lib = core()
    _check(lib, lib.qil_head_gate(_p(y), c_longlong(y.shape[1]), c_int(width),
                                  c_void_p(gate.data_ptr() + gate_column * gate.element_size()), c_longlong(gate.shape[1]),
                                  c_int(n), c_int(y.shape[1] // width), c_int(dtype_code(y.dtype)), _stream()), "head_gate")
    return y


def moe_route(x, router, bias, top, *, softmax_all=False, correction=None, weight_scale=1.0, gate_row=False,
              renormalize=True):
    """(chosen int32 [N, top], weights float32 [N, top]): the ``top`` largest of x R^T + b per row (float32
    arithmetic; the lower index wins a tie) and the softmax over those logits alone.

    ``softmax_all``: scores are the softmax over all outputs; the choice goes by score + ``correction`` (float32
    [outputs]), the weights are the chosen scores divided by their sum (+ 1e-20), times ``weight_scale``; with
    ``renormalize=False`` the chosen scores themselves, undivided.
    ``gate_row``: the last row of ``router`` is not an output but a gate's weights: its dot products are returned
    as a third result, float32 [N]."""
    _need(x, "x", ndim=2); _need(router, "router", ndim=2)
    if router.shape[1] != x.shape[1]:
        raise KernelError("moe_route: the router's width differs from x's")
    if bias is not None:
        _need(bias, "bias", router.dtype, 1)
    n = x.shape[0]
    outputs = router.shape[0] - (1 if gate_row else 0)
    if not renormalize and not softmax_all:
        raise KernelError("moe_route: only scores of a softmax over all outputs can stay as they are")
    if correction is not None:
        _need(correction, "correction", torch.float32, 1)
        if correction.shape[0] != outputs:
            raise KernelError("moe_route: one correction per output of the router")
    chosen = torch.empty((n, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=x.device)
    gate = torch.empty((n,), dtype=torch.float32, device=x.device) if gate_row else None
    lib = core()
    _check(lib, lib.qil_moe_route(_p(x), _p(router), _p(bias), c_int(n), c_int(x.shape[1]), c_int(outputs),
                                  c_int(top), _p(chosen), _p(weights), c_int((1 if renormalize else 2) if softmax_all else 0),
                                  _p(correction),
                                  c_float(weight_scale), _p(gate), c_int(dtype_code(x.dtype)),
                                  c_int(dtype_code(router.dtype)), _stream()), "moe_route")
    return (chosen, weights, gate) if gate_row else (chosen, weights)


def moe_experts(x, chosen, weights, gate_w, up_w, down_w, kind, *, limit=0.0, alpha=1.0, residual=None, out=None,
                identity=False, extra=None, extra_gate=None, col_scale=None):
    """out = residual + sum over a token's chosen experts of weight * down_e(act(gate_e x, up_e x)).

    gate_w, up_w [E, ff, width]; down_w [E, width, ff]; ``kind`` as in ``gated_activation`` (``silu`` or
    ``clamped_swish``).  ``residual`` and ``out`` [N, width] share a dtype (the residual stream's).
    ``up_w`` None: experts without a gate matrix, down_e(act(gate_w_e x)) with ``kind`` in ``PLAIN_ACTIVATIONS``.
    ``identity``: a choice >= E names no expert and adds weight * x.  ``extra`` float32 [N, width]: added too,
    times sigmoid(``extra_gate``) (float32 [N]) when that is given.  ``col_scale`` float32 [width] multiplies
    everything that is added to the residual."""
    _need(x, "x", ndim=2); _need(chosen, "chosen", torch.int32, 2); _need(weights, "weights", torch.float32, 2)
    _need(gate_w, "gate_w", ndim=3); _need(down_w, "down_w", gate_w.dtype, 3)
    if up_w is not None:
        _need(up_w, "up_w", gate_w.dtype, 3)
    n, width = x.shape
    experts, ff, _ = gate_w.shape
    top = chosen.shape[1]
    if (gate_w.shape != (experts, ff, width) or (up_w is not None and up_w.shape != gate_w.shape)
            or down_w.shape != (experts, width, ff) or chosen.shape[0] != n or weights.shape != chosen.shape):
        raise KernelError("moe_experts: shapes do not fit together")
    if kind not in (("silu", "clamped_swish") if up_w is not None else PLAIN_ACTIVATIONS):
        raise KernelError(f"moe_experts: activation {kind!r}")
    if extra is not None:
        _need(extra, "extra", torch.float32, 2)
        if extra.shape != (n, width):
            raise KernelError("moe_experts: extra has the wrong shape")
    if extra_gate is not None:
        _need(extra_gate, "extra_gate", torch.float32, 1)
    if col_scale is not None:
        _need(col_scale, "col_scale", torch.float32, 1)
    stream_dtype = residual.dtype if residual is not None else (out.dtype if out is not None else x.dtype)
    if out is None:
        out = torch.empty((n, width), dtype=stream_dtype, device=x.device)
    _need(out, "out", stream_dtype, 2)
    if residual is not None:
        _need(residual, "residual", stream_dtype, 2)
    lib = core()
    pairs = n * top
    tile_rows = lib.qil_moe_tile_rows()
    max_tiles = min(pairs, pairs // tile_rows + experts)
    work = torch.empty(1 + experts + pairs + 3 * max_tiles, dtype=torch.int32, device=x.device)
    info, sorted_pairs, tiles = work[:1 + experts], work[1 + experts:1 + experts + pairs], work[1 + experts + pairs:]
    hidden = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
    y = torch.empty((pairs, width), dtype=torch.float32, device=x.device)
    act, wt = c_int(dtype_code(x.dtype)), c_int(dtype_code(gate_w.dtype))
    _check(lib, lib.qil_moe_group(_p(chosen), c_int(pairs), c_int(experts), _p(sorted_pairs), _p(info), _p(tiles),
                                  c_int(max_tiles), _stream()), "moe_group", kernels=1 if pairs <= lib.qil_moe_one_block_pairs() else 2)
    _check(lib, lib.qil_moe_gate_up(_p(x), c_int(width), _p(gate_w), _p(up_w), _p(tiles), _p(info), c_int(max_tiles),
                                    _p(sorted_pairs), c_int(top), _p(hidden), c_int(ff), c_int(width),
                                    c_int(ACTIVATIONS[kind]), c_float(limit), c_float(alpha), act, wt, _stream()),
           "moe_gate_up")
    _check(lib, lib.qil_moe_down(_p(hidden), _p(down_w), _p(tiles), _p(info), c_int(max_tiles), _p(sorted_pairs),
                                 _p(weights), _p(y), c_int(width), c_int(ff), act, wt, _stream()), "moe_down")
    _check(lib, lib.qil_moe_combine(_p(y), _p(residual), _p(out), c_int(n), c_int(width), c_int(top),
                                    c_int(dtype_code(stream_dtype)), _p(chosen), _p(weights), _p(x if identity else None),
                                    c_int(dtype_code(x.dtype)), c_int(experts), _p(extra), _p(extra_gate), _p(col_scale),
                                    _stream()), "moe_combine")
    return out


def sample_rows(logits, temperature=None, seed=None, counter=None, tokens=None, nonfinite=None, state=None,
                owner=None):
    """Choose one token per row of float32 ``logits`` [R,V]; returns (tokens, nonfinite) int32 [R].

    Settings per row come from arrays: temperature float32 [R] (0 = greedy), seed and counter int64 [R], all
    optional (greedy); or from state slots: ``state`` int64 [slots, 4] = (the temperature's float32 bits,
    seed, draws so far, unused) per request and ``owner`` int32 [R], the slot of each row.  With slots
    the kernel adds one to the draws of every row's slot.
    """
    _need(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("seed", seed, torch.int64),
                        ("counter", counter, torch.int64), ("owner", owner, torch.int32)):
        if t is not None:
            _need(t, name, dt, 1)
            if t.shape[0] != rows:
                raise KernelError(f"sample_rows: {name} needs one entry per row")
    if state is not None:
        _need(state, "state", torch.int64, 2)
        if state.shape[1] != 4 or owner is None:
            raise KernelError("sample_rows: state slots are int64 [slots, 4] and need the rows' owners")
    if tokens is None:
        tokens = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if nonfinite is None:
        nonfinite = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = core()
    _check(lib, lib.qil_sample_rows(_p(logits), c_int(rows), c_int(vocab), c_longlong(logits.stride(0)),
                                    _p(temperature), _p(seed), _p(counter), _p(state), _p(owner), _p(tokens),
                                    _p(nonfinite), _stream()),
           "sample_rows")
    return tokens, nonfinite
