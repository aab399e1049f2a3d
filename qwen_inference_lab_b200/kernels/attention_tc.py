"""The tcgen05/TMA attention for whole 128-token query tiles (bfloat16, head size 128).

``prefill`` takes tiles of exactly 128 tokens; :func:`attention_mma.prefill` takes what is left.
The kernel's mbarrier waits are bounded and report through an error word that ``check()`` reads.
"""
from __future__ import annotations

from ctypes import c_float, c_int

import torch

from . import build
from . import ops
from .ops import KernelError, _check, _need, _p, _stream

HEAD_DIM = 128
TILE = 128
_lib = None
_fault = ops.ErrorWord(lambda code: f"attention_tc: a wait inside the kernel ran out (code {code}: 1x producer, "
                                    f"13-17 MMA issuer, 2x softmax warps)")


def library():
    global _lib
    if _lib is None:
        _lib = build.load("qil_attn_tc", ["attention_tc.cu"])
        ops.register_post_step_check(check)
        if _lib.qil_attn_tc_head_dim() != HEAD_DIM:
            raise KernelError("attention_tc was built for another head size")
    return _lib


def supports(head_dim, page_size, window) -> bool:
    return head_dim == HEAD_DIM and window == 0 and page_size in (8, 16, 32, 64)


def takes(options) -> bool:
    """Of the score options (``attention_mma.ScoreOptions``) this kernel has the cap, chunks and a learned sink."""
    return options.distance_bias is None and (not options.sink or options.sink_logits is not None)


def prefill(q, pages, out, tile_info, n_tiles, block_table, n_q_heads, n_kv_heads, page_size, scale, trace=None,
            lib=None, slopes_log2=None, chunk=0, sink_log2=None, softcap=0.0):
    """q, out bfloat16 [N, Hq*128]; pages [num_pages, 2, Hkv, page_size, 128];
    tile_info int32 [n_tiles * 4] = (first token, its position, 128, block-table row).
    ``slopes_log2`` float32 [Hq] on the device: slope_h * log2(e) of a bias slope_h * (query position - key
    position) taken off the scaled score.  ``chunk`` > 0: a query sees the keys of its own chunk of that many
    positions only.  ``sink_log2`` float32 [Hq] on the device: learned scores times log2(e) whose exponentials join
    the softmax's denominator.  ``softcap`` > 0: score <- cap * tanh(score / cap) on the scaled product."""
    if sink_log2 is not None:
        _need(sink_log2, "sink_log2", torch.float32, 1)
        if sink_log2.shape[0] != n_q_heads:
            raise KernelError("attention_tc: one sink score per query head")
    if slopes_log2 is not None:
        _need(slopes_log2, "slopes_log2", torch.float32, 1)
        if slopes_log2.shape[0] != n_q_heads:
            raise KernelError("attention_tc: one slope per query head")
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2); _need(pages, "pages", torch.bfloat16, 5)
    if tuple(pages.shape[1:]) != (2, n_kv_heads, page_size, HEAD_DIM) or q.shape[1] != n_q_heads * HEAD_DIM:
        raise KernelError("attention_tc: shapes do not match the head counts")
    lib = lib or library()
    word = _fault.tensor(q.device)
    _fault.mark()
    _check(lib, lib.qil_attn_tc_prefill_capped(
        _p(q), _p(pages), _p(out), _p(tile_info), c_int(n_tiles), c_int(q.shape[0]), _p(block_table),
        c_int(block_table.shape[1]), c_int(n_q_heads), c_int(n_kv_heads), c_int(page_size), c_int(pages.shape[0]),
        c_float(scale), _p(slopes_log2), c_int(int(chunk or 0)), _p(sink_log2), c_float(float(softcap or 0.0)), _p(word),
        _p(trace), _stream()),
        "attention (128-token tiles)")


def check(wait=True) -> None:
    """Raise if a bounded wait inside a launch ran out (see ``ops.ErrorWord.check``)."""
    _fault.check(wait)
