"""Larolorn on the GPU: every mechanism alone against its plain function, keys made to stand out at the edges of
windows and chunks and far away, then whole models under four ways of cutting the work, long decoding, slots and
pages used again, generation through the engine, the replay program and the command line."""
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import harness
from tests import larolorn_cases as cases
from tests.plain import larolorn_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["float32", "bfloat16"]
F64 = torch.float64


def low_of(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


def close(actual, expected, dtype, scale=1.0):
    """float32: element by element.  bfloat16: the expected rows carry the plain implementation's own bfloat16
    roundings, and the engine rounds at other points, so the bar is on the root mean square of the difference
    (1.5 % of the rows' own) and on the largest one (6 % of the largest value)."""
    actual, expected = actual.float().cpu(), expected.float()
    assert torch.isfinite(actual).all()
    if dtype == torch.float32:
        torch.testing.assert_close(actual, expected, atol=3e-5 * scale, rtol=3e-5)
        return
    difference = actual - expected
    assert difference.pow(2).mean().sqrt() <= 0.015 * expected.pow(2).mean().sqrt() + 1e-6, \
        f"rms difference {difference.pow(2).mean().sqrt():.3e} against rows of {expected.pow(2).mean().sqrt():.3e}"
    assert difference.abs().max() <= 0.06 * expected.abs().max() + 1e-6, \
        f"largest difference {difference.abs().max():.3e} against a largest value of {expected.abs().max():.3e}"


def fill(part, seed, dtype, values=None):
    """Random parameters (``cases.draw_weights``) or the given ones; returns name -> CPU float32."""
    drawn = cases.draw_weights(part.all_named_params(), seed)
    drawn.update(values or {})
    for name, param in part.all_named_params().items():
        drawn[name] = drawn[name].to(torch.bfloat16).float()
        param.data = drawn[name].to(dtype).cuda()
    part.finalize(torch.device("cuda"), dtype)
    return drawn


def rows(count, width, seed, scale=1.0):
    return (torch.randn(count, width, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16).float()


class Ctx:
    """The little of a step's context that parts without a cache read."""
    def __init__(self, dtype):
        self.dtype, self.device, self.stream_dtype = dtype, torch.device("cuda"), torch.float32

    def empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# ------------------------------------------------------------------ mechanisms without a cache
@pytest.mark.parametrize("width", [70, 96, 1000, 4100])
def test_a_normed_branch_joins_the_stream(width):
    """x += m * rms(a) * w on a float32 stream, and the two-branch form with the side-by-side mixers' own norms."""
    from qwen_inference_lab_b200.kernels import ops
    stream, a, b = rows(5, width, 1, 4.0), rows(5, width, 2, 3.0), rows(5, width, 3, 0.02)
    w, wa, wb = (1 + 0.1 * rows(1, width, 4 + i)[0] for i in range(3))
    for eps in (1e-6, 0.5):
        out = ops.rms_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, 0.3)
        torch.testing.assert_close(out.cpu(), (stream.double() + 0.3 * plain.rms_norm(a.double(), w, eps)).float(), atol=1e-5, rtol=1e-6)
        out = ops.rms_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, 0.3, b=b.cuda(), weight_a=wa.cuda(), weight_b=wb.cuda(), pre=0.5)
        y = 0.5 * (plain.rms_norm(a.double(), wa, eps) + plain.rms_norm(b.double(), wb, eps))
        torch.testing.assert_close(out.cpu(), (stream.double() + 0.3 * plain.rms_norm(y, w, eps)).float(), atol=1e-5, rtol=1e-6)
        # the rounded copy for the next product is the new stream rounded once, bit for bit, from either form
        for two in (False, True):
            copy = torch.full((5, width), float("nan"), dtype=torch.bfloat16, device="cuda")
            more = dict(b=b.cuda(), weight_a=wa.cuda(), weight_b=wb.cuda(), pre=0.5) if two else {}
            again = ops.rms_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, 0.3, rows=copy, **more)
            assert torch.equal(copy, again.to(torch.bfloat16))
            assert two or torch.equal(again, ops.rms_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, 0.3))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,width,ff,limit", [(1, 96, 72, 3.0), (9, 70, 37, 0.5), (300, 64, 48, 7.0)])
def test_clamped_feed_forward(dtype, n, width, ff, limit):
    """Inputs large enough that the gate passes its upper bound and the other branch both of its bounds."""
    from qwen_inference_lab_b200.parts import GatedMLP
    part = GatedMLP(width, ff, names=dict(gate="f.gate", up="f.up", down="f.down"), activation="clamped_swish", limit=limit,
                    alpha=1.702, suffixes=("", ".b"))
    w = fill(part, 3, dtype)
    x = rows(n, width, 4, 2.5)
    gate = x.double() @ w["f.gate"].double().t()
    assert (gate > limit).any() and (gate < -limit).any()
    expected = plain.clamped_feed_forward(x.double(), w, "f.", dict(limit=limit), low_of(dtype))
    out = part.forward(Ctx(dtype), x.to(dtype).cuda(), out_float32=True)
    assert out.dtype == torch.float32
    close(out, expected, dtype, scale=float(expected.abs().max()))


@pytest.mark.parametrize("layout", ["halves", "interleaved"])
@pytest.mark.parametrize("dims,head", [(16, 16), (4, 20), (2, 6), (80, 80)])
def test_rotation_from_frequencies_in_float32(layout, dims, head):
    """The rotation kernel alone, float32, positions up to a million: float32 angles as the design computes them."""
    from qwen_inference_lab_b200.kernels import ops
    from qwen_inference_lab_b200.parts import RotaryFrequencies
    rotation = RotaryFrequencies(dims, 5000.0, layout)
    rotation.finalize(torch.device("cuda"), torch.float32)
    heads, n = 3, 6
    positions = [0, 1, 17, 4095, 70001, 999999]
    x = rows(n, heads * head, 5)
    q = torch.empty(n, heads * head, device="cuda")
    # no key/value heads: the kernel rotates the queries and touches no page
    ops.qk_rotate_store(x.cuda(), (0, heads * head, heads * head), q, None, None, None, 0.0, rotation.freq, dims, rotation.layout,
                        torch.tensor(positions, dtype=torch.int32, device="cuda"), torch.arange(n, dtype=torch.int32, device="cuda"),
                        None, heads, 0, head, head, 4)
    rot = dict(base=5000.0, dims=dims)
    for i, p in enumerate(positions):
        expected = _at_position(x[i].view(1, heads, head), p, rot, layout)
        torch.testing.assert_close(q[i].cpu().view(heads, head), expected[0], atol=2e-6, rtol=1e-5)
    # the plain functions count positions from the sequence's start: the first rows agree with them too
    short = rows(4, heads * head, 6)
    ops.qk_rotate_store(short.cuda(), (0, heads * head, heads * head), q[:4], None, None, None, 0.0, rotation.freq, dims,
                        rotation.layout, torch.arange(4, dtype=torch.int32, device="cuda"),
                        torch.zeros(4, dtype=torch.int32, device="cuda"), None, heads, 0, head, head, 4)
    turn = plain.rotate_halves if layout == "halves" else plain.rotate_interleaved
    torch.testing.assert_close(q[:4].cpu().view(4, heads, head), turn(short.view(4, heads, head), rot), atol=2e-6, rtol=1e-5)


def _at_position(x, position, rot, layout):
    """x [1, H, n] rotated as the token at ``position``: float32 angles position * f_i, cos and sin in float64."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).float()
    a = (torch.tensor(float(position), dtype=torch.float32) * f).double()
    cos, sin = a.cos(), a.sin()
    out = x.double().clone()
    if layout == "halves":
        u, v = x[..., :dims // 2].double(), x[..., dims // 2:dims].double()
        out[..., :dims // 2], out[..., dims // 2:dims] = u * cos - v * sin, v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2].double(), x[..., 1:dims:2].double()
        out[..., 0:dims:2], out[..., 1:dims:2] = u * cos - v * sin, v * cos + u * sin
    return out.float()


# ------------------------------------------------------------------ the mixers alone, through the step function
SUFFIX = ("", ".b")


def latent_part(hidden, m, eps=1e-5):
    from qwen_inference_lab_b200.parts import LatentAttention, RotaryFrequencies
    names = {k: "m." + k for k in ("q", "dkv", "uk", "uv", "g", "o")}
    names["dkv_norm"] = "m.dkv.norm"
    return LatentAttention(hidden, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], scale=m["scale"],
                           window=m["mask"]["size"], position=RotaryFrequencies(m["rot"]["dims"], m["rot"]["base"], "interleaved"),
                           norm_eps=eps, names=names, suffixes=SUFFIX, norm_suffix="")


def left_part(hidden, m, eps=1e-5, prefix="m."):
    from qwen_inference_lab_b200.parts import GroupedQueryAttention, RotaryFrequencies
    names = {k: prefix + k for k in ("q", "k", "v", "o", "sink")}
    names.update(q_norm=prefix + "q.norm", k_norm=prefix + "k.norm")
    return GroupedQueryAttention(hidden, m["heads"], m["kv_heads"], m["dim"], names=names, bias=True, scale=m["scale"],
                                 v_head_dim=m["vdim"], suffixes=SUFFIX, chunk=m["mask"]["size"], sink="learned",
                                 position=RotaryFrequencies(m["rot"]["dims"], m["rot"]["base"], "halves"),
                                 whole_qk_norm_eps=eps, norm_suffix="")


def right_part(hidden, m, eps=1e-5, prefix="m."):
    from qwen_inference_lab_b200.parts import DecayLinearAttention
    names = {k: prefix + k for k in ("q", "k", "v", "g", "o", "norm")}
    return DecayLinearAttention(hidden, m["heads"], m["dim"], m["vdim"], m["decay"], norm_eps=eps, names=names, suffixes=SUFFIX,
                                norm_suffix="")


def through_the_step_function(part, hidden, dtype, inputs, cuts, page_size=4, num_pages=64):
    body = lambda ctx, x, view: part.forward(ctx, x, view, out_float32=True)
    return harness.run_part(part, hidden, dtype, body, inputs, cuts, page_size=page_size, num_pages=num_pages)


CUTS = ({"a": [75], "b": [41]}, {"a": [3, 1, 1, 2, 30, 1, 5, 2, 30], "b": [1] * 9 + [2] * 6 + [20]}, {"a": [1] * 75, "b": [17, 24]})

LATENTS = [cases.latent(3, 24, 8, 40, 24, 0.17, 10000.0, 20),      # key rows of 32: the tensor-core kernels in bfloat16
           cases.latent(5, 12, 4, 20, 10, 0.25, 2000.0, 1),        # rows of 14: the float32 kernel; a token sees itself
           cases.latent(1, 6, 2, 10, 30, 0.4, 7.0, 4096),          # one head, one rotated pair, no window in reach
           cases.latent(2, 16, 16, 16, 48, 0.18, 100.0, 33),       # rows of 64
           cases.latent(4, 40, 24, 8, 72, 0.1, 1e6, 5),            # rows of 96, values smaller than keys, a window of five
           cases.latent(3, 48, 32, 56, 128, 0.09, 50000.0, 40),    # rows of 160
           cases.latent(2, 128, 64, 128, 192, 0.07, 10000.0, 70)]  # rows of 256, the widest the tensor-core kernels take


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m", LATENTS, ids=[f"row{m['kv_rank'] + m['rot_dim']}" for m in LATENTS])
def test_latent_attention_whole_cut_and_side_by_side(dtype, m):
    """The mixer over whole sequences, over portions down to one and two tokens, and with two requests in every
    step, against the plain mixer that writes every head's keys and values out."""
    part = latent_part(88, m)
    w = fill(part, 11, dtype)
    inputs = {"a": rows(75, 88, 12), "b": rows(41, 88, 13)}
    expected = {rid: plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    for cuts in CUTS:
        got = through_the_step_function(part, 88, dtype, inputs, cuts, num_pages=48)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


LEFTS = [cases.left(4, 2, 32, 32, 0.2, 300000.0, 16, 24),          # the tensor-core kernels in bfloat16; half a head rotated
         cases.left(6, 3, 16, 8, 0.3, 1000.0, 16, 7),              # values smaller than keys: the float32 kernel
         cases.left(3, 3, 20, 12, 0.22, 50.0, 4, 1),               # a chunk of one position: a token and the sink
         cases.left(2, 1, 80, 80, 0.11, 500.0, 80, 4096),          # one key/value head, no chunk edge in reach
         cases.left(6, 1, 16, 16, 0.25, 10000.0, 2, 33),           # six query heads on one key/value head, one rotated pair
         cases.left(8, 2, 128, 128, 0.08, 500000.0, 64, 50),       # heads of 128, half of each rotated
         cases.left(4, 4, 48, 48, 0.15, 20000.0, 48, 19)]          # heads of 48, as many key/value heads as query heads


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m", LEFTS, ids=[f"d{m['dim']}c{m['mask']['size']}" for m in LEFTS])
def test_chunked_attention_with_whole_norms_and_sinks_whole_cut_and_side_by_side(dtype, m):
    part = left_part(72, m)
    w = fill(part, 21, dtype)
    inputs = {"a": rows(75, 72, 22), "b": rows(41, 72, 23)}
    expected = {rid: plain.chunk_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    for cuts in CUTS:
        got = through_the_step_function(part, 72, dtype, inputs, cuts, num_pages=48)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


@pytest.mark.parametrize("chunk", [50, 128, 200, 4096])
def test_whole_tiles_of_heads_of_128_take_the_tensor_memory_kernel_with_chunks_and_sinks(monkeypatch, chunk):
    """Whole 128-token tiles of a prompt go to the tcgen05 kernel, which starts at the chunk of a tile's first row and
    masks, row by row, what lies before a later row's chunk (chunk edges inside a tile, at a tile's edge, one edge in
    the prompt, none); the sink's score joins every row's denominator.  Leftovers and single tokens take the tiled
    kernels."""
    from qwen_inference_lab_b200.kernels import attention_tc
    calls = []
    original = attention_tc.prefill
    monkeypatch.setattr(attention_tc, "prefill",
                        lambda *a, **k: (calls.append((k.get("chunk"), k.get("sink_log2") is not None)), original(*a, **k))[1])
    m = cases.left(4, 2, 128, 128, 0.09, 10000.0, 128, chunk)
    part = left_part(64, m)
    w = fill(part, 31, torch.bfloat16)
    inputs = {"a": rows(330, 64, 32), "b": rows(140, 64, 33)}
    expected = {rid: plain.chunk_attention_mixer(x.double(), w, "m.", m, 1e-5, torch.bfloat16) for rid, x in inputs.items()}
    for cuts in ({"a": [330], "b": [140]}, {"a": [129, 1, 200], "b": [7, 133]}):
        got = through_the_step_function(part, 64, torch.bfloat16, inputs, cuts, page_size=16, num_pages=40)
        for rid in inputs:
            close(got[rid], expected[rid], torch.bfloat16)
    assert calls and all(call == (chunk, True) for call in calls)


def test_the_sink_takes_its_share_and_is_not_scaled():
    """All projections zero but the values' bias: every key scores zero, so a token n positions into its chunk gets
    n / (n + e^sink) of the value (sink about log 2), whatever the scale says."""
    m = cases.left(2, 1, 16, 16, 37.0, 100.0, 16, 6)
    part = left_part(24, m)
    zero = {name: torch.zeros(p.shape) for name, p in part.all_named_params().items() if name.split(".")[-1] not in ("norm",)}
    zero["m.v.b"] = torch.ones(16)
    zero["m.o"] = torch.eye(24, 32)
    sink = float(torch.tensor(math.log(2.0)).to(torch.bfloat16))            # what the checkpoint can hold
    zero["m.sink"] = torch.tensor([sink, -30.0])
    fill(part, 1, torch.float32, zero)
    got = through_the_step_function(part, 24, torch.float32, {"a": rows(15, 24, 3)}, {"a": [4, 1, 1, 9]})["a"]
    for t in range(15):
        n = t % 6 + 1
        assert abs(float(got[t, 0]) - n / (n + math.exp(sink))) < 1e-6 and abs(float(got[t, 20]) - 1.0) < 1e-6


RIGHTS = [cases.right(2, 16, 24, (0.9, 0.5)), cases.right(3, 40, 8, (1.0, 0.0, 0.97)), cases.right(1, 64, 64, (0.99,)),
          cases.right(5, 10, 6, (0.3, 0.999, 0.8, 1.0, 0.61)), cases.right(2, 128, 32, (0.95, 0.999))]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m", RIGHTS, ids=[f"h{m['heads']}d{m['dim']}" for m in RIGHTS])
def test_decayed_linear_attention_whole_cut_and_side_by_side(dtype, m):
    """Short portions run token by token, portions of more than 128 tokens as chunks with a carry: the state a
    portion leaves is what the next one starts from, whichever way each ran.  A decay of one forgets nothing (a lost
    state shows at once), a decay of zero keeps the current token only."""
    part = right_part(56, m)
    w = fill(part, 31, dtype)
    inputs = {"a": rows(300, 56, 32), "b": rows(41, 56, 33)}
    expected = {rid: plain.decay_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    for cuts in ({"a": [300], "b": [41]}, {"a": [2, 129, 1, 1, 64, 3, 100], "b": [1] * 9 + [2] * 6 + [20]},
                 {"a": [150, 150], "b": [17, 24]}, {"a": [1] * 40 + [260], "b": [41]}):
        got = through_the_step_function(part, 56, dtype, inputs, cuts, page_size=16, num_pages=24)
        for rid in inputs:
            close(got[rid], expected[rid], dtype, scale=float(expected[rid].abs().max()))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_two_mixers_side_by_side(dtype):
    """Half the sum of the two normed outputs; one output is made a thousand times the other's size, which the
    norms must undo."""
    from qwen_inference_lab_b200.parts import ParallelMixers
    ml, mr = cases.left(4, 2, 32, 32, 0.2, 300000.0, 16, 24), cases.right(3, 24, 8, (1.0, 0.5, 0.97))
    part = ParallelMixers(80, left_part(80, ml, prefix="m.left."), right_part(80, mr, prefix="m.right."), norm_eps=1e-5,
                          share=0.5, norm_suffix="", names=dict(left_out="m.left.out", right_out="m.right.out"))
    drawn = cases.draw_weights(part.all_named_params(), 41)
    w = fill(part, 41, dtype, {"m.right.o": drawn["m.right.o"] * 1024.0})
    inputs = {"a": rows(75, 80, 42), "b": rows(41, 80, 43)}
    expected = {rid: plain.parallel_mixer(x.double(), w, "m.", dict(left=ml, right=mr), 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    body = lambda ctx, x, view: part.forward(ctx, x, view)
    for cuts in CUTS:
        got = harness.run_part(part, 80, dtype, body, inputs, cuts, page_size=4, num_pages=48)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


# ------------------------------------------------------------------ one key made to stand out
def _run_with_the_query_last(part, hidden, dtype, x, query, single, page_size=8):
    """The rows up to ``query`` through the step function; the query comes as a single token or as the last of a
    five-token portion, behind one large portion and a two-token one."""
    tail = 1 if single else min(5, query + 1)
    head = query + 1 - tail
    cuts = ([head - 2, 2] if head > 3 else [head] if head else []) + [tail]
    pages = (query + 1) // page_size + 3
    return through_the_step_function(part, hidden, dtype, {"a": x[:query + 1]}, {"a": cuts}, page_size=page_size, num_pages=pages)["a"]


WINDOW_EDGES = [(64, 127, 64, True), (64, 128, 64, False), (20, 19, 0, True), (20, 20, 0, False), (100, 200, 101, True),
                (100, 200, 100, False), (600, 650, 51, True), (600, 651, 51, False), (1, 9, 9, None), (1, 9, 8, False),
                (33, 64, 32, True), (33, 65, 32, False), (4096, 500, 0, True)]


def _judge_the_query(got, expected, exact, alone, query, inside, dtype):
    """The portion's last rows against the plain mixer; the query's row against the far token's value alone."""
    assert inside is None or ((exact[query] - alone).abs().max() < 1e-6 * alone.abs().max()) == inside, \
        "the far key does not stand out as the test wants"
    count = min(5, query + 1)
    close(got[-count:], expected[query + 1 - count:query + 1], dtype)
    if inside:
        close(got[-1], alone, dtype)
    elif inside is False:
        assert (got[-1].double() - alone).abs().max() > 0.02 * alone.abs().max()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query,far,inside", WINDOW_EDGES)
def test_a_key_just_inside_and_just_outside_the_window(dtype, single, window, query, far, inside):
    """The far token's input is eight times the others', so its rotated key part (which no norm touches) is the
    largest by far.  The query's input is solved for: no plain part, a rotated part that, turned at the query's
    position, points along the far token's turned key part (score 80, every other key at most some 15), a rotated
    key part of its own of zero and a gate of one half.  Just inside the window every head's output is then the far
    token's value alone; one position further that token is not seen at all.  The rotation has to hold over the
    distance: a wrong angle or position loses the key."""
    hidden = 96
    m = cases.latent(2, 24, 8, 16, 24, 0.2, 10000.0, window)
    H, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    part = latent_part(hidden, m)
    w = fill(part, 51, dtype)
    W = {k: v.double() for k, v in w.items()}
    x = rows(query + 1, hidden, 52 + query, 0.5)
    if far != query:
        x[far] *= 8.0
        shared = x[far].double() @ W["m.dkv"][c:].t()                              # the far token's key part, not yet turned
        freq = torch.tensor([m["rot"]["base"] ** (-2.0 * i / r) for i in range(r // 2)], dtype=F64)
        pairs = torch.view_as_complex(shared.view(r // 2, 2).contiguous()) * torch.exp(1j * (far - query) * freq)
        q_rot = torch.view_as_real(pairs).flatten() * (80.0 / (float(shared @ shared) * m["scale"]))
        target = torch.cat([torch.zeros(H, d, dtype=F64), q_rot.expand(H, r)], dim=1).flatten()
        system = torch.cat([W["m.q"], W["m.dkv"][c:], W["m.g"]])
        x[query] = (torch.linalg.pinv(system) @ torch.cat([target, torch.zeros(r + H, dtype=F64)])).to(torch.bfloat16).float()
    expected = plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype))
    exact = plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5)
    z_far = plain.rms_norm((x[far].double() @ W["m.dkv"].t())[:c], W["m.dkv.norm"], 1e-5)
    gate = torch.sigmoid(x[query].double() @ W["m.g"].t())
    alone = ((W["m.uv"] @ z_far).view(H, e) * gate[:, None]).flatten() @ W["m.o"].t()
    got = _run_with_the_query_last(part, hidden, dtype, x, query, single)
    _judge_the_query(got, expected, exact, alone, query, inside, dtype)


CHUNK_EDGES = [(64, 127, 64, True), (64, 128, 127, False), (64, 128, 64, False), (24, 47, 24, True), (24, 48, 47, False),
               (7, 13, 7, True), (7, 14, 13, False), (1024, 700, 3, True), (300, 599, 300, True), (300, 600, 599, False),
               (1, 5, 5, None), (1, 5, 4, False), (33, 65, 33, True), (33, 66, 65, False)]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk,query,far,inside", CHUNK_EDGES)
def test_a_key_just_inside_and_just_outside_the_chunk(dtype, single, chunk, query, far, inside):
    """The same for the chunked attention: the query's input is solved for so that, after the norm over the whole
    projection, every head's query points along the far token's normed key of its group (q and k are normed, so a
    key stands out by its direction only: the far token's input is drawn again until its score leads every other
    key of the sequence by 30 in every head).  Seen from the far token's own chunk the output is that token's value;
    from the first position of the next chunk it is not seen, however close it is.  Chunks that are over have given
    their pages back by then."""
    hidden = 160
    m = cases.left(4, 2, 32, 32, 3.0, 10000.0, 4, chunk)
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    part = left_part(hidden, m)
    w = fill(part, 61, dtype)
    W = {k: v.double() for k, v in w.items()}
    x = rows(query + 1, hidden, 62 + query, 0.5)
    normed_keys = lambda t: plain.rms_norm(t.double() @ W["m.k"].t() + W["m.k.b"], W["m.k.norm"], 1e-5).view(-1, G, d)
    for attempt in range(40):
        if far == query:
            break
        x[far] = rows(1, hidden, 1000 + attempt, 0.5)[0]
        k_far = normed_keys(x[far:far + 1])[0]
        target = torch.stack([k_far[a // (H // G)] / k_far[a // (H // G)].norm() for a in range(H)]).flatten() / W["m.q.norm"]
        x[query] = (torch.linalg.pinv(W["m.q"]) @ (target - W["m.q.b"])).to(torch.bfloat16).float()
        q = plain.rms_norm(x.double() @ W["m.q"].t() + W["m.q.b"], W["m.q.norm"], 1e-5).view(-1, H, d)
        turned_q, turned_k = plain.rotate_halves(q, m["rot"])[query], plain.rotate_halves(normed_keys(x), m["rot"])
        scores = torch.stack([turned_k[:, a // (H // G)] @ turned_q[a] for a in range(H)]) * m["scale"]      # [H, T]
        others = torch.cat([scores[:, :far], scores[:, far + 1:]], dim=1)
        if float((scores[:, far] - others.max(dim=1).values).min()) > 30.0:
            break
    else:
        raise AssertionError("no input found whose key stands out")
    expected = plain.chunk_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype))
    exact = plain.chunk_attention_mixer(x.double(), w, "m.", m, 1e-5)
    v_far = (x[far].double() @ W["m.v"].t() + W["m.v.b"]).view(G, e)
    alone = torch.stack([v_far[a // (H // G)] for a in range(H)]).flatten() @ W["m.o"].t() + W["m.o.b"]
    got = _run_with_the_query_last(part, hidden, dtype, x, query, single)
    _judge_the_query(got, expected, exact, alone, query, inside, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
def test_the_state_remembers_a_token_from_far_back(dtype, single):
    """A head that forgets nothing (decay one) beside one that forgets fast: token 2 has the only large key and value, the
    query 600 positions later asks for it.  The first head's output is then that value times the match, the second
    head's is next to nothing."""
    hidden, query = 64, 602
    m = cases.right(2, 16, 8, (1.0, 0.5))
    part = right_part(hidden, m)
    w = fill(part, 71, dtype)
    x = rows(query + 1, hidden, 72, 0.05)
    x[2] = rows(1, hidden, 73, 6.0)[0]
    x[query] = x[2]
    expected = plain.decay_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype))
    lost = x.clone(); lost[2] = x[3]
    without = plain.decay_mixer(lost.double(), w, "m.", m, 1e-5)
    assert (expected[query].double() - without[query]).abs().max() > 0.1 * expected[query].abs().max()
    tail = 1 if single else 5
    cuts = [130, 2, 200, 1, query + 1 - 333 - tail, tail]
    got = through_the_step_function(part, hidden, dtype, {"a": x}, {"a": cuts}, page_size=16, num_pages=40)["a"]
    close(got[-5:], expected[-5:], dtype, scale=float(expected.abs().max()))


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    result = {}
    for name, case in cases.CASES.items():
        folder = tmp_path_factory.mktemp(f"larolorn{name}")
        weights = cases.write_folder(case["config"], case["seed"], folder)
        requests = {f"r{i}": cases.random_tokens(case["config"], n, 60 + i) for i, n in enumerate(case["lengths"])}
        result[name] = (folder, weights, requests)
    return result


@pytest.fixture(scope="module")
def truth(folders):
    """The plain rows of every case, in float64 and with bfloat16 roundings: computed once."""
    return {name: (cases.plain_rows(requests, weights, cases.CASES[name]["config"]),
                   cases.plain_rows(requests, weights, cases.CASES[name]["config"], torch.bfloat16))
            for name, (folder, weights, requests) in folders.items()}


def judge(actual, expected, low, dtype, what):
    """float32: every row, element by element, against the float64 rows (1e-4 of the largest logit: what float32 sums
    of this depth cost).

    bfloat16: the yardstick is what bfloat16 costs the plain implementation itself (``low``).  The mean row error
    may be 1.5 times the yardstick's; no row's largest error may pass twice the yardstick's largest; a row's own
    error may be 1.5 times the yardstick's in that row or 2.25 times its mean, which one row in twenty-five may
    pass, by a factor of two at most (branches normed by their own root mean square make single rows sensitive,
    and the engine does not round where the plain code does); and wherever the float64 row's best logit leads by
    four times the yardstick's largest error in that row, the engine's best token is the same."""
    assert set(actual) == set(expected), f"{what}: different (request, position) sets"
    keys = sorted(expected)
    assert all(torch.isfinite(actual[k]).all() for k in keys), f"{what}: non-finite logits"
    if dtype == torch.float32:
        bar = 1e-4 * max(float(expected[k].abs().max()) for k in keys)
        bad = [k for k in keys if not torch.allclose(actual[k], expected[k], atol=bar, rtol=1e-5)]
        assert not bad, f"{what}: {len(bad)} rows differ, first {bad[0]} by {(actual[bad[0]] - expected[bad[0]]).abs().max():.3e}"
        return
    rms = lambda rows_, k: (rows_[k] - expected[k]).pow(2).mean().sqrt().item()
    peak = lambda rows_, k: (rows_[k] - expected[k]).abs().max().item()
    mean_bar = 1.5 * sum(rms(low, k) for k in keys) / len(keys)
    peak_bar = 2.0 * max(peak(low, k) for k in keys)
    mean_rms = sum(rms(actual, k) for k in keys) / len(keys)
    assert mean_rms <= mean_bar, f"{what}: mean row error {mean_rms:.3e} against a bar of {mean_bar:.3e}"
    worst = max(keys, key=lambda k: peak(actual, k))
    assert peak(actual, worst) <= peak_bar, f"{what}: row {worst} is off by {peak(actual, worst):.3e}, the bar is {peak_bar:.3e}"
    row_bar = lambda k: max(1.5 * mean_bar, 1.5 * rms(low, k))
    over = [k for k in keys if rms(actual, k) > row_bar(k)]
    assert len(over) <= max(1, len(keys) // 25) and all(rms(actual, k) <= 2 * row_bar(k) for k in over), \
        f"{what}: {len(over)} of {len(keys)} rows are further off than their bar, first {over[0]}: " \
        f"{rms(actual, over[0]):.3e} against {row_bar(over[0]):.3e}"
    judged = 0
    for k in keys:
        best = expected[k].topk(2).values
        if (best[0] - best[1]).item() > 4 * peak(low, k):
            judged += 1
            assert actual[k].argmax().item() == expected[k].argmax().item(), f"{what}: another best token at {k}"
    assert judged > len(keys) // 4, f"{what}: only {judged} of {len(keys)} rows have a clear best token; use other weights"


SCHEDULES = {"whole": harness.whole_schedule, "tail_decode": harness.tail_decode_schedule,
             "chunks": harness.chunk_schedule, "mixed": harness.mixed_schedule}


def peak_live_pages(schedule, model, page_size):
    """The most pages of any group the schedule holds at once when windows that have passed and chunks that are
    over give their pages back: found by walking the schedule through a cache manager on the CPU."""
    from qwen_inference_lab_b200.cache import CacheManager
    cache = CacheManager(model.cache_specs(), num_pages=4096, page_size=page_size, max_requests=8, max_context=1 << 20,
                         dtype=torch.float32, device="cpu")
    peak = 0
    for entries, ended in schedule:
        for rid, tokens, _ in entries:
            if rid not in cache.rows:
                assert cache.admit(rid)
            cache.ensure(rid, cache.written(rid) + len(tokens))
        peak = max(peak, max(g.capacity - len(g.free) for g in cache.kv_groups))
        for rid, tokens, _ in entries:
            cache.advance(rid, cache.written(rid) + len(tokens))
        for rid in ended:
            cache.release(rid)
    return peak


def replay(folders, case, schedule_name, dtype):
    folder, weights, requests = folders[case]
    page_size = cases.CASES[case]["page_size"]
    schedule = SCHEDULES[schedule_name](requests)
    from qwen_inference_lab_b200.config import registry
    entry = registry.lookup(cases.CASES[case]["config"])
    shell = entry.build(entry.config_class.from_dict(cases.CASES[case]["config"]))
    num_pages = peak_live_pages(schedule, shell, page_size) + 1
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    for _, _, tensor in cache.state_groups:
        tensor.fill_(float("nan"))             # a slot that is not zeroed at admission shows
    ledger = harness.PageLedger(cache)
    actual = harness.run_schedule(runner, cache, schedule, ledger)
    assert cache.free_pages() == num_pages and not cache.owners()
    assert ledger.handovers > 0, "no page was used again by another request: the pool is too large"
    return actual


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("case", list(cases.CASES))
def test_replay_matches_plain(folders, truth, case, schedule, dtype):
    actual = replay(folders, case, schedule, dtype)
    expected, low = truth[case]
    judge(actual, expected, low, dtype, f"larolorn {case} {schedule} {dtype}")


@pytest.mark.parametrize("case", list(cases.CASES))
def test_float32_rows_agree_under_every_schedule(folders, case):
    """Portions of up to 128 tokens and single tokens walk the recurrent state token by token, attention walks key
    tiles aligned to positions and float32 products sum in ascending order: such schedules give the same bits.  A
    longer portion's state comes through the chunked scan's carry, which rounds differently in the last bits."""
    runs = {name: replay(folders, case, name, torch.float32) for name in SCHEDULES}
    longest = max(cases.CASES[case]["lengths"])
    for name, got in runs.items():
        if longest <= 128:
            different = [key for key in sorted(got) if not torch.equal(got[key], runs["chunks"][key])]
        else:
            different = [key for key in sorted(got) if not torch.allclose(got[key], runs["chunks"][key], atol=2e-5, rtol=1e-5)]
        assert not different, \
            f"larolorn {case}: {len(different)} rows of schedule {name} differ from the run in portions, first {different[0]}"
    for name in ("tail_decode", "mixed"):
        short = [key for key in sorted(runs[name]) if len(folders[case][2][key[0]]) <= 128]
        assert all(torch.equal(runs[name][key], runs["chunks"][key]) for key in short)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("case", ["A", "B"])
def test_long_decoding_and_the_first_tokens(folders, dtype, case):
    """Three tokens as a prompt, then 300 single tokens (recorded graphs) across many window and chunk edges, every
    position judged; the pool holds fewer pages than the positions need, because windows that have passed and chunks
    that are over give theirs back."""
    folder, weights, _ = folders[case]
    config, page_size = cases.CASES[case]["config"], cases.CASES[case]["page_size"]
    tokens = cases.random_tokens(config, 303, 99)
    schedule = [([("r", tokens[:3], [0, 1, 2])], [])]
    schedule += [([("r", [tokens[i]], [0])], ["r"] if i == 302 else []) for i in range(3, 303)]
    num_pages = {"A": 10, "B": 303 // page_size + 2}[case]       # case B's chunk is longer than the request: it keeps all
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = cases.plain_rows({"r": tokens}, weights, config)
    low = cases.plain_rows({"r": tokens}, weights, config, torch.bfloat16) if dtype == torch.bfloat16 else None
    judge(actual, expected, low, dtype, f"larolorn {case} long decoding {dtype}")


def test_a_state_slot_and_pages_that_another_request_used_before(folders):
    """"x" runs and ends; "y" takes its slot and its pages: its logits are those of "y" in a fresh cache, bit for bit."""
    folder, weights, _ = folders["A"]
    config = cases.CASE_A
    x, y = cases.random_tokens(config, 37, 1), cases.random_tokens(config, 29, 2)
    def run(first):
        _, cache, runner = harness.build_engine_parts(folder, torch.float32, num_pages=12, page_size=4, max_requests=1)
        schedule = []
        if first:
            schedule += [([("x", x[:30], [])], [])] + [([("x", [t], [0])], []) for t in x[30:]]
            schedule[-1] = (schedule[-1][0], ["x"])
        schedule += [([("y", y[:11], list(range(11)))], []), ([("y", y[11:13], [0, 1])], [])]
        schedule += [([("y", [t], [0])], []) for t in y[13:]]
        schedule[-1] = (schedule[-1][0], ["y"])
        got = harness.run_schedule(runner, cache, schedule)
        return torch.stack([got[("y", p)] for p in range(len(y))])
    assert torch.equal(run(first=True), run(first=False))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_engine(folders, dtype):
    """Prompts of unequal length through ``Engine.generate`` (scheduler, chunked prompts, sampler): every token is
    the plain implementation's best one, or in bfloat16 inside what bfloat16 costs the plain implementation."""
    from qwen_inference_lab_b200 import Engine, load_model
    folder, weights, _ = folders["A"]
    config = cases.CASE_A
    model = load_model(folder, device="cuda", dtype=dtype)
    engine = Engine(model, num_pages=48, page_size=4, token_budget=24, prefill_chunk=10, max_active=3)
    prompts = [cases.random_tokens(config, n, 40 + n) for n in (2, 31, 17, 5)]
    results = engine.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert engine.idle and engine.cache.free_pages() == 48
    for prompt, row in zip(prompts, results):
        assert len(row["token_ids"]) == 12
        sequence = list(prompt)
        for token in row["token_ids"]:
            logits = plain.forward(config, weights, sequence, torch.float32)[-1]
            best = int(logits.argmax())
            if token != best:
                assert dtype == torch.bfloat16, f"token {token} instead of {best} after {len(sequence)} tokens"
                noise = (plain.forward(config, weights, sequence, torch.float32, torch.bfloat16)[-1] - logits).abs().max().item()
                assert float(logits[best] - logits[token]) < 4 * noise
            sequence.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_runs_a_mixed_schedule(folders, truth, tmp_path, dtype):
    folder, weights, requests = folders["B"]
    schedule = harness.mixed_schedule(requests)
    peak = harness.peak_pages(schedule, 64, round_to=64) * 64
    process = subprocess.Popen([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                                "--out", str(tmp_path / "out"), "--max-tokens", str(peak)],
                               stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    got, position = {}, {}
    for number, (entries, ended) in enumerate(schedule):
        step = dict(step=number, entries=[dict(id=rid, tokens=tokens, want=want) for rid, tokens, want in entries], end=ended)
        process.stdin.write(json.dumps(step) + "\n")
        process.stdin.flush()
        assert process.stdout.readline().strip() == f"done {number}"
        wanted = [(rid, position.get(rid, 0) + w) for rid, tokens, want in entries for w in want]
        data = np.fromfile(tmp_path / "out" / f"{number}.f32", dtype="<f4").reshape(len(wanted), cases.CASE_B["vocab"])
        for key, row in zip(wanted, data):
            got[key] = torch.from_numpy(row.copy())
        for rid, tokens, _ in entries:
            position[rid] = position.get(rid, 0) + len(tokens)
    process.stdin.close()
    assert process.wait(timeout=60) == 0
    expected, low = truth["B"]
    judge(got, expected, low, torch.float32 if dtype == "float32" else torch.bfloat16, f"larolorn replay program {dtype}")


def test_command_line_generates_with_written_and_with_random_weights(folders, tmp_path):
    folder, weights, _ = folders["C"]
    prompt = cases.random_tokens(cases.CASE_C, 9, 77)          # ids that every case's vocabulary holds
    run = lambda model, *extra: subprocess.run(
        [sys.executable, "-m", "qwen_inference_lab_b200", "--model", str(model), "--token-ids", json.dumps(prompt),
         "--dtype", "float32", "--max-new-tokens", "4", "--pages", "24", "--page-size", "4", "--chunk-size", "5",
         "--ignore-eos", *extra], capture_output=True, text=True, cwd=str(ROOT))
    done = run(folder)
    assert done.returncode == 0, done.stderr
    tokens = json.loads(done.stdout)["token_ids"]
    sequence = list(prompt)
    for token in tokens:
        assert token == int(plain.forward(cases.CASE_C, weights, sequence, torch.float32)[-1].argmax())
        sequence.append(token)
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(cases.CASE_A))
    done = run(bare, "--random-weights", "3")
    assert done.returncode == 0, done.stderr
    assert len(json.loads(done.stdout)["token_ids"]) == 4 and (bare / "model.safetensors").is_file()
