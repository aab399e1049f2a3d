"""Gogotar on the GPU: every mechanism alone against its plain function, keys made to stand out at the edges of chunks,
at page borders and far away, then whole models under four ways of cutting the work, long decoding, slots and pages
used again, generation through the engine, the replay program and the command line."""
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import gogotar_cases as cases
from tests import harness
from tests.plain import gogotar_plain as plain
from tests.test_larolorn_gpu import (SCHEDULES, Ctx, _judge_the_query, _run_with_the_query_last, close, low_of,
                                     peak_live_pages, rows, through_the_step_function)
from tests.test_larolorn_gpu import judge as judge_rows

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["float32", "bfloat16"]
F64 = torch.float64
SUFFIX = ("", ".b")


def fill(part, seed, dtype, values=None):
    """Random parameters (``cases.draw_weights``) or the given ones; returns name -> CPU float32."""
    drawn = cases.draw_weights(part.all_named_params(), seed)
    drawn.update(values or {})
    for name, param in part.all_named_params().items():
        drawn[name] = drawn[name].to(torch.bfloat16).float()
        param.data = drawn[name].to(dtype).cuda()
    part.finalize(torch.device("cuda"), dtype)
    return drawn


# ------------------------------------------------------------------ mechanisms without a cache
@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("width", [70, 96, 1000, 1025, 2048, 3000, 4096, 4100])
def test_a_normed_branch_joins_the_stream_and_the_next_norm_rides_along(kind, width):
    """x += norm(a) w on a float32 stream; the same kernel norms the new stream for the next sublayer (float32 and
    bfloat16 rows), or hands it on rounded.  The branch carries a large mean, which the layer norm takes off.  Rows
    of up to 4096 values stay in registers (4, 8 or 16 a thread), wider ones are read again."""
    from qwen_inference_lab_b200.kernels import ops
    norm = plain.layer_norm if kind == "layer" else plain.rms_norm
    stream, a = rows(5, width, 1, 4.0) + 2.0, rows(5, width, 2, 3.0) + 5.0
    w, w_next = (1 + 0.1 * rows(1, width, 4 + i)[0] for i in range(2))
    for eps in (1e-6, 0.5):
        joined = (stream.double() + norm(a.double(), w, eps)).float()
        out = ops.norm_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, kind)
        torch.testing.assert_close(out.cpu(), joined, atol=1e-5, rtol=1e-6)
        for row_dtype in DTYPES:
            after = torch.full((5, width), float("nan"), dtype=row_dtype, device="cuda")
            again = ops.norm_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, kind, next_weight=w_next.cuda(), rows=after)
            assert torch.equal(again, out)
            expected = norm(out.cpu().double(), w_next, eps)
            if row_dtype == torch.float32:
                torch.testing.assert_close(after.cpu(), expected.float(), atol=2e-6, rtol=1e-5)
            else:
                assert (after.float().cpu() - expected).abs().max() <= 2.0 ** -8 * expected.abs().max()
            copy = torch.full((5, width), float("nan"), dtype=row_dtype, device="cuda")
            ops.norm_join(stream.clone().cuda(), a.cuda(), w.cuda(), eps, kind, rows=copy)
            assert torch.equal(copy, out.to(row_dtype))
    # the other kind of norm behind this one, with an eps of its own
    other = "rms" if kind == "layer" else "layer"
    after = torch.empty((5, width), device="cuda")
    out = ops.norm_join(stream.clone().cuda(), a.cuda(), w.cuda(), 1e-5, kind, next_weight=w_next.cuda(), next_eps=0.3,
                        next_kind=other, rows=after)
    expected = (plain.rms_norm if kind == "layer" else plain.layer_norm)(out.cpu().double(), w_next, 0.3)
    torch.testing.assert_close(after.cpu(), expected.float(), atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_layer_norm_without_a_bias_and_the_rms_norm_of_a_column_range(dtype):
    from qwen_inference_lab_b200.kernels import ops
    x = rows(7, 150, 3, 2.0) + 1.5
    w = (1 + 0.1 * rows(1, 150, 4)[0])
    got = ops.layernorm_exact(x.cuda(), w.to(dtype).cuda(), None, 1e-5, out_dtype=dtype, rows=torch.tensor([6, 0, 3], dtype=torch.int32, device="cuda"))
    close(got, plain.layer_norm(x.double(), w.to(dtype).double(), 1e-5)[[6, 0, 3]], dtype)
    piece = ops.rmsnorm_exact(x.to(dtype).cuda(), w[:37].to(dtype).cuda(), 1e-5, out_dtype=dtype, columns=(51, 37))
    close(piece, plain.rms_norm(x.to(dtype).double()[:, 51:88], w[:37].to(dtype).double(), 1e-5), dtype)


def test_the_embedding_is_scaled_and_the_logits_are_capped():
    from qwen_inference_lab_b200.kernels import ops
    table = rows(20, 33, 5)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device="cuda")
    for dtype in DTYPES:
        out = torch.empty(4, 33, device="cuda")
        ops.embed_gather(table.to(dtype).cuda(), ids, out, 12.5)
        assert torch.equal(out.cpu(), table[[3, 19, 0, 3]] * 12.5)
    logits = rows(3, 50, 6, 40.0)
    got = ops.softcap_inplace(logits.clone().cuda(), 20.0)
    torch.testing.assert_close(got.cpu(), (20.0 * torch.tanh(logits.double() / 20.0)).float(), atol=1e-5, rtol=1e-6)
    assert got.abs().max() <= 20.0 and (logits.abs() > 60).any()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,width,experts,top,ff", [(1, 96, 5, 2, 24), (9, 70, 7, 7, 11), (75, 64, 3, 1, 48), (200, 128, 16, 4, 32)])
def test_routed_experts_with_unrenormalised_scores(dtype, n, width, experts, top, ff):
    """Choice and weights against the plain router (the kernel's float32 scores: rows whose choice is a close call are
    left out), then the experts' weighted sum; a token alone gives what it gives in the batch."""
    from qwen_inference_lab_b200.kernels import ops
    from qwen_inference_lab_b200.parts import RoutedExperts
    names = dict(router="f.router", router_bias=None, expert=lambda index, which: f"f.e{index}.{which}")
    part = RoutedExperts(width, ff, experts, top, names=names, activation="silu", routing="softmax_all", renormalize=False)
    w = fill(part, 7, dtype)
    x = rows(n, width, 8)
    chosen, weights = ops.moe_route(x.to(dtype).cuda(), part.router.data, None, top, softmax_all=True, renormalize=False)
    want_chosen, want_weights = plain.route(x.double(), w["f.router"], top)
    margins = []
    plain.routed_experts(x.double(), w, "f.", dict(router=dict(top=top, experts=experts)), margins=margins)
    clear = torch.ones(n, dtype=torch.bool) if not margins else margins[0] > 1e-3
    assert clear.sum() >= n // 2 + 1
    assert torch.equal(chosen.cpu()[clear].long(), want_chosen[clear])
    torch.testing.assert_close(weights.cpu()[clear], want_weights[clear].float(), atol=1e-6, rtol=1e-5)
    if top < experts:
        assert (weights.sum(dim=1) < 1.0).all()
    expected = plain.routed_experts(x.double(), w, "f.", dict(router=dict(top=top, experts=experts)), low_of(dtype))
    ctx = Ctx(dtype)
    out = part.forward(ctx, x.to(dtype).cuda(), out_float32=True)
    assert out.dtype == torch.float32
    close(out[clear.cuda()], expected[clear], dtype, scale=float(expected.abs().max()))
    alone = part.forward(ctx, x[n // 2:n // 2 + 1].to(dtype).cuda(), out_float32=True)
    torch.testing.assert_close(alone[0], out[n // 2], atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-5 if dtype == torch.float32 else 2e-2)


# ------------------------------------------------------------------ the mixers alone, through the step function
def attention_part(hidden, m, eps=1e-5):
    from qwen_inference_lab_b200.parts import GroupedQueryAttention, RotaryFrequencies
    names = {k: "m." + k for k in ("q", "k", "o", "sink")}
    names.update(q_norm="m.q.norm", k_norm="m.k.norm")
    scaling = m["rot"].get("scaling")
    position = RotaryFrequencies(m["rot"]["dims"], m["rot"]["base"], "halves",
                                 scaling=None if scaling is None else tuple(scaling[k] for k in ("factor", "low", "high", "original")))
    return GroupedQueryAttention(hidden, m["heads"], m["kv_heads"], m["dim"], names=names, scale=m["scale"], suffixes=SUFFIX,
                                 position=position, qk_norm_eps=eps, norm_suffix="", chunk=(m.get("mask") or {}).get("size", 0),
                                 softcap=m.get("softcap") or 0.0, sink="learned", values_from_keys=True, head_gate="m.g")


def latent_part(hidden, m, eps=1e-5):
    from qwen_inference_lab_b200.parts import LatentAttention
    names = {k: "m." + k for k in ("dq", "uq", "dkv", "uk", "uv", "g", "o", "sink")}
    names.update(dq_norm="m.dq.norm", dkv_norm="m.dkv.norm")
    return LatentAttention(hidden, m["heads"], m["dim"], 0, m["vdim"], m["kv_rank"], scale=m["scale"], window=0, position=None,
                           norm_eps=eps, names=names, suffixes=SUFFIX, norm_suffix="", query_latent=m["q_rank"],
                           sink="learned", gate="element")


CUTS = ({"a": [75], "b": [41]}, {"a": [3, 1, 1, 2, 30, 1, 5, 2, 30], "b": [1] * 9 + [2] * 6 + [20]}, {"a": [1] * 75, "b": [17, 24]})

ATTENTIONS = [cases.attention(4, 2, 32, 0.2, 10000.0, 16, 24, 20.0, (4.0, 1.0, 2.0, 64)),   # tensor-core kernels; half a head rotated
              cases.attention(6, 6, 16, 0.9, 300.0, 16, 7, 1.5),                            # a cap that bites; chunks of seven
              cases.attention(3, 3, 20, 0.22, 50.0, 4, 1, 2.5),                             # heads of 20: the float32 kernel; a token and the sink
              cases.attention(2, 1, 80, 0.11, 500.0, 80, 4096, 30.0, (2.0, 2.0, 8.0, 32)),  # one key/value head, no chunk edge in reach
              cases.attention(6, 1, 16, 0.25, 10000.0, 2),                                  # no mask, no cap; one rotated pair
              cases.attention(8, 2, 128, 0.08, 250000.0, 64, 50, 45.0, (6.0, 1.0, 3.0, 16)),  # heads of 128
              cases.attention(4, 4, 48, 0.15, 20000.0, 48, 19, 10.0)]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m", ATTENTIONS, ids=[f"d{m['dim']}h{m['heads']}" for m in ATTENTIONS])
def test_attention_with_keys_as_values_whole_cut_and_side_by_side(dtype, m):
    """The mixer over whole sequences, over portions down to one and two tokens, and with two requests in every step."""
    part = attention_part(72, m)
    w = fill(part, 21, dtype)
    inputs = {"a": rows(75, 72, 22), "b": rows(41, 72, 23)}
    expected = {rid: plain.attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    for cuts in CUTS:
        got = through_the_step_function(part, 72, dtype, inputs, cuts, num_pages=48)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


def test_whole_tiles_of_heads_of_128_take_the_tensor_memory_kernel_with_capped_scores(monkeypatch):
    """Whole 128-token tiles of a prompt go to the tcgen05 kernel, which caps the scores itself (a cap that bites, a mild
    one, none), inside chunks whose edges fall inside a tile, with the sinks; leftovers and single tokens take the
    tiled kernels."""
    from qwen_inference_lab_b200.kernels import attention_tc
    calls = []
    original = attention_tc.prefill
    monkeypatch.setattr(attention_tc, "prefill", lambda *a, **k: (calls.append(k.get("softcap")), original(*a, **k))[1])
    for softcap in (3.0, 40.0, None):
        del calls[:]
        m = cases.attention(4, 2, 128, 0.09, 10000.0, 64, 200, softcap, (6.0, 1.0, 3.0, 64))
        part = attention_part(64, m)
        w = fill(part, 31, torch.bfloat16)
        inputs = {"a": rows(330, 64, 32), "b": rows(140, 64, 33)}
        want = {rid: plain.attention_mixer(x.double(), w, "m.", m, 1e-5, torch.bfloat16) for rid, x in inputs.items()}
        for cuts in ({"a": [330], "b": [140]}, {"a": [129, 1, 200], "b": [7, 133]}):
            got = through_the_step_function(part, 64, torch.bfloat16, inputs, cuts, page_size=16, num_pages=40)
            for rid in inputs:
                close(got[rid], want[rid], torch.bfloat16)
        assert calls and all(call == (softcap or 0.0) for call in calls)


LATENTS = [cases.latent(3, 24, 40, 32, 20, 0.17),      # key rows of 32: the tensor-core kernels in bfloat16
           cases.latent(5, 12, 20, 10, 8, 0.25),       # rows of 10: the float32 kernel
           cases.latent(1, 6, 10, 30, 7, 0.4),         # one head
           cases.latent(2, 16, 16, 48, 56, 0.2),       # a query latent larger than the key latent
           cases.latent(4, 40, 8, 96, 72, 0.1),        # values smaller than keys
           cases.latent(3, 48, 56, 160, 33, 0.09),
           cases.latent(2, 128, 128, 256, 192, 0.07)]  # rows of 256, the widest the tensor-core kernels take


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("m", LATENTS, ids=[f"row{m['kv_rank']}" for m in LATENTS])
def test_latent_attention_whole_cut_and_side_by_side(dtype, m):
    part = latent_part(88, m)
    w = fill(part, 11, dtype)
    inputs = {"a": rows(75, 88, 12), "b": rows(41, 88, 13)}
    expected = {rid: plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype)) for rid, x in inputs.items()}
    for cuts in CUTS:
        got = through_the_step_function(part, 88, dtype, inputs, cuts, num_pages=48)
        for rid in inputs:
            close(got[rid], expected[rid], dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_latent_attention_in_long_portions_takes_the_batched_products(dtype):
    """Portions of more than 64 tokens hand the per-head products to batched library products in bfloat16."""
    m = cases.latent(3, 24, 40, 32, 20, 0.17)
    part = latent_part(88, m)
    w = fill(part, 11, dtype)
    inputs = {"a": rows(300, 88, 12)}
    expected = plain.latent_attention_mixer(inputs["a"].double(), w, "m.", m, 1e-5, low_of(dtype))
    for cuts in ({"a": [300]}, {"a": [130, 1, 2, 167]}):
        got = through_the_step_function(part, 88, dtype, inputs, cuts, page_size=16, num_pages=24)
        close(got["a"], expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_the_sink_takes_its_share_and_is_neither_scaled_nor_capped(dtype):
    """Zero query projections: every key scores zero, so a token n positions into its chunk gets the sum of the keys
    it sees (as projected: the values) over n + e^sink, whatever scale and cap say, times the gate of one half."""
    m = cases.attention(2, 1, 16, 37.0, 100.0, 16, 6, 0.01)
    part = attention_part(24, m)
    sink = float(torch.tensor(math.log(2.0)).to(torch.bfloat16))
    w = fill(part, 1, dtype, {"m.q": torch.zeros(32, 24), "m.g": torch.zeros(2, 24), "m.o": torch.eye(24, 32),
                              "m.sink": torch.tensor([sink, -30.0])})
    x = rows(15, 24, 3)
    got = through_the_step_function(part, 24, dtype, {"a": x}, {"a": [4, 1, 1, 9]})["a"].float().cpu()
    keys = x.double() @ w["m.k"].double().t()
    if dtype == torch.bfloat16:
        keys = keys.to(torch.bfloat16).double()
    for t in range(15):
        first, n = t // 6 * 6, t % 6 + 1
        with_sink = 0.5 * keys[first:t + 1].sum(0) / (n + math.exp(sink))
        without = 0.5 * keys[first:t + 1].mean(0)
        want = torch.cat([with_sink, without[:8]])
        assert (got[t] - want).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(want.abs().max()))
    # the latent attention: zero queries, so the mean of the values seen so far with the sink's share taken off
    m = cases.latent(2, 8, 8, 16, 12, 9.0)
    part = latent_part(24, m)
    w = fill(part, 2, dtype, {"m.uq": torch.zeros(16, 12), "m.g": torch.zeros(16, 24), "m.o": torch.eye(24, 16),
                              "m.sink": torch.tensor([sink, -30.0])})
    got = through_the_step_function(part, 24, dtype, {"a": x}, {"a": [4, 1, 1, 9]})["a"].float().cpu()
    z = plain.rms_norm(x.double() @ w["m.dkv"].double().t(), w["m.dkv.norm"].double(), 1e-5)
    values = z @ w["m.uv"].double().t()
    for t in range(15):
        want = 0.5 * torch.cat([values[:t + 1, :8].sum(0) / (t + 1 + math.exp(sink)), values[:t + 1, 8:].mean(0)])
        assert (got[t, :16] - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2) * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------ one key made to stand out
CHUNK_EDGES = [(64, 127, 64, True), (64, 128, 127, False), (64, 128, 64, False), (24, 47, 24, True), (24, 48, 47, False),
               (7, 13, 7, True), (7, 14, 13, False), (1024, 700, 3, True), (300, 599, 300, True), (300, 600, 599, False),
               (1, 5, 5, None), (1, 5, 4, False), (33, 65, 33, True), (33, 66, 65, False), (None, 700, 8, True)]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk,query,far,inside", CHUNK_EDGES)
def test_a_key_just_inside_and_just_outside_the_chunk(dtype, single, chunk, query, far, inside):
    """The query's input is solved for so that, after the per-head norm, every head's query points along the far
    token's normed key of its group (q and k are normed, so a key stands out by its direction only: the far token's
    input is drawn again until its score leads every other key of the sequence by 30 in every head).  Seen from the
    far token's own chunk the output is that token's value, its key as projected, under the query's gates; from the
    first position of the next chunk it is not seen, however close it is.  Chunks that are over have given their
    pages back by then; without a mask a key hundreds of positions back, at a page's border, is still seen."""
    hidden = 160
    m = cases.attention(4, 2, 32, 3.0, 10000.0, 4, chunk, 400.0, (4.0, 1.0, 2.0, 16))
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    part = attention_part(hidden, m)
    w = fill(part, 61, dtype)
    W = {k: v.double() for k, v in w.items()}
    x = rows(query + 1, hidden, 62 + query, 0.5)
    normed_keys = lambda t: plain.rms_norm((t.double() @ W["m.k"].t()).view(-1, G, d), W["m.k.norm"], 1e-5)
    for attempt in range(40):
        if far == query:
            break
        x[far] = rows(1, hidden, 1000 + attempt, 0.5)[0]
        k_far = normed_keys(x[far:far + 1])[0]
        target = torch.stack([k_far[a // (H // G)] / W["m.q.norm"] for a in range(H)]).flatten()
        x[query] = (torch.linalg.pinv(torch.cat([W["m.q"], W["m.g"]])) @ torch.cat([target, torch.zeros(H, dtype=F64)])).to(torch.bfloat16).float()
        q = plain.rms_norm((x.double() @ W["m.q"].t()).view(-1, H, d), W["m.q.norm"], 1e-5)
        turned_q, turned_k = plain.rotate_halves(q, m["rot"])[query], plain.rotate_halves(normed_keys(x), m["rot"])
        scores = torch.stack([turned_k[:, a // (H // G)] @ turned_q[a] for a in range(H)]) * m["scale"]      # [H, T]
        others = torch.cat([scores[:, :far], scores[:, far + 1:]], dim=1)
        if float((scores[:, far] - others.max(dim=1).values).min()) > 30.0:
            break
    else:
        raise AssertionError("no input found whose key stands out")
    expected = plain.attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype))
    exact = plain.attention_mixer(x.double(), w, "m.", m, 1e-5)
    v_far = (x[far].double() @ W["m.k"].t()).view(G, d)
    gate = torch.sigmoid(x[query].double() @ W["m.g"].t())
    alone = torch.stack([v_far[a // (H // G)] * gate[a] for a in range(H)]).flatten() @ W["m.o"].t()
    got = _run_with_the_query_last(part, hidden, dtype, x, query, single)
    _judge_the_query(got, expected, exact, alone, query, inside, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("single", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("query,far", [(700, 7), (700, 8), (515, 0), (130, 127), (64, 63), (9, 9)])
def test_the_latent_attention_finds_a_key_far_back(dtype, single, query, far):
    """Causal without a window: the query's input is solved for through both of the queries' products and their norm, so
    that every head's query points along the far token's key of that head; the output is then that token's value
    alone under the query's gates.  Far tokens sit at page borders and at the very first position."""
    hidden = 192
    # keys are products of normed latents, all of about one length: heads and latents of 64 leave room for one
    # direction to stand out, and a large score scale turns the lead into dozens
    m = cases.latent(2, 64, 12, 64, 128, 100.0)
    H, d, e = m["heads"], m["dim"], m["vdim"]
    part = latent_part(hidden, m)
    w = fill(part, 51, dtype, {"m.sink": torch.tensor([-8.0, -8.0])})       # the sink's share has a test of its own
    W = {k: v.double() for k, v in w.items()}
    x = rows(query + 1, hidden, 52 + query, 0.5)
    latent_of = lambda t: plain.rms_norm(t.double() @ W["m.dkv"].t(), W["m.dkv.norm"], 1e-5)
    for attempt in range(60):
        if far == query:
            break
        x[far] = rows(1, hidden, 2000 + attempt, 0.5)[0]
        k_far = W["m.uk"] @ latent_of(x[far])                                  # [H * d]
        q_latent = torch.linalg.pinv(W["m.uq"]) @ k_far                        # the queries' latent that expands to it
        x[query] = (torch.linalg.pinv(torch.cat([W["m.dq"], W["m.g"]])) @ torch.cat([q_latent / W["m.dq.norm"], torch.zeros(H * e, dtype=F64)])).to(torch.bfloat16).float()
        q = (plain.rms_norm(x[query].double() @ W["m.dq"].t(), W["m.dq.norm"], 1e-5) @ W["m.uq"].t()).view(H, d)
        keys = (latent_of(x) @ W["m.uk"].t()).view(-1, H, d)
        scores = torch.einsum("thd,hd->ht", keys, q) * m["scale"]
        others = torch.cat([scores[:, :far], scores[:, far + 1:]], dim=1)
        if float((scores[:, far] - others.max(dim=1).values).min()) > 30.0:
            break
    else:
        raise AssertionError("no input found whose key stands out")
    expected = plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5, low_of(dtype))
    exact = plain.latent_attention_mixer(x.double(), w, "m.", m, 1e-5)
    gate = torch.sigmoid(x[query].double() @ W["m.g"].t())
    alone = ((W["m.uv"] @ latent_of(x[far])) * gate) @ W["m.o"].t()
    got = _run_with_the_query_last(part, hidden, dtype, x, query, single)
    if dtype == torch.float32:
        _judge_the_query(got, expected, exact, alone, query, None if far == query else True, dtype)
    elif far != query:
        # under this score scale bfloat16 rounding moves the other rows' softmax about; the query's own row is clear
        assert (exact[query] - alone).abs().max() < 1e-6 * alone.abs().max()
        close(got[-1], alone, dtype)


# ------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    result = {}
    for name, case in cases.CASES.items():
        folder = tmp_path_factory.mktemp(f"gogotar{name}")
        weights = cases.write_folder(case["config"], case["seed"], folder)
        requests = {f"r{i}": cases.random_tokens(case["config"], n, 60 + i) for i, n in enumerate(case["lengths"])}
        result[name] = (folder, weights, requests)
    return result


@pytest.fixture(scope="module")
def truth(folders):
    """The plain rows of every case, in float64 and with bfloat16 roundings, and the rows whose routing is a close call."""
    return {name: (cases.plain_rows(requests, weights, cases.CASES[name]["config"]),
                   cases.plain_rows(requests, weights, cases.CASES[name]["config"], torch.bfloat16),
                   cases.close_calls(requests, weights, cases.CASES[name]["config"]))
            for name, (folder, weights, requests) in folders.items()}


def judge(actual, expected, low, skip, dtype, what):
    """``tests.test_larolorn_gpu.judge``; bfloat16 rows whose choice of experts is a close call are not judged."""
    assert set(actual) == set(expected), f"{what}: different (request, position) sets"
    if dtype == torch.bfloat16:
        actual, expected, low = ({k: v for k, v in rows_.items() if k not in skip} for rows_ in (actual, expected, low))
    judge_rows(actual, expected, low, dtype, what)


def replay(folders, case, schedule_name, dtype):
    folder, weights, requests = folders[case]
    page_size = cases.CASES[case]["page_size"]
    schedule = SCHEDULES[schedule_name](requests)
    from qwen_inference_lab_b200.config import registry
    entry = registry.lookup(cases.CASES[case]["config"])
    shell = entry.build(entry.config_class.from_dict(cases.CASES[case]["config"]))
    num_pages = peak_live_pages(schedule, shell, page_size) + 1
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=num_pages, page_size=page_size)
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
    expected, low, skip = truth[case]
    judge(actual, expected, low, skip, dtype, f"gogotar {case} {schedule} {dtype}")


@pytest.mark.parametrize("case", list(cases.CASES))
def test_float32_rows_are_the_same_bits_under_every_schedule(folders, case):
    """Attention walks key tiles aligned to positions, float32 products sum in ascending order, every norm is over one
    token's row and a token's experts are summed in the order of its own choice: every cut gives the same bits."""
    runs = {name: replay(folders, case, name, torch.float32) for name in SCHEDULES}
    for name, got in runs.items():
        different = [key for key in sorted(got) if not torch.equal(got[key], runs["chunks"][key])]
        assert not different, \
            f"gogotar {case}: {len(different)} rows of schedule {name} differ from the run in portions, first {different[0]}"


@pytest.mark.parametrize("case,dtype", [("A", torch.float32), ("C", torch.float32), ("C", torch.bfloat16)],
                         ids=["A-float32", "C-float32", "C-bfloat16"])
def test_long_decoding_and_the_first_tokens(folders, dtype, case):
    """Three tokens as a prompt, then 300 single tokens (recorded graphs) across many chunk edges, every position
    judged.  (In bfloat16 only the case whose tokens use every expert: elsewhere a close call in the choice of experts
    early on reaches every later position.)"""
    folder, weights, _ = folders[case]
    config, page_size = cases.CASES[case]["config"], cases.CASES[case]["page_size"]
    tokens = cases.random_tokens(config, 303, 99)
    schedule = [([("r", tokens[:3], [0, 1, 2])], [])]
    schedule += [([("r", [tokens[i]], [0])], ["r"] if i == 302 else []) for i in range(3, 303)]
    _, cache, runner = harness.build_engine_parts(folder, dtype, num_pages=303 // page_size + 2, page_size=page_size)
    actual = harness.run_schedule(runner, cache, schedule)
    assert runner._graphs, "single-token steps should have been recorded"
    expected = cases.plain_rows({"r": tokens}, weights, config)
    low = cases.plain_rows({"r": tokens}, weights, config, torch.bfloat16) if dtype == torch.bfloat16 else None
    judge(actual, expected, low, cases.close_calls({"r": tokens}, weights, config), dtype, f"gogotar {case} long decoding {dtype}")


def test_pages_that_another_request_used_before(folders):
    """"x" runs and ends; "y" takes its row and its pages: its logits are those of "y" in a fresh cache, bit for bit."""
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
    expected, low, skip = truth["B"]
    judge(got, expected, low, skip, torch.float32 if dtype == "float32" else torch.bfloat16, f"gogotar replay program {dtype}")


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
