"""Larolorn without a GPU: configuration and refusals, tensor names and shapes, cache specs, layers that run with
another layer's tensors, the step plan of the recurrent mixer, and the plain functions against closed forms."""
import math

import pytest
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.config.model_config import ConfigError, LarolornConfig
from qwen_inference_lab_b200.parts import KVCacheSpec, StateSpec
from tests import larolorn_cases as cases
from tests.plain import larolorn_plain as plain

F64 = torch.float64


def test_the_registry_builds_the_model_with_the_design_names():
    entry = registry.lookup(cases.CASE_A)
    assert entry.config_class is LarolornConfig
    model = entry.build(LarolornConfig.from_dict(cases.CASE_A))
    params = model.all_named_params()
    for expected in ("embed", "final.norm", "head", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm",
                     "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down",
                     "l1.mix.left.q", "l1.mix.left.q.b", "l1.mix.left.k.b", "l1.mix.left.v.b", "l1.mix.left.o.b",
                     "l1.mix.left.q.norm", "l1.mix.left.k.norm", "l1.mix.left.sink", "l1.mix.left.out", "l1.mix.right.out",
                     "l1.mix.right.q", "l1.mix.right.k", "l1.mix.right.v", "l1.mix.right.g", "l1.mix.right.o",
                     "l1.mix.right.norm", "l3.norm1", "l3.mix.left.sink"):
        assert expected in params, expected
    # layers 2 and 4 run with the tensors of layers 0 and 1; the latent attention's projections have no biases
    assert not any(name.startswith(("l2.", "l4.")) for name in params) and "l0.mix.q.b" not in params
    assert "l1.mix.right.q.b" not in params and params["l3.norm2"].optional and not params["l1.norm2"].optional
    assert params["l0.mix.q"].shape == (3 * (24 + 8), 96) and params["l0.mix.dkv"].shape == (24 + 8, 96)
    assert params["l0.mix.uk"].shape == (3 * 24, 24) and params["l0.mix.uv"].shape == (3 * 40, 24)
    assert params["l0.mix.g"].shape == (3, 96) and params["l0.mix.o"].shape == (96, 3 * 40)
    assert params["l1.mix.left.q.norm"].shape == (4 * 32,) and params["l1.mix.left.k.norm"].shape == (2 * 32,)
    assert params["l1.mix.left.sink"].shape == (4,) and params["l1.mix.right.norm"].shape == (2 * 24,)
    assert params["l3.mix.left.o"].shape == (96, 6 * 8) and params["l3.mix.right.k"].shape == (3 * 40, 96)
    assert len(model.layers) == 3 and [call.layer for call in model.order] == [0, 1, 0, 2, 1]
    assert model.logit_scale == 0.5 and model.stream_dtype == torch.float32


def test_every_layer_run_has_a_cache_of_its_own():
    model = registry.lookup(cases.CASE_A).build(LarolornConfig.from_dict(cases.CASE_A))
    specs = model.cache_specs()
    assert len(specs) == 5
    # the latent layers keep one row [latent, rotated key part] per token, inside a window of 20; the value is
    # the row's first 24 columns and has no row of its own
    assert specs[0] == specs[2] == KVCacheSpec(1, 32, 20, 24, shared_rows=True)
    # the parallel layers keep pages for the chunked attention and a float32 matrix per recurrent head
    assert specs[1] == specs[4] == (KVCacheSpec(2, 32, 0, 0, chunk=24), StateSpec((2, 16, 24), torch.float32))
    assert specs[3] == (KVCacheSpec(3, 16, 0, 8, chunk=7), StateSpec((3, 40, 8), torch.float32))
    cache = CacheManager(specs, num_pages=8, page_size=4, max_requests=2, max_context=64, dtype=torch.float32, device="cpu")
    views = cache.views()
    assert views[0].pages.data_ptr() != views[2].pages.data_ptr() and tuple(views[0].pages.shape) == (8, 1, 1, 4, 32)
    assert views[1][1].slots.data_ptr() != views[4][1].slots.data_ptr()
    # whatever the key row's size: one row per token
    model = registry.lookup(cases.CASE_B).build(LarolornConfig.from_dict(cases.CASE_B))
    assert model.cache_specs()[2] == KVCacheSpec(1, 14, 1, 10, shared_rows=True)
    assert model.cache_specs()[1] == KVCacheSpec(1, 64, 33, 48, shared_rows=True)


def _changed(change, case=cases.CASE_A):
    data = LarolornConfig.from_dict(case).to_dict()
    change(data)
    return data


@pytest.mark.parametrize("change", [
    lambda c: c.update(vocab=0), lambda c: c.update(width=-3), lambda c: c["norm"].update(eps=0), lambda c: c.update(layers=[]),
    lambda c: c.update(residual_mult="x"), lambda c: c.update(architecture="Other"),
    lambda c: c["layers"][0].update(type="attention"), lambda c: c["layers"][0]["mixer"].update(heads=0),
    lambda c: c["layers"][0]["mixer"].pop("kv_rank"), lambda c: c["layers"][0]["mixer"].update(scale=0),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), lambda c: c["layers"][0]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][1]["mixer"].pop("right"), lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
    lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=34), lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5, 1.5]),
    lambda c: c["layers"][1]["mlp"].update(kind="moe"), lambda c: c["layers"][1]["mlp"].update(limit=0),
    lambda c: c["layers"][2].update(weights_of=2), lambda c: c["layers"][2].update(weights_of=1),
    lambda c: c["layers"][4].update(weights_of=2),
])
def test_configurations_that_are_refused(change):
    with pytest.raises(ConfigError):
        LarolornConfig.from_dict(_changed(change))


def test_configuration_round_trip_and_defaults():
    config = LarolornConfig.from_dict(cases.CASE_C)
    assert LarolornConfig.from_dict(config.to_dict()) == config
    assert config.residual_mult == 0.25 and config.logit_scale == 2.0 and config.eps == 1e-5
    bare = _changed(lambda c: (c.pop("residual_mult"), c.pop("logit_scale")))
    config = LarolornConfig.from_dict(bare)
    assert config.residual_mult == 1.0 and config.logit_scale == 1.0
    # "weights_of": null is a layer with tensors of its own
    explicit = _changed(lambda c: c["layers"][1].update(weights_of=None))
    model = registry.lookup(explicit).build(LarolornConfig.from_dict(explicit))
    assert "l1.mix.left.q" in model.all_named_params()


def test_a_layer_may_run_with_the_tensors_of_a_later_layer():
    data = _changed(lambda c: (c["layers"][0].update(weights_of=2), c["layers"][2].pop("weights_of")))
    model = registry.lookup(data).build(LarolornConfig.from_dict(data))
    params = model.all_named_params()
    assert "l2.mix.q" in params and not any(name.startswith("l0.") for name in params)
    assert [call.layer for call in model.order][0] == [call.layer for call in model.order][2]
    weights = cases.draw_weights(params, 3)
    tokens = cases.random_tokens(data, 12, 1)
    assert torch.isfinite(plain.forward(data, weights, tokens)).all()


def test_the_recurrent_mixers_step_plan_cuts_long_segments_into_chunks():
    from types import SimpleNamespace
    import numpy as np
    from qwen_inference_lab_b200.parts.linear_attention import CHUNK, LONG_SEGMENT, ScanPlanner
    lens = [1, LONG_SEGMENT, LONG_SEGMENT + 1, 3 * CHUNK + 5]
    first = np.cumsum([0] + lens[:-1])
    plan = ScanPlanner().plan(SimpleNamespace(lens=lens, first=first, rows=[3, 0, 2, 1]))
    assert plan["short_len"].tolist() == [1, LONG_SEGMENT] and plan["short_row"].tolist() == [3, 0]
    pieces = -(-(LONG_SEGMENT + 1) // CHUNK)
    assert plan["carry"].tolist() == [2, 0, pieces, 1, pieces, 4]
    assert plan["chunk_len"].sum() == lens[2] + lens[3] and plan["chunk_len"].max() == CHUNK
    assert plan["chunk_start"][0] == first[2] and plan["chunk_start"][pieces] == first[3]
    assert plan["chunk_index"].tolist() == list(range(pieces + 4))


# ------------------------------------------------------------------ the plain functions against closed forms
def test_plain_norm_activation_and_feed_forward():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(plain.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0), torch.tensor([[3.0, 8.0]], dtype=F64) / math.sqrt(12.5))
    # eps sits inside the root
    assert torch.allclose(plain.rms_norm(torch.zeros(1, 4, dtype=F64) + 1e-9, torch.ones(4), 1.0), torch.full((1, 4), 1e-9, dtype=F64))
    w = {"f.gate": torch.tensor([[1.0]]), "f.up": torch.tensor([[1.0]]), "f.down": torch.tensor([[1.0]])}
    ff = lambda h: float(plain.clamped_feed_forward(torch.tensor([[h]], dtype=F64), w, "f.", dict(limit=2.0)))
    swish = lambda g: g / (1 + math.exp(-1.702 * g))
    assert abs(ff(1.0) - swish(1.0) * 2.0) < 1e-12
    assert abs(ff(5.0) - swish(2.0) * 3.0) < 1e-12                  # both clamped from above
    assert abs(ff(-5.0) - swish(-5.0) * (-2.0 + 1.0)) < 1e-12      # the gate has no lower bound, the other branch has


def test_plain_rotations_pair_the_right_dimensions():
    rot = dict(base=100.0, dims=4)
    x = torch.zeros(3, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0                     # the first dimension of pair 0 in both layouts
    x[:, 0, 5] = 7.0                     # beyond the rotated dimensions
    a = plain.rotate_interleaved(x, rot)
    b = plain.rotate_halves(x, rot)
    for t in range(3):
        assert torch.allclose(a[t, 0], torch.tensor([math.cos(t), math.sin(t), 0, 0, 0, 7.0], dtype=F64))
        assert torch.allclose(b[t, 0], torch.tensor([math.cos(t), 0, math.sin(t), 0, 0, 7.0], dtype=F64))
    # pair 1 turns by base^(-2 / dims) a position
    y = torch.zeros(2, 1, 4, dtype=F64); y[:, 0, 2] = 1.0
    assert torch.allclose(plain.rotate_interleaved(y, rot)[1, 0], torch.tensor([0, 0, math.cos(0.1), math.sin(0.1)], dtype=F64))
    z = torch.zeros(2, 1, 4, dtype=F64); z[:, 0, 1] = 1.0
    assert torch.allclose(plain.rotate_halves(z, rot)[1, 0], torch.tensor([0, math.cos(0.1), 0, math.sin(0.1)], dtype=F64))
    # a rotated query against a rotated key depends on the distance only
    q = torch.randn(9, 1, 4, dtype=F64).expand(9, 1, 4)[0:1].repeat(9, 1, 1)
    turned = plain.rotate_halves(q, rot)
    assert torch.allclose((turned[8] * turned[5]).sum(), (turned[3] * turned[0]).sum())


def test_plain_window_and_chunk_edges_and_the_sink():
    T = 12
    q = torch.zeros(T, 1, 2, dtype=F64); q[:, 0, 0] = 50.0
    k = torch.zeros(T, 1, 2, dtype=F64); k[4, 0, 0] = 50.0       # one key that outweighs everything
    v = torch.arange(T, dtype=F64).view(T, 1, 1) + 1.0
    out = plain.window_softmax_attention(q, k, v, 1.0, 5).flatten()
    assert abs(out[8] - 5.0) < 1e-9                                # 8 - 4 < 5: just inside
    assert abs(out[9] - (6 + 7 + 8 + 9 + 10) / 5.0) < 1e-9        # 9 - 4 = 5: just outside, five equal keys
    assert abs(out[2] - 2.0) < 1e-9                                # the first tokens see what there is
    none = torch.full((1,), -1e9, dtype=F64)                       # a sink that weighs nothing
    out = plain.chunk_sink_attention(q, k, v, 1.0, 5, none).flatten()
    assert abs(out[4] - 5.0) < 1e-9                                # the chunk's last position sees the key
    assert abs(out[5] - 6.0) < 1e-9                                # the next chunk's first position sees itself only
    assert abs(out[9] - (6 + 7 + 8 + 9 + 10) / 5.0) < 1e-9
    # a sink of score s beside one key of score zero: the key's weight is 1 / (1 + e^s); the sink is not scaled
    one = plain.chunk_sink_attention(torch.zeros(1, 1, 2, dtype=F64), torch.zeros(1, 1, 2, dtype=F64), torch.ones(1, 1, 1, dtype=F64),
                                     123.0, 4, torch.tensor([math.log(3.0)], dtype=F64))
    assert abs(float(one) - 0.25) < 1e-12
    # query heads read the key/value head of their group
    qq = torch.zeros(1, 4, 2, dtype=F64); kk = torch.zeros(1, 2, 2, dtype=F64)
    vv = torch.tensor([[[1.0], [2.0]]], dtype=F64)
    assert plain.chunk_sink_attention(qq, kk, vv, 1.0, 4, none.expand(4)).flatten().tolist() == [1.0, 1.0, 2.0, 2.0]


def test_plain_decayed_state_is_a_geometric_sum():
    T = 6
    q = torch.ones(T, 2, 1, dtype=F64); k = torch.ones(T, 2, 1, dtype=F64); v = torch.ones(T, 2, 1, dtype=F64)
    out, state = plain.decayed_state_scan(q, k, v, [0.5, 1.0])
    assert torch.allclose(out[:, 0, 0], torch.tensor([sum(0.5 ** i for i in range(t + 1)) for t in range(T)], dtype=F64))
    assert torch.allclose(out[:, 1, 0], torch.arange(1, T + 1, dtype=F64))
    # going on from a state equals never having stopped
    first, s = plain.decayed_state_scan(q[:2], k[:2], v[:2], [0.5, 1.0])
    rest, s = plain.decayed_state_scan(q[2:], k[2:], v[2:], [0.5, 1.0], s)
    assert torch.allclose(torch.cat([first, rest]), out) and torch.allclose(s, state)


def test_plain_latent_attention_equals_attention_over_expanded_keys():
    """The mixer's keys and values written out per head and fed to a textbook softmax give the mixer's output."""
    m = cases.CASE_A["layers"][0]["mixer"]
    model = registry.lookup(cases.CASE_A).build(LarolornConfig.from_dict(cases.CASE_A))
    w = {k: v.double() for k, v in cases.draw_weights(model.all_named_params(), 2).items()}
    T, H, d, r, e, c = 9, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    h = torch.randn(T, 96, dtype=F64, generator=torch.Generator().manual_seed(1))
    got = plain.latent_attention_mixer(h, w, "l0.mix.", m, 1e-5)
    q = (h @ w["l0.mix.q"].t()).view(T, H, d + r)
    down = h @ w["l0.mix.dkv"].t()
    z = plain.rms_norm(down[:, :c], w["l0.mix.dkv.norm"], 1e-5)
    gate = torch.sigmoid(h @ w["l0.mix.g"].t())
    freq = torch.tensor([m["rot"]["base"] ** (-2.0 * i / r) for i in range(r // 2)], dtype=F64)
    def turn(x, t):
        u, v = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = u * torch.cos(t * freq) - v * torch.sin(t * freq)
        out[..., 1::2] = v * torch.cos(t * freq) + u * torch.sin(t * freq)
        return out
    heads_out = torch.zeros(T, H, e, dtype=F64)
    for t in range(T):
        for a in range(H):
            scores = []
            for j in range(max(0, t - m["mask"]["size"] + 1), t + 1):
                key = w["l0.mix.uk"][a * d:(a + 1) * d] @ z[j]
                scores.append((q[t, a, :d] @ key + turn(q[t, a, d:], t) @ turn(down[j, c:], j)) * m["scale"])
            p = torch.softmax(torch.stack(scores), 0)
            for weight, j in zip(p, range(max(0, t - m["mask"]["size"] + 1), t + 1)):
                heads_out[t, a] += weight * (w["l0.mix.uv"][a * e:(a + 1) * e] @ z[j])
    expected = (heads_out * gate[:, :, None]).reshape(T, H * e) @ w["l0.mix.o"].t()
    assert torch.allclose(got, expected, atol=1e-10)
