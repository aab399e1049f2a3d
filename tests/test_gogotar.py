"""Gogotar without a GPU: configuration and refusals, tensor names and shapes, looped layers with caches of their own,
the stretched rotary frequencies, and the plain functions against closed forms."""
import copy
import math

import pytest
import torch

from qwen_inference_lab_b200.cache import CacheManager
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.config.model_config import ConfigError, GogotarConfig
from qwen_inference_lab_b200.parts import KVCacheSpec, RotaryFrequencies
from tests import gogotar_cases as cases
from tests.plain import gogotar_plain as plain

F64 = torch.float64


def build(config):
    return registry.lookup(config).build(GogotarConfig.from_dict(config))


def test_the_registry_builds_the_model_with_the_design_names():
    entry = registry.lookup(cases.CASE_A)
    assert entry.config_class is GogotarConfig
    model = build(cases.CASE_A)
    params = model.all_named_params()
    for expected in ("embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.k",
                     "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.router",
                     "l0.mlp.e0.gate", "l0.mlp.e4.up", "l0.mlp.e4.down", "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq",
                     "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.sink", "l1.mix.g", "l1.mix.o",
                     "l1.mlp.gate", "l1.mlp.up", "l1.mlp.down", "l3.mix.sink"):
        assert expected in params, expected
    # no value projection, no biases, no head of its own (the embedding is the head), five experts
    assert not any(name in params for name in ("l0.mix.v", "l0.mix.q.b", "head", "l0.mlp.e5.gate", "final.norm.b"))
    assert params["l2.norm2"].optional and params["l2.norm2b"].optional and not params["l1.norm2b"].optional
    assert params["l0.mix.q"].shape == (4 * 32, 96) and params["l0.mix.k"].shape == (2 * 32, 96)
    assert params["l0.mix.q.norm"].shape == (32,) and params["l0.mix.g"].shape == (4, 96) and params["l0.mix.sink"].shape == (4,)
    assert params["l0.mix.o"].shape == (96, 4 * 32) and params["l0.mlp.router"].shape == (5, 96)
    assert params["l1.mix.dq"].shape == (20, 96) and params["l1.mix.uq"].shape == (3 * 24, 20)
    assert params["l1.mix.dkv"].shape == (32, 96) and params["l1.mix.uk"].shape == (3 * 24, 32)
    assert params["l1.mix.uv"].shape == (3 * 40, 32) and params["l1.mix.g"].shape == (3 * 40, 96)
    assert params["l1.mix.o"].shape == (96, 3 * 40) and params["l1.mix.sink"].shape == (3,)
    assert model.head.weight is model.embedding.weight and model.embedding.scale == 3.0 and model.logit_softcap == 25.0
    assert model.stream_dtype == torch.float32


def test_looped_layers_run_in_a_row_with_a_cache_for_every_pass():
    model = build(cases.CASE_A)
    assert len(model.layers) == 4 and [call.layer for call in model.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert plain.layer_runs(cases.CASE_A) == [0, 1, 2, 1, 2, 1, 2, 3]
    specs = model.cache_specs()
    assert len(specs) == 8
    # the values are the keys as projected: pages of keys and values of one size, given back chunk by chunk
    assert specs[0] == KVCacheSpec(2, 32, 0, 0, chunk=24) and specs[7] == KVCacheSpec(6, 16, 0, 0, chunk=7)
    # the latent layers keep one normed row per token; the value is the row itself
    assert specs[1] == specs[3] == specs[5] == KVCacheSpec(1, 32, 0, 32, shared_rows=True)
    cache = CacheManager(specs, num_pages=8, page_size=4, max_requests=2, max_context=64, dtype=torch.float32, device="cpu")
    views = cache.views()
    assert len({views[i].pages.data_ptr() for i in (1, 3, 5)}) == 3 and tuple(views[1].pages.shape) == (8, 1, 1, 4, 32)
    assert [call.layer for call in build(cases.CASE_B).order] == [0, 1, 2]             # no loop
    assert [call.layer for call in build(cases.CASE_C).order] == [0, 1, 2, 0, 1, 2]    # all layers, twice
    once = copy.deepcopy(cases.CASE_C)
    once["loop"] = dict(start=1, stop=1, times=5)                                      # an empty run of layers
    assert [call.layer for call in build(once).order] == [0, 1, 2]
    # no mask: keys and values of the whole request stay
    assert build(cases.CASE_B).cache_specs()[2] == KVCacheSpec(1, 48, 0, 0, chunk=0)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0]["mixer"].update(vdim=16), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "do not divide"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(low=2.0), "scaling"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][1].update(type="parallel"), "neither"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "neither dense nor moe"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c["embedding"].update(scale=0), "embedding.scale"),
])
def test_refused_configurations(change, message):
    config = copy.deepcopy(cases.CASE_A)
    change(config)
    with pytest.raises(ConfigError, match=message):
        GogotarConfig.from_dict(config)


def test_stretched_frequencies():
    """Short waves stay, long waves slow down by the factor, and between the two the blend runs from one to the other;
    the part's frequencies are the plain function's, and without scaling both are the plain powers of the base."""
    rot = dict(base=10000.0, dims=16, scaling=dict(factor=4.0, low=1.0, high=2.0, original=64))
    plain_f = plain.scaled_frequencies(rot)
    bare = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    kinds = set()
    for f, b in zip(plain_f, bare):
        wave = 2 * math.pi / b
        if wave < 32:
            assert f == b; kinds.add("short")
        elif wave > 64:
            assert f == b / 4.0; kinds.add("long")
        else:
            assert b / 4.0 < f < b; kinds.add("between")
            s = (64 / wave - 1.0) / (2.0 - 1.0)
            assert abs(f - ((1 - s) * b / 4.0 + s * b)) < 1e-15
    assert kinds == {"short", "long", "between"}
    part = RotaryFrequencies(16, 10000.0, "halves", scaling=(4.0, 1.0, 2.0, 64))
    assert part.frequencies() == plain_f
    assert RotaryFrequencies(16, 10000.0, "halves").frequencies() == bare == plain.scaled_frequencies(dict(base=10000.0, dims=16))
    with pytest.raises(ValueError):
        RotaryFrequencies(16, 10000.0, "halves", scaling=(4.0, 2.0, 2.0, 64))


def test_rotation_pairs_a_dimension_with_the_one_half_the_rotated_size_further():
    rot = dict(base=100.0, dims=4)
    x = torch.zeros(3, 1, 6, dtype=F64)
    x[:, 0, 0], x[:, 0, 5] = 1.0, 7.0
    out = plain.rotate_halves(x, rot)
    for p in range(3):
        assert abs(out[p, 0, 0] - math.cos(p)) < 1e-12 and abs(out[p, 0, 2] - math.sin(p)) < 1e-12
        assert out[p, 0, 1] == 0 and out[p, 0, 3] == 0 and out[p, 0, 4] == 0 and out[p, 0, 5] == 7.0
    assert torch.equal(plain.rotate_halves(x[2:], rot, first=2), out[2:])


def test_the_layer_norm_takes_the_mean_off_and_has_no_bias():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=F64)
    centred = x - 3.0
    expected = centred / math.sqrt(float(centred.pow(2).mean()) + 0.1) * w
    torch.testing.assert_close(plain.layer_norm(x, w, 0.1), expected)
    torch.testing.assert_close(plain.layer_norm(x + 100.0, w, 0.1), expected)


def test_who_sees_whom_and_what_the_sink_takes():
    """Zero queries: every key scores zero whatever the scale and the cap, so position i inside its chunk gets the
    mean of the values it sees times n / (n + e^sink)."""
    T, chunk = 9, 4
    q, k = torch.zeros(T, 2, 3, dtype=F64), torch.randn(T, 1, 3, dtype=F64)
    sinks = torch.tensor([math.log(3.0), -40.0], dtype=F64)
    out = plain.sink_attention(q, k, k, 5.0, sinks, chunk, softcap=2.0)
    for i in range(T):
        first = i // chunk * chunk
        n = i - first + 1
        torch.testing.assert_close(out[i, 0], k[first:i + 1, 0].sum(0) / (n + 3.0))
        torch.testing.assert_close(out[i, 1], k[first:i + 1, 0].mean(0))
    whole = plain.sink_attention(q, k, k, 5.0, sinks)
    torch.testing.assert_close(whole[8, 1], k[:, 0].mean(0))
    # the cap bounds a score: one huge product counts as the cap, not as itself
    q[5, 0, 0], k[4, 0, 0], k[5, 0, 0] = 100.0, 100.0, 0.0
    capped = plain.sink_attention(q, k, k, 1.0, torch.tensor([-40.0, -40.0], dtype=F64), chunk, softcap=2.0)
    weight = math.exp(2.0) / (math.exp(2.0) + 1.0)
    torch.testing.assert_close(capped[5, 0], weight * k[4, 0] + (1 - weight) * k[5, 0])


def test_routing_keeps_the_scores_as_they_are():
    h = torch.randn(6, 5, dtype=F64)
    router = torch.randn(4, 5, dtype=F64)
    chosen, weights = plain.route(h, router, 2)
    scores = torch.softmax(h @ router.t(), dim=-1)
    for t in range(6):
        order = sorted(range(4), key=lambda e: -float(scores[t, e]))[:2]
        assert chosen[t].tolist() == order
        torch.testing.assert_close(weights[t], scores[t, order])
    assert (weights.sum(dim=1) < 1.0).all()
    everything = plain.route(h, router, 4)[1]
    torch.testing.assert_close(everything.sum(dim=1), torch.ones(6, dtype=F64))


def test_attention_over_the_latent_equals_attention_over_expanded_keys():
    """What the engine does (the query folded through the key expansion, one row per token, the value expansion
    applied to the weighted sum of latents) is the plain mixer's arithmetic reassociated."""
    m = cases.latent(2, 6, 5, 7, 9, 0.3)
    width, T = 12, 8
    g = torch.Generator().manual_seed(3)
    w = {"m." + k: torch.randn(s, generator=g, dtype=F64) * 0.4 for k, s in dict(
        dq=(9, width), uq=(12, 9), dkv=(7, width), uk=(12, 7), uv=(10, 7), g=(10, width), o=(width, 10)).items()}
    w["m.dq.norm"], w["m.dkv.norm"] = 1 + 0.1 * torch.randn(9, generator=g, dtype=F64), 1 + 0.1 * torch.randn(7, generator=g, dtype=F64)
    w["m.sink"] = torch.tensor([0.3, -0.8], dtype=F64)
    h = torch.randn(T, width, generator=g, dtype=F64)
    expected = plain.latent_attention_mixer(h, w, "m.", m, 1e-5)
    z = plain.rms_norm(h @ w["m.dkv"].t(), w["m.dkv.norm"], 1e-5)
    q = (plain.rms_norm(h @ w["m.dq"].t(), w["m.dq.norm"], 1e-5) @ w["m.uq"].t()).view(T, 2, 6)
    folded = torch.einsum("thd,hdc->thc", q, w["m.uk"].view(2, 6, 7))
    sums = plain.sink_attention(folded, z[:, None, :], z[:, None, :], 0.3, w["m.sink"])
    mixed = torch.einsum("thc,hec->the", sums, w["m.uv"].view(2, 5, 7)).reshape(T, 10) * torch.sigmoid(h @ w["m.g"].t())
    torch.testing.assert_close(mixed @ w["m.o"].t(), expected)
