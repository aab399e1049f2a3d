"""Small Gogotar configurations and random weights for the tests.

The sizes differ from layer to layer and between the cases: head sizes the tensor-core attention takes and ones it
does not, one to three query heads per key/value head, rotations over all and over two of a head's dimensions, with
and without stretched frequencies, chunks of one position, of a few and longer than every request or none at all,
latents whose key row is and is not a size the tensor-core attention takes, value heads larger than, smaller than
and equal to key heads, one expert a token, a few, and all of them, layers without a feed-forward, loops of one,
two and three passes, at the start, in the middle and over all layers, no loop, scales and caps of one and absent.
"""
import json
from pathlib import Path

import torch

import qwen_inference_lab_b200.models  # noqa: F401  (registers the architectures)
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.weights import write_safetensors
from tests.plain import gogotar_plain as plain


def attention(heads, kv_heads, dim, scale, base, dims, chunk=None, softcap=None, scaling=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, rot=dict(base=base, dims=dims))
    if chunk is not None:
        m["mask"] = dict(size=chunk)
    if softcap is not None:
        m["softcap"] = softcap
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def latent(heads, dim, vdim, kv_rank, q_rank, scale):
    return dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


CASE_A = dict(architecture="Gogotar", vocab=173, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.0), logit_softcap=25.0,
              loop=dict(start=1, stop=3, times=3), layers=[
    dict(type="attention", mixer=attention(4, 2, 32, 0.2, 10000.0, 16, 24, 20.0, (4.0, 1.0, 2.0, 64)), mlp=moe(5, 2, 24)),
    dict(type="latent_attention", mixer=latent(3, 24, 40, 32, 20, 0.17), mlp=dense(72, 3.0)),
    dict(type="latent_attention", mixer=latent(2, 16, 16, 48, 56, 0.2), mlp=None),
    dict(type="attention", mixer=attention(6, 6, 16, 0.3, 300.0, 16, 7, 5.0), mlp=dense(40, 1.5)),
])
# no loop, no cap on the logits, an embedding scale of one; a chunk longer than every request and a layer without a mask; one
# key/value head under two query heads of 80; a latent row of 10, which no tensor-core kernel takes; one expert a token
CASE_B = dict(architecture="Gogotar", vocab=97, width=64, norm=dict(eps=1e-6), embedding=dict(scale=1.0), layers=[
    dict(type="latent_attention", mixer=latent(5, 12, 20, 10, 8, 0.25), mlp=moe(3, 1, 48)),
    dict(type="attention", mixer=attention(2, 1, 80, 0.11, 500.0, 80, 4096, 30.0, (2.0, 2.0, 8.0, 32)), mlp=dense(48, 7.0)),
    dict(type="attention", mixer=attention(3, 1, 48, 0.15, 20000.0, 2), mlp=None),
])
# awkward sizes: a width that is a multiple of nothing, heads of 20 (the float32 kernel), a chunk of one position (a token sees
# itself and the sink), one latent head, every expert for every token, a loop over all layers, a first layer without a feed-forward
CASE_C = dict(architecture="Gogotar", vocab=53, width=70, norm=dict(eps=1e-5), embedding=dict(scale=0.5), logit_softcap=35.0,
              loop=dict(start=0, stop=3, times=2), layers=[
    dict(type="attention", mixer=attention(3, 3, 20, 0.22, 50.0, 4, 1, 2.5), mlp=None),
    dict(type="latent_attention", mixer=latent(1, 6, 10, 30, 7, 0.4), mlp=moe(7, 7, 11)),
    dict(type="attention", mixer=attention(4, 2, 16, 0.3, 1e6, 16, 33, None, (16.0, 1.0, 3.0, 8)), mlp=dense(37, 0.5)),
])
# longer requests over pages of 16: heads of 128 whose whole 128-token tiles take the tensor-memory kernel, with a chunk that is a
# multiple of neither a page nor a key tile and a cap; every expert for every token (no close calls: bfloat16 is judged everywhere);
# a latent row of 80; a looped pair of layers in front
CASE_D = dict(architecture="Gogotar", vocab=301, width=256, norm=dict(eps=1e-5), embedding=dict(scale=2.0), logit_softcap=20.0,
              loop=dict(start=0, stop=2, times=2), layers=[
    dict(type="attention", mixer=attention(8, 2, 128, 0.09, 100000.0, 48, 100, 12.0, (4.0, 1.0, 4.0, 128)), mlp=moe(4, 4, 40)),
    dict(type="latent_attention", mixer=latent(4, 48, 24, 80, 50, 0.14), mlp=dense(136, 2.0)),
    dict(type="attention", mixer=attention(2, 2, 64, 0.125, 10000.0, 64, 300, 8.0), mlp=None),
])
CASES = {"A": dict(config=CASE_A, seed=5, page_size=4, lengths=(70, 9, 33, 150, 1, 50)),
         "B": dict(config=CASE_B, seed=6, page_size=16, lengths=(40, 3, 300, 64, 25)),
         "C": dict(config=CASE_C, seed=7, page_size=2, lengths=(31, 2, 77, 20, 45)),
         "D": dict(config=CASE_D, seed=8, page_size=16, lengths=(400, 130, 17, 260))}


def draw_weights(params: dict, seed: int) -> dict:
    """name -> CPU float32 tensor of bfloat16-representable values for ``params`` (name -> Param): weights of norms
    around one, sink scores of order one, the embedding of order a half, matrices scaled by their input size (the router's
    less, so that its scores are spread)."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, param in params.items():
        draw = torch.randn(param.shape, generator=generator)
        leaf = name.split(".")[-1]
        if leaf == "sink":
            value = draw
        elif len(param.shape) == 1:
            value = 1.0 + draw * 0.1
        elif leaf == "embed":
            value = draw * 0.5
        elif leaf == "router":
            value = draw * 2.0 * (param.shape[-1] ** -0.5)
        else:
            value = draw * (param.shape[-1] ** -0.5)
        weights[name] = value.to(torch.bfloat16).float()
    return weights


def make_weights(config: dict, seed: int) -> dict:
    entry = registry.lookup(config)
    model = entry.build(entry.config_class.from_dict(config))
    return draw_weights(model.all_named_params(), seed)


def write_folder(config: dict, seed: int, folder) -> dict:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    weights = make_weights(config, seed)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return weights


def random_tokens(config, count, seed):
    return torch.randint(0, config["vocab"], (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def plain_rows(requests, weights, config, low=None):
    """{(id, position): logits row} of the plain implementation (float64 arithmetic; with ``low`` float32
    arithmetic that rounds what the design allows in bfloat16)."""
    rows = {}
    for rid, tokens in requests.items():
        logits = plain.forward(config, weights, tokens, torch.float64 if low is None else torch.float32, low)
        for position in range(len(tokens)):
            rows[(rid, position)] = logits[position].float()
    return rows


CLOSE_CALL = 0.05      # a router margin below this fraction of the score is a choice that bfloat16 rounding can flip


def close_calls(requests, weights, config):
    """The (id, position) that a close call in the choice of experts can reach: the position of the close call itself
    (in any layer run) and, since later tokens attend to it, every later position of its request.  bfloat16 runs are
    not judged there (another expert is another function; the float32 runs are judged everywhere)."""
    found = set()
    for rid, tokens in requests.items():
        margins = []
        plain.forward(config, weights, tokens, torch.float64, margins=margins)
        if margins:
            close = (torch.stack(margins).min(dim=0).values < CLOSE_CALL).nonzero().flatten()
            if len(close):
                found |= {(rid, p) for p in range(int(close[0]), len(tokens))}
    return found
