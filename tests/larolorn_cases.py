"""Small Larolorn configurations and random weights for the tests.

The sizes differ from layer to layer and between the cases: latents whose key row is and is not a size the
tensor-core attention takes, value heads larger than, smaller than and equal to key heads, one to three query
heads per key/value head, rotations over all and over a few of a head's dimensions, windows and chunks of one
position, of a few and longer than every request, decays of exactly one and exactly zero, layers that run with
an earlier layer's tensors (of both kinds), layers without a feed-forward, multipliers of one and others.
"""
import json
from pathlib import Path

import torch

import qwen_inference_lab_b200.models  # noqa: F401  (registers the architectures)
from qwen_inference_lab_b200.config import registry
from qwen_inference_lab_b200.weights import write_safetensors
from tests.plain import larolorn_plain as plain


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, window):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                rot=dict(base=base, dims=rot_dim), mask=dict(size=window))


def left(heads, kv_heads, dim, vdim, scale, base, dims, chunk):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(base=base, dims=dims),
                mask=dict(size=chunk))


def right(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


_A0 = latent(3, 24, 8, 40, 24, 0.17, 10000.0, 20)
_A1 = dict(left=left(4, 2, 32, 32, 0.2, 300000.0, 16, 24), right=right(2, 16, 24, (0.9, 0.5)))
_A3 = dict(left=left(6, 3, 16, 8, 0.3, 1000.0, 16, 7), right=right(3, 40, 8, (1.0, 0.0, 0.97)))
CASE_A = dict(architecture="Larolorn", vocab=173, width=96, norm=dict(eps=1e-5), residual_mult=0.4, logit_scale=0.5, layers=[
    dict(type="latent_attention", mixer=_A0, mlp=dense(72, 3.0)),
    dict(type="parallel", mixer=_A1, mlp=dense(40, 1.5)),
    dict(type="latent_attention", mixer=_A0, mlp=dense(72, 3.0), weights_of=0),
    dict(type="parallel", mixer=_A3, mlp=None),
    dict(type="parallel", mixer=_A1, mlp=dense(40, 1.5), weights_of=1),
])
# a parallel layer first; a latent whose key row is 64 wide and one whose row of 14 no tensor-core kernel takes; a window of one
# position (a token sees itself); a chunk longer than every request; one key/value head and one recurrent head; multipliers of one
CASE_B = dict(architecture="Larolorn", vocab=97, width=64, norm=dict(eps=1e-6), residual_mult=1.0, logit_scale=1.0, layers=[
    dict(type="parallel", mixer=dict(left=left(2, 1, 80, 80, 0.11, 500.0, 80, 4096), right=right(1, 64, 64, (0.99,))),
         mlp=dense(48, 7.0)),
    dict(type="latent_attention", mixer=latent(2, 16, 16, 16, 48, 0.18, 100.0, 33), mlp=None),
    dict(type="latent_attention", mixer=latent(5, 12, 4, 20, 10, 0.25, 2000.0, 1), mlp=dense(24, 0.8)),
])
# awkward sizes: a width that is a multiple of nothing, one head, two rotated dimensions, a chunk of one position (a token
# sees itself and the sink), a window longer than every request, five small recurrent heads, both kinds of layer run twice
_C0 = latent(1, 6, 2, 10, 30, 0.4, 7.0, 4096)
_C1 = dict(left=left(3, 3, 20, 12, 0.22, 50.0, 4, 1), right=right(5, 10, 6, (0.3, 0.999, 0.8, 1.0, 0.61)))
CASE_C = dict(architecture="Larolorn", vocab=53, width=70, norm=dict(eps=1e-5), residual_mult=0.25, logit_scale=2.0, layers=[
    dict(type="latent_attention", mixer=_C0, mlp=dense(37, 0.5)),
    dict(type="parallel", mixer=_C1, mlp=dense(11, 2.5)),
    dict(type="parallel", mixer=_C1, mlp=dense(11, 2.5), weights_of=1),
    dict(type="latent_attention", mixer=_C0, mlp=dense(37, 0.5), weights_of=0),
])
CASES = {"A": dict(config=CASE_A, seed=5, page_size=4, lengths=(70, 9, 33, 150, 1, 50)),
         "B": dict(config=CASE_B, seed=6, page_size=16, lengths=(40, 3, 300, 64, 25)),
         "C": dict(config=CASE_C, seed=7, page_size=2, lengths=(31, 2, 77, 20, 45))}


def draw_weights(params: dict, seed: int) -> dict:
    """name -> CPU float32 tensor of bfloat16-representable values for ``params`` (name -> Param): weights of
    norms around one, biases small, sink scores of order one, the embedding of order one, matrices scaled by
    their input size."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, param in params.items():
        draw = torch.randn(param.shape, generator=generator)
        leaf = name.split(".")[-1]
        if leaf == "b":
            value = draw * 0.1
        elif leaf == "sink":
            value = draw
        elif len(param.shape) == 1:
            value = 1.0 + draw * 0.1
        elif leaf == "embed":
            value = draw
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
