"""Tiny Fuzelorn configurations and weights for the tests.

The weights are drawn so that the mechanisms show in the logits: projections keep activations of order one, the
matrices behind attention scores are larger (a peaked softmax: a key wrongly seen or missed changes the output), sinks
are of the scores' size, decays range from forgetful to nearly none, corrections reorder the experts, routers look at
the token.  ``router_gain`` small gives routers that hardly look at the token (the corrections then decide), for
comparisons in bfloat16, where a close call of the router would otherwise flip an expert."""
from __future__ import annotations

import json
import os

import torch

from neurogrid_b200.config import config_from_dict
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.weights import write_file


def _left(heads, kv, dim, vdim, scale, window, temp=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        d["mask"] = {"size": window}
    if temp:
        d["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return d


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, ff, limit, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    d = {"kind": "moe", "router": r, "expert": {"ff": ff, "limit": limit}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def _layer(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


# S: grouped heads on both sides, every option, the middle layers looped; sizes differ wherever two could be equal
FUZE_S = {
    "architecture": "Fuzelorn", "vocab": 151, "width": 72, "norm": {"eps": 3e-6}, "logit_softcap": 9.0,
    "embedding": {"scale": 1.6, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 11}},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(_left(4, 2, 16, 24, 0.3, 9, (0.7, 5)), _right(4, 2, 8, 12, 3), {"kind": "dense", "ff": 40}),
        _layer(_left(6, 2, 8, 12, 0.4, 13, (0.3, 2)), _right(2, 1, 24, 20, 4), _moe(6, 2, 24, 1.5, (3, 2), (32, 0.8))),
        _layer(_left(2, 2, 24, 8, 0.25, 30), _right(3, 3, 12, 16, 2), None),
        _layer(_left(4, 1, 16, 16, 0.35, 17, (1.1, 16)), _right(4, 2, 16, 8, 5), _moe(8, 3, 16, 0.9, (2, 1), (16, 2.5))),
    ],
}

# U: values that could be equal are, or are 1: one head, a window of one token, one tap, one expert chosen, one group
# (none named), no shared expert, no loop, no pairs, no temperature, no cap, no embedding scale, no mask in one layer
FUZE_U = {
    "architecture": "Fuzelorn", "vocab": 61, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_left(1, 1, 8, 8, 0.35, 1), _right(1, 1, 8, 8, 1), {"kind": "dense", "ff": 24}),
        _layer(_left(2, 1, 6, 10, 0.5, None), _right(2, 2, 5, 7, 2), _moe(2, 1, 12, 1.0)),
        _layer(_left(1, 1, 12, 5, 0.3, 6), _right(2, 1, 9, 3, 8), _moe(3, 3, 8, 0.6, (3, 3))),
    ],
}

# W: windows over many pages, head sizes the tensor-core kernels take, the whole stack looped three times, groups of
# one expert, more experts kept than chosen, recurrent heads wider than a warp's share
FUZE_W = {
    "architecture": "Fuzelorn", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
    "embedding": {"scale": 0.75, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 1}},
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _layer(_left(4, 2, 32, 16, 0.2, 70, (0.4, 32)), _right(2, 2, 40, 20, 4), _moe(4, 2, 16, 1.2, (4, 3), (24, 1.0))),
        _layer(_left(8, 2, 16, 32, 0.3, 33), _right(4, 1, 72, 36, 3), {"kind": "dense", "ff": 48}),
    ],
}

# V: layers whose scratch needs differ: attention without a mask over hundreds of keys (a step of few rows cuts them
# into runs) with other head counts and value sizes in every layer, recurrent heads of two sizes that both run chunk by
# chunk; a step's fixed workspace must hold every layer's share
FUZE_V = {
    "architecture": "Fuzelorn", "vocab": 120, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
    "embedding": {"scale": 1.25, "bigram": {"buckets": 19, "mul_prev": 5, "mul_cur": 2}},
    "layers": [
        _layer(_left(2, 1, 16, 16, 0.3, None), _right(2, 1, 16, 16, 3), {"kind": "dense", "ff": 32}),
        _layer(_left(8, 2, 32, 48, 0.25, None, (0.2, 50)), _right(4, 2, 32, 48, 4), _moe(4, 2, 16, 1.0, (2, 1), (16, 1.5))),
        _layer(_left(4, 4, 16, 32, 0.3, 150), _right(3, 3, 8, 32, 2), None),
    ],
}

CONFIGS = {"S": (FUZE_S, 31), "U": (FUZE_U, 32), "W": (FUZE_W, 33), "V": (FUZE_V, 34)}
PAGE_SIZE = {"S": 8, "U": 16, "W": 8, "V": 16}


def draw_weights(config: dict, seed: int, router_gain: float = 3.0):
    """name -> bfloat16 tensor for every tensor the configuration declares."""
    decls = declare_tensors(config_from_dict(config).model_spec())
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(decls):
        d = decls[name]
        leaf = name.split(".")[-1]
        rnd = lambda *s: torch.randn(*s, generator=g)
        if leaf in ("norm", "norm1", "norm2", "out"):
            t = 1.0 + 0.2 * rnd(d.shape)
        elif leaf == "sink":
            t = 1.5 * rnd(d.shape)
        elif leaf == "A_log":
            t = torch.linspace(-3.0, 0.5, d.shape[0]) + 0.2 * rnd(d.shape)
        elif leaf == "dt_bias":
            t = rnd(d.shape)
        elif leaf == "correction":
            t = 0.4 * rnd(d.shape)
        elif leaf == "conv":
            t = 0.6 * rnd(d.shape)
        elif leaf == "b" and len(d.shape) == 1:
            t = 0.3 * rnd(d.shape)
        elif name in ("embed", "bigram"):
            t = rnd(d.shape)
        else:
            gain = {"q": 2.5, "k": 2.5, "head": 2.0, "router": router_gain, "sg": 2.0, "a": 2.0, "b": 2.0}.get(leaf, 1.0)
            if ".right." in name and leaf in ("q", "k", "v"):
                gain = 2.0
            t = gain * rnd(d.shape) / d.shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(config: dict, seed: int, folder: str, weights=None, router_gain: float = 3.0) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_file(os.path.join(folder, "model.safetensors"), weights or draw_weights(config, seed, router_gain))
    return folder


def load_plain(folder: str):
    """(config mapping, name -> float64 tensor) of a model folder."""
    from neurogrid_b200.weights.safetensors_io import MappedFiles, read_header
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    files = MappedFiles()
    w = {k: files.read(e).double() for k, e in read_header(os.path.join(folder, "model.safetensors")).items()}
    files.close()
    return cfg, w
