"""Tiny Dodilix configurations and weights for the tests.

The weights are drawn so that the mechanisms show in the logits: projections keep activations of order one, the matrices
behind attention scores are larger (a peaked softmax: a key wrongly seen or missed changes the output), sinks are of the
scores' size, the decay's bias ranges from forgetful to nearly none, the stream's copies are mixed by matrices far from
the identity, routers look at the token.  ``same_experts`` gives every routed expert of a layer the weights of its
first one, for comparisons in bfloat16: a close call of the router, which rounding may decide the other way, then
changes nothing (the weights still have to sum to the router's scale); the choice itself is tested in float32."""
from __future__ import annotations

import json
import os

import torch

from neurogrid_b200.config import config_from_dict
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.weights import write_file


def _left(heads, kv, dim, vdim, scale, chunk, rot=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        d["mask"] = {"size": chunk}
    if rot:
        d["rot"] = {"base": rot[0], "dims": rot[1]}
    return d


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def _parallel(left, right, mlp, scales=None):
    m = {"left": left, "right": right}
    if scales:
        m["left_scale"], m["right_scale"] = scales
    return {"type": "parallel", "mixer": m, "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, mlp, kv_from=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if rot_dim and base:
        m["rot"] = {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _moe(experts, top, ff, groups=None, shared=None, scale=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    d = {"kind": "moe", "router": r, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


# A: three copies of the stream, every option, a reader of an earlier layer's latents, grouped heads; sizes differ
# wherever two could be equal
DODI_A = {
    "architecture": "Dodilix", "vocab": 131, "width": 56, "streams": 3, "norm": {"eps": 2e-6}, "logit_scale": 0.6,
    "embedding": {"scale": 1.7},
    "layers": [
        _latent(3, 8, 4, 6, 20, 24, 0.3, 500.0, _moe(6, 2, 16, (3, 1), 24, 1.7)),
        _parallel(_left(4, 2, 16, 12, 0.3, 13, (1000.0, 8)), _right(3, 8, 10, 7.0, 5), {"kind": "dense", "ff": 40}, (0.7, 1.3)),
        _latent(2, 12, 4, 10, 16, 24, 0.25, 500.0, None, kv_from=0),
        _parallel(_left(6, 2, 8, 20, 0.4, 9, (50.0, 8)), _right(2, 24, 12, 3.0, 9), _moe(10, 3, 8, (5, 2), 16, 2.25), (1.2, 0.85)),
    ],
}

# B: values that could be equal are, or are 1, and what can be left out is: one stream's copy / none, one head, a chunk
# of one position, no mask, no rotation and a rotation of the whole head, no rotated part, one chosen expert, no groups,
# no shared expert, no scales
DODI_B = {
    "architecture": "Dodilix", "vocab": 61, "width": 40, "streams": 1, "norm": {"eps": 1e-5},
    "layers": [
        _parallel(_left(1, 1, 8, 8, 0.35, 1), _right(1, 8, 8, 1.0, 1), {"kind": "dense", "ff": 24}),
        _latent(1, 6, 0, 6, 6, 6, 0.4, 0.0, _moe(2, 1, 12)),
        _parallel(_left(2, 2, 6, 10, 0.5, None, (10000.0, 6)), _right(2, 5, 7, 11.0, 3), _moe(3, 3, 8, (3, 3))),
        _latent(2, 4, 6, 5, 7, 6, 0.5, 0.0, None),          # coordinates beside the head's that no rotation turns
    ],
}
DODI_B0 = {**{k: v for k, v in DODI_B.items() if k != "streams"}, "vocab": 67}      # plain residual sums

# C: chunks over many pages, head sizes the tensor-core kernels take (a KV group of four heads), a latent row of 64
# columns, recurrent heads the chunk-by-chunk kernels take, two readers of one layer's latents
DODI_C = {
    "architecture": "Dodilix", "vocab": 90, "width": 64, "streams": 2, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "embedding": {"scale": 0.75},
    "layers": [
        _parallel(_left(4, 1, 64, 64, 0.15, 70, (10000.0, 32)), _right(2, 32, 16, 8.0, 4), _moe(4, 2, 16, (4, 3), 24, 1.0), (0.9, 1.15)),
        _latent(4, 16, 8, 16, 24, 56, 0.2, 1000.0, {"kind": "dense", "ff": 48}),
        _parallel(_left(8, 2, 32, 16, 0.2, 33, (100.0, 32)), _right(4, 16, 48, 2.0, 8), None),
        _latent(5, 8, 8, 24, 16, 56, 0.3, 1000.0, _moe(4, 1, 16, None, 16), kv_from=1),
        _latent(2, 24, 8, 8, 32, 56, 0.2, 1000.0, None, kv_from=1),
    ],
}

# D: a width that is no multiple of four, five copies, a cached row wider than the latent cores take (272 columns: the
# plain attention kernel serves, with the gate behind it) and a reader of it, a key/value group of more heads than a tile has rows
DODI_D = {
    "architecture": "Dodilix", "vocab": 70, "width": 50, "streams": 5, "norm": {"eps": 1e-5}, "logit_scale": 0.8,
    "layers": [
        _latent(2, 10, 8, 14, 12, 264, 0.2, 300.0, {"kind": "dense", "ff": 30}, rot_dims=4),
        _parallel(_left(34, 2, 8, 6, 0.35, 21, (10.0, 4)), _right(1, 12, 20, 4.0, 2), None, (1.0, 0.5)),
        _latent(3, 6, 8, 9, 10, 264, 0.25, 300.0, _moe(5, 2, 10, None, None, 0.7), kv_from=0, rot_dims=4),
    ],
}

CONFIGS = {"A": (DODI_A, 41), "B": (DODI_B, 42), "B0": (DODI_B0, 43), "C": (DODI_C, 44), "D": (DODI_D, 45)}
PAGE_SIZE = {"A": 8, "B": 16, "B0": 4, "C": 8, "D": 8}


def draw_weights(config: dict, seed: int, router_gain: float = 3.0, same_experts: bool = False):
    """name -> bfloat16 tensor for every tensor the configuration declares."""
    decls = declare_tensors(config_from_dict(config).model_spec())
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(decls):
        d = decls[name]
        parts = name.split(".")
        leaf = parts[-1]
        rnd = lambda *s: torch.randn(*s, generator=g)
        if len(parts) > 1 and parts[1] in ("hc1", "hc2"):
            n = d.shape[0]
            if leaf == "in":
                t = 1.0 / n + 0.3 * rnd(d.shape)
            elif leaf == "out":
                t = 1.0 + 0.4 * rnd(d.shape)
            else:                                           # mixes the copies; columns sum to about one
                t = 0.6 * torch.eye(n) + 0.4 / n + 0.15 * rnd(d.shape)
        elif leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.2 * rnd(d.shape)
        elif leaf == "sink":
            t = 1.5 * rnd(d.shape)
        elif leaf == "b":                                   # the decay's bias: from forgetful to nearly no decay
            t = torch.linspace(-2.0, 6.0, d.shape[0])[torch.randperm(d.shape[0], generator=g)] + 0.3 * rnd(d.shape)
        elif name == "embed":
            t = rnd(d.shape)
        else:
            gain = {"q": 2.5, "k": 2.5, "uq": 2.5, "uk": 2.5, "dkv": 1.5, "head": 2.0, "router": router_gain, "sg": 2.0,
                    "a1": 2.0, "a2": 2.0}.get(leaf, 1.0)
            t = gain * rnd(d.shape) / d.shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    if same_experts:
        for name in out:
            parts = name.split(".")
            if len(parts) == 4 and parts[1] == "mlp" and parts[2][0] == "e" and parts[2][1:].isdigit():
                out[name] = out[".".join([parts[0], "mlp", "e0", parts[3]])]
    return out


def write_model(config: dict, seed: int, folder: str, weights=None, router_gain: float = 3.0, same_experts: bool = False) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_file(os.path.join(folder, "model.safetensors"), weights or draw_weights(config, seed, router_gain, same_experts))
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
