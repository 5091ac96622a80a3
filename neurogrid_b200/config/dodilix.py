"""Typed configuration of the Dodilix decoder, read from its own ``config.json`` keys.

Dodilix is a pre-norm decoder (RMS norms with plain weights) whose layers are listed one by one in ``layers``; with
``streams`` the residual stream is that many copies tied by hyper-connections (every sublayer reads a weighted sum of
the copies and writes into all of them through a mixing matrix), and the final norm reads their sum.

* ``type`` ``parallel``: two mixers side by side on the same normed input, result left_scale * left + right_scale *
  right.  ``mixer.left``: grouped-query softmax attention; a partial rotation in pairs (i, i + dims/2); q and k over
  their root mean square per head after the rotation (no weights); a chunked mask (a query sees the earlier keys of
  its own chunk of ``mask.size`` positions, chunks counted from the sequence's start); a learned sink per head in the
  softmax's denominator; a sigmoid output gate per coordinate of the concatenated heads.  ``mixer.right``: gated
  linear attention, a recurrence with a float32 state per head and a decay per key channel and token,
  sigmoid(z)^(1/tau) with z from a low-rank pair of projections; heads RMS-normed with a shared weight, a silu gate.
* ``type`` ``latent_attention``: causal softmax attention whose queries pass a normed latent (``q_rank``) and whose
  keys and values are expanded from a normed latent (``kv_rank``) per token; q and k also have ``rot_dim`` rotated
  coordinates (pairs (2i, 2i+1)), the key's shared by all heads; a sigmoid output gate per coordinate.  ``kv_from: j``:
  the layer has no latent projection of its own and reads what layer j cached.

The feed-forward (``mlp``, or null for none) is ``dense`` (down(silu(gate x) * up x)) or ``moe``: softmax scores over all
experts, the choice limited to the best groups (a group's score: its largest), the chosen scores over their sum times
``router.scale``, and a shared expert times the sigmoid of one more projection.  Token embeddings are multiplied by
``embedding.scale`` and the logits by ``logit_scale``.

Keys: ``architecture``, ``vocab``, ``width``, ``streams``, ``norm.eps``, ``embedding.scale``, ``logit_scale``,
``layers[i].type``, ``layers[i].mixer.{left_scale, right_scale}``, ``layers[i].mixer.left.{heads, kv_heads, dim, vdim,
scale, mask.size, rot.{base, dims}}``, ``layers[i].mixer.right.{heads, dim, vdim, tau}``, ``layers[i].mixer.{heads, dim,
rot_dim, vdim, q_rank, kv_rank, scale, rot.{base, dims}, kv_from}``, ``layers[i].mlp.{kind, ff}`` or
``layers[i].mlp.{kind, router.{experts, top, scale, groups.{count, keep}}, expert.ff, shared.ff}``.  Sizes that no key
gives (the decay's low rank) are read from the tensors' shapes when the model is loaded: ``decay_rank`` defaults to
the value ``layers[i].mixer.right.decay_rank`` or 16.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.hc1.{in, out, mix}``, ``l<i>.hc2.{in, out, mix}``, ``l<i>.mix.left.{q, k, v, g, o, sink}``,
``l<i>.mix.right.{q, k, v, g, o, norm, a1, a2, a2.b}``, ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}``,
``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, e<j>.{gate, up, down}, shared.{gate, up, down, sg}}``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .metanex import _need
from .specs import (GatedLinearAttentionSpec, LatentAttentionSpec, LayerSpec, MappedAttentionSpec, ModelSpec, MoESpec,
                    NoPositionSpec, RMSNormSpec, RopeSpec, ScheduleEntry, SideBySideSpec, SwiGLUSpec)

LAYER_TYPES = ("parallel", "latent_attention")
MAX_STREAMS = 16
DEFAULT_DECAY_RANK = 16


def _rot(m: Mapping[str, Any], path: str, whole: int) -> Optional[Tuple[float, int]]:
    """(base, dims) of a mixer's ``rot`` or None; dims even and at most ``whole``."""
    rot = m.get("rot")
    if rot is None:
        return None
    base = _need(rot, path + "rot.", "base", float)
    dims = _need(rot, path + "rot.", "dims", int, positive=False) if rot.get("dims") is not None else whole
    if dims < 0 or dims % 2 or dims > whole:
        raise ConfigError(f"{path}rot.dims = {dims} must be even and at most {whole}")
    return (base, dims) if dims else None


@dataclass(frozen=True)
class DodilixConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    logit_scale: float
    streams: int                                  # 0: one stream and plain residual sums
    layers: Tuple[Mapping[str, Any], ...]
    decay_ranks: Tuple[Optional[int], ...]        # per layer, what ``with_shapes`` read off the weight files
    raw: Mapping[str, Any]

    architecture = "Dodilix"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DodilixConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks required key 'layers' (a list of layer descriptions)")
        for i, layer in enumerate(layers):
            path = f"layers[{i}]."
            t = _need(layer, path, "type", str)
            if t not in LAYER_TYPES:
                raise ConfigError(f"{path}type = {t!r}; allowed: {', '.join(LAYER_TYPES)}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json lacks required key {path}mixer")
            if t == "parallel":
                left, lp = m.get("left"), path + "mixer.left."
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _need(left, lp, key, int)
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{lp}heads = {left['heads']} is not a multiple of kv_heads = {left['kv_heads']}")
                _need(left, lp, "scale", float)
                if left.get("mask") is not None:
                    _need(left["mask"], lp + "mask.", "size", int)
                _rot(left, lp, left["dim"])
                right, rp = m.get("right"), path + "mixer.right."
                for key in ("heads", "dim", "vdim"):
                    _need(right, rp, key, int)
                _need(right, rp, "tau", float)
                for key in ("left_scale", "right_scale"):
                    if m.get(key) is not None:
                        _need(m, path + "mixer.", key, float, positive=False)
            else:
                mp = path + "mixer."
                for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _need(m, mp, key, int)
                _need(m, mp, "scale", float)
                rot_dim = _need(m, mp, "rot_dim", int, positive=False) if m.get("rot_dim") is not None else 0
                if rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"{mp}rot_dim = {rot_dim} must be even and not negative")
                _rot(m, mp, rot_dim)                    # rot.dims at most rot_dim: the part's first coordinates are rotated
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
                        raise ConfigError(f"{mp}kv_from = {src!r} must name an earlier layer")
                    sm = layers[src].get("mixer", {})
                    if layers[src].get("type") != "latent_attention" or sm.get("kv_from") is not None:
                        raise ConfigError(f"{mp}kv_from = {src}: that layer keeps no latents of its own")
                    mine, theirs = (m["kv_rank"], rot_dim, m.get("rot")), (sm.get("kv_rank"), sm.get("rot_dim") or 0, sm.get("rot"))
                    if mine != theirs:
                        raise ConfigError(f"{mp}kv_from = {src}: kv_rank, rot_dim and rot must equal that layer's")
            mlp = layer.get("mlp")
            if mlp is not None:
                mp = path + "mlp."
                kind = mlp.get("kind", "dense")
                if kind == "dense":
                    _need(mlp, mp, "ff", int)
                elif kind == "moe":
                    r = mlp.get("router")
                    e = _need(r, mp + "router.", "experts", int)
                    top = _need(r, mp + "router.", "top", int)
                    if r.get("scale") is not None:
                        _need(r, mp + "router.", "scale", float)
                    groups = r.get("groups")
                    count = _need(groups, mp + "router.groups.", "count", int) if groups is not None else 1
                    keep = _need(groups, mp + "router.groups.", "keep", int) if groups is not None else 1
                    if e % count or keep > count or top > keep * (e // count):
                        raise ConfigError(f"{mp}router: {e} experts in {count} groups of which {keep} are kept cannot give {top} experts")
                    _need(mlp.get("expert"), mp + "expert.", "ff", int)
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], mp + "shared.", "ff", int)
                else:
                    raise ConfigError(f"{mp}kind = {kind!r}; allowed: dense, moe")
        emb = d.get("embedding") or {}
        streams = 0
        if d.get("streams") is not None:
            streams = _need(d, "", "streams", int)
            if streams > MAX_STREAMS:
                raise ConfigError(f"streams = {streams}; at most {MAX_STREAMS}")
        cfg = cls(vocab=_need(d, "", "vocab", int), width=_need(d, "", "width", int),
                  norm_eps=_need(d.get("norm"), "norm.", "eps", float),
                  embed_scale=_need(emb, "embedding.", "scale", float) if emb.get("scale") is not None else 1.0,
                  logit_scale=_need(d, "", "logit_scale", float) if d.get("logit_scale") is not None else 1.0,
                  streams=streams, layers=tuple(layers), decay_ranks=(None,) * len(layers), raw=dict(d))
        if not math.isfinite(cfg.norm_eps):
            raise ConfigError("norm.eps must be finite")
        return cfg

    def to_dict(self) -> dict:
        return dict(self.raw)

    def with_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "DodilixConfig":
        """The configuration with the sizes that only the weight files give: the low rank between the decay's two
        projections, the first dimension of ``l<i>.mix.right.a1``."""
        ranks = []
        for i, layer in enumerate(self.layers):
            shape = shapes.get(f"l{i}.mix.right.a1")
            ranks.append(int(shape[0]) if shape and layer["type"] == "parallel" else None)
        return DodilixConfig(**{**self.__dict__, "decay_ranks": tuple(ranks)})

    # ------------------------------------------------------------------ the model, as data
    def _mixer_spec(self, i: int, layer: Mapping[str, Any]):
        D, m = self.width, layer["mixer"]
        if layer["type"] == "latent_attention":
            rot_dim = int(m.get("rot_dim") or 0)
            rot = _rot(m, f"layers[{i}].mixer.", rot_dim)
            position = RopeSpec(rot_dim, rot[0] if rot else 1.0, "adjacent", rotary_dims=rot[1] if rot else 0) if rot_dim else None
            return LatentAttentionSpec(hidden=D, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], q_rank=m["q_rank"],
                                       kv_rank=m["kv_rank"], softmax_scale=float(m["scale"]), eps=self.norm_eps, window=None,
                                       rope_dim=rot_dim, position=position, gate="element")
        l, r = m["left"], m["right"]
        rot = _rot(l, f"layers[{i}].mixer.left.", l["dim"])
        position = RopeSpec(l["dim"], rot[0], "half", rotary_dims=rot[1]) if rot else NoPositionSpec()
        chunk = int(l["mask"]["size"]) if l.get("mask") else None
        left = MappedAttentionSpec(
            hidden=D, n_heads=l["heads"], n_kv_heads=l["kv_heads"], key_dim=l["dim"], value_dim=l["vdim"], position=position,
            softmax_scale=float(l["scale"]), n_maps=1, qk_norm=True, norm_weight=False, eps=self.norm_eps, chunk=chunk,
            cache_window=chunk, sink=True, out_gate=True)
        rank = self.decay_ranks[i] or int(r.get("decay_rank") or DEFAULT_DECAY_RANK)
        right = GatedLinearAttentionSpec(hidden=D, n_heads=r["heads"], key_dim=r["dim"], value_dim=r["vdim"], decay_rank=rank,
                                         tau=float(r["tau"]), eps=self.norm_eps)
        return SideBySideSpec(hidden=D, left=left, right=right, eps=self.norm_eps, combine="weighted",
                              left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)))

    def _ffn_spec(self, layer: Mapping[str, Any]):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if mlp.get("kind", "dense") == "dense":
            return SwiGLUSpec(self.width, mlp["ff"], names=dict(gate="gate", up="up", down="down"), weight_suffix="")
        r, shared = mlp["router"], mlp.get("shared")
        groups = r.get("groups")
        return MoESpec(hidden=self.width, n_experts=r["experts"], top_k=r["top"], expert_ff=mlp["expert"]["ff"],
                       shared_ff=shared["ff"] if shared else 0, scoring="softmax_all",
                       n_groups=int(groups["count"]) if groups else 1, keep_groups=int(groups["keep"]) if groups else 1,
                       group_score="max", route_scale=float(r.get("scale", 1.0)), shared_gate=bool(shared))

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = RMSNormSpec(D, self.norm_eps, tensor="")
        specs = []
        for i, layer in enumerate(self.layers):
            ffn = self._ffn_spec(layer)
            names = dict(mixer="mix", ffn="mlp", mixer_norm="norm1", ffn_norm="norm2", mixer_hc="hc1", ffn_hc="hc2")
            specs.append(LayerSpec(mixer=self._mixer_spec(i, layer), ffn=ffn, mixer_norm=norm,
                                   ffn_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=names,
                                   block="hyper" if self.streams else "prenorm",
                                   options=dict(streams=self.streams) if self.streams else {}))
        # a layer with ``kv_from`` reads the pages its source layer wrote: the same cache id, no write of its own
        schedule = []
        for i, layer in enumerate(self.layers):
            src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            schedule.append(ScheduleEntry(i, i if src is None else int(src), writes=src is None))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=D, layers=tuple(specs),
                         schedule=tuple(schedule), final_norm=norm, tie_head=False, max_positions=0,
                         embed_name="embed", final_norm_name="final.norm", head_name="head",
                         embed_scale=self.embed_scale, logit_scale=self.logit_scale, streams=self.streams)
