"""Typed configuration of the Fuzelorn decoder, read from its own ``config.json`` keys.

Fuzelorn is a pre-norm decoder (RMS norms with plain weights) whose layers are listed one by one in ``layers``.  A
layer of ``type`` ``parallel`` has two mixers side by side that read the same normed input, and the layer adds half the
sum of their outputs, each first RMS-normed over the width with a weight of its own:

* ``mixer.left``: grouped-query softmax attention without rotation.  One RMS norm over the whole q projection and one
  over the whole k projection (before the split into heads); q times a temperature that grows with the logarithm of
  the position; a distance bias slope_h (i - j) with slope_h = 2^(-8 (h + 1) / heads) taken off the scaled score; a
  sliding window; a learned sink per head in the softmax's denominator.
* ``mixer.right``: the gated delta rule (a recurrence with a float32 state per head) behind short causal
  convolutions of q, k and v.

The feed-forward (``mlp``, or null for none) is ``dense`` (down(relu(up x + b)^2) + b) or ``moe``: routed experts with
sigmoid scores, a correction added for the choice only, a choice limited to the best groups of experts, a clamped
gated activation, and a gated shared expert.  ``loop`` runs layers ``start`` .. ``stop`` - 1 ``times`` times in a row
with the same weights, each pass with a cache and state of its own.  Token embeddings are multiplied by
``embedding.scale``; ``embedding.bigram`` adds an embedding of the pair (previous token, token); the logits pass
``logit_softcap * tanh(logits / logit_softcap)``.

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.{scale, bigram.{buckets, mul_prev, mul_cur}}``,
``logit_softcap``, ``loop.{start, stop, times}``, ``layers[i].type``, ``layers[i].mixer.left.{heads, kv_heads, dim, vdim,
scale, mask.size, q_temp.{coef, every}}``, ``layers[i].mixer.right.{heads, kv_heads, dim, vdim, conv}``,
``layers[i].mlp.{kind, ff}`` or ``layers[i].mlp.{kind, router.{experts, top, groups.{count, keep}}, expert.{ff, limit},
shared.{ff, limit}}``.  Tensor names: ``embed``, ``bigram``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.left.{q, k, v, o,
q.norm, k.norm, sink, out}``, ``l<i>.mix.right.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, norm, g, o, out}``,
``l<i>.mlp.{up, up.b, down, down.b}`` or ``l<i>.mlp.{router, correction, e<j>.{gate, up, down}, shared.{gate, up, down,
sg}}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .metanex import _need
from .specs import (DistanceBiasSpec, GatedDeltaSpec, LayerSpec, MLPSpec, MappedAttentionSpec, ModelSpec, MoESpec,
                    RMSNormSpec, ScheduleEntry, SideBySideSpec, TokenPairSpec)

LAYER_TYPES = ("parallel",)
SLOPE_EXPONENT = 8.0        # slope_h = 2^(-8 (h + 1) / heads)
GLU_ALPHA = 1.702           # the clamped activation's sigmoid(alpha g)


@dataclass(frozen=True)
class FuzelornConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    bigram: Optional[Tuple[int, int, int]]        # (buckets, mul_prev, mul_cur)
    logit_softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times)
    layers: Tuple[Mapping[str, Any], ...]
    raw: Mapping[str, Any]

    architecture = "Fuzelorn"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FuzelornConfig":
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
            left, lp = m.get("left"), path + "mixer.left."
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _need(left, lp, key, int)
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"{lp}heads = {left['heads']} is not a multiple of kv_heads = {left['kv_heads']}")
            _need(left, lp, "scale", float)
            if left.get("mask") is not None:
                _need(left["mask"], lp + "mask.", "size", int)
            if left.get("q_temp") is not None:
                _need(left["q_temp"], lp + "q_temp.", "coef", float, positive=False)
                _need(left["q_temp"], lp + "q_temp.", "every", int)
            right, rp = m.get("right"), path + "mixer.right."
            for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                _need(right, rp, key, int)
            if right["heads"] % right["kv_heads"]:
                raise ConfigError(f"{rp}heads = {right['heads']} is not a multiple of kv_heads = {right['kv_heads']}")
            if right["conv"] > 8 or right["dim"] > 256:
                raise ConfigError(f"{rp}conv must be at most 8 and dim at most 256")
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
                    groups = r.get("groups")
                    count = _need(groups, mp + "router.groups.", "count", int) if groups is not None else 1
                    keep = _need(groups, mp + "router.groups.", "keep", int) if groups is not None else 1
                    if e % count or keep > count or top > keep * (e // count):
                        raise ConfigError(f"{mp}router: {e} experts in {count} groups of which {keep} are kept cannot give {top} experts")
                    _need(mlp.get("expert"), mp + "expert.", "ff", int)
                    _need(mlp.get("expert"), mp + "expert.", "limit", float)
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], mp + "shared.", "ff", int)
                        _need(mlp["shared"], mp + "shared.", "limit", float)
                else:
                    raise ConfigError(f"{mp}kind = {kind!r}; allowed: dense, moe")
        emb = d.get("embedding") or {}
        big = emb.get("bigram")
        bigram = None
        if big is not None:
            bigram = (_need(big, "embedding.bigram.", "buckets", int), _need(big, "embedding.bigram.", "mul_prev", int, positive=False),
                      _need(big, "embedding.bigram.", "mul_cur", int, positive=False))
            if bigram[1] < 0 or bigram[2] < 0:
                raise ConfigError("embedding.bigram: the multipliers must not be negative")
        loop = d.get("loop")
        lp3 = None
        if loop is not None:
            lp3 = (_need(loop, "loop.", "start", int, positive=False), _need(loop, "loop.", "stop", int, positive=False),
                   _need(loop, "loop.", "times", int))
            if not 0 <= lp3[0] <= lp3[1] <= len(layers):
                raise ConfigError(f"loop: start = {lp3[0]} and stop = {lp3[1]} must lie in order within 0..{len(layers)}")
        cfg = cls(vocab=_need(d, "", "vocab", int), width=_need(d, "", "width", int),
                  norm_eps=_need(d.get("norm"), "norm.", "eps", float),
                  embed_scale=_need(emb, "embedding.", "scale", float) if emb.get("scale") is not None else 1.0,
                  bigram=bigram,
                  logit_softcap=_need(d, "", "logit_softcap", float) if d.get("logit_softcap") is not None else None,
                  loop=lp3, layers=tuple(layers), raw=dict(d))
        if not math.isfinite(cfg.norm_eps):
            raise ConfigError("norm.eps must be finite")
        return cfg

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ------------------------------------------------------------------ the model, as data
    def layer_runs(self) -> Tuple[int, ...]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    def _mixer_spec(self, layer: Mapping[str, Any]) -> SideBySideSpec:
        D, m = self.width, layer["mixer"]
        l, r = m["left"], m["right"]
        mask, temp = l.get("mask"), l.get("q_temp")
        window = int(mask["size"]) if mask else None
        left = MappedAttentionSpec(
            hidden=D, n_heads=l["heads"], n_kv_heads=l["kv_heads"], key_dim=l["dim"], value_dim=l["vdim"],
            position=DistanceBiasSpec(l["heads"], SLOPE_EXPONENT), softmax_scale=float(l["scale"]), n_maps=1, qk_norm=True,
            eps=self.norm_eps, window=window, cache_window=window, norm_scope="projection",
            q_temp_coef=float(temp["coef"]) if temp else 0.0, q_temp_every=int(temp["every"]) if temp else 1, sink=True)
        right = GatedDeltaSpec(hidden=D, n_heads=r["heads"], n_qk_heads=r["kv_heads"], key_dim=r["dim"], value_dim=r["vdim"],
                               taps=r["conv"], eps=self.norm_eps)
        return SideBySideSpec(hidden=D, left=left, right=right, eps=self.norm_eps)

    def _ffn_spec(self, layer: Mapping[str, Any]):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if mlp.get("kind", "dense") == "dense":
            return MLPSpec(self.width, mlp["ff"], activation="relu2", bias=True)
        r, shared = mlp["router"], mlp.get("shared")
        groups = r.get("groups")
        return MoESpec(hidden=self.width, n_experts=r["experts"], top_k=r["top"], expert_ff=mlp["expert"]["ff"],
                       shared_ff=shared["ff"] if shared else 0, scoring="sigmoid", correction=True,
                       n_groups=int(groups["count"]) if groups else 1, keep_groups=int(groups["keep"]) if groups else 1,
                       activation="clamped_glu", limit=float(mlp["expert"]["limit"]),
                       shared_limit=float(shared["limit"]) if shared else 0.0, glu_alpha=GLU_ALPHA, shared_gate=bool(shared))

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = RMSNormSpec(D, self.norm_eps, tensor="")
        specs = []
        for i, layer in enumerate(self.layers):
            ffn = self._ffn_spec(layer)
            specs.append(LayerSpec(mixer=self._mixer_spec(layer), ffn=ffn, mixer_norm=norm,
                                   ffn_norm=norm if ffn is not None else None, prefix=f"l{i}.",
                                   names=dict(mixer="mix", ffn="mlp", mixer_norm="norm1", ffn_norm="norm2"),
                                   block="prenorm"))
        # every run of a layer has a cache id of its own: a looped layer shares weights, not keys, values or state
        schedule = tuple(ScheduleEntry(layer, run) for run, layer in enumerate(self.layer_runs()))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=D, layers=tuple(specs),
                         schedule=schedule, final_norm=norm, tie_head=False, max_positions=0,
                         embed_name="embed", final_norm_name="final.norm", head_name="head",
                         embed_scale=self.embed_scale,
                         token_pair=TokenPairSpec(*self.bigram) if self.bigram else None,
                         logit_softcap=self.logit_softcap)
