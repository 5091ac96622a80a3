"""Architecture-neutral descriptions of a decoder, produced by a typed model configuration.

A model configuration (one class per architecture, e.g. ``Lfm2Config``) turns the keys of
its ``config.json`` into a :class:`ModelSpec`: a tuple of :class:`LayerSpec` (one per
distinct layer, each naming its mixer, feed-forward, norms and block arrangement by
*spec objects*) and a ``schedule`` that says in which order layers run and whose cache
each run uses.  Parts are built from specs alone; no part sees the model configuration.

Every spec carries ``kind``: the key under which the part class is registered
(:mod:`neurogrid_b200.parts.registry`).  A new part brings its own frozen dataclass with a
``kind`` field; nothing here needs to change for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


def _names(**kw) -> Mapping[str, str]:
    return dict(kw)


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * w  (weight multiplies directly, no 1+w).
    ``tensor``: the weight's name relative to the norm's ("": it is stored under the norm's own name)."""
    size: int
    eps: float
    tensor: str = "weight"
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class LayerNormSpec:
    """y = (x - mean(x)) * rsqrt(var(x) + eps) * w, var the mean of the squared deviations; a weight and no bias.
    ``tensor``: the weight's name relative to the norm's ("": it is stored under the norm's own name)."""
    size: int
    eps: float
    tensor: str = "weight"
    kind: str = "layernorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the whole head.

    ``pairing`` "adjacent" rotates (2i, 2i+1); "half" rotates (i, i+head_dim/2).
    ``scale`` divides positions before the angle is formed (linear position scaling).
    ``rotary_dims`` (None: the whole head) rotates only the first that many coordinates of a head:
    pair i is (i, i + rotary_dims/2) or (2i, 2i+1), its angle pos * theta^(-2i/rotary_dims), and the
    rest of the head passes unchanged.
    ``freq_scaling`` = (factor, low, high, original) rescales the frequencies by their wavelength l = 2 pi / f:
    f stays where l < original / high, becomes f / factor where l > original / low, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
    """
    head_dim: int
    theta: float
    pairing: str = "half"
    scale: float = 1.0
    rotary_dims: Optional[int] = None
    freq_scaling: Optional[Tuple[float, float, float, float]] = None
    kind: str = "rope"

    def __post_init__(self):
        if self.pairing not in ("adjacent", "half"):
            raise ValueError(f"rope pairing must be 'adjacent' or 'half', got {self.pairing!r}")
        if self.head_dim % 2:
            raise ValueError("rope needs an even head_dim")
        if self.rotary_dims is not None and (self.rotary_dims % 2 or not 0 <= self.rotary_dims <= self.head_dim):
            raise ValueError(f"rotary_dims must be even and at most head_dim, got {self.rotary_dims}")


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding (queries and keys pass unchanged)."""
    kind: str = "none"


@dataclass(frozen=True)
class DistanceBiasSpec:
    """No rotation; positions enter the scores only: slope_h * (query position - key position) is taken off head h's
    score, slope_h = 2^(-``exponent`` * (h + 1) / n_heads)."""
    n_heads: int
    exponent: float = 8.0
    kind: str = "distance_bias"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache.

    ``window`` None = every earlier key is visible; W = only the last W keys (the query's own
    position included).  ``qk_norm`` applies an RMSNorm over head_dim to q and k (weights
    shared by all heads) before the position encoding.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: object
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None
    softmax_scale: Optional[float] = None      # None -> 1/sqrt(head_dim)
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        q="q_proj", k="k_proj", v="v_proj", o="o_proj", q_norm="q_norm", k_norm="k_norm"))
    kind: str = "attention"

    def __post_init__(self):
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if self.head_dim % 16 or not (16 <= self.head_dim <= 256):
            raise ValueError(f"head_dim must be a multiple of 16 in [16, 256], got {self.head_dim}")
        if self.window is not None and self.window < 1:
            raise ValueError("attention window must be >= 1")


@dataclass(frozen=True)
class MappedAttentionSpec:
    """Grouped-query attention whose scores and softmax weights are float32, with ``n_maps`` score maps per head.

    Query head h has ``n_maps`` queries of ``key_dim`` coordinates (rows of the q projection head by head as
    [map 0, map 1]), KV head g as many keys and ONE value of ``value_dim``.  Per map: RMS norm of q and k over
    key_dim (``qk_norm``; one weight each, shared by heads and maps), ``position`` on q and k,
    s = softcap * tanh(scale * q.k / softcap) (``softcap`` None: scale * q.k), softmax over the keys j <= i with
    i - j < ``window`` or j < ``keep_first`` (``window`` None: every j <= i).  One map: the head's output is the
    weighted values.  Two maps: o = a_0 - lambda a_1 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` (four
    vectors of key_dim, one lambda per layer), then o over its root mean square (``eps``, no weight) times
    (1 - diff).  ``bias``: q, k, v and the output projection have biases.
    ``cache_window`` / ``cache_keep_first``: what the layer's pages must keep: its own mask, or the widest mask among
    the layers that read its keys and values.
    ``norm_scope`` "projection": ONE RMS norm over all of q (before it is split into heads) and one over all of k, the
    weights as long as the projections, instead of a norm per head.  ``q_temp_coef`` c, ``q_temp_every`` m: q is
    multiplied by 1 + c ln(floor((p + 1) / m) + 1) at position p (c = 0: not).  ``sink``: a learned number per head
    whose exponential is one more term of the softmax's denominator; it has no key and no value, is not scaled and
    gets no bias.  A ``position`` with score slopes takes slope_h (i - j) off the scaled (and capped) score.
    ``chunk`` c: a query also sees only the keys of its own chunk, floor(j / c) = floor(i / c), chunks counted from the
    sequence's position 0 (``cache_window`` is then c: no later query reads further back).  ``norm_weight`` False: the
    RMS norm of q and k has no weights, and since a rotation keeps a head's sum of squares it may be taken on either
    side of ``position``.  ``out_gate``: the concatenated heads are multiplied element by element by the sigmoid of
    one more projection of the mixer's input (rows ``g``) before the output projection.
    """
    hidden: int
    n_heads: int
    n_kv_heads: int
    key_dim: int
    value_dim: int
    position: object
    softmax_scale: float
    n_maps: int = 1
    qk_norm: bool = False
    eps: float = 1e-6
    window: Optional[int] = None
    keep_first: int = 0
    softcap: Optional[float] = None
    diff: float = 0.0
    bias: bool = False
    cache_window: Optional[int] = None
    cache_keep_first: int = 0
    norm_scope: str = "head"
    q_temp_coef: float = 0.0
    q_temp_every: int = 1
    sink: bool = False
    chunk: Optional[int] = None
    norm_weight: bool = True
    out_gate: bool = False
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", o_bias="o.b", q_norm="q.norm",
        k_norm="k.norm", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2", sink="sink", out_gate="g"))
    kind: str = "mapped_attention"

    def __post_init__(self):
        if self.n_maps not in (1, 2):
            raise ValueError(f"mapped attention has one or two maps per head, got {self.n_maps}")
        if self.n_heads < 1 or self.n_kv_heads < 1 or self.n_heads % self.n_kv_heads:
            raise ValueError(f"n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if not (1 <= self.key_dim <= 512) or not (1 <= self.value_dim <= 256):
            raise ValueError(f"mapped attention: key_dim in [1, 512] and value_dim in [1, 256], got {self.key_dim}, {self.value_dim}")
        if self.window is not None and self.window < 1:
            raise ValueError("attention window must be >= 1")
        if self.keep_first < 0 or (self.softcap is not None and not self.softcap > 0):
            raise ValueError("keep_first must be >= 0 and softcap positive")
        if self.norm_scope not in ("head", "projection") or self.q_temp_every < 1:
            raise ValueError("norm_scope is 'head' or 'projection', q_temp_every at least 1")
        if self.chunk is not None and (self.chunk < 1 or self.window is not None or self.keep_first):
            raise ValueError("a chunked mask has a positive size and goes without a window or kept first tokens")
        if not self.norm_weight and self.norm_scope != "head":
            raise ValueError("a norm without weights is a norm per head")


@dataclass(frozen=True)
class ShortConvSpec:
    """Gated causal depthwise convolution of width ``width`` (state: last width-1 inputs)."""
    hidden: int
    width: int
    bias: bool = False
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        in_proj="in_proj", conv="conv", out_proj="out_proj"))
    kind: str = "short_conv"

    def __post_init__(self):
        if not (2 <= self.width <= 8):
            raise ValueError(f"short-conv width must be in [2, 8], got {self.width}")


@dataclass(frozen=True)
class SwiGLUSpec:
    """down( act(gate(x)) * up(x) ), no biases; ``activation`` "silu" or "gelu_tanh" (the tanh form of gelu).
    A tensor's name is its role's name plus ``weight_suffix``."""
    hidden: int
    intermediate: int
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        gate="gate_proj", up="up_proj", down="down_proj"))
    activation: str = "silu"
    weight_suffix: str = ".weight"
    kind: str = "swiglu"

    def __post_init__(self):
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: activation must be silu or gelu_tanh, got {self.activation!r}")


@dataclass(frozen=True)
class ScalarRMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * g with ONE gain g for all coordinates (the tensor has no dimensions)."""
    size: int
    eps: float
    kind: str = "rmsnorm_scalar"


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head and no softmax or denominator.

    Per head (key size ``key_dim``, value size ``value_dim``): S_t = decay * S_(t-1) + k_t v_t^T and
    o_t = S_t^T q_t, with q and k rotated by ``position`` and k scaled by key_dim^(-1/2) after the
    rotation.  Each head's o is divided by its root mean square (``eps``, no weight), the heads are
    gated by silu of a fourth projection and projected back.  State per request: S, float32, zero.
    """
    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    position: object
    eps: float
    names: Mapping[str, str] = field(default_factory=lambda: _names(q="q", k="k", v="v", gate="g", o="o"))
    kind: str = "retention"

    def __post_init__(self):
        if len(self.decay) != self.n_heads:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.n_heads} heads")
        if min(self.n_heads, self.key_dim, self.value_dim) < 1:
            raise ValueError("retention: heads and head sizes must be positive")


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention without positions whose keys and values are expanded from one latent per token.

    c_q = rmsnorm(W_dq x) (``q_rank`` wide), q = W_uq c_q;  c = rmsnorm(W_dkv x) (``kv_rank`` wide), per
    head k = W_uk c and v = W_uv c; only c is cached.  ``window`` None = every earlier key, W = the last W
    keys with the query's own.  Head h's output is multiplied by sigmoid(W_g x)_h before the output
    projection.  Both norms have plain weights and ``eps``.
    ``rope_dim`` r > 0: q has r more coordinates per head (laid out [key_dim | r]) and W_dkv r more rows, one key
    part shared by all heads and not normed; both are rotated by ``position`` (over all r coordinates) and the score
    is the sum of the two dot products.  The latent and the rotated key part are cached.  ``gate`` "element": the
    gate has a row per coordinate of the concatenated heads instead of one per head.
    """
    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    softmax_scale: float
    eps: float
    window: Optional[int] = None
    rope_dim: int = 0
    position: object = None
    gate: str = "head"
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", gate="g", o="o"))
    kind: str = "latent_attention"

    def __post_init__(self):
        if self.window is not None and self.window < 1:
            raise ValueError("attention window must be >= 1")
        if not (1 <= self.kv_rank <= 512):
            raise ValueError(f"latent attention: kv_rank must be in [1, 512], got {self.kv_rank}")
        if self.rope_dim < 0 or self.rope_dim % 2 or (self.rope_dim > 0) != (self.position is not None):
            raise ValueError("latent attention: a rotated key part has an even size and a position encoding")
        if self.gate not in ("head", "element"):
            raise ValueError("latent attention: the gate is per head or per element")


@dataclass(frozen=True)
class MoESpec:
    """Routed experts: of ``n_experts`` gated experts of width ``expert_ff`` each token uses ``top_k``; a shared expert
    of width ``shared_ff`` (0: none) runs for every token and is added.

    ``scoring`` "softmax": the top_k largest router logits (float32, with a bias), weighted by the softmax over the
    chosen logits.  ``scoring`` "sigmoid": scores s = sigmoid(logits), no bias; experts are chosen by s +
    ``correction`` (a stored vector, if ``correction``) among the ``keep_groups`` best of ``n_groups`` equal groups of
    neighbouring experts (a group's score: the sum of its two largest choice scores; the other groups' experts cannot
    be chosen), and weighted by s over the sum of the chosen s (+ 1e-20).
    ``activation`` "swiglu": silu(gate) * up.  "clamped_glu": g = min(gate, limit), u = clamp(up, -limit, limit),
    g sigmoid(``glu_alpha`` g) (u + 1); the shared expert has a ``shared_limit`` of its own.
    ``shared_gate``: the shared expert's output is multiplied by sigmoid(w . x), one number per token.
    ``scoring`` "softmax_all": scores s = softmax(logits) over ALL experts, no bias, and then as for sigmoid scores
    (correction, groups, s over the chosen sum).  ``group_score`` "top2" (the sum of a group's two largest choice
    scores) or "max".  ``route_scale`` multiplies the routing weights."""
    hidden: int
    n_experts: int
    top_k: int
    expert_ff: int
    shared_ff: int = 0
    scoring: str = "softmax"
    correction: bool = False
    n_groups: int = 1
    keep_groups: int = 1
    activation: str = "swiglu"
    limit: float = 0.0
    shared_limit: float = 0.0
    glu_alpha: float = 1.702
    shared_gate: bool = False
    group_score: str = "top2"
    route_scale: float = 1.0
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        expert="e{}", gate="gate", up="up", down="down", router="router", router_bias="router.b", shared="shared",
        correction="correction", shared_gate="shared.sg"))
    kind: str = "moe"

    def __post_init__(self):
        if not (1 <= self.top_k <= self.n_experts):
            raise ValueError(f"moe: top_k {self.top_k} must be in 1..{self.n_experts}")
        if self.top_k > 32:
            raise ValueError("moe: top_k above 32 is not supported")
        if self.scoring not in ("softmax", "sigmoid", "softmax_all") or self.activation not in ("swiglu", "clamped_glu"):
            raise ValueError("moe: scoring is softmax, sigmoid or softmax_all, activation swiglu or clamped_glu")
        if self.group_score not in ("top2", "max"):
            raise ValueError("moe: a group's score is top2 or max")
        if self.scoring == "softmax" and self.route_scale != 1.0:
            raise ValueError("moe: a scale of the routing weights goes with sigmoid or softmax_all scoring")
        if self.n_groups < 1 or self.n_experts % self.n_groups or not (1 <= self.keep_groups <= self.n_groups):
            raise ValueError(f"moe: {self.n_experts} experts do not form {self.n_groups} equal groups of which {self.keep_groups} are kept")
        if self.top_k > self.keep_groups * (self.n_experts // self.n_groups):
            raise ValueError("moe: the kept groups hold fewer experts than top_k")
        if self.scoring == "softmax" and (self.correction or self.n_groups > 1):
            raise ValueError("moe: a correction and groups go with sigmoid scoring")
        if self.activation == "clamped_glu" and not (self.limit > 0 and (self.shared_ff == 0 or self.shared_limit > 0)):
            raise ValueError("moe: the clamped activation needs positive limits")
        if self.shared_gate and not (self.shared_ff and self.scoring != "softmax"):
            raise ValueError("moe: a gate of the shared expert needs a shared expert and sigmoid or softmax_all scoring")


@dataclass(frozen=True)
class MLPSpec:
    """down(act(up x + b_up)) + b_down: an ungated feed-forward; ``activation`` "relu2" is the square of relu.
    ``bias``: both projections have biases."""
    hidden: int
    intermediate: int
    activation: str = "relu2"
    bias: bool = True
    names: Mapping[str, str] = field(default_factory=lambda: _names(up="up", down="down", up_bias="up.b", down_bias="down.b"))
    kind: str = "mlp"

    def __post_init__(self):
        if self.activation not in ("relu2",):
            raise ValueError(f"feed-forward: activation must be relu2, got {self.activation!r}")


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule: a recurrence per value head with a float32 state S [key_dim, value_dim],

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q      (the read-out sees the token's own write)

    q and k (``n_qk_heads`` heads of ``key_dim``; value head h uses head h // (n_heads / n_qk_heads)) and v (``n_heads``
    heads of ``value_dim``) are projections passed through a causal convolution over time per channel (``taps``
    taps, the last on the current token, no bias, zeros before the start) and silu; q and k are then unit vectors
    per head (x / sqrt(sum x^2 + 1e-6)), q times key_dim^(-1/2).  beta = sigmoid(W_b x) and the decay
    g = exp(-exp(A_log) softplus(W_a x + dt_bias)) are one number per value head.  Each head's o is divided by its root
    mean square (``eps``), multiplied by a weight of ``value_dim`` (shared by heads) and by silu(W_g x), then
    projected back.  State per request: S (zero at the start) and the convolution's last taps - 1 inputs."""
    hidden: int
    n_heads: int
    n_qk_heads: int
    key_dim: int
    value_dim: int
    taps: int
    eps: float
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", decay="a", a_log="A_log",
        dt_bias="dt_bias", norm="norm", gate="g", o="o"))
    kind: str = "gated_delta"

    def __post_init__(self):
        if self.n_heads < 1 or self.n_qk_heads < 1 or self.n_heads % self.n_qk_heads:
            raise ValueError(f"gated delta: {self.n_heads} value heads are not a multiple of {self.n_qk_heads} query/key heads")
        if not (1 <= self.key_dim <= 256) or self.value_dim < 1:
            raise ValueError(f"gated delta: key_dim in [1, 256] and a positive value_dim, got {self.key_dim}, {self.value_dim}")
        if not (1 <= self.taps <= 8):
            raise ValueError(f"gated delta: taps must be in [1, 8], got {self.taps}")


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is half the sum of their outputs, each first divided by its
    root mean square over the model width (``eps``) and multiplied by a plain weight of its own.
    ``combine`` "weighted": the result is left_scale * left + right_scale * right instead (no norms, no weights)."""
    hidden: int
    left: object
    right: object
    eps: float
    combine: str = "norm_mean"
    left_scale: float = 1.0
    right_scale: float = 1.0
    names: Mapping[str, str] = field(default_factory=lambda: _names(left="left", right="right", left_out="left.out",
                                                                   right_out="right.out"))
    kind: str = "side_by_side"

    def __post_init__(self):
        if self.combine not in ("norm_mean", "weighted"):
            raise ValueError("side by side: combine is norm_mean or weighted")


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention whose state decays per key channel and token:

        S <- diag(alpha_t) S + k_t v_t^T;   o_t = S^T q_t       (S [key_dim, value_dim] per head, float32, zero at the start)

    q = W_q x * key_dim^(-1/2), k = W_k x (``n_heads`` heads of ``key_dim``), v = W_v x (heads of ``value_dim``);
    alpha = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 x) + b, laid out heads x key_dim, through a low-rank pair of
    matrices (``decay_rank`` columns between them).  Each head's o is RMS-normed over value_dim with a plain weight
    shared by the heads (``eps``), the heads are multiplied by silu(W_g x) and projected back."""
    hidden: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    eps: float
    names: Mapping[str, str] = field(default_factory=lambda: _names(
        q="q", k="k", v="v", gate="g", o="o", norm="norm", decay_down="a1", decay_up="a2", decay_bias="a2.b"))
    kind: str = "gated_linear_attention"

    def __post_init__(self):
        if min(self.n_heads, self.key_dim, self.value_dim, self.decay_rank) < 1 or not self.tau > 0:
            raise ValueError("gated linear attention: heads, sizes and tau must be positive")


@dataclass(frozen=True)
class TokenPairSpec:
    """An embedding of the pair (previous token, token), added to the token's: row (previous * mul_prev + token * mul_cur)
    mod buckets of a table [buckets + 1, hidden]; a sequence's first token takes the last row."""
    buckets: int
    mul_prev: int
    mul_cur: int
    table_name: str = "bigram"

    def __post_init__(self):
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("token pairs: buckets must be positive and the multipliers not negative")


@dataclass(frozen=True)
class InputConvSpec:
    """What a sublayer reads, u, is replaced by u + conv(u): a causal convolution over time on each channel,
    conv(u)_t = sum_j w[:, j] * u_(t - taps + 1 + j), no bias.  State per request: the last taps-1 inputs."""
    hidden: int
    taps: int
    kind: str = "input_conv"

    def __post_init__(self):
        if not (1 <= self.taps <= 8):
            raise ValueError(f"input conv taps must be in [1, 8], got {self.taps}")


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, added after the feed-forward: e = table[token] (``dim`` wide,
    columns ``offset``..``offset+dim`` of a table shared by all layers), g = gelu_tanh(W_gate x) * e,
    y = W_proj g, x += rmsnorm(y) * w (plain weight)."""
    hidden: int
    dim: int
    offset: int
    table_name: str
    table_width: int
    vocab_size: int
    eps: float
    names: Mapping[str, str] = field(default_factory=lambda: _names(gate="gate", proj="proj", norm="norm"))
    kind: str = "token_side"


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: a block arrangement around a mixer and a feed-forward.

    ``prefix`` is the tensor-name prefix of the layer; ``names`` maps the four roles
    (mixer, ffn, mixer_norm, ffn_norm) to the sub-prefix used in the weight files.
    """
    mixer: object
    ffn: object
    mixer_norm: object
    ffn_norm: object
    prefix: str
    names: Mapping[str, str]
    block: str = "prenorm"
    options: Mapping[str, object] = field(default_factory=dict)   # what a block arrangement has besides the four parts


@dataclass(frozen=True)
class ScheduleEntry:
    """Run ``layer`` (index into ModelSpec.layers) with cache ``cache``.

    Cache ids form a namespace of their own; ``cache == layer`` with ``writes`` is the ordinary
    case.  The same ``layer`` may appear twice (shared weights), each time with a cache id of
    its own.  ``writes=False`` lets a layer read the keys and values that another entry wrote
    under that cache id, without adding its own; such a layer needs no k/v weights.
    """
    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    tie_head: bool
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    eos_token_ids: Tuple[int, ...] = ()
    embed_scale: float = 1.0                     # the token embeddings are multiplied by this
    position_table_name: Optional[str] = None    # a table [max_positions, hidden] of learned positions, added to the
                                                 # token embeddings (no LFM2 configuration has one)
    token_pair: Optional[object] = None          # a TokenPairSpec: an embedding of (previous token, token), added too
    logit_softcap: Optional[float] = None        # logits <- cap * tanh(logits / cap)
    logit_scale: float = 1.0                     # logits <- logits * scale
    streams: int = 0                             # > 0: the residual stream is that many copies (hyper-connections); every
                                                 # layer's block arrangement then keeps them ("hyper")

    def __post_init__(self):
        n = len(self.layers)
        if self.position_table_name and self.max_positions <= 0:
            raise ValueError("a table of learned positions needs max_positions")
        if self.streams < 0 or (self.streams > 0) != any(l.block == "hyper" for l in self.layers) \
                or (self.streams > 0 and not all(l.block == "hyper" for l in self.layers)):
            raise ValueError("a model with several copies of the stream has hyper blocks in every layer, and only such a model")
        writers = set()
        for e in self.schedule:
            if not (0 <= e.layer < n) or e.cache < 0:
                raise ValueError(f"schedule entry {e} names a layer outside 0..{n - 1} or a negative cache id")
            if e.writes:
                if e.cache in writers:
                    raise ValueError(f"schedule entry {e}: cache {e.cache} already has a writer")
                writers.add(e.cache)
            elif e.cache not in writers:
                raise ValueError(f"schedule entry {e} reads cache {e.cache} before any entry writes it")
