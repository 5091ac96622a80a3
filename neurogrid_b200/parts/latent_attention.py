"""Latent attention: softmax attention whose keys and values are expanded from one cached latent per token."""
from __future__ import annotations

import torch

from ..cache.manager import PagedNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from . import registry
from .base import PositionArgs
from .registry import register


@register("mixer", "latent_attention")
class LatentAttention:
    """c_q = rmsnorm(W_dq x), q_h = W_uq,h c_q;  c = rmsnorm(W_dkv x), k_h = W_uk,h c, v_h = W_uv,h c;
    out = W_o concat_h( sigmoid(W_g x)_h * softmax(q_h k_h^T * scale) v_h ) over a window; no positions.

    Only c is cached (pages without a value half, one "head" of kv_rank columns, padded to a multiple
    of 16 with zeros).  The expansions are folded into the neighbouring matrices when the weights are
    bound (in float64, rounded once to the compute dtype):
        q_h . k_h = (W_uk,h^T W_uq,h c_q) . c        -> one matrix [heads * rank, q_rank] makes the queries
        W_o,h (g_h * W_uv,h sum_j p_j c_j)           -> one matrix [hidden, heads * rank] ends the mixer
    so the attention core is a multi-query attention in which every head reads the latent pages both as
    keys and as values: a block per row stages each tile of latents once for all heads.  Scores, softmax
    weights and their sum with the values are float32, keys are walked in ascending order, and the two
    norms and the gate are float32 too.  Long bfloat16 steps run the core on the tensor cores with the heads
    of a row as the rows of an MMA tile (exact products, float32 sums; the weights as three bfloat16 terms).

    With a rotated key part (``spec.rope_dim`` r): a cached row is [c | rotated key part | zeros], a head's query
    [W_uk,h^T q_h unrotated | q_h rotated part | zeros] (one product makes both, a row kernel then rotates the part), so
    the core's dot product over the whole row is the sum of the two scores; the head's weighted rows carry r
    coordinates that nothing reads.  With a gate per element (``spec.gate`` "element") W_uv cannot be folded into the
    output projection: a kernel expands each head's weighted latent by W_uv,h and applies the gate, then W_o follows.
    ``owns_cache`` False builds a layer that reads another latent layer's pages: it has no W_dkv and no norm of c."""

    graph_safe = True      # launches depend on device data and on launch-time constants only
    SPLIT_MAX_ROWS = 32    # steps of up to this many rows cut each row's keys into runs
    MAX_SPLITS = 16

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device, self.owns_cache = spec, dtype, device, owns_cache
        self.rope = getattr(spec, "rope_dim", 0)
        self.by_element = getattr(spec, "gate", "head") == "element"
        if not owns_cache and not self.rope and not self.by_element:
            raise ValueError("a latent attention layer of this form keeps its own cache")
        self.rank_p = -(-(spec.kv_rank + self.rope) // 16) * 16
        self.n_gate = spec.n_heads * spec.value_dim if self.by_element else spec.n_heads
        self.position = registry.build("position", spec.position, device=device) if self.rope else None
        self.w_down = self.w_q = self.w_out = self.w_uv = self.dq_norm = self.dkv_norm = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        d = {n["dq"]: TensorDecl((s.q_rank, s.hidden)), n["dq_norm"]: TensorDecl((s.q_rank,), "norm"),
             n["uq"]: TensorDecl((s.n_heads * (s.key_dim + self.rope), s.q_rank)),
             n["uk"]: TensorDecl((s.n_heads * s.key_dim, s.kv_rank)),
             n["uv"]: TensorDecl((s.n_heads * s.value_dim, s.kv_rank)),
             n["gate"]: TensorDecl((self.n_gate, s.hidden)),
             n["o"]: TensorDecl((s.hidden, s.n_heads * s.value_dim))}
        if self.owns_cache:
            d[n["dkv"]] = TensorDecl((s.kv_rank + self.rope, s.hidden))
            d[n["dkv_norm"]] = TensorDecl((s.kv_rank,), "norm")
        return d

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        H, rp = s.n_heads, self.rank_p
        self.w_down = torch.cat([t[n[p]].to(**kw) for p in (("dq", "dkv", "gate") if self.owns_cache else ("dq", "gate"))]).contiguous()
        self.dq_norm = t[n["dq_norm"]].to(**f32).contiguous()
        self.dkv_norm = t[n["dkv_norm"]].to(**f32).contiguous() if self.owns_cache else None
        uq = t[n["uq"]].double().view(H, s.key_dim + self.rope, s.q_rank)
        uk = t[n["uk"]].double().view(H, s.key_dim, s.kv_rank)
        uv = t[n["uv"]].double().view(H, s.value_dim, s.kv_rank)
        wo = t[n["o"]].double().view(s.hidden, H, s.value_dim)
        wq = torch.zeros(H, rp, s.q_rank, dtype=torch.float64)
        wq[:, :s.kv_rank] = torch.einsum("hdr,hdq->hrq", uk, uq[:, :s.key_dim])
        wq[:, s.kv_rank:s.kv_rank + self.rope] = uq[:, s.key_dim:]          # the part that is rotated: as it is stored
        self.w_q = wq.view(H * rp, s.q_rank).to(**kw).contiguous()
        if self.by_element:
            self.w_uv = t[n["uv"]].to(**kw).view(H, s.value_dim, s.kv_rank).contiguous()
            self.w_out = t[n["o"]].to(**kw).contiguous()
        else:
            wout = torch.zeros(s.hidden, H, rp, dtype=torch.float64)
            wout[:, :, :s.kv_rank] = torch.einsum("ohv,hvr->ohr", wo, uv)
            self.w_out = wout.view(s.hidden, H * rp).to(**kw).contiguous()

    def cache_need(self):
        return PagedNeed(1, self.rank_p, self.spec.window, values=False)

    def _position_args(self):
        """The rotation of the rotated part as the row kernels take it: a frequency per pair of the part; pairs behind
        the encoding's rotated coordinates get the frequency zero (they pass unchanged)."""
        if getattr(self, "_pa", None) is None:
            pa = PositionArgs.of(self.position.kernel_args())
            if pa.pos_scale != 1.0 or (pa.half_pairing and pa.inv_freq is not None and pa.inv_freq.numel() != self.rope // 2):
                raise NotImplementedError("the rotated part takes unscaled positions, and pairs (i, i + half) only whole")
            f = torch.zeros(self.rope // 2, dtype=torch.float32, device=self.device)
            if pa.inv_freq is not None:
                f[: pa.inv_freq.numel()] = pa.inv_freq.to(self.device)
            pa.inv_freq = f
            self._pa = pa
        return self._pa

    def kernels(self):
        jobs = [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("latent", None)]
        if ops.latent_core_mma_takes(self.spec.n_heads, self.rank_p, self.dtype):
            jobs.append(("latent_mma", {"NG_LAT_RANK": self.rank_p}))
        if not ops.latent_core_takes(self.spec.n_heads, self.rank_p):
            jobs.append(("attention_generic", None))
        return jobs

    def forward(self, x, ctx, cache):
        s = self.spec
        n, H, rp = x.shape[0], s.n_heads, self.rank_p
        if cache.writes and not self.owns_cache:
            raise RuntimeError("a latent attention layer without W_dkv cannot write a cache")
        writes = cache.writes
        w_down = self.w_down
        if self.owns_cache and not writes:       # has W_dkv but this run reads another cache: its rows are left out
            if getattr(self, "w_down_reader", None) is None:
                keep = list(range(s.q_rank)) + list(range(s.q_rank + s.kv_rank + self.rope, self.w_down.shape[0]))
                self.w_down_reader = self.w_down[keep].contiguous()
            w_down = self.w_down_reader
        down = ctx.ws.buf("lat_down", n, w_down.shape[0], self.dtype)
        ops.linear(x, w_down, None, down)
        cq = ctx.ws.buf("lat_cq", n, s.q_rank, self.dtype)
        gate = ctx.ws.buf("lat_gate", n, self.n_gate, torch.float32)
        pa = self._position_args() if self.rope else None
        ops.latent_prep(down, self.dq_norm, self.dkv_norm if writes else None, cq, cache.k_pages if writes else None, gate,
                        cache.table, ctx.positions, ctx.row_entry, self.n_gate, s.eps, ctx.status,
                        rot=self.rope if writes else 0, inv_freq=pa.inv_freq if pa else None,
                        half_pairing=bool(pa and pa.half_pairing))
        q = ctx.ws.buf("lat_q", n, H * rp, self.dtype)
        ops.linear(cq, self.w_q, None, q)
        if self.rope:
            ops.latent_rope_q(q, ctx.positions, ctx.row_entry, pa.inv_freq, H, s.kv_rank, pa.half_pairing)
        o = ctx.ws.buf("lat_o", n, H * rp, self.dtype)
        head_gate = None if self.by_element else gate
        if n > self.SPLIT_MAX_ROWS and ops.latent_core_mma_takes(H, rp, self.dtype):
            ops.latent_core_mma(q, cache.k_pages, cache.table, ctx.positions, ctx.row_entry, head_gate, o, H, s.window,
                                s.softmax_scale)
        elif ops.latent_core_takes(H, rp):
            # a step of few rows has too few blocks for the GPU: every row's keys are cut into runs, a block each
            n_splits = 1
            if n <= self.SPLIT_MAX_ROWS:
                longest = s.window or cache.table.shape[1] * cache.k_pages.shape[2]
                n_splits = max(1, min(self.MAX_SPLITS, 128 // n, longest // 64))
            partial = None
            if n_splits > 1:
                partial = ctx.ws.flat(f"lat_partial_{H}x{rp}", ops.latent_core_partial_floats(n, H, rp, n_splits), torch.float32,
                                      reserve=ops.latent_core_partial_floats(self.SPLIT_MAX_ROWS, H, rp, self.MAX_SPLITS))
            ops.latent_core(q, cache.k_pages, cache.table, ctx.positions, ctx.row_entry, head_gate, o, H, s.window,
                            s.softmax_scale, n_splits, partial)
        else:                                   # very many heads or a very wide latent: the plain kernel, then the gate
            ops.attention_generic(q, cache.k_pages, cache.k_pages, cache.table, ctx.positions, ctx.row_entry, o,
                                  H, s.window, s.softmax_scale)
            if head_gate is not None:
                ops.head_gate(o, gate, H)
        if self.by_element:                     # expand every head's weighted latent to its values, gate them, project
            a = ctx.ws.buf("lat_heads", n, H * s.value_dim, self.dtype)
            ops.head_up_gate(o, self.w_uv, gate, a)
            return ops.linear_to_residual(a, self.w_out, None, ctx.ws, "mixer_out", residual=ctx.residual)
        return ops.linear_to_residual(o, self.w_out, None, ctx.ws, "mixer_out", residual=ctx.residual)
