#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the LFM2-1.2B shape, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]
                    [--shape 1.2b|700m|350m] [--prompt-len N] [--workload mixed350m|long700m|metanex|rofulorn|fuzelorn|dodilix]

A "step" is one decode step of the batch.  The default run has the layer sizes of the
LFM2-1.2B configuration, a batch of 8 and requests that hold 2,048-token prompts and grow
toward a context of 4,096.  One JSON line is printed:

* ``value``     decoded tokens a second, timed on the device around regions of K steps of the step
                function; a region is repeated until the regions together last a quarter of a second,
                ``ms_per_step`` is the median of the regions' means and ``spread`` their extremes;
* ``e2e``       the same through ``Engine.step()``: host token ids in (pinned host memory ->
                device every step) and sampled token ids back on the host every step;
* ``prefill``   one 2,048-token prompt in one step, logits of the last row;
* ``roofline``  bytes a decode step has to read (every weight once, the live requests' keys,
                values and states) / its time, against the measured copy bandwidth;
* ``points``    decode tokens a second at batch 1 and 64;
* ``mixed_step`` a step that holds a 100-token prompt portion beside the batch's decode tokens: device
                milliseconds and the host's milliseconds to launch it;
* ``step_ms``   the distribution of single decode steps (one CUDA event per step);
* ``kernels``   device time of the kernels that carry a step: decode attention, the gate/up
                product with its gate, the down product and the LM head at decode sizes; portion
                attention, gate/up (+ gate kernel) and down at 2,048 rows;
* ``gpu_launches``  kernel nodes of the decode graph that the timed steps replay (asked from the
                CUDA runtime) times the steps timed.

``--impl reference`` runs the reference's own CUDA library through its stock C entry points
(baseline/reference_arm.py) for the same metric and prints the same line with ``"impl":
"reference"``.  ``--workload`` runs one of the other two workloads of the benchmark set through
``Engine.generate`` and prints a line of its own.  For N > 1 GPUs it prints one line that says so
and exits with 2: the engine is single-GPU.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# LFM2-1.2B layer sizes (the benchmark configuration); random weights N(0, 0.02)
LFM2_1_2B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=65536, hidden_size=2048,
    num_hidden_layers=16,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv",
                 "full_attention", "conv", "full_attention", "conv", "full_attention", "conv", "full_attention", "conv"],
    num_attention_heads=32, num_key_value_heads=8, block_ff_dim=12288, block_auto_adjust_ff_dim=True,
    block_multiple_of=256, block_ffn_dim_multiplier=1.0, conv_L_cache=3, conv_bias=False, tie_embedding=True,
    rope_theta=1000000.0, norm_eps=1e-5, max_position_embeddings=128000,
)
PROMPT, CONTEXT, PREFILL_TOKENS = 2048, 4096, 2048
MIN_REGION_S = 0.25                    # timed regions are repeated until they last this long together
# the other published LFM2 shapes (same layer pattern, 8 KV heads of 64): --shape
SHAPES = {"1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288),
          "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10240),
          "350m": dict(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656)}
SHAPE_NAMES = {"1.2b": "LFM2-1.2B", "700m": "LFM2-700M", "350m": "LFM2-350M"}
PUBLISHED_BASELINE_TOK_S = 362.0      # the reference's best published batch-1 decode figure (GH200)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    out = dict(FALLBACK_PEAKS)
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            flat = {}

            def walk(o):
                if isinstance(o, dict):
                    for k, v in o.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat:
                out["hbm_gbs"] = flat["hbm_gbs"]
                src = "measured"
            if "bf16_tflops" in flat:
                out["bf16_tflops"] = flat["bf16_tflops"]
        except (ValueError, OSError):
            pass
    out["source"] = src
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu=0):
        self.rows, self.proc, self.gpu = [], None, gpu

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, lo=0, hi=None):
        rows = self.rows[lo:hi]
        sm = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(rows[0][1]) if rows and rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def shape_config(args):
    cfg = dict(LFM2_1_2B)
    cfg.update(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["layer_types"] = cfg["layer_types"][: args.layers]
    return cfg, full_layers


def ffn_width(cfg):
    """SwiGLU width of an LFM2 config.json (2/3 of block_ff_dim, scaled, rounded up to the multiple)."""
    if not cfg.get("block_auto_adjust_ff_dim"):
        return cfg["block_ff_dim"]
    d = int(cfg.get("block_ffn_dim_multiplier", 1.0) * int(2 * cfg["block_ff_dim"] / 3))
    m = cfg["block_multiple_of"]
    return m * ((d + m - 1) // m)


def model_numbers(c):
    """Parameter bytes a decode step reads, flops per token, KV bytes per token, state bytes of a
    configuration object (``Lfm2Config``)."""
    H, I, V = c.hidden_size, c.intermediate_size, c.vocab_size
    qd, kd = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    n_attn = sum(t == "full_attention" for t in c.layer_types)
    n_conv = len(c.layer_types) - n_attn
    conv_p = 3 * H * H + H * H + H * c.conv_L_cache
    attn_p = (qd + 2 * kd) * H + H * qd + 2 * c.head_dim
    ffn_p = 3 * H * I
    layer_p = n_conv * (conv_p + ffn_p + 2 * H) + n_attn * (attn_p + ffn_p + 2 * H)
    head_p = V * H
    mm_per_tok = 2 * (n_conv * (4 * H * H) + n_attn * ((qd + 2 * kd) * H + H * qd) + len(c.layer_types) * ffn_p)
    return dict(weight_bytes=2 * (layer_p + head_p + H), layer_params=layer_p, head_params=head_p,
                kv_bytes_per_token=n_attn * 2 * kd * 2, state_bytes=n_conv * (c.conv_L_cache - 1) * H * 4,
                mm_flops_per_token=mm_per_tok, head_flops_per_row=2 * head_p, n_attn=n_attn, qd=qd,
                head_dim=c.head_dim, n_heads=c.num_attention_heads)


def describe(c, shape, full_layers, batch, page_size, prompt, context, weight_bytes):
    """The flat ``config`` of the JSON line, read from the configuration that ran."""
    return {"model": f"{SHAPE_NAMES[shape]} shape, random weights", "hidden": c.hidden_size, "ffn": c.intermediate_size,
            "vocab": c.vocab_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
            "head_dim": c.head_dim, "conv_L": c.conv_L_cache, "layers": c.num_hidden_layers, "layers_full": full_layers,
            "attn_layers": sum(t == "full_attention" for t in c.layer_types), "global_batch": batch,
            "seq_len": context, "prompt_len": prompt, "page_size": page_size, "parallelism": "1 GPU",
            "l2": f"not flushed: each step reads {weight_bytes / 1e9:.1f} GB of weights, far more than L2",
            "weights_gb": round(weight_bytes / 1e9, 3)}


def flush_l2(buf):
    buf.add_(1)                                    # a buffer larger than L2, written between timed steps


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def run_ours(args):
    import torch
    from neurogrid_b200 import Engine
    from neurogrid_b200.engine import StepEntry
    from neurogrid_b200.sampling import SamplingParams

    prompt_len, context = (args.prompt_len, 2 * args.prompt_len) if args.prompt_len else (PROMPT, CONTEXT)
    cfg, full_layers = shape_config(args)
    pk = peaks()
    clocks = ClockSampler(0)
    clocks.start()
    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    # long contexts: no batch-64 point; one request more than the batch for the mixed step's portion
    max_batch = max(args.batch + 1, 64 if not args.prompt_len else 0)
    eng = Engine(config=cfg, random_weights=0, dtype="bf16", gpu=0, max_seq_len=context, page_size=args.page_size,
                 max_requests=max_batch, max_tokens_per_step=max(PREFILL_TOKENS, max_batch),
                 num_pages=max_batch * context // args.page_size)
    runner = eng.runner
    runner.keep_graphs = True
    nums = model_numbers(eng.config)
    l2 = torch.zeros(192 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    if args.profile_only:
        runner.cuda_graphs = False
        ids = [f"p{i}" for i in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (prompt_len,), generator=g).tolist(), [])])
        for _ in range(args.warmup + args.steps):
            runner.step([StepEntry(r, [5], [0]) for r in ids])
        torch.cuda.synchronize()
        clocks.stop()
        print("profile run done")
        return

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(3 + 7):
        flush_l2(l2)
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry("pf", prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.finish("pf")
        if i >= 3:
            times.append(a.elapsed_time(b))
    pf_ms = median(times)
    T = PREFILL_TOKENS
    attn_flops = nums["n_attn"] * 4 * nums["qd"] * (T * (T + 1) // 2)
    pf_flops = T * nums["mm_flops_per_token"] + attn_flops + nums["head_flops_per_row"]
    prefill = {"value": round(T / pf_ms * 1e3, 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(pf_flops / (pf_ms * 1e-3) / 1e12, 1), "of": pk["source"],
               "spread_ms": [round(min(times), 3), round(max(times), 3)]}

    # ---------------------------------------------------------------- decode, device-timed
    def decode_point(batch, steps, warmup, distribution=False):
        """Requests with `prompt_len` tokens in the cache, then regions of `steps` timed decode steps
        until the regions last MIN_REGION_S together (at least three)."""
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            toks_p = torch.randint(0, V, (prompt_len,), generator=g).tolist()
            for at in range(0, prompt_len, PREFILL_TOKENS):              # long prompts go in portions
                runner.step([StepEntry(rid, toks_p[at:at + PREFILL_TOKENS], [])])
        toks = torch.randint(0, V, (batch,), generator=g).tolist()
        entries = lambda: [StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]
        for _ in range(warmup):
            runner.step(entries())
        mark = clocks.mark()
        room = context - prompt_len - warmup - 2
        regions, total_ms, used = [], 0.0, 0
        while (len(regions) < 3 or total_ms < MIN_REGION_S * 1e3) and used + steps <= room:
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            for _ in range(steps):                           # exactly `steps` steps in one timed region
                runner.step(entries())
            b.record()
            torch.cuda.synchronize()
            regions.append(a.elapsed_time(b) / steps)
            total_ms += regions[-1] * steps
            used += steps
        ctx_mid = prompt_len + warmup + used // 2
        dist = None
        if distribution and used + 128 <= room:
            evs = [ev() for _ in range(129)]
            torch.cuda.synchronize()
            evs[0].record()
            for i in range(128):
                runner.step(entries())
                evs[i + 1].record()
            torch.cuda.synchronize()
            per = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(128))
            dist = {"p50": round(per[64], 4), "p90": round(per[115], 4), "p99": round(per[126], 4),
                    "max": round(per[-1], 4), "steps": 128}
        span = (mark, clocks.mark())
        for rid in ids:
            runner.finish(rid)
        return median(regions), regions, ctx_mid, dist, span

    t_first = clocks.mark()
    ms, regions, ctx_mid, dist, _ = decode_point(args.batch, args.steps, args.warmup, distribution=True)
    nodes = runner.graph_kernel_nodes()
    decode_nodes = max((n for k, n in nodes.items() if k[0] != "portion"), default=0)
    step_bytes = nums["weight_bytes"] + args.batch * (ctx_mid * nums["kv_bytes_per_token"] + 2 * nums["state_bytes"])
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    for b in (1, 64):
        if b > max_batch:
            continue
        if b == args.batch:
            points[f"decode_b{b}"] = round(b / ms * 1e3, 1)
            continue
        pms, _, _, _, _ = decode_point(b, max(8, args.steps // 2), args.warmup)
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)

    # ---------------------------------------------------------------- a mixed step: a 100-token portion beside the batch's decode tokens
    def mixed_point(portion=100):
        ids = [f"m{i}" for i in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (min(prompt_len, 1024),), generator=g).tolist(), [])])
        def one():
            entries = [StepEntry("mp", torch.randint(0, V, (portion,), generator=g).tolist(), [portion - 1])] + \
                      [StepEntry(r, [5], [0]) for r in ids]
            t0 = time.perf_counter()
            runner.step(entries)
            return (time.perf_counter() - t0) * 1e3

        # what the host needs to launch one such step, the device idle (the first two meet the shape and capture it)
        host = []
        for it in range(5):
            torch.cuda.synchronize()
            host.append(one())
        # the steps launched back to back, as a serving loop does: the period between the ends of two steps is the
        # device's time for one as long as the host needs less
        ends = [ev() for _ in range(9)]
        torch.cuda.synchronize()
        ends[0].record()
        for it in range(8):
            one()
            ends[it + 1].record()
        torch.cuda.synchronize()
        dev_ms = [ends[i].elapsed_time(ends[i + 1]) for i in range(8)]
        for rid in ids + ["mp"]:
            runner.finish(rid)
        return {"portion": portion, "decode_tokens": args.batch, "ms": round(median(dev_ms[2:]), 4),
                "host_ms": round(median(host[2:]), 4)}

    mixed = mixed_point() if context - 8 * 100 > 1100 else None

    # ---------------------------------------------------------------- decode, end to end through Engine.step()
    budget = context - prompt_len - 4
    for i in range(args.batch):
        eng.add_request(torch.randint(0, V, (prompt_len,), generator=g).tolist(),
                        SamplingParams(temperature=0.0, max_new_tokens=budget, ignore_eos=True))
    while any(r.pending > 1 or not r.output for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()                                                    # prefill until every request decodes
    for _ in range(args.warmup):
        eng.step()
    h0, d0 = eng.h2d_bytes, eng.d2h_bytes
    e2e_regions, total_s, used = [], 0.0, args.warmup + 2
    while (len(e2e_regions) < 3 or total_s < MIN_REGION_S) and used + args.steps < budget:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        e2e_regions.append(dt * 1e3 / args.steps)
        total_s += dt
        used += args.steps
    e2e_ms = median(e2e_regions)
    n_e2e = len(e2e_regions) * args.steps
    e2e = {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "spread_ms": [round(min(e2e_regions), 4), round(max(e2e_regions), 4)], "regions": len(e2e_regions),
           "h2d_bytes_per_step": (eng.h2d_bytes - h0) // n_e2e, "d2h_bytes_per_step": (eng.d2h_bytes - d0) // n_e2e}
    time.sleep(0.06)                                   # let the last clock sample of the timed regions arrive
    clocks.stop()
    clock_summary = clocks.summary(t_first, None)

    kernels = kernel_times(eng, args.batch, prompt_len, l2) if not args.no_kernels else None

    value = args.batch / ms * 1e3
    shape_name = SHAPE_NAMES[args.shape]
    line = {"metric": f"decode tok/s @ batch {args.batch} ({shape_name} shape)", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
            "spread_ms": [round(min(regions), 4), round(max(regions), 4)], "regions": len(regions),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(points.get("decode_b1", 0.0) / PUBLISHED_BASELINE_TOK_S, 2),
            "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02)",
            "config": describe(eng.config, args.shape, full_layers, args.batch, args.page_size, prompt_len, context,
                               nums["weight_bytes"]),
            "e2e": e2e, "gpu_launches": decode_nodes * args.steps, "launches_per_step": decode_nodes, "prefill": prefill,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes),
                         "of": pk["source"]},
            "points": points, "mixed_step": mixed, "step_ms": dist, "kernels": kernels, "clocks": clock_summary, "impl": "ours"}
    print(json.dumps(line))


def kernel_times(eng, batch, ctx_len, l2):
    """Device microseconds of the kernels that carry a step, each alone with the model's own weights
    (a different layer's every launch, so that nothing is left in L2 from the launch before): the
    launches are captured in a CUDA graph, as the step's are, and CUDA events time its replays, so
    that a kernel of a few microseconds is not measured by the host's launch rate.  Back-to-back
    launches of one kernel overlap their edges (programmatic dependent launch), as they do in the step."""
    import torch
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts.attention import decode_splits
    model, dev = eng.model, eng.device
    ffns = [b.ffn for b in model.blocks]
    attn = next((b.mixer for b in model.blocks if type(b.mixer).__name__ == "Attention"), None)
    H, I = model.spec.hidden, ffns[0].spec.intermediate
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=dev) * 0.05).to(torch.bfloat16)

    def timed(fn, n=48, reps=4):
        for i in range(4):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                fn(i)
        graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return round(a.elapsed_time(b) / (n * reps) * 1e3, 2)

    out = {"unit": "us", "decode_rows": batch, "prefill_rows": PREFILL_TOKENS}
    L = len(ffns)
    # ---- decode sizes
    x, act = rnd(batch, H), rnd(batch, I)
    o_act = torch.empty(batch, I, dtype=torch.bfloat16, device=dev)
    h = torch.zeros(batch, H, dtype=torch.float32, device=dev)
    from neurogrid_b200.parts.base import Workspace
    ws = Workspace(max(batch, 16), dev)
    out["decode_gate_up_swiglu"] = timed(lambda i: ops.gemm_swiglu_sm100(x, ffns[i % L].w_gate_up, o_act))
    out["decode_down_residual"] = timed(lambda i: ops.linear_to_residual(act, ffns[i % L].w_down, None, ws, "k", residual=h))
    # the smaller products, the norm and the conv of a decode step
    convs = [b.mixer for b in model.blocks if type(b.mixer).__name__ == "ShortConv"]
    norms = [b.ffn_norm for b in model.blocks]
    nbuf = torch.empty(batch, H, dtype=torch.bfloat16, device=dev)
    hs = torch.randn(batch, H, generator=g, device=dev)
    out["decode_norm"] = timed(lambda i: ops.add_rmsnorm(hs, None, norms[i % L].weight, nbuf, 1e-5))
    if convs:
        C = len(convs)
        out["decode_conv_in_proj"] = timed(lambda i: ops.linear_to_residual(x, convs[i % C].w_in, None, ws, "ci"))
        out["decode_out_proj_residual"] = timed(lambda i: ops.linear_to_residual(x, convs[i % C].w_out, None, ws, "co", residual=h))
        p_in = ops.linear_to_residual(x, convs[0].w_in, None, ws, "ci")
        st = torch.zeros(batch, convs[0].spec.width - 1, H, device=dev)
        cu1 = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        cb1 = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
        sl1 = torch.arange(batch, dtype=torch.int32, device=dev)
        out["decode_shortconv"] = timed(lambda i: ops.shortconv(p_in, convs[i % C].w_conv, None, st, nbuf, cu1, cb1, sl1, batch, 1))
    logits = torch.empty(batch, model.spec.vocab_size, dtype=torch.float32, device=dev)

    def head(i):
        l2.add_(1)                                    # there is one head: clear L2 of it between launches
        ops.linear(x, model.head_weight, None, logits)

    def flush_only(i):
        l2.add_(1)

    out["decode_lm_head"] = round(timed(head, 12) - timed(flush_only, 12), 2)
    if attn is not None:
        s = attn.spec
        ps = eng.runner.storage.page_size
        pages_each = -(-(ctx_len + 1) // ps)
        n_pages = batch * pages_each
        kp = [rnd(n_pages, s.n_kv_heads, ps, s.head_dim) for _ in range(3)]
        vp = [rnd(n_pages, s.n_kv_heads, ps, s.head_dim) for _ in range(3)]
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, pages_each).contiguous()
        cu = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        cb = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
        q = rnd(batch, s.n_heads * s.head_dim)
        o = torch.empty_like(q)
        n_splits = decode_splits(batch, s.n_kv_heads, ctx_len + 1, None, dev)
        scratch = torch.empty(max(1, ops.attn_decode_scratch_floats(batch, s.n_heads, s.head_dim, n_splits)), device=dev)
        out["decode_attention"] = timed(lambda i: ops.attn_decode_bf16(q, kp[i % 3], vp[i % 3], table, cu, cb, o, scratch,
                                                                      batch, s.n_heads, None, attn.scale, n_splits, ctx_len + 1))
        out["decode_attention_ctx"] = ctx_len
        out["decode_qkv"] = timed(lambda i: ops.linear_to_residual(x, attn.w_qkv, None, ws, "qk"))
        qkv1 = ops.linear_to_residual(x, attn.w_qkv, None, ws, "qk")
        pa1 = attn.position.kernel_args()
        pos1 = torch.full((batch,), ctx_len, dtype=torch.int32, device=dev)
        re1 = torch.arange(batch, dtype=torch.int32, device=dev)
        out["decode_rope_cache"] = timed(lambda i: ops.rope_cache(
            qkv1, q, attn.q_norm, attn.k_norm, pa1.inv_freq, pa1.half_pairing, pa1.pos_scale, kp[i % 3], vp[i % 3], table,
            pos1, re1, s.n_heads, s.n_kv_heads, s.head_dim, s.qk_norm_eps, eng.runner.status))
        # ---- a 2,048-token portion
        T = PREFILL_TOKENS
        pages_p = -(-T // ps)
        kq, vq = rnd(pages_p, s.n_kv_heads, ps, s.head_dim), rnd(pages_p, s.n_kv_heads, ps, s.head_dim)
        tab_p = torch.arange(pages_p, dtype=torch.int32, device=dev).view(1, pages_p)
        cu_p = torch.tensor([0, T], dtype=torch.int32, device=dev)
        cb_p = torch.zeros(1, dtype=torch.int32, device=dev)
        qp = rnd(T, s.n_heads * s.head_dim)
        op = torch.empty_like(qp)
        qkv_p = rnd(T, (s.n_heads + 2 * s.n_kv_heads) * s.head_dim)
        pos_p = torch.arange(T, dtype=torch.int32, device=dev)
        re_p = torch.zeros(T, dtype=torch.int32, device=dev)
        pa = attn.position.kernel_args()
        out["prefill_rope_cache"] = timed(lambda i: ops.rope_cache(
            qkv_p, qp, attn.q_norm, attn.k_norm, pa.inv_freq, pa.half_pairing, pa.pos_scale, kq, vq, tab_p, pos_p, re_p,
            s.n_heads, s.n_kv_heads, s.head_dim, s.qk_norm_eps, eng.runner.status), 16)
        pf = ops.attn_prefill_sm100 if ops.attn_prefill_sm100_takes(s.head_dim, ps) else ops.attn_prefill_bf16
        out["prefill_attention"] = timed(lambda i: pf(qp, kq, vq, tab_p, cu_p, cb_p, op, 1, T, s.n_heads, None, attn.scale,
                                                      False), 16)
    T = PREFILL_TOKENS
    xp, gu, ap = rnd(T, H), torch.empty(T, 2 * I, dtype=torch.bfloat16, device=dev), rnd(T, I)
    acts, outp = torch.empty(T, I, dtype=torch.bfloat16, device=dev), torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def gate_up(i):
        ops.linear(xp, ffns[i % L].w_gate_up, None, gu)
        ops.swiglu(gu, acts)

    out["prefill_gate_up_swiglu"] = timed(gate_up, 16)
    out["prefill_down"] = timed(lambda i: ops.linear(ap, ffns[i % L].w_down, None, outp), 16)
    return out


def run_workload(args):
    """The two other workloads of the benchmark set, through the Python entry point."""
    import torch
    from neurogrid_b200 import Engine

    g = torch.Generator().manual_seed(0)
    cfg = dict(LFM2_1_2B)
    if args.workload == "mixed350m":
        # LFM2-350M shape: 64 requests, prompts of 128..8,192 tokens, 256 new tokens each at temperature 0.7, 32k context
        cfg.update(SHAPES["350m"])
        n_req, new = 64, 256
        lens = torch.randint(128, 8193, (n_req,), generator=g).tolist()
        eng = Engine(config=cfg, random_weights=0, dtype="bf16", max_seq_len=32768, max_requests=n_req,
                     max_tokens_per_step=8192, chunk_size=2048, num_pages=n_req * 8448 // 16 + n_req)
        kw = dict(max_new_tokens=new, temperature=0.7, seed=1, ignore_eos=True)
        name = "LFM2-350M shape, 64 requests, prompts 128..8192, 256 new tokens at temperature 0.7"
    else:
        # LFM2-700M shape: 8 requests of 32,768-token prompts in 2,048-token portions, then 512 greedy tokens each
        cfg.update(SHAPES["700m"])
        n_req, new = 8, 512
        lens = [32768] * n_req
        eng = Engine(config=cfg, random_weights=0, dtype="bf16", max_seq_len=33792, max_requests=n_req,
                     max_tokens_per_step=2048 + n_req, chunk_size=2048, num_pages=n_req * 33792 // 16)
        kw = dict(max_new_tokens=new, temperature=0.0, ignore_eos=True)
        name = "LFM2-700M shape, 8 requests of 32768-token prompts in 2048-token portions, 512 greedy tokens"
    prompts = [torch.randint(0, 65536, (n,), generator=g).tolist() for n in lens]
    clocks = ClockSampler(0)
    clocks.start()
    runs = []
    for _ in range(max(1, args.repeat)):
        s0 = eng.stats()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, **kw)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        s1 = eng.stats()
        assert all(len(o) == new for o in outs)
        steps = s1["steps"] - s0["steps"]
        runs.append({"total_s": round(dt, 3), "new_tokens_per_s": round(n_req * new / dt, 1),
                     "tokens_per_s": round((sum(lens) + n_req * new) / dt, 1), "steps": steps,
                     "eager_step_share": round((s1["eager_steps"] - s0["eager_steps"]) / max(1, steps), 4),
                     "preemptions": s1["preemptions"] - s0["preemptions"]})
    time.sleep(0.06)
    clocks.stop()
    best = min(runs, key=lambda r: r["total_s"])
    print(json.dumps({"workload": args.workload, "what": name, "prompt_tokens": sum(lens), "new_tokens": n_req * new,
                      **best, "runs": runs, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
                      "clocks": clocks.summary(), "impl": "ours"}))


# ---------------------------------------------------------------------------------------------- --workload metanex
def metanex_config(width, layers):
    """A Metanex configuration with layers of a real model's sizes: three retention layers to one latent
    attention layer, routed experts whose widths add up to about four times the model's, a shared expert."""
    heads = width // 128
    ret = {"type": "retention", "mixer": {"heads": heads, "dim": 128, "vdim": 128,
                                          "decay": [1.0 - 2.0 ** (-5 - 6 * h / max(1, heads - 1)) for h in range(heads)],
                                          "rot": {"dims": 64, "base": 1000000.0}}}
    lat = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "q_rank": 768, "kv_rank": 128,
                                                 "scale": 128 ** -0.5, "mask": {"size": 1024}}}
    mlp = {"kind": "moe", "router": {"experts": 16, "top": 4}, "expert": {"ff": width // 4}, "shared": {"ff": width // 2}}
    pattern = [ret, ret, lat, ret]
    return {"architecture": "Metanex", "vocab": 65536, "width": width, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
            "token_side": {"dim": 64},
            "layers": [dict(pattern[i % 4], mlp=mlp) for i in range(layers)]}


def design_arm(arm, cfg, row, args, l2):
    """One configuration with random weights through the engine's step function: prefill of one 2,048-token prompt
    in one step, then decode at batch 8 and 1 after 2,048 tokens; fills ``row`` under the arm's name and returns
    the engine.  CUDA events; the L2 is flushed between timed steps."""
    import torch
    from neurogrid_b200 import Engine
    from neurogrid_b200.engine import StepEntry
    eng = Engine(config=cfg, random_weights=0, dtype="bf16", max_seq_len=8192, max_requests=8,
                 max_tokens_per_step=2048, num_pages=8 * 4096 // 16)
    r = eng.runner
    r.keep_graphs = True            # for the count of kernel nodes in the decode graph
    V = eng.model.spec.vocab_size
    g = torch.Generator().manual_seed(1)
    toks = lambda n: torch.randint(0, V, (n,), generator=g).tolist()

    def timed(fn, reps):
        ts = []
        for _ in range(reps):
            flush_l2(l2)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return median(ts)

    # prefill: one request's 2,048-token prompt in one step (the third meeting of the shape replays its graph)
    n_pre = [0]

    def prefill():
        rid = ("p", n_pre[0])
        n_pre[0] += 1
        r.step([StepEntry(rid, toks(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
        r.finish(rid)

    for _ in range(3):
        prefill()
    torch.cuda.synchronize()
    ms = timed(prefill, 5)
    row[arm + "_prefill_ms"] = round(ms, 3)
    row[arm + "_prefill_tok_s"] = round(PREFILL_TOKENS / ms * 1e3)
    # decode: 8 requests (and 1) that hold 2,048 tokens each, one token a step
    for i in range(8):
        r.step([StepEntry(("d", i), toks(PREFILL_TOKENS), [])])
    for batch in (8, 1):
        step = lambda: r.step([StepEntry(("d", i), toks(1), [0]) for i in range(batch)])
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        ms = timed(step, 24)
        row[f"{arm}_decode{batch}_ms"] = round(ms, 4)
        row[f"{arm}_decode{batch}_tok_s"] = round(batch / ms * 1e3)
    r.check_status()
    row[arm + "_weights_gb"] = round(eng.model.weight_bytes() / 1e9, 3)
    row[arm + "_decode_launches"] = max((n for k, n in r.graph_kernel_nodes().items() if k[0] != "portion"), default=0)
    return eng


def run_metanex(args):
    """Prefill and decode throughput of the Metanex design at layer sizes of a real model, beside LFM2 (the closest
    existing model: a hybrid of state layers and attention layers) at equal width and depth, and the design's own
    kernels one by one with what they must move or compute.  One JSON line.  Random weights, synthetic token ids;
    CUDA events; the L2 is flushed between timed steps."""
    import torch
    from neurogrid_b200 import Engine
    from neurogrid_b200.engine import StepEntry
    pk = peaks()
    l2 = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda:0")
    clocks = ClockSampler(0)
    clocks.start()
    results = []
    for width, layers in ((1024, 16), (2048, 16)):
        lfm2 = dict(LFM2_1_2B)
        lfm2.update(SHAPES["350m" if width == 1024 else "1.2b"])
        arms = {"metanex": metanex_config(width, layers), "lfm2": lfm2}
        row = {"width": width, "layers": layers}
        for arm, cfg in arms.items():
            eng = design_arm(arm, cfg, row, args, l2)
            if arm == "metanex" and not args.no_kernels:
                row["kernels"] = metanex_kernel_times(eng, l2, pk)
            del eng
            torch.cuda.empty_cache()
        results.append(row)
    time.sleep(0.06)
    clocks.stop()
    print(json.dumps({"workload": "metanex", "what": "Metanex beside LFM2 at equal width and depth: prefill of 2,048 tokens, "
                      "decode at batch 8 and 1 after 2,048 tokens", "results": results, "dtype": "bf16",
                      "data": "synthetic token ids, random-init weights", "peaks": pk, "clocks": clocks.summary(),
                      "impl": "ours"}))


def metanex_kernel_times(eng, l2, pk):
    """The design's own kernels alone (CUDA events around one launch, L2 flushed before it, median of 7), with the
    bytes each must move and the float32 operations it must do: microseconds, and the fraction of the measured copy
    bandwidth (or, for the chunked retention, of the float32 FFMA rate of the SMs at the clock seen)."""
    import torch
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts.base import Workspace
    from neurogrid_b200.parts import PagedView, SlotView, StepContext
    model, dev = eng.model, eng.device
    D = model.spec.hidden
    ret = next(b.mixer for b in model.blocks if type(b.mixer).__name__ == "Retention")
    lat = next(b.mixer for b in model.blocks if type(b.mixer).__name__ == "LatentAttention")
    blk = model.blocks[0]
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=dev)).to(torch.bfloat16)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)

    def timed(fn):
        ts = []
        for _ in range(9):
            flush_l2(l2)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return median(ts[2:])

    out = {"unit": "us"}
    bw = pk["hbm_gbs"] * 1e9

    def mem(name, us, nbytes):
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "of_copy_bandwidth": round(nbytes / (us * 1e-6) / bw, 3)}

    for rows, entries in ((PREFILL_TOKENS, 1), (8, 8)):
        tag = "prefill" if entries == 1 else "decode8"
        q = rows // entries
        cu, cb, sl = i32([q * e for e in range(entries + 1)]), i32([2048] * entries), i32(list(range(entries)))
        pos = i32([2048 + t for e in range(entries) for t in range(q)])
        re = i32([e for e in range(entries) for _ in range(q)])
        # input convolution
        u, o = rnd(rows, D), torch.empty(rows, D, dtype=torch.bfloat16, device=dev)
        st = torch.zeros(8, blk.mixer_conv.spec.taps - 1, D, device=dev)
        us = timed(lambda: ops.input_conv(u, blk.mixer_conv.weight, st, o, cu, cb, sl, entries, q))
        mem(f"{tag}_input_conv", us, 2 * rows * D * 2 + 2 * entries * st[0].numel() * 4)
        # retention
        s = ret.spec
        x = rnd(rows, ret.w_in.shape[0])
        ro = torch.empty(rows, s.n_heads * s.value_dim, dtype=torch.bfloat16, device=dev)
        state = torch.zeros(8, s.n_heads, s.key_dim, s.value_dim, device=dev)
        chunked = q >= ret.CHUNKED_MIN_ROWS
        scr = torch.empty(rows, s.n_heads * s.value_dim, device=dev) if chunked else None
        sts = torch.empty(ops.retention_chunked_scratch(rows, entries, s.n_heads, s.key_dim, s.value_dim), device=dev) if chunked else None
        us = timed(lambda: ops.retention(x, ret.position.inv_freq, s.position.rotary_dims, ret.decay, state, ro, cu, cb, sl,
                                         entries, s.n_heads, s.key_dim, s.value_dim, s.eps, scratch=scr, state_scratch=sts,
                                         max_q=q))
        nbytes = x.numel() * 2 + ro.numel() * 2 + 2 * entries * state[0].numel() * 4 + (3 * sts.numel() * 4 + 2 * scr.numel() * 4 if chunked else 0)
        mem(f"{tag}_retention", us, nbytes)
        if chunked:
            C = 32
            flops = 2 * rows * s.n_heads * (s.key_dim * (C + 1) / 2 + s.value_dim * (C + 1) / 2 + 2 * s.key_dim * s.value_dim)
            out[f"{tag}_retention"]["fp32_flops"] = int(flops)
            out[f"{tag}_retention"]["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)
        # token input
        h = torch.randn(rows, D, generator=g, device=dev)
        tok = torch.randint(0, model.spec.vocab_size, (rows,), generator=g, device=dev).to(torch.int32)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        sd = blk.side
        ssc = torch.empty(max(1, ops.token_side_scratch(rows, D, sd.spec.dim)), device=dev) if rows < 128 else None
        us = timed(lambda: ops.token_side(h, tok, sd.table, sd.w_gate, sd.w_proj, sd.w_norm, re, sd.spec.eps, status, ssc))
        mem(f"{tag}_token_side", us, 2 * rows * D * 4 + (sd.w_gate.numel() + sd.w_proj.numel()) * 4)
        # router and weighting of the experts' activations
        f = blk.ffn
        xs, wts = rnd(rows, D), torch.empty(rows, f.spec.n_experts, device=dev)
        us = timed(lambda: ops.moe_router(xs, f.w_router, f.b_router, wts, f.spec.top_k))
        mem(f"{tag}_moe_router", us, rows * D * 2 + f.w_router.numel() * 4 + wts.numel() * 4)
        act = rnd(rows, f.width)
        us = timed(lambda: ops.moe_scale(act, wts, f.spec.expert_ff))
        mem(f"{tag}_moe_scale", us, 2 * rows * f.spec.n_experts * f.spec.expert_ff * 2)
        # latent attention: norms + cache write + gate, then the attention core over the latent pages
        ls = lat.spec
        ps, n_pages = 16, 8 * 4096 // 16
        pages = rnd(n_pages, 1, ps, lat.rank_p)
        table = torch.arange(entries * 256, dtype=torch.int32, device=dev).view(entries, 256)
        down = rnd(rows, lat.w_down.shape[0])
        cq = torch.empty(rows, ls.q_rank, dtype=torch.bfloat16, device=dev)
        gate = torch.empty(rows, ls.n_heads, device=dev)
        us = timed(lambda: ops.latent_prep(down, lat.dq_norm, lat.dkv_norm, cq, pages, gate, table, pos, re, ls.n_heads,
                                           ls.eps, status))
        mem(f"{tag}_latent_prep", us, down.numel() * 2 + cq.numel() * 2 + rows * lat.rank_p * 2 + gate.numel() * 4)
        qa = rnd(rows, ls.n_heads * lat.rank_p)
        ao = torch.empty_like(qa)
        nsp = max(1, min(lat.MAX_SPLITS, 128 // rows, ls.window // 64)) if rows <= lat.SPLIT_MAX_ROWS else 1
        part = torch.empty(max(1, ops.latent_core_partial_floats(rows, ls.n_heads, lat.rank_p, nsp)), device=dev)
        if rows > lat.SPLIT_MAX_ROWS and ops.latent_core_mma_takes(ls.n_heads, lat.rank_p, torch.bfloat16):
            us = timed(lambda: ops.latent_core_mma(qa, pages, table, pos, re, gate, ao, ls.n_heads, ls.window, ls.softmax_scale))
        else:
            us = timed(lambda: ops.latent_core(qa, pages, table, pos, re, gate, ao, ls.n_heads, ls.window, ls.softmax_scale, nsp, part))
        keys = min(ls.window, 2048 + q)
        flops = 4 * rows * ls.n_heads * keys * lat.rank_p
        out[f"{tag}_latent_attention_core"] = {"us": round(us, 2), "fp32_flops": int(flops),
                                               "tflops": round(flops / (us * 1e-6) / 1e12, 2),
                                               "bytes": int(2 * qa.numel() * 2 + entries * keys * lat.rank_p * 2)}
    return out



# ---------------------------------------------------------------------------------------------- --workload rofulorn
def rofulorn_config(width, layers, ff):
    """A Rofulorn configuration with layers of a real model's sizes: plain windowed attention layers (heads of 64,
    four query heads to a key/value head) alternate with two-map attention layers (half as many heads, values of
    128), every fourth layer reading the keys and values of the two-map layer two before it; windows of 1,024
    tokens, four kept first tokens; a gated feed-forward as wide as LFM2's at the same width."""
    heads = width // 64
    a2 = {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 64, "vdim": 64, "scale": 0.125,
                                           "mask": {"size": 1024}, "rot": {"dims": 32, "base": 1000000.0}}}
    diff = {"heads": heads // 2, "kv_heads": max(1, heads // 8), "dim": 64, "vdim": 128, "scale": 0.125, "softcap": 30.0,
            "diff": 0.5, "mask": {"size": 1024, "keep_first": 4},
            "rot": {"dims": 32, "base": 20000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 2048}}}
    out = []
    for i in range(layers):
        if i % 2 == 0:
            layer = dict(a2)
        else:
            layer = {"type": "attention", "mixer": dict(diff, **({"kv_from": i - 2} if i % 4 == 3 else {}))}
        out.append(dict(layer, mlp={"kind": "dense", "ff": ff}))
    return {"architecture": "Rofulorn", "vocab": 65536, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
            "layers": out}


def run_rofulorn(args):
    """Prefill and decode throughput of the Rofulorn design at layer sizes of a real model, beside LFM2 (the closest
    existing model: grouped-query attention layers with a gated feed-forward) at equal width, depth and feed-forward
    width, and the design's attention kernels alone beside LFM2's.  One JSON line.  Random weights, synthetic token
    ids; CUDA events; the L2 is flushed between timed steps."""
    import torch
    pk = peaks()
    l2 = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda:0")
    clocks = ClockSampler(0)
    clocks.start()
    results = []
    for width, layers in ((1024, 16), (2048, 16)):
        lfm2 = dict(LFM2_1_2B)
        lfm2.update(SHAPES["350m" if width == 1024 else "1.2b"])
        row = {"width": width, "layers": layers}
        for arm, cfg in {"rofulorn": rofulorn_config(width, layers, ffn_width(lfm2)), "lfm2": lfm2}.items():
            eng = design_arm(arm, cfg, row, args, l2)
            if not args.no_kernels:
                row[arm + "_kernels"] = attention_kernel_times(eng, l2, pk)
            del eng
            torch.cuda.empty_cache()
        results.append(row)
    time.sleep(0.06)
    clocks.stop()
    print(json.dumps({"workload": "rofulorn", "what": "Rofulorn beside LFM2 at equal width, depth and feed-forward width: "
                      "prefill of 2,048 tokens, decode at batch 8 and 1 after 2,048 tokens; attention kernels alone",
                      "results": results, "dtype": "bf16", "data": "synthetic token ids, random-init weights", "peaks": pk,
                      "clocks": clocks.summary(), "impl": "ours"}))


def attention_kernel_times(eng, l2, pk):
    """Every attention layer kind of the model alone, through the mixer's own launch plan: the q/k preparation with
    the page write, and the attention core, for a 2,048-token portion and for 8 single tokens after 2,048 (CUDA
    events around the launches, L2 flushed before, median of 7): microseconds, the multiply-adds of the two products
    as TFLOP/s with the fraction of the measured tensor peak, and the bytes a decode step must read with the fraction
    of the measured copy bandwidth."""
    import torch
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts import PagedView, StepContext
    from neurogrid_b200.parts.base import Workspace
    model, dev = eng.model, eng.device
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(torch.bfloat16)

    def timed(fn):
        ts = []
        for _ in range(9):
            flush_l2(l2)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return median(ts[2:])

    out = {"unit": "us"}
    seen = set()
    for blk in model.blocks:
        mixer = blk.mixer
        kind = type(mixer).__name__
        s = mixer.spec
        if kind not in ("MappedAttention", "Attention") or not mixer.owns_cache:
            continue
        maps = getattr(s, "n_maps", 1)
        d = getattr(s, "key_dim", None) or s.head_dim
        dv = getattr(s, "value_dim", None) or s.head_dim
        tag = f"{kind}_{maps}map_{s.n_heads}x{d}"
        if tag in seen:
            continue
        seen.add(tag)
        need = mixer.cache_need()
        ps, n_pages = 16, 8 * 4096 // 16
        vh, vd = need.value_shape()
        kp, vp = rnd(n_pages, need.n_kv_heads, ps, need.head_dim), rnd(n_pages, vh, ps, vd)
        for rows, entries in ((PREFILL_TOKENS, 1), (8, 8)):
            q_len = rows // entries
            before = 0 if entries == 1 else 2048
            table = torch.arange(entries * 256, dtype=torch.int32, device=dev).view(entries, 256)
            ctx = StepContext(n_rows=rows, n_entries=entries, max_q=q_len, tokens=i32([0] * rows),
                              positions=i32([before + t for e in range(entries) for t in range(q_len)]),
                              row_entry=i32([e for e in range(entries) for _ in range(q_len)]),
                              cu_q=i32([q_len * e for e in range(entries + 1)]), ctx_before=i32([before] * entries),
                              slots=i32(list(range(entries))), status=torch.zeros(1, dtype=torch.int32, device=dev),
                              ws=Workspace(4096, dev), dtype=torch.bfloat16, q_lens=[q_len] * entries,
                              ctx_lens=[before] * entries, slot_ids=list(range(entries)))
            view = PagedView(kp, vp, table)
            o = torch.empty(rows, s.n_heads * dv, dtype=torch.bfloat16, device=dev)
            if kind == "MappedAttention":
                qkv = rnd(rows, mixer.w_qkv.shape[0])
                qb = torch.empty(rows, s.n_heads * maps * d, dtype=torch.bfloat16, device=dev)
                pa = mixer.position.kernel_args()
                prep = lambda: ops.qkv_prep(qkv, qb, mixer.q_norm, mixer.k_norm, pa.inv_freq, kp, vp, table, ctx.positions,
                                            ctx.row_entry, s.n_heads * maps, need.n_kv_heads, vh, d, dv, s.eps, ctx.status)
                core = lambda: mixer.attend(qb, view, ctx, o)
            else:
                qkv = rnd(rows, mixer.w_qkv.shape[0])
                qb = torch.empty(rows, s.n_heads * d, dtype=torch.bfloat16, device=dev)
                pa = mixer.position.kernel_args()
                prep = lambda: ops.rope_cache(qkv, qb, mixer.q_norm, mixer.k_norm, pa.inv_freq, pa.half_pairing, pa.pos_scale, kp,
                                              vp, table, ctx.positions, ctx.row_entry, s.n_heads, s.n_kv_heads, d, s.qk_norm_eps,
                                              ctx.status)
                core = lambda: mixer.attend(qb, view, ctx, o)
            prep()
            core()
            torch.cuda.synchronize()
            name = ("prefill2048_" if entries == 1 else "decode8_") + tag
            window = getattr(s, "window", None)
            if entries == 1:
                pairs = sum(min(t + 1, window) if window else t + 1 for t in range(rows))
            else:
                pairs = rows * (min(before + 1, window) if window else before + 1)
            flops = 2 * pairs * s.n_heads * (maps * d + maps * dv)
            keys = min(before + q_len, window) if window else before + q_len
            kv_bytes = entries * keys * need.elements_per_token() * 2
            us_p, us_c = timed(prep), timed(core)
            out[name] = {"prep_us": round(us_p, 2), "core_us": round(us_c, 2), "core_flops": int(flops),
                         "core_tflops": round(flops / (us_c * 1e-6) / 1e12, 2),
                         "core_of_tensor_peak": round(flops / (us_c * 1e-6) / 1e12 / pk["bf16_tflops"], 4),
                         "kv_bytes": int(kv_bytes),
                         "core_of_copy_bandwidth": round(kv_bytes / (us_c * 1e-6) / (pk["hbm_gbs"] * 1e9), 4)}
    return out


# ---------------------------------------------------------------------------------------------- --workload fuzelorn
def fuzelorn_config(width, layers):
    """A Fuzelorn configuration with layers of a real model's sizes: in every layer a windowed attention (heads of 128,
    four query heads to a key/value head, a window of 1,024) beside a gated delta rule (as many value heads of
    128 x 128, half as many query/key heads, four taps); the first layer's feed-forward dense, the others' routed
    (16 experts of width/4 in four groups of which two are kept, top 4, a gated shared expert of width/2)."""
    heads = width // 128
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "mask": {"size": 1024}, "q_temp": {"coef": 0.1, "every": 1024}}
    right = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": width // 4, "limit": 7.0}, "shared": {"ff": width // 2, "limit": 7.0}}
    dense = {"kind": "dense", "ff": 4 * width}
    return {"architecture": "Fuzelorn", "vocab": 65536, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "embedding": {"scale": 2.0, "bigram": {"buckets": 100003, "mul_prev": 36313, "mul_cur": 27191}},
            "layers": [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": dense if i == 0 else moe}
                       for i in range(layers)]}


def run_fuzelorn(args):
    """Prefill and decode throughput of the Fuzelorn design at layer sizes of a real model, beside Metanex (the closest
    existing model: layers with a float32 recurrent state, windowed attention with float32 weights, routed experts
    with a shared one) at equal width and depth, and the design's own kernels one by one beside Metanex's like
    kernels.  One JSON line.  Random weights, synthetic token ids; CUDA events; the L2 is flushed between timed steps."""
    import torch
    pk = peaks()
    l2 = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda:0")
    clocks = ClockSampler(0)
    clocks.start()
    results = []
    for width, layers in ((1024, 16), (2048, 16)):
        row = {"width": width, "layers": layers}
        for arm, cfg in {"fuzelorn": fuzelorn_config(width, layers), "metanex": metanex_config(width, layers)}.items():
            eng = design_arm(arm, cfg, row, args, l2)
            if not args.no_kernels:
                row[arm + "_kernels"] = (fuzelorn_kernel_times if arm == "fuzelorn" else metanex_kernel_times)(eng, l2, pk)
            del eng
            torch.cuda.empty_cache()
        results.append(row)
    time.sleep(0.06)
    clocks.stop()
    print(json.dumps({"workload": "fuzelorn", "what": "Fuzelorn beside Metanex at equal width and depth: prefill of 2,048 "
                      "tokens, decode at batch 8 and 1 after 2,048 tokens; each design's own kernels alone",
                      "results": results, "dtype": "bf16", "data": "synthetic token ids, random-init weights", "peaks": pk,
                      "clocks": clocks.summary(), "impl": "ours"}))


def fuzelorn_kernel_times(eng, l2, pk):
    """The design's own kernels alone, through the parts' own launch plans (CUDA events around the launches, L2 flushed
    before, median of 7), for a 2,048-token portion and for 8 single tokens after 2,048: microseconds, the bytes each
    must move with the fraction of the measured copy bandwidth, and for the recurrence and the attention core the
    multiply-adds they must do as TFLOP/s."""
    import torch
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts import PagedView, StepContext
    from neurogrid_b200.parts.base import Workspace
    model, dev = eng.model, eng.device
    D = model.spec.hidden
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(torch.bfloat16)

    def timed(fn):
        ts = []
        for _ in range(9):
            flush_l2(l2)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return median(ts[2:])

    out = {"unit": "us"}
    bw = pk["hbm_gbs"] * 1e9

    def mem(name, us, nbytes, flops=0):
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "of_copy_bandwidth": round(nbytes / (us * 1e-6) / bw, 3)}
        if flops:
            out[name]["flops"] = int(flops)
            out[name]["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)

    blk = next(b for b in model.blocks if type(b.ffn).__name__ == "MoE")
    side, f = blk.mixer, blk.ffn
    left, right = side.left, side.right
    ls, rs = left.spec, right.spec
    need = left.cache_need()
    ps, n_pages = 16, 8 * 4096 // 16
    kp, vp = rnd(n_pages, need.n_kv_heads, ps, need.head_dim), rnd(n_pages, *need.value_shape()[:1], ps, need.value_shape()[1])
    for rows, entries in ((PREFILL_TOKENS, 1), (8, 8)):
        tag = "prefill2048" if entries == 1 else "decode8"
        q_len = rows // entries
        before = 0 if entries == 1 else 2048
        table = torch.arange(entries * 256, dtype=torch.int32, device=dev).view(entries, 256)
        ctx = StepContext(n_rows=rows, n_entries=entries, max_q=q_len, tokens=i32([0] * rows),
                          positions=i32([before + t for e in range(entries) for t in range(q_len)]),
                          row_entry=i32([e for e in range(entries) for _ in range(q_len)]),
                          cu_q=i32([q_len * e for e in range(entries + 1)]), ctx_before=i32([before] * entries),
                          slots=i32(list(range(entries))), status=torch.zeros(1, dtype=torch.int32, device=dev),
                          ws=Workspace(4096, dev), dtype=torch.bfloat16, q_lens=[q_len] * entries,
                          ctx_lens=[before] * entries, slot_ids=list(range(entries)))
        # the pair embedding
        tp = model.spec.token_pair
        h = torch.randn(rows, D, generator=g, device=dev)
        tok = torch.randint(0, model.spec.vocab_size, (rows,), generator=g, device=dev).to(torch.int32)
        prev = torch.zeros(8, dtype=torch.int32, device=dev)
        us = timed(lambda: ops.pair_embed(model.pair_table, tok, prev, ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.row_entry, h,
                                          entries, model.spec.vocab_size, tp.buckets, tp.mul_prev, tp.mul_cur, ctx.status))
        mem(f"{tag}_pair_embed", us, rows * D * (2 + 4 + 4))
        # left: norms over the projections, temperature, page write; then the attention core
        d, dv, H = ls.key_dim, ls.value_dim, ls.n_heads
        vh = need.value_shape()[0]
        qkv = rnd(rows, left.w_qkv.shape[0])
        qb = torch.empty(rows, H * d, dtype=torch.bfloat16, device=dev)
        pa = left.position.kernel_args()
        view = PagedView(kp, vp, table)
        o = torch.empty(rows, H * dv, dtype=torch.bfloat16, device=dev)
        prep = lambda: ops.qkv_prep(qkv, qb, left.q_norm, left.k_norm, None, kp, vp, table, ctx.positions, ctx.row_entry, H,
                                    need.n_kv_heads, vh, d, dv, ls.eps, ctx.status, whole=True, q_temp_coef=ls.q_temp_coef,
                                    q_temp_every=ls.q_temp_every)
        core = lambda: left.attend(qb, view, ctx, o, pa.score_slopes)
        prep()
        core()
        torch.cuda.synchronize()
        mem(f"{tag}_attention_prep", timed(prep), 2 * qkv.numel() * 2)
        window = ls.window
        pairs = sum(min(t + 1, window) for t in range(rows)) if entries == 1 else rows * min(before + 1, window)
        keys = min(before + q_len, window)
        kv_bytes = entries * keys * need.elements_per_token() * 2
        us = timed(core)
        mem(f"{tag}_attention_core", us, kv_bytes + 2 * rows * H * d * 2, 2 * pairs * H * (d + dv))
        out[f"{tag}_attention_core"]["of_tensor_peak"] = round(2 * pairs * H * (d + dv) / (us * 1e-6) / 1e12 / pk["bf16_tflops"], 4)
        # right: convolution + silu, the recurrence, head norm and gate (one call of the part's launcher)
        nH, nG, dk, dvr = rs.n_heads, rs.n_qk_heads, rs.key_dim, rs.value_dim
        C = right.channels
        p = rnd(rows, right.w_in.shape[0])
        state = torch.zeros(8, nH, dk, dvr, device=dev)
        cst = torch.zeros(8, right.taps - 1, C, device=dev)
        conv = torch.empty(rows, C, device=dev)
        oraw = torch.empty(rows, nH * dvr, device=dev)
        og = torch.empty(rows, nH * dvr, dtype=torch.bfloat16, device=dev)
        chunks = None           # as the part chooses: long portions chunk by chunk, single tokens one by one
        if q_len >= right.CHUNKED_MIN_ROWS and right._chunked():
            chunks = torch.empty(ops.gated_delta_chunked_scratch(rows, entries, nH, dk, dvr), device=dev)
        run = lambda: ops.gated_delta(p, right.w_conv, right.a_log, right.dt_bias, right.norm, cst, state, conv, oraw, og,
                                      ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.row_entry, entries, q_len, nH, nG, dk, dvr, rs.eps,
                                      chunk_scratch=chunks)
        run()
        torch.cuda.synchronize()
        nbytes = p.numel() * 2 + 2 * conv.numel() * 4 + 2 * oraw.numel() * 4 + og.numel() * 2 + 2 * entries * state[0].numel() * 4
        mem(f"{tag}_gated_delta", timed(run), nbytes, 6 * rows * nH * dk * dvr)
        # the two mixers' outputs: norms over the width and the mean
        a, b = rnd(rows, D), rnd(rows, D)
        y = torch.empty(rows, D, device=dev)
        us = timed(lambda: ops.pair_norm_mean(a, b, side.w_left, side.w_right, y, side.spec.eps, torch.bfloat16))
        mem(f"{tag}_pair_norm_mean", us, 2 * rows * D * 2 + rows * D * 4)
        # router and the clamped activation with the routing weights
        fs = f.spec
        xs, wts = rnd(rows, D), torch.empty(rows, fs.n_experts + 1, device=dev)
        us = timed(lambda: ops.moe_router_sigmoid(xs, f.w_router, f.correction, f.w_shared_gate, wts, fs.top_k, fs.n_groups,
                                                  fs.keep_groups))
        mem(f"{tag}_moe_router", us, rows * D * 2 + f.w_router.numel() * 4 + wts.numel() * 4)
        gu, act = rnd(rows, 2 * f.width), torch.empty(rows, f.width, dtype=torch.bfloat16, device=dev)
        us = timed(lambda: ops.moe_clamped_glu_scaled(gu, wts, act, fs.n_experts, fs.expert_ff, fs.limit, fs.shared_limit,
                                                      fs.glu_alpha, True))
        mem(f"{tag}_moe_clamped_glu", us, 3 * rows * f.width * 2)
    return out


# ---------------------------------------------------------------------------------------------- --workload dodilix
def dodilix_config(width, layers):
    """A Dodilix configuration with layers of a real model's sizes: four copies of the stream; layers alternate between
    a parallel mixer (chunked attention, heads of 128 with half of each head rotated, four query heads to a key/value
    head, chunks of 1,024, beside a gated linear attention with as many heads of 128 x 128) and a latent attention
    (heads of 128 + 64 rotated coordinates, a latent of 192 beside the 64 shared rotated ones, queries through a latent
    of width/2), every fourth layer reading the latents of the latent layer before it; the first layer's feed-forward
    dense, the others' routed (16 experts of width/4 in four groups of which two are kept, top 4, a gated shared
    expert of width/2)."""
    heads = width // 128
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "mask": {"size": 1024}, "rot": {"base": 10000.0, "dims": 64}}
    right = {"heads": heads, "dim": 128, "vdim": 128, "tau": 8.0, "decay_rank": 64}
    parallel = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.9, "right_scale": 1.2}}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": width // 2, "kv_rank": 192,
              "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 4, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": width // 4}, "shared": {"ff": width // 2}}
    dense = {"kind": "dense", "ff": 4 * width}
    out = []
    for i in range(layers):
        if i % 2 == 0:
            layer = dict(parallel)
        else:
            layer = {"type": "latent_attention", "mixer": dict(latent, **({"kv_from": i - 2} if i % 4 == 3 else {}))}
        layer["mlp"] = dense if i == 0 else moe
        out.append(layer)
    return {"architecture": "Dodilix", "vocab": 65536, "width": width, "streams": 4, "norm": {"eps": 1e-5},
            "logit_scale": 0.5, "embedding": {"scale": 2.0}, "layers": out}


def run_dodilix(args):
    """Prefill and decode throughput of the Dodilix design at layer sizes of a real model, beside Fuzelorn (the closest
    existing model: a windowed attention with float32 weights beside a recurrence with a float32 state in every layer,
    routed experts in groups with a gated shared one) at equal width and depth, and the design's own kernels one by
    one.  One JSON line.  Random weights, synthetic token ids; CUDA events; the L2 is flushed between timed steps."""
    import torch
    pk = peaks()
    l2 = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda:0")
    clocks = ClockSampler(0)
    clocks.start()
    results = []
    for width, layers in ((1024, 16), (2048, 16)):
        row = {"width": width, "layers": layers}
        for arm, cfg in {"dodilix": dodilix_config(width, layers), "fuzelorn": fuzelorn_config(width, layers)}.items():
            eng = design_arm(arm, cfg, row, args, l2)
            if not args.no_kernels:
                row[arm + "_kernels"] = (dodilix_kernel_times if arm == "dodilix" else fuzelorn_kernel_times)(eng, l2, pk)
            del eng
            torch.cuda.empty_cache()
        results.append(row)
    time.sleep(0.06)
    clocks.stop()
    print(json.dumps({"workload": "dodilix", "what": "Dodilix beside Fuzelorn at equal width and depth: prefill of 2,048 "
                      "tokens, decode at batch 8 and 1 after 2,048 tokens; each design's own kernels alone",
                      "results": results, "dtype": "bf16", "data": "synthetic token ids, random-init weights", "peaks": pk,
                      "clocks": clocks.summary(), "impl": "ours"}))


def dodilix_kernel_times(eng, l2, pk):
    """The design's own kernels alone, through the parts' own launch plans (CUDA events around the launches, L2 flushed
    before, median of 7), for a 2,048-token portion and for 8 single tokens after 2,048: microseconds, the bytes each
    must move with the fraction of the measured copy bandwidth, and for the recurrence and the attention cores the
    multiply-adds they must do as TFLOP/s."""
    import torch
    from neurogrid_b200.csrc import ops
    from neurogrid_b200.parts import PagedView, StepContext
    from neurogrid_b200.parts.base import Workspace
    model, dev = eng.model, eng.device
    D, S = model.spec.hidden, model.spec.streams
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev).to(torch.bfloat16)

    def timed(fn):
        ts = []
        for _ in range(9):
            flush_l2(l2)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return median(ts[2:])

    out = {"unit": "us"}
    bw = pk["hbm_gbs"] * 1e9

    def mem(name, us, nbytes, flops=0):
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "of_copy_bandwidth": round(nbytes / (us * 1e-6) / bw, 3)}
        if flops:
            out[name]["flops"] = int(flops)
            out[name]["tflops"] = round(flops / (us * 1e-6) / 1e12, 2)

    par = next(b for b in model.blocks if type(b.mixer).__name__ == "SideBySide" and type(b.ffn).__name__ == "MoE")
    lat = next(b.mixer for b in model.blocks if type(b.mixer).__name__ == "LatentAttention" and b.mixer.owns_cache)
    side, f = par.mixer, par.ffn
    left, right = side.left, side.right
    ls, rs, ts_ = left.spec, right.spec, lat.spec
    need = left.cache_need()
    ps, n_pages = 16, 8 * 4096 // 16
    kp, vp = rnd(n_pages, need.n_kv_heads, ps, need.head_dim), rnd(n_pages, need.value_shape()[0], ps, need.value_shape()[1])
    lp = rnd(n_pages, 1, ps, lat.rank_p)
    for rows, entries in ((PREFILL_TOKENS, 1), (8, 8)):
        tag = "prefill2048" if entries == 1 else "decode8"
        q_len = rows // entries
        before = 0 if entries == 1 else 2048
        table = torch.arange(entries * 256, dtype=torch.int32, device=dev).view(entries, 256)
        ctx = StepContext(n_rows=rows, n_entries=entries, max_q=q_len, tokens=i32([0] * rows),
                          positions=i32([before + t for e in range(entries) for t in range(q_len)]),
                          row_entry=i32([e for e in range(entries) for _ in range(q_len)]),
                          cu_q=i32([q_len * e for e in range(entries + 1)]), ctx_before=i32([before] * entries),
                          slots=i32(list(range(entries))), status=torch.zeros(1, dtype=torch.int32, device=dev),
                          ws=Workspace(4096, dev), dtype=torch.bfloat16, q_lens=[q_len] * entries,
                          ctx_lens=[before] * entries, slot_ids=list(range(entries)))
        # between two sublayers: the copies' update, the read-out and its norm
        X, y = torch.randn(rows, S * D, generator=g, device=dev), rnd(rows, D)
        w_in, w_out, mix = par.hc["hc1"]
        normed = torch.empty(rows, D, dtype=torch.bfloat16, device=dev)
        us = timed(lambda: ops.hc_step(X, S, delta=y, mix=mix, out_w=w_out, in_w=w_in, norm_w=par.mixer_norm.weight, out=normed,
                                       eps=1e-5))
        mem(f"{tag}_stream_copies", us, rows * D * (2 * 4 * S + 2 + 2))
        # left: rotation, norms, page write; the attention core; the output gate
        d, dv, H = ls.key_dim, ls.value_dim, ls.n_heads
        vh = need.value_shape()[0]
        qkv = rnd(rows, left.w_qkv.shape[0])
        qb = torch.empty(rows, H * d, dtype=torch.bfloat16, device=dev)
        pa = left.position.kernel_args()
        view = PagedView(kp, vp, table)
        o = torch.empty(rows, H * dv, dtype=torch.bfloat16, device=dev)
        prep = lambda: ops.qkv_prep(qkv, qb, None, None, pa.inv_freq, kp, vp, table, ctx.positions, ctx.row_entry, H,
                                    need.n_kv_heads, vh, d, dv, ls.eps, ctx.status, half_pairing=True, unit_norm=True)
        core = lambda: left.attend(qb, view, ctx, o, None)
        prep()
        core()
        torch.cuda.synchronize()
        mem(f"{tag}_attention_prep", timed(prep), 2 * (H + need.n_kv_heads) * d * rows * 2 + 2 * vh * dv * rows * 2)
        chunk = ls.chunk
        pairs = sum(t % chunk + 1 for t in range(rows)) if entries == 1 else rows * (before % chunk + 1)
        keys = min(before % chunk + q_len, chunk)
        kv_bytes = entries * keys * need.elements_per_token() * 2
        us = timed(core)
        mem(f"{tag}_attention_core", us, kv_bytes + 2 * rows * H * d * 2, 2 * pairs * H * (d + dv))
        out[f"{tag}_attention_core"]["of_tensor_peak"] = round(2 * pairs * H * (d + dv) / (us * 1e-6) / 1e12 / pk["bf16_tflops"], 4)
        gate = qkv[:, qkv.shape[1] - H * dv:]
        mem(f"{tag}_output_gate", timed(lambda: ops.gate_mul(o, gate, "sigmoid", 0.9)), 3 * rows * H * dv * 2)
        # right: the recurrence with its decay, head norm and gate (one call of the part's launcher)
        nH, dk, dvr = rs.n_heads, rs.key_dim, rs.value_dim
        p, z = rnd(rows, right.w_in.shape[0]), rnd(rows, nH * dk)
        state = torch.zeros(8, nH, dk, dvr, device=dev)
        og = torch.empty(rows, nH * dvr, dtype=torch.bfloat16, device=dev)
        scratch = states = None         # as the part chooses: long portions chunk by chunk, single tokens one by one
        if right._chunked(ctx):
            scratch = torch.empty(rows, nH * dvr, device=dev)
            states = torch.empty(ops.gated_linear_chunked_scratch(rows, entries, nH, dk, dvr), device=dev)
        run = lambda: ops.gated_linear(p, z, right.norm, state, og, ctx.cu_q, ctx.ctx_before, ctx.slots, entries, nH, dk, dvr,
                                       rs.tau, rs.eps, 1.2, scratch=scratch, state_scratch=states, max_q=q_len)
        run()
        torch.cuda.synchronize()
        nbytes = (p.numel() + z.numel() + og.numel()) * 2 + 2 * entries * state[0].numel() * 4
        mem(f"{tag}_gated_linear", timed(run), nbytes, 4 * rows * nH * dk * dvr)
        # latent attention: the row kernel, the rotation of q, the core, the heads' expansion with the gate
        Hl, rp = ts_.n_heads, lat.rank_p
        down = rnd(rows, lat.w_down.shape[0])
        cq, gl = torch.empty(rows, ts_.q_rank, dtype=torch.bfloat16, device=dev), torch.empty(rows, lat.n_gate, device=dev)
        la = lat.position.kernel_args()
        us = timed(lambda: ops.latent_prep(down, lat.dq_norm, lat.dkv_norm, cq, lp, gl, table, ctx.positions, ctx.row_entry,
                                           lat.n_gate, ts_.eps, ctx.status, rot=lat.rope, inv_freq=la.inv_freq))
        mem(f"{tag}_latent_prep", us, down.numel() * 2 + cq.numel() * 2 + rows * rp * 2 + gl.numel() * 4)
        ql, ol = rnd(rows, Hl * rp), torch.empty(rows, Hl * rp, dtype=torch.bfloat16, device=dev)
        mem(f"{tag}_latent_rope_q", timed(lambda: ops.latent_rope_q(ql, ctx.positions, ctx.row_entry, la.inv_freq, Hl, ts_.kv_rank)),
            2 * rows * Hl * lat.rope * 2)
        if entries == 1:
            corel = lambda: ops.latent_core_mma(ql, lp, table, ctx.positions, ctx.row_entry, None, ol, Hl, None, ts_.softmax_scale)
        else:
            n_splits = max(1, min(lat.MAX_SPLITS, 128 // rows, (before + 1) // 64))
            part = torch.empty(max(1, ops.latent_core_partial_floats(rows, Hl, rp, n_splits)), device=dev)
            corel = lambda: ops.latent_core(ql, lp, table, ctx.positions, ctx.row_entry, None, ol, Hl, None, ts_.softmax_scale,
                                            n_splits, part)
        corel()
        torch.cuda.synchronize()
        pairs = sum(t + 1 for t in range(rows)) if entries == 1 else rows * (before + 1)
        us = timed(corel)
        mem(f"{tag}_latent_core", us, entries * (before + q_len) * rp * 2 + 2 * rows * Hl * rp * 2, 4 * pairs * Hl * rp)
        out[f"{tag}_latent_core"]["of_tensor_peak"] = round(4 * pairs * Hl * rp / (us * 1e-6) / 1e12 / pk["bf16_tflops"], 4)
        heads_out = torch.empty(rows, Hl * ts_.value_dim, dtype=torch.bfloat16, device=dev)
        us = timed(lambda: ops.head_up_gate(ol, lat.w_uv, gl, heads_out))
        mem(f"{tag}_heads_expanded", us, ol.numel() * 2 + lat.w_uv.numel() * 2 + gl.numel() * 4 + heads_out.numel() * 2,
            2 * rows * Hl * ts_.value_dim * ts_.kv_rank)
        # router and the activation with the routing weights
        fs = f.spec
        xs, wts = rnd(rows, D), torch.empty(rows, fs.n_experts + 1, device=dev)
        us = timed(lambda: ops.moe_router_sigmoid(xs, f.w_router, None, f.w_shared_gate, wts, fs.top_k, fs.n_groups,
                                                  fs.keep_groups, softmax_scores=True, group_max=True, route_scale=fs.route_scale))
        mem(f"{tag}_moe_router", us, rows * D * 2 + f.w_router.numel() * 4 + wts.numel() * 4)
        gu, act = rnd(rows, 2 * f.width), torch.empty(rows, f.width, dtype=torch.bfloat16, device=dev)
        us = timed(lambda: ops.moe_swiglu_scaled(gu, wts, act, fs.expert_ff, shared_gated=True))
        mem(f"{tag}_moe_activation", us, 3 * rows * f.width * 2)
    return out


def run_reference(args):
    """The reference's own library through its stock entry points; same metric, same line."""
    shape_name = SHAPE_NAMES[args.shape]
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
    except Exception as e:                              # numpy missing, or the like
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm cannot start: {e!r}"}))
        return
    cfg, full_layers = shape_config(args)
    cfg["intermediate_size"] = ffn_width(cfg)
    cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    prompt_len = args.prompt_len or PROMPT
    clocks = ClockSampler(0)
    clocks.start()
    try:
        m = reference_arm.run(cfg, batch=args.batch, steps=args.steps, warmup=max(3, args.warmup), prompt_len=prompt_len)
    except reference_arm.Unavailable as e:
        clocks.stop()
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return
    time.sleep(0.06)
    clocks.stop()
    pk = peaks()
    bn_kernel = m.get("bN_kernel_ms", m["b1_kernel_ms"])
    bn_stock = m.get("bN_stock_ms", m["b1_stock_ms"])
    line = {"metric": f"decode tok/s @ batch {args.batch} ({shape_name} shape)",
            "value": round(args.batch / bn_kernel * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(bn_kernel, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(1e3 / m["b1_kernel_ms"] / PUBLISHED_BASELINE_TOK_S, 2), "dtype": "bf16",
            "data": "synthetic token ids, random-init weights N(0, 0.02)",
            "config": {"model": f"{shape_name} shape, random weights", "hidden": cfg["hidden_size"],
                       "ffn": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "heads": cfg["num_attention_heads"],
                       "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "conv_L": cfg["conv_L_cache"],
                       "layers": cfg["num_hidden_layers"], "layers_full": full_layers, "global_batch": args.batch,
                       "seq_len": CONTEXT, "prompt_len": prompt_len, "page_size": 16, "parallelism": "1 GPU",
                       "how": "libgpu_engine.so built by the reference's `make cuda-only`, driven with ctypes in the "
                              "order of pkg/inference; value = device time of its model and LM-head calls, "
                              "e2e = its scheduler's whole per-token sequence"},
            "e2e": {"value": round(args.batch / bn_stock * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(bn_stock, 4),
                    "h2d_bytes_per_step": m["h2d_bytes_per_step"], "d2h_bytes_per_step": m["d2h_bytes_per_step"]},
            "gpu_launches": 0, "launches_note": m["launch_note"],
            "prefill": {"value": round(m["prefill_tokens"] / m["prefill_ms"] * 1e3, 1), "tokens": m["prefill_tokens"],
                        "ms": round(m["prefill_ms"], 2), "first_ms": round(m["prefill_first_ms"], 2)},
            "points": {"decode_b1": round(1e3 / m["b1_kernel_ms"], 1), "decode_b1_e2e": round(1e3 / m["b1_stock_ms"], 1)},
            "peaks": {"hbm_gbs": pk["hbm_gbs"], "of": pk["source"]},
            "clocks": clocks.summary(), "impl": "reference"}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--shape", default="1.2b", choices=sorted(SHAPES), help="layer sizes: another published LFM2 shape")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="tokens each request holds before decoding (default 2,048; the context is twice this)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="", choices=["", "mixed350m", "long700m", "metanex", "rofulorn", "fuzelorn", "dodilix"],
                    help="run another workload of the benchmark set through Engine.generate instead; metanex / rofulorn: "
                         "that design beside LFM2 at equal width and depth, prefill and decode, and its kernels alone")
    ap.add_argument("--repeat", type=int, default=2, help="--workload: runs (the first also warms up and captures graphs)")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel timings")
    ap.add_argument("--profile-only", action="store_true",
                    help="a short eager run for a profiler: prefill once, then the decode steps, no CUDA graphs, no JSON")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"error": "this engine runs on one GPU; bench.py measures N=1 only", "n_gpus": args.gpus}))
        return 2
    if args.impl == "reference":
        run_reference(args)
        return 0
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "metanex":
        run_metanex(args)
        return 0
    if args.workload == "dodilix":
        run_dodilix(args)
        return 0
    if args.workload == "fuzelorn":
        run_fuzelorn(args)
        return 0
    if args.workload == "rofulorn":
        run_rofulorn(args)
        return 0
    if args.workload:
        run_workload(args)
        return 0
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
