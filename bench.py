#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the LFM2-1.2B shape, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]
                    [--shape 1.2b|700m|350m] [--prompt-len N] [--workload mixed350m|long700m]

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
    ap.add_argument("--workload", default="", choices=["", "mixed350m", "long700m"],
                    help="run another workload of the benchmark set through Engine.generate instead")
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
    if args.workload:
        run_workload(args)
        return 0
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
