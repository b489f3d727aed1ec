#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the LFM2-1.2B shape, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

A "step" is one decode step of the batch.  The default run has the layer sizes of the
LFM2-1.2B configuration, a batch of 8 and requests that hold 2,048-token prompts and grow
toward a context of 4,096.  One JSON line is printed:

* ``value``     decoded tokens a second, timed on the device around K steps of the step function;
* ``e2e``       the same through ``Engine.step()``: host token ids in (pinned host memory ->
                device every step) and sampled token ids back on the host every step;
* ``prefill``   one 2,048-token prompt in one step, logits of the last row;
* ``roofline``  bytes a decode step has to read (every weight once, the live requests' keys,
                values and states) / its time, against the measured copy bandwidth;
* ``points``    decode tokens a second at batch 1 and 64.

For N > 1 GPUs it prints one line that says so and exits with 2: the engine is single-GPU.
"""
from __future__ import annotations

import argparse
import json
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
# the other published LFM2 shapes (same layer pattern, 8 KV heads of 64): --shape
SHAPES = {"1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288),
          "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10240),
          "350m": dict(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656)}
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


def model_numbers(cfg_dict, n_layers_run):
    """Parameter bytes a decode step reads, flops per token, KV bytes per token, state bytes."""
    from neurogrid_b200.config import config_from_dict
    c = config_from_dict(cfg_dict)
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


def flush_l2(buf):
    buf.add_(1)                                    # a buffer larger than L2, written between timed steps


def run_ours(args):
    import torch
    from neurogrid_b200 import Engine
    from neurogrid_b200.engine import StepEntry
    from neurogrid_b200.sampling import SamplingParams

    global PROMPT, CONTEXT
    cfg = dict(LFM2_1_2B)
    cfg.update(SHAPES[args.shape])
    if args.prompt_len:
        PROMPT, CONTEXT = args.prompt_len, 2 * args.prompt_len
    full_layers = cfg["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["layer_types"] = cfg["layer_types"][: args.layers]
    pk = peaks()
    clocks = ClockSampler(0)
    clocks.start()
    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    max_batch = max(args.batch, 64 if not args.prompt_len else args.batch)     # long contexts: no batch-64 point
    eng = Engine(config=cfg, random_weights=0, dtype="bf16", gpu=0, max_seq_len=CONTEXT, page_size=args.page_size,
                 max_requests=max_batch, max_tokens_per_step=max(PREFILL_TOKENS, max_batch),
                 num_pages=max_batch * CONTEXT // args.page_size)
    runner = eng.runner
    nums = model_numbers(cfg, cfg["num_hidden_layers"])
    l2 = torch.zeros(192 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator().manual_seed(1)
    V = cfg["vocab_size"]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    if args.profile_only:
        runner.cuda_graphs = False
        ids = [f"p{i}" for i in range(args.batch)]
        for rid in ids:
            runner.step([StepEntry(rid, torch.randint(0, V, (PROMPT,), generator=g).tolist(), [])])
        for _ in range(args.warmup + args.steps):
            runner.step([StepEntry(r, [5], [0]) for r in ids])
        torch.cuda.synchronize()
        clocks.stop()
        print("profile run done")
        return

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(3 + 5):
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
    pf_ms = sorted(times)[len(times) // 2]
    T = PREFILL_TOKENS
    attn_flops = nums["n_attn"] * 4 * nums["qd"] * (T * (T + 1) // 2)
    pf_flops = T * nums["mm_flops_per_token"] + attn_flops + nums["head_flops_per_row"]
    prefill = {"value": round(T / pf_ms * 1e3, 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(pf_flops / (pf_ms * 1e-3) / 1e12, 1), "of": pk["source"]}

    # ---------------------------------------------------------------- decode, device-timed
    def decode_point(batch, steps, warmup):
        """Requests with PROMPT tokens in the cache, then `steps` timed decode steps."""
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:
            toks_p = torch.randint(0, V, (PROMPT,), generator=g).tolist()
            for at in range(0, PROMPT, PREFILL_TOKENS):              # long prompts go in portions
                runner.step([StepEntry(rid, toks_p[at:at + PREFILL_TOKENS], [])])
        toks = torch.randint(0, V, (batch,), generator=g).tolist()
        launches0 = kernel_launches(runner, batch)
        for _ in range(warmup):
            runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        mark = clocks.mark()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):                               # exactly `steps` steps in one timed region
            runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)])
        b.record()
        torch.cuda.synchronize()
        per = [a.elapsed_time(b) / steps]
        ctx_mid = PROMPT + warmup + steps // 2
        for rid in ids:
            runner.finish(rid)
        ms = sum(per) / len(per)
        return ms, ctx_mid, launches0, (mark, clocks.mark())

    t_first = clocks.mark()
    ms, ctx_mid, launches, span = decode_point(args.batch, args.steps, args.warmup)
    step_bytes = nums["weight_bytes"] + args.batch * (ctx_mid * nums["kv_bytes_per_token"] + 2 * nums["state_bytes"])
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    for b in (1, 64):
        if b > max_batch:
            continue
        if b == args.batch:
            points[f"decode_b{b}"] = round(b / ms * 1e3, 1)
            continue
        pms, _, _, _ = decode_point(b, max(8, args.steps // 2), args.warmup)
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)

    # ---------------------------------------------------------------- decode, end to end through Engine.step()
    for i in range(args.batch):
        eng.add_request(torch.randint(0, V, (PROMPT,), generator=g).tolist(),
                        SamplingParams(temperature=0.0, max_new_tokens=args.warmup + args.steps + 64 + args.batch, ignore_eos=True))
    while any(r.pending > 1 or not r.output for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()                                                    # prefill until every request decodes
    for _ in range(args.warmup):
        eng.step()
    h0, d0 = eng.h2d_bytes, eng.d2h_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e = {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": (eng.h2d_bytes - h0) // args.steps,
           "d2h_bytes_per_step": (eng.d2h_bytes - d0) // args.steps}
    time.sleep(0.06)                                   # let the last clock sample of the timed regions arrive
    clocks.stop()

    value = args.batch / ms * 1e3
    from neurogrid_b200.config import config_from_dict
    shape_name = {"1.2b": "LFM2-1.2B", "700m": "LFM2-700M", "350m": "LFM2-350M"}[args.shape]
    config = {"model": f"{shape_name} shape, random weights", "hidden": cfg["hidden_size"],
              "ffn": config_from_dict(cfg).intermediate_size,
              "vocab": V, "heads": cfg["num_attention_heads"], "kv_heads": 8, "head_dim": 64, "conv_L": 3,
              "layers": cfg["num_hidden_layers"], "layers_full": full_layers, "attn_layers": nums["n_attn"],
              "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": args.page_size,
              "parallelism": "1 GPU", "l2": f"not flushed: each step reads {nums['weight_bytes'] / 1e9:.1f} GB of weights, far more than L2",
              "weights_gb": round(nums["weight_bytes"] / 1e9, 3)}
    line = {"metric": f"decode tok/s @ batch {args.batch} ({shape_name} shape)", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(points.get("decode_b1", 0.0) / PUBLISHED_BASELINE_TOK_S, 2),
            "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02)", "config": config,
            "e2e": e2e, "gpu_launches": launches * args.steps, "prefill": prefill,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes),
                         "of": pk["source"]},
            "points": points, "clocks": clocks.summary(t_first, None), "impl": "ours"}
    print(json.dumps(line))


def kernel_launches(runner, batch):
    """Kernel launches of one decode step, all of this package at decode sizes (the products
    included), counted from the model's structure: embedding; per layer two norms, the mixer's
    kernels (short conv: product, conv, product; attention: product, rope/cache, attention,
    combine, product) and two feed-forward products (the gate rides in the first); final norm
    and the head's product."""
    spec = runner.model.spec
    n = 1 + 2
    for e in spec.schedule:
        kind = spec.layers[e.layer].mixer.kind
        n += 2 + 2 + (5 if kind == "attention" else 3)
    return n


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Go program over a CUDA library (cgo); no Go toolchain is installed and it "
                      "has no Python package to install offline"}))


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
    ap.add_argument("--profile-only", action="store_true",
                    help="a short eager run for a profiler: prefill once, then the decode steps, no CUDA graphs, no JSON")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"error": "this engine runs on one GPU; bench.py measures N=1 only", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    run_ours(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
