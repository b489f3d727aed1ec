"""A mixer with state of its own, a feed-forward with routing, another position encoding and a
whole toy architecture, all defined here, are registered, built, loaded and stepped without touching the
framework's files.  The toy parts are plain PyTorch on the GPU: they are test fixtures that
show the interfaces, not product kernels."""
import dataclasses
import math
from dataclasses import dataclass

import pytest
import torch

import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.cache import SlotNeed
from neurogrid_b200.config import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                                   SwiGLUSpec, register_architecture)
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.parts import register
from neurogrid_b200.weights import TensorDecl, write_random_model

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class DecaySpec:
    hidden: int
    decay: float
    kind: str = "toy_decay"


@register("mixer", "toy_decay")
class DecayMixer:
    """s[t] = decay * s[t-1] + gate * x[t];  y[t] = W s[t].  One state vector per request."""

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def tensors(self):
        return {"gate": TensorDecl((self.spec.hidden,), "norm"), "mix.weight": TensorDecl((self.spec.hidden,) * 2)}

    def bind(self, t):
        self.gate = t["gate"].to(self.device, torch.float32)
        self.w = t["mix.weight"].to(self.device, torch.float32)

    def cache_need(self):
        return SlotNeed((self.spec.hidden,))

    def forward(self, x, ctx, cache):
        out = ctx.ws.buf("mixer_out", x.shape[0], self.spec.hidden, self.dtype)
        row = 0
        for q, before, slot in zip(ctx.q_lens, ctx.ctx_lens, ctx.slot_ids):
            s = cache.state[slot] if before > 0 else torch.zeros_like(cache.state[slot])
            for t in range(q):
                s = self.spec.decay * s + self.gate * x[row + t].float()
                out[row + t] = (self.w @ s).to(self.dtype)
            cache.state[slot] = s
            row += q
        return out


@dataclass(frozen=True)
class Top1Spec:
    hidden: int
    experts: int
    kind: str = "toy_top1"


@register("ffn", "toy_top1")
class Top1Experts:
    """Router logits in float32 -> the best expert's matrix is applied to the token."""

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def tensors(self):
        s = self.spec
        return {"router.weight": TensorDecl((s.experts, s.hidden)),
                **{f"experts.{e}.weight": TensorDecl((s.hidden, s.hidden)) for e in range(s.experts)}}

    def bind(self, t):
        self.router = t["router.weight"].to(self.device, torch.float32)
        self.experts = torch.stack([t[f"experts.{e}.weight"].to(self.device, torch.float32)
                                    for e in range(self.spec.experts)])

    def forward(self, x, ctx):
        xf = x.float()
        pick = torch.argmax(xf @ self.router.T, -1)
        out = ctx.ws.buf("ffn_out", x.shape[0], self.spec.hidden, self.dtype)
        out.copy_(torch.einsum("nij,nj->ni", self.experts[pick], xf).to(self.dtype))
        return out


class ToyConfig:
    """Layers: decay mixer + routed ffn, attention + SwiGLU, decay mixer + SwiGLU, an attention
    layer without k/v weights.  The schedule runs the first attention layer twice (each run
    with a cache of its own) and lets the last layer read the cache the first run wrote."""
    architecture = "ToyForCausalLM"

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def model_spec(self):
        H, V = self.d["width"], self.d["vocab_size"]
        norm = RMSNormSpec(H, 1e-5)
        names = dict(mixer="mixer", ffn="ffn", mixer_norm="norm1", ffn_norm="norm2")
        decay = DecaySpec(H, self.d["decay"])
        attn = AttentionSpec(H, 4, 2, 16, RopeSpec(16, 1e4, "half"))
        layers = (LayerSpec(decay, Top1Spec(H, 3), norm, norm, "toy.0.", names),
                  LayerSpec(attn, SwiGLUSpec(H, 96), norm, norm, "toy.1.", names),
                  LayerSpec(decay, SwiGLUSpec(H, 96), norm, norm, "toy.2.", names),
                  LayerSpec(attn, SwiGLUSpec(H, 96), norm, norm, "toy.3.", names))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2), ScheduleEntry(1, 7),
                    ScheduleEntry(3, 1, writes=False))
        return ModelSpec("ToyForCausalLM", V, H, layers, schedule, norm, True, 256,
                         embed_name="toy.embed.weight", final_norm_name="toy.norm.weight")


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    register_architecture("ToyForCausalLM", ToyConfig)
    folder = write_random_model({"architectures": ["ToyForCausalLM"], "width": 48, "vocab_size": 120, "decay": 0.8},
                                5, str(tmp_path / "toy"))
    runner = make_runner(folder, dtype=torch.float32, device="cuda", num_pages=16, page_size=16, max_seq_len=256)
    st = runner.storage
    assert len(st.slot_needs) == 1 and st.state[0].shape == (2, 4, 48)        # two decay layers share a group
    assert len(st.paged_needs) == 1 and st.k[0].shape[0] == 2                 # caches 1 and 7
    assert "toy.3.mixer.k_proj.weight" not in runner.model.tensors()          # the reader has no k/v weights
    assert "toy.1.mixer.k_proj.weight" in runner.model.tensors()
    reqs = scenarios.make_requests([40, 9, 70], 120, seed=1)

    def replay(steps):
        got = []
        for s in steps:
            got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
            for r in s["end"]:
                runner.finish(r)
        runner.cache.check()
        return scenarios.collect(steps, lambda i: got[i])

    whole = replay(scenarios.whole(reqs))
    cut = replay(scenarios.portions(reqs))
    mixed = replay(scenarios.mixed(reqs, 256, round_to=16))
    for r in reqs:
        assert torch.isfinite(whole[r]).all() and float(whole[r].abs().max()) > 0
        assert rel_err(cut[r], whole[r]) < 1e-4 and rel_err(mixed[r], whole[r]) < 1e-4
    # the state matters: the same token at the same place after another prefix gives other logits
    a = runner.step([StepEntry("p", [3, 4, 5, 6], [3])]).clone()
    runner.finish("p")
    b = runner.step([StepEntry("p", [9, 4, 5, 6], [3])]).clone()
    runner.finish("p")
    assert rel_err(a, b) > 1e-3
    assert runner.cache.pages_free() == [16] and runner.cache.slots_free() == 4


# ---------------------------------------------------------------------------------------------
# another position encoding, defined here: only the first `rotary_dims` of a head are rotated
# (the other pairs keep angle 0), with a frequency base of its own.  Nothing of the framework
# changes: the part hands the q/k kernel its table of frequencies.
@dataclasses.dataclass(frozen=True)
class PartialRopeSpec:
    head_dim: int
    rotary_dims: int
    theta: float
    kind: str = "toy_partial_rope"


@register("position", "toy_partial_rope")
class PartialRope:
    def __init__(self, spec, *, device):
        self.spec = spec
        i = torch.arange(spec.head_dim // 2, dtype=torch.float64)
        inv = float(spec.theta) ** (-2.0 * i / spec.rotary_dims)
        inv[spec.rotary_dims // 2:] = 0.0                          # angle 0: these pairs pass unchanged
        self.inv_freq = inv.to(torch.float32).to(device)

    def kernel_args(self):
        return self.inv_freq, False, 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_position_encoding_in_the_attention_part(dtype):
    from neurogrid_b200.config import AttentionSpec
    from neurogrid_b200.parts import PagedView, build
    from neurogrid_b200.weights import draw
    from helpers import make_ctx, rel_err
    H, nH, nKV, hd, rot, T, ps = 64, 4, 2, 32, 16, 37, 8
    spec = AttentionSpec(H, nH, nKV, hd, PartialRopeSpec(hd, rot, 777.0), qk_norm=False)
    part = build("mixer", spec, dtype=dtype, device="cuda")
    w = draw(part.tensors(), 3)
    part.bind(w)
    w = {k: v.double() for k, v in w.items()}
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dtype).to("cuda")
    # plain statement: rotate the first `rot` dims of every head in adjacent pairs, then causal attention
    xs = x.double().cpu()
    rb = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t)
    q = rb(xs @ w["q_proj.weight"].T).reshape(T, nH, hd)
    k = rb(xs @ w["k_proj.weight"].T).reshape(T, nKV, hd)
    v = rb(xs @ w["v_proj.weight"].T).reshape(T, nKV, hd)
    pos = torch.arange(T, dtype=torch.float64)
    inv = 777.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
    ang = (pos[:, None].float() * inv[None, :].float()).double()   # the kernel forms the angle in float32
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot_first(t):
        a, b = t[..., 0:rot:2], t[..., 1:rot:2]
        o = t.clone()
        o[..., 0:rot:2], o[..., 1:rot:2] = a * c - b * s, a * s + b * c
        return rb(o)

    q, k = rot_first(q), rot_first(k)
    mask = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    heads = []
    for h in range(nH):
        sc = (q[:, h] @ k[:, h // (nH // nKV)].T) / math.sqrt(hd)
        p = torch.softmax(sc.masked_fill(mask, -1e300), -1)
        heads.append((rb(p) if dtype == torch.bfloat16 else p) @ v[:, h // (nH // nKV)])
    want = rb(torch.stack(heads, 1).reshape(T, -1)) @ w["o_proj.weight"].T

    pages = 16
    kp = torch.randn(pages, nKV, ps, hd, device="cuda").to(dtype)
    vp = torch.randn(pages, nKV, ps, hd, device="cuda").to(dtype)
    table = torch.full((1, pages), -1, dtype=torch.int32)
    table[0, : -(-T // ps)] = torch.randperm(pages)[: -(-T // ps)].to(torch.int32)
    view = PagedView(kp, vp, table.to("cuda"))
    got, at = [], 0
    for n in (20, 1, 1, 15):
        got.append(part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [0], dtype=dtype), view).clone())
        at += n
    assert rel_err(torch.cat(got), want) < (1e-4 if dtype == torch.float32 else 2e-2)


# ---------------------------------------------------------------------------------------------
# a windowed model, defined here: the LFM2 layers with every attention layer limited to the last
# `sliding_window` keys.  Its pages are given back as the window passes them, inside the step
# function, the portion graphs and the decode graphs.
class WindowedConfig:
    architecture = "ToyWindowedForCausalLM"

    def __init__(self, d):
        from neurogrid_b200.config import Lfm2Config
        self.inner = Lfm2Config.from_dict(d)
        self.window = int(d["sliding_window"])

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def model_spec(self):
        spec = self.inner.model_spec()
        layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, window=self.window))
                       if isinstance(l.mixer, AttentionSpec) else l for l in spec.layers)
        return dataclasses.replace(spec, layers=layers, architecture=self.architecture)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_windowed_model_gives_pages_back_and_keeps_the_logits(tmp_path, dtype):
    import plain_lfm2
    from tiny_configs import TINY_B
    register_architecture("ToyWindowedForCausalLM", WindowedConfig)
    ps, window = 8, 21                                          # the window is no multiple of the page size
    cfg = dict(TINY_B, architectures=["ToyWindowedForCausalLM"], sliding_window=window)
    folder = write_random_model(cfg, 9, str(tmp_path / "windowed"))
    pcfg, w = plain_lfm2.load_plain(folder)
    toks = scenarios.make_requests([150], pcfg["vocab_size"], seed=4)["r0"]
    want = plain_lfm2.forward(pcfg, w, toks, round_bf16=(dtype == torch.bfloat16))
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    # far fewer pages than the request's 150 tokens would need without a window
    runner = make_runner(folder, dtype=dtype, device="cuda", num_pages=10, page_size=ps, max_requests=2, max_seq_len=256)
    assert runner.cache.windowed
    # portions that straddle the window's edge and page edges: two tokens, one page and a token, ...
    cuts = [2, ps + 1, 2, 2, 13, ps + 1, 2, 30, 2, 2, 2] + [ps] * 4 + [ps] * 2
    assert sum(cuts) < len(toks)
    got, at, held = [], 0, []
    for n in cuts:
        got.append(runner.step([StepEntry("x", toks[at:at + n], list(range(n)))]).clone())
        at += n
        held.append(runner.cache.pages_held("x")[0])
    while at < len(toks):                                       # decode past pages that were given back
        got.append(runner.step([StepEntry("x", toks[at:at + 1], [0])]).clone())
        at += 1
        held.append(runner.cache.pages_held("x")[0])
    runner.check_status()
    runner.cache.check()
    assert max(held) <= 10 and held[-1] <= -(-window // ps) + 1   # only the window's pages are held
    assert rel_err(torch.cat(got), want) < tol
    # a second request beside the first: pages freed and retaken within the same steps
    a, b = toks[:90], scenarios.make_requests([70], pcfg["vocab_size"], seed=6)["r0"]
    want_b = plain_lfm2.forward(pcfg, w, b, round_bf16=(dtype == torch.bfloat16))
    runner.finish("x")
    out_a, out_b, ia, ib = [], [], 0, 0
    while ia < len(a) or ib < len(b):
        entries = []
        na, nb = min(7, len(a) - ia), min(1 if ib >= 40 else 9, len(b) - ib)
        if na:
            entries.append(StepEntry("a", a[ia:ia + na], list(range(na))))
        if nb:
            entries.append(StepEntry("b", b[ib:ib + nb], list(range(nb))))
        lg = runner.step(entries).clone()
        out_a.append(lg[:na])
        out_b.append(lg[na:na + nb])
        ia, ib = ia + na, ib + nb
    runner.check_status()
    runner.cache.check()
    assert rel_err(torch.cat(out_a), want[:90]) < tol and rel_err(torch.cat(out_b), want_b) < tol
    runner.finish("a")
    runner.finish("b")
    assert runner.cache.pages_free() == [10]


# ---------------------------------------------------------------------------------------------
# a position encoding that is no rotation at all, defined here: a bias on the scores that grows
# with the distance between query and key, one slope per head.  The part hands the slopes to the
# attention kernels through PositionArgs; no kernel and no framework file changes.
@dataclasses.dataclass(frozen=True)
class DistanceBiasSpec:
    n_heads: int
    kind: str = "toy_distance_bias"


@register("position", "toy_distance_bias")
class DistanceBias:
    def __init__(self, spec, *, device):
        from neurogrid_b200.parts import PositionArgs
        self.slopes = torch.tensor([2.0 ** (-(h + 1) * 8.0 / spec.n_heads) for h in range(spec.n_heads)],
                                   dtype=torch.float32, device=device)
        self.args = PositionArgs(score_slopes=self.slopes)

    def kernel_args(self):
        return self.args


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,ps", [(64, 16), (32, 8)])
def test_toy_score_bias_reaches_every_attention_kernel(dtype, hd, ps):
    """Head size 64 with pages of 16 runs the tcgen05 portion kernel and the split decode kernel in
    bfloat16, head size 32 the mma.sync portion kernel; float32 runs the order-fixed kernel."""
    from neurogrid_b200.parts import PagedView, build
    from neurogrid_b200.weights import draw
    from helpers import make_ctx
    nH, nKV, T = 4, 2, 150
    H = nH * hd
    spec = AttentionSpec(H, nH, nKV, hd, DistanceBiasSpec(nH), qk_norm=False)
    part = build("mixer", spec, dtype=dtype, device="cuda")
    w = draw(part.tensors(), 3)
    part.bind(w)
    w = {k: v.double() for k, v in w.items()}
    g = torch.Generator().manual_seed(2)
    x = (3 * torch.randn(T, H, generator=g)).to(torch.bfloat16).to(dtype).to("cuda")
    xs = x.double().cpu()
    rb = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t)
    q = rb(xs @ w["q_proj.weight"].T).reshape(T, nH, hd)
    k = rb(xs @ w["k_proj.weight"].T).reshape(T, nKV, hd)
    v = rb(xs @ w["v_proj.weight"].T).reshape(T, nKV, hd)
    pos = torch.arange(T, dtype=torch.float64)
    dist = pos[:, None] - pos[None, :]
    mask = dist < 0
    slopes = part.position.slopes.double().cpu()
    heads = []
    for h in range(nH):
        sc = (q[:, h] @ k[:, h // (nH // nKV)].T) / math.sqrt(hd) - slopes[h] * dist
        p = torch.softmax(sc.masked_fill(mask, -1e300), -1)
        heads.append(p @ v[:, h // (nH // nKV)])
    want = rb(torch.stack(heads, 1).reshape(T, -1)) @ w["o_proj.weight"].T
    # the bias matters: without it the output differs
    plain = torch.stack([torch.softmax(((q[:, h] @ k[:, h // (nH // nKV)].T) / math.sqrt(hd)).masked_fill(mask, -1e300), -1)
                         @ v[:, h // (nH // nKV)] for h in range(nH)], 1).reshape(T, -1) @ w["o_proj.weight"].T
    assert rel_err(plain, want) > 5e-2
    pages = 32
    kp = torch.randn(pages, nKV, ps, hd, device="cuda").to(dtype)
    vp = torch.randn(pages, nKV, ps, hd, device="cuda").to(dtype)
    table = torch.full((1, pages), -1, dtype=torch.int32)
    table[0, : -(-T // ps)] = torch.randperm(pages)[: -(-T // ps)].to(torch.int32)
    view = PagedView(kp, vp, table.to("cuda"))
    got, at = [], 0
    for n in (70, 1, 1, 40, 1, 37):
        got.append(part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [0], dtype=dtype), view).clone())
        at += n
    assert at == T
    assert rel_err(torch.cat(got), want) < (1e-4 if dtype == torch.float32 else 2e-2)


# ---------------------------------------------------------------------------------------------
# a state in bfloat16 that starts at a value of its own, learned absolute positions, and CUDA
# graphs around parts that are not graph-safe: a toy architecture of two mixer kinds.
@dataclass(frozen=True)
class EmaSpec:
    hidden: int
    rate: float
    start: float
    kind: str = "toy_ema"


@register("mixer", "toy_ema")
class EmaMixer:
    """s[t] = (1 - rate) * s[t-1] + rate * x[t], kept in bfloat16, starting at ``start``;  y[t] = s[t] * gain."""

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def tensors(self):
        return {"gain": TensorDecl((self.spec.hidden,), "norm")}

    def bind(self, t):
        self.gain = t["gain"].to(self.device, torch.float32)

    def cache_need(self):
        return SlotNeed((self.spec.hidden,), dtype="bfloat16", init=self.spec.start)

    def forward(self, x, ctx, cache):
        assert cache.state.dtype == torch.bfloat16
        out = ctx.ws.buf("mixer_out", x.shape[0], self.spec.hidden, self.dtype)
        row, r = 0, self.spec.rate
        for q, slot in zip(ctx.q_lens, ctx.slot_ids):
            s = cache.state[slot].float()
            for t in range(q):
                s = ((1 - r) * s + r * x[row + t].float()).to(torch.bfloat16).float()
                out[row + t] = (s * self.gain).to(self.dtype)
            cache.state[slot] = s.to(torch.bfloat16)
            row += q
        return out


class EmaConfig:
    architecture = "ToyEmaForCausalLM"

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def model_spec(self):
        H, V = self.d["width"], self.d["vocab_size"]
        norm = RMSNormSpec(H, 1e-5)
        names = dict(mixer="mixer", ffn="ffn", mixer_norm="norm1", ffn_norm="norm2")
        attn = AttentionSpec(H, 4, 2, 16, RopeSpec(16, 1e4, "half"))
        ema = EmaSpec(H, 0.25, self.d["start"])
        layers = (LayerSpec(attn, SwiGLUSpec(H, 96), norm, norm, "toy.0.", names),
                  LayerSpec(ema, SwiGLUSpec(H, 96), norm, norm, "toy.1.", names),
                  LayerSpec(attn, SwiGLUSpec(H, 96), norm, norm, "toy.2.", names))
        return ModelSpec("ToyEmaForCausalLM", V, H, layers, tuple(ScheduleEntry(i, i) for i in range(3)), norm, True,
                         128, embed_name="toy.embed.weight", final_norm_name="toy.norm.weight",
                         position_table_name="toy.positions.weight")


def _ema_plain(w, tokens, start, dtype):
    """The toy model restated with the plain implementation's parts (float64, whole sequence)."""
    import plain_lfm2 as P
    rb = dtype == torch.bfloat16
    r = (lambda t: t.to(torch.bfloat16).double()) if rb else (lambda t: t)
    w = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    h = w["toy.embed.weight"][torch.tensor(tokens)] + w["toy.positions.weight"][:T]
    for i in range(3):
        p = f"toy.{i}."
        n = r(P.rmsnorm(h, w[p + "norm1.weight"], 1e-5))
        if i == 1:
            s = torch.full((h.shape[1],), start, dtype=torch.float64).to(torch.bfloat16).double()
            rows = []
            for t in range(T):
                s = (0.75 * s.float() + 0.25 * n[t].float()).to(torch.bfloat16).double()
                rows.append(r(s.float() * w[p + "mixer.gain"].float()).double() if rb else s * w[p + "mixer.gain"])
            m = torch.stack(rows)
        else:
            m = P.attention(n, w[p + "mixer.q_proj.weight"], w[p + "mixer.k_proj.weight"], w[p + "mixer.v_proj.weight"],
                            w[p + "mixer.o_proj.weight"], None, None, n_heads=4, n_kv=2, hd=16, eps=1e-6, theta=1e4,
                            pairing="half", rb=rb)
        h = h + m
        n = r(P.rmsnorm(h, w[p + "norm2.weight"], 1e-5))
        h = h + P.swiglu(n, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"], rb)
    return r(P.rmsnorm(h, w["toy.norm.weight"], 1e-5)) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_state_dtype_start_value_positions_and_graphs_around_eager_parts(tmp_path, dtype):
    from safetensors.torch import load_file
    register_architecture("ToyEmaForCausalLM", EmaConfig)
    folder = write_random_model({"architectures": ["ToyEmaForCausalLM"], "width": 64, "vocab_size": 90, "start": 0.5},
                                11, str(tmp_path / "ema"))
    w = load_file(folder + "/model.safetensors")
    assert w["toy.positions.weight"].shape == (128, 64)
    runner = make_runner(folder, dtype=dtype, device="cuda", num_pages=16, page_size=16, max_seq_len=128)
    assert runner.storage.state[0].dtype == torch.bfloat16 and float(runner.storage.state[0].float().mean()) == 0.5
    # graphs stay on although the middle layer's mixer is plain PyTorch: it runs between two graphs
    assert runner.cuda_graphs and [s for s, _ in runner._pieces] == [True, False, True]
    toks = scenarios.make_requests([60], 90, seed=5)["r0"]
    want = _ema_plain(w, toks, 0.5, dtype)
    got = [runner.step([StepEntry("x", toks[:20], list(range(20)))]).clone()]
    got += [runner.step([StepEntry("x", [t], [0])]).clone() for t in toks[20:]]
    runner.check_status()
    assert runner.stats()["graph_replays"] >= 30                 # the single-token steps replayed graphs
    assert rel_err(torch.cat(got), want) < (1e-4 if dtype == torch.float32 else 2e-2)
    # a slot handed to the next request starts at the start value again, not where the last one left it
    runner.finish("x")
    again = runner.step([StepEntry("y", toks[:20], list(range(20)))]).clone()
    assert rel_err(again, want[:20]) < (1e-4 if dtype == torch.float32 else 2e-2)


# ------------------------------------------------------------------------------------------------------
# another norm: a LayerNorm with a bias (mean-centred), in plain PyTorch, for every norm of a toy model.
@dataclass(frozen=True)
class CentredNormSpec:
    size: int
    eps: float
    kind: str = "toy_layernorm"


@register("norm", "toy_layernorm")
class CentredNorm:
    """h += delta (float32; delta is nothing, a tensor of the activation dtype, or a float32 stack of
    partial sums), then y = (h - mean) / sqrt(var + eps) * w + b for the rows asked for."""

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def tensors(self):
        return {"weight": TensorDecl((self.spec.size,), "norm"), "bias": TensorDecl((self.spec.size,), "bias")}

    def bind(self, t):
        self.w = t["weight"].to(self.device, torch.float32)
        self.b = t["bias"].to(self.device, torch.float32)

    def forward(self, h, delta, out, rows=None):
        if delta is not None:
            h += delta.float().sum(0) if delta.dim() == 3 else delta.float()
        x = h if rows is None else h[rows.long()]
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        out.copy_(((x - mu) * torch.rsqrt(var + self.spec.eps) * self.w + self.b).to(out.dtype))
        return out


class CentredConfig:
    architecture = "ToyCentredForCausalLM"

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def model_spec(self):
        H, V = self.d["width"], self.d["vocab_size"]
        norm = CentredNormSpec(H, 1e-5)
        names = dict(mixer="mixer", ffn="ffn", mixer_norm="norm1", ffn_norm="norm2")
        attn = AttentionSpec(H, 4, 2, 16, RopeSpec(16, 1e4, "half"))
        layers = tuple(LayerSpec(attn, SwiGLUSpec(H, 80), norm, norm, f"toy.{i}.", names) for i in range(2))
        return ModelSpec("ToyCentredForCausalLM", V, H, layers, tuple(ScheduleEntry(i, i) for i in range(2)), norm, True,
                         128, embed_name="toy.embed.weight", final_norm_name="toy.norm.weight")


def _centred_plain(w, tokens, dtype):
    import plain_lfm2 as P
    rb = dtype == torch.bfloat16
    r = (lambda t: t.to(torch.bfloat16).double()) if rb else (lambda t: t)
    w = {k: v.double() for k, v in w.items()}

    def norm(x, name):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return r((x - mu) / torch.sqrt(var + 1e-5) * w[name + ".weight"] + w[name + ".bias"])

    h = w["toy.embed.weight"][torch.tensor(tokens)]
    for i in range(2):
        p = f"toy.{i}."
        n = norm(h, p + "norm1")
        h = h + P.attention(n, w[p + "mixer.q_proj.weight"], w[p + "mixer.k_proj.weight"], w[p + "mixer.v_proj.weight"],
                            w[p + "mixer.o_proj.weight"], None, None, n_heads=4, n_kv=2, hd=16, eps=1e-6, theta=1e4,
                            pairing="half", rb=rb)
        n = norm(h, p + "norm2")
        h = h + P.swiglu(n, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"], rb)
    return norm(h, "toy.norm") @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_norm_is_registered_and_used_for_every_norm_of_a_model(tmp_path, dtype):
    from safetensors.torch import load_file
    register_architecture("ToyCentredForCausalLM", CentredConfig)
    folder = write_random_model({"architectures": ["ToyCentredForCausalLM"], "width": 64, "vocab_size": 77}, 4,
                                str(tmp_path / "centred"))
    w = load_file(folder + "/model.safetensors")
    assert "toy.0.norm1.bias" in w and "toy.norm.bias" in w
    runner = make_runner(folder, dtype=dtype, device="cuda", num_pages=16, page_size=16, max_seq_len=128)
    toks = scenarios.make_requests([50], 77, seed=2)["r0"]
    want = _centred_plain(w, toks, dtype)
    got = [runner.step([StepEntry("x", toks[:30], list(range(30)))]).clone()]
    got += [runner.step([StepEntry("x", [t], [0])]).clone() for t in toks[30:]]
    runner.check_status()
    assert rel_err(torch.cat(got), want) < (1e-4 if dtype == torch.float32 else 2e-2)


# ------------------------------------------------------------------------------------------------------
# another arrangement of a block: mixer and feed-forward side by side on one norm,
# y = x + mixer(norm(x)) + ffn(norm(x)).
@register("block", "toy_parallel")
class ParallelBlock:
    def __init__(self, spec, *, dtype, device, owns_cache=True):
        from neurogrid_b200.parts import registry
        self.spec, self.dtype = spec, dtype
        kw = dict(dtype=dtype, device=device)
        self.mixer = registry.build("mixer", spec.mixer, **kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw)
        self.norm = registry.build("norm", spec.mixer_norm, **kw)

    def parts(self):
        n = self.spec.names
        return {n["mixer"]: self.mixer, n["ffn"]: self.ffn, n["mixer_norm"]: self.norm}

    def tensors(self):
        return {f"{sub}.{name}": decl for sub, part in self.parts().items() for name, decl in part.tensors().items()}

    def bind(self, t):
        for sub, part in self.parts().items():
            part.bind({k[len(sub) + 1:]: v for k, v in t.items() if k.startswith(sub + ".")})

    def cache_need(self):
        return self.mixer.cache_need()

    def kernels(self):
        return [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    graph_safe = False                                  # the sum below is a PyTorch expression

    def forward(self, h, pending, ctx, cache):
        ctx.residual = None                             # both outputs come back as tensors
        x = self.norm.forward(h, pending, ctx.ws.buf("normed", h.shape[0], h.shape[1], self.dtype))
        m = self.mixer.forward(x, ctx, cache)
        f = self.ffn.forward(x, ctx)
        out = ctx.ws.buf("parallel_out", h.shape[0], h.shape[1], self.dtype)
        torch.add(m if m.dim() == 2 else m.sum(0).to(self.dtype), f if f.dim() == 2 else f.sum(0).to(self.dtype), out=out)
        return out


class ParallelConfig:
    architecture = "ToyParallelForCausalLM"

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def model_spec(self):
        H, V = self.d["width"], self.d["vocab_size"]
        norm = RMSNormSpec(H, 1e-5)
        names = dict(mixer="mixer", ffn="ffn", mixer_norm="norm", ffn_norm="unused")
        attn = AttentionSpec(H, 4, 2, 16, RopeSpec(16, 1e4, "half"))
        layers = tuple(LayerSpec(attn, SwiGLUSpec(H, 80), norm, norm, f"toy.{i}.", names, block="toy_parallel")
                       for i in range(3))
        return ModelSpec("ToyParallelForCausalLM", V, H, layers, tuple(ScheduleEntry(i, i) for i in range(3)), norm, True,
                         128, embed_name="toy.embed.weight", final_norm_name="toy.norm.weight")


def _parallel_plain(w, tokens, dtype):
    import plain_lfm2 as P
    rb = dtype == torch.bfloat16
    r = (lambda t: t.to(torch.bfloat16).double()) if rb else (lambda t: t)
    w = {k: v.double() for k, v in w.items()}
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    for i in range(3):
        p = f"toy.{i}."
        n = r(P.rmsnorm(h, w[p + "norm.weight"], 1e-5))
        m = P.attention(n, w[p + "mixer.q_proj.weight"], w[p + "mixer.k_proj.weight"], w[p + "mixer.v_proj.weight"],
                        w[p + "mixer.o_proj.weight"], None, None, n_heads=4, n_kv=2, hd=16, eps=1e-6, theta=1e4,
                        pairing="half", rb=rb)
        f = P.swiglu(n, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"], rb)
        h = h + r(m + f)
    return r(P.rmsnorm(h, w["toy.norm.weight"], 1e-5)) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_block_arrangement_is_registered_and_stepped(tmp_path, dtype):
    from safetensors.torch import load_file
    register_architecture("ToyParallelForCausalLM", ParallelConfig)
    folder = write_random_model({"architectures": ["ToyParallelForCausalLM"], "width": 64, "vocab_size": 83}, 6,
                                str(tmp_path / "parallel"))
    w = load_file(folder + "/model.safetensors")
    assert "toy.0.norm.weight" in w and not any("unused" in k for k in w)
    runner = make_runner(folder, dtype=dtype, device="cuda", num_pages=16, page_size=16, max_seq_len=128)
    toks = scenarios.make_requests([45], 83, seed=8)["r0"]
    want = _parallel_plain(w, toks, dtype)
    got = [runner.step([StepEntry("x", toks[:25], list(range(25)))]).clone()]
    got += [runner.step([StepEntry("x", [t], [0])]).clone() for t in toks[25:]]
    runner.check_status()
    assert rel_err(torch.cat(got), want) < (1e-4 if dtype == torch.float32 else 2e-2)
