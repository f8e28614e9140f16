"""Redodra: a decoder-only language model lowered to op lists (seq_ops.StepBuilder) for seq_engine.SequenceEngine.

With N(v; n) = tanh(alpha_n v) * w_n + b_n (dynamic-tanh norm: no statistics), layer i (tensors `l<i>.*`) turns its input x into
    y  = x + N(mixer(N(x; norm1)); norm1b)
    X  = y + N(ff(N(y; norm2)); norm2b)                       (no feed-forward: X = y)
and hands on  sum_(j <= i + 1) dwa_i[j] * X_j,  X_0 being the embedding output and X_(j + 1) layer j's own X: every layer's output
is kept for the step (`hist`), and FQ3C_DEPTH_MIX forms the sum.  Mixers: gated delta rule (state: conv inputs, S), gated sink
attention with partial rotary positions (state: key / value cache, or another layer's), or windowed attention and a state-space
scan side by side (state: cache; conv inputs, S).  Feed-forward: xIELU.  Output: N(x; final.norm), then the head.

This file only packs the checkpoint's tensors into the layouts the mechanisms take and strings the mechanisms together in the
configured order; the kernels, the state manager and the step loop are the shared ones.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .config import DeltaRuleConfig, ParallelMixerConfig, RedodraConfig, SoftmaxAttentionConfig
from .seq_ops import StepBuilder
from .seq_state import StateSpec

NORMS = ("norm1", "norm1b", "norm2", "norm2b")


def _attention_specs(p: str, m: SoftmaxAttentionConfig, W: int) -> Dict[str, tuple]:
    out = {p + "q": (m.heads * m.dim, W), p + "o": (W, m.heads * m.vdim)}
    if m.kv_from is None:
        out.update({p + "k": (m.kv_heads * m.dim, W), p + "v": (m.kv_heads * m.vdim, W)})
    if m.bias:
        out.update({k + ".b": (s[0],) for k, s in list(out.items())})
    if m.sink:
        out[p + "sink"] = (m.heads,)
    if m.gate:
        out[p + "g"] = (m.heads, W)
    if m.distance:
        out.update({p + "r1": (m.heads,), p + "r2": (m.heads,)})
    return out


def tensor_specs(cfg: RedodraConfig) -> Dict[str, tuple]:
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    W = cfg.width
    out = {"embed": (cfg.vocab, W), "head": (cfg.vocab, W)}

    def norm(name):
        out.update({name: (W,), name + ".b": (W,), name + ".alpha": ()})

    norm("final.norm")
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        norm(p + "norm1")
        norm(p + "norm1b")
        m = L.mixer
        if isinstance(m, DeltaRuleConfig):
            qk, v = m.kv_heads * m.dim, m.heads * m.vdim
            out.update({p + "mix.q": (qk, W), p + "mix.q.conv": (qk, m.conv), p + "mix.k": (qk, W), p + "mix.k.conv": (qk, m.conv),
                        p + "mix.v": (v, W), p + "mix.v.conv": (v, m.conv), p + "mix.b": (m.heads, W), p + "mix.a": (m.heads, W),
                        p + "mix.A_log": (m.heads,), p + "mix.dt_bias": (m.heads,), p + "mix.norm": (m.vdim,), p + "mix.g": (v, W),
                        p + "mix.o": (W, v)})
        elif isinstance(m, SoftmaxAttentionConfig):
            out.update(_attention_specs(p + "mix.", m, W))
        else:
            r = m.right
            nconv = r.inner + 2 * r.groups * r.state
            out.update(_attention_specs(p + "mix.left.", m.left, W))
            out.update({p + "mix.right.in": (r.inner + nconv + r.heads, W), p + "mix.right.conv": (nconv, r.conv),
                        p + "mix.right.conv.b": (nconv,), p + "mix.right.dt_bias": (r.heads,), p + "mix.right.A_log": (r.heads,),
                        p + "mix.right.D": (r.heads,), p + "mix.right.norm": (r.inner,), p + "mix.right.o": (W, r.inner),
                        p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        if L.mlp is not None:
            norm(p + "norm2")
            norm(p + "norm2b")
            out.update({p + "mlp.up": (L.mlp.ff, W), p + "mlp.down": (W, L.mlp.ff), p + "mlp.act": (2,)})
        out[p + "dwa"] = (i + 2,)
    return out


def init_synthetic(cfg: RedodraConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a configuration (no checkpoint offline): products scaled by 1/sqrt(fan-in)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_specs(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = 0.6 + 0.3 * torch.rand((), generator=g)
        elif last == "dwa":
            t = torch.full(shape, 0.25 / shape[0]) + 0.1 * torch.randn(shape, generator=g)
            t[-1] += 0.8
        elif last in NORMS or name.endswith(("final.norm", "mix.norm", ".out")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.tensor([0.3, -0.2]) + 0.1 * torch.randn(2, generator=g)
        elif last == "A_log":
            t = torch.log(0.5 + 4.0 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = -1.5 + torch.randn(shape, generator=g)
        elif last in ("r1", "r2"):
            t = 0.05 + 0.5 * torch.rand(shape, generator=g)
        elif last in ("sink", "b", "D") and len(shape) <= 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


class Packer:
    """Checkpoint tensors -> the layouts the mechanisms of seq_ops.StepBuilder take.  `raw(name)` gives a CPU f32 tensor."""

    def __init__(self, raw: Callable[[str], torch.Tensor], device, f32: bool):
        self.raw, self.device, self.wdt = raw, torch.device(device), torch.float32 if f32 else torch.bfloat16

    def W(self, t):   # product operand
        return t.to(self.device, self.wdt).contiguous()

    def F(self, t):   # always-f32 parameter
        return t.to(self.device, torch.float32).contiguous()

    def norm(self, name: str) -> dict:
        w, b = self.raw(name), self.raw(name + ".b")
        return {"alpha": float(self.raw(name + ".alpha")), "w": self.F(w), "b": self.F(b), "wb": self.F(torch.cat([w, b]))}

    def attention(self, p: str, m: SoftmaxAttentionConfig) -> dict:
        raw, W, F = self.raw, self.W, self.F
        parts = [p + "q"] + ([p + "k", p + "v"] if m.kv_from is None else [])
        rows = [raw(n) for n in parts] + ([raw(p + "g")] if m.gate else [])
        d = {"wqkv": W(torch.cat(rows, 0)), "o": W(raw(p + "o")), "bqkv": None, "o_b": None, "freq": None, "sink": None, "r12": None}
        if m.bias:
            d["bqkv"] = F(torch.cat([raw(n + ".b") for n in parts] + ([torch.zeros(m.heads)] if m.gate else [])))
            d["o_b"] = F(raw(p + "o.b"))
        if m.rot_dims > 0:
            i = torch.arange(m.rot_dims // 2, dtype=torch.float64)
            d["freq"] = F(torch.as_tensor(m.rot_base, dtype=torch.float64) ** (-2.0 * i / m.rot_dims))
        if m.sink:
            d["sink"] = F(raw(p + "sink"))
        if m.distance:
            d["r12"] = F(torch.cat([raw(p + "r1"), raw(p + "r2")]))
        return d

    def delta_rule(self, q: str) -> dict:
        raw, W, F = self.raw, self.W, self.F
        return {"win": W(torch.cat([raw(q + n) for n in ("q", "k", "v", "g", "a", "b")], 0)),
                "conv": F(torch.cat([raw(q + n + ".conv") for n in ("q", "k", "v")], 0)), "A_log": F(raw(q + "A_log")),
                "dt_bias": F(raw(q + "dt_bias")), "norm": F(raw(q + "norm")), "o": W(raw(q + "o"))}

    def state_space(self, r: str) -> dict:
        raw, W, F = self.raw, self.W, self.F
        return {"win": W(raw(r + "in")), "conv": F(raw(r + "conv")), "conv_b": F(raw(r + "conv.b")), "A_log": F(raw(r + "A_log")),
                "dt_bias": F(raw(r + "dt_bias")), "D": F(raw(r + "D")), "norm": F(raw(r + "norm")), "o": W(raw(r + "o"))}

    def xielu_ff(self, p: str) -> dict:
        return {"up": self.W(self.raw(p + "up")), "down": self.W(self.raw(p + "down")), "act": self.F(self.raw(p + "act"))}


class RedodraModel:
    def __init__(self, cfg: RedodraConfig, get: Callable[[str], Optional[torch.Tensor]], device, f32: bool = False):
        """`get(name)` returns a CPU tensor or None."""
        self.cfg, self.device, self.f32 = cfg, torch.device(device), bool(f32)
        self.wdt = torch.float32 if f32 else torch.bfloat16
        self.vocab, self.width = cfg.vocab, cfg.width
        specs = tensor_specs(cfg)

        def raw(name):
            t = get(name)
            if t is None:
                raise KeyError(f"tensor {name!r} is missing")
            if tuple(t.shape) != tuple(specs[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration implies {tuple(specs[name])}")
            return t.to(torch.float32)

        pk = Packer(raw, self.device, self.f32)
        self.g: Dict[str, object] = {"embed": pk.W(raw("embed")), "final.norm": pk.norm("final.norm"), "head": pk.W(raw("head"))}
        self.layers: List[dict] = []
        for i, L in enumerate(cfg.layers):
            p = f"l{i}."
            d: dict = {"norm1": pk.norm(p + "norm1"), "norm1b": pk.norm(p + "norm1b"), "dwa": pk.F(raw(p + "dwa"))}
            m = L.mixer
            q = p + "mix."
            if isinstance(m, DeltaRuleConfig):
                d["mix"] = pk.delta_rule(q)
            elif isinstance(m, SoftmaxAttentionConfig):
                d["mix"] = pk.attention(q, m)
            else:
                # the halving of the sum is folded into the two output norms' weights (exact: a power of two)
                d["mix"] = {"left": pk.attention(q + "left.", m.left), "right": pk.state_space(q + "right."),
                            "left_out": pk.F(0.5 * raw(q + "left.out")), "right_out": pk.F(0.5 * raw(q + "right.out"))}
            if L.mlp is not None:
                d["norm2"], d["norm2b"] = pk.norm(p + "norm2"), pk.norm(p + "norm2b")
                d["ff"] = pk.xielu_ff(p + "mlp.")
            self.layers.append(d)

    # ---- what a sequence keeps between steps ------------------------------------------------------
    def state_specs(self) -> List[StateSpec]:
        out = []

        def cache(i, m: SoftmaxAttentionConfig):
            if m.kv_from is None:
                out.append(StateSpec(f"l{i}.k", "append", m.kv_heads * m.dim, dtype=self.wdt))
                out.append(StateSpec(f"l{i}.v", "append", m.kv_heads * m.vdim, dtype=self.wdt))

        for i, L in enumerate(self.cfg.layers):
            m = L.mixer
            if isinstance(m, DeltaRuleConfig):
                if m.conv > 1:
                    out.append(StateSpec(f"l{i}.dr.conv", "carry", 2 * m.kv_heads * m.dim + m.heads * m.vdim, m.conv - 1))
                out.append(StateSpec(f"l{i}.dr.s", "carry", m.vdim, m.heads * m.dim))
            elif isinstance(m, SoftmaxAttentionConfig):
                cache(i, m)
            else:
                cache(i, m.left)
                r = m.right
                if r.conv > 1:
                    out.append(StateSpec(f"l{i}.ss.conv", "carry", r.inner + 2 * r.groups * r.state, r.conv - 1))
                out.append(StateSpec(f"l{i}.ss.s", "carry", r.vdim, r.heads * r.state))
        return out

    # ---- one step of M tokens -----------------------------------------------------------------------
    def build_step(self, b: StepBuilder, ids: torch.Tensor, layer_taps: Optional[list] = None):
        """ids: device int32 [M].  Returns the f32 stream that the output norm reads, [M, width].  `layer_taps`, when given, receives
        one f32 buffer per layer holding what that layer hands on (debugging, tests)."""
        c, M, Wd = self.cfg, b.M, self.cfg.width
        n = len(c.layers)
        hist = torch.zeros(n + 1, M, Wd, dtype=torch.float32, device=self.device)      # X_0 .. X_n of this step
        b.plan.keep.append(hist)
        hn = b.buf("hn", M, Wd, b.adt)        # a norm's output: what the next products read
        b.embed(ids, self.g["embed"], hist[0])
        x = hist[0]
        if n:
            b.dyt(x, self.layers[0]["norm1"], hn)
        for i, (L, w) in enumerate(zip(c.layers, self.layers)):
            m, X = L.mixer, hist[i + 1]
            mo = b.buf("mo", M, Wd)
            if isinstance(m, DeltaRuleConfig):
                b.delta_rule(hn, m, w["mix"], f"l{i}.dr", c.norm_eps, mo)
            elif isinstance(m, SoftmaxAttentionConfig):
                j = i if m.kv_from is None else m.kv_from
                b.softmax_attention(hn, m, w["mix"], f"l{j}.k", f"l{j}.v", mo)
            else:
                lo = b.softmax_attention(hn, m.left, w["mix"]["left"], f"l{i}.k", f"l{i}.v", b.buf("par.l", M, Wd))
                ro = b.state_space(hn, m.right, w["mix"]["right"], f"l{i}.ss", c.norm_eps, b.buf("par.r", M, Wd))
                b.group_norm(lo, w["mix"]["left_out"], 1, c.norm_eps, mo)
                b.group_norm(ro, w["mix"]["right_out"], 1, c.norm_eps, mo, residual=mo)
            if L.mlp is not None:
                b.dyt(mo, w["norm1b"], X, residual=x, chain=(w["norm2"], hn))
                fo = b.xielu_ff(hn, w["ff"], b.buf("fo", M, Wd))
                b.dyt(fo, w["norm2b"], X, residual=X)
            else:
                b.dyt(mo, w["norm1b"], X, residual=x)
            nxt = self.layers[i + 1]["norm1"] if i + 1 < n else None
            x = torch.zeros(M, Wd, dtype=torch.float32, device=self.device) if layer_taps is not None else b.buf("xmix", M, Wd)
            b.depth_mix(hist, i + 2, w["dwa"], x, chain=(nxt, hn) if nxt is not None else None)
            if layer_taps is not None:
                b.plan.keep.append(x)
                layer_taps.append(x)
        b.commit()
        return x

    def build_head(self, b: StepBuilder, x: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
        """`b` is a builder of b.M = wanted rows.  Logits f32 [b.M, vocab] of the rows of x (f32, a step's output) named by
        the device int32 index list `want`."""
        c = self.cfg
        rows = b.embed(want, x, b.buf("head.rows", b.M, c.width))
        xn = b.dyt(rows, self.g["final.norm"], b.buf("head.xn", b.M, c.width, b.adt))
        return b.linear(xn, self.g["head"], b.buf("head.logits", b.M, c.vocab))
