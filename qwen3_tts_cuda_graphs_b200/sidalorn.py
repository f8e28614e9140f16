"""Sidalorn: a decoder-only language model lowered to op lists (seq_ops.StepBuilder) for seq_engine.SequenceEngine.

Layer i (tensors `l<i>.*`), on the f32 residual stream x:
    h  = x + conv_t(x)                      `canon1` [width, taps]: causal, per channel; the last taps - 1 inputs are state
    x += gnorm(mixer(h)) * norm1            mixer: latent attention (state: the latent cache) or RG-LRU block (state: conv inputs, S)
    x += gnorm(ff(x)) * norm2               ff reads x itself: PolyNorm dense, or routed experts + identity experts + shared expert
gnorm = RMS norm inside each of `norm_groups` equal consecutive groups.  Output: gnorm(x) * final.norm, then the head.

This file only packs the checkpoint's tensors into the layouts the mechanisms take and strings the mechanisms together in the
configured order; the kernels, the state manager and the step loop are the shared ones.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .config import DenseFFConfig, LatentAttentionConfig, MoEFFConfig, RglruConfig, SidalornConfig
from .seq_ops import StepBuilder
from .seq_state import StateSpec


def tensor_specs(cfg: SidalornConfig) -> Dict[str, tuple]:
    """name -> shape of every tensor a checkpoint of this configuration holds (optional ones included)."""
    W = cfg.width
    out = {"embed": (cfg.vocab, W), "final.norm": (W,), "head": (cfg.vocab, W)}
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        out[p + "norm1"] = (W,)
        if cfg.canon_taps > 0:
            out[p + "canon1"] = (W, cfg.canon_taps)
        m = L.mixer
        if isinstance(m, LatentAttentionConfig):
            out.update({p + "mix.q": (m.heads * m.dim, W), p + "mix.dkv": (m.kv_rank, W), p + "mix.dkv.norm": (m.kv_rank,),
                        p + "mix.uk": (m.heads * m.dim, m.kv_rank), p + "mix.uv": (m.heads * m.vdim, m.kv_rank),
                        p + "mix.sink": (m.heads,), p + "mix.o": (W, m.heads * m.vdim)})
        else:
            bs = m.width // m.blocks
            out.update({p + "mix.y": (m.width, W), p + "mix.y.b": (m.width,), p + "mix.x": (m.width, W), p + "mix.x.b": (m.width,),
                        p + "mix.conv": (m.width, m.conv), p + "mix.conv.b": (m.width,), p + "mix.ra": (m.blocks, bs, bs),
                        p + "mix.ra.b": (m.blocks, bs), p + "mix.ri": (m.blocks, bs, bs), p + "mix.ri.b": (m.blocks, bs),
                        p + "mix.lam": (m.width,), p + "mix.o": (W, m.width)})
        f = L.mlp
        if f is None:
            continue
        out[p + "norm2"] = (W,)
        if isinstance(f, DenseFFConfig):
            out.update({p + "mlp.up": (f.ff, W), p + "mlp.down": (W, f.ff), p + "mlp.act": (4,)})
        else:
            out.update({p + "mlp.router": (f.routed, W), p + "mlp.correction": (f.routed,)})
            for e in range(f.experts):
                out[p + f"mlp.e{e}.up"] = (f.expert_ff, W)
                out[p + f"mlp.e{e}.down"] = (W, f.expert_ff)
            if f.shared_ff:
                out.update({p + "mlp.shared.up": (f.shared_ff, W), p + "mlp.shared.down": (W, f.shared_ff)})
    return out


OPTIONAL_SUFFIXES = (".sink", ".correction", ".y.b", ".x.b", ".conv.b", ".ra.b", ".ri.b")


def init_synthetic(cfg: SidalornConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a configuration (no checkpoint offline): products scaled by 1/sqrt(fan-in)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_specs(cfg).items():
        if name.endswith(("norm1", "norm2", "final.norm", "dkv.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".act"):
            t = torch.tensor([0.6, 0.3, 0.1, 0.05]) + 0.05 * torch.randn(4, generator=g)
        elif name.endswith((".sink", ".correction", ".b", ".lam")):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(("canon1", ".conv")):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


class SidalornModel:
    def __init__(self, cfg: SidalornConfig, get: Callable[[str], Optional[torch.Tensor]], device, f32: bool = False):
        """`get(name)` returns a CPU tensor or None (optional tensors)."""
        self.cfg, self.device, self.f32 = cfg, torch.device(device), bool(f32)
        self.wdt = torch.float32 if f32 else torch.bfloat16
        self.vocab, self.width = cfg.vocab, cfg.width
        specs = tensor_specs(cfg)

        def raw(name, optional=False):
            t = get(name)
            if t is None:
                if optional or name.endswith(OPTIONAL_SUFFIXES):
                    return None
                raise KeyError(f"tensor {name!r} is missing")
            if tuple(t.shape) != tuple(specs[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration implies {tuple(specs[name])}")
            return t.to(torch.float32)

        def W(t):   # product operand
            return None if t is None else t.to(self.device, self.wdt).contiguous()

        def F(t):   # always-f32 parameter
            return None if t is None else t.to(self.device, torch.float32).contiguous()

        self.g: Dict[str, object] = {"embed": W(raw("embed")), "final.norm": F(raw("final.norm")), "head": W(raw("head"))}
        self.layers: List[dict] = []
        for i, L in enumerate(cfg.layers):
            p = f"l{i}."
            d: dict = {"norm1": F(raw(p + "norm1"))}
            if cfg.canon_taps > 0:
                d["canon"] = F(raw(p + "canon1"))
            m = L.mixer
            if isinstance(m, LatentAttentionConfig):
                uk = raw(p + "mix.uk").reshape(m.heads, m.dim, m.kv_rank)
                d["mix"] = {"wqd": W(torch.cat([raw(p + "mix.q"), raw(p + "mix.dkv")], 0)), "dkv_norm": F(raw(p + "mix.dkv.norm")),
                            "uk_t": W(uk.transpose(1, 2)), "uv": W(raw(p + "mix.uv").reshape(m.heads, m.vdim, m.kv_rank)),
                            "sink": F(raw(p + "mix.sink")), "o": W(raw(p + "mix.o"))}
            else:
                yb, xb = raw(p + "mix.y.b"), raw(p + "mix.x.b")
                byx = None
                if yb is not None or xb is not None:
                    z = torch.zeros(m.width)
                    byx = torch.cat([yb if yb is not None else z, xb if xb is not None else z])
                rab, rib = raw(p + "mix.ra.b"), raw(p + "mix.ri.b")
                gb = None
                if rab is not None or rib is not None:
                    z = torch.zeros(m.width)
                    gb = torch.cat([(rab if rab is not None else z).reshape(-1), (rib if rib is not None else z).reshape(-1)])
                d["mix"] = {"wyx": W(torch.cat([raw(p + "mix.y"), raw(p + "mix.x")], 0)), "byx": F(byx), "conv": F(raw(p + "mix.conv")),
                            "conv_b": F(raw(p + "mix.conv.b")), "gates": W(torch.cat([raw(p + "mix.ra"), raw(p + "mix.ri")], 0)),
                            "gates_b": F(gb), "lam": F(raw(p + "mix.lam")), "o": W(raw(p + "mix.o"))}
            f = L.mlp
            if f is not None:
                d["norm2"] = F(raw(p + "norm2"))
                if isinstance(f, DenseFFConfig):
                    d["ff"] = {"up": W(raw(p + "mlp.up")), "down": W(raw(p + "mlp.down")), "act": F(raw(p + "mlp.act"))}
                else:
                    d["ff"] = {"router": W(raw(p + "mlp.router")), "correction": F(raw(p + "mlp.correction")),
                               "up": W(torch.stack([raw(p + f"mlp.e{e}.up") for e in range(f.experts)])),
                               "down": W(torch.stack([raw(p + f"mlp.e{e}.down") for e in range(f.experts)])),
                               "shared_up": W(raw(p + "mlp.shared.up")) if f.shared_ff else None,
                               "shared_down": W(raw(p + "mlp.shared.down")) if f.shared_ff else None}
            self.layers.append(d)

    # ---- what a sequence keeps between steps ------------------------------------------------------
    def state_specs(self) -> List[StateSpec]:
        c, out = self.cfg, []
        for i, L in enumerate(c.layers):
            if c.canon_taps > 1:
                out.append(StateSpec(f"l{i}.canon", "carry", c.width, c.canon_taps - 1))
            m = L.mixer
            if isinstance(m, LatentAttentionConfig):
                out.append(StateSpec(f"l{i}.latent", "append", m.kv_rank, dtype=self.wdt))
            else:
                if m.conv > 1:
                    out.append(StateSpec(f"l{i}.lru.conv", "carry", m.width, m.conv - 1))
                out.append(StateSpec(f"l{i}.lru.s", "carry", m.width, 1))
        return out

    # ---- one step of M tokens -----------------------------------------------------------------------
    def build_step(self, b: StepBuilder, ids: torch.Tensor, layer_taps: Optional[list] = None):
        """ids: device int32 [M].  Returns the f32 residual stream after the last layer, [M, width].  `layer_taps`, when given,
        receives one f32 buffer per layer that the step also fills with the stream after that layer (debugging, tests)."""
        c, M = self.cfg, b.M
        x = b.buf("x", M, c.width)
        # x as a product operand: the stream itself in 32-bit mode, else a bf16 copy that every norm refreshes as it updates x
        xb = None if b.f32 else b.buf("xb", M, c.width, torch.bfloat16)
        b.embed(ids, self.g["embed"], x)
        if xb is not None and (c.canon_taps == 0 or not c.layers):
            b.time_conv(x, self._one_tap(), "", xb)      # one tap of weight 1: the rounded copy
        for i, (L, w) in enumerate(zip(c.layers, self.layers)):
            if c.canon_taps > 0:
                h = b.time_conv(x, w["canon"], f"l{i}.canon", b.buf("h", M, c.width, b.adt), add_input=True)
            else:
                h = x if b.f32 else xb
            mo = b.buf("mo", M, c.width)
            if isinstance(L.mixer, LatentAttentionConfig):
                b.latent_attention(h, L.mixer, w["mix"], f"l{i}.latent", c.norm_eps, mo)
            else:
                b.rglru(h, L.mixer, w["mix"], f"l{i}.lru", mo)
            b.group_norm(mo, w["norm1"], c.norm_groups, c.norm_eps, x, residual=x, out_bf16=xb)
            if L.mlp is not None:
                fo = b.buf("fo", M, c.width)
                if isinstance(L.mlp, DenseFFConfig):
                    b.polynorm_ff(x if b.f32 else xb, w["ff"], c.norm_eps, fo)
                else:
                    b.moe_ff(x, x if b.f32 else xb, L.mlp, w["ff"], fo)
                b.group_norm(fo, w["norm2"], c.norm_groups, c.norm_eps, x, residual=x, out_bf16=xb)
            if layer_taps is not None:
                t = torch.zeros(M, c.width, dtype=torch.float32, device=self.device)
                b.time_conv(x, self._one_tap(), "", t)
                layer_taps.append(t)
        b.commit()
        return x

    def _one_tap(self) -> torch.Tensor:
        if "one" not in self.g:
            self.g["one"] = torch.ones(self.cfg.width, 1, dtype=torch.float32, device=self.device)
        return self.g["one"]

    def build_head(self, b: StepBuilder, x: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
        """`b` is a builder of b.M = wanted rows.  Logits f32 [b.M, vocab] of the rows of x (f32, a step's output) named by
        the device int32 index list `want`."""
        c = self.cfg
        rows = b.embed(want, x, b.buf("head.rows", b.M, c.width))
        xn = b.group_norm(rows, self.g["final.norm"], c.norm_groups, c.norm_eps, b.buf("head.xn", b.M, c.width, b.adt))
        return b.linear(xn, self.g["head"], b.buf("head.logits", b.M, c.vocab))
