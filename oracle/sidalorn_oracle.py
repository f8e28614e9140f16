"""Plain, slow restatement of the Sidalorn design in float64 PyTorch on the CPU — the yardstick the CUDA path is held against.

One function per mechanism, written from the design's equations; it shares no code with the product path (it reads the raw
config dictionary and the checkpoint's tensor names directly) and keeps no cache: a sequence is always recomputed whole.

Notation: T tokens, x [T, width] the residual stream, W[name] the checkpoint tensor `name` as float64, linear weights [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def grouped_rms_norm(v: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Split the last axis into `groups` equal consecutive parts, unit-RMS each part, multiply the whole by weight."""
    shape = v.shape
    parts = v.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms_unit(parts, eps).reshape(shape) * weight


def causal_time_conv(v: torch.Tensor, taps_w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, c] = bias[c] + sum_j taps_w[c, j] * v[t - (taps - 1) + j, c], zeros before the start (last column = current token)."""
    T, C = v.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=v.dtype), v], 0)
    out = torch.zeros_like(v)
    for j in range(taps):
        out = out + taps_w[:, j] * padded[j:j + T]
    return out if bias is None else out + bias


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Keys and values are per-head up-projections of one normed low-rank latent per position; causal; softmax with a sink."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    latent = rms_unit(h @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]
    k = (latent @ W[p + "uk"].T).reshape(T, H, dk)
    v = (latent @ W[p + "uv"].T).reshape(T, H, dv)
    sink = W[p + "sink"] if (p + "sink") in W else None
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):                                         # query i sees keys 0..i
        s = torch.einsum("jhd,hd->hj", k[: i + 1], q[i]) * m["scale"]          # [H, i + 1]
        top = s.max(-1).values if sink is None else torch.maximum(s.max(-1).values, sink)
        e = torch.exp(s - top[:, None])
        den = e.sum(-1) + (0.0 if sink is None else torch.exp(sink - top))     # the sink counts once, has no value
        out[i] = torch.einsum("hj,jhd->hd", e / den[:, None], v[: i + 1])
    return out.reshape(T, H * dv) @ W[p + "o"].T


def rglru_block(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """y = gelu_tanh(W_y h + b); u = conv(W_x h + b); block-diagonal sigmoid gates r, i from u; log a = -8 r softplus(lam);
    S_t = a S_(t-1) + sqrt(1 - a^2) (i * u), S_(-1) = 0; out = W_o (S * y)."""
    T = h.shape[0]
    B, width = m["blocks"], m["width"]

    def opt(name):
        return W[p + name] if (p + name) in W else 0.0

    y = gelu_tanh(h @ W[p + "y"].T + opt("y.b"))
    u = causal_time_conv(h @ W[p + "x"].T + opt("x.b"), W[p + "conv"], W.get(p + "conv.b"))
    ub = u.reshape(T, B, width // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ra"]) + opt("ra.b")).reshape(T, width)
    g = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ri"]) + opt("ri.b")).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(W[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * g * u
    S = torch.zeros(width, dtype=h.dtype)
    rows = []
    for t in range(T):
        S = a[t] * S + drive[t]
        rows.append(S * y[t])
    return torch.stack(rows) @ W[p + "o"].T


def polynorm_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    z = h @ W[p + "up"].T
    a, b, c, e = W[p + "act"]
    return (a * rms_unit(z, eps) + b * rms_unit(z ** 2, eps) + c * rms_unit(z ** 3, eps) + e) @ W[p + "down"].T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, r: dict):
    """Returns (chosen ids [T, top], weights [T, top]) — softmax scores, correction only for the choice, neighbour groups."""
    T = h.shape[0]
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ W[p + "router"].T, -1)
    choice = s + (W[p + "correction"] if (p + "correction") in W else 0.0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    gc, gk = groups["count"], groups["keep"]
    ids = torch.zeros(T, r["top"], dtype=torch.long)
    wts = torch.zeros(T, r["top"], dtype=h.dtype)
    for t in range(T):
        ch = choice[t].clone()
        gscore = ch.reshape(gc, n // gc).max(-1).values
        kept = set(torch.argsort(gscore, descending=True, stable=True)[:gk].tolist())
        for gidx in range(gc):
            if gidx not in kept:
                ch[gidx * (n // gc):(gidx + 1) * (n // gc)] = -math.inf
        order = torch.argsort(ch, descending=True, stable=True)[: r["top"]]
        ids[t] = order
        w = s[t, order]
        wts[t] = w / (w.sum() + 1e-20) * r.get("scale", 1.0)
    return ids, wts


def moe_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    r = f["router"]
    ids, wts = route(h, W, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            if e >= r["experts"]:
                out[t] += wts[t, j] * h[t]              # identity expert
            else:
                out[t] += wts[t, j] * (gelu_erf(h[t] @ W[p + f"e{e}.up"].T) @ W[p + f"e{e}.down"].T)
    if f.get("shared"):
        out = out + gelu_erf(h @ W[p + "shared.up"].T) @ W[p + "shared.down"].T
    return out


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; `layer_outputs` receives the stream after every layer."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    taps = (cfg.get("canon") or {}).get("taps", 0)
    x = W["embed"][torch.tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + causal_time_conv(x, W[p + "canon1"]) if taps > 0 else x
        if L["type"] == "latent_attention":
            mixed = latent_attention(h, W, p + "mix.", L["mixer"], eps)
        else:
            mixed = rglru_block(h, W, p + "mix.", L["mixer"])
        x = x + grouped_rms_norm(mixed, W[p + "norm1"], groups, eps)
        f = L.get("mlp")
        if f is not None:
            y = polynorm_ff(x, W, p + "mlp.", eps) if f["kind"] == "dense" else moe_ff(x, W, p + "mlp.", f)
            x = x + grouped_rms_norm(y, W[p + "norm2"], groups, eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return grouped_rms_norm(x, W["final.norm"], groups, eps) @ W["head"].T
