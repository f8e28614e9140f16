"""Plain, slow restatement of the Redodra design in float64 PyTorch on the CPU — the yardstick the CUDA path is held against.

One function per mechanism, written from the design's equations; it shares no code with the product path (it reads the raw
config dictionary and the checkpoint's tensor names directly) and keeps no cache: a sequence is always recomputed whole.

Notation: T tokens, x [T, width] the residual stream, W[name] the checkpoint tensor `name` as float64, linear weights [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---- element-wise pieces -------------------------------------------------------------------------------------------------
def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dyt_norm(v: torch.Tensor, W: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """Dynamic tanh: tanh(alpha v) * w + b; no mean, no variance, no eps."""
    return torch.tanh(W[name + ".alpha"] * v) * W[name] + W[name + ".b"]


def rms_unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def l2_unit(v: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return v / torch.sqrt((v * v).sum(-1, keepdim=True) + eps)


def causal_time_conv(v: torch.Tensor, taps_w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, c] = bias[c] + sum_j taps_w[c, j] * v[t - (taps - 1) + j, c]; zeros before the start; last column = current token."""
    T, C = v.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=v.dtype), v], 0)
    out = torch.zeros_like(v)
    for j in range(taps):
        out = out + taps_w[:, j] * padded[j:j + T]
    return out if bias is None else out + bias


def rotate_interleaved(v: torch.Tensor, dims: int, base: float, first_position: int = 0) -> torch.Tensor:
    """v [T, heads, d]: the first `dims` entries of each head turn in pairs (2i, 2i + 1) by the angle p * base^(-2i / dims)."""
    T = v.shape[0]
    out = v.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ang = (torch.arange(T, dtype=F64) + first_position) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ---- softmax attention (both attention mixers) ---------------------------------------------------------------------------
def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, softcap: Optional[float],
                     window: Optional[int] = None, keep_first: int = 0, sink: Optional[torch.Tensor] = None,
                     r1: Optional[torch.Tensor] = None, r2: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H / G).  Position i sees j <= i with
    (i - j < window or j < keep_first) when a window is given.  score = cap(scale q.k) - r1_h ln(1 + r2_h (i - j)); the
    denominator also holds exp(sink_h) when a sink is given."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            jt = torch.arange(i + 1)
            if window is not None:
                jt = jt[(i - jt < window) | (jt < keep_first)]
            s = (k[jt, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if r1 is not None:
                s = s - r1[h] * torch.log1p(r2[h] * (i - jt).to(F64))
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[jt, g]
    return out


def gated_sink_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, shared_kv=None):
    """The 'attention' mixer.  Returns (output [T, width], (k after rotation, v)) so that a later layer can borrow them."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    if rot:
        q = rotate_interleaved(q, rot["dims"], rot["base"])
    if shared_kv is None:
        k = (h @ W[p + "k"].T).reshape(T, G, d)
        if rot:
            k = rotate_interleaved(k, rot["dims"], rot["base"])
        v = (h @ W[p + "v"].T).reshape(T, G, dv)
    else:
        k, v = shared_kv
    o = masked_attention(q, k, v, m["scale"], m.get("softcap"), sink=W.get(p + "sink"))
    gate = torch.sigmoid(h @ W[p + "g"].T)                     # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T, (k, v)


def windowed_bias_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """Left half of the 'parallel' mixer: biased projections, no rotation, log-distance penalty, window with kept first tokens."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    mask = m.get("mask") or {}
    o = masked_attention(q, k, v, m["scale"], m.get("softcap"), window=mask.get("size"), keep_first=mask.get("keep_first", 0),
                         r1=W[p + "r1"], r2=W[p + "r2"])
    return o.reshape(T, H * dv) @ W[p + "o"].T + W[p + "o.b"]


# ---- recurrences ---------------------------------------------------------------------------------------------------------
def gated_delta_rule(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """The 'delta' mixer: S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  per head, S [dim, vdim] from zero."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_time_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_time_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_time_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = l2_unit(q) * d ** -0.5
    k = l2_unit(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                         # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(h @ W[p + "g"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = rms_unit(out, eps) * W[p + "norm"] * gate
    return out.reshape(T, H * dv) @ W[p + "o"].T


def state_space_duality(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Right half of the 'parallel' mixer: S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T (S [N, vdim]), y = S^T C + D x."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = h @ W[p + "in"].T
    z = zxbcdt[:, :inner]
    xbc = silu(causal_time_conv(zxbcdt[:, inner:2 * inner + 2 * G * N], W[p + "conv"], W[p + "conv.b"]))
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + W[p + "dt_bias"])            # [T, H]
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    A = torch.exp(W[p + "A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m.get("norm_groups", 1)
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def parallel_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = windowed_bias_attention(h, W, p + "left.", m["left"])
    right = state_space_duality(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * W[p + "left.out"] + rms_unit(right, eps) * W[p + "right.out"])


def xielu_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    act = W[p + "act"]
    return xielu(h @ W[p + "up"].T, act[0], act[1]) @ W[p + "down"].T


# ---- the model -----------------------------------------------------------------------------------------------------------
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  `taps`, when a list, receives the stream after every layer (after the depth average)."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(list(tokens))]
    history = [x]                                   # X_0 and every layer's own result
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        hin = dyt_norm(x, W, p + "norm1")
        m = L["mixer"]
        if L["type"] == "delta":
            mo = gated_delta_rule(hin, W, p + "mix.", m, eps)
        elif L["type"] == "parallel":
            mo = parallel_mixer(hin, W, p + "mix.", m, eps)
        elif L["type"] == "attention":
            mo, kv[i] = gated_sink_attention(hin, W, p + "mix.", m, kv.get(m.get("kv_from")) if m.get("kv_from") is not None else None)
        else:
            raise ValueError(L["type"])
        x = x + dyt_norm(mo, W, p + "norm1b")
        if L.get("mlp") is not None:
            x = x + dyt_norm(xielu_ff(dyt_norm(x, W, p + "norm2"), W, p + "mlp."), W, p + "norm2b")
        history.append(x)
        x = sum(W[p + "dwa"][j] * history[j] for j in range(i + 2))
        if taps is not None:
            taps.append(x)
    return dyt_norm(x, W, "final.norm") @ W["head"].T
