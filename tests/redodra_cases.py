"""Small Redodra configurations and random weights for the tests (raw config dictionaries, checkpoint tensor names)."""
import torch

from sidalorn_cases import save_checkpoint, tokens  # noqa: F401  (same checkpoint format and token streams)


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def attn_mixer(heads, kv_heads, dim, vdim, scale, softcap=None, rot=None, mask=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def attn(*a, **k):
    return {"type": "attention", "mixer": attn_mixer(*a, **k)}


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel(left, right):
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(vocab, width, layers, eps=1e-6):
    return {"architecture": "Redodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def odd():
    """Sizes that are multiples of nothing convenient; every mixer, a layer without feed-forward, a borrowed cache two layers back,
    fewer query / key heads than value heads in the delta rule, key size unlike value size, one and several groups."""
    return config(61, 56, [
        layer(attn(6, 2, 14, 10, 0.3, softcap=4.0, rot=(6, 777.0)), dense(40)),
        layer(delta(6, 3, 10, 7, 3), None),
        layer(parallel(attn_mixer(4, 1, 6, 9, 0.4, softcap=3.0, mask=(9, 2)), ssm(3, 5, 7, 1, 2, 3)), dense(24)),
        layer(attn(6, 2, 14, 10, 0.3, softcap=4.0, rot=(6, 777.0), kv_from=0), dense(32)),
        layer(delta(2, 2, 5, 33, 1), dense(16)),
        layer(parallel(attn_mixer(3, 3, 8, 8, 0.35, mask=(300, 0)), ssm(4, 9, 12, 4, 4, 1)), None),
        layer(attn(6, 2, 14, 10, 0.3, softcap=4.0, rot=(6, 777.0), kv_from=0), None),
    ], eps=1e-2)      # large enough to change every RMS norm visibly: a norm that ignores the configured value fails


def unaligned():
    """Width not a multiple of 8 (no tensor-core product takes it); the whole head rotates; a window of one position."""
    return config(31, 36, [
        layer(parallel(attn_mixer(2, 2, 10, 6, 0.4, softcap=2.5, mask=(1, 3)), ssm(2, 40, 3, 2, 1, 2)), dense(20)),
        layer(attn(2, 1, 4, 6, 0.5, rot=(4, 50.0)), dense(12)),
        layer(delta(1, 1, 34, 3, 4), dense(28)),
    ])


def aligned():
    """Sizes the tensor-core products take (multiples of 64)."""
    return config(320, 128, [
        layer(delta(4, 2, 32, 64, 4), dense(256)),
        layer(attn(4, 4, 64, 32, 0.125, softcap=20.0, rot=(32, 10000.0)), dense(192)),
        layer(parallel(attn_mixer(2, 1, 64, 64, 0.125, softcap=15.0, mask=(40, 4)), ssm(8, 16, 64, 2, 3, 4)), dense(128)),
        layer(attn(4, 4, 64, 32, 0.125, softcap=20.0, rot=(32, 10000.0), kv_from=1), dense(64)),
    ], eps=1e-5)


def _attn_weights(W, p, m, width, rnd, kind, peaky):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    W[p + "q"] = rnd(H * d, width, s=width ** -0.5) * (peaky if peaky else 1.0)
    W[p + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
    if m.get("kv_from") is None:
        W[p + "k"] = rnd(G * d, width, s=width ** -0.5)
        W[p + "v"] = rnd(G * dv, width, s=width ** -0.5)
    if kind == "attention":
        W[p + "sink"] = rnd(H)
        W[p + "g"] = rnd(H, width, s=2.0 * width ** -0.5)
    else:
        for n in [k for k in ("q", "k", "v", "o") if p + k in W]:
            W[p + n + ".b"] = rnd(W[p + n].shape[0], s=0.3)
        W[p + "r1"] = rnd(H, s=0.3).abs() + 0.1
        W[p + "r2"] = rnd(H, s=0.5).abs() + 0.05


def weights(cfg, seed=0, peaky=0.0, sink=None):
    """Random weights rounded to bf16 (so that bf16 and f32 runs hold the same numbers).  peaky > 0 multiplies the query
    projections of the softmax attentions: rows collapse onto single keys, so a key that is one position off, a window edge or a
    kept position changes the output visibly.  sink: a value for every head's sink (None: random)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return (s * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(torch.float32)

    def norm(W, name, width):
        W[name] = 1.0 + rnd(width, s=0.2)
        W[name + ".b"] = rnd(width, s=0.1)
        W[name + ".alpha"] = (0.5 + 0.4 * torch.rand((), generator=g)).to(torch.bfloat16).to(torch.float32)

    W, width = {}, cfg["width"]
    W["embed"] = rnd(cfg["vocab"], width)
    W["head"] = rnd(cfg["vocab"], width, s=width ** -0.5)
    norm(W, "final.norm", width)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(W, p + "norm1", width)
        norm(W, p + "norm1b", width)
        q = p + "mix."
        if L["type"] == "delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[q + n] = rnd(rows, width, s=2.0 * width ** -0.5)
                W[q + n + ".conv"] = rnd(rows, taps, s=0.6)
            W[q + "b"] = rnd(H, width, s=2.0 * width ** -0.5)
            W[q + "a"] = rnd(H, width, s=2.0 * width ** -0.5)
            W[q + "A_log"] = torch.log(0.3 + 2.0 * torch.rand(H, generator=g)).to(torch.bfloat16).float()
            W[q + "dt_bias"] = rnd(H) - 2.0
            W[q + "norm"] = 1.0 + rnd(dv, s=0.2)
            W[q + "g"] = rnd(H * dv, width, s=2.0 * width ** -0.5)
            W[q + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
        elif L["type"] == "attention":
            _attn_weights(W, q, m, width, rnd, "attention", peaky)
            if sink is not None:
                W[q + "sink"] = torch.full((m["heads"],), float(sink))
        else:
            _attn_weights(W, q + "left.", m["left"], width, rnd, "left", peaky)
            r = m["right"]
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            W[q + "right.in"] = rnd(2 * inner + 2 * gn + r["heads"], width, s=2.0 * width ** -0.5)
            W[q + "right.conv"] = rnd(inner + 2 * gn, r["conv"], s=0.6)
            W[q + "right.conv.b"] = rnd(inner + 2 * gn, s=0.3)
            W[q + "right.dt_bias"] = rnd(r["heads"]) - 1.0
            W[q + "right.A_log"] = torch.log(0.3 + 2.0 * torch.rand(r["heads"], generator=g)).to(torch.bfloat16).float()
            W[q + "right.D"] = rnd(r["heads"])
            W[q + "right.norm"] = 1.0 + rnd(inner, s=0.2)
            W[q + "right.o"] = rnd(width, inner, s=inner ** -0.5)
            W[q + "left.out"] = 1.0 + rnd(width, s=0.2)
            W[q + "right.out"] = 1.0 + rnd(width, s=0.2)
        if L.get("mlp") is not None:
            ff = L["mlp"]["ff"]
            norm(W, p + "norm2", width)
            norm(W, p + "norm2b", width)
            W[p + "mlp.up"] = rnd(ff, width, s=2.0 * width ** -0.5)
            W[p + "mlp.down"] = rnd(width, ff, s=ff ** -0.5)
            W[p + "mlp.act"] = (torch.tensor([0.4, -0.3]) + rnd(2, s=0.2))
        dw = rnd(i + 2, s=0.15)
        dw[-1] += 0.9
        W[p + "dwa"] = dw
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}      # what a bf16 checkpoint holds
