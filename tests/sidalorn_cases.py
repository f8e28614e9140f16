"""Small Sidalorn configurations and random weights for the tests (raw config dictionaries, checkpoint tensor names)."""
import torch


def attn(heads, dim, vdim, rank, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}}


def lru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, count, keep, scale, ff, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None,
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


def config(vocab, width, groups, taps, layers, eps=1e-6):
    out = {"architecture": "Sidalorn", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if taps:
        out["canon"] = {"taps": taps}
    return out


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def odd():
    """Sizes that are multiples of nothing convenient; every mechanism and every optional part in both states."""
    return config(53, 72, 3, 2, [
        layer(lru(48, 3, 2), dense(40)),
        layer(attn(3, 24, 40, 20, 0.3), moe(6, 2, 3, 4, 2, 1.7, 24, 24)),
        layer(attn(2, 8, 8, 12, 0.5), None),
        layer(lru(40, 1, 1), moe(4, 0, 1, 1, 1, 1.0, 16, 0)),
        layer(attn(5, 16, 8, 36, 0.25), moe(5, 3, 2, 2, 1, 2.5, 32, 40)),
    ], eps=1e-2)      # large enough to change every norm visibly: a norm that ignores the configured value fails


def unaligned():
    """Width not a multiple of 8 (no tensor-core path takes it), no input convolution, one norm group."""
    return config(31, 36, 1, 0, [
        layer(attn(2, 10, 6, 14, 0.4), dense(20)),
        layer(lru(30, 2, 3), moe(3, 1, 2, 1, 1, 1.0, 12, 10)),
    ])


def aligned():
    """Sizes the tensor-core products take (multiples of 64)."""
    return config(320, 128, 2, 4, [
        layer(lru(128, 4, 4), dense(256)),
        layer(attn(4, 32, 32, 64, 0.18), moe(8, 2, 2, 2, 1, 2.0, 64, 128)),
        layer(attn(4, 32, 32, 64, 0.18), dense(192)),
    ])


def mid():
    """Sizes at which every product takes its real-size kernel (128-row tensor-core tiles, the attention's 16-head blocks with
    a second, part-filled block, two accumulator widths, grouped expert tiles), still quick for the float64 oracle."""
    return config(1000, 256, 4, 3, [
        layer(attn(20, 32, 48, 144, 0.2), moe(12, 4, 3, 4, 2, 2.0, 128, 256)),
        layer(lru(384, 6, 4), dense(512)),
        layer(attn(4, 64, 32, 256, 0.15), moe(8, 0, 2, 1, 1, 1.0, 192, 0)),
        layer(lru(128, 2, 2), None),
    ], eps=1e-5)


def weights(cfg, seed=0, peaky=0.0, sink=None, optional=True):
    """Random weights rounded to bf16 (so that bf16 and f32 runs hold the same numbers).  peaky > 0 multiplies the query
    projections: softmax rows collapse onto single keys, so a key that is one position off changes the output visibly.
    sink: a value for every head's sink (None: random).  optional=False leaves every optional tensor out."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return (s * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(torch.float32)

    W, width = {}, cfg["width"]
    W["embed"] = rnd(cfg["vocab"], width)
    W["head"] = rnd(cfg["vocab"], width, s=width ** -0.5)
    W["final.norm"] = 1.0 + rnd(width, s=0.2)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = 1.0 + rnd(width, s=0.2)
        if taps:
            W[p + "canon1"] = rnd(width, taps, s=0.4)
        if L["type"] == "latent_attention":
            H, dk, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            W[p + "mix.q"] = rnd(H * dk, width, s=width ** -0.5) * (peaky if peaky else 1.0)
            W[p + "mix.dkv"] = rnd(R, width, s=width ** -0.5)
            W[p + "mix.dkv.norm"] = 1.0 + rnd(R, s=0.2)
            W[p + "mix.uk"] = rnd(H * dk, R, s=R ** -0.5)
            W[p + "mix.uv"] = rnd(H * dv, R, s=R ** -0.5)
            W[p + "mix.o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
            if optional:
                W[p + "mix.sink"] = rnd(H) if sink is None else torch.full((H,), float(sink))
        else:
            Wd, B = m["width"], m["blocks"]
            bs = Wd // B
            W[p + "mix.y"] = rnd(Wd, width, s=width ** -0.5)
            W[p + "mix.x"] = rnd(Wd, width, s=width ** -0.5)
            W[p + "mix.conv"] = rnd(Wd, m["conv"], s=0.5)
            W[p + "mix.ra"] = rnd(B, bs, bs, s=bs ** -0.5)
            W[p + "mix.ri"] = rnd(B, bs, bs, s=bs ** -0.5)
            W[p + "mix.lam"] = rnd(Wd, s=1.0) - 2.0
            W[p + "mix.o"] = rnd(width, Wd, s=Wd ** -0.5)
            if optional:
                for n, shape in (("y.b", (Wd,)), ("x.b", (Wd,)), ("conv.b", (Wd,)), ("ra.b", (B, bs)), ("ri.b", (B, bs))):
                    W[p + "mix." + n] = rnd(*shape, s=0.3)
        f = L.get("mlp")
        if f is None:
            continue
        W[p + "norm2"] = 1.0 + rnd(width, s=0.2)
        if f["kind"] == "dense":
            W[p + "mlp.up"] = rnd(f["ff"], width, s=width ** -0.5)
            W[p + "mlp.down"] = rnd(width, f["ff"], s=f["ff"] ** -0.5)
            W[p + "mlp.act"] = torch.tensor([0.7, 0.25, 0.1, 0.05]) + rnd(4, s=0.05)
        else:
            r, ff = f["router"], f["expert"]["ff"]
            n = r["experts"] + r["identity"]
            W[p + "mlp.router"] = rnd(n, width, s=2.0 * width ** -0.5)
            if optional:
                W[p + "mlp.correction"] = rnd(n, s=0.3) - 0.4          # choice scores go negative
            for e in range(r["experts"]):
                W[p + f"mlp.e{e}.up"] = rnd(ff, width, s=width ** -0.5)
                W[p + f"mlp.e{e}.down"] = rnd(width, ff, s=ff ** -0.5)
            if f.get("shared"):
                W[p + "mlp.shared.up"] = rnd(f["shared"]["ff"], width, s=width ** -0.5)
                W[p + "mlp.shared.down"] = rnd(width, f["shared"]["ff"], s=f["shared"]["ff"] ** -0.5)
    return W


def tokens(cfg, n, seed=0):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def save_checkpoint(folder, cfg, W):
    """config.json and model.safetensors (bf16) in `folder`: 8-byte little-endian header length, JSON header, tensor bytes."""
    import json
    import os
    import struct

    header, blobs, at = {}, [], 0
    for name, t in W.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
