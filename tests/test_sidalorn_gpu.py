"""The Sidalorn sequence model on the CUDA op-list path against the float64 oracle (oracle/sidalorn_oracle.py).

Mechanisms alone (seq_ops.StepBuilder fragments), then whole models: prompts, prompts in portions down to two tokens, token by
token decoding through the carried state, slots that are given back and used again, requests that take turns, keys far back and
at the borders of the attention kernel's key tiles and splits, sinks, long decoding, sizes that are multiples of nothing, and
greedy generation through the engine's entry point and the scheduler.
"""
import math

import pytest
import torch

import sidalorn_cases as cases
from oracle import sidalorn_oracle as so

pytestmark = pytest.mark.gpu

F64 = torch.float64


def make_engine(cfg, W, f32=True, max_tokens=700, max_slots=2):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict
    from qwen3_tts_cuda_graphs_b200.seq_engine import SequenceEngine, model_class

    model = model_class(cfg["architecture"])(sequence_config_from_dict(cfg), W.get, "cuda", f32=f32)
    return SequenceEngine(model, max_tokens, max_slots)


def row_errors(got, want):
    """Per position: RMS over the vocabulary of the mean-free difference, relative to the RMS of the wanted logits."""
    got, want = got.to(F64).cpu(), want.to(F64)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def rel_err(got, want):
    return float(row_errors(got, want).max())


TOL = {True: 3e-4, False: 6e-2}      # true 32-bit / bf16 products


def close_enough(got, want, f32):
    """True 32-bit: every position within the tolerance.  bf16 products: rounding noise can flip a router's close call or a
    peaked softmax's near-tie at a few positions of these tiny random models, so nine positions in ten must be within the
    tolerance and the typical one well within it; a wrong key, state or sink moves all of them."""
    e = row_errors(got, want)
    if f32:
        return float(e.max()) < TOL[True]
    return float(e.quantile(0.9)) < TOL[False] and float(e.median()) < TOL[False] / 2


def run_schedule(eng, toks, portions, name="r"):
    """Feed toks in the given portions (the rest one by one); logits of every position, [T, vocab]."""
    rows, at = [], 0
    sizes = list(portions) + [1] * (len(toks) - sum(portions))
    for n in sizes:
        part = toks[at:at + n]
        rows.append(eng.step(name, part, list(range(len(part)))).clone())
        at += n
    eng.close(name)
    return torch.cat(rows, 0)


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
class Bench:
    """A StepBuilder around hand-made state: runs one mechanism for a sequence of portions."""

    def __init__(self, specs, f32=True, max_pos=700):
        from qwen3_tts_cuda_graphs_b200 import codec
        from qwen3_tts_cuda_graphs_b200.seq_state import SequenceStateManager

        self.codec, self.f32 = codec, f32
        self.lib = codec.load_lib()
        self.mgr = SequenceStateManager(specs, max_pos, torch.device("cuda"), 1)
        self.slot = self.mgr.acquire("t")

    def run(self, M, build):
        from qwen3_tts_cuda_graphs_b200.seq_ops import StepBuilder

        b = StepBuilder(torch.device("cuda"), M, self.slot, self.f32)
        out = build(b)
        b.commit()
        self.codec.run_op_plan(self.lib, b.finish(), False)
        torch.cuda.synchronize()
        return out


def cuda(t, dtype=torch.float32):
    return t.to("cuda", dtype).contiguous()


@pytest.mark.parametrize("n,groups", [(60, 3), (64, 1), (14, 7)])
def test_group_norm_alone(n, groups):
    torch.manual_seed(0)
    x, w, res = torch.randn(5, n), torch.randn(n), torch.randn(5, n)
    bench = Bench([])
    out = torch.zeros(5, n, device="cuda")
    copy = torch.zeros(5, n, device="cuda", dtype=torch.bfloat16)
    bench.run(5, lambda b: b.group_norm(cuda(x), cuda(w), groups, 1e-5, out, residual=cuda(res), out_bf16=copy))
    want = res.to(F64) + so.grouped_rms_norm(x.to(F64), w.to(F64), groups, 1e-5)
    assert torch.allclose(out.cpu().to(F64), want, atol=1e-5, rtol=1e-5)
    assert torch.equal(copy.cpu(), out.cpu().to(torch.bfloat16))


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_time_conv_carries_its_inputs_across_portions(taps):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    torch.manual_seed(1)
    C, T = 19, 17
    x, w, bias = torch.randn(T, C), torch.randn(C, taps), torch.randn(C)
    bench = Bench([StateSpec("c", "carry", C, taps - 1)])
    rows, at = [], 0
    for n in (1, 1, 2, 5, 1, 3, 4):          # portions shorter than the history included
        part = cuda(x[at:at + n])
        out = torch.zeros(n, C, device="cuda")
        bench.run(n, lambda b: b.time_conv(part, cuda(w), "c", out, bias=cuda(bias), add_input=True))
        rows.append(out.cpu())
        at += n
    want = x.to(F64) + so.causal_time_conv(x.to(F64), w.to(F64), bias.to(F64))
    assert torch.allclose(torch.cat(rows).to(F64), want, atol=1e-5, rtol=1e-5)


def _attn_weights(H, dk, dv, R, width, sink, seed=2, peaky=1.0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, k=1.0: (k * torch.randn(*s, generator=g)).to(torch.bfloat16).float()
    W = {"q": r(H * dk, width, k=peaky * width ** -0.5), "dkv": r(R, width, k=width ** -0.5), "dkv.norm": 1 + r(R, k=0.2),
         "uk": r(H * dk, R, k=R ** -0.5), "uv": r(H * dv, R, k=R ** -0.5), "o": r(width, H * dv, k=(H * dv) ** -0.5)}
    if sink is not None:
        W["sink"] = torch.full((H,), float(sink)) if not isinstance(sink, str) else r(H)
    return W


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("sink", [None, "random", 6.0])
def test_latent_attention_alone(sink, f32):
    from qwen3_tts_cuda_graphs_b200.config import LatentAttentionConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, dk, dv, R, width, T = 3, 24, 40, 20, 48, 75
    W = _attn_weights(H, dk, dv, R, width, sink, peaky=4.0)
    m = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": R, "scale": 0.3}
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).float()
    want = so.latent_attention(h.to(F64), {"m." + k: v.to(F64) for k, v in W.items()}, "m.", m, 1e-6)
    wdt = torch.float32 if f32 else torch.bfloat16
    pw = {"wqd": cuda(torch.cat([W["q"], W["dkv"]]), wdt), "dkv_norm": cuda(W["dkv.norm"]),
          "uk_t": cuda(W["uk"].reshape(H, dk, R).transpose(1, 2), wdt), "uv": cuda(W["uv"].reshape(H, dv, R), wdt),
          "sink": cuda(W["sink"]) if "sink" in W else None, "o": cuda(W["o"], wdt)}
    bench = Bench([StateSpec("lat", "append", R, dtype=wdt)], f32=f32)
    rows, at = [], 0
    for n in (30, 1, 1, 2, 3, 33, 1, 4):     # crosses the 32-key tile of the kernel inside a portion and while decoding
        part = cuda(h[at:at + n], wdt)
        out = torch.zeros(n, width, device="cuda")
        bench.run(n, lambda b: b.latent_attention(part, LatentAttentionConfig(H, dk, dv, R, 0.3), pw, "lat", 1e-6, out))
        rows.append(out.cpu())
        at += n
    got = torch.cat(rows).to(F64)
    err = float((got - want).abs().max() / want.abs().max())
    assert err < (2e-5 if f32 else 3e-2), err
    if sink == 6.0:   # a sink this large takes much of the mass: leaving it out moves the output far beyond the tolerance
        no_sink = so.latent_attention(h.to(F64), {"m." + k: v.to(F64) for k, v in W.items() if k != "sink"}, "m.", m, 1e-6)
        assert float((no_sink - want).abs().max() / want.abs().max()) > 0.3


@pytest.mark.parametrize("H,R", [(3, 48), (18, 80), (5, 128), (2, 256), (17, 336)])
def test_latent_attention_tensor_core_tiles(H, R):
    """bf16 cache with a rank the MMA tiles divide: every accumulator width of the tensor-core kernel, one and two column slices
    per query, an odd tile count per slice, head counts on both sides of a 16-head block; portions that cross its 64- and 32-key
    tiles, its 4-query blocks and its key-range splits, and single decoded tokens.  Peaky queries: one key off shows."""
    from qwen3_tts_cuda_graphs_b200.config import LatentAttentionConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    dk, dv, width, T = 16, 8, 64, 209
    W = _attn_weights(H, dk, dv, R, width, "random", seed=5, peaky=4.0)
    m = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": R, "scale": 0.3}
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).float()
    want = so.latent_attention(h.to(F64), {"m." + k: v.to(F64) for k, v in W.items()}, "m.", m, 1e-6)
    wdt = torch.bfloat16
    pw = {"wqd": cuda(torch.cat([W["q"], W["dkv"]]), wdt), "dkv_norm": cuda(W["dkv.norm"]),
          "uk_t": cuda(W["uk"].reshape(H, dk, R).transpose(1, 2), wdt), "uv": cuda(W["uv"].reshape(H, dv, R), wdt),
          "sink": cuda(W["sink"]), "o": cuda(W["o"], wdt)}
    bench = Bench([StateSpec("lat", "append", R, dtype=wdt)], f32=False)
    rows, at = [], 0
    for n in (70, 1, 1, 2, 5, 50, 1, 3, 67, 9):
        part = cuda(h[at:at + n], wdt)
        out = torch.zeros(n, width, device="cuda")
        bench.run(n, lambda b: b.latent_attention(part, LatentAttentionConfig(H, dk, dv, R, 0.3), pw, "lat", 1e-6, out))
        rows.append(out.cpu())
        at += n
    assert at == T
    got = torch.cat(rows).to(F64)
    err = (got - want).abs().amax(-1) / want.abs().max()
    assert float(err.max()) < 3e-2, (float(err.max()), int(err.argmax()))


@pytest.mark.parametrize("blocks,conv,T", [(3, 4, 40), (1, 1, 9), (2, 2, 600)])
def test_rglru_alone(blocks, conv, T):
    from qwen3_tts_cuda_graphs_b200.config import RglruConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    Wd, width = 48, 40
    bs = Wd // blocks
    g = torch.Generator().manual_seed(4)
    r = lambda *s, k=1.0: (k * torch.randn(*s, generator=g)).to(torch.bfloat16).float()
    W = {"y": r(Wd, width, k=width ** -0.5), "y.b": r(Wd, k=0.3), "x": r(Wd, width, k=width ** -0.5), "x.b": r(Wd, k=0.3),
         "conv": r(Wd, conv, k=0.5), "conv.b": r(Wd, k=0.3), "ra": r(blocks, bs, bs, k=bs ** -0.5), "ra.b": r(blocks, bs, k=0.3),
         "ri": r(blocks, bs, bs, k=bs ** -0.5), "ri.b": r(blocks, bs, k=0.3), "lam": r(Wd) - 3.0, "o": r(width, Wd, k=Wd ** -0.5)}
    h = torch.randn(T, width, generator=g).to(torch.bfloat16).float()
    want = so.rglru_block(h.to(F64), {"m." + k: v.to(F64) for k, v in W.items()}, "m.", {"width": Wd, "blocks": blocks, "conv": conv})
    pw = {"wyx": cuda(torch.cat([W["y"], W["x"]])), "byx": cuda(torch.cat([W["y.b"], W["x.b"]])), "conv": cuda(W["conv"]),
          "conv_b": cuda(W["conv.b"]), "gates": cuda(torch.cat([W["ra"], W["ri"]])),
          "gates_b": cuda(torch.cat([W["ra.b"].reshape(-1), W["ri.b"].reshape(-1)])), "lam": cuda(W["lam"]), "o": cuda(W["o"])}
    bench = Bench([StateSpec("r.conv", "carry", Wd, conv - 1), StateSpec("r.s", "carry", Wd, 1)])
    rows, at = [], 0
    sizes = [3, 1, 1, 2] + ([T - 7 - 2, 1, 1] if T > 9 else [1, 1])     # a long portion takes the piecewise scan
    for n in sizes:
        part = cuda(h[at:at + n])
        out = torch.zeros(n, width, device="cuda")
        bench.run(n, lambda b: b.rglru(part, RglruConfig(Wd, blocks, conv), pw, "r", out))
        rows.append(out.cpu())
        at += n
    assert at == T
    got = torch.cat(rows).to(F64)
    assert float((got - want).abs().max() / want.abs().max()) < 2e-5


def test_polynorm_ff_alone():
    g = torch.Generator().manual_seed(5)
    width, ff, T = 24, 52, 6
    W = {"up": torch.randn(ff, width, generator=g) * width ** -0.5, "down": torch.randn(width, ff, generator=g) * ff ** -0.5,
         "act": torch.tensor([0.6, -0.3, 0.2, 0.1])}
    h = torch.randn(T, width, generator=g)
    want = so.polynorm_ff(h.to(F64), {"m." + k: v.to(F64) for k, v in W.items()}, "m.", 1e-6)
    out = torch.zeros(T, width, device="cuda")
    Bench([]).run(T, lambda b: b.polynorm_ff(cuda(h), {k: cuda(v) for k, v in W.items()}, 1e-6, out))
    assert float((out.cpu().to(F64) - want).abs().max() / want.abs().max()) < 2e-5


@pytest.mark.parametrize("experts,identity,top,count,keep,shared", [(6, 2, 3, 4, 2, 24), (4, 0, 1, 1, 1, 0), (5, 3, 2, 2, 1, 8), (3, 1, 4, 1, 1, 0)])
def test_moe_ff_alone(experts, identity, top, count, keep, shared):
    from qwen3_tts_cuda_graphs_b200.config import MoEFFConfig

    g = torch.Generator().manual_seed(6)
    width, ff, T, n = 20, 12, 70, experts + identity
    W = {"router": torch.randn(n, width, generator=g), "correction": torch.randn(n, generator=g) * 0.3 - 0.5}
    for e in range(experts):
        W[f"e{e}.up"] = torch.randn(ff, width, generator=g) * width ** -0.5
        W[f"e{e}.down"] = torch.randn(width, ff, generator=g) * ff ** -0.5
    if shared:
        W["shared.up"] = torch.randn(shared, width, generator=g) * width ** -0.5
        W["shared.down"] = torch.randn(width, shared, generator=g) * shared ** -0.5
    h = torch.randn(T, width, generator=g)
    f = {"router": {"experts": experts, "identity": identity, "top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}},
         "shared": {"ff": shared} if shared else None}
    W64 = {"m." + k: v.to(F64) for k, v in W.items()}
    want = so.moe_ff(h.to(F64), W64, "m.", f)
    ids, _ = so.route(h.to(F64), W64, "m.", f["router"])
    assert identity == 0 or bool((ids >= experts).any())        # identity experts are really chosen in this case
    pw = {"router": cuda(W["router"]), "correction": cuda(W["correction"]),
          "up": cuda(torch.stack([W[f"e{e}.up"] for e in range(experts)])), "down": cuda(torch.stack([W[f"e{e}.down"] for e in range(experts)])),
          "shared_up": cuda(W["shared.up"]) if shared else None, "shared_down": cuda(W["shared.down"]) if shared else None}
    out = torch.zeros(T, width, device="cuda")
    bench = Bench([])
    x = cuda(h)
    bench.run(T, lambda b: b.moe_ff(x, x, MoEFFConfig(experts, identity, top, count, keep, 1.7, ff, shared), pw, out))
    assert float((out.cpu().to(F64) - want).abs().max() / want.abs().max()) < 2e-5


def test_moe_ff_many_tokens_per_expert_bf16():
    """Hundreds of rows per expert in bf16: the grouped products take their tall tensor-core tiles, with gathered rows, segments
    that end inside a tile, an expert nobody chooses (its correction is very negative) and identity choices that leave no row."""
    from qwen3_tts_cuda_graphs_b200.config import MoEFFConfig

    g = torch.Generator().manual_seed(12)
    experts, identity, top, width, ff, T = 4, 1, 2, 136, 152, 700
    n = experts + identity
    r = lambda *sh, k=1.0: (k * torch.randn(*sh, generator=g)).to(torch.bfloat16).float()
    W = {"router": r(n, width, k=width ** -0.5), "correction": torch.tensor([0.0, -50.0, 0.1, 0.0, 0.05])}
    for e in range(experts):
        W[f"e{e}.up"] = r(ff, width, k=width ** -0.5)
        W[f"e{e}.down"] = r(width, ff, k=ff ** -0.5)
    h = r(T, width)
    f = {"router": {"experts": experts, "identity": identity, "top": top, "scale": 1.3, "groups": {"count": 1, "keep": 1}}, "shared": None}
    W64 = {"m." + k: v.to(F64) for k, v in W.items()}
    want = so.moe_ff(h.to(F64), W64, "m.", f)
    ids, _ = so.route(h.to(F64), W64, "m.", f["router"])
    assert not bool((ids == 1).any()) and bool((ids == 4).any()) and int((ids == 0).sum()) > 128
    bf = torch.bfloat16
    pw = {"router": cuda(W["router"], bf), "correction": cuda(W["correction"]),
          "up": cuda(torch.stack([W[f"e{e}.up"] for e in range(experts)]), bf), "down": cuda(torch.stack([W[f"e{e}.down"] for e in range(experts)]), bf),
          "shared_up": None, "shared_down": None}
    out = torch.zeros(T, width, device="cuda")
    bench = Bench([], f32=False, max_pos=T)
    bench.run(T, lambda b: b.moe_ff(cuda(h), cuda(h, bf), MoEFFConfig(experts, identity, top, 1, 1, 1.3, ff, 0), pw, out))
    err = (out.cpu().to(F64) - want).abs().amax(-1) / want.abs().max()
    assert float(err.quantile(0.98)) < 2e-2 and float(err.median()) < 5e-3, (float(err.max()), float(err.median()))


# ---------------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------------
CASES = {"odd": cases.odd, "unaligned": cases.unaligned, "aligned": cases.aligned}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(CASES))
def test_prompt_portions_and_decoding_agree_with_the_oracle(case, f32):
    cfg = CASES[case]()
    W = cases.weights(cfg, seed=7)
    toks = cases.tokens(cfg, 90)
    want = so.forward(cfg, W, toks)
    eng = make_engine(cfg, W, f32)
    whole = run_schedule(eng, toks, [90])
    assert close_enough(whole, want, f32)
    # the slot of the request above is used again by each of these
    for portions in ([2, 3, 1, 5, 2, 37, 2, 33], [60], [1] * 20, [89]):
        got = run_schedule(eng, toks, portions)
        assert close_enough(got, want, f32), portions
        assert close_enough(got, whole.cpu(), f32), portions
    eng.close_all()


@pytest.mark.parametrize("f32", [True, False])
def test_real_size_kernel_paths_agree_with_the_oracle(f32):
    """A prompt long enough for full 128-row product tiles and several key tiles, in one step and in portions, then decoding."""
    cfg = cases.mid()
    W = cases.weights(cfg, seed=11)
    toks = cases.tokens(cfg, 300)
    want = so.forward(cfg, W, toks)
    eng = make_engine(cfg, W, f32)
    for portions in ([300], [130, 2, 140], [257, 9, 31]):
        assert close_enough(run_schedule(eng, toks, portions), want, f32), portions
    eng.close_all()


def test_optional_tensors_may_be_absent():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=8, optional=False)
    assert not any(k.endswith((".sink", ".correction", ".b")) for k in W)
    toks = cases.tokens(cfg, 40)
    eng = make_engine(cfg, W, True)
    assert rel_err(run_schedule(eng, toks, [17, 2]), so.forward(cfg, W, toks)) < TOL[True]


@pytest.mark.parametrize("f32", [True, False])
def test_far_keys_tile_borders_and_sinks(f32):
    """Peaky attention (queries scaled up) puts each row's mass on single keys, mostly far back; wanted positions sit on both sides
    of the kernel's 32-key tiles and of its key-range splits, in a prompt portion and decoded alone."""
    cfg = cases.config(64, 64, 2, 3, [cases.layer(cases.attn(4, 16, 16, 24, 0.25), cases.dense(64)),
                                      cases.layer(cases.attn(2, 32, 8, 40, 0.2), cases.moe(4, 1, 2, 1, 1, 1.5, 32, 16))])
    W = cases.weights(cfg, seed=9, peaky=6.0, sink=7.0)
    T = 530
    toks = cases.tokens(cfg, T)
    want = so.forward(cfg, W, toks)
    # the oracle's attention really is peaky and looks far back: check the premise on layer 0, head 0
    eng = make_engine(cfg, W, f32, max_tokens=T)
    got_a = run_schedule(eng, toks, [T])                       # every border inside one portion
    got_b = run_schedule(eng, toks, [31, 33, 190, 2, 255])     # portions end at 31, 64, 254, 256, 511; the rest decoded
    for got in (got_a, got_b):
        assert close_enough(got, want, f32)
    # a model whose sink is left out answers differently by more than the tolerance at most positions
    W2 = {k: v for k, v in W.items() if not k.endswith(".sink")}
    assert float(row_errors(so.forward(cfg, W2, toks[:64]), want[:64]).median()) > 2 * TOL[False]
    eng.close_all()


def test_peaky_premise_holds():
    """The crafted weights of the test above do what they are for: softmax rows concentrate on single keys far back."""
    cfg = cases.config(64, 64, 2, 3, [cases.layer(cases.attn(4, 16, 16, 24, 0.25), cases.dense(64))])
    W = {k: v.to(F64) for k, v in cases.weights(cfg, seed=9, peaky=6.0, sink=7.0).items()}
    toks = cases.tokens(cfg, 300)
    x = W["embed"][torch.tensor(toks)]
    h = x + so.causal_time_conv(x, W["l0.canon1"])
    q = (h @ W["l0.mix.q"].T).reshape(300, 4, 16)
    lat = so.rms_unit(h @ W["l0.mix.dkv"].T, 1e-6) * W["l0.mix.dkv.norm"]
    k = (lat @ W["l0.mix.uk"].T).reshape(300, 4, 16)
    s = torch.einsum("hd,jhd->hj", q[299], k) * 0.25
    p = torch.softmax(s, -1)
    assert float(p.max(-1).values.mean()) > 0.3            # mass on single keys
    assert int((299 - p.argmax(-1)).max()) > 50            # some of them far back


def test_requests_take_turns_in_two_slots_and_slots_are_reused():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=10)
    eng = make_engine(cfg, W, True, max_slots=2)
    reqs = {n: cases.tokens(cfg, L, seed=i) for i, (n, L) in enumerate([("a", 23), ("b", 9), ("c", 41), ("d", 2)])}
    want = {n: so.forward(cfg, W, t) for n, t in reqs.items()}
    got = {n: [] for n in reqs}
    at = {n: 0 for n in reqs}
    # a and b interleaved with unequal portions; when b ends, c takes its slot while a is still running; then d
    plan = [("a", 5), ("b", 2), ("a", 1), ("b", 7), ("c", 30), ("a", 10), ("c", 1), ("a", 7), ("d", 2), ("c", 10)]
    for n, k in plan:
        part = reqs[n][at[n]:at[n] + k]
        got[n].append(eng.step(n, part, list(range(k))).clone())
        at[n] += k
        if at[n] == len(reqs[n]):
            eng.close(n)
    assert len(eng.states.slots) == 2
    for n in reqs:
        assert rel_err(torch.cat(got[n]), want[n]) < TOL[True], n


def test_long_decoding():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=11)
    toks = cases.tokens(cfg, 340)
    want = so.forward(cfg, W, toks)
    for f32 in (True, False):
        eng = make_engine(cfg, W, f32)
        got = run_schedule(eng, toks, [3])          # 337 tokens one by one through the carried state
        assert close_enough(got, want, f32)
        eng.close_all()


def test_capacity_and_bad_input_are_refused():
    cfg = cases.unaligned()
    eng = make_engine(cfg, cases.weights(cfg), True, max_tokens=10, max_slots=1)
    eng.step("a", [1, 2, 3, 4, 5, 6], [])
    with pytest.raises(RuntimeError):
        eng.step("a", [1, 2, 3, 4, 5], [])
    with pytest.raises(RuntimeError):
        eng.open("b")                                # the only slot is taken
    with pytest.raises(ValueError):
        eng.step("a", [cfg["vocab"]], [])
    eng.close("a")
    eng.step("b", [1, 2], [1])


def _oracle_greedy(cfg, W, prompt, n):
    """Greedy continuation by the oracle, with the margin between the two best logits of every choice."""
    toks, margins = list(prompt), []
    for _ in range(n):
        lg = so.forward(cfg, W, toks)[-1]
        top = torch.topk(lg, 2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(lg.argmax()))
    return toks[len(prompt):], margins


def test_greedy_generation_through_engine_and_scheduler():
    from qwen3_tts_cuda_graphs_b200.serving import TokenRequest, TokenScheduler

    cfg = cases.odd()
    W = cases.weights(cfg, seed=12)
    prompts = [cases.tokens(cfg, L, seed=20 + i) for i, L in enumerate((12, 3, 27))]
    n_new = 10
    eng = make_engine(cfg, W, True, max_tokens=64, max_slots=2)
    want = []
    for p in prompts:
        ids, margins = _oracle_greedy(cfg, W, p, n_new)
        cut = next((i for i, m in enumerate(margins) if m < 1e-3), n_new)     # compare up to the first near-tie
        want.append(ids[:cut])
        assert cut >= 3
    for p, w in zip(prompts, want):
        assert eng.generate(p, n_new, prefill_chunk=5)[:len(w)] == w
    sched = TokenScheduler(eng, prefill_chunk=4)       # three requests, two slots: the third waits for a slot
    handles = [sched.submit(TokenRequest(p, n_new)) for p in prompts]
    sched.run()
    for h, w in zip(handles, want):
        assert h.done and h.reason == "length" and h.result()[:len(w)] == w
    # sampling goes through the framework's sampler: top-k 1 at any temperature is the greedy choice
    h = sched.submit(TokenRequest(prompts[0], 4, do_sample=True, temperature=0.7, top_k=1, seed=3))
    sched.run()
    assert h.result()[:min(4, len(want[0]))] == want[0][:4]
    eng.close_all()


def test_replayer_reads_a_checkpoint_from_disk_and_writes_the_wanted_logits(tmp_path):
    """bin/trace_run as a child process: config.json + model.safetensors on disk, steps on standard input (a portion with
    several wanted places, a two-token portion with none, single tokens, a finished request whose slot the next one takes),
    one file of little-endian f32 logits per step that wants some, "done <step>" after every step."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    cfg = cases.odd()
    W = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in cases.weights(cfg, seed=21).items()}   # what the file holds
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    cases.save_checkpoint(str(model_dir), cfg, W)
    a, b = cases.tokens(cfg, 14, seed=5), cases.tokens(cfg, 6, seed=6)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [0, 3, 8]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[9:11], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[11:12], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[12:14], "want": [1, 0]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                        "--out", str(out_dir), "--max-tokens", "16", "--max-slots", "1"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(5)]
    assert not (out_dir / "1.f32").exists()
    ref_a, ref_b = so.forward(cfg, W, a), so.forward(cfg, W, b)
    for step, ref, places in ((0, ref_a, [0, 3, 8]), (2, ref_a, [11]), (3, ref_a, [13, 12]), (4, ref_b, [5])):
        got = torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(places), cfg["vocab"]))
        assert rel_err(got, ref[places]) < TOL[True], step
