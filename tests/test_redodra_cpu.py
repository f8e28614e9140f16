"""Host-side parts of the Redodra sequence model (no GPU): configuration reader, tensor inventory, state declaration, and the
float64 oracle's own consistency (oracle/redodra_oracle.py)."""
import json
import math

import pytest
import torch

import redodra_cases as cases
from oracle import redodra_oracle as ro
from qwen3_tts_cuda_graphs_b200.config import (DeltaRuleConfig, DenseFFConfig, ParallelMixerConfig, SEQUENCE_ARCHITECTURES,
                                               SoftmaxAttentionConfig, StateSpaceConfig, sequence_config_from_dict)

F64 = torch.float64


def test_config_reader_takes_every_size_and_constant_from_the_dictionary():
    c = sequence_config_from_dict(json.loads(json.dumps(cases.odd())))
    assert (c.vocab, c.width, c.norm_eps, len(c.layers)) == (61, 56, 1e-2, 7)
    a = c.layers[0].mixer
    assert a == SoftmaxAttentionConfig(6, 2, 14, 10, 0.3, 4.0, 6, 777.0, 0, 0, sink=True, gate=True)
    assert c.layers[1].mixer == DeltaRuleConfig(6, 3, 10, 7, 3) and c.layers[1].mlp is None
    p = c.layers[2].mixer
    assert isinstance(p, ParallelMixerConfig) and p.right == StateSpaceConfig(3, 5, 7, 1, 2, 3) and p.right.inner == 15
    assert (p.left.window, p.left.keep_first, p.left.bias, p.left.distance, p.left.sink, p.left.gate) == (9, 2, True, True, False, False)
    assert c.layers[3].mixer.kv_from == 0 and c.layers[6].mixer.kv_from == 0 and c.layers[0].mlp == DenseFFConfig(40)
    assert c.layers[5].mixer.left.softcap == 0.0          # no cap configured
    assert "Redodra" in SEQUENCE_ARCHITECTURES
    bad = cases.odd()
    bad["layers"][3]["mixer"]["kv_from"] = 1               # not an attention layer
    with pytest.raises(ValueError):
        sequence_config_from_dict(bad)
    bad = cases.odd()
    bad["layers"][6]["mixer"]["kv_from"] = 3               # that layer borrows its cache itself
    with pytest.raises(ValueError):
        sequence_config_from_dict(bad)


def test_model_declares_the_tensors_the_test_checkpoint_holds():
    from qwen3_tts_cuda_graphs_b200.redodra import init_synthetic, tensor_specs

    for make in (cases.odd, cases.unaligned, cases.aligned):
        cfg = make()
        W = cases.weights(cfg)
        specs = tensor_specs(sequence_config_from_dict(cfg))
        assert set(W) == set(specs)
        assert all(tuple(W[k].shape) == tuple(specs[k]) for k in W)
        S = init_synthetic(sequence_config_from_dict(cfg))
        assert set(S) == set(specs) and all(tuple(S[k].shape) == tuple(specs[k]) for k in S)


def test_state_declaration_follows_the_layers():
    from qwen3_tts_cuda_graphs_b200.redodra import RedodraModel

    cfg = cases.odd()
    m = RedodraModel(sequence_config_from_dict(cfg), cases.weights(cfg).get, "cpu", f32=True)
    specs = {s.name: s for s in m.state_specs()}
    assert {"l0.k", "l0.v", "l2.k", "l2.v", "l5.k", "l5.v"} == {n for n, s in specs.items() if s.kind == "append"}
    assert (specs["l0.k"].cols, specs["l0.v"].cols, specs["l2.k"].cols, specs["l2.v"].cols) == (28, 20, 6, 9)
    assert (specs["l1.dr.conv"].rows, specs["l1.dr.conv"].cols) == (2, 2 * 3 * 10 + 6 * 7)
    assert (specs["l1.dr.s"].rows, specs["l1.dr.s"].cols) == (6 * 10, 7)
    assert "l4.dr.conv" not in specs                        # one tap: nothing to carry
    assert (specs["l2.ss.conv"].rows, specs["l2.ss.conv"].cols) == (1, 15 + 2 * 7)
    assert (specs["l5.ss.s"].rows, specs["l5.ss.s"].cols) == (4 * 12, 9)


def test_oracle_elementwise_pieces():
    z = torch.tensor([-3.0, -1e-9, 0.0, 1e-9, 2.0], dtype=F64)
    p, q = torch.tensor(0.3, dtype=F64), torch.tensor(-0.7, dtype=F64)
    y = ro.xielu(z, p, q)
    sp = lambda v: math.log1p(math.exp(v))
    assert abs(float(y[4]) - (sp(0.3) * 4 + 1)) < 1e-12
    assert abs(float(y[0]) - ((0.5 + sp(-0.7)) * (math.exp(-3) - 1 + 3) - 1.5)) < 1e-12
    assert abs(float(y[1]) - float(y[3])) < 1e-8 and float(y[2]) == 0.0          # continuous through zero
    v = torch.randn(3, 2, 8, dtype=F64)
    r = ro.rotate_interleaved(v, 4, 100.0)
    assert torch.equal(r[..., 4:], v[..., 4:]) and torch.allclose(r[0], v[0])        # rest untouched; position 0 is the identity
    assert torch.allclose(r[..., :4].pow(2).sum(-1), v[..., :4].pow(2).sum(-1))      # a rotation
    a = 2 * 100.0 ** (-2 * 1 / 4)
    assert torch.allclose(r[2, 1, 2], v[2, 1, 2] * math.cos(a) - v[2, 1, 3] * math.sin(a))
    n = ro.dyt_norm(torch.tensor([[0.5, -2.0]], dtype=F64), {"n": torch.tensor([2.0, 3.0], dtype=F64), "n.b": torch.tensor([0.1, 0.2], dtype=F64),
                                                            "n.alpha": torch.tensor(0.5, dtype=F64)}, "n")
    assert torch.allclose(n, torch.tensor([[2 * math.tanh(0.25) + 0.1, 3 * math.tanh(-1.0) + 0.2]], dtype=F64))


def test_oracle_attention_mask_sink_and_sharing():
    torch.manual_seed(0)
    T, H, G, d, dv = 12, 4, 2, 6, 5
    q, k, v = torch.randn(T, H, d, dtype=F64), torch.randn(T, G, d, dtype=F64), torch.randn(T, G, dv, dtype=F64)
    base = ro.masked_attention(q, k, v, 0.4, 3.0, window=4, keep_first=2)
    v2 = v.clone()
    v2[5] += 1.0                    # position 5 is outside query 9's window (6..9) and not among the first two
    out = ro.masked_attention(q, k, v2, 0.4, 3.0, window=4, keep_first=2)
    assert torch.equal(out[9:], base[9:]) and not torch.allclose(out[8], base[8]) and torch.equal(out[:5], base[:5])
    v3 = v.clone()
    v3[1] += 1.0                    # a kept first position: every later query sees it
    assert not torch.allclose(ro.masked_attention(q, k, v3, 0.4, 3.0, window=4, keep_first=2)[11], base[11])
    # a sink only grows the denominator: outputs shrink by the same factor in every column
    plain = ro.masked_attention(q, k, v, 0.4, None)
    sunk = ro.masked_attention(q, k, v, 0.4, None, sink=torch.full((H,), 1.5, dtype=F64))
    ratio = sunk / plain
    assert torch.allclose(ratio, ratio[..., :1].expand_as(ratio)) and float(ratio.max()) < 1.0
    # a distance penalty with r1 = 0 changes nothing; with r1 > 0 the current position gains weight
    z, one = torch.zeros(H, dtype=F64), torch.ones(H, dtype=F64)
    assert torch.allclose(ro.masked_attention(q, k, v, 0.4, None, r1=z, r2=one), plain)


def test_oracle_is_causal_and_recurrences_start_from_zero():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=3)
    toks = cases.tokens(cfg, 20)
    a = ro.forward(cfg, W, toks)
    other = list(toks)
    other[15] = (other[15] + 1) % cfg["vocab"]
    b = ro.forward(cfg, W, other)
    assert torch.equal(a[:15], b[:15]) and not torch.allclose(a[15:], b[15:])
    assert torch.allclose(ro.forward(cfg, W, toks[:7]), a[:7], atol=1e-12)


def test_command_lines_accept_the_model():
    from qwen3_tts_cuda_graphs_b200.cli import build_parser

    a = build_parser().parse_args(["lm", "--model", "m", "--tokens", "1 2 3", "--greedy", "--prefill-chunk", "7"])
    assert a.fn.__name__ == "cmd_lm" and a.prefill_chunk == 7


def test_peaky_weights_put_the_mass_on_single_keys_far_back():
    """The premise of the GPU test of far keys: with the query projections scaled up, a full-attention row concentrates on
    single keys, many of them far back, and the windowed rows reach their window's far edge and the kept first positions."""
    cfg = cases.config(64, 64, [
        cases.layer(cases.attn(4, 2, 16, 16, 0.25, softcap=25.0, rot=(8, 2000.0)), cases.dense(64)),
        cases.layer(cases.parallel(cases.attn_mixer(4, 2, 16, 8, 0.25, softcap=25.0, mask=(37, 3)), cases.ssm(4, 8, 16, 2, 3, 2)), cases.dense(32)),
    ])
    W = {k: v.to(F64) for k, v in cases.weights(cfg, seed=9, peaky=20.0, sink=8.0).items()}
    T = 300
    toks = cases.tokens(cfg, T)
    h = ro.dyt_norm(W["embed"][torch.tensor(toks)], W, "l0.norm1")
    q = ro.rotate_interleaved((h @ W["l0.mix.q"].T).reshape(T, 4, 16), 8, 2000.0)
    k = ro.rotate_interleaved((h @ W["l0.mix.k"].T).reshape(T, 2, 16), 8, 2000.0)
    top, dist = [], []
    for i in range(200, T):
        for hd in range(4):
            s = (k[: i + 1, hd // 2] @ q[i, hd]) * 0.25
            s = 25.0 * torch.tanh(s / 25.0)
            p = torch.softmax(s, 0)                      # among the keys (the sink only scales the row)
            top.append(float(p.max()))
            dist.append(i - int(p.argmax()))
    assert sum(top) / len(top) > 0.3 and max(dist) > 150 and sum(d > 50 for d in dist) > len(dist) // 4
    # windowed layer: rows whose heaviest key is the window's last visible position or a kept one do occur
    taps = []
    ro.forward(cfg, {k_: v for k_, v in W.items()}, toks, taps)
    h1 = ro.dyt_norm(taps[0], W, "l1.norm1")
    p_ = "l1.mix.left."
    q1 = (h1 @ W[p_ + "q"].T + W[p_ + "q.b"]).reshape(T, 4, 16)
    k1 = (h1 @ W[p_ + "k"].T + W[p_ + "k.b"]).reshape(T, 2, 16)
    edge = kept = 0
    for i in range(60, T):
        for hd in range(4):
            js = torch.tensor([j for j in range(i + 1) if i - j < 37 or j < 3])
            s = 25.0 * torch.tanh((k1[js, hd // 2] @ q1[i, hd]) * 0.25 / 25.0) - W[p_ + "r1"][hd] * torch.log1p(W[p_ + "r2"][hd] * (i - js).to(F64))
            j = int(js[int(s.argmax())])
            edge += int(i - j >= 33)
            kept += int(j < 3)
    assert edge > 10 and kept > 10
