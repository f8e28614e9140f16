"""Host-side parts of the sequence models (no GPU): configuration reader, state slots, and the oracle's own consistency."""
import json
import math

import pytest
import torch

import sidalorn_cases as cases
from oracle import sidalorn_oracle as so
from qwen3_tts_cuda_graphs_b200.config import (DenseFFConfig, LatentAttentionConfig, MoEFFConfig, RglruConfig, SEQUENCE_ARCHITECTURES,
                                               sequence_config_from_dict)
from qwen3_tts_cuda_graphs_b200.seq_state import SequenceStateManager, StateSpec


def test_config_reader_takes_every_size_and_constant_from_the_dictionary():
    raw = json.loads(json.dumps(cases.odd()))       # through JSON, as a checkpoint's config.json
    c = sequence_config_from_dict(raw)
    assert (c.vocab, c.width, c.norm_groups, c.canon_taps, c.norm_eps) == (53, 72, 3, 2, 1e-2)
    assert [L.type for L in c.layers] == ["rglru", "latent_attention", "latent_attention", "rglru", "latent_attention"]
    assert c.layers[0].mixer == RglruConfig(48, 3, 2) and c.layers[0].mlp == DenseFFConfig(40)
    assert c.layers[1].mixer == LatentAttentionConfig(3, 24, 40, 20, 0.3)
    assert c.layers[1].mlp == MoEFFConfig(6, 2, 3, 4, 2, 1.7, 24, 24) and c.layers[1].mlp.routed == 8
    assert c.layers[2].mlp is None
    assert c.layers[3].mlp.shared_ff == 0 and c.layers[3].mlp.identity == 0
    assert sequence_config_from_dict(cases.unaligned()).canon_taps == 0
    with pytest.raises(ValueError):
        sequence_config_from_dict({"architecture": "nope"})
    assert "Sidalorn" in SEQUENCE_ARCHITECTURES


def test_model_declares_the_tensors_the_test_checkpoint_holds():
    from qwen3_tts_cuda_graphs_b200.sidalorn import tensor_specs

    for make in (cases.odd, cases.unaligned, cases.aligned):
        cfg = make()
        W = cases.weights(cfg)
        specs = tensor_specs(sequence_config_from_dict(cfg))
        assert set(W) == set(specs)
        assert all(tuple(W[k].shape) == tuple(specs[k]) for k in W)


def test_state_slots_are_reset_reused_and_bounded():
    specs = [StateSpec("tail", "carry", 6, 3), StateSpec("none", "carry", 6, 0), StateSpec("cache", "append", 4, dtype=torch.bfloat16)]
    m = SequenceStateManager(specs, max_pos=10, device="cpu", max_slots=2)
    a = m.acquire("a")
    assert a.cur["cache"].shape == (10, 4) and a.cur["tail"].shape == (3, 6) and "none" not in a.cur
    assert a.commit.shape == (1, 3) and int(a.commit[0, 2]) == 3 * 6 * 4
    assert m.reserve(a, 4) == 0 and m.reserve(a, 6) == 4
    with pytest.raises(RuntimeError):
        m.reserve(a, 1)
    a.cur["tail"].fill_(3.0); a.next["tail"].fill_(2.0); a.pos.fill_(10)
    b = m.acquire("b")
    assert b.index == 1 and m.free_slots() == 0
    with pytest.raises(RuntimeError):
        m.acquire("c")
    with pytest.raises(KeyError):
        m.acquire("a")
    m.release("a")
    c = m.acquire("c")                   # takes a's slot, cleared
    assert c is a and c.length == 0 and int(c.pos) == 0 and float(c.cur["tail"].abs().sum() + c.next["tail"].abs().sum()) == 0
    assert m.get("a") is None and m.get("c") is c
    with pytest.raises(ValueError):
        SequenceStateManager([StateSpec("x", "carry", 1), StateSpec("x", "carry", 1)], 4, "cpu")


def test_oracle_is_causal_and_its_parts_mean_what_they_say():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=3)
    toks = cases.tokens(cfg, 30)
    full = so.forward(cfg, W, toks)
    assert torch.allclose(so.forward(cfg, W, toks[:17]), full[:17], atol=1e-9)       # later tokens change nothing earlier
    # grouped norm: every group of the output (before the weight) has unit RMS
    v = torch.randn(4, 12, dtype=torch.float64)
    n = so.grouped_rms_norm(v, torch.ones(12, dtype=torch.float64), 3, 0.0).reshape(4, 3, 4)
    assert torch.allclose((n * n).mean(-1), torch.ones(4, 3, dtype=torch.float64))
    # convolution: the last column weighs the current token, nothing comes from the future
    x = torch.zeros(5, 1, dtype=torch.float64); x[2] = 1.0
    out = so.causal_time_conv(x, torch.tensor([[10.0, 20.0, 30.0]], dtype=torch.float64))
    assert out[:, 0].tolist() == [0.0, 0.0, 30.0, 20.0, 10.0]


def test_oracle_router_groups_mask_with_minus_infinity_and_identity_experts_pass_the_input():
    W = {"m.router": torch.zeros(4, 3, dtype=torch.float64), "m.correction": torch.tensor([-0.9, -0.8, -0.5, -0.7], dtype=torch.float64)}
    h = torch.ones(1, 3, dtype=torch.float64)
    r = {"experts": 2, "identity": 2, "top": 2, "scale": 3.0, "groups": {"count": 2, "keep": 1}}
    ids, w = so.route(h, W, "m.", r)
    # scores are all 0.25; choices -0.65, -0.55 | -0.25, -0.45: group 1 wins, and with the loser at minus infinity (not 0, which
    # would beat every negative choice) both picks come from it, best first
    assert ids.tolist() == [[2, 3]]
    assert torch.allclose(w, torch.tensor([[1.5, 1.5]], dtype=torch.float64))
    out = so.moe_ff(h, W, "m.", {"router": r, "shared": None})
    assert torch.allclose(out, 3.0 * h)                                              # two identity experts, weights 1.5 each


def test_oracle_sink_only_enlarges_the_denominator():
    H, dk, dv, R, width = 2, 4, 3, 5, 6
    g = torch.Generator().manual_seed(0)
    W = {"m." + k: torch.randn(*s, generator=g, dtype=torch.float64) for k, s in
         [("q", (H * dk, width)), ("dkv", (R, width)), ("uk", (H * dk, R)), ("uv", (H * dv, R))]}
    W["m.dkv.norm"] = torch.ones(R, dtype=torch.float64)
    W["m.o"] = torch.eye(width, dtype=torch.float64)[:, :H * dv]
    m = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": R, "scale": 0.5}
    h = torch.randn(1, width, generator=g, dtype=torch.float64)
    plain = so.latent_attention(h, W, "m.", m, 1e-6)
    # one token: without a sink the weight of the only key is 1; with sink s it is e^z / (e^z + e^s)
    q = (h @ W["m.q"].T).reshape(H, dk)
    lat = so.rms_unit(h @ W["m.dkv"].T, 1e-6)
    z = ((lat @ W["m.uk"].T).reshape(H, dk) * q).sum(-1) * 0.5
    W["m.sink"] = torch.tensor([0.3, -1.0], dtype=torch.float64)
    with_sink = so.latent_attention(h, W, "m.", m, 1e-6)
    ratio = (torch.exp(z) / (torch.exp(z) + torch.exp(W["m.sink"]))).repeat_interleave(dv)
    assert torch.allclose(with_sink[0, :H * dv], plain[0, :H * dv] * ratio)


def test_trace_runner_and_cli_parse_their_arguments():
    from qwen3_tts_cuda_graphs_b200 import cli

    a = cli.build_parser().parse_args(["lm", "--model", "m", "--tokens", "1 2 3", "--tokens", "4,5", "--greedy", "--max-new-tokens", "7"])
    assert a.tokens == ["1 2 3", "4,5"] and a.greedy and a.max_new_tokens == 7 and a.fn is cli.cmd_lm
