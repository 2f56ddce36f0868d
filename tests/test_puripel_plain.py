"""Puripel without a GPU: the configuration reader, the run order it makes, the tensors the parts ask for, and the plain
implementation's own consistency (what it computes for a prefix does not change when the sequence goes on; a key
outside a window changes nothing; the pieces of a mechanism add up)."""

import copy
import math

import pytest
import torch

from tests import plain_puripel as P
from tests import puripel_configs as C


def test_the_reader_names_every_tensor_of_the_design():
    from tandemllm_b200.config import PuripelConfig, architecture_of
    from tandemllm_b200.parts.model import DecoderModel
    for name, cfg in C.CONFIGS.items():
        assert architecture_of(cfg).name == "puripel"
        spec = PuripelConfig.from_dict(cfg).to_spec()
        got = {s.name: tuple(s.shape) for s in DecoderModel(spec).weight_specs(None)}
        assert got == C.tensor_shapes(cfg), name


def test_the_run_order_repeats_the_looped_layers_with_caches_of_their_own():
    from tandemllm_b200.config import PuripelConfig
    spec = PuripelConfig.from_dict(C.P1).to_spec()
    assert [s.layer for s in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [s.add.row if s.add else None for s in spec.schedule] == [None, 0, None, 1, None, 2, None, None]
    assert all(s.cache_of is None for s in spec.schedule)
    assert [(i, t) for i, t in P.run_order(C.P1)] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    plain = copy.deepcopy(C.P2)
    assert [s.layer for s in PuripelConfig.from_dict(plain).to_spec().schedule] == [0, 1, 2]
    once = PuripelConfig.from_dict(C.P4).to_spec().schedule
    assert [s.layer for s in once] == [0, 1, 2, 3] and once[1].add.row == 0 and once[1].add.rows == 1


def test_unknown_keys_and_bad_sizes_are_refused_by_name():
    from tandemllm_b200.config import PuripelConfig
    bad = copy.deepcopy(C.P2)
    bad["layers"][0]["mixer"]["heads_kv"] = 2
    with pytest.raises(ValueError, match="heads_kv"):
        PuripelConfig.from_dict(bad)
    bad = copy.deepcopy(C.P2)
    bad["layers"][1]["mlp"]["router"]["groups"]["count"] = 3
    with pytest.raises(ValueError, match="groups"):
        PuripelConfig.from_dict(bad)
    bad = copy.deepcopy(C.P1)
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError, match="loop"):
        PuripelConfig.from_dict(bad)
    bad = copy.deepcopy(C.P1)
    bad["layers"][0]["type"] = "mamba3"
    with pytest.raises(ValueError, match="mamba3"):
        PuripelConfig.from_dict(bad)
    assert PuripelConfig.from_dict(C.P3).to_dict() == C.P3


def test_the_plain_model_is_causal_and_its_windows_end_where_they_should():
    cfg, W = C.P1, C.weights("p1")
    toks = C.tokens("p1", 40, seed=1)
    whole = P.forward(cfg, W, toks)
    assert torch.allclose(P.forward(cfg, W, toks[:17]), whole[:17], atol=1e-10)
    # latent attention alone: a key `window` back is not seen, the one after it is
    m = cfg["layers"][1]["mixer"]
    w64 = {k: v.double() for k, v in W.items()}
    g = torch.Generator().manual_seed(3)
    h = torch.randn(12, cfg["width"], generator=g, dtype=torch.float64)
    base = P.latent_attention_mixer(h, m, w64, "l1.mix.", 1e-4)
    h2 = h.clone()
    h2[11 - m["mask"]["size"]] += 3.0            # just outside the last row's window
    assert torch.allclose(P.latent_attention_mixer(h2, m, w64, "l1.mix.", 1e-4)[11], base[11], atol=1e-12)
    h3 = h.clone()
    h3[11 - m["mask"]["size"] + 1] += 3.0        # the oldest key it sees
    assert not torch.allclose(P.latent_attention_mixer(h3, m, w64, "l1.mix.", 1e-4)[11], base[11], atol=1e-6)


def test_the_state_space_recurrence_equals_its_unrolled_sum():
    """y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (C_t . B_s) x_s + D x_t, written out for one head."""
    cfg, W = C.P3, {k: v.double() for k, v in C.weights("p3").items()}
    m = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(5)
    T = 9
    h = torch.randn(T, cfg["width"], generator=g, dtype=torch.float64)
    p = "l0.mix."
    H, Pc, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * Pc
    proj = h @ W[p + "in"].T
    xbc = P.silu(P.causal_conv(proj[:, inner:2 * inner + 2 * G * N], W[p + "conv"], W[p + "conv.b"]))
    x, B, Cm = xbc[:, :inner].view(T, H, Pc), xbc[:, inner:inner + G * N].view(T, G, N), xbc[:, inner + G * N:].view(T, G, N)
    dt = P.softplus(proj[:, 2 * inner + 2 * G * N:] + W[p + "dt_bias"])
    a = torch.exp(-torch.exp(W[p + "A_log"]) * dt)
    y = torch.zeros(T, H, Pc, dtype=torch.float64)
    for hd in range(H):
        gi = hd // (H // G)
        for t in range(T):
            for s in range(t + 1):
                y[t, hd] += a[s + 1:t + 1, hd].prod() * dt[s, hd] * (Cm[t, gi] @ B[s, gi]) * x[s, hd]
            y[t, hd] += W[p + "D"][hd] * x[t, hd]
    v = y.reshape(T, inner) * P.silu(proj[:, :inner])
    parts = m["norm_groups"]
    v = P.rms_norm(v.view(T, parts, -1), None, 1e-5).reshape(T, inner) * W[p + "norm"]
    assert torch.allclose(P.mamba2_mixer(h, m, W, p, 1e-5), v @ W[p + "o"].T, atol=1e-9)


def test_the_router_keeps_to_the_best_groups_and_the_correction_moves_the_choice_only():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    w = {"x.router": torch.eye(6, dtype=torch.float64), "x.correction": torch.zeros(6, dtype=torch.float64)}
    # scores: group 0 holds the single best expert, group 1 the best pair
    z = torch.tensor([[3.0, -5.0, 1.0, 1.2, -1.0, 0.0]], dtype=torch.float64)
    ids, wts = P.route(z, w, "x.", r)
    assert sorted(ids[0].tolist()) == [2, 3]
    s = torch.sigmoid(z[0])
    assert torch.allclose(wts[0].sum(), torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(wts[0, ids[0].tolist().index(3)], 2.0 * s[3] / (s[2] + s[3]))
    # a correction lifts group 2 into the choice; the weights still come from the uncorrected scores
    w["x.correction"] = torch.tensor([0.0, 0.0, 0.0, 0.0, 1.0, 1.0], dtype=torch.float64)
    ids, wts = P.route(z, w, "x.", r)
    assert sorted(ids[0].tolist()) == [4, 5]
    assert torch.allclose(wts[0, ids[0].tolist().index(5)], 2.0 * s[5] / (s[4] + s[5]))
    # negative choice scores: a dropped group's experts lose against them all the same
    w["x.correction"] = torch.full((6,), -3.0, dtype=torch.float64)
    ids, _ = P.route(z, w, "x.", r)
    assert sorted(ids[0].tolist()) == [2, 3]
    assert P.choice_margin(z, w, "x.", r) > 0


def test_an_expert_is_clamped_before_its_gate():
    w = {"e.gate": torch.tensor([[1.0]], dtype=torch.float64), "e.up": torch.tensor([[1.0]], dtype=torch.float64),
         "e.down": torch.tensor([[1.0]], dtype=torch.float64)}
    for x, limit in [(0.5, 2.0), (5.0, 2.0), (-5.0, 2.0)]:
        g, u = min(x, limit), max(-limit, min(x, limit))
        want = g / (1 + math.exp(-1.702 * g)) * (u + 1)
        got = P.expert(torch.tensor([[x]], dtype=torch.float64), w, "e.", limit)
        assert abs(float(got) - want) < 1e-12
