"""CPU tests of Sifupel: the configuration reader and registry, the model's tensor list against the design's names, and
the plain implementation's own mechanisms (its window, its activation, causality, what the head mix reduces to)."""

import copy

import pytest
import torch

from tests import plain_sifupel as P
from tests import sifupel_configs as S


def test_the_registry_chooses_the_reader_by_the_architecture_string():
    from tandemllm_b200.config import SifupelConfig, architecture_of
    arch = architecture_of(S.S1)
    assert arch.name == "sifupel"
    cfg = arch.read_config(S.S1, "", None)
    assert isinstance(cfg, SifupelConfig) and cfg.to_dict()["layers"][1]["mlp"] is None
    assert SifupelConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("where", ["top", "layer", "mixer", "mask", "mlp", "norm"])
def test_an_unknown_key_is_refused_by_name(where):
    from tandemllm_b200.config import SifupelConfig
    raw = copy.deepcopy(S.S1)
    {"top": raw, "layer": raw["layers"][0], "mixer": raw["layers"][0]["mixer"], "mask": raw["layers"][0]["mixer"]["mask"],
     "mlp": raw["layers"][0]["mlp"], "norm": raw["norm"]}[where]["surprise"] = 1
    with pytest.raises(ValueError, match="surprise"):
        SifupelConfig.from_dict(raw)


def test_values_that_do_not_fit_are_refused():
    from tandemllm_b200.config import SifupelConfig
    for change in (lambda r: r["layers"][0]["mixer"].update(vdim=8), lambda r: r["layers"][0]["mixer"].update(kv_heads=3),
                   lambda r: r["layers"][0].update(type="recurrent"), lambda r: r["layers"][0]["mlp"].update(kind="routed"),
                   lambda r: r["layers"][0]["mixer"].pop("scale")):
        raw = copy.deepcopy(S.S1)
        change(raw)
        with pytest.raises(ValueError):
            SifupelConfig.from_dict(raw)


@pytest.mark.parametrize("name", ["s1", "s2", "s3", "s4"])
def test_the_parts_read_the_designs_tensors_and_no_others(name):
    from tandemllm_b200.config import SifupelConfig
    from tandemllm_b200.parts.model import DecoderModel
    spec = SifupelConfig.from_dict(S.CONFIGS[name]).to_spec()
    want = S.tensor_shapes(S.CONFIGS[name])
    got = {s.name: tuple(s.shape) for s in DecoderModel(spec).weight_specs(set(want))}
    assert got == want
    # a layer without a feed-forward declares no second norm when the folder has none, and binds one that is there
    assert {s.name for s in DecoderModel(spec).weight_specs(None)} == set(want)


def test_window_activation_and_causality_of_the_plain_model():
    vis = P.visible(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[0].tolist() == [True] + [False] * 5
    pq = torch.tensor([0.3, -0.2], dtype=torch.float64)
    z = torch.tensor([-1e-9, 0.0, 1e-9], dtype=torch.float64)
    y = P.xielu(z, pq)
    assert float(y[1]) == 0.0 and abs(float(y[2] - y[0]) - 1e-9) < 1e-12        # continuous, slope 1/2 at 0
    cfg, W = S.CONFIGS["s1"], S.weights("s1")
    toks = S.tokens("s1", 40, seed=1)
    full = P.forward(cfg, W, toks)
    assert torch.allclose(P.forward(cfg, W, toks[:17]), full[:17], atol=1e-10)


def test_the_head_mix_with_the_identity_is_ordinary_attention():
    cfg = copy.deepcopy(S.CONFIGS["s3"])
    W = S.weights("s3")
    m = cfg["layers"][0]["mixer"]
    W["l0.mix.talk"] = torch.eye(m["heads"])
    n = torch.randn(12, cfg["width"], dtype=torch.float64)
    got = P.head_mixed_attention(n, W, "l0", m, 1e-5)
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = P.unit_rms((n @ W["l0.mix.q"].double().T).view(12, H, D), 1e-5)
    kr = (n @ W["l0.mix.k"].double().T).view(12, G, D)
    k = P.unit_rms(kr, 1e-5)
    outs = []
    for h in range(H):
        c = h // (H // G)
        s = (q[:, h] @ k[:, c].T) * m["scale"]
        s = s.masked_fill(~P.visible(12, m["mask"]["size"]), float("-inf"))
        outs.append(torch.softmax(s, -1) @ kr[:, c] * torch.sigmoid(n @ W["l0.mix.g"].double().T)[:, h:h + 1])
    want = torch.cat(outs, -1) @ W["l0.mix.o"].double().T
    assert torch.allclose(got, want, atol=1e-10)


def test_the_command_line_writes_and_audits_a_folder_of_this_design(tmp_path):
    import json

    from tandemllm_b200.__main__ import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(S.S1))
    out = tmp_path / "model"
    assert main(["random-weights", "--config", str(cfg), "--seed", "3", "--out", str(out)]) == 0
    from tandemllm_b200.config import read_model_config, spec_of
    from tandemllm_b200.parts.model import DecoderModel
    from tandemllm_b200.weights.loader import FolderWeights
    arch, config = read_model_config(str(out))
    spec = spec_of(config)
    weights = FolderWeights(str(out), spec.name_prefixes)
    weights.check(DecoderModel(spec).weight_specs(weights.present()))
    assert arch.name == "sifupel" and set(weights.present()) == set(S.tensor_shapes(S.S1))
    assert main(["audit", "--model", str(out)]) == 0
