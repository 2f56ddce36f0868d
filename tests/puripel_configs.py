"""Tiny Puripel configurations of the tests (config.json dictionaries), their random weights and prompts.

p1: sizes no kernel is tuned for: an odd vocabulary, a width that is no multiple of 8, three state-space heads of 12
    columns over a state of 5 with one group, two taps, one norm part; a latent of 20 with 3 heads of 8 + 6, values of 10,
    a window of 5 and only 4 of the 6 rotated entries turned; a layer without a feed-forward; four heads that are their
    own groups with four taps and two norm parts; top-1 of 6 experts in 3 groups of which 1 is kept, experts without groups, no shared
    expert in one layer. Layers 1..2 run three times.
p2: widths the tensor-core kernels of the bfloat16 path take; latent attention first; a window that is a page's
    multiple; 8 experts top-3 in 2 groups, 1 kept; no loop.
p3: a window longer than any test's sequence, a state of 128 rows with columns of 40, the whole model run twice, every
    group kept (the groups then decide nothing), top equal to the number of experts in one layer.
p4: a loop that runs once, starting after the first layer; one head everywhere; a window of 1 (a row sees itself only);
    a state of one row.
No two layers of a model agree in their sizes, scales differ from (dim + rot_dim)^-1/2, eps differs from model to model.
"""

from __future__ import annotations

import json
import os

import torch


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, window, mlp, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, limit, scale=1.0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


P1 = {"architecture": "Puripel", "vocab": 97, "width": 44, "norm": {"eps": 1e-4},
      "layers": [mamba(3, 12, 5, 1, 2, 1, moe(6, 1, 10, 0.7, 1.5, (3, 1), (12, 1.1))),
                 latent(3, 8, 6, 10, 20, 12, 0.21, 100.0, 5, None, dims=4),
                 mamba(4, 8, 16, 4, 4, 2, moe(5, 2, 14, 1.2, 0.8, None, None)),
                 latent(2, 12, 4, 6, 9, 7, 0.4, 30.0, 33, moe(4, 2, 9, 0.9, 2.0, (2, 1), (20, 0.5)))],
      "loop": {"start": 1, "stop": 3, "times": 3}}
P2 = {"architecture": "Puripel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
      "layers": [latent(4, 64, 32, 64, 128, 96, 0.08, 10000.0, 48, moe(8, 3, 64, 1.0, 1.0, (2, 1), (128, 1.5))),
                 mamba(8, 16, 64, 2, 4, 1, moe(8, 2, 48, 2.5, 2.5, (4, 2), (64, 3.0))),
                 latent(16, 16, 16, 32, 64, 64, 0.15, 500.0, 70, moe(16, 4, 32, 1.5, 1.0, (8, 3), (96, 1.0)))]}
P3 = {"architecture": "Puripel", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
      "layers": [mamba(2, 40, 128, 1, 3, 2, moe(4, 4, 24, 1.3, 1.0, (2, 2), (40, 2.0))),
                 latent(5, 24, 8, 16, 40, 48, 0.12, 1000.0, 300, moe(6, 2, 16, 0.6, 3.0, (3, 2), (24, 0.8)))],
      "loop": {"start": 0, "stop": 2, "times": 2}}
P4 = {"architecture": "Puripel", "vocab": 211, "width": 56, "norm": {"eps": 3e-6},
      "layers": [latent(1, 16, 2, 24, 17, 11, 0.3, 7.0, 1, moe(3, 1, 8, 1.0, 1.0, None, (8, 1.0))),
                 mamba(1, 24, 1, 1, 5, 3, None),
                 mamba(6, 4, 9, 3, 2, 2, moe(9, 3, 12, 0.4, 1.7, (3, 2), (16, 2.2))),
                 latent(7, 4, 12, 3, 33, 20, 0.25, 64.0, 16, moe(10, 2, 6, 2.0, 0.5, (5, 4), None))],
      "loop": {"start": 1, "stop": 4, "times": 1}}
CONFIGS = {"p1": P1, "p2": P2, "p3": P3, "p4": P4}
SEEDS = {"p1": 21, "p2": 22, "p3": 23, "p4": 24}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}"
        out[p + ".norm1"], out[p + ".norm1b"] = (W,), (W,)
        if layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + ".mix.in"] = (2 * inner + 2 * gn + m["heads"], W)
            out[p + ".mix.conv"] = (inner + 2 * gn, m["conv"])
            out[p + ".mix.conv.b"] = (inner + 2 * gn,)
            for name in ("dt_bias", "A_log", "D"):
                out[f"{p}.mix.{name}"] = (m["heads"],)
            out[p + ".mix.norm"] = (inner,)
            out[p + ".mix.o"] = (W, inner)
        else:
            H = m["heads"]
            out[p + ".mix.dq"], out[p + ".mix.dq.norm"] = (m["q_rank"], W), (m["q_rank"],)
            out[p + ".mix.uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            out[p + ".mix.dkv"], out[p + ".mix.dkv.norm"] = (m["kv_rank"] + m["rot_dim"], W), (m["kv_rank"],)
            out[p + ".mix.uk"], out[p + ".mix.uv"] = (H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"])
            out[p + ".mix.o"] = (W, H * m["vdim"])
        mlp = layer["mlp"]
        if mlp is not None:
            out[p + ".norm2"], out[p + ".norm2b"] = (W,), (W,)
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[p + ".mlp.router"], out[p + ".mlp.correction"] = (E, W), (E,)
            for e in range(E):
                out[f"{p}.mlp.e{e}.gate"], out[f"{p}.mlp.e{e}.up"], out[f"{p}.mlp.e{e}.down"] = (ff, W), (ff, W), (W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out[p + ".mlp.shared.gate"], out[p + ".mlp.shared.up"] = (sf, W), (sf, W)
                out[p + ".mlp.shared.down"], out[p + ".mlp.shared.sg"] = (W, sf), (1, W)
    out["final.norm"] = (W,)
    return out


def weights_of(cfg: dict, seed: int, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    """32-bit random weights by stored name; with `bf16_exact` every value is a bfloat16 value, so that the engine in
    either precision and the plain model read the same numbers. Sizes are chosen so that every mechanism matters: gates
    and experts reach their limits, the corrections reorder the choice, step sizes and decays spread over (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for key, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g)
        if key == "embed":
            t = t * 0.8
        elif key == "loop.step":
            t = t * 0.5
        elif key.endswith(".correction"):
            t = t * 0.3
        elif key.endswith(".conv"):
            t = t * 0.6
        elif key.endswith(".conv.b") or key.endswith(".dt_bias"):
            t = t * 0.5
        elif key.endswith(".A_log"):
            t = t * 0.7 - 0.5
        elif key.endswith(".D"):
            t = 1.0 + 0.5 * t
        elif "norm" in key.rsplit(".", 1)[-1] or key.endswith("final.norm"):
            t = 1.0 + 0.2 * t
        elif key.endswith(".router") or key.endswith(".sg"):
            t = t * 1.5 * (shape[1] ** -0.5)
        elif key.endswith(".gate") or key.endswith(".up"):
            t = t * 1.6 * (shape[1] ** -0.5)
        else:
            t = t * (shape[1] ** -0.5)
        out[key] = t.to(torch.bfloat16).float() if bf16_exact else t
    return out


def weights(name: str, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    return weights_of(CONFIGS[name], SEEDS[name], bf16_exact)


def tokens(name: str, n: int, seed: int = 0) -> list[int]:
    g = torch.Generator().manual_seed(seed * 7919 + n)
    return torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist()


def write_folder(folder: str, name: str) -> str:
    """config.json and model.safetensors (bfloat16, as the design stores them) of the tiny model `name`."""
    from tandemllm_b200.weights.safetensors_io import write_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    write_file(os.path.join(folder, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in weights(name).items()})
    return folder
