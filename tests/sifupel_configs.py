"""Tiny Sifupel configurations of the tests (config.json dictionaries), their random weights and prompts.

s1: three layers that differ in everything: grouped heads with a window of 5; as many KV heads as heads, a head size that
    is no multiple of 16, a window of 33 and no feed-forward; one KV head, a head size of 8 and a window of 1 (a row sees
    itself only). Width and vocabulary are no multiples of 8.
s2: widths and head sizes that the tensor-core kernels of the bfloat16 path take (multiples of 8, heads of 64 and 32),
    windows of 70 and 48 (a page's multiple).
s3: a head size of 128, a window longer than any test's sequence (nothing is ever masked but the future), and a layer
    whose window is exactly four pages.
s4: sizes no kernel is tuned for: an odd vocabulary and a width that is no multiple of 8, head sizes of 20, 72, 40 and 256,
    one head, five heads that are their own KV heads, forty heads over eight KV heads (more than the tensor-core kernel
    takes), feed-forward widths that are no multiples of 8, windows of 100, 7, 64 and 3, six layers, two without a feed-forward.
No scale equals dim^-1/2, eps differs, and the norms' alpha, weight and bias are random.
"""

from __future__ import annotations

import json
import os

import torch


def _attn(heads, kv, dim, window, scale, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": window}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


S1 = {"architecture": "Sifupel", "vocab": 97, "width": 44, "norm": {"eps": 1e-4},
      "layers": [_attn(4, 2, 16, 5, 0.31, 80), _attn(3, 3, 24, 33, 0.17, None), _attn(6, 1, 8, 1, 0.5, 52)]}
S2 = {"architecture": "Sifupel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
      "layers": [_attn(4, 2, 64, 70, 0.2, 192), _attn(8, 4, 32, 48, 0.11, 256)]}
S3 = {"architecture": "Sifupel", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
      "layers": [_attn(2, 1, 128, 300, 0.05, 96), _attn(2, 2, 32, 64, 0.4, 72)]}
S4 = {"architecture": "Sifupel", "vocab": 1001, "width": 100, "norm": {"eps": 3e-6},
      "layers": [_attn(5, 5, 20, 100, 0.21, 136), _attn(1, 1, 72, 7, 0.09, None), _attn(12, 3, 40, 64, 0.13, 28),
                 _attn(40, 8, 64, 50, 0.12, 44), _attn(2, 2, 256, 3, 0.06, None), _attn(9, 3, 48, 31, 0.19, 60)]}
CONFIGS = {"s1": S1, "s2": S2, "s3": S3, "s4": S4}
SEEDS = {"s1": 11, "s2": 12, "s3": 13, "s4": 14}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}"
        norm(p + ".norm1")
        out[p + ".mix.q"] = (m["heads"] * m["dim"], W)
        out[p + ".mix.k"] = (m["kv_heads"] * m["dim"], W)
        out[p + ".mix.talk"] = (m["heads"], m["heads"])
        out[p + ".mix.g"] = (m["heads"], W)
        out[p + ".mix.o"] = (W, m["heads"] * m["vdim"])
        if layer["mlp"] is not None:
            norm(p + ".norm2")
            out[p + ".mlp.up"] = (layer["mlp"]["ff"], W)
            out[p + ".mlp.down"] = (W, layer["mlp"]["ff"])
            out[p + ".mlp.act"] = (2,)
    norm("final.norm")
    return out


def weights(name: str, bf16_exact: bool = True) -> dict[str, torch.Tensor]:
    """32-bit random weights by stored name; with `bf16_exact` every value is a bfloat16 value, so that the engine in
    either precision and the plain model read the same numbers."""
    cfg = CONFIGS[name]
    g = torch.Generator().manual_seed(SEEDS[name])
    out = {}
    for key, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g)
        if key == "embed":
            t = t * 0.8
        elif key.endswith(".alpha"):
            t = 0.6 + 0.2 * t.abs()
        elif key.endswith(".b"):
            t = 0.1 * t
        elif ".norm" in key:
            t = 1.0 + 0.2 * t
        elif key.endswith(".talk"):
            t = torch.eye(shape[0]) + 0.3 * t
        elif key.endswith(".act"):
            t = 0.5 * t
        else:
            t = t * (shape[1] ** -0.5)
        out[key] = t.to(torch.bfloat16).float() if bf16_exact else t
    return out


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
