"""A plain, slow implementation of the Sifupel decoder: whole sequences, no cache, one function per mechanism,
plain torch on the CPU in 64-bit or 32-bit. It shares no code with the package: tests hold the engine to it.

The design, in this file's notation (x: a row of the residual stream, n: a normed row, W: a matrix stored
[out, in] and applied as W n):

  norm      dyt(x) = tanh(a x) * w + b, a one scalar a norm; no mean, no variance
  mixer     q = W_q n, k = W_k n, values = the keys as projected; q and k are brought to unit root mean square per
            head; s_g(i, j) = scale * <q_g(i), k_c(g)(j)> for i - window < j <= i; p_g = softmax_j s_g;
            p'_h = sum_g M[h, g] p_g  (the heads' weights are mixed after the softmax);
            o_h(i) = sigmoid(W_g n)_h * sum_j p'_h(i, j) k_raw_c(h)(j);  out = W_o concat_h o_h
  ff        W_down f(W_up n),  f(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (expm1(z) - z) + z / 2 else
  layer     x += mixer(dyt_1(x)); x += ff(dyt_2(x));   logits = E dyt_final(x), E the embedding table

Weights are a dict by stored name; the configuration is the config.json dict.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def dyt(x: torch.Tensor, W: dict, name: str) -> torch.Tensor:
    return torch.tanh(W[name + ".alpha"].to(x.dtype) * x) * W[name].to(x.dtype) + W[name + ".b"].to(x.dtype)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    ap = F.softplus(pq[0].to(z.dtype))
    an = 0.5 + F.softplus(pq[1].to(z.dtype))
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def visible(n: int, window: int) -> torch.Tensor:
    """[n, n] bool: row i sees column j when 0 <= i - j < window."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (i - j >= 0) & (i - j < window)


def head_mixed_attention(n: torch.Tensor, W: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The mixer on the normed rows n [T, width]; `m` is the layer's "mixer" dict, `p` the layer's name."""
    T = n.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    if m["vdim"] != D:
        raise ValueError("the values are the keys: vdim must equal dim")
    dt = n.dtype
    q = (n @ W[p + ".mix.q"].to(dt).T).view(T, H, D)
    k_raw = (n @ W[p + ".mix.k"].to(dt).T).view(T, G, D)
    gate = torch.sigmoid(n @ W[p + ".mix.g"].to(dt).T)              # [T, H]
    qn, kn = unit_rms(q, eps), unit_rms(k_raw, eps)
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", qn, kn[:, kv_of]) * m["scale"]   # [H, T, T]
    s = s.masked_fill(~visible(T, int(m["mask"]["size"]))[None], float("-inf"))
    w = torch.softmax(s, dim=-1)
    w = torch.einsum("hg,gij->hij", W[p + ".mix.talk"].to(dt), w)
    o = torch.einsum("hij,jhd->ihd", w, k_raw[:, kv_of]) * gate[:, :, None]
    return o.reshape(T, H * D) @ W[p + ".mix.o"].to(dt).T


def dense_ff(n: torch.Tensor, W: dict, p: str) -> torch.Tensor:
    dt = n.dtype
    return xielu(n @ W[p + ".mlp.up"].to(dt).T, W[p + ".mlp.act"]) @ W[p + ".mlp.down"].to(dt).T


def forward(cfg: dict, W: dict, tokens: list[int], dtype=torch.float64, keep_layers: bool = False):
    """Logits [T, vocab] of the whole sequence (and, with `keep_layers`, the residual stream after each layer)."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    kept = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        if layer["type"] != "attention":
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + head_mixed_attention(dyt(x, W, p + ".norm1"), W, p, layer["mixer"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            x = x + dense_ff(dyt(x, W, p + ".norm2"), W, p)
        if keep_layers:
            kept.append(x.clone())
    logits = dyt(x, W, "final.norm") @ W["embed"].to(dtype).T
    return (logits, kept) if keep_layers else logits


def greedy(cfg: dict, W: dict, prompt: list[int], n_new: int, dtype=torch.float64) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, W, toks, dtype)[-1].argmax()))
    return toks[len(prompt):]
