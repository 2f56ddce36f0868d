"""A plain, slow Puripel: one function a mechanism, float64 on the CPU, whole sequences at once, no cache.

It shares no code with the engine: the tests hold the engine's logits (whole prompts, portions, decoding, batches)
against this. `weights` maps tensor names to tensors, `cfg` is the configuration as config.json holds it.

  layer        x += norm1b(mixer(norm1 x));  x += norm2b(ff(norm2 x))     (both pairs of RMS norms with weights)
  run order    layers [start, stop) are run `times` times with the same weights; before each pass the pass's row of
               `loop.step` is added to x; then the layers from `stop` on
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotate_pairs(x, positions, base, dims):
    """Interleaved rotary on the first `dims` entries of the last axis: entries (2i, 2i+1) turn by p * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(F64)[:, None] * f[None, :]                     # [T, dims/2]
    shape = [a.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def causal_conv(x, taps, bias):
    """x [T, C]; taps [C, K], the last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for k in range(K):
        out += padded[k:k + T] * taps[:, k]
    return out + bias


def mamba2_mixer(h, m, w, p, eps):
    """h [T, width]; m the mixer's sizes; w the weights; p the tensors' prefix ('l0.mix.')."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)              # [T, H]
    y = torch.zeros(T, H, P, dtype=h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    group = torch.arange(H) // (H // G)                              # head -> its group's B and C
    for t in range(T):
        Bt, Ct = B[t, group], C[t, group]                            # [H, N]
        S = decay[t, :, None, None] * S + dt[t, :, None, None] * Bt[:, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + w[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def latent_attention_mixer(h, m, w, p, eps):
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :L], w[p + "dkv.norm"], eps)
    rot = m.get("rot") or {}
    base, dims = rot.get("base", 10000.0), rot.get("dims", R)
    k_rot = rotate_pairs(kv[:, L:], pos, base, dims)               # [T, R], shared by the heads
    q_rot = rotate_pairs(q[..., D:], pos, base, dims)
    k_nope = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], k_nope) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i)
    if m.get("mask"):
        seen &= (i - j) < m["mask"]["size"]
    s = s.masked_fill(~seen, -math.inf)
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", a, v).reshape(T, H * V)
    return o @ w[p + "o"].T


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def route(h, w, p, r):
    """(ids [T, top], weights [T, top]) of the rows h."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        by_group = choice.view(-1, n, per)
        gscore = by_group.topk(min(2, per), dim=-1).values.sum(-1)          # [T, n]
        kept = gscore.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), -math.inf)
    ids = choice.topk(top, dim=-1).indices
    wts = s.gather(1, ids)
    wts = wts / (wts.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return ids, wts


def choice_margin(h, w, p, r):
    """How far the router's decisions are from going the other way: the smallest gap between the last chosen and the
    first unchosen choice score of a row and, with groups, between the last kept and the first dropped group's score."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    gap = math.inf
    groups = r.get("groups")
    if groups and groups["keep"] < groups["count"]:
        per = E // groups["count"]
        gs = choice.view(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(-1).sort(dim=-1, descending=True).values
        gap = float((gs[:, groups["keep"] - 1] - gs[:, groups["keep"]]).min())
        kept = gs[:, groups["keep"] - 1:groups["keep"]]
        full = choice.view(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(-1)
        allowed = (full >= kept)[:, :, None].expand(-1, -1, per).reshape(-1, E)
        choice = choice.masked_fill(~allowed, -math.inf)
    if top < E:
        c = choice.sort(dim=-1, descending=True).values
        d = c[:, top - 1] - c[:, top]
        gap = min(gap, float(d[torch.isfinite(d)].min()) if torch.isfinite(d).any() else math.inf)
    return gap


def greedy(cfg, weights, prompt, n):
    """The n tokens the model continues `prompt` with when it always takes the most likely one."""
    text = list(prompt)
    for _ in range(n):
        text.append(int(forward(cfg, weights, text)[-1].argmax()))
    return text[len(prompt):]


def moe(h, mlp, w, p, forced=None):
    """`forced` (ids [T, top]): the experts to use instead of the router's own choice; the weights follow the ids."""
    T = h.shape[0]
    r = mlp["router"]
    ids, wts = route(h, w, p, r)
    if forced is not None:
        ids = torch.as_tensor(forced, dtype=torch.long)
        s = torch.sigmoid(h @ w[p + "router"].T).gather(1, ids)
        wts = s / (s.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    out = torch.zeros_like(h)
    limit = mlp["expert"]["limit"]
    for t in range(T):
        for e, a in zip(ids[t].tolist(), wts[t]):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", limit)[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)             # [T, 1]
        out = out + gate * expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def run_order(cfg):
    """[(layer, pass number when the layer is a pass's first, else None)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, weights, tokens, layer_outputs: list | None = None, routes: list | None = None, margins: list | None = None,
            halves: bool = False):
    """Logits float64 [T, vocab] of one sequence; `layer_outputs` collects the residual stream after every layer run.
    `routes`: for every routed feed-forward in run order, the expert ids [T, top] to use instead of the router's choice.
    `margins` collects, for every routed feed-forward run, the smallest gap between a chosen and an unchosen choice score.
    With `halves`, `layer_outputs` also gets the stream after every mixer's half of a layer."""
    routes = list(routes) if routes is not None else None
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, t in run_order(cfg):
        if t is not None:
            x = x + w["loop.step"][t]
        layer = cfg["layers"][i]
        p = f"l{i}."
        n = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mamba2":
            d = mamba2_mixer(n, layer["mixer"], w, p + "mix.", eps)
        elif layer["type"] == "latent_attention":
            d = latent_attention_mixer(n, layer["mixer"], w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(d, w[p + "norm1b"], eps)
        if layer_outputs is not None and halves:
            layer_outputs.append(x.clone())
        if layer.get("mlp"):
            n = rms_norm(x, w[p + "norm2"], eps)
            if margins is not None:
                margins.append(choice_margin(n, w, p + "mlp.", layer["mlp"]["router"]))
            x = x + rms_norm(moe(n, layer["mlp"], w, p + "mlp.", routes.pop(0) if routes else None), w[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
