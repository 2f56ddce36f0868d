"""Sifupel on the GPU against the plain implementation (`tests/plain_sifupel.py`): every mechanism alone at the
kernels' own entry points, then whole models through the step function and the scheduler.

The tiny models differ from one another in every size and constant (head counts and grouping, head size, window,
scale, feed-forward width or none, eps, width, vocabulary, layer count), none has a scale of dim^-1/2, and the layers
of one model differ among themselves. Where random weights would hide a fault (one far key among hundreds, a window's
edge), one query and one key are scaled up so that one score stands out.

Tolerances as for the engine's other models: 32-bit within 1e-4 of a row's largest magnitude, bfloat16 within 3e-2.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import plain_sifupel as P
from tests import sifupel_configs as S

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float(((a - b).abs() / b.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)).max())


def engine_of(name, dtype, pages=64, parallel=4, **kw):
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.config import SifupelConfig
    from tandemllm_b200.weights.loader import DictWeights
    cfg = S.CONFIGS[name]
    W = S.weights(name, bf16_exact=True)
    spec = SifupelConfig.from_dict(cfg).to_spec()
    args = EngineArgs(dtype=dtype, max_len=4096, parallel=parallel, block_size=16, kv_blocks=pages, graph=False, **kw)
    return Engine._build(None, spec, DictWeights({k: v.clone() for k, v in W.items()}), args), cfg, W


@pytest.fixture(scope="module")
def plain_logits():
    memo = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in memo:
            memo[key] = P.forward(S.CONFIGS[name], S.weights(name, bf16_exact=True), list(tokens))
        return memo[key]
    return get


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [48, 50])
def test_dynamic_tanh_with_the_residual_add(dtype, hidden):
    from tandemllm_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    R = 9
    res = torch.randn(R, hidden, generator=g)
    parts = torch.randn(3, R, hidden, generator=g)
    w, b, a = 1 + 0.3 * torch.randn(hidden, generator=g), 0.2 * torch.randn(hidden, generator=g), torch.tensor([0.7])
    W = {"n": w.double(), "n.b": b.double(), "n.alpha": a.double()[0]}
    dev = "cuda"
    # a plain tensor
    r1 = res.clone().to(dev)
    out = torch.empty(R, hidden, dtype=DT[dtype], device=dev)
    ops.add_dyt(r1, parts[0].to(dev), w.to(dev), b.to(dev), a.to(dev), out)
    want_res = res.double() + parts[0].double()
    assert rel(r1, want_res) < 1e-6
    assert rel(out.float(), P.dyt(want_res, W, "n")) < (1e-6 if dtype == "float32" else 1e-2)
    # partial sums, added in order
    r2 = res.clone().to(dev)
    ps = ops.PartialSums(parts.to(dev).contiguous().view(-1), 3, R, hidden)
    ops.add_dyt(r2, ps, w.to(dev), b.to(dev), a.to(dev), out)
    want_res = res.double() + parts.double().sum(0)
    assert rel(r2, want_res) < 1e-6
    assert rel(out.float(), P.dyt(want_res, W, "n")) < (1e-6 if dtype == "float32" else 1e-2)
    # chosen rows only: the residual stays
    r3 = res.clone().to(dev)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=dev)
    out3 = torch.empty(3, hidden, dtype=DT[dtype], device=dev)
    ops.add_dyt(r3, parts[1].to(dev), w.to(dev), b.to(dev), a.to(dev), out3, rows)
    assert torch.equal(r3.cpu(), res)
    assert rel(out3.float(), P.dyt((res.double() + parts[1].double())[[7, 0, 3]], W, "n")) < (1e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_xielu_both_branches(dtype):
    from tandemllm_b200.kernels import ops
    z = torch.linspace(-9, 9, 1001).to(DT[dtype])
    pq = torch.tensor([0.4, -0.8])
    sp = torch.nn.functional.softplus(pq)
    out = torch.empty_like(z, device="cuda")
    ops.activation(z.cuda(), out, ops.ACTIVATIONS["xielu"], float(sp[0]), float(0.5 + sp[1]))
    want = P.xielu(z.double(), pq.double())
    assert rel(out.float()[None], want[None]) < (1e-6 if dtype == "float32" else 5e-3)
    assert float(want[-1]) > 30 and abs(float(want[0]) - (float(0.5 + sp[1]) * (np.exp(-9.0) + 8.0) - 4.5)) < 1e-5


def _paged(k, v, page_size, seed):
    """Scatter k, v [T, G, D] into shuffled pages of a pool; returns (k_cache, v_cache, table [1, pages])."""
    T_, G, D = k.shape
    n = -(-T_ // page_size)
    pool = n + 5
    order = torch.randperm(pool, generator=torch.Generator().manual_seed(seed))[:n]
    kc = torch.full((pool, G, page_size, D), float("nan"), dtype=k.dtype)
    vc = torch.full((pool, G, page_size, D), float("nan"), dtype=k.dtype)
    for t in range(T_):
        kc[order[t // page_size], :, t % page_size] = k[t]
        vc[order[t // page_size], :, t % page_size] = v[t]
    return kc, vc, order.to(torch.int32)[None].contiguous()


def _plain_headmix(q, k, v, scale, window, mix, gate):
    T_, H, D = q.shape
    G = k.shape[1]
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q.double(), k.double()[:, kv_of]) * scale
    s = s.masked_fill(~P.visible(T_, window if window else T_ + 1)[None], float("-inf"))
    w = torch.einsum("hg,gij->hij", mix.double(), torch.softmax(s, -1))
    return torch.einsum("hij,jhd->ihd", w, v.double()[:, kv_of]) * torch.sigmoid(gate.double())[:, :, None]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,window,T_", [(4, 2, 16, 5, 70), (3, 3, 24, 33, 100), (6, 1, 8, 1, 40), (8, 4, 64, 45, 130),
                                               (4, 4, 20, 0, 90), (2, 1, 64, 0, 1500)])
def test_head_mixed_attention_kernel(dtype, H, G, D, window, T_):
    """All rows of a sequence at once (a prompt), then the last rows one at a time against many keys (decoding: few
    rows, so long contexts are cut into spans), on shuffled pages."""
    from tandemllm_b200.kernels import ops
    from tandemllm_b200.parts.base import Runtime
    g = torch.Generator().manual_seed(H * 100 + D)
    dt = DT[dtype]
    q = torch.randn(T_, H, D, generator=g).to(dt)
    k = torch.randn(T_, G, D, generator=g).to(dt)
    v = torch.randn(T_, G, D, generator=g).to(dt)
    mix = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    gate = torch.randn(T_, H + 3, generator=g).to(dt)           # logits inside wider rows, as in the fused product
    want = _plain_headmix(q.float(), k.float(), v.float(), 0.37, window, mix, gate[:, :H].float())
    kc, vc, table = _paged(k, v, 16, seed=T_)
    dev = torch.device("cuda")
    rt = Runtime(dev, dt)
    kc, vc, table = kc.to(dev), vc.to(dev), table.to(dev)
    out = torch.empty(T_, H, D, dtype=dt, device=dev)
    pos = torch.arange(T_, dtype=torch.int32, device=dev)
    req = torch.zeros(T_, dtype=torch.int32, device=dev)
    gd = gate.to(dev)
    ops.attention_headmix(q.to(dev), kc, vc, table, 16, req, pos, 0.37, window, mix.to(dev), gd, gd.stride(0), out, T_, rt,
                          rt.status)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert int(rt.status.item()) == 0
    assert rel(out.float().view(T_, -1), want.reshape(T_, -1)) < tol
    last = 3
    out2 = torch.empty(last, H, D, dtype=dt, device=dev)
    ops.attention_headmix(q[-last:].to(dev).contiguous(), kc, vc, table, 16, req[:last], pos[-last:].contiguous(), 0.37, window,
                          mix.to(dev), gd[-last:], gd.stride(0), out2, T_, rt, rt.status)
    assert int(rt.status.item()) == 0
    assert rel(out2.float().view(last, -1), want[-last:].reshape(last, -1)) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,T_", [(37, 300), (0, 1100)])
def test_one_key_that_stands_out_far_back_and_at_the_windows_edge(dtype, window, T_):
    """The last row's query and one key are scaled so that this key takes all of the softmax if the row sees it. At
    distance window - 1 (or at position 0 without a window) the output is that key's value; one step further it is not
    seen at all and the output equals the one computed without it."""
    from tandemllm_b200.kernels import ops
    from tandemllm_b200.parts.base import Runtime
    H, G, D = 4, 2, 32
    dt, dev = DT[dtype], torch.device("cuda")
    rt = Runtime(dev, dt)
    g = torch.Generator().manual_seed(5)
    for distance in ([window - 1, window] if window else [T_ - 1]):
        q = torch.randn(T_, H, D, generator=g)
        k = torch.randn(T_, G, D, generator=g)
        v = torch.randn(T_, G, D, generator=g)
        j = T_ - 1 - distance
        direction = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
        q[-1] = 30 * direction
        k[j] = 30 * direction
        q, k, v = q.to(dt), k.to(dt), v.to(dt)
        mix = torch.eye(H)
        gate = torch.full((T_, H), 20.0).to(dt)                 # sigmoid = 1
        kc, vc, table = _paged(k, v, 16, seed=distance)
        out = torch.empty(1, H, D, dtype=dt, device=dev)
        ops.attention_headmix(q[-1:].to(dev).contiguous(), kc.to(dev), vc.to(dev), table.to(dev), 16,
                              torch.zeros(1, dtype=torch.int32, device=dev),
                              torch.tensor([T_ - 1], dtype=torch.int32, device=dev), 1.0, window, mix.to(dev), gate[-1:].to(dev),
                              H, out, T_, rt, rt.status)
        want = _plain_headmix(q.float(), k.float(), v.float(), 1.0, window, mix, gate.float())[-1]
        assert rel(out.float().view(1, -1), want.reshape(1, -1)) < (2e-5 if dtype == "float32" else 2e-2)
        seen = v.float()[j][torch.arange(H) // (H // G)]
        close = float((out.float().cpu()[0] - seen).abs().max())
        if distance < (window or T_):
            assert close < 2e-2, "the key that stands out was not seen"
        else:
            assert close > 0.3, "a key outside the window was seen"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unit_norm_and_keys_kept_as_values(dtype):
    """The q/k kernel with both flags: q and k at unit root mean square without a weight, the key as projected stored as
    the value, on the rows' pages."""
    from tandemllm_b200.kernels import ops
    from tandemllm_b200.parts.base import Runtime
    dt, dev = DT[dtype], torch.device("cuda")
    for H, G, D in [(4, 2, 64), (3, 1, 24), (5, 5, 128)]:
        rt = Runtime(dev, dt)
        g = torch.Generator().manual_seed(D)
        R, eps = 21, 1e-3
        width = (H + G) * D + 8
        qk = (3 * torch.randn(R, width, generator=g)).to(dt)
        kc = torch.zeros(4, G, 16, D, dtype=dt, device=dev)
        vc = torch.zeros_like(kc)
        table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=dev)
        pos = torch.arange(5, 5 + R, dtype=torch.int32, device=dev)
        q_out = torch.empty(R, H, D, dtype=dt, device=dev)
        ops.qk_prepare(qk.to(dev), None, None, eps, None, 0, pos, torch.zeros(R, dtype=torch.int32, device=dev), table, 16,
                       q_out, kc, vc, None, None, H, G, D, rt.status, ops.QK_UNIT_NORM | ops.QK_VALUES_ARE_KEYS)
        assert int(rt.status.item()) == 0
        qf = qk.double()[:, :H * D].view(R, H, D)
        kf = qk.double()[:, H * D:(H + G) * D].view(R, G, D)
        tol = 1e-5 if dtype == "float32" else 1e-2
        assert rel(q_out.float().view(R, -1), P.unit_rms(qf, eps).view(R, -1)) < tol
        for r in range(R):
            p = 5 + r
            page = int(table[0, p // 16])
            assert rel(kc[page, :, p % 16].float().reshape(1, -1), P.unit_rms(kf[r], eps).view(1, -1)) < tol
            assert torch.equal(vc[page, :, p % 16].cpu(), qk[r, H * D:(H + G) * D].view(G, D))


# ------------------------------------------------------------------------------------------ whole models
def run_schedule(engine, requests, schedule):
    """`schedule`: steps of [(request, count), ...]; every position's logits are wanted. Returns request -> logits."""
    from tandemllm_b200.engine import StepEntry
    at = {r: 0 for r in requests}
    got = {r: [] for r in requests}
    for step in schedule:
        entries = []
        for r, n in step:
            if not engine.cache.has(r):
                engine.admit(r)
            entries.append(StepEntry(r, requests[r][at[r]:at[r] + n], list(range(n))))
        logits = engine.step(entries).float().cpu()
        o = 0
        for r, n in step:
            got[r].append(logits[o:o + n])
            o += n
            at[r] += n
            if at[r] == len(requests[r]):
                engine.release(r)
    engine.cache.check()
    return {r: torch.cat(v) for r, v in got.items()}


def cuts(n, sizes):
    out, i = [], 0
    while n:
        c = min(n, sizes[i % len(sizes)])
        out.append(c)
        n -= c
        i += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["s1", "s2", "s3", "s4"])
def test_whole_prompts_decoding_and_portions_agree_with_the_plain_model(name, dtype, plain_logits):
    engine, cfg, W = engine_of(name, dtype)
    toks = S.tokens(name, 150, seed=3)
    want = plain_logits(name, toks)
    reqs = {"a": toks}
    whole = run_schedule(engine, reqs, [[("a", len(toks))]])["a"]
    assert rel(whole, want) < TOL[dtype]
    # the layers one by one on the way: the first tokens of a sequence alone
    first = run_schedule(engine, {"a": toks[:3]}, [[("a", 1)], [("a", 1)], [("a", 1)]])["a"]
    assert rel(first, want[:3]) < TOL[dtype]
    # most of it at once, then token by token across windows' and pages' edges
    decode = run_schedule(engine, reqs, [[("a", 60)]] + [[("a", 1)]] * 90)["a"]
    assert rel(decode, want) < TOL[dtype]
    # token by token from the very first
    every = run_schedule(engine, {"a": toks[:70]}, [[("a", 1)]] * 70)["a"]
    assert rel(every, want[:70]) < TOL[dtype]
    # portions of changing size, down to two tokens
    for sizes in ([2], [7, 2, 33, 3, 16, 5], [64, 2, 31]):
        got = run_schedule(engine, reqs, [[("a", c)] for c in cuts(len(toks), sizes)])["a"]
        assert rel(got, want) < TOL[dtype]
        # how the prompt was cut changes nothing beyond rounding
        assert rel(got, whole) < (2e-5 if dtype == "float32" else TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["s1", "s2", "s4"])
def test_unequal_requests_in_one_batch_on_pages_and_slots_that_are_used_again(name, dtype, plain_logits):
    """Seven requests of unequal length through four slots and a pool too small for all of them: portions beside
    single tokens, requests that pause, pages and slots that come back and are taken again."""
    lengths = [90, 5, 47, 130, 1, 33, 64]
    reqs = {f"q{i}": S.tokens(name, n, seed=10 + i) for i, n in enumerate(lengths)}
    engine, cfg, W = engine_of(name, dtype, pages=20, parallel=4)
    rng = np.random.default_rng(0)
    at = {r: 0 for r in reqs}
    waiting, live, schedule = list(reqs), [], []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        step = []
        for r in list(live):
            left = len(reqs[r]) - at[r]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            n = min(left, int(rng.choice([1, 1, 2, 3, 16, 29])))
            # the pool holds 20 pages of 16 tokens: a request never brings more than fits beside the others' windows
            step.append((r, n))
            at[r] += n
            if at[r] == len(reqs[r]):
                live.remove(r)
        if step:
            schedule.append(step)
    got = run_schedule(engine, reqs, schedule)
    for r, toks in reqs.items():
        assert rel(got[r], plain_logits(name, toks)) < TOL[dtype], r
    stats = engine.cache.stats()
    assert all(g["reused"] > 0 for g in stats["groups"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(dtype, plain_logits):
    name = "s1"
    engine, cfg, W = engine_of(name, dtype, pages=12)
    toks = S.tokens(name, 400, seed=8)
    got = run_schedule(engine, {"a": toks}, [[("a", 9)]] + [[("a", 1)]] * 391)["a"]
    assert rel(got, plain_logits(name, toks)) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype, tmp_path):
    """A folder on disk (config.json chooses the architecture), `Engine.generate`, several requests at once."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    name = "s2"
    folder = S.write_folder(str(tmp_path / "m"), name)
    engine = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=256, parallel=3, chunk_size=32, max_batched_tokens=64))
    assert engine.model.spec.architecture == "Sifupel"
    prompts = [S.tokens(name, n, seed=40 + n) for n in (70, 3, 21, 45)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    cfg, W = S.CONFIGS[name], S.weights(name, bf16_exact=True)
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        if dtype == "float32":
            assert out == P.greedy(cfg, W, prompt, 12)
        else:
            # bfloat16 may take another token where two logits are close: every token must be the plain model's choice
            # given the text so far, or within the precision's noise of it
            text = list(prompt)
            for t in out:
                row = P.forward(cfg, W, text)[-1]
                assert float(row.max() - row[t]) <= 3e-2 * float(row.abs().max())
                text.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_on_a_folder(dtype, tmp_path, plain_logits):
    name = "s3"
    folder = S.write_folder(str(tmp_path / "m"), name)
    toks = {"x": S.tokens(name, 40, seed=1), "y": S.tokens(name, 19, seed=2)}
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks["x"][:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks["x"][25:], "want": [14]},
                                     {"id": "y", "tokens": toks["y"], "want": [18]}], "end": ["x", "y"]},
             {"step": 2, "entries": [{"id": "z", "tokens": toks["y"][:2], "want": []}], "end": ["z"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                        str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    V = S.CONFIGS[name]["vocab"]
    a = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    b = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    wx, wy = plain_logits(name, toks["x"]), plain_logits(name, toks["y"])
    assert rel(a, wx[[0, 24]]) < TOL[dtype]
    assert rel(b, torch.stack([wx[39], wy[18]])) < TOL[dtype]
    assert not (out / "2.f32").exists()


@pytest.mark.parametrize("H,G,D,window,T_", [(8, 4, 64, 45, 150), (4, 1, 64, 0, 100), (16, 4, 64, 70, 120), (32, 8, 64, 33, 90),
                                               (24, 6, 64, 64, 110), (12, 4, 128, 50, 130), (10, 5, 128, 97, 140), (3, 3, 128, 1, 40)])
def test_head_mixed_attention_on_the_tensor_cores(H, G, D, window, T_):
    """The prompt kernel of the bfloat16 path at its own entry point: tiles of 16 rows and a last, shorter one, a second
    request that begins in the middle of a page's worth of rows, every number of heads a warp (1, 2, 4), windows' edges
    inside and across key tiles, on shuffled pages."""
    from tandemllm_b200.kernels import tensorcore
    from tandemllm_b200.parts.base import Runtime
    lib = tensorcore.lib()
    assert lib.tl_attention_headmix_mma_supported(H, G, D)
    dt, dev = torch.bfloat16, torch.device("cuda")
    rt = Runtime(dev, dt)
    g = torch.Generator().manual_seed(H + D + T_)
    q = torch.randn(T_, H, D, generator=g).to(dt)
    k = torch.randn(T_, G, D, generator=g).to(dt)
    v = torch.randn(T_, G, D, generator=g).to(dt)
    mix = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    gate = torch.randn(T_, H + 5, generator=g).to(dt)
    want = _plain_headmix(q.float(), k.float(), v.float(), 0.23, window, mix, gate[:, :H].float())
    kc, vc, table = _paged(k, v, 16, seed=T_ + 1)
    # the step brings the sequence's last rows only (the earlier keys are in the cache), cut into tiles of 16 rows
    first = 37
    rows = T_ - first
    tiles = torch.tensor([(0, r0, min(16, rows - r0)) for r0 in range(0, rows, 16)], dtype=torch.int32, device=dev)
    out = torch.zeros(rows, H, D, dtype=dt, device=dev)
    gd = gate[first:].contiguous().to(dev)
    qd, kd, vd, td, md = q[first:].contiguous().to(dev), kc.to(dev), vc.to(dev), table.to(dev), mix.to(dev)
    pos = torch.arange(first, T_, dtype=torch.int32, device=dev)
    code = lib.tl_attention_headmix_mma(
        qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), td.data_ptr(), td.shape[1], 16, kd.shape[0], tiles.data_ptr(),
        tiles.shape[0], pos.data_ptr(), 0.23, window, md.data_ptr(), gd.data_ptr(), gd.stride(0), out.data_ptr(), H, G, D,
        rt.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == 0
    torch.cuda.synchronize()
    assert int(rt.status.item()) == 0
    assert rel(out.float().view(rows, -1), want[first:].reshape(rows, -1)) < 2e-2


def test_the_activation_in_the_prompt_products_epilogue():
    """The ungated feed-forward's up product with xIELU applied to the 32-bit accumulator before it is rounded, against
    the plain activation of the plain product; a decode step's few rows are told to take the unfused way."""
    from tandemllm_b200.kernels import ops, tensorcore
    from tandemllm_b200.parts.base import Runtime
    dev = torch.device("cuda")
    rt = Runtime(dev, torch.bfloat16)
    tc = tensorcore.enable(rt)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(300, 136, generator=g).to(torch.bfloat16)
    w = (torch.randn(200, 136, generator=g) * 0.2).to(torch.bfloat16)
    pq = torch.tensor([0.3, -0.4])
    sp = torch.nn.functional.softplus(pq)
    got = tc.linear_act(x.to(dev), w.to(dev), ops.ACTIVATIONS["xielu"], float(sp[0]), float(0.5 + sp[1]))
    assert got is not None and int(rt.status.item()) == 0
    want = P.xielu(x.double() @ w.double().T, pq.double())
    assert rel(got.float(), want) < 1e-2
    assert tc.linear_act(x[:8].to(dev), w.to(dev), ops.ACTIVATIONS["xielu"], 1.0, 1.0) is None
