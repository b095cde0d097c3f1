"""Bevuvik on the device against the plain implementation (tests/plain_bevuvik.py): each mechanism
alone (with weights made so that a lost key, a window that is one token off or a lost state shows),
then whole models replayed through bin/trace_run (whole prompts, the last tokens one by one,
portions down to two tokens, mixed batches on a pool so small that pages and slots are used again),
then greedy generation through the engine's entry point and scheduler."""
import math
import os

import numpy as np
import pytest
import torch

import bevuvik_tools as bt
import plain_bevuvik as P
import trace_tools as tt

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, f32=2e-5, bf16=2.5e-2):
    err = float((got.double().cpu() - want.double()).abs().max() / want.abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16), f"relative error {err:.2e}"
    return err


def bf(t):
    """Values that are exact in bfloat16, as float64."""
    return t.to(torch.bfloat16).double()


@pytest.fixture(scope="module")
def kit(cuda_device):
    from gollmgo_b200 import parts
    from gollmgo_b200.cache import CacheManager
    from gollmgo_b200.csrc import ops
    from gollmgo_b200.engine.batch import BatchBuilder, StepEntry
    parts.set_matmul_precision()

    class Kit:
        pass
    k = Kit()
    k.parts, k.ops, k.CacheManager, k.BatchBuilder, k.StepEntry = parts, ops, CacheManager, BatchBuilder, StepEntry
    return k


def ctx_for(kit, dtype, page=16, max_tokens=640):
    return kit.parts.BuildContext(dtype, "cuda", max_tokens=max_tokens, max_seqs=8, page_size=page)


class MixerRun:
    """A mixer with a cache manager of its own: sequences are fed in portions, several a step."""

    def __init__(self, kit, mixer, dtype, page, pages=64, slots=4):
        self.kit, self.mixer, self.dtype = kit, mixer, dtype
        self.need = mixer.cache_need()
        self.cm = kit.CacheManager([self.need], page, pages, slots, dtype=dtype, device="cuda")
        self.bb = kit.BatchBuilder(self.cm, "cuda", query_tiles=getattr(mixer, "query_tiles", lambda: ())())

    def step(self, parts):
        """parts: {sequence: rows [n, width]} -> {sequence: output rows}"""
        for s in parts:
            if s not in self.cm.requests:
                self.cm.admit(s)
        batch = self.bb.build([self.kit.StepEntry(s, [0] * x.shape[0], []) for s, x in parts.items()])
        x = torch.cat(list(parts.values())).cuda().to(self.dtype).contiguous()
        y = self.mixer.forward(x, batch, self.cm.cache_view(0, self.need)).clone()
        out, at = {}, 0
        for s, rows in parts.items():
            out[s] = y[at:at + rows.shape[0]]
            at += rows.shape[0]
        return out

    def feed(self, x, cuts, seq="s", keep=False):
        outs, at = [], 0
        for c in cuts:
            outs.append(self.step({seq: x[at:at + c]})[seq])
            at += c
        assert at == x.shape[0]
        if not keep:
            self.cm.free(seq)
        return torch.cat(outs)


def cuts_of(n, sizes):
    out, at, i = [], 0, 0
    while at < n:
        c = min(sizes[i % len(sizes)], n - at)
        if n - at - c == 1:
            c += 1
        out.append(c)
        at += c
        i += 1
    return out


# ------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_gated_feed_forward(kit, dtype):
    """Gates above the limit and ups beyond it on both sides are cut; the up branch is shifted by one."""
    torch.manual_seed(0)
    D, F, T = 72, 100, 19
    f = {"kind": "dense", "ff": F, "limit": 0.9}
    ff = kit.parts.build_feed_forward(kit.parts.PartSpec("gated_mlp", {
        "hidden_size": D, "intermediate_size": F, "activation": "clamped_swish", "limit": 0.9, "names": ("gate", "up", "down")}),
        ctx_for(kit, dtype))
    w = {"gate": bf(torch.randn(F, D) * 0.3), "up": bf(torch.randn(F, D) * 0.3), "down": bf(torch.randn(D, F) / F ** 0.5)}
    ff.load(lambda n: w[n].cuda().to(dtype))
    x = bf(torch.randn(T, D))
    g, u = x @ w["gate"].T, x @ w["up"].T
    assert (g > 0.9).any() and (u > 0.9).any() and (u < -0.9).any()
    want = P.clamped_gated_ff(x, {"p.gate": w["gate"], "p.up": w["up"], "p.down": w["down"]}, "p.", f)
    close(ff.forward(x.cuda().to(dtype), None), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_branch_mix_and_scaled_add(kit, dtype):
    torch.manual_seed(1)
    T, W, eps = 11, 100, 1e-5
    ys = [bf(torch.randn(T, W) * s) for s in (0.3, 7.0, 1.0)]
    ws = [bf(1 + 0.3 * torch.randn(W)) for _ in ys]
    out = torch.empty(T, W, device="cuda", dtype=dtype)
    kit.ops.rms_mix([y.cuda().to(dtype) for y in ys], [w.float().cuda() for w in ws], 1 / 3, eps, out)
    close(out, sum(P.rms_norm(y, w, eps) for y, w in zip(ys, ws)) / 3, dtype, bf16=5e-3)
    resid0 = torch.randn(T, W)
    for b in (ys[2], None):
        resid = resid0.clone().cuda()
        kit.ops.scaled_add(resid, ys[0].cuda().to(dtype), None if b is None else b.cuda().to(dtype), 0.7)
        close(resid, resid0.double() + 0.7 * (ys[0] + (b if b is not None else 0)), torch.float32, f32=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 2, 16, 1, 24, 8, True, True), (4, 4, 32, 2, 40, 32, False, False),
                                   (2, 1, 12, 1, 12, 6, False, True), (5, 5, 20, 5, 20, 0, True, False)])
def test_rotation_bias_and_cache_write(kit, dtype, shape):
    """The kernel that adds the bias, rotates part of every q and k head (adjacent pairs or halves,
    cosines and sines scaled) and scatters k and v into caches of different shapes."""
    nh, nkv, d, nv, dv, rot_dims, interleaved, bias = shape
    torch.manual_seed(2)
    T, page, pages = 37, 8, 9
    width = (nh + nkv) * d + nv * dv
    x = bf(torch.randn(T, width))
    b = bf(torch.randn(width) * 0.5) if bias else None
    rot = {"dims": rot_dims, "base": 1000.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 0.5}} if rot_dims else None
    pos = torch.randint(0, 3000, (T,), dtype=torch.int32)
    slots = torch.randperm(page * pages)[:T].to(torch.int32)
    slots[5] = -1
    qkv = x.cuda().to(dtype)
    kc = torch.zeros(pages, nkv, page, d, device="cuda", dtype=dtype)
    vc = torch.zeros(pages, nv, page, dv, device="cuda", dtype=dtype)
    table, mag = None, 1.0
    if rot:
        f, mag = P.rotary_frequencies(rot)
        table = f.cuda()
    kit.ops.rope_kv_write_x(qkv, pos.cuda(), slots.cuda(), table, mag, None if b is None else b.float().cuda(),
                            kc, vc, nh, nkv, d, nv, dv, page, interleaved, True)
    xb = x + (b if bias else 0)
    q, k = xb[:, :nh * d].view(T, nh, d), xb[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = xb[:, (nh + nkv) * d:].view(T, nv, dv)
    if rot:
        q, k = P.rotate(q, pos, rot, interleaved), P.rotate(k, pos, rot, interleaved)
    close(qkv[:, :nh * d], q.reshape(T, -1), dtype, bf16=8e-3)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        close(kc[s // page, :, s % page], k[t], dtype, bf16=8e-3)
        close(vc[s // page, :, s % page], v[t], dtype, bf16=8e-3)
    assert int((kc != 0).any(-1).sum()) == (T - 1) * nkv          # the token without a slot wrote nothing


# ------------------------------------------------------------------ softmax attention with capped scores
def tagged(D, heads, d, scale, n_tags, tag_dim0, seed, boost=24.0):
    """Query and key weights [heads * d, D] under which one score can be made to stand out: the last
    2 * n_tags input channels are tags.  Key tag t lands on dimension tag_dim0 + t of every key head,
    query tag t on the same dimension of every query head with a large weight; a token with key tag t
    set is then the one key that a token with query tag t set looks at.  Other channels are random."""
    g = torch.Generator().manual_seed(seed)
    C = D - 2 * n_tags
    q = torch.zeros(heads, d, D)
    k = torch.zeros(heads, d, D)
    free = [i for i in range(d) if not (tag_dim0 <= i < tag_dim0 + n_tags)]
    q[:, free, :C] = torch.randn(heads, len(free), C, generator=g) / C ** 0.5
    k[:, free, :C] = torch.randn(heads, len(free), C, generator=g) / C ** 0.5
    for t in range(n_tags):
        q[:, tag_dim0 + t, C + n_tags + t] = boost / scale
        k[:, tag_dim0 + t, C + t] = 1.0
    return q.reshape(heads * d, D), k.reshape(heads * d, D)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(96, 4, 2, 32, 16, 16, 20.0, 16), (128, 6, 1, 24, 40, 0, 0.0, 8),
                                   (160, 4, 4, 128, 128, 64, 30.0, 32), (104, 3, 3, 20, 12, 8, 12.0, 16),
                                   (160, 4, 2, 128, 64, 32, 25.0, 16), (128, 4, 1, 64, 64, 16, 14.0, 8),
                                   (128, 34, 1, 64, 128, 0, 0.0, 16)])
def test_capped_attention_finds_one_key_among_hundreds(kit, dtype, shape):
    """Queries made to pick out single keys: the very first tokens, keys at both sides of page
    borders, keys hundreds of tokens back, a key that was itself decoded; asked for from prompt
    portions of several sizes (down to two tokens) and from single decoded tokens.  Values of another
    size than keys, rotation of part of the head, capped scores (the cap is below the boosted score)."""
    D, H, G, d, dv, rot_dims, cap, page = shape
    scale = 1.2 / math.sqrt(d)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale}
    if cap:
        m["softcap"] = cap
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": 50000.0}
    TAGS = 8
    pos = kit.parts.PartSpec("rope", {"head_dim": d, "rotary_dim": rot_dims, "theta": 50000.0, "scaling": None}) \
        if rot_dims else kit.parts.PartSpec("none")
    mixer = kit.parts.build_mixer(kit.parts.PartSpec("attention", {
        "hidden_size": D, "num_heads": H, "num_kv_heads": G, "head_dim": d, "v_head_dim": dv, "window": None,
        "position": pos, "scale": scale, "softcap": cap or None, "names": ("q", "k", "v", "o")}), ctx_for(kit, dtype, page))
    g = torch.Generator().manual_seed(5)
    wq, _ = tagged(D, H, d, scale, TAGS, rot_dims, 6, boost=18.0 if cap else 24.0)
    _, wk = tagged(D, G, d, scale, TAGS, rot_dims, 7)
    w = {"q": bf(wq), "k": bf(wk), "v": bf(torch.randn(G * dv, D, generator=g) / D ** 0.5),
         "o": bf(torch.randn(D, H * dv, generator=g) / (H * dv) ** 0.5)}
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    n, C = 420, D - 2 * TAGS
    x = torch.zeros(n, D)
    x[:, :C] = torch.randn(n, C, generator=g)
    keys = [0, 1, page - 1, page, 2 * page - 1, 2 * page, 5 * page - 1, 400]
    for t, k in enumerate(keys):
        x[k, C + t] = 8.0
    queries = {150: 0, 151: 1, 152: 2, 153: 3, 154: 4, 155: 5, 300: 0, 301: 6, 401: 0, 402: 3, 403: 6, 404: 7,
               410: 1, 419: 4, 418: 7, 405: 2}
    for qi, t in queries.items():
        x[qi, C + TAGS + t] = 1.0
    x = bf(x)
    pw = {"p." + k: v for k, v in w.items()}
    # such a query puts nearly all its weight on its key
    qq, kk = (x @ w["q"].T).view(n, H, d), (x @ w["k"].T).view(n, G, d)
    if rot_dims:
        qq, kk = P.rotate(qq, torch.arange(n), m["rot"], False), P.rotate(kk, torch.arange(n), m["rot"], False)
    for qi, t in queries.items():
        sc = torch.einsum("hd,jhd->hj", qq[qi], kk[:qi + 1].repeat_interleave(H // G, 1)) * scale
        if cap:
            sc = cap * torch.tanh(sc / cap)
        assert float(torch.softmax(sc, -1)[:, keys[t]].min()) > 0.98, (qi, keys[t])
    want = P.capped_attention(x, pw, "p.", m)
    run = MixerRun(kit, mixer, dtype, page)
    cuts = [130, 2, 17, 3, 64, 100, 2, 82] + [1] * 20
    close(run.feed(x, cuts, "a"), want, dtype)
    close(run.feed(x, [n], "b"), want, dtype)


# ------------------------------------------------------------------ differential attention
def diff_weights(D, H, G, d, dv, scale, rot_dims, seed, tags=8):
    """Map 1 of every head carries tags 0..tags/2-1, map 2 the rest: a fault in either map shows."""
    g = torch.Generator().manual_seed(seed)
    half = tags // 2
    q1, k1 = tagged(D, H, d, scale, tags, rot_dims, seed + 1)
    q2, k2 = tagged(D, H, d, scale, tags, rot_dims, seed + 2)
    C = D - 2 * tags
    # map 1 answers only to the first half of the tags, map 2 to the second half
    q1.view(H, d, D)[:, rot_dims + half:rot_dims + tags] = 0
    q2.view(H, d, D)[:, rot_dims:rot_dims + half] = 0
    q = torch.stack([q1.view(H, d, D), q2.view(H, d, D)], 1).reshape(H * 2 * d, D)
    kk1, kk2 = k1.view(H, d, D)[:G], k2.view(H, d, D)[:G]
    k = torch.stack([kk1, kk2], 1).reshape(G * 2 * d, D)
    w = {"q": q, "k": k, "v": torch.randn(G * dv, D, generator=g) / D ** 0.5,
         "o": torch.randn(D, H * dv, generator=g) / (H * dv) ** 0.5,
         "q.b": 0.1 * torch.randn(H * 2 * d, generator=g), "k.b": 0.1 * torch.randn(G * 2 * d, generator=g),
         "v.b": 0.3 * torch.randn(G * dv, generator=g), "o.b": 0.3 * torch.randn(D, generator=g)}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        w[n] = 0.4 * torch.randn(d, generator=g)
    return {k: bf(v) for k, v in w.items()}


def diff_mixer(kit, dtype, D, m, page, eps, max_tokens=640):
    rot = m.get("rot")
    pos = kit.parts.PartSpec("none")
    if rot:
        from gollmgo_b200.parts.position import YarnScaling
        sc = rot.get("scaling")
        pos = kit.parts.PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"],
                                          "interleaved": True,
                                          "scaling": YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None})
    return kit.parts.build_mixer(kit.parts.PartSpec("diff_attention", {
        "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "v_head_dim": m["vdim"], "window": (m.get("mask") or {}).get("size"), "position": pos, "scale": m["scale"],
        "diff": m["diff"], "eps": eps, "biases": True, "names": ("q", "k", "v", "o")}), ctx_for(kit, dtype, page, max_tokens))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(96, 4, 2, 24, 16, 8, 70, 16), (128, 2, 2, 32, 48, 16, 33, 8), (112, 6, 1, 16, 24, 0, 129, 32),
                                   (160, 2, 1, 64, 128, 32, 64, 16)])
def test_differential_attention_at_the_windows_edge(kit, dtype, shape):
    """Keys just inside and just outside the window of a query, for queries in prompt portions and
    for single decoded tokens, with keys at page borders and among the first tokens: a query whose key
    is the oldest one it may see puts nearly all weight of one map on it; one token later the key is
    gone and the map falls back on the others.  A window that is one token off changes the row wholesale."""
    D, H, G, d, dv, rot_dims, W, page = shape
    scale, eps, TAGS = 1.1 / math.sqrt(d), 1e-5, 8
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale, "diff": 0.25, "mask": {"size": W}}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": 10000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 0.5}}
    mixer = diff_mixer(kit, dtype, D, m, page, eps)
    w = diff_weights(D, H, G, d, dv, scale, rot_dims, seed=11)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    n, C = 3 * W + 150, D - 2 * TAGS
    g = torch.Generator().manual_seed(12)
    x = torch.zeros(n, D)
    x[:, :C] = torch.randn(n, C, generator=g)
    # key tag t at position k; queries at k + W - 1 (the last that sees it) and k + W (the first that does not)
    keys = [0, 1, page - 1, page, W + 3, 2 * W + 7, 2 * W + 40, 3 * W + 20]
    queries = []                                  # (query, tag); a query may carry two tags
    for t, k in enumerate(keys):
        x[k, C + t] = 8.0
        queries += [(qi, t) for qi in (k + 1, k + W - 1, k + W) if qi < n]
    for qi, t in queries:
        x[qi, C + TAGS + t] += 1.0
    assert sum(qi in (keys[4] + W - 1, keys[4] + W) for qi, _ in queries) == 2      # those two carry one tag each
    x = bf(x)
    pw = {"p." + k: v for k, v in w.items()}
    want = P.differential_attention(x, pw, "p.", m, eps)
    # the rows just inside differ clearly from what they would be without their key: the test has teeth
    x_nokey = x.clone()
    x_nokey[keys[4], C + 4] = 0
    other = P.differential_attention(x_nokey, pw, "p.", m, eps)
    inside, outside = keys[4] + W - 1, keys[4] + W
    assert float((want[inside] - other[inside]).abs().max()) > 0.05 * float(want[inside].abs().max())
    torch.testing.assert_close(want[outside], other[outside], rtol=0, atol=1e-9)
    run = MixerRun(kit, mixer, dtype, page, pages=4 * (W // page + 8))
    first = 2 * W + 35
    cuts = cuts_of(first, [W - 1, 2, 17, 3, page, 2, 50]) + [1] * (n - first)       # the later queries are decoded alone
    close(run.feed(x, cuts, "a", keep=True), want, dtype)
    # the windowed group gave pages back as the window passed
    held = [p for p in run.cm.block_table("a", 0) if p >= 0]
    assert len(held) <= W // page + 2 < len(run.cm.block_table("a", 0))
    run.cm.free("a")
    close(run.feed(x, [n], "b"), want, dtype)                                         # all queries inside one portion
    close(run.feed(x, cuts_of(n, [2, 5, W, 3, W + 1]), "c"), want, dtype)


# ------------------------------------------------------------------ gated delta rule
def delta_weights(D, H, G, d, dv, taps, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)

    def conv(c):
        t = r(c, taps) / taps
        t[:, -1] += 1.0
        return t
    w = {"q": r(G * d, D) / D ** 0.5, "k": r(G * d, D) / D ** 0.5, "v": r(H * dv, D) / D ** 0.5, "g": r(H * dv, D) / D ** 0.5,
         "b": r(H, D) / D ** 0.5, "a": r(H, D) / D ** 0.5, "A_log": r(H) - 1.5, "dt_bias": 0.5 * r(H),
         "norm": 1 + 0.2 * r(dv), "o": r(D, H * dv) / (H * dv) ** 0.5,
         "q.conv": conv(G * d), "k.conv": conv(G * d), "v.conv": conv(H * dv)}
    return {k: bf(v) for k, v in w.items()}


def delta_mixer(kit, dtype, D, m, eps, page=16):
    return kit.parts.build_mixer(kit.parts.PartSpec("gated_delta", {
        "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "v_head_dim": m["vdim"], "conv": m["conv"], "eps": eps}), ctx_for(kit, dtype, page))


DELTA_SHAPES = [(64, 4, 2, 16, 24, 3), (96, 3, 3, 32, 32, 2), (100, 6, 2, 20, 36, 5), (128, 2, 1, 128, 128, 4),
                (72, 2, 2, 8, 40, 1), (80, 1, 1, 200, 16, 4)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", DELTA_SHAPES)
def test_gated_delta_rule_in_portions_and_token_by_token(kit, dtype, shape):
    """The whole sequence in one step, in portions of several sizes down to two tokens (shorter than
    the convolution's window), and token by token, two sequences beside each other: the state matrix
    and the convolution's last inputs carry over in the request's slot."""
    D, H, G, d, dv, taps = shape
    eps = 1e-5
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    mixer = delta_mixer(kit, dtype, D, m, eps)
    w = delta_weights(D, H, G, d, dv, taps, seed=21)
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    g = torch.Generator().manual_seed(22)
    xa, xb = bf(torch.randn(75, D, generator=g)), bf(torch.randn(41, D, generator=g))
    pw = {"p." + k: v for k, v in w.items()}
    wa, wb = P.gated_delta_rule(xa, pw, "p.", m, eps), P.gated_delta_rule(xb, pw, "p.", m, eps)
    tol = dict(f32=1e-4, bf16=3e-2)
    run = MixerRun(kit, mixer, dtype, 16)
    close(run.feed(xa, [75], "whole"), wa, dtype, **tol)
    close(run.feed(xa, cuts_of(75, [2, 3, 2, 17, 5, 2, 30]), "cut"), wa, dtype, **tol)
    close(run.feed(xa, [1] * 75, "single"), wa, dtype, **tol)
    # two sequences in the same steps, unequal portions, one sitting steps out
    outs = {"a": [], "b": []}
    plan = [{"a": (0, 9), "b": (0, 2)}, {"a": (9, 10)}, {"b": (2, 19), "a": (10, 11)}, {"a": (11, 12), "b": (19, 20)},
            {"a": (12, 60), "b": (20, 41)}, {"a": (60, 75)}]
    run2 = MixerRun(kit, mixer, dtype, 16)
    for step in plan:
        got = run2.step({s: (xa if s == "a" else xb)[lo:hi] for s, (lo, hi) in step.items()})
        for s in step:
            outs[s].append(got[s])
    close(torch.cat(outs["a"]), wa, dtype, **tol)
    close(torch.cat(outs["b"]), wb, dtype, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_delta_rule_remembers_far_back_and_slots_start_clean(kit, dtype):
    """A head that barely decays keeps a value written hundreds of tokens ago: with weights made so,
    the read-out at the end is that value.  Then the slot is given back and used by another request,
    which must see none of it, also when its first portion is a single token."""
    D, H, G, d, dv, taps, eps = 64, 2, 1, 16, 16, 3, 1e-5
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    mixer = delta_mixer(kit, dtype, D, m, eps)
    w = delta_weights(D, H, G, d, dv, taps, seed=23)
    w["A_log"] = bf(torch.tensor([-9.0, 0.5]))                 # head 0 all but never forgets, head 1 forgets fast
    mixer.load(lambda n: w[n].cuda().to(dtype))
    pw = {"p." + k: v for k, v in w.items()}
    g = torch.Generator().manual_seed(24)
    x = bf(torch.randn(400, D, generator=g) * 0.3)
    x[3] = bf(torch.randn(D, generator=g) * 4)                  # one loud token early on
    x2 = x.clone()
    x2[3] = bf(torch.randn(D, generator=g) * 4)
    want, want2 = P.gated_delta_rule(x, pw, "p.", m, eps), P.gated_delta_rule(x2, pw, "p.", m, eps)
    assert float((want[399] - want2[399]).abs().max()) > 0.02 * float(want[399].abs().max())     # token 3 still matters at 399
    run = MixerRun(kit, mixer, dtype, 16, slots=1)
    close(run.feed(x, cuts_of(380, [64, 2, 100, 7]) + [1] * 20, "first"), want, dtype, f32=1e-4, bf16=3e-2)
    y = bf(torch.randn(30, D, generator=g))
    close(run.feed(y, [1, 2, 27], "second", keep=True), P.gated_delta_rule(y, pw, "p.", m, eps), dtype, f32=1e-4, bf16=3e-2)
    assert run.cm.state_slot("second") == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_mixer(kit, dtype):
    """Both branches read the same rows; each result is RMS-normed with its own weight; half the sum."""
    cfg, page = bt.get("bev_c")
    D, eps = cfg["width"], cfg["norm"]["eps"]
    m = cfg["layers"][0]["mixer"]
    from gollmgo_b200.architectures.bevuvik import bevuvik_spec
    from gollmgo_b200.config.bevuvik_config import BevuvikConfig
    spec = bevuvik_spec(BevuvikConfig.from_dict(cfg)).layers[0].mixer
    mixer = kit.parts.build_mixer(spec, ctx_for(kit, dtype, page))
    w = {k[len("l0.mix."):]: v for k, v in bt.random_weights(cfg, 25).items() if k.startswith("l0.mix.")}
    assert set(mixer.weights()) == set(w)
    mixer.load(lambda n: w[n].cuda().to(dtype))
    x = bf(torch.randn(90, D, generator=torch.Generator().manual_seed(26)))
    want = P.parallel_mixer(x, {"p." + k: v.double() for k, v in w.items()}, "p.", m, eps)
    run = MixerRun(kit, mixer, dtype, page)
    close(run.feed(x, [90], "a"), want, dtype, f32=1e-4, bf16=3e-2)
    close(run.feed(x, cuts_of(70, [33, 2, 9]) + [1] * 20, "b"), want, dtype, f32=1e-4, bf16=3e-2)


# ------------------------------------------------------------------ whole models through bin/trace_run
LENGTHS = {"bev_a": [1, 5, 37, 70, 130, 96], "bev_b": [2, 64, 65, 131, 200, 33], "bev_c": [3, 66, 40, 150, 97, 129],
           "bev_d": [4, 17, 250, 33, 65, 120]}
# float32: every row to a few units of rounding.  bfloat16: nine rows in ten within 4 % of the row's largest
# logit and none further off than what a lost key or state would cause (such a row is off by its whole size).
TOL = {"float32": (5e-5, 5e-5), "bfloat16": (4e-2, 0.15)}


def compare(trace, out_dir, reference, vocab, dtype):
    errs = []
    for step, exp in trace.expect.items():
        path = os.path.join(out_dir, f"{step}.f32")
        assert os.path.exists(path), f"step {step} wrote no file"
        got = np.fromfile(path, dtype="<f4").reshape(-1, vocab)
        assert got.shape[0] == len(exp), f"step {step}: {got.shape[0]} rows, expected {len(exp)}"
        for row, (name, pos) in zip(got, exp):
            ref = reference[name][pos].numpy()
            assert np.isfinite(row).all(), f"step {step} {name}@{pos}: non-finite logits"
            errs.append((float(np.abs(row - ref).max() / max(np.abs(ref).max(), 1e-6)), step, name, pos))
    most, worst = TOL[dtype]
    p90 = float(np.percentile([e[0] for e in errs], 90))
    top = max(errs)
    assert p90 <= most, f"90th percentile of the rows' errors is {p90:.3e}"
    assert top[0] <= worst, f"worst relative error {top[0]:.3e} at (step, request, position) {top[1:]}"
    return p90, top[0]


def plain_logits(cfg, weights, requests):
    w = {k: v.double() for k, v in weights.items()}
    return {name: P.forward(w, cfg, toks).float() for name, toks in requests.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(bt.TINY))
def test_replay_matches_plain(tmp_path, cuda_device, name, dtype):
    cfg, page = bt.get(name)
    weights = bt.random_weights(cfg, seed=31)
    model_dir = bt.model_folder(tmp_path, name, cfg, weights)
    requests = tt.random_requests(cfg["vocab"], LENGTHS[name], seed=5)
    reference = plain_logits(cfg, weights, requests)
    trace = tt.Trace()
    tt.whole(trace, requests)
    tt.tail_decode(trace, requests, tail=48)
    tt.portions(trace, requests)
    tt.mixed(trace, requests, max_live=4, seed=3)
    tt.mixed(trace, dict(reversed(list(requests.items()))), max_live=3, seed=4, tag="n")
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page)
    p90, worst = compare(trace, out, reference, cfg["vocab"], dtype)
    pool, asked, shared = tt.pages_were_used_again(trace, out + "/pages.jsonl", page)
    print(f"{name} {dtype}: {len(trace.steps)} steps, {pool} pages for {asked} asked, {shared} held by several, "
          f"errors: 90 % within {p90:.2e}, worst {worst:.2e}")


@pytest.mark.parametrize("name,dtype", [("bev_a", "bfloat16"), ("bev_b", "float32"), ("bev_c", "bfloat16")])
def test_pages_given_back_are_never_read(tmp_path, cuda_device, name, dtype):
    """The mixed trace with every page overwritten by NaN the moment it is given back (the windowed
    layers give pages back all the time)."""
    cfg, page = bt.get(name)
    weights = bt.random_weights(cfg, seed=32)
    model_dir = bt.model_folder(tmp_path, name, cfg, weights)
    requests = tt.random_requests(cfg["vocab"], LENGTHS[name], seed=6)
    reference = plain_logits(cfg, weights, requests)
    trace = tt.Trace()
    tt.mixed(trace, requests, max_live=4, seed=7)
    tt.portions(trace, requests)
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page, env=dict(os.environ, GOLLMGO_B200_POISON_FREED="1"))
    compare(trace, out, reference, cfg["vocab"], dtype)
    tt.pages_were_used_again(trace, out + "/pages.jsonl", page)


# ------------------------------------------------------------------ the entry point
def plain_greedy(cfg, weights, prompt, n):
    w = {k: v.double() for k, v in weights.items()}
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(P.forward(w, cfg, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_engine(tmp_path, cuda_device):
    """Requests of unequal length through Engine.generate (scheduler, chunked prompts, captured
    decode steps, the device's arg-max): the plain implementation's tokens, alone and together."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = bt.get("bev_a")
    weights = bt.random_weights(cfg, seed=33)
    d = bt.model_folder(tmp_path, "bev_a", cfg, weights)
    prompts = list(tt.random_requests(cfg["vocab"], [1, 9, 40, 23], seed=8).values())
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=24, max_batch_size=4, max_token_budget=32,
                 prefill_chunk_size=16)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    want = [plain_greedy(cfg, weights, pr, 12) for pr in prompts]
    assert [o.token_ids for o in outs] == want
    assert eng.generate([prompts[2]], SamplingParams(max_tokens=12, ignore_eos=True))[0].token_ids == want[2]
    eng.runner.cache.audit()
    assert eng.runner.cache.min_free_pages() == 24
    assert eng.runner.cache.slots.num_free == eng.runner.cache.slots.max_requests


def test_long_decoding_in_bfloat16_stays_near_the_plain_choice(tmp_path, cuda_device):
    """200 decoded tokens, past the window and over many pages, through captured decode steps: the tokens
    are (nearly) the plain implementation's best given the same history."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = bt.get("bev_b")
    weights = bt.random_weights(cfg, seed=34)
    d = bt.model_folder(tmp_path, "bev_b", cfg, weights)
    prompt = tt.random_requests(cfg["vocab"], [11], seed=9)["r0"]
    eng = Engine(d, dtype="bfloat16", block_size=page, num_blocks=40, max_batch_size=2, max_token_budget=64)
    toks = eng.generate([prompt], SamplingParams(max_tokens=200, ignore_eos=True))[0].token_ids
    assert len(toks) == 200
    logits = P.forward({k: v.double() for k, v in weights.items()}, cfg, prompt + toks)
    near = sum(float(row.max() - row[tok]) <= 0.06 * float(row.abs().max())
               for tok, row in zip(toks, logits[len(prompt) - 1:]))
    assert near >= 190, f"only {near} of 200 tokens are near the plain choice"
    assert eng.runner.cache.min_free_pages() == 40


def test_command_line_generates(tmp_path, cuda_device):
    import json
    import subprocess
    import sys
    cfg, page = bt.get("bev_c")
    weights = bt.random_weights(cfg, seed=35)
    d = bt.model_folder(tmp_path, "bev_c", cfg, weights)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "gollmgo_b200", "generate", "--model", d, "--dtype", "float32",
                        "--block-size", str(page), "--num-blocks", "16", "--max-batch-size", "4", "--max-token-budget", "64",
                        "--log-level", "error", "--prompt-ids", "5,6,7", "--prompt-ids", "9", "--max-tokens", "5", "--ignore-eos"],
                       capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    lines = [json.loads(l) for l in p.stdout.strip().splitlines()]
    assert lines[0]["token_ids"] == plain_greedy(cfg, weights, [5, 6, 7], 5)
    assert lines[1]["token_ids"] == plain_greedy(cfg, weights, [9], 5)
