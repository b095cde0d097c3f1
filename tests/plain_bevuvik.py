"""A plain, slow implementation of the Bevuvik decoder: float64, whole sequences, no cache,
one function per mechanism, written from the design's equations.  It shares no code with
the package and is what the package's kernels are compared with.

``w`` is a dict name -> float64 tensor, ``cfg`` the dict of config.json.
"""
import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


# ------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    """Per pair i < dims/2: (frequency, factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):            # the pair index whose wave makes `turns` turns over the original length
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, interleaved):
    """x [T, heads, d]: the first rot.dims values of every head are rotated; pairs are
    (2i, 2i+1) if interleaved, else (i, i + dims/2)."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions.to(F)[:, None] * f[None, :]            # [T, dims/2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        h = dims // 2
        u, v = x[..., :h], x[..., h:dims]
        out[..., :h] = u * c - v * s
        out[..., h:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------ softmax attention
def softmax_attention(q, k, v, scale, window=None, softcap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; head h reads kv head h // (H/G);
    token i sees j <= i, and with a window only i - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    out = torch.empty(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~ok, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // rep]
    return out


def differential_attention(h, w, p, m, eps):
    """The 'attention' mixer.  h [T, width]; w names under prefix p; m = the mixer's config."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate(q.reshape(T, 2 * H, d), pos, rot, True).view(T, H, 2, d)
        k = rotate(k.reshape(T, 2 * G, d), pos, rot, True).view(T, G, 2, d)
    window = (m.get("mask") or {}).get("size")
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], window)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], window)
    diff = float(m["diff"])
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + diff
    o = a1 - lam * a2
    o = rms(o, eps) * (1.0 - diff)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def capped_attention(h, w, p, m):
    """The left branch of the 'parallel' mixer: grouped-query attention with rotate-half
    positions on part of the head and tanh-capped scores."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    pos = torch.arange(T)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"], False), rotate(k, pos, m["rot"], False)
    a = softmax_attention(q, k, v, m["scale"], None, m.get("softcap"))
    return a.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ gated delta rule
def short_convolution(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] * x_{t - (taps-1) + j}, zeros before 0."""
    T, C = x.shape
    taps = taps_w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + xp[j:j + T] * taps_w[:, j]
    return y


def gated_delta_rule(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                     # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).view(T, H, dv)
    out = torch.empty(T, H, dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, hd] = S.T @ qt
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = capped_attention(h, w, p + "left.", m["left"])
    right = gated_delta_rule(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ------------------------------------------------------------------ feed-forward, layer, model
def clamped_gated_ff(h, w, p, f):
    lim = float(f["limit"])
    g = torch.clamp(h @ w[p + "gate"].T, max=lim)
    u = torch.clamp(h @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def layer(x, w, cfg, i):
    lc = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    if lc["type"] == "attention":
        y = differential_attention(h, w, p + "mix.", lc["mixer"], eps)
    elif lc["type"] == "parallel":
        y = parallel_mixer(h, w, p + "mix.", lc["mixer"], eps)
    else:
        raise ValueError(lc["type"])
    if lc.get("mlp"):
        y = y + clamped_gated_ff(h, w, p + "mlp.", lc["mlp"])
    return x + float(cfg.get("residual_mult", 1.0)) * y


def layer_runs(cfg):
    """The layers in the order they run, with a mark on the first of each pass of the loop."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(w, cfg, tokens, streams=None):
    """Logits [T, vocab]; ``streams`` (a list) receives the residual stream after every layer run."""
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x0 = x
    for i, first_of_pass in layer_runs(cfg):
        if first_of_pass:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        x = layer(x, w, cfg, i)
        if streams is not None:
            streams.append(x)
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T
