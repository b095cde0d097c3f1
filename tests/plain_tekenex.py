"""A plain, slow Tekenex for the tests: one function per mechanism, written from the design's
equations in float64 (or any dtype given), whole sequences at once, no cache, no batching.
It shares no code with the package.

Notation: x [n, D] is the residual stream of one sequence of n tokens, W matrices are stored
[out, in] and applied as x @ W.T, ``p`` is a dict of the checkpoint's tensors by name.
"""
import math

import torch


def layer_norm(y, w, b, eps):
    mu = y.mean(-1, keepdim=True)
    var = ((y - mu) ** 2).mean(-1, keepdim=True)
    return (y - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(y, w, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def latent_attention(h, p, pre, heads, dim, vdim, rank, scale, eps):
    """Causal softmax attention whose keys and values are expanded from one latent row per token;
    a sigmoid gate per head on the output.  No position encoding."""
    n = h.shape[0]
    q = (h @ p[pre + "q"].T).view(n, heads, dim)
    c = rms_norm(h @ p[pre + "dkv"].T, p[pre + "dkv.norm"], eps)            # [n, rank]: all that a cache keeps
    k = (c @ p[pre + "uk"].T).view(n, heads, dim)
    v = (c @ p[pre + "uv"].T).view(n, heads, vdim)
    gate = torch.sigmoid(h @ p[pre + "g"].T)                                 # [n, heads]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhe->ihe", a, v) * gate[:, :, None]
    return o.reshape(n, heads * vdim) @ p[pre + "o"].T


def dense_ff(h, p, pre):
    return (torch.relu(h @ p[pre + "up"].T) ** 2) @ p[pre + "down"].T


def gated_expert(h, p, pre):
    g = h @ p[pre + "gate"].T
    return (g * torch.sigmoid(g) * (h @ p[pre + "up"].T)) @ p[pre + "down"].T


def route(h, p, pre, top):
    """(chosen experts [n, top], their weights [n, top]): the largest logits, softmax over those alone."""
    z = h @ p[pre + "router"].T + p[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def route_gap(h, p, pre, top):
    """Per token, how far the last chosen logit lies above the first one left out, as a share of
    the largest logit's size: a small gap is a choice that rounding can turn."""
    z = h @ p[pre + "router"].T + p[pre + "router.b"]
    if top >= z.shape[-1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    val = torch.topk(z, top + 1, dim=-1).values
    return (val[:, top - 1] - val[:, top]) / z.abs().max(-1).values


def moe_ff(h, p, pre, experts, top, shared, gaps=None):
    idx, w = route(h, p, pre, top)
    if gaps is not None:
        gaps.append(route_gap(h, p, pre, top))
    out = torch.zeros(h.shape[0], p[pre + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(experts):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero()[:, 0]             # the tokens whose j-th choice is expert e
            if rows.numel():
                out[rows] += w[rows, j, None] * gated_expert(h[rows], p, f"{pre}e{e}.")
    if shared:
        out = out + gated_expert(h, p, pre + "shared.")
    return out


def layer(x, p, i, lc, eps, gaps=None):
    pre = f"l{i}."
    m = lc["mixer"]
    if lc["type"] != "latent_attention":
        raise ValueError(lc["type"])
    y = latent_attention(x, p, pre + "mix.", m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["scale"], eps)
    x = x + p[pre + "ls1"] * layer_norm(y, p[pre + "norm1"], p[pre + "norm1.b"], eps)
    f = lc.get("mlp")
    if f is None:
        return x
    if f["kind"] == "dense":
        y = dense_ff(x, p, pre + "mlp.")
    elif f["kind"] == "moe":
        y = moe_ff(x, p, pre + "mlp.", f["router"]["experts"], f["router"]["top"], f.get("shared"), gaps)
    else:
        raise ValueError(f["kind"])
    return x + p[pre + "ls2"] * layer_norm(y, p[pre + "norm2"], p[pre + "norm2.b"], eps)


def forward(config, p, tokens, dtype=torch.float64, trace=None, gaps=None):
    """Logits [n, vocab] of one sequence.  ``trace``: a list that receives the residual stream
    after every layer; ``gaps``: a list that receives every routed layer's route_gap."""
    p = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in p.items()}
    eps = config["norm"]["eps"]
    x = p["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, lc in enumerate(config["layers"]):
        x = layer(x, p, i, lc, eps, gaps)
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, p["final.norm"], p["final.norm.b"], eps) @ p["embed"].T
