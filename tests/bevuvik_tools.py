"""Small Bevuvik configurations and weights for the tests.  The configurations differ in every size,
in the order of their layers and in which optional features they have: with and without a repeated
run of layers (of one layer, of several, starting at 0 and later), windows shorter and longer than a
page and than the requests, rotary tables on part of a head and on all of it, with and without
stretching, with and without capped scores, one kv head, as many kv heads as heads, a layer without
feed-forward, sizes that are no multiple of 8, and sizes that reach the widest kernels."""
import copy
import json
import os

import torch


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _diff(heads, kv, dim, vdim, scale, diff, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    return m


def _left(heads, kv, dim, vdim, scale, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = rot
    return m


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _attention(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _parallel(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


_YARN = (4.0, 64, 8.0, 1.0)

BEV_A = {"architecture": "Bevuvik", "vocab": 203, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
         "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
             _attention(_diff(4, 2, 16, 24, 0.3, 0.2, window=40, rot=_rot(8, 10000.0, _YARN)), _mlp(100, 2.5)),
             _parallel(_left(4, 2, 32, 16, 0.2, softcap=20.0, rot=_rot(16, 50000.0)), _right(4, 2, 16, 24, 3), _mlp(72, 2.5)),
             _attention(_diff(4, 2, 16, 24, 0.3, 0.2, window=40, rot=_rot(8, 10000.0, _YARN)), None),
             _parallel(_left(2, 1, 16, 16, 0.25, softcap=8.0, rot=_rot(16, 1000.0)), _right(2, 1, 8, 40, 4), _mlp(40, 1.5)),
         ]}
# no loop, one kv head, kv heads = heads, a window shorter than a page, full-width rotation without stretching, no cap
BEV_B = {"architecture": "Bevuvik", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "layers": [
    _parallel(_left(4, 1, 32, 32, 0.18, rot=_rot(32, 10000.0)), _right(3, 3, 32, 32, 2), _mlp(136, 0.8)),
    _attention(_diff(2, 2, 32, 32, 0.2, 0.35, window=5, rot=_rot(32, 100000.0)), _mlp(136, 0.8)),
    _attention(_diff(4, 1, 8, 16, 0.35, 0.1, window=17), _mlp(64, 0.8)),
]}
# sizes that are no multiple of 8, a loop of one layer from the start, a window of exactly four pages
BEV_C = {"architecture": "Bevuvik", "vocab": 150, "width": 100, "norm": {"eps": 3e-6}, "residual_mult": 0.8,
         "loop": {"start": 0, "stop": 1, "times": 2}, "layers": [
             _parallel(_left(3, 3, 12, 20, 0.3, softcap=15.0, rot=_rot(6, 20000.0)), _right(6, 2, 20, 36, 5), _mlp(52, 1.0)),
             _attention(_diff(6, 2, 12, 20, 0.3, 0.25, window=64, rot=_rot(12, 500000.0, (16.0, 32, 4.0, 0.5))), _mlp(28, 3.0)),
         ]}
# the widest kernels: heads of 128, a state of 128 x 128, a window longer than most requests; the loop ends the model
BEV_D = {"architecture": "Bevuvik", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
         "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [
             _attention(_diff(2, 1, 64, 128, 0.125, 0.3, window=200, rot=_rot(64, 1000000.0, (8.0, 128, 32.0, 1.0))), _mlp(256, 1.0)),
             _parallel(_left(4, 2, 128, 128, 0.09, softcap=30.0, rot=_rot(64, 500000.0)), _right(2, 1, 128, 128, 4), _mlp(384, 1.0)),
         ]}

# name -> (config, page size)
TINY = {"bev_a": (BEV_A, 16), "bev_b": (BEV_B, 8), "bev_c": (BEV_C, 16), "bev_d": (BEV_D, 32)}


def get(name):
    cfg, page = TINY[name]
    return copy.deepcopy(cfg), page


def tensor_shapes(cfg):
    """Names and shapes of a checkpoint of ``cfg``, from the design's naming rules."""
    D, s = cfg["width"], {}
    s["embed"] = (cfg["vocab"], D)
    if cfg.get("loop"):
        s["loop.in"] = (D, 2 * D)
    for i, lc in enumerate(cfg["layers"]):
        p = f"l{i}."
        s[p + "norm1"] = (D,)
        m = lc["mixer"]
        if lc["type"] == "attention":
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * 2 * d, D), p + "mix.q.b": (H * 2 * d,), p + "mix.k": (G * 2 * d, D),
                      p + "mix.k.b": (G * 2 * d,), p + "mix.v": (G * v, D), p + "mix.v.b": (G * v,),
                      p + "mix.o": (D, H * v), p + "mix.o.b": (D,)})
            s.update({p + "mix." + n: (d,) for n in ("lq1", "lk1", "lq2", "lk2")})
        else:
            l, r = m["left"], m["right"]
            H, G, d, v = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            s.update({p + "mix.left.q": (H * d, D), p + "mix.left.k": (G * d, D), p + "mix.left.v": (G * v, D),
                      p + "mix.left.o": (D, H * v), p + "mix.left.out": (D,), p + "mix.right.out": (D,)})
            H, G, d, v, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            s.update({p + "mix.right.q": (G * d, D), p + "mix.right.q.conv": (G * d, taps),
                      p + "mix.right.k": (G * d, D), p + "mix.right.k.conv": (G * d, taps),
                      p + "mix.right.v": (H * v, D), p + "mix.right.v.conv": (H * v, taps),
                      p + "mix.right.b": (H, D), p + "mix.right.a": (H, D), p + "mix.right.A_log": (H,),
                      p + "mix.right.dt_bias": (H,), p + "mix.right.norm": (v,), p + "mix.right.g": (H * v, D),
                      p + "mix.right.o": (D, H * v)})
        f = lc["mlp"]
        if f is not None:
            s.update({p + "mlp.gate": (f["ff"], D), p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
    s["final.norm"] = (D,)
    s["head"] = (cfg["vocab"], D)
    return s


def random_weights(cfg, seed):
    """Float32 tensors whose values are exact in bfloat16, so that the same checkpoint serves both
    modes.  Matrices N(0, 1/fan_in) with a gain, norm weights around 1, biases away from 0, decays
    spread between fast and slow, taps of the size of an average with weight on the current token."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "conv":
            t = torch.randn(shape, generator=g) / shape[1]
            t[:, -1] += 1.0
        elif len(shape) == 2:
            gain = 1.0 if name == "embed" else 1.5
            t = torch.randn(shape, generator=g) * gain / (shape[1] ** 0.5 if name != "embed" else 1.0)
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=g)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif last == "A_log":
            t = torch.randn(shape, generator=g) - 1.0
        elif last == "dt_bias":
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


def model_folder(tmp, name, cfg, weights, dtype="bfloat16"):
    from gollmgo_b200.weights import save_file
    d = os.path.join(str(tmp), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    td = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    save_file(((k, v.to(td)) for k, v in weights.items()), os.path.join(d, "model.safetensors"), metadata={"format": "pt"})
    return d
