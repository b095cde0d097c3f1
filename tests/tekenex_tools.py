"""Small Tekenex configurations and weights for the tests.  The configurations differ in every
size and in the order of their layers: odd and even head counts, more heads than one tile of the
decode kernels holds, query/key size equal to and different from the value size, latents that
take the general, the mma.sync and the tcgen05 attention kernels, one expert per token and every
expert per token, with and without a shared expert, a layer without feed-forward, vocabularies
that are no power of two."""
import copy
import json
import os

import torch


def _layer(heads, dim, vdim, rank, scale, mlp):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


TEK_A = {"architecture": "Tekenex", "vocab": 203, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    _layer(3, 16, 24, 40, 0.31, _dense(100)),
    _layer(3, 16, 24, 40, 0.31, _moe(4, 1, 40, 56)),
    _layer(3, 16, 24, 40, 0.31, None),
    _layer(3, 16, 24, 40, 0.31, _moe(5, 3, 24)),
]}
TEK_B = {"architecture": "Tekenex", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    _layer(4, 32, 32, 64, 0.15, _moe(8, 2, 72, 72)),
    _layer(4, 32, 32, 64, 0.15, _dense(136)),
    _layer(2, 24, 40, 64, 0.2, _moe(8, 2, 72, 72)),
]}
TEK_C = {"architecture": "Tekenex", "vocab": 257, "width": 96, "norm": {"eps": 3e-6}, "layers": [
    _layer(18, 8, 12, 128, 0.4, _dense(96)),
    _layer(18, 8, 12, 128, 0.4, _moe(3, 3, 48, 80)),
]}
# sizes that are no multiple of 8: no kernel may count on 16-byte rows; the second layer's latent is wider than
# an attention head can be, so that layer caches expanded keys and values (a second cache group)
TEK_D = {"architecture": "Tekenex", "vocab": 150, "width": 100, "norm": {"eps": 2e-6}, "layers": [
    _layer(2, 12, 20, 28, 0.3, _moe(3, 2, 20, 28)),
    _layer(5, 6, 10, 260, 0.45, _dense(52)),
]}

# name -> (config, page size)
TINY = {"tek_a": (TEK_A, 16), "tek_b": (TEK_B, 8), "tek_c": (TEK_C, 32), "tek_d": (TEK_D, 16)}


def get(name):
    cfg, page = TINY[name]
    return copy.deepcopy(cfg), page


def tensor_shapes(cfg):
    """Names and shapes of a checkpoint of ``cfg``, from the design's naming rules."""
    D, s = cfg["width"], {}
    s["embed"] = (cfg["vocab"], D)
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        H, d, v, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        s.update({p + "norm1": (D,), p + "norm1.b": (D,), p + "ls1": (D,),
                  p + "mix.q": (H * d, D), p + "mix.dkv": (r, D), p + "mix.dkv.norm": (r,),
                  p + "mix.uk": (H * d, r), p + "mix.uv": (H * v, r), p + "mix.g": (H, D), p + "mix.o": (D, H * v)})
        f = lc["mlp"]
        if f is None:
            continue
        s.update({p + "norm2": (D,), p + "norm2.b": (D,), p + "ls2": (D,)})
        if f["kind"] == "dense":
            s.update({p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            s.update({p + "mlp.router": (E, D), p + "mlp.router.b": (E,)})
            for e in range(E):
                s.update({f"{p}mlp.e{e}.gate": (ff, D), f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
            if f.get("shared"):
                sf = f["shared"]["ff"]
                s.update({p + "mlp.shared.gate": (sf, D), p + "mlp.shared.up": (sf, D), p + "mlp.shared.down": (D, sf)})
    s["final.norm"] = (D,)
    s["final.norm.b"] = (D,)
    return s


def random_weights(cfg, seed):
    """Float32 tensors whose values are exact in bfloat16, so that the same checkpoint serves both
    modes.  Matrices N(0, 1/fan_in) with a gain, norm weights around 1, biases and layer scales
    that are far from 0 and 1, router biases large enough to move choices."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 2:
            gain = 1.0 if name == "embed" else 1.6
            t = torch.randn(shape, generator=g) * gain / (shape[1] ** 0.5 if name != "embed" else 1.0)
        elif name.endswith("router.b"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("ls1") or name.endswith("ls2"):
            t = 0.6 + 0.3 * torch.rand(shape, generator=g)
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


def steady_requests(cfg, weights, lengths, seed, min_gap=0.06):
    """Random requests in which no token's choice of experts is a close call (the plain
    implementation's router gaps all exceed ``min_gap``): a reduced-precision run then makes the
    same choices, and its logits can be compared with a tolerance of rounding.  A token that makes a
    close call is drawn again; tokens before it are not affected (attention is causal)."""
    import random

    import plain_tekenex as P
    rng = random.Random(seed)
    out = {}
    for i, n in enumerate(lengths):
        toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
        for _ in range(40 * n):
            gaps = []
            P.forward(cfg, weights, toks, gaps=gaps)
            if not gaps:
                break
            bad = (torch.stack(gaps).min(0).values < min_gap).nonzero()
            if bad.numel() == 0:
                break
            toks[int(bad[0])] = rng.randrange(cfg["vocab"])
        else:
            raise AssertionError("no request without close calls found")
        out[f"r{i}"] = toks
    return out
