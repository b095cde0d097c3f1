"""Tekenex without a device: its configuration, its place in the registry, the names and shapes
of its tensors, and the plain implementation's own consistency (the latent form of the attention
that the engine computes equals the expanded form of the equations)."""
import json

import pytest
import torch

import plain_tekenex as P
import tekenex_tools as tk


def test_registry_finds_the_design_by_its_singular_key():
    from gollmgo_b200.config import TekenexConfig, resolve_architecture
    import gollmgo_b200.architectures  # noqa: F401
    cfg, _ = tk.get("tek_a")
    arch = resolve_architecture(cfg)
    assert arch.name == "Tekenex"
    typed = arch.parse(cfg)
    assert isinstance(typed, TekenexConfig) and typed.width == 64 and typed.vocab == 203 and typed.eps == 1e-5
    assert [l.mlp.kind if l.mlp else None for l in typed.layers] == ["dense", "moe", None, "moe"]
    assert typed.layers[1].mlp.top == 1 and typed.layers[1].mlp.shared.ff == 56 and typed.layers[3].mlp.shared is None
    assert typed.layers[0].mixer.scale == 0.31
    spec = arch.spec(typed)
    assert spec.tie_embeddings and spec.layers[2].feed_forward is None and spec.layers[2].ffn_norm is None
    assert spec.layers[0].block.kind == "post_norm" and spec.layers[0].mixer.kind == "latent_attention"
    assert spec.layers[1].feed_forward.kind == "moe" and spec.layers[0].feed_forward.kind == "mlp"


@pytest.mark.parametrize("name", ["tek_a", "tek_b", "tek_c", "tek_d"])
def test_manifest_is_the_designs_tensor_list(name):
    from gollmgo_b200.parts import manifest_for_config
    cfg, _ = tk.get(name)
    m = {k: tuple(v.shape) for k, v in manifest_for_config(cfg).items() if not v.optional}
    assert m == tk.tensor_shapes(cfg)


@pytest.mark.parametrize("change,match", [
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "not known"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 0), "positive"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "picks"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv"), "kind"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_bad_configurations_are_refused(change, match):
    from gollmgo_b200.config import ConfigError, TekenexConfig
    cfg, _ = tk.get("tek_a")
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        TekenexConfig.from_dict(cfg)


def test_checkpoint_round_trip_and_wrong_shapes(tmp_path):
    from gollmgo_b200.parts import manifest_for_config
    from gollmgo_b200.weights import WeightError, checkpoint_source
    cfg, _ = tk.get("tek_a")
    w = tk.random_weights(cfg, 3)
    d = tk.model_folder(tmp_path, "ok", cfg, w)
    get = checkpoint_source(d, manifest_for_config(cfg), torch.bfloat16, "cpu")
    assert torch.equal(get("l1.mlp.router.b").float(), w["l1.mlp.router.b"])
    assert get("head") is None                       # the head is the embedding table
    bad = dict(w)
    bad["l0.mix.g"] = torch.zeros(4, 64)
    del bad["l3.ls2"]
    d2 = tk.model_folder(tmp_path, "bad", cfg, bad)
    with pytest.raises(WeightError) as e:
        checkpoint_source(d2, manifest_for_config(cfg), torch.bfloat16, "cpu")
    assert "l3.ls2" in str(e.value) and "l0.mix.g" in str(e.value)


def test_latent_form_of_the_attention_equals_the_expanded_form():
    """score = q . (Wuk c) = (Wuk^T q) . c and sum p v = Wuv (sum p c): what lets a cache of
    latents be read like a multi-query cache."""
    torch.manual_seed(0)
    n, D, H, d, v, r = 9, 32, 3, 8, 10, 12
    p = {"q": torch.randn(H * d, D), "dkv": torch.randn(r, D), "dkv.norm": torch.rand(r) + 0.5,
         "uk": torch.randn(H * d, r), "uv": torch.randn(H * v, r), "g": torch.randn(H, D), "o": torch.randn(D, H * v)}
    p = {k: t.double() for k, t in p.items()}
    h = torch.randn(n, D).double()
    want = P.latent_attention(h, p, "", H, d, v, r, 0.3, 1e-6)
    q = (h @ p["q"].T).view(n, H, d)
    c = P.rms_norm(h @ p["dkv"].T, p["dkv.norm"], 1e-6)
    ql = torch.einsum("ihd,hdr->ihr", q, p["uk"].view(H, d, r))
    s = torch.einsum("ihr,jr->hij", ql, c) * 0.3
    s = s.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf"))
    ol = torch.einsum("hij,jr->ihr", torch.softmax(s, -1), c)
    o = torch.einsum("ihr,her->ihe", ol, p["uv"].view(H, v, r)) * torch.sigmoid(h @ p["g"].T)[:, :, None]
    torch.testing.assert_close(o.reshape(n, H * v) @ p["o"].T, want, rtol=1e-10, atol=1e-10)


def test_plain_routing_picks_the_largest_and_weights_sum_to_one():
    torch.manual_seed(1)
    p = {"router": torch.randn(6, 16).double(), "router.b": torch.tensor([0., 0., 50., 0., 0., -50.]).double()}
    h = torch.randn(20, 16).double()
    idx, w = P.route(h, p, "", 2)
    z = h @ p["router"].T + p["router.b"]
    assert torch.equal(idx[:, 0], z.argmax(-1))
    torch.testing.assert_close(w.sum(-1), torch.ones(20).double())
    assert (idx != 5).all() and (idx[:, 0] == 2).all()          # the bias takes part in the choice
    idx1, w1 = P.route(h, p, "", 1)
    assert torch.equal(w1, torch.ones(20, 1).double())
