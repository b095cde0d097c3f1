"""Bevuvik without a device: registry and typed configuration, refused configurations, the
manifest against the design's naming rules, the run order of a repeated run of layers, the
rotary table with stretching, cache needs, and properties of the plain implementation that
the device tests lean on."""
import copy
import math

import pytest
import torch

import bevuvik_tools as bt
import plain_bevuvik as P


def test_registry_and_typed_config():
    from gollmgo_b200.config import resolve_architecture
    cfg, _ = bt.get("bev_a")
    arch = resolve_architecture(cfg)
    assert arch.name == "Bevuvik"
    c = arch.parse(cfg)
    assert (c.vocab, c.width, c.eps, c.residual_mult) == (203, 64, 1e-5, 0.5)
    assert (c.loop.start, c.loop.stop, c.loop.times) == (1, 3, 3)
    a, p = c.layers[0].mixer, c.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.diff) == (4, 2, 16, 24, 40, 0.2)
    assert a.rot.dims == 8 and a.rot.scaling == (4.0, 64.0, 8.0, 1.0)
    assert (p.left.softcap, p.left.rot.scaling, p.right.conv) == (20.0, None, 3)
    assert c.layers[2].mlp is None and c.layers[0].mlp.limit == 2.5
    b = arch.parse(bt.get("bev_b")[0])
    assert b.loop is None and b.layers[0].mixer.left.softcap is None and b.layers[2].mixer.rot is None


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "more than dim"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3), "loop"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "left"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refused_configurations(edit, word):
    from gollmgo_b200.config import ConfigError, resolve_architecture
    cfg, _ = bt.get("bev_a")
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        resolve_architecture(cfg).parse(cfg)


@pytest.mark.parametrize("name", sorted(bt.TINY))
def test_manifest_follows_the_naming_rules(name):
    from gollmgo_b200.parts.model import manifest_for_config
    cfg, _ = bt.get(name)
    m = manifest_for_config(cfg)
    want = bt.tensor_shapes(cfg)
    assert set(m) == set(want)
    assert all(tuple(m[k].shape) == tuple(want[k]) for k in want)


def test_run_order_of_a_repeated_run():
    from gollmgo_b200.architectures.bevuvik import bevuvik_spec
    from gollmgo_b200.config.bevuvik_config import BevuvikConfig
    for name in sorted(bt.TINY):
        cfg, _ = bt.get(name)
        spec = bevuvik_spec(BevuvikConfig.from_dict(cfg))
        got = [(e.layer, e.mix_input) for e in spec.run_order]
        assert got == P.layer_runs(cfg)
        assert [e.cache for e in spec.run_order] == list(range(len(got)))       # every run a cache entry of its own
        assert (spec.input_mix_name == "loop.in") == bool(cfg.get("loop"))
    cfg, _ = bt.get("bev_a")
    assert [l for l, _ in P.layer_runs(cfg)] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [f for _, f in P.layer_runs(cfg)] == [False, True, False, True, False, True, False, False]


def test_rotary_table_with_stretching():
    from gollmgo_b200.parts.position import YarnScaling, inverse_frequencies
    for dims, base, sc in [(8, 10000.0, (4.0, 64, 8.0, 1.0)), (12, 500000.0, (16.0, 32, 4.0, 0.5)),
                           (64, 1e6, (8.0, 128, 32.0, 1.0)), (16, 1000.0, None)]:
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        f, mag = P.rotary_frequencies(rot)
        got = inverse_frequencies(dims, base, YarnScaling(*sc) if sc else None)
        torch.testing.assert_close(got, f, rtol=1e-14, atol=0)
        if sc:
            assert YarnScaling(*sc).magnitude == mag == 0.1 * math.log(sc[0]) + 1.0
            plain = inverse_frequencies(dims, base, None)
            assert (got <= plain).all() and (got < plain).any() and (got >= plain / sc[0] * (1 - 1e-12)).all()


def test_cache_needs_of_the_mixers():
    from gollmgo_b200.cache import CacheManager, FixedStateNeed, PagedKVNeed
    from gollmgo_b200.parts import BuildContext, build_model
    cfg, page = bt.get("bev_a")
    _, spec, model = build_model(cfg, BuildContext(torch.float32, "cpu", 64, 4, page))
    needs = model.cache_needs()
    assert len(needs) == 8
    # differential attention: keys per map (2 x kv heads of size dim), values once per kv head, the window
    assert needs[0] == PagedKVNeed(4, 16, 40, v_heads=2, v_head_dim=24) == needs[2] == needs[4]
    # the parallel mixer: pages for the attention branch; a state matrix and the convolution's window for the other
    assert needs[1] == (PagedKVNeed(2, 32, None, v_heads=2, v_head_dim=16),
                        (FixedStateNeed((4, 24, 16)), FixedStateNeed((2, 2 * 2 * 16 + 4 * 24))))
    cm = CacheManager(needs, page, 6, 4)
    assert len(cm.groups) == 3                              # the windowed layers, and the two kinds of attention branch
    assert len(cm.state_needs) == 8                         # two per run of a parallel layer
    assert CacheManager.bytes_per_page(needs, page, 2) == \
        (4 * (4 * 16 + 2 * 24) + 3 * (2 * 32 + 2 * 16) + (1 * 16 + 1 * 16)) * page * 2


def test_plain_model_is_causal_and_windowed():
    """What the device tests lean on: a token's logits depend on earlier tokens only, and a
    differential attention layer forgets what has left its window."""
    cfg, _ = bt.get("bev_b")
    w = {k: v.double() for k, v in bt.random_weights(cfg, 1).items()}
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, cfg["vocab"], (30,), generator=g).tolist()
    b = list(a)
    b[20] = (b[20] + 1) % cfg["vocab"]
    la, lb = P.forward(w, cfg, a), P.forward(w, cfg, b)
    torch.testing.assert_close(la[:20], lb[:20], rtol=0, atol=0)
    assert float((la[20:] - lb[20:]).abs().max()) > 1e-3
    # the mixer alone, window 5: row 12 does not see token 7, row 11 does
    m = cfg["layers"][1]["mixer"]
    h = torch.randn(16, cfg["width"], generator=g, dtype=torch.float64)
    h2 = h.clone()
    h2[7] += 1.0
    y, y2 = (P.differential_attention(x, w, "l1.mix.", m, 1e-6) for x in (h, h2))
    torch.testing.assert_close(y[12:], y2[12:], rtol=0, atol=1e-12)
    assert float((y[11] - y2[11]).abs().max()) > 1e-4


def test_plain_delta_rule_overwrites_with_unit_keys():
    """With decay one, beta one and orthonormal keys the rule stores each value under its key:
    a spot check of the rule itself, beside a run of the whole mixer on a configuration."""
    k = torch.eye(4, dtype=torch.float64)
    S = torch.zeros(4, 3, dtype=torch.float64)
    v = torch.arange(12, dtype=torch.float64).view(4, 3)
    for t in range(4):
        S = S + torch.outer(k[t], 1.0 * (v[t] - S.T @ k[t]))
    torch.testing.assert_close(S, v)
    cfg, _ = bt.get("bev_c")
    w = {k: v.double() for k, v in bt.random_weights(cfg, 2).items()}
    m = cfg["layers"][0]["mixer"]["right"]
    h = torch.randn(40, cfg["width"], generator=torch.Generator().manual_seed(3), dtype=torch.float64)
    whole = P.gated_delta_rule(h, w, "l0.mix.right.", m, 3e-6)
    assert whole.shape == (40, cfg["width"]) and torch.isfinite(whole).all()
    # causal: the first rows do not depend on later ones
    torch.testing.assert_close(P.gated_delta_rule(h[:17], w, "l0.mix.right.", m, 3e-6), whole[:17], rtol=0, atol=1e-12)
