"""Tekenex on the device against the plain implementation (tests/plain_tekenex.py): each
mechanism alone, then whole models replayed through bin/trace_run (whole prompts, the last tokens
one by one, portions down to two tokens, mixed batches on a pool so small that pages and slots
are used again), then greedy generation through the engine's entry point and scheduler."""
import math

import numpy as np
import pytest
import torch

import plain_tekenex as P
import tekenex_tools as tk
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


def ctx_for(kit, dtype, page=16, max_tokens=512):
    return kit.parts.BuildContext(dtype, "cuda", max_tokens=max_tokens, max_seqs=8, page_size=page)


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
def test_norm_on_a_sublayers_output(kit, dtype, kind):
    """x += s * norm(y), and the rounded copy of x; with and without the scale; a mean far from 0."""
    torch.manual_seed(0)
    H, T, eps = 72, 7, 3e-5
    n = kit.parts.build_norm(kit.parts.PartSpec(kind, {"size": H, "eps": eps}), ctx_for(kit, dtype))
    w, b, s = bf(1 + 0.3 * torch.randn(H)), bf(0.4 * torch.randn(H)), bf(0.5 + torch.rand(H))
    n.load(lambda local: (b if local == ".b" else w).cuda().to(dtype))
    y = bf(torch.randn(T, H) * 3 + 5)
    x0 = torch.randn(T, H).double()
    normed = P.layer_norm(y, w, b, eps) if kind == "layernorm" else P.rms_norm(y, w, eps)
    for scale in (s, None):
        resid = x0.float().cuda()
        copy = torch.empty(T, H, device="cuda", dtype=dtype)
        n.norm_scale_add(resid, y.cuda().to(dtype), None if scale is None else scale.float().cuda(), copy)
        want = x0.float().double() + (normed * scale if scale is not None else normed)
        close(resid, want, torch.float32, f32=2e-6)
        close(copy, want, dtype, bf16=5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_before_the_head_takes_rows(kit, dtype):
    torch.manual_seed(1)
    H, eps = 40, 1e-6
    n = kit.parts.build_norm(kit.parts.PartSpec("layernorm", {"size": H, "eps": eps}), ctx_for(kit, dtype))
    w, b = bf(1 + 0.3 * torch.randn(H)), bf(torch.randn(H))
    n.load(lambda local: (b if local == ".b" else w).cuda().to(dtype))
    resid = (torch.randn(9, H) * 2 - 3).cuda()
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    out = torch.empty(3, H, device="cuda", dtype=dtype)
    n.add_norm(resid, None, out, rows=rows, write_back=False)
    close(out, P.layer_norm(resid.cpu().double()[[8, 0, 3]], w, b, eps), dtype, bf16=8e-3)


# ------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", DTYPES)
def test_squared_relu_feed_forward(kit, dtype):
    torch.manual_seed(2)
    D, F, T = 48, 100, 21
    ff = kit.parts.build_feed_forward(kit.parts.PartSpec("mlp", {"hidden_size": D, "intermediate_size": F,
                                                                  "activation": "relu2"}), ctx_for(kit, dtype))
    p = {"up": bf(torch.randn(F, D) / 7), "down": bf(torch.randn(D, F) / 10)}
    ff.load(lambda local: p[local].cuda().to(dtype))
    x = bf(torch.randn(T, D))
    close(ff.forward(x.cuda().to(dtype), None), P.dense_ff(x, p, ""), dtype)


def test_activations(kit):
    z = torch.linspace(-6, 6, 1001)
    for kind, f in (("relu2", lambda t: torch.relu(t) ** 2), ("gelu_tanh", P.gelu_tanh), ("silu", lambda t: t * torch.sigmoid(t))):
        out = torch.empty_like(z, device="cuda")
        kit.ops.act(z.cuda(), out, kind)
        torch.testing.assert_close(out.cpu().double(), f(z.double()), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top", [(6, 2), (5, 1), (3, 3), (40, 4)])
def test_router(kit, dtype, experts, top):
    """The chosen experts and their weights, with a bias that changes choices."""
    torch.manual_seed(3)
    D, T = 56, 33
    moe = kit.parts.build_feed_forward(kit.parts.PartSpec("moe", {"hidden_size": D, "intermediate_size": 8,
                                                                   "experts": experts, "top": top}), ctx_for(kit, dtype))
    p = {"router": bf(torch.randn(experts, D) / 4), "router.b": bf(torch.randn(experts))}
    moe.w_router, moe.b_router = p["router"].cuda().to(dtype), p["router.b"].float().cuda()
    x = bf(torch.randn(T, D))
    idx, wgt = moe.route(x.cuda().to(dtype))
    want_idx, want_w = P.route(x, p, "", top)
    assert torch.equal(idx.cpu().long().sort(-1).values, want_idx.sort(-1).values)
    got = torch.zeros(T, experts).double().scatter_(1, idx.cpu().long(), wgt.cpu().double())
    want = torch.zeros(T, experts).double().scatter_(1, want_idx, want_w)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,shared,T,D,F", [(6, 2, 24, 37, 40, 24), (4, 1, 0, 5, 40, 24), (3, 3, 40, 1, 40, 24),
                                                      (12, 2, 16, 150, 40, 24), (6, 2, 24, 700, 40, 24), (20, 3, 0, 400, 40, 24),
                                                      (6, 2, 72, 9, 320, 264), (5, 2, 0, 70, 264, 328)])
def test_mixture_of_experts(kit, dtype, experts, top, shared, T, D, F):
    """Few rows (the kernels that stream the chosen experts' weights: K in one or two steps, and, from
    256 values of K, through a ring of cp.async stages with a ragged last step) and many rows (in bfloat16
    the tcgen05 product over rows gathered into whole tiles per expert, some experts with no row at all)."""
    torch.manual_seed(4)
    sh = kit.parts.PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": shared, "names": ("gate", "up", "down")}) \
        if shared else None
    moe = kit.parts.build_feed_forward(kit.parts.PartSpec("moe", {"hidden_size": D, "intermediate_size": F, "experts": experts,
                                                                   "top": top, "shared": sh}), ctx_for(kit, dtype, max_tokens=1024))
    p = {"router": bf(torch.randn(experts, D) / 3), "router.b": bf(torch.randn(experts) / 2)}
    if experts == 20:
        p["router.b"][15:] = -100.0                  # experts that no token ever picks
    for e in [f"e{i}." for i in range(experts)] + (["shared."] if shared else []):
        f = shared if e == "shared." else F
        p.update({e + "gate": bf(torch.randn(f, D) / 6), e + "up": bf(torch.randn(f, D) / 6), e + "down": bf(torch.randn(D, f) / 5)})
    assert set(moe.weights()) == set(p)
    moe.load(lambda local: p[local].cuda().to(dtype))
    x = bf(torch.randn(T, D))
    want = P.moe_ff(x, p, "", experts, top, shared)
    close(moe.forward(x.cuda().to(dtype), None), want, dtype)
    # a token's result does not depend on the others in the step
    if T > 4:
        alone = moe.forward(x[3:4].cuda().to(dtype).contiguous(), None).clone()
        close(alone, want[3:4], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_grouped_product_per_head(kit, dtype):
    """Every group takes all rows and its own columns; the result padded with zeros; a sigmoid gate per row and group."""
    torch.manual_seed(5)
    T, G, K, N, Kp, Np = 45, 3, 20, 37, 24, 48
    a = bf(torch.randn(T, G * Kp + 8))
    w = bf(torch.randn(G, N, K) / 4)
    out = torch.full((T, G * Np), 7.0, device="cuda", dtype=dtype)
    kit.ops.grouped_gemm(a.cuda().to(dtype), w.cuda().to(dtype), out, N, K, G, a_group_cols=Kp, o_group_cols=Np,
                         n_padded=Np, rows=T, gate=a.cuda().to(dtype), gate_col0=G * Kp)
    want = torch.zeros(T, G, Np).double()
    for g in range(G):
        want[:, g, :N] = (a[:, g * Kp:g * Kp + K] @ w[g].T) * torch.sigmoid(a[:, G * Kp + g])[:, None]
    close(out, want.view(T, G * Np), dtype, bf16=1e-2)
    assert (out.view(T, G, Np)[:, :, N:] == 0).all()


# ------------------------------------------------------------------ latent attention
def make_mixer(kit, dtype, D, H, d, v, r, scale, page, seed=6):
    torch.manual_seed(seed)
    eps = 1e-6
    ctx = ctx_for(kit, dtype, page)
    mixer = kit.parts.build_mixer(kit.parts.PartSpec("latent_attention", {
        "hidden_size": D, "num_heads": H, "head_dim": d, "v_head_dim": v, "kv_rank": r, "scale": scale, "eps": eps}), ctx)
    p = {"q": bf(torch.randn(H * d, D) / D ** 0.5), "dkv": bf(torch.randn(r, D) / D ** 0.5), "dkv.norm": bf(1 + 0.2 * torch.randn(r)),
         "uk": bf(torch.randn(H * d, r) / r ** 0.5), "uv": bf(torch.randn(H * v, r) / r ** 0.5), "g": bf(torch.randn(H, D) / 3),
         "o": bf(torch.randn(D, H * v) / (H * v) ** 0.5)}
    assert set(mixer.weights()) == set(p)
    mixer.load(lambda local: p[local].cuda().to(dtype))
    return mixer, p, eps


def run_mixer(kit, mixer, x_parts, dtype, page, pages=64):
    cm = kit.CacheManager([mixer.cache_need()], page, pages, 4, dtype=dtype, device="cuda")
    bb = kit.BatchBuilder(cm, "cuda", query_tiles=mixer.query_tiles())
    cm.admit("s")
    outs = []
    for x in x_parts:
        batch = bb.build([kit.StepEntry("s", [0] * x.shape[0], [])])
        outs.append(mixer.forward(x.cuda().to(dtype).contiguous(), batch, cm.layer_cache(0)).clone())
    return torch.cat(outs)


TAGS = 8


def tagged_weights(D, H, d, v, r, scale, seed):
    """Weights under which one score can be made to stand out: the last 2 * TAGS input channels are
    tags.  Key tag t goes to latent row t and on to key dimension t of every head; query tag t goes
    to query dimension t of every head with a large weight.  A token with key tag t set is then
    the one key that a token with query tag t set looks at; all other channels are random."""
    g = torch.Generator().manual_seed(seed)
    m, C = TAGS, D - 2 * TAGS
    rn = lambda *shape: torch.randn(*shape, generator=g)
    q = torch.zeros(H, d, D)
    q[:, m:, :C] = rn(H, d - m, C) / C ** 0.5
    dkv = torch.zeros(r, D)
    dkv[m:, :C] = rn(r - m, C) / C ** 0.5
    uk = torch.zeros(H, d, r)
    uk[:, m:, m:] = rn(H, d - m, r - m) / (r - m) ** 0.5
    for t in range(m):
        q[:, t, C + m + t] = 24.0 / scale
        dkv[t, C + t] = 1.0
        uk[:, t, t] = 1.0
    p = {"q": q.reshape(H * d, D), "dkv": dkv, "dkv.norm": torch.ones(r), "uk": uk.reshape(H * d, r),
         "uv": rn(H * v, r) / r ** 0.5, "g": rn(H, D) / 3, "o": rn(D, H * v) / (H * v) ** 0.5}
    return {k: bf(t) for k, t in p.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(64, 3, 16, 24, 40, 16), (96, 4, 32, 32, 64, 8), (128, 18, 8, 12, 128, 32),
                                   (80, 2, 24, 8, 200, 16), (96, 2, 16, 40, 300, 16), (96, 2, 64, 48, 264, 8)])
def test_latent_attention_finds_one_key_among_hundreds(kit, dtype, shape):
    """Queries made to pick out single keys: the very first tokens, keys at both sides of page
    borders, keys hundreds of tokens back, a key that was itself decoded; asked for from prompt
    portions of several sizes (down to two tokens) and from single decoded tokens.  A kernel that
    loses one of these keys returns another token's values.  The last two shapes have latents wider
    than an attention head can be: the layer then caches expanded keys and values."""
    D, H, d, v, r, page = shape
    scale, eps = 1.3 / math.sqrt(d), 1e-6
    mixer, _, _ = make_mixer(kit, dtype, D, H, d, v, r, scale, page)
    p = tagged_weights(D, H, d, v, r, scale, seed=6)
    mixer.load(lambda local: p[local].cuda().to(dtype))
    n, m, C = 420, TAGS, D - 2 * TAGS
    x = torch.zeros(n, D)
    x[:, :C] = torch.randn(n, C, generator=torch.Generator().manual_seed(7))
    x = bf(x)
    keys = [0, 1, page - 1, page, 2 * page - 1, 2 * page, 5 * page - 1, 400]
    for t, k in enumerate(keys):
        x[k, C + t] = 8.0
    queries = {150: 0, 151: 1, 152: 2, 153: 3, 154: 4, 155: 5, 300: 0, 301: 6, 401: 0, 402: 3, 403: 6, 404: 7,
               410: 1, 419: 4, 418: 7, 405: 2}
    for qi, t in queries.items():
        x[qi, C + m + t] = 1.0
    # the plain attention puts nearly all weight of such a query on its key
    qq = (x @ p["q"].T).view(n, H, d)
    kk = (P.rms_norm(x @ p["dkv"].T, p["dkv.norm"], eps) @ p["uk"].T).view(n, H, d)
    for qi, t in queries.items():
        sc = torch.einsum("hd,jhd->hj", qq[qi], kk[:qi + 1]) * scale
        assert float(torch.softmax(sc, -1)[:, keys[t]].min()) > 0.99, (qi, keys[t])
    want = P.latent_attention(x, p, "", H, d, v, r, scale, eps)
    cuts = [130, 2, 17, 3, 64, 100, 2, 82]                 # 400 tokens in portions, then 20 single tokens
    parts, at = [], 0
    for c in cuts:
        parts.append(x[at:at + c])
        at += c
    parts += [x[i:i + 1] for i in range(at, n)]
    close(run_mixer(kit, mixer, parts, dtype, page), want, dtype)
    close(run_mixer(kit, mixer, [x], dtype, page), want, dtype)          # the same in one portion


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_token_by_token_equals_prefill(kit, dtype):
    mixer, p, eps = make_mixer(kit, dtype, 64, 5, 8, 16, 48, 0.4, 16, seed=8)
    x = bf(torch.randn(70, 64, generator=torch.Generator().manual_seed(9)))
    want = P.latent_attention(x, p, "", 5, 8, 16, 48, 0.4, eps)
    close(run_mixer(kit, mixer, [x[i:i + 1] for i in range(70)], dtype, 16), want, dtype)
    close(run_mixer(kit, mixer, [x[:1], x[1:3], x[3:70]], dtype, 16), want, dtype)


def test_latent_cache_keeps_one_row_per_token(kit):
    wide, _, _ = make_mixer(kit, torch.bfloat16, 64, 3, 16, 24, 300, 0.3, 16)
    assert wide.cache_need() == kit.parts.latent_attention.PagedKVNeed(3, 24, None)      # expanded: heads x max(dim, vdim)
    mixer, _, _ = make_mixer(kit, torch.bfloat16, 64, 3, 16, 24, 40, 0.3, 16)
    need = mixer.cache_need()
    assert need.shared_kv and need.n_kv_heads == 1 and need.head_dim == 48        # 40 padded to a multiple of 16
    cm = kit.CacheManager([need], 16, 10, 4, dtype=torch.bfloat16, device="cuda")
    k, v, _ = cm.layer_cache(0)
    assert k.data_ptr() == v.data_ptr() and cm.groups[0].kv.shape == (1, 1, 10, 1, 16, 48)
    assert kit.CacheManager.bytes_per_page([need], 16, 2) == 16 * 48 * 2


# ------------------------------------------------------------------ whole models through bin/trace_run
LENGTHS = {"tek_a": [1, 5, 37, 70, 130, 96], "tek_b": [2, 64, 65, 131, 300, 33], "tek_c": [3, 66, 40, 150, 97, 129],
           "tek_d": [4, 17, 80, 33, 65, 120]}
# float32: every row to a few units of rounding.  bfloat16: these models are narrow and deep enough in norms that
# a row's error varies widely with its content, so nine rows in ten must be within 4 % of the row's largest logit and
# none further off than what a lost or foreign key would cause (such a row is off by its whole size).
TOL = {"float32": (3e-5, 3e-5), "bfloat16": (4e-2, 0.2)}


def compare(trace, out_dir, reference, vocab, dtype):
    """Every written row against the plain logits of its (request, position); the error of a row is
    max|diff| / max|reference row|.  Returns (90th percentile, worst)."""
    import os
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
    p95 = float(np.percentile([e[0] for e in errs], 90))
    top = max(errs)
    assert p95 <= most, f"90th percentile of the rows' errors is {p95:.3e}"
    assert top[0] <= worst, f"worst relative error {top[0]:.3e} at (step, request, position) {top[1:]}"
    return p95, top[0]


def plain_logits(cfg, weights, requests):
    return {name: P.forward(cfg, weights, toks).float() for name, toks in requests.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tek_a", "tek_b", "tek_c", "tek_d"])
def test_replay_matches_plain(tmp_path, cuda_device, name, dtype):
    cfg, page = tk.get(name)
    weights = tk.random_weights(cfg, seed=31)
    model_dir = tk.model_folder(tmp_path, name, cfg, weights)
    requests = tk.steady_requests(cfg, weights, LENGTHS[name], seed=5)
    reference = plain_logits(cfg, weights, requests)
    trace = tt.Trace()
    tt.whole(trace, requests)
    tt.tail_decode(trace, requests)
    tt.portions(trace, requests)
    tt.mixed(trace, requests, max_live=4, seed=3)
    tt.mixed(trace, dict(reversed(list(requests.items()))), max_live=3, seed=4, tag="n")
    out = str(tmp_path / "out")
    tt.run_trace(model_dir, dtype, trace, out, block_size=page)
    p95, worst = compare(trace, out, reference, cfg["vocab"], dtype)
    pool, asked, shared = tt.pages_were_used_again(trace, out + "/pages.jsonl", page)
    print(f"{name} {dtype}: {len(trace.steps)} steps, {pool} pages for {asked} asked, {shared} held by several, "
          f"errors: 90 % within {p95:.2e}, worst {worst:.2e}")


@pytest.mark.parametrize("name,dtype", [("tek_a", "bfloat16"), ("tek_b", "float32"), ("tek_c", "bfloat16")])
def test_pages_given_back_are_never_read(tmp_path, cuda_device, name, dtype):
    """The mixed trace with every page overwritten by NaN the moment it is given back."""
    import os
    cfg, page = tk.get(name)
    weights = tk.random_weights(cfg, seed=32)
    model_dir = tk.model_folder(tmp_path, name, cfg, weights)
    requests = tk.steady_requests(cfg, weights, LENGTHS[name], seed=6)
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
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(P.forward(cfg, weights, toks, dtype=torch.float32)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_engine(tmp_path, cuda_device):
    """Requests of unequal length through Engine.generate (scheduler, chunked prompts, captured
    decode steps, the device's arg-max): the plain implementation's tokens, alone and together."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = tk.get("tek_a")
    weights = tk.random_weights(cfg, seed=33)
    d = tk.model_folder(tmp_path, "tek_a", cfg, weights)
    prompts = list(tt.random_requests(cfg["vocab"], [1, 9, 40, 23], seed=8).values())
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=24, max_batch_size=4, max_token_budget=32,
                 prefill_chunk_size=16)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    want = [plain_greedy(cfg, weights, pr, 12) for pr in prompts]
    assert [o.token_ids for o in outs] == want
    assert eng.generate([prompts[2]], SamplingParams(max_tokens=12, ignore_eos=True))[0].token_ids == want[2]
    eng.runner.cache.audit()
    assert eng.runner.cache.free_pages() == 24


def test_long_decoding_in_bfloat16_stays_near_the_plain_choice(tmp_path, cuda_device):
    """150 decoded tokens over many pages: the tokens are (nearly) the plain implementation's best
    given the same history (all but a few: rounding may turn a close choice of experts)."""
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = tk.get("tek_b")
    weights = tk.random_weights(cfg, seed=34)
    d = tk.model_folder(tmp_path, "tek_b", cfg, weights)
    prompt = tt.random_requests(cfg["vocab"], [11], seed=9)["r0"]
    eng = Engine(d, dtype="bfloat16", block_size=page, num_blocks=32, max_batch_size=2, max_token_budget=64)
    toks = eng.generate([prompt], SamplingParams(max_tokens=150, ignore_eos=True))[0].token_ids
    assert len(toks) == 150
    logits = P.forward(cfg, weights, prompt + toks)
    near = sum(float(row.max() - row[tok]) <= 0.06 * float(row.abs().max())
               for tok, row in zip(toks, logits[len(prompt) - 1:]))
    assert near >= 143, f"only {near} of 150 tokens are near the plain choice"
    assert eng.runner.cache.free_pages() == 32


def test_command_line_and_seeded_sampling(tmp_path, cuda_device):
    """`python -m gollmgo_b200 generate` and `bench` on a Tekenex folder; sampling with a temperature and a
    seed gives the same tokens alone and in a batch (the logits do not depend on the batch)."""
    import json
    import os
    import subprocess
    import sys
    from gollmgo_b200 import Engine, SamplingParams
    cfg, page = tk.get("tek_c")
    weights = tk.random_weights(cfg, seed=35)
    d = tk.model_folder(tmp_path, "tek_c", cfg, weights)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, "-m", "gollmgo_b200"]
    common = ["--model", d, "--dtype", "float32", "--block-size", str(page), "--num-blocks", "16",
              "--max-batch-size", "4", "--max-token-budget", "64", "--log-level", "error"]
    p = subprocess.run(base + ["generate", *common, "--prompt-ids", "5,6,7", "--prompt-ids", "9", "--max-tokens", "5",
                               "--ignore-eos"], capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    lines = [json.loads(l) for l in p.stdout.strip().splitlines()]
    assert lines[0]["token_ids"] == plain_greedy(cfg, weights, [5, 6, 7], 5)
    assert lines[1]["token_ids"] == plain_greedy(cfg, weights, [9], 5)
    p = subprocess.run(base + ["bench", *common, "--mode", "offline", "--num-prompts", "5", "--prompt-len", "12",
                               "--output-len", "4"], capture_output=True, text=True, cwd=root)
    assert p.returncode == 0, p.stderr
    res = json.loads(p.stdout)
    assert res["num_prompts"] == 5 and res["tokens_per_second"] > 0 and res["error_count"] == 0
    prompts = list(tt.random_requests(cfg["vocab"], [3, 30, 11], seed=10).values())
    params = [SamplingParams(temperature=0.9, top_k=20, seed=70 + i, max_tokens=10, ignore_eos=True) for i in range(3)]
    eng = Engine(d, dtype="float32", block_size=page, num_blocks=16, max_batch_size=4, max_token_budget=48,
                 prefill_chunk_size=16)
    together = [o.token_ids for o in eng.generate(prompts, params)]
    alone = [eng.generate([pr], [pa])[0].token_ids for pr, pa in zip(prompts, params)]
    assert together == alone
    assert eng.runner.cache.free_pages() == 16
