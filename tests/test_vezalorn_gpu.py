"""The Vezalorn design against its plain restatement (tests/plain_vezalorn.py): each mechanism's kernels alone, whole
models in every cutting of the requests, windows of pages and state slots that are used again, keys far away and
at page borders, long decoding, sizes that differ in everything, and greedy generation through the engine."""
import json
import os

import numpy as np
import pytest
import torch

import plain_vezalorn as plain
import traces
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu


def attention(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}}


def gru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model_config(vocab, width, scale, eps, groups, layers):
    return {"architecture": "Vezalorn", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps, "groups": groups}, "layers": layers}


# Two configurations that differ in every size; neither has the recurrent width equal to the model's, the latent as
# wide as a head, or all attention layers alike. A starts with attention, has a feed-forward after a recurrence and an
# attention layer without one; B has one norm group, one head in one layer and sizes that are no multiples of 16.
CONFIG_A = model_config(300, 96, 6.0, 1e-5, 4, [
    attention(3, 32, 16, 24, 48, base=10000.0, mlp=dense(160)),
    gru(64, mlp=dense(72)),
    gru(128),
    attention(6, 16, 8, 16, 80, base=500000.0),
    gru(96),
])
CONFIG_B = model_config(211, 72, 1.0, 1e-6, 1, [
    gru(40),
    attention(1, 24, 12, 20, 28, base=1000.0, mlp=dense(100)),
    attention(5, 8, 4, 12, 36, base=300000.0, mlp=dense(64)),
    gru(72, mlp=dense(90)),
])
# sizes at which the tensor-core kernels serve the bfloat16 path (multiples of 16 everywhere)
CONFIG_C = model_config(512, 128, 3.0, 1e-5, 2, [
    gru(192),
    attention(4, 32, 16, 48, 64, base=100000.0, mlp=dense(256)),
    gru(128, mlp=dense(128)),
    attention(8, 16, 32, 16, 96, base=10000.0),
])
# sizes that are multiples of nothing: no 16-byte row anywhere, so every kernel's plain form serves both element types
CONFIG_D = model_config(101, 54, 2.5, 1e-5, 3, [
    attention(2, 10, 6, 14, 22, base=5000.0, mlp=dense(50)),
    gru(30),
    attention(7, 6, 2, 5, 9, base=20000.0),
    gru(54, mlp=dense(33)),
])
CONFIGS = {"a": CONFIG_A, "b": CONFIG_B, "c": CONFIG_C, "d": CONFIG_D}
LENGTHS = {"a": [1, 9, 40, 64, 131, 77, 2], "b": [3, 55, 150, 18, 97], "c": [200, 1, 65, 129, 30, 260], "d": [70, 2, 33, 140, 17]}
PAGE = {"a": 8, "b": 16, "c": 16, "d": 4}


def write_model(folder, config, seed, dtype="bfloat16", init=None):
    from cellm_b200.weights import InitSpec, write_random_model
    # matrices five times as large as a trained model's 0.02, so that a wrong key or a stale state moves the logits; larger
    # ones make gates and softmax so steep that bfloat16's own rounding of their inputs comes near the bound of the comparison
    init = init or InitSpec(linear_std=0.1, embedding_std=0.08, bias_std=0.1, norm_jitter=0.2)
    return write_random_model(str(folder), config, seed, dtype, init)


def load_plain(folder):
    from cellm_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n).clone() for n in sf.names()}


def run_trace(folder, dtype, steps, page, use_graphs=True, max_tokens=None):
    from cellm_b200.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or traces.max_live_tokens(steps), page, 4, use_graphs=use_graphs)
    outs = [rp.step(s["entries"], s["end"]) for s in steps]
    assert rp.cache.live == 0
    assert all(rp.cache.free_pages(g) == rp.cache.group_pages[g] for g in range(len(rp.cache.group_pages)))
    return traces.collect(steps, outs)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    d = tmp_path_factory.mktemp("vz")
    out = {}
    for i, (name, config) in enumerate(CONFIGS.items()):
        folder = write_model(d / name, config, 31 + i)
        cfg, w = load_plain(folder)
        rng = np.random.default_rng(17 + i)
        reqs = {f"r{j}": rng.integers(0, cfg["vocab"], n).tolist() for j, n in enumerate(LENGTHS[name])}
        ref = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
        out[name] = (folder, reqs, ref)
    return out


FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_matches_plain(models, name, dtype):
    folder, reqs, ref = models[name]
    results = {}
    for fam, make in FAMILIES.items():
        got = results[fam] = run_trace(folder, dtype, make(reqs), PAGE[name])
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} {fam} {rid}")
    for fam in ("tail", "portions", "mixed"):
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(results[fam][rid], len(toks)), traces.as_matrix(results["whole"][rid], len(toks)),
                        dtype, f"{name} {dtype} {fam} vs whole {rid}", k=K_SELF[dtype])
    got = run_trace(folder, dtype, traces.mixed(reqs), PAGE[name], use_graphs=False)
    for rid, toks in reqs.items():
        check_close(traces.as_matrix(got[rid], len(toks)), traces.as_matrix(results["mixed"][rid], len(toks)), dtype,
                    f"{name} {dtype} mixed: kernel by kernel vs graphs {rid}", k=K_SELF[dtype])


def test_mixed_trace_reuses_pages_and_slots(models):
    folder, reqs, _ = models["a"]
    steps = traces.mixed(reqs)
    assert len(reqs) > 4                                     # more requests than state slots
    assert traces.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_two_and_odd_sizes(models, dtype):
    folder, reqs, ref = models["b"]
    for sizes in ((2,), (3, 2, 5), (17, 2, 2, 31)):
        got = run_trace(folder, dtype, traces.portions(reqs, sizes), PAGE["b"])
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"b {dtype} portions {sizes} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_pages(models, dtype):
    """Most of the sequence decoded token by token: every page border and every state update on the decode path."""
    folder, reqs, ref = models["c"]
    some = {rid: reqs[rid] for rid in ("r0", "r5")}
    got = run_trace(folder, dtype, traces.tail_one_by_one(some, tail=190), 8)
    for rid, toks in some.items():
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"c {dtype} long tail {rid}")


# --------------------------------------------------------------------- keys far away, the first tokens, page borders
def sharp_attention_model(folder, seed, scale):
    """One attention layer between two recurrences, its softmax so peaked (a large score scale, large query and key
    matrices) that a position's output is a few single keys, wherever they lie: a key lost at a page border, a wrong
    block of keys or a wrong rotation changes the logits outright."""
    from cellm_b200.weights import InitSpec
    config = model_config(128, 64, 4.0, 1e-5, 2, [gru(64), attention(4, 16, 16, 16, 32, base=10000.0, scale=scale), gru(48)])
    return write_model(folder, config, seed, init=InitSpec(linear_std=0.25, embedding_std=0.1, bias_std=0.05, norm_jitter=0.1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_reaches_far_keys(tmp_path, dtype):
    # bfloat16 rounds a score of size s by s / 256, which a peaked softmax turns into that share of its weights: the
    # 16-bit run gets smaller scores (up to 27 instead of 200), still so peaked that the heaviest key has two fifths of
    # the weight in the median and one lost key shows
    folder = sharp_attention_model(tmp_path / "sharp", 5, 1.5 if dtype == "float32" else 0.2)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg["vocab"], 700).tolist()
    reqs = {"long": toks, "short": toks[:70]}
    ref = {rid: plain.forward(cfg, w, t) for rid, t in reqs.items()}
    # the attention really is peaked and really reaches back: the plain model's heaviest key is often hundreds back
    t64 = {k: v.double() for k, v in w.items()}
    lo = []
    plain.forward(cfg, w, toks, layers_out=lo)
    x1 = lo[0]
    p = cfg["layers"][1]["mixer"]
    T = len(toks)
    q = (x1 @ t64["l1.mix.q"].T).reshape(T, p["heads"], -1)
    down = x1 @ t64["l1.mix.dkv"].T
    c = plain.unit_rms(down[:, :p["kv_rank"]], cfg["norm"]["eps"]) * t64["l1.mix.dkv.norm"]
    kt = plain.rotate_pairs(down[:, p["kv_rank"]:], torch.arange(T), p["rot"]["base"], p["rot"]["dims"])
    kp = (c @ t64["l1.mix.uk"].T).reshape(T, p["heads"], p["dim"])
    qt = plain.rotate_pairs(q[..., p["dim"]:], torch.arange(T), p["rot"]["base"], p["rot"]["dims"])
    s = (torch.einsum("ihd,jhd->hij", q[..., :p["dim"]], kp) + torch.einsum("ihr,jr->hij", qt, kt)) * p["scale"]
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    wts = torch.softmax(s, -1)
    top, where = wts[:, 600:].max(-1)
    assert float(top.median()) > (0.3 if dtype == "float32" else 0.1) and float((torch.arange(600, T)[None] - where).float().median()) > 100
    for fam in ("whole", "tail", "portions", "mixed"):
        for page in (8, 32):
            got = run_trace(folder, dtype, FAMILIES[fam](reqs), page)
            for rid, t in reqs.items():
                check_close(traces.as_matrix(got[rid], len(t)), ref[rid].numpy(), dtype, f"sharp {dtype} {fam} page {page} {rid}")


# ------------------------------------------------------------------------------------------ generation
def check_greedy_tokens(cfg, w, prompt, out, dtype):
    """Teacher-forced on the engine's own tokens: each is the plain model's arg-max given the tokens before it, or lies
    within the precision's bound of it."""
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(cfg, w, seq)[len(prompt) - 1:].numpy()
    tol = 2 * K[dtype] * (1 + np.abs(ref).max())
    for j, t in enumerate(out):
        best = int(ref[j].argmax())
        assert t == best or ref[j][best] - ref[j][t] <= tol, f"token {j}: {t} where the plain model has {best}"


@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_engine(models, name):
    from cellm_b200 import Engine, SamplingParams
    folder, reqs, _ = models[name]
    cfg, w = load_plain(folder)
    prompts = [t for t in reqs.values() if len(t) < 140][:5]
    eng = Engine(folder, dtype="float32", tokens_per_block=8, total_blocks=96, max_num_seqs=3, max_batch_tokens=48,
                 prefill_chunk=24)
    outs = eng.generate(prompts, SamplingParams.greedy(12, stop_eos=False))
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        check_greedy_tokens(cfg, w, prompt, out, "float32")
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"] and s["free_slots"] == 3


def test_bfloat16_generation_runs_ahead_and_frees(models):
    from cellm_b200 import Engine, SamplingParams
    folder, reqs, _ = models["c"]
    cfg, w = load_plain(folder)
    prompts = list(reqs.values())
    eng = Engine(folder, dtype="bfloat16", tokens_per_block=16, total_blocks=80, max_num_seqs=4, max_batch_tokens=64,
                 prefill_chunk=32)
    outs = eng.generate(prompts, SamplingParams.greedy(20, stop_eos=False))
    assert all(len(o) == 20 for o in outs)
    for prompt, out in zip(prompts, outs):
        check_greedy_tokens(cfg, w, prompt, out, "bfloat16")
    # slots and pages given back and used again: the plain model's tokens again (in another batch the kernels that serve
    # a step may differ, so a near-tie may fall the other way: each run is held to the plain model, not to the other)
    again = eng.generate(prompts[:2], SamplingParams.greedy(20, stop_eos=False))
    for prompt, out in zip(prompts[:2], again):
        check_greedy_tokens(cfg, w, prompt, out, "bfloat16")
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]


# ------------------------------------------------------------------------------------- the kernels by themselves
DEV = "cuda:0"


def _t(x, dtype):
    return x.to(dtype).to(DEV).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,groups,gate", [(96, 1, True), (96, 4, True), (120, 3, False), (2048, 2, True)])
def test_gated_norm_add(dtype, H, groups, gate):
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(1)
    T = 7
    x = torch.randn(T, H, generator=g)
    m, z = _t(torch.randn(T, H, generator=g) * 3, dtype), _t(torch.randn(T, H, generator=g) * 2, dtype)
    b, w = _t(torch.randn(H, generator=g), dtype), _t(1 + 0.3 * torch.randn(H, generator=g), dtype)
    md, zd, bd, wd = (v.cpu().double() for v in (m, z, b, w))
    c = _t(torch.randn(H, generator=g), dtype) if H == 96 else None          # a bias the result has not taken yet
    if c is not None:
        md = md + c.cpu().double()
    v = md * torch.sigmoid(zd + bd) if gate else md
    want = x.double() + plain.group_rms_norm(v, wd, groups, 1e-5)
    xd = x.to(DEV)
    if gate and groups == 2:        # the gate as 32-bit columns of a wider matrix (where a sublayer's first product leaves it)
        wide = torch.zeros(T, H + 24, device=DEV)
        wide[:, 16:16 + H] = z.float()
        z = wide[:, 16:16 + H]
    y = ops.gated_norm_add(xd, m, z if gate else None, b if gate else None, w, groups, 1e-5, m_bias=c)
    torch.testing.assert_close(xd.cpu().double(), want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(y.cpu().double(), want.to(dtype).double(), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-5)


@pytest.mark.parametrize("groups", [1, 2, 5])
def test_rms_norm_in_groups(groups):
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(2)
    x, w = torch.randn(6, 80, generator=g) * 4, 1 + 0.2 * torch.randn(80, generator=g)
    want = plain.group_rms_norm(x.double(), w.double(), groups, 1e-6)
    y = ops.add_rmsnorm(x.to(DEV), None, w.to(DEV), 1e-6, torch.float32, None, groups)
    torch.testing.assert_close(y.cpu().double(), want, rtol=1e-5, atol=1e-5)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    y = ops.add_rmsnorm(x.to(DEV), None, w.to(DEV), 1e-6, torch.float32, rows, groups)
    torch.testing.assert_close(y.cpu().double(), want[[4, 1]], rtol=1e-5, atol=1e-5)


def test_embedding_scale():
    from cellm_b200 import ops
    from cellm_b200.ops._state import error_word
    table = torch.randn(20, 24).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 19, 0], dtype=torch.int32, device=DEV)
    out = ops.embed(table, ids, error_word(torch.device(DEV)), 7.5)
    torch.testing.assert_close(out.cpu(), table.cpu().float()[[3, 19, 0]] * 7.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mingru_scan_whole_against_token_by_token(dtype):
    """The recurrence over a portion, over the same tokens one by one, and in two requests side by side whose slots
    are not in order, against the plain recurrence; a decay near one keeps the first tokens visible at the end."""
    from cellm_b200 import ops
    from cellm_b200.ops._state import error_word
    g = torch.Generator().manual_seed(3)
    T, W = 150, 72
    proj = torch.randn(T, 3 * W, generator=g) * 2
    proj[:, :W] -= 3.0                               # small z: a long memory
    bz, bx = torch.randn(W, generator=g) * 0.3, torch.randn(W, generator=g) * 0.3
    z = torch.sigmoid(proj[:, :W].double() + bz.double())
    u = proj[:, W:2 * W].double() + bx.double()
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = proj[:, 2 * W:].double()
    S, rows = torch.zeros(W, dtype=torch.float64), []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t] * torch.sigmoid(gate[t]))
    want = torch.stack(rows)
    err = error_word(torch.device(DEV))
    pd, bzd, bxd = proj.to(DEV), _t(bz, torch.float32), _t(bx, torch.float32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    state = torch.zeros(3, W, device=DEV)
    out = ops.mingru_scan(pd, bzd, bxd, state, i32([2]), i32([0, T]), dtype, err)
    torch.testing.assert_close(out.cpu().double(), want, **tol)
    torch.testing.assert_close(state[2].cpu().double(), S, rtol=1e-5, atol=1e-6)
    assert float(state[:2].abs().max()) == 0.0
    state2 = torch.zeros(3, W, device=DEV)
    outs = [ops.mingru_scan(pd[t:t + 1], bzd, bxd, state2, i32([1]), i32([0, 1]), dtype, err) for t in range(T)]
    assert torch.equal(torch.cat(outs), out) and torch.equal(state2[1], state[2])        # cut anywhere: the same bits
    # two requests in one launch: the first 60 tokens in slot 2, tokens 60.. continuing the state slot 0 holds
    state3 = torch.zeros(3, W, device=DEV)
    ops.mingru_scan(pd[:60], bzd, bxd, state3, i32([0]), i32([0, 60]), dtype, err)
    both = ops.mingru_scan(torch.cat([pd[:60], pd[60:]]), bzd, bxd, state3, i32([2, 0]), i32([0, 60, T]), dtype, err)
    assert torch.equal(both, out) and torch.equal(state3[0], state[2])
    # long portions under bfloat16 are walked in runs side by side: the same recurrence up to rounding, also for
    # a request of one token and one whose runs are not all full beside the long one
    state4 = torch.zeros(3, W, device=DEV)
    ops.mingru_scan(pd[:1], bzd, bxd, state4, i32([1]), i32([0, 1]), dtype, err)
    runs = ops.mingru_scan(torch.cat([pd, pd[1:2]]), bzd, bxd, state4, i32([0, 1]), i32([0, T, T + 1]), dtype, err, max_q_len=T)
    torch.testing.assert_close(runs[:T].cpu().double(), want, **tol)
    torch.testing.assert_close(runs[T:].cpu().double(), want[1:2], **tol)
    torch.testing.assert_close(state4[0].cpu().double(), S, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_product_with_pitches(dtype):
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(4)
    T, heads, N, K = 37, 3, 20, 28
    x, w = _t(torch.randn(T, heads, K + 5, generator=g), dtype), _t(torch.randn(heads, N, K, generator=g), dtype)
    out = torch.zeros(T, heads, N + 7, dtype=dtype, device=DEV)
    ops.head_product(x[:, :, :K], w, out[:, :, 3:3 + N])
    want = torch.einsum("thk,hnk->thn", x[:, :, :K].cpu().double(), w.cpu().double())
    tol = dict(rtol=2e-2, atol=5e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out[:, :, 3:3 + N].cpu().double(), want, **tol)
    assert float(out[:, :, :3].abs().max()) == 0.0 and float(out[:, :, 3 + N:].abs().max()) == 0.0


@pytest.mark.parametrize("T,heads,N,K", [(5, 3, 40, 128), (16, 2, 16, 64), (1, 4, 100, 192)])
def test_head_product_of_few_tokens(T, heads, N, K):
    """bfloat16 and at most 16 tokens: the form that reads each matrix row once."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(6)
    x, w = _t(torch.randn(T, heads, K, generator=g), torch.bfloat16), _t(torch.randn(heads, N, K, generator=g), torch.bfloat16)
    out = ops.head_product(x, w)
    want = torch.einsum("thk,hnk->thn", x.cpu().double(), w.cpu().double())
    torch.testing.assert_close(out.cpu().double(), want, rtol=2e-2, atol=8e-2)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_act(act):
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(5)
    gu, bg, bu = torch.randn(9, 2 * 50, generator=g) * 3, torch.randn(50, generator=g), torch.randn(50, generator=g)
    a, u = gu[:, :50].double() + bg.double(), gu[:, 50:].double() + bu.double()
    want = (plain.gelu_tanh(a) if act == "gelu_tanh" else a * torch.sigmoid(a)) * u
    h = ops.gated_act(gu.to(DEV), bg.to(DEV), bu.to(DEV), act, torch.float32)
    torch.testing.assert_close(h.cpu().double(), want, rtol=1e-5, atol=1e-5)
    h = ops.gated_act(gu.to(DEV), None, None, act, torch.float32)
    a, u = gu[:, :50].double(), gu[:, 50:].double()
    want = (plain.gelu_tanh(a) if act == "gelu_tanh" else a * torch.sigmoid(a)) * u
    torch.testing.assert_close(h.cpu().double(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [gru(40), gru(64, mlp=dense(48)), attention(2, 16, 8, 24, 20, mlp=dense(56)),
                                   attention(4, 16, 16, 16, 32)])
def test_one_layer_alone(tmp_path, dtype, layer):
    """A model of a single layer: the mixer, its gate and norm (and feed-forward) with nothing around them."""
    config = model_config(97, 48, 2.0, 1e-5, 2, [layer])
    folder = write_model(tmp_path / "one", config, 9)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(1)
    reqs = {"x": rng.integers(0, 97, 45).tolist(), "y": rng.integers(0, 97, 3).tolist()}
    for fam in ("whole", "portions", "mixed"):
        got = run_trace(folder, dtype, FAMILIES[fam](reqs), 8)
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), plain.forward(cfg, w, toks).numpy(), dtype, f"{layer['type']} {fam} {rid}")


@pytest.mark.parametrize("nh,kw,dv,page", [(8, 80, 64, 16), (16, 576, 512, 32), (5, 48, 32, 8), (3, 64, 48, 16), (2, 144, 128, 64),
                                              (4, 400, 384, 16), (2, 112, 96, 8), (3, 96, 80, 16), (70, 32, 16, 16)])
def test_latent_attention_kernel_against_plain_kernel_and_torch(nh, kw, dv, page):
    """The tensor-core kernel alone: portions of several requests at contexts that end inside a page and inside a block
    of keys, whole and cut into pieces, against 64-bit torch over the same rounded inputs and the plain kernel."""
    from cellm_b200 import ops
    from cellm_b200.ops._state import error_word
    g = torch.Generator().manual_seed(nh * 1000 + kw)
    q_lens, ctx_lens = [70, 1, 9, 1], [131, 300, 0, 63]
    B, T = len(q_lens), sum(q_lens)
    width = max((c + n + page - 1) // page for c, n in zip(ctx_lens, q_lens))
    n_pages = B * width + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, width), -1, dtype=torch.int32)
    for b in range(B):
        for i in range((ctx_lens[b] + q_lens[b] + page - 1) // page):
            table[b, i] = order.pop()
    pool = (torch.randn(n_pages, 1, page, kw, generator=g) * 0.7).to(torch.bfloat16)
    q = (torch.randn(T, nh * kw, generator=g) * 0.7).to(torch.bfloat16)
    scale = 1.7 * kw ** -0.5
    want = torch.zeros(T, nh, dv, dtype=torch.float64)
    t = 0
    for b in range(B):
        total = ctx_lens[b] + q_lens[b]
        keys = torch.stack([pool[table[b, j // page], 0, j % page] for j in range(total)]).double()
        for i in range(q_lens[b]):
            qi = q[t].double().reshape(nh, kw)
            s = (qi @ keys[:ctx_lens[b] + i + 1].T) * scale
            want[t] = torch.softmax(s, -1) @ keys[:ctx_lens[b] + i + 1, :dv]
            t += 1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu = i32([0] + list(np.cumsum(q_lens)))
    err = error_word(torch.device(DEV))
    positions = i32([c + j for c, n in zip(ctx_lens, q_lens) for j in range(n)])
    seq = i32([b for b, n in enumerate(q_lens) for _ in range(n)])
    poold, qd, tabled = pool.to(DEV), q.to(DEV), table.to(DEV)
    plain_out = ops.attention_plain(qd, poold, poold, positions, seq, tabled, nh, scale, 0, err, value_dim=dv)
    torch.testing.assert_close(plain_out.cpu().double().reshape(T, nh, dv), want, rtol=2e-2, atol=2e-2)
    for nsplit in (1, 3, 8):
        out = ops.attention_latent(qd, poold, cu, i32(ctx_lens), tabled, q_lens, nh, dv, scale, nsplit, err)
        torch.testing.assert_close(out.cpu().double().reshape(T, nh, dv), want, rtol=2e-2, atol=2e-2)
    assert int(err.item()) == 0


def test_latent_attention_takes_the_tensor_core_kernel(models):
    from cellm_b200.runtime import program
    folder, reqs, ref = models["c"]
    before = program.CALLS["cellm_attention_latent"]
    run_trace(folder, "bfloat16", traces.whole({"r0": reqs["r0"]}), 16)
    assert program.CALLS["cellm_attention_latent"] > before
    before = program.CALLS["cellm_attention_latent"]
    run_trace(folder, "float32", traces.whole({"r0": reqs["r0"]}), 16)
    assert program.CALLS["cellm_attention_latent"] == before


# --------------------------------------------------------------------------------------------- command lines
def test_command_lines_take_the_design(models, tmp_path):
    """bin/infer generates greedily from a folder of this design as the plain model does; bin/trace_run replays a mixed
    trace of it from standard input."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, reqs, ref = models["a"]
    cfg, w = load_plain(folder)
    prompt = reqs["r1"]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "infer"), "--model", folder, "--dtype", "float32", "--tokens",
                        ",".join(map(str, prompt)), "--gen", "6", "--temperature", "0", "--stop-eos", "false",
                        "--tokens-per-block", "8"], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    out = [int(t) for t in [l for l in p.stdout.splitlines() if l.startswith("tokens:")][0].split(":")[1].split(",")]
    seq = list(prompt) + out[:-1]
    want = plain.forward(cfg, w, seq)[len(prompt) - 1:].numpy()
    tol = 2 * K["float32"] * (1 + np.abs(want).max())
    assert all(want[j].max() - want[j][t] <= tol for j, t in enumerate(out))
    steps = traces.mixed(reqs, seed=4)
    out_dir = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "bfloat16",
                        "--out", str(out_dir), "--max-tokens", str(traces.max_live_tokens(steps))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outs = []
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        outs.append(np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, cfg["vocab"]) if n_want else None)
    got = traces.collect(steps, outs)
    for rid, toks in reqs.items():
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], "bfloat16", f"trace_run {rid}")


def test_latent_attention_kernel_refuses_what_it_does_not_take():
    """Widths that are no multiples of 16, values wider than its warps can split: the entry point says so (the executor
    sends these to the plain kernel)."""
    from cellm_b200.ops import _lib
    supports = _lib.fn("attention_latent", "cellm_attention_latent_supports")
    assert supports(576, 512) == 1 and supports(80, 64) == 1 and supports(640, 512) == 1
    assert supports(88, 64) == 0 and supports(80, 72) == 0 and supports(800, 768) == 0 and supports(64, 80) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gates_as_products_of_their_own(models, dtype):
    """A sublayer that declines the gate's rows (here: every one, by the arrangement's `stack_gates` parameter) leaves
    the gate a product of its own before the gate-and-norm kernel; the logits are the plain model's either way."""
    import dataclasses
    from cellm_b200.config import load_config, parse_dtype
    from cellm_b200.models.decoder import DecoderModel
    from cellm_b200.runtime import program
    from cellm_b200.weights import load_weights
    folder, reqs, ref = models["a"]
    cfg, plan = load_config(folder)
    layers = tuple(dataclasses.replace(l, block=dataclasses.replace(l.block, params={**l.block.params, "stack_gates": False}))
                   for l in plan.layers)
    plan = dataclasses.replace(plan, layers=layers)
    model = DecoderModel(plan, load_weights(folder, plan, parse_dtype(dtype), "cuda:0"), parse_dtype(dtype), "cuda:0")
    assert not any(b.stacked.get(n) for b in model.blocks for n in ("mixer", "feed_forward"))
    some = {rid: reqs[rid] for rid in ("r2", "r4", "r6")}
    for fam in ("whole", "mixed"):
        got = run_trace((cfg, plan, model), dtype, FAMILIES[fam](some), PAGE["a"])
        for rid, toks in some.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"own gate products {dtype} {fam} {rid}")
