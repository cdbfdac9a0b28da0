"""The Tufadra design against its plain restatement (tests/plain_tufadra.py): each mechanism's kernels alone, whole
models in every cutting of the requests, pages and slots that are used again, keys far away and at page borders, the
edges of the query temperature's steps, long decoding, sizes that differ in everything, and greedy generation through
the engine.

A mixture of experts chooses by comparing scores, and a score that bfloat16 moved by its rounding can fall on the
other side of a near tie, after which the logits differ outright. So whole models under bfloat16 get routers whose
choice does not hang on the last bits (`steady_routers`), while the routing itself, token by token with random
scores, is tested in 32-bit through whole models and in both types on the part alone, where the plain function is
given the very input the kernels read."""
import json
import os

import numpy as np
import pytest
import torch

import plain_tufadra as plain
import traces
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def attn(heads, kv_heads, dim, vdim, scale=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def moe(ff, experts, top, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    d = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp=None, weights_of=None):
    d = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


def model_config(vocab, width, max_positions, eps, layers):
    return {"architecture": "Tufadra", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps},
            "layers": layers}


# A: key and value widths differ both ways, a layer without a feed-forward, a layer that runs another's weights again,
# groups of one expert, no shared expert in one layer, one key/value head in one layer and as many as heads in another.
_A0 = layer(attn(6, 2, 16, 24, q_temp=(0.4, 16)), moe(40, 12, 4, 2.0, groups=(3, 2), shared=56))
_A3 = layer(attn(3, 1, 8, 8, scale=0.5), moe(24, 6, 1, 1.0, groups=(6, 3)))
CONFIG_A = model_config(300, 96, 400, 1e-5, [_A0, layer(attn(4, 4, 32, 16, q_temp=(1.0, 1))), dict(_A0, weights_of=0), _A3,
                                             dict(_A3, weights_of=3)])
# B: sizes that are multiples of nothing (no 16-byte row anywhere), no groups, top = all but one, no temperature
CONFIG_B = model_config(211, 54, 300, 1e-6, [
    layer(attn(3, 3, 10, 14), moe(21, 5, 4, 0.7, shared=33)),
    layer(attn(2, 1, 6, 5, q_temp=(0.25, 7)), moe(9, 4, 2, 1.3, groups=(2, 2))),
])
# C: heads of 64 with values as wide (the tensor-core attention kernels serve bfloat16), many experts
CONFIG_C = model_config(512, 128, 600, 1e-5, [
    layer(attn(4, 2, 64, 64, q_temp=(0.5, 32)), moe(64, 16, 3, 1.5, groups=(4, 2), shared=96)),
    layer(attn(8, 1, 32, 32), None),
    layer(attn(4, 2, 64, 64, q_temp=(0.5, 32)), moe(64, 16, 3, 1.5, groups=(4, 2), shared=96), weights_of=0),
])
# D: a width that is a multiple of 4 only beside products whose K is a multiple of 8, eight experts all kept
CONFIG_D = model_config(157, 100, 350, 1e-5, [
    layer(attn(4, 2, 24, 40, q_temp=(0.6, 50)), moe(48, 8, 8, 1.0, groups=(2, 2), shared=64)),
    layer(attn(5, 5, 16, 8), moe(32, 8, 2, 2.5, groups=(8, 5))),
])
CONFIGS = {"a": CONFIG_A, "b": CONFIG_B, "c": CONFIG_C, "d": CONFIG_D}
LENGTHS = {"a": [1, 9, 40, 64, 131, 77, 2], "b": [3, 55, 150, 18, 97], "c": [200, 1, 65, 129, 30, 260], "d": [70, 2, 33, 140, 17]}
PAGE = {"a": 8, "b": 16, "c": 16, "d": 4}


def write_model(folder, config, seed, dtype="bfloat16", init=None):
    from cellm_b200.weights import InitSpec, write_random_model
    init = init or InitSpec(linear_std=0.1, embedding_std=0.08, bias_std=0.1, norm_jitter=0.2)
    return write_random_model(str(folder), config, seed, dtype, init)


def load_plain(folder):
    from cellm_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n).clone() for n in sf.names()}


def steady_routers(folder):
    """Rewrites the model's routers so that no choice is a close call: router rows a hundred times smaller (all scores
    near one half, moved by the token in the fourth digit) and corrections, kept in 32-bit, that put the groups 0.1 apart
    in a shuffled order and the experts of a group 0.01 apart, so that neither two experts nor the sums of two groups'
    best pairs come near each other."""
    from cellm_b200.weights.safetensors_io import save_file
    cfg, w = load_plain(folder)
    g = torch.Generator().manual_seed(5)
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("mlp") is None or lay.get("weights_of") is not None:
            continue
        r = lay["mlp"]["router"]
        count = (r.get("groups") or {"count": 1})["count"]
        size = r["experts"] // count
        w[f"l{i}.mlp.router"] = (w[f"l{i}.mlp.router"].float() * 0.01).to(w[f"l{i}.mlp.router"].dtype)
        band = torch.randperm(count, generator=g).float() * 0.1
        within = torch.stack([torch.randperm(size, generator=g).float() * 0.01 for _ in range(count)])
        w[f"l{i}.mlp.correction"] = (band[:, None] + within).reshape(-1) - 0.05 * count
    save_file(w, os.path.join(folder, "model.safetensors"), {"format": "pt"})
    return folder


def run_trace(folder, dtype, steps, page, use_graphs=True, max_tokens=None):
    from cellm_b200.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or traces.max_live_tokens(steps), page, 4, use_graphs=use_graphs)
    outs = [rp.step(s["entries"], s["end"]) for s in steps]
    assert rp.cache.live == 0
    assert all(rp.cache.free_pages(g) == rp.cache.group_pages[g] for g in range(len(rp.cache.group_pages)))
    return traces.collect(steps, outs)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> dtype -> (folder, requests, plain logits). The bfloat16 folder has steady routers."""
    d = tmp_path_factory.mktemp("tf")
    out = {}
    for i, (name, config) in enumerate(CONFIGS.items()):
        rng = np.random.default_rng(17 + i)
        reqs = {f"r{j}": rng.integers(0, config["vocab"], n).tolist() for j, n in enumerate(LENGTHS[name])}
        out[name] = {}
        for dtype in ("float32", "bfloat16"):
            folder = write_model(d / f"{name}_{dtype}", config, 31 + i)
            if dtype == "bfloat16":
                steady_routers(folder)
            cfg, w = load_plain(folder)
            out[name][dtype] = (folder, reqs, {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()})
    return out


FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_matches_plain(models, name, dtype):
    folder, reqs, ref = models[name][dtype]
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
    folder, reqs, _ = models["a"]["float32"]
    steps = traces.mixed(reqs)
    assert len(reqs) > 4                                     # more requests than state slots
    assert traces.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_two_and_odd_sizes(models, dtype):
    folder, reqs, ref = models["b"][dtype]
    for sizes in ((2,), (3, 2, 5), (17, 2, 2, 31)):
        got = run_trace(folder, dtype, traces.portions(reqs, sizes), PAGE["b"])
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"b {dtype} portions {sizes} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_pages(models, dtype):
    """Most of the sequence decoded token by token: every page border and every step of the temperature on the decode path."""
    folder, reqs, ref = models["c"][dtype]
    some = {rid: reqs[rid] for rid in ("r0", "r5")}
    got = run_trace(folder, dtype, traces.tail_one_by_one(some, tail=190), 8)
    for rid, toks in some.items():
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"c {dtype} long tail {rid}")


def test_a_layer_that_runs_again_has_a_cache_of_its_own(models):
    from cellm_b200.config import load_config
    folder, _, _ = models["a"]["float32"]
    cfg, plan = load_config(folder)
    assert [e.layer for e in plan.order] == [0, 1, 0, 2, 2] and all(e.cache_of is None for e in plan.order)
    assert len(plan.layers) == 3


# ------------------------------------------------------- keys far away, page borders, the temperature's steps
def sharp_model(folder, seed, scale, dtype):
    """One layer of attention alone, its softmax so peaked (a large score scale) that a position's output is a few
    single keys, wherever they lie: a key lost at a page border, a wrong position's vector or a temperature that steps
    one token early or late changes the logits outright."""
    from cellm_b200.weights import InitSpec
    config = model_config(128, 64, 800, 1e-5, [layer(attn(4, 2, 16, 24, scale=scale, q_temp=(0.9, 64))),
                                               layer(attn(2, 1, 32, 16, scale=scale / 2, q_temp=(0.9, 64)))])
    return write_model(folder, config, seed, init=InitSpec(linear_std=0.25, embedding_std=0.1, bias_std=0.05, norm_jitter=0.1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_reaches_far_keys(tmp_path, dtype):
    # the norm over the projection leaves q and k with a root mean square of one, so q . k of 16 entries is about 4 wide,
    # and the temperature triples it far out; a rounding of the score by e moves the weights by that share, so the
    # 32-bit run has scores of a dozen or two and bfloat16, which rounds a score of size s by s / 256, the smaller scale
    folder = sharp_model(tmp_path / "sharp", 5, 1.0 if dtype == "float32" else 0.5, dtype)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg["vocab"], 700).tolist()
    reqs = {"long": toks, "short": toks[:70]}
    ref = {rid: plain.forward(cfg, w, t) for rid, t in reqs.items()}
    # the attention really is peaked and really reaches back
    t64 = {k: v.double() for k, v in w.items()}
    x0 = plain.embed_with_positions(t64["embed"], t64["pos"], toks)
    weights = []
    plain.attention(plain.offset_norm(x0, t64["l0.norm1"], 1e-5), t64, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5, weights)
    top, where = torch.stack(weights)[:, 600:].max(-1)
    assert float(top.median()) > (0.3 if dtype == "float32" else 0.08)
    assert float((torch.arange(600, 700)[None] - where).float().median()) > 100
    for fam in ("whole", "tail", "portions", "mixed"):
        for page in (8, 32):
            got = run_trace(folder, dtype, FAMILIES[fam](reqs), page)
            for rid, t in reqs.items():
                check_close(traces.as_matrix(got[rid], len(t)), ref[rid].numpy(), dtype, f"sharp {dtype} {fam} page {page} {rid}")


def test_temperature_steps_where_it_should():
    """The factor alone: it changes exactly at positions every * n - 1, in prompts and in single tokens."""
    from cellm_b200.ops._lib import fn, ptr, stream_of, tag
    from cellm_b200.ops._state import error_word
    for coef, every in ((0.5, 64), (1.25, 1), (0.3, 7)):
        positions = torch.tensor([0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 5 * every - 1, 5 * every, 1000],
                                 dtype=torch.int32).clamp_min(0)
        T, nh, hd = positions.numel(), 2, 8
        q = torch.ones(T, nh * hd, device=DEV)
        out = torch.empty_like(q)
        pos = positions.to(DEV)
        seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        rc = fn("kernels_common", "cellm_attn_prep")(ptr(out), ptr(q), nh * hd, None, None, 0, 1e-5, 0, coef, every, ptr(pos), ptr(seq),
                                                      None, 0, None, None, 0, 16, T, nh, 0, hd, hd, 0, 0, tag(q), ptr(error_word(torch.device(DEV))),
                                                      stream_of(q))
        assert rc == 0
        want = plain.query_temperature(1001, coef, every)[positions.long()]
        torch.testing.assert_close(out[:, 0].cpu().double(), want, rtol=1e-6, atol=1e-6)


# ------------------------------------------------------------------------------------------ generation
def check_greedy_tokens(cfg, w, prompt, out, dtype):
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(cfg, w, seq)[len(prompt) - 1:].numpy()
    tol = 2 * K[dtype] * (1 + np.abs(ref).max())
    for j, t in enumerate(out):
        best = int(ref[j].argmax())
        assert t == best or ref[j][best] - ref[j][t] <= tol, f"token {j}: {t} where the plain model has {best}"


@pytest.mark.parametrize("name", ["a", "d"])
def test_greedy_generation_through_the_engine(models, name):
    from cellm_b200 import Engine, SamplingParams
    folder, reqs, _ = models[name]["float32"]
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
    folder, reqs, _ = models["c"]["bfloat16"]
    cfg, w = load_plain(folder)
    prompts = list(reqs.values())
    eng = Engine(folder, dtype="bfloat16", tokens_per_block=16, total_blocks=80, max_num_seqs=4, max_batch_tokens=64,
                 prefill_chunk=32)
    outs = eng.generate(prompts, SamplingParams.greedy(20, stop_eos=False))
    assert all(len(o) == 20 for o in outs)
    for prompt, out in zip(prompts, outs):
        check_greedy_tokens(cfg, w, prompt, out, "bfloat16")
    again = eng.generate(prompts[:2], SamplingParams.greedy(20, stop_eos=False))
    for prompt, out in zip(prompts[:2], again):
        check_greedy_tokens(cfg, w, prompt, out, "bfloat16")
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]


def test_a_prompt_beyond_the_position_table_is_refused(models):
    from cellm_b200 import Engine, SamplingParams
    folder, _, _ = models["b"]["float32"]
    eng = Engine(folder, dtype="float32", tokens_per_block=16, total_blocks=64, max_num_seqs=2)
    with pytest.raises(Exception):
        eng.generate([[1] * 295], SamplingParams.greedy(10, stop_eos=False))       # 300 position vectors


# ------------------------------------------------------------------------------------- the parts by themselves
def _t(x, dtype):
    return x.to(dtype).to(DEV).contiguous()


def _ctx(T, dtype):
    from cellm_b200.ops._state import error_word
    from cellm_b200.parts.base import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return StepContext(T=T, B=1, dtype=dtype, device=torch.device(DEV), token_ids=i32([0] * T), positions=i32(list(range(T))),
                       seq_of_token=i32([0] * T), cu_seqlens=i32([0, T]), ctx_lens=i32([0]), slot_ids=i32([0]),
                       err=error_word(torch.device(DEV)), q_lens=[T], ctx_lens_host=[0], max_q_len=T, max_total_len=T)


ROUTED = [  # H, experts, top, ff, groups, keep, shared_ff
    (96, 12, 4, 40, 3, 2, 56), (54, 5, 4, 21, 1, 1, 33), (128, 16, 1, 64, 16, 5, 0), (64, 8, 8, 32, 2, 2, 16),
    (2048, 64, 6, 256, 8, 4, 512), (100, 6, 2, 24, 3, 3, 8), (256, 32, 3, 128, 4, 1, 0),
    (64, 4, 4, 4096, 1, 1, 0),          # a token's middles beyond 48 KB of shared memory in the second row-by-row kernel
]


@pytest.mark.parametrize("T", [1, 5, 16, 17, 150, 300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,E,top,ff,groups,keep,sff", ROUTED)
def test_routed_experts_against_plain(dtype, T, H, E, top, ff, groups, keep, sff):
    """The part alone on random inputs: the plain function reads the same (rounded) input and weights, so every choice
    is the same one unless two scores lie within 32-bit rounding of each other. Few tokens take the row-by-row kernels,
    many (under bfloat16) the grouped products."""
    from cellm_b200.parts.routed_experts import RoutedExperts
    if H == 2048 and T not in (5, 150):
        pytest.skip("the large shape at two sizes")
    g = torch.Generator().manual_seed(H * 7 + E)
    w = {"router": torch.randn(E, H, generator=g) * 3 / H ** 0.5, "correction": torch.randn(E, generator=g) * 0.2}
    for e in range(E):
        w[f"up_{e}"] = torch.randn(ff, H, generator=g) / H ** 0.5
        w[f"down_{e}"] = torch.randn(H, ff, generator=g) / ff ** 0.5
    if sff:
        w.update(shared_up=torch.randn(sff, H, generator=g) / H ** 0.5, shared_down=torch.randn(H, sff, generator=g) / sff ** 0.5,
                 shared_gate=torch.randn(1, H, generator=g) / H ** 0.5)
    w = {k: _t(v, dtype) for k, v in w.items()}
    params = {"hidden_size": H, "experts": E, "top": top, "ff_dim": ff, "activation": "gelu", "route_scale": 1.7, "groups": groups,
              "keep_groups": keep, "shared_ff": sff}
    part = RoutedExperts(params, w, dtype)
    x = _t(torch.randn(T, H, generator=g), dtype)
    got = part.forward(x, _ctx(T, dtype)).cpu().double()
    pw = {"router": w["router"], "correction": w["correction"]}
    for e in range(E):
        pw[f"e{e}.up"], pw[f"e{e}.down"] = w[f"up_{e}"], w[f"down_{e}"]
    if sff:
        pw.update({"shared.up": w["shared_up"], "shared.down": w["shared_down"], "shared.sg": w["shared_gate"]})
    pw = {k: v.cpu().double() for k, v in pw.items()}
    f = {"router": {"top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}, "shared": {"ff": sff} if sff else None}
    want = plain.mixture(x.cpu().double(), pw, "", f)
    tol = dict(rtol=3e-2, atol=3e-2 * float(want.abs().max())) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=2e-5 * float(want.abs().max()))
    torch.testing.assert_close(got, want, **tol)


def test_route_choice_and_weights():
    """The router alone against the plain choice, with ties (equal scores go to the lower index), groups of one, negative
    choice scores (a group that is not kept counts as minus infinity, not as zero) and a top of one."""
    from cellm_b200.ops._lib import fn, ptr, stream_of, tag
    g = torch.Generator().manual_seed(2)
    for E, top, groups, keep in ((8, 3, 4, 3), (6, 1, 6, 2), (12, 5, 1, 1), (16, 4, 4, 2), (64, 6, 8, 4)):
        T, H = 40, 32
        x = torch.randn(T, H, generator=g)
        router = torch.randn(E, H, generator=g) * 0.5
        x[3] = 0.0                                   # all scores one half: the correction alone chooses, with ties
        correction = torch.randn(E, generator=g) * 0.3 - 1.5            # choice scores below zero
        correction[1] = correction[0]
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, top, device=DEV)
        z = (x @ router.T).contiguous()
        zd, cd = z.to(DEV), correction.to(DEV)
        rc = fn("kernels_common", "cellm_route")(ptr(idx), ptr(wts), None, ptr(zd), E, ptr(cd), tag(cd), T, E, top, groups, keep, 2.5, 0,
                                                  stream_of(zd))
        assert rc == 0
        want_idx, want_w = plain.route(z.double(), correction.double(), top, {"count": groups, "keep": keep}, 2.5)
        assert torch.equal(idx.cpu().long(), want_idx), (E, top, groups, keep)
        torch.testing.assert_close(wts.cpu().double(), want_w, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [96, 100, 2048])
def test_norm_with_an_offset_and_two_addends(dtype, H):
    from cellm_b200.ops._lib import check, fn, ptr, stream_of, tag
    from cellm_b200.parts.norm import RMSNorm
    g = torch.Generator().manual_seed(3)
    T = 9
    x = torch.randn(T, H, generator=g) * 2
    a, b = _t(torch.randn(T, H, generator=g), dtype), _t(torch.randn(T, H, generator=g), dtype)
    w = _t(torch.randn(H, generator=g) * 0.1, dtype)
    norm = RMSNorm({"dim": H, "eps": 1e-5, "offset": 1.0}, {"weight": w}, dtype)
    assert norm.weight.dtype == torch.float32
    xd = x.to(DEV)
    y = torch.empty(T, H, dtype=dtype, device=DEV)
    check(fn("kernels_common", "cellm_add2_rmsnorm")(ptr(xd), ptr(a), ptr(b), ptr(norm.weight), tag(norm.weight), ptr(y), None, T, H, 1, 1e-5,
                                                     tag(dtype), stream_of(xd)), "add2_rmsnorm")
    s = x.double() + (a.cpu().double() + b.cpu().double())
    torch.testing.assert_close(xd.cpu().double(), s, rtol=1e-6, atol=1e-6)
    want = plain.offset_norm(s, w.cpu().double(), 1e-5)
    torch.testing.assert_close(y.cpu().double(), want, **(dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)))
    # the wanted rows only: the stream stays as it was
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    x2 = x.to(DEV)
    y2 = torch.empty(2, H, dtype=dtype, device=DEV)
    check(fn("kernels_common", "cellm_add2_rmsnorm")(ptr(x2), ptr(a), ptr(b), ptr(norm.weight), tag(norm.weight), ptr(y2), ptr(rows), 2, H, 1,
                                                     1e-5, tag(dtype), stream_of(x2)), "add2_rmsnorm")
    assert torch.equal(x2.cpu(), x)
    torch.testing.assert_close(y2.cpu().double(), want[[7, 2]], **(dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)))


def test_embedding_with_learned_positions():
    from cellm_b200 import ops
    from cellm_b200.ops._state import error_word
    table = torch.randn(20, 24).to(torch.bfloat16).to(DEV)
    pos_table = torch.randn(11, 24).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32, device=DEV)
    positions = torch.tensor([10, 0, 5, 4], dtype=torch.int32, device=DEV)
    out = ops.embed(table, ids, error_word(torch.device(DEV)), 1.0, pos_table, positions)
    torch.testing.assert_close(out.cpu(), table.cpu().float()[[3, 19, 0, 3]] + pos_table.cpu().float()[[10, 0, 5, 4]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention alone", "with experts", "one head, wide values", "equal widths", "wider than any fast kernel",
                                   "equal and odd", "five query heads a key head", "seven", "twelve", "sixteen"])
def test_one_layer_alone(tmp_path, dtype, which):
    lay = {"attention alone": layer(attn(4, 2, 16, 24, q_temp=(0.5, 8))),
           "with experts": layer(attn(2, 2, 8, 8), moe(24, 6, 2, 1.5, groups=(3, 2), shared=16)),
           "one head, wide values": layer(attn(1, 1, 16, 48, q_temp=(2.0, 3))),
           "equal widths": layer(attn(4, 1, 32, 32)),
           "wider than any fast kernel": layer(attn(2, 1, 136, 40, q_temp=(0.5, 8))),      # values in rows of their own width
           "equal and odd": layer(attn(3, 3, 20, 20)),
           "five query heads a key head": layer(attn(10, 2, 32, 32, q_temp=(0.3, 16))), "seven": layer(attn(7, 1, 64, 64)),
           "twelve": layer(attn(12, 1, 16, 24)), "sixteen": layer(attn(32, 2, 8, 8))}[which]
    config = model_config(97, 48, 64, 1e-5, [lay])
    folder = write_model(tmp_path / "one", config, 9)
    if dtype == "bfloat16":
        steady_routers(folder)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(1)
    reqs = {"x": rng.integers(0, 97, 45).tolist(), "y": rng.integers(0, 97, 3).tolist()}
    for fam in ("whole", "portions", "mixed"):
        got = run_trace(folder, dtype, FAMILIES[fam](reqs), 8)
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(got[rid], len(toks)), plain.forward(cfg, w, toks).numpy(), dtype, f"{which} {fam} {rid}")


@pytest.mark.parametrize("name", ["c", "a", "d"])
def test_bfloat16_takes_the_fast_attention_kernels(models, name):
    """Heads of 64 as they are, and heads of other and of unequal widths padded with zeros to 32, 64 or 128."""
    from cellm_b200.runtime import program
    folder, reqs, _ = models[name]["bfloat16"]
    rid = max(reqs, key=lambda r: len(reqs[r]))
    watched = ("cellm_attention_flash", "cellm_attention_decode", "cellm_attention_plain_wide", "cellm_attention_plain")
    before = {k: program.CALLS[k] for k in watched}
    run_trace(folder, "bfloat16", traces.tail_one_by_one({rid: reqs[rid]}, tail=8), 16)
    assert program.CALLS["cellm_attention_flash"] > before["cellm_attention_flash"]
    assert program.CALLS["cellm_attention_decode"] > before["cellm_attention_decode"]
    assert program.CALLS["cellm_attention_plain_wide"] == before["cellm_attention_plain_wide"]
    assert program.CALLS["cellm_attention_plain"] == before["cellm_attention_plain"]


# --------------------------------------------------------------------------------------------- command lines
def test_command_lines_take_the_design(models, tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, reqs, ref = models["a"]["float32"]
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
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
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
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], "float32", f"trace_run {rid}")
