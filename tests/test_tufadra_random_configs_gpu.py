"""Random Tufadra configurations (fixed seeds): widths that are and are not multiples of 8, key and value widths of every
relation (equal, either wider, wider than any fast kernel takes), one to four key/value heads with one to eight query
heads each, with and without a temperature, layers without a feed-forward, layers that run another's weights again,
experts with and without groups, groups of one, a top of one and of many, with and without a shared expert. Each is
replayed whole and as a mixed trace in both element types against the plain restatement, and generates through the
engine."""
import numpy as np
import pytest

import plain_tufadra as plain
import traces
from test_tufadra_gpu import attn, layer, load_plain, model_config, moe, run_trace, steady_routers, write_model
from tolerances import check_close

pytestmark = pytest.mark.gpu

SEEDS = list(range(14))


def random_config(seed):
    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([48, 54, 64, 96, 100, 128, 160])
    own = []
    for _ in range(int(rng.integers(1, 4))):
        kv = pick([1, 2, 3, 4])
        heads = kv * pick([1, 2, 3, 4, 8])
        dim = pick([8, 16, 20, 24, 32, 48, 64, 72, 136])
        vdim = pick([dim, dim, 8, 16, 24, 40, 64, 80, 136])
        temp = (round(float(rng.uniform(0.1, 1.0)), 3), pick([1, 3, 16, 64])) if rng.random() < 0.7 else None
        mixer = attn(heads, kv, dim, vdim, scale=round(dim ** -0.5 * float(rng.uniform(0.5, 2.0)), 4), q_temp=temp)
        mlp = None
        if rng.random() < 0.8:
            experts = pick([2, 4, 6, 8, 12, 16, 32])
            groups = None
            if rng.random() < 0.7:
                count = pick([c for c in (1, 2, 3, 4, 6, 8, 16, 32) if experts % c == 0])
                groups = (count, int(rng.integers(1, count + 1)))
            reach = experts if groups is None else groups[1] * (experts // groups[0])
            top = int(rng.integers(1, min(reach, 8) + 1))
            mlp = moe(pick([8, 16, 24, 40, 64]), experts, top, round(float(rng.uniform(0.5, 2.5)), 3), groups=groups,
                      shared=pick([None, 16, 33, 48]))
        own.append(layer(mixer, mlp))
    layers = list(own)
    for _ in range(int(rng.integers(0, 3))):          # some layers once more, anywhere behind their first run
        j = int(rng.integers(0, len(own)))
        at = int(rng.integers(layers.index(own[j]) + 1, len(layers) + 1))
        layers.insert(at, dict(own[j], weights_of=None))
    # weights_of names the place of the layer that has the tensors in the final list
    place = {id(l): i for i, l in enumerate(layers) if "weights_of" not in l}
    final = []
    for l in layers:
        if "weights_of" in l:
            src = next(o for o in own if o["mixer"] is l["mixer"] and o["mlp"] is l["mlp"])
            final.append(dict(src, weights_of=place[id(src)]))
        else:
            final.append(l)
    return model_config(int(rng.integers(50, 400)), width, 256, pick([1e-5, 1e-6]), final)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(tmp_path, seed):
    config = random_config(seed)
    rng = np.random.default_rng(seed)
    reqs = {f"r{j}": rng.integers(0, config["vocab"], int(n)).tolist() for j, n in enumerate(rng.integers(1, 90, 3))}
    page = [4, 8, 16, 32][seed % 4]
    for dtype in ("float32", "bfloat16"):
        folder = write_model(tmp_path / dtype, config, 77 + seed)
        if dtype == "bfloat16":
            steady_routers(folder)
        cfg, w = load_plain(folder)
        ref = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
        for fam, make in (("whole", traces.whole), ("mixed", traces.mixed)):
            got = run_trace(folder, dtype, make(reqs), page)
            for rid, toks in reqs.items():
                check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"seed {seed} {dtype} {fam} {rid}")


@pytest.mark.parametrize("seed", SEEDS[:4])
def test_random_configuration_generates(tmp_path, seed):
    from cellm_b200 import Engine, SamplingParams
    from test_tufadra_gpu import check_greedy_tokens
    config = random_config(seed)
    folder = write_model(tmp_path / "m", config, 5 + seed)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], int(n)).tolist() for n in (3, 40, 17)]
    eng = Engine(folder, dtype="float32", tokens_per_block=8, total_blocks=64, max_num_seqs=2, max_batch_tokens=32, prefill_chunk=16)
    outs = eng.generate(prompts, SamplingParams.greedy(8, stop_eos=False))
    for prompt, out in zip(prompts, outs):
        check_greedy_tokens(cfg, w, prompt, out, "float32")
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]
