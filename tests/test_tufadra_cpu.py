"""Tufadra without a GPU: its configuration reader, its plan (tensor names, run order, cache needs), which kernels a
step of it launches (entry points replaced by recorders), and the plain restatement's own pieces."""
import copy

import pytest
import torch

import plain_tufadra as plain
from launch_recorder import Recorder, run_step, zero_model

MIXER = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "q_temp": {"coef": 0.4, "every": 16}}
MLP = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 12, "top": 4, "scale": 2.0, "groups": {"count": 3, "keep": 2}},
       "shared": {"ff": 56}}
CONFIG = {"architecture": "Tufadra", "vocab": 300, "width": 96, "max_positions": 400, "norm": {"eps": 1e-5}, "layers": [
    {"type": "attention", "mixer": MIXER, "mlp": MLP},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 32, "vdim": 32, "scale": 0.2}, "mlp": None},
    {"type": "attention", "mixer": MIXER, "mlp": MLP, "weights_of": 0},
]}


def test_config_round_trip_and_plan():
    from cellm_b200 import parts  # noqa: F401
    from cellm_b200.config import config_from_dict
    from cellm_b200.parts.base import PagedKV
    from cellm_b200.weights.loader import expected_tensors
    cfg, plan = config_from_dict(copy.deepcopy(CONFIG))
    assert cfg.to_dict() == CONFIG
    assert [e.layer for e in plan.order] == [0, 1, 0] and len(plan.layers) == 2 and plan.max_positions == 400
    names = expected_tensors(plan)
    assert names["pos"].shape == (400, 96) and names["l0.mix.q.norm"].shape == (96,) and names["l0.mix.k.norm"].shape == (32,)
    assert names["l0.mix.v"].shape == (48, 96) and names["l0.mix.o"].shape == (96, 144)
    assert names["l0.mlp.e11.up"].shape == (40, 96) and names["l0.mlp.shared.sg"].shape == (1, 96) and names["l0.mlp.correction"].shape == (12,)
    assert not any(n.startswith("l2.") for n in names) and "l1.mlp.router" not in names
    assert plan.tied
    from cellm_b200.parts.attention import AttentionMixer
    # keys of 16 and values of 24 are kept in heads of 32 (zeros behind their entries); heads of 32 as they are
    assert AttentionMixer.cache_need(plan.layers[0].mixer.params) == PagedKV(2, 32, 0, True, 0)
    assert AttentionMixer.cache_need(plan.layers[1].mixer.params) == PagedKV(4, 32, 0, True, 0)
    assert AttentionMixer.cache_need({**plan.layers[0].mixer.params, "pad_heads": False}) == PagedKV(2, 16, 0, True, 24)
    assert AttentionMixer.cache_need({**plan.layers[0].mixer.params, "head_dim": 136}) == PagedKV(2, 136, 0, True, 24)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "feed-forward kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(groups={"count": 5, "keep": 2}), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(groups={"count": 6, "keep": 1}), "cannot give"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("max_positions"), "max_positions"),
])
def test_config_faults_name_the_key(change, message):
    from cellm_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(CONFIG)
    change(c)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(c)


def test_what_the_file_leaves_out_does_not_exist():
    from cellm_b200.config import config_from_dict
    c = copy.deepcopy(CONFIG)
    c["layers"][0]["mixer"].pop("q_temp")
    c["layers"][0]["mlp"].pop("shared")
    c["layers"][0]["mlp"]["router"].pop("groups")
    c["layers"][2] = dict(copy.deepcopy(c["layers"][0]), weights_of=0)
    cfg, plan = config_from_dict(c)
    assert plan.layers[0].mixer.params["query_temperature"] is None
    p = plan.layers[0].feed_forward.params
    assert p["shared_ff"] == 0 and p["groups"] == 1 and p["keep_groups"] == 1
    assert "shared_up" not in plan.layers[0].feed_forward.weights
    assert cfg.to_dict() == c


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_launches_of_a_step(monkeypatch, dtype):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(copy.deepcopy(CONFIG), dtype)
    run_step(model, plan, [5, 1], [0, 7])
    names = rec.names()
    product = "cellm_gemm_tcgen05" if dtype == torch.bfloat16 else "cellm_gemm_plain"
    experts = [product, "cellm_route", "cellm_experts_rowwise"]          # few tokens: the shared expert is walked with the chosen ones
    # portions of at most 16 (token, head) rows a key/value head: the decode kernel, also for the heads padded to 32
    attend = "cellm_attention_decode" if dtype == torch.bfloat16 else "cellm_attention_plain"
    wide = ["cellm_add_rmsnorm", product, "cellm_attn_prep", attend, product]
    equal = [product, "cellm_attn_prep", attend, product]
    assert names == (["cellm_embed_pos"] + wide + experts + ["cellm_add2_rmsnorm"] + equal + ["cellm_add_rmsnorm"] + wide[1:] + experts +
                     ["cellm_add2_rmsnorm", product])
    # both addends of a layer wait for the next norm: nothing is added into the stream by a kernel of its own
    assert "cellm_residual_add" not in names
    prep = rec.of("cellm_attn_prep")[0]
    assert prep[7] == 2 and abs(prep[8] - 0.4) < 1e-6 and prep[9] == 16 and prep[19:25] == (6, 2, 16, 24, 32, 32)
    prep = rec.of("cellm_attn_prep")[1]
    assert prep[7] == 2 and prep[8] == 0.0 and prep[19:25] == (4, 4, 32, 32, 32, 32)
    out_proj = rec.of(product)[1]
    assert out_proj[5] == 6 * 32           # K of the output product: the padded heads
    route = rec.of("cellm_route")[0]
    assert route[4] == 13 and route[7:12] == (6, 12, 4, 3, 2) and route[13] == 1       # 12 router rows and the gate's


def test_decoded_tokens_of_equal_widths_take_the_decode_kernel(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(copy.deepcopy(CONFIG), torch.bfloat16)
    run_step(model, plan, [1, 1, 1], [40, 7, 300])
    assert rec.names().count("cellm_attention_decode") == 3 and "cellm_attention_plain_wide" not in rec.names()


def test_heads_wider_than_the_fast_kernels_keep_their_widths(monkeypatch):
    rec = Recorder(monkeypatch)
    c = copy.deepcopy(CONFIG)
    c["layers"] = [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 136, "vdim": 40, "scale": 0.1}, "mlp": None}]
    cfg, plan, model = zero_model(c, torch.bfloat16)
    run_step(model, plan, [5, 1], [0, 7])
    assert rec.names().count("cellm_attention_plain_wide") == 1
    prep = rec.of("cellm_attn_prep")[0]
    assert prep[19:25] == (2, 1, 136, 40, 136, 40)


def test_plain_route_against_topk():
    g = torch.Generator().manual_seed(1)
    z = torch.randn(50, 12, generator=g, dtype=torch.float64)
    corr = torch.randn(12, generator=g, dtype=torch.float64) * 0.3
    chosen, weights = plain.route(z, corr, 4, None, 1.5)
    s = torch.sigmoid(z)
    assert torch.equal(chosen, (s + corr).topk(4, -1).indices)
    torch.testing.assert_close(weights.sum(-1), torch.full((50,), 1.5, dtype=torch.float64))
    # groups: an expert outside the kept groups is never chosen, however large its score
    z[:, 0] = 30.0
    z[:, 1] = -30.0
    corr[:] = 0.0
    chosen, _ = plain.route(z, corr, 2, {"count": 6, "keep": 1}, 1.0)      # groups of two: (0, 1) scores about 1.0
    s = torch.sigmoid(z).reshape(50, 6, 2).sum(-1)
    best = s.argmax(-1)
    assert all(set(chosen[t].tolist()) == {2 * int(best[t]), 2 * int(best[t]) + 1} for t in range(50))


def test_plain_temperature_and_norm():
    f = plain.query_temperature(130, 0.5, 64)
    assert float(f[0]) == 1.0 and float(f[62]) == 1.0 and abs(float(f[63]) - (1 + 0.5 * 0.6931471805599453)) < 1e-12
    assert float(f[126]) == float(f[63]) and abs(float(f[127]) - (1 + 0.5 * 1.0986122886681098)) < 1e-12
    x = torch.randn(3, 10, dtype=torch.float64)
    y = plain.offset_norm(x, torch.zeros(10, dtype=torch.float64), 0.0)
    torch.testing.assert_close((y * y).mean(-1), torch.ones(3, dtype=torch.float64))


def test_many_tokens_take_the_grouped_products(monkeypatch):
    """Under bfloat16 a step of 17 tokens or more sorts its (token, choice) slots by expert and runs both expert products
    as grouped tensor-core products over rows padded to whole tiles; fewer tokens, and 32-bit, walk the experts row by row."""
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(copy.deepcopy(CONFIG), torch.bfloat16)
    run_step(model, plan, [40, 1], [0, 7])
    names = rec.names()
    assert names.count("cellm_moe_sort") == 2 and names.count("cellm_gemm_grouped_tcgen05") == 6 and "cellm_experts_rowwise" not in names
    i = names.index("cellm_route")
    assert names[i - 1:i + 4] == ["cellm_gemm_tcgen05", "cellm_route", "cellm_gemm_grouped_tcgen05", "cellm_gemm_tcgen05",
                                  "cellm_moe_sort"]       # the router's sums, the choice, the shared expert (gelu in its first product)
    i = names.index("cellm_moe_sort")
    assert names[i:i + 5] == ["cellm_moe_sort", "cellm_moe_gather", "cellm_gemm_grouped_tcgen05", "cellm_gemm_grouped_tcgen05", "cellm_moe_combine"]
    S, E = 41 * 4, 12
    rows = -(-(S + E * 127) // 128) * 128
    sort = rec.of("cellm_moe_sort")[0]
    assert sort[4:7] == (S, E, rows // 128)
    shared_up, up, down = rec.of("cellm_gemm_grouped_tcgen05")[:3]
    assert shared_up[3:7] == (41, 56, 96, 1) and shared_up[11] is None and shared_up[12] == 0
    assert up[3:7] == (rows, 40, 96, 12) and up[12] == 0            # the exact gelu in the first product's epilogue
    assert down[3:7] == (rows, 96, 40, 12) and down[12] == -1
    rec2 = Recorder(monkeypatch)
    cfg, plan, model = zero_model(copy.deepcopy(CONFIG), torch.float32)
    run_step(model, plan, [40, 1], [0, 7])
    assert "cellm_moe_sort" not in rec2.names() and rec2.names().count("cellm_experts_rowwise") == 2
