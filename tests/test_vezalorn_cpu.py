"""The Vezalorn design without a GPU: its configuration reader, the plan and tensor table it builds, what its
cache needs, and which kernels a step launches (entry points replaced by recorders, zero weights)."""
import copy

import pytest
import torch

from launch_recorder import Recorder, run_step, zero_model


def config(layers=None, **over):
    attn = {"heads": 4, "dim": 32, "rot_dim": 16, "vdim": 48, "kv_rank": 64, "scale": 0.125, "rot": {"base": 10000.0, "dims": 16}}
    d = {"architecture": "Vezalorn", "vocab": 1000, "width": 128, "embedding": {"scale": 3.0},
         "norm": {"eps": 1e-5, "groups": 2},
         "layers": layers if layers is not None else [
             {"type": "mingru", "mixer": {"width": 192}, "mlp": None},
             {"type": "latent_attention", "mixer": attn, "mlp": {"kind": "dense", "ff": 256}}]}
    d.update(over)
    return d


def test_config_round_trip_and_plan():
    from cellm_b200.config import config_from_dict
    from cellm_b200.parts.base import FixedState, PagedKV
    from cellm_b200.weights.loader import expected_tensors
    cfg, plan = config_from_dict(config())
    assert cfg.to_dict() == config()
    assert (plan.hidden_size, plan.vocab_size, plan.tied) == (128, 1000, True)
    assert plan.embedding.params["scale"] == 3.0 and plan.final_norm.params["groups"] == 2
    want = {n: tuple(ts.shape) for n, ts in expected_tensors(plan).items()}
    assert want == {
        "embed": (1000, 128), "final.norm": (128,),
        "l0.norm1": (128,), "l0.rg1": (128, 128), "l0.rg1.b": (128,),
        "l0.mix.z": (192, 128), "l0.mix.z.b": (192,), "l0.mix.x": (192, 128), "l0.mix.x.b": (192,), "l0.mix.g": (192, 128),
        "l0.mix.o": (128, 192),
        "l1.norm1": (128,), "l1.norm2": (128,), "l1.rg1": (128, 128), "l1.rg1.b": (128,), "l1.rg2": (128, 128), "l1.rg2.b": (128,),
        "l1.mix.q": (4 * 48, 128), "l1.mix.dkv": (80, 128), "l1.mix.dkv.norm": (64,), "l1.mix.uk": (4 * 32, 64),
        "l1.mix.uv": (4 * 48, 64), "l1.mix.o": (128, 4 * 48),
        "l1.mlp.gate": (256, 128), "l1.mlp.gate.b": (256,), "l1.mlp.up": (256, 128), "l1.mlp.up.b": (256,),
        "l1.mlp.down": (128, 256), "l1.mlp.down.b": (128,)}
    cfg, plan, model = zero_model(config())
    assert model.cache_needs() == [FixedState((192,), torch.float32), PagedKV(1, 80, 0, values=False)]
    assert model.graph_safe


@pytest.mark.parametrize("change,message", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].update(groups=3), "norm groups"),
    (lambda d: d["layers"][0].update(type="lstm"), "mixer type"),
    (lambda d: d["layers"][1]["mlp"].update(kind="routed"), "feed-forward kind"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"].update(width=0), "width"),
])
def test_config_faults_are_named(change, message):
    from cellm_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(config())
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_the_architecture_is_found_by_its_one_string():
    from cellm_b200.config import ConfigError, resolve_architecture
    assert resolve_architecture({"architecture": "Vezalorn"}) == "Vezalorn"
    assert resolve_architecture({"model_type": "vezalorn"}) == "Vezalorn"
    with pytest.raises(ConfigError, match="unsupported model"):
        resolve_architecture({"architecture": "Nothing"})


def test_cache_group_without_values_keeps_one_pool():
    from cellm_b200.cache.manager import CacheManager
    from cellm_b200.parts.base import PagedKV
    cm = CacheManager([PagedKV(1, 80, 0, values=False), PagedKV(2, 16, 0), PagedKV(1, 80, 0, values=False)], [None] * 3, 8, 6, 2,
                      torch.bfloat16, "cpu")
    assert tuple(cm.k_pools[0].shape) == (2, 6, 1, 8, 80) and cm.v_pools[0] is None and cm.v_pools[1] is not None
    assert cm.bytes_per_token() == 2 * (2 * 80 + 2 * 2 * 16)
    b = cm.bindings([torch.zeros(1, 6, dtype=torch.int32)] * 2)
    assert b[0].v is None and b[1].v is not None and b[2].k.data_ptr() != b[0].k.data_ptr()


def names_of(rec):
    return [n.replace("cellm_", "") for n in rec.names()]


def test_decode_step_kernels(monkeypatch):
    """One token for each of three requests: a recurrent layer without a feed-forward, a latent attention layer with
    one. The stream is cast once; after that every gate-and-norm kernel leaves the next sublayer's input."""
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(config())
    run_step(model, plan, [1, 1, 1], [40, 7, 300])
    assert names_of(rec) == [
        "embed", "stream_cast",
        "gemm_tcgen05", "mingru_scan", "gemm_tcgen05",                          # z | candidate | gate | the stream's gate, the recurrence, the way out
        "gated_norm_add",                                                        # gate + norm + sum (the gate lies behind the product's own columns)
        "gemm_tcgen05", "latent_prep", "head_product", "attention_latent", "head_product", "gemm_tcgen05",
        "gated_norm_add",
        "gemm_tcgen05", "gated_act", "gemm_tcgen05",                             # gate | up | the stream's gate, activation, the way back
        "gated_norm_add",                                                        # (its bias is added by the gate-and-norm kernel)
        "add_rmsnorm", "gemm_tcgen05"]
    prep = rec.of("cellm_latent_prep")[0]
    assert prep[15:22] == (3, 4, 32, 16, 64, 16, prep[21]) and prep[12] is not None          # tokens, heads, dim, rot_dim, rank, rot; a cache to write
    att = rec.of("cellm_attention_latent")[0]
    assert (att[9], att[10], att[14], att[15], att[16]) == (3, 3, 4, 80, 64)                 # requests, tokens, heads, row width, value width
    norm = rec.of("cellm_gated_norm_add")[0]
    assert (norm[10], norm[11], norm[12]) == (3, 128, 2) and norm[3] is not None and norm[9] is not None and norm[2] is None
    assert (norm[4], norm[5]) == (3 * 192 + 128, 0)                                           # the gate: 32-bit, behind z, candidate and gate
    assert rec.of("cellm_gated_norm_add")[1][4:6] == (4 * 48 + 80 + 128, 1)                   # behind queries, latent and key part
    assert rec.of("cellm_gated_norm_add")[2][2] is not None                                   # the feed-forward's last bias
    assert [g[4] for g in rec.of("cellm_gemm_tcgen05")][:1] == [3 * 192 + 128]
    final = rec.of("cellm_add_rmsnorm")[0]
    assert final[8] == 2                                                                      # the model's norm is in groups too
    assert rec.of("cellm_embed")[0][7] == 3.0


def test_thirty_two_bit_takes_the_plain_kernels(monkeypatch):
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(config(), dtype=torch.float32)
    run_step(model, plan, [5, 1], [0, 19])
    names = set(names_of(rec))
    assert "attention_plain" in names and "gemm_plain" in names
    assert not names & {"attention_latent", "gemm_tcgen05", "stream_cast"}                   # the 32-bit stream is read as it is
    plain = rec.of("cellm_attention_plain")[0]
    assert (plain[11], plain[12], plain[13], plain[14]) == (4, 1, 80, 64)                     # heads on one key/value head; values: a row's first 64


def test_prompt_step_kernels(monkeypatch):
    """A long portion: the recurrence in runs (the same entry point, told the longest portion), per-head products on
    the tensor cores."""
    rec = Recorder(monkeypatch)
    cfg, plan, model = zero_model(config())
    run_step(model, plan, [600], [0])
    scan = rec.of("cellm_mingru_scan")[0]
    assert scan[11:16] == (600, 1, 192, scan[14], 600)
    assert "head_product" not in names_of(rec)                      # all heads in one tensor-core launch, twice
    per_head = rec.of("cellm_head_product_mma")
    assert [(g[1], g[2], g[7], g[8], g[9], g[10]) for g in per_head] == [(4 * 80, 80, 600, 4, 64, 32), (4 * 48, 48, 600, 4, 48, 64)]
    att = rec.of("cellm_attention_latent")[0]
    # 38 tiles leave most of 148 SMs idle: the keys in pieces (two CTAs an SM wanted, at least two blocks of keys a piece)
    assert att[11] == (600 * 4 + 63) // 64 and att[18] == 5 and att[1] is not None
    rec.calls.clear()
    run_step(model, plan, [4096, 4096], [0, 0])
    att = rec.of("cellm_attention_latent")[0]
    assert att[11] == 2 * 4096 * 4 // 64 and att[18] == 1 and att[1] is None             # tiles enough: one piece
