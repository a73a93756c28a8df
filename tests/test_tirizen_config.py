"""Configuration, specification and build units of the Tirizen decoder (no GPU)."""

import copy
import json

import pytest

from quanta_b200.config import ConfigError, TirizenConfig
from quanta_b200.config.registry import load_config, resolve

RAW = {
    "architecture": "Tirizen", "vocab": 50, "width": 32, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-4},
    "streams": 2, "residual_mult": 0.6, "logit_scale": 0.25, "max_positions": 40,
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "tau": 8.0}, "mlp": None},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 24},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "q_temp": {"coef": 0.2, "every": 5}}},
        {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 5, "top": 2}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "kv_from": 1}},
    ],
}


def test_registry_finds_the_architecture_by_its_key():
    assert resolve(RAW).name == "Tirizen"
    assert resolve({"architectures": ["Tirizen"]}).config_cls is TirizenConfig


def test_fields_and_round_trip():
    cfg = TirizenConfig.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps) == (50, 32, 1.5, 1e-4)
    assert (cfg.streams, cfg.residual_mult, cfg.logit_scale, cfg.max_positions) == (2, 0.6, 0.25, 40)
    assert [l.type for l in cfg.layers] == ["gla", "attention", "attention"]
    assert cfg.layers[0].mlp is None and cfg.layers[2].mixer["kv_from"] == 1
    again = TirizenConfig.from_dict(cfg.to_dict())
    assert again == cfg and again.to_dict() == cfg.to_dict()
    plain = TirizenConfig.from_dict({k: v for k, v in RAW.items() if k not in ("streams", "residual_mult", "logit_scale")})
    assert (plain.streams, plain.residual_mult, plain.logit_scale) == (0, 1.0, 1.0)
    assert "streams" not in plain.to_dict()


@pytest.mark.parametrize("change,what", [
    (lambda r: r["layers"][0].update(type="sliding"), "type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="gated"), "kind"),
    (lambda r: r["layers"][1]["mixer"].pop("vdim"), "lacks"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"]["q_temp"].update(every=0), "q_temp"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=8), "differ"),
    (lambda r: r["layers"][2]["mlp"]["router"].update(top=6), "router.top"),
    (lambda r: r["layers"][0]["mixer"].update(dim=300), "between"),
    (lambda r: r["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda r: r.update(streams=17), "streams"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_refusals(change, what):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=what):
        TirizenConfig.from_dict(raw)


def test_specification_names_every_tensor_once(tmp_path):
    from quanta_b200.engine.model import Model, write_random_model
    cfg = TirizenConfig.from_dict(RAW)
    out = write_random_model(cfg, 1, tmp_path / "m")
    arch, again = load_config(out)
    assert arch.name == "Tirizen" and again.layers[0].mixer["decay_rank"] == 16
    model = Model(arch.build_spec(again), dtype="float32", device="cpu")
    names = [s.name for s in model.tensor_specs()]
    assert len(names) == len(set(names))
    shapes = {s.name: s.shape for s in model.tensor_specs()}
    assert shapes["embed"] == (50, 32) and shapes["pos"] == (40, 32) and "head" not in shapes
    assert shapes["l0.mix.a1"] == (16, 32) and shapes["l0.mix.a2"] == (16, 16) and shapes["l0.mix.norm"] == (12,)
    assert shapes["l0.mix.v"] == (24, 32) and shapes["l0.mix.o"] == (32, 24)
    assert shapes["l1.mix.q.norm"] == (32,) and shapes["l1.mix.k.norm"] == (16,) and shapes["l1.mix.g"] == (4, 32)
    assert shapes["l1.mix.v"] == (12, 32) and shapes["l1.mix.o"] == (32, 24)
    assert "l2.mix.k" not in shapes and "l2.mix.k.norm" not in shapes and "l2.mix.v" not in shapes
    assert shapes["l2.mlp.router"] == (5, 32) and shapes["l2.mlp.router.b"] == (5,) and shapes["l2.mlp.e4.down"] == (32, 16)
    assert shapes["l0.hc1.mix"] == (2, 2) and "l0.hc2.in" not in shapes and shapes["l1.hc2.out"] == (2,)
    # the run order: every layer once, the third reading the second's cache; caches and state per entry
    assert [(e.layer, e.read_cache_of) for e in model.schedule] == [(0, None), (1, None), (2, 1)]
    needs = model.cache_needs()
    assert needs[0] is None and needs[2] is None
    assert [(s.name, s.heads, s.width) for s in needs[1].streams] == [("k", 2, 8), ("v", 2, 6)]
    assert list(model.state_needs()[0]) == ["gla_state"] and model.state_needs()[0]["gla_state"][0] == (2, 8, 12)


def test_sizes_that_only_the_checkpoint_knows():
    cfg = TirizenConfig.from_dict({k: v for k, v in RAW.items() if k != "max_positions"})
    shapes = {"l0.mix.a1": (7, 32), "pos": (99, 32)}
    full = cfg.with_tensor_shapes(lambda n: shapes.get(n))
    assert full.layers[0].mixer["decay_rank"] == 7 and full.max_positions == 99
    with pytest.raises(ConfigError, match="a1"):
        cfg.with_tensor_shapes(lambda n: None)


def test_plain_residual_has_no_connection_tensors():
    from quanta_b200.engine.model import Model
    raw = {k: v for k, v in RAW.items() if k != "streams"}
    cfg = TirizenConfig.from_dict(raw)
    from quanta_b200.models.tirizen import build_spec
    model = Model(build_spec(cfg), dtype="float32", device="cpu")
    assert not [s.name for s in model.tensor_specs() if ".hc" in s.name]


def test_the_recurrence_is_a_build_unit_of_its_own():
    from quanta_b200.csrc import build
    where = build.entry_points()
    assert where["qb_gla"] == "linear_attention" and build.UNITS["linear_attention"] == ["gla.cu"]
    assert where["qb_streams_mix_rmsnorm"] == "core" and where["qb_head_norm_gate"] == "core"
