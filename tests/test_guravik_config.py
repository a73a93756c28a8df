"""Configuration, run order, specification and build units of the Guravik decoder (no GPU)."""

import copy
import json

import pytest

from quanta_b200.config import ConfigError, GuravikConfig
from quanta_b200.config.registry import load_config, resolve
from tests.plain import guravik_plain as P

RAW = {
    "architecture": "Guravik", "vocab": 50, "width": 32, "canon": {"taps": 2}, "embedding": {"scale": 1.5},
    "norm": {"eps": 1e-4}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "general_delta", "mixer": {"heads": 2, "dim": 8}, "mlp": None},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 24},
         "mixer": {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3,
                   "rot": {"base": 100.0, "dims": 4}}},
        {"type": "general_delta", "mixer": {"heads": 1, "dim": 16}, "mlp": {"kind": "dense", "ff": 20}},
        {"type": "general_delta", "mixer": {"heads": 1, "dim": 8}, "mlp": None},
    ],
}


def test_registry_finds_the_architecture_by_its_key():
    assert resolve(RAW).name == "Guravik"
    assert resolve({"architectures": ["Guravik"]}).config_cls is GuravikConfig


def test_fields_and_round_trip():
    cfg = GuravikConfig.from_dict(RAW)
    assert (cfg.vocab, cfg.width, cfg.canon_taps, cfg.embedding_scale, cfg.norm_eps) == (50, 32, 2, 1.5, 1e-4)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 3, 3)
    assert [l.type for l in cfg.layers] == ["general_delta", "latent_attention", "general_delta", "general_delta"]
    assert cfg.layers[0].mlp is None and cfg.layers[1].mlp["ff"] == 24
    again = GuravikConfig.from_dict(cfg.to_dict())
    assert again == cfg and again.to_dict() == cfg.to_dict()


def test_run_order_matches_the_plain_reading():
    cfg = GuravikConfig.from_dict(RAW)
    assert cfg.run_order() == P.run_order(RAW)
    assert cfg.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    for loop in ({"start": 0, "stop": 0, "times": 1}, {"start": 0, "stop": 4, "times": 2}, {"start": 3, "stop": 4, "times": 4},
                 {"start": 2, "stop": 2, "times": 5}):
        raw = dict(RAW, loop=loop)
        assert GuravikConfig.from_dict(raw).run_order() == P.run_order(raw)
    no_loop = {k: v for k, v in RAW.items() if k != "loop"}
    assert [i for i, _ in GuravikConfig.from_dict(no_loop).run_order()] == [0, 1, 2, 3]


@pytest.mark.parametrize("change,what", [
    (lambda r: r["layers"][0].update(type="sliding"), "type"),
    (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "dense"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].pop("kv_rank"), "lacks"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["canon"].update(taps=0), "tap"),
    (lambda r: r["layers"][2]["mixer"].update(dim=300), "limit"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_refusals(change, what):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=what):
        GuravikConfig.from_dict(raw)


def test_specification_names_every_tensor_once(tmp_path):
    from quanta_b200.engine.model import Model
    from quanta_b200.weights.safetensors_io import write_safetensors
    weights = P.draw_weights(RAW, seed=1, decay_rank=5)
    write_safetensors(tmp_path / "model.safetensors", weights)
    (tmp_path / "config.json").write_text(json.dumps(RAW))
    arch, cfg = load_config(tmp_path)
    assert [l.mixer.get("decay_rank") for l in cfg.layers] == [5, None, 5, 5]      # read from the checkpoint's shapes
    model = Model(arch.build_spec(cfg), dtype="float32", device="cpu")
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == {n: tuple(shape) for n, (shape, _) in P.tensor_shapes(RAW, 5).items()}
    assert [(e.layer, e.add_embedding) for e in model.schedule] == cfg.run_order()
    # a cache for every run of the attention layer, a state (recurrence and convolution inputs) for every run
    needs = model.cache_needs()
    assert [n is not None for n in needs] == [i == 1 for i, _ in cfg.run_order()]
    assert needs[1].streams[0].width == 12 + 4 and needs[1].streams[0].heads == 1
    states = model.state_needs()
    assert states[0]["delta_state"][0] == (2, 8, 8) and states[0]["conv_inputs"][0] == (1, 32)
    assert "delta_state" not in states[1] and states[1]["conv_inputs"][0] == (1, 32)


def test_every_entry_point_belongs_to_one_unit():
    from quanta_b200.csrc import build
    where = build.entry_points()
    assert where["qb_delta_rule"] == "recurrent" and where["qb_latent_attend"] == "latent" and where["qb_add_rmsnorm"] == "core"
    assert build._unassigned() == []
    assert sorted({p.name for u in build.UNITS for p in build.sources(u)}) == sorted(p.name for p in build.SRC_DIR.glob("*.cu"))
