"""Guravik decoder: from its configuration to a model specification.

Layers ``l<i>.``: RMS norm, a short convolution over time on the mixer's input (``canon1``), a mixer
(``general_delta``: the delta-rule recurrence with a decay per key channel; ``latent_attention``: softmax
attention through low-rank latents with a shared rotated key part and a sink), RMS norm on the mixer's
output, and where the layer has one a dense gated feed-forward between two more RMS norms.  A range of
layers may run several times with the same weights; every run has a cache and state of its own, and each
pass after the first starts from the residual stream plus the embedded tokens.  The embedding is scaled
by a constant; the head is the final RMS norm and a linear map.
"""

from __future__ import annotations

import math

from ..config.guravik import GuravikConfig
from ..config.registry import register_architecture
from ..parts.spec import ModelSpec, ScheduleEntry

# constants of the design
DECAY_SCALE = math.exp(-0.5)      # w = exp(-DECAY_SCALE * sigmoid(.))
UNIT_KEY_EPS = 1e-6               # u = k / sqrt(|k|^2 + UNIT_KEY_EPS)
DEFAULT_DECAY_RANK = 16           # inner rank of the decay when no checkpoint says otherwise (random models)


def layer_choice(cfg: GuravikConfig, i: int) -> tuple[str, dict]:
    layer = cfg.layers[i]
    p, m = f"l{i}.", layer.mixer
    mix = p + "mix."
    norm = lambda n: ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=p + n))  # noqa: E731
    if layer.type == "general_delta":
        mixer = ("delta_rule", dict(
            hidden_size=cfg.width, n_heads=m["heads"], dim=m["dim"], decay_rank=m.get("decay_rank", DEFAULT_DECAY_RANK),
            decay_scale=DECAY_SCALE, unit_eps=UNIT_KEY_EPS, norm_eps=cfg.norm_eps,
            names={"r": mix + "r", "k": mix + "k", "v": mix + "v", "g": mix + "g", "a": mix + "a", "a_bias": mix + "a.b",
                   "w1": mix + "w1", "w2": mix + "w2", "w_bias": mix + "w0", "gain": mix + "norm", "o": mix + "o"}))
    else:
        position = ("partial_rotary", dict(head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"]))
        mixer = ("latent_attention", dict(
            hidden_size=cfg.width, n_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
            q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], norm_eps=cfg.norm_eps, position=position,
            names={"dq": mix + "dq", "dq_norm": mix + "dq.norm", "uq": mix + "uq", "dkv": mix + "dkv",
                   "dkv_norm": mix + "dkv.norm", "uk": mix + "uk", "uv": mix + "uv", "o": mix + "o",
                   "sink": mix + "sink"}))
    params = dict(hidden_size=cfg.width, mixer=mixer, mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
                  conv=("residual_short_conv", dict(channels=cfg.width, taps=cfg.canon_taps, weight_name=p + "canon1")))
    if layer.mlp is not None:
        mlp = p + "mlp."
        params.update(
            feed_forward=("gated_dense", dict(hidden_size=cfg.width, inner_size=layer.mlp["ff"],
                                              names={"gate": mlp + "gate", "up": mlp + "up", "down": mlp + "down"})),
            feed_forward_norm=norm("norm2"), feed_forward_post_norm=norm("norm2b"))
    return ("sandwich_norm", params)


def build_spec(cfg: GuravikConfig) -> ModelSpec:
    return ModelSpec(
        name="Guravik", vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
        layers=[layer_choice(cfg, i) for i in range(len(cfg.layers))],
        final_norm=("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="final.norm")),
        head_name="head",
        embedding=("token_table", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="embed",
                                       scale=cfg.embedding_scale)),
        schedule=[ScheduleEntry(i, add_embedding=again) for i, again in cfg.run_order()],
    )


ARCHITECTURE = register_architecture(["Guravik", "guravik"], GuravikConfig, build_spec)
