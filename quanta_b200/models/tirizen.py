"""Tirizen decoder: from its configuration to a model specification.

The embedding is the token table times a constant plus a learned vector per position.  Layers ``l<i>.`` are
pre-norm sublayers (RMS norm) connected to one or several residual streams (``hc1`` / ``hc2``: how the mixer
and the feed-forward read the streams and write back); two kinds of mixer (``gla``: a linear recurrence with a
decay per key channel; ``attention``: softmax attention with a norm over the whole query / key projection, no
rotation, a query temperature that grows with the position, a gate per head, and optionally the keys and values
of an earlier layer); feed-forwards with the square of relu, dense or as routed experts whose weights are the
softmax over the chosen logits.  The head is the final RMS norm and the token table itself, times a constant.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tirizen import DEFAULT_DECAY_RANK, TirizenConfig
from ..parts.spec import ModelSpec, ScheduleEntry


def layer_choice(cfg: TirizenConfig, i: int) -> tuple[str, dict]:
    layer = cfg.layers[i]
    p, m = f"l{i}.", layer.mixer
    mix = p + "mix."
    norm = lambda n: ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=p + n))  # noqa: E731
    if layer.type == "gla":
        mixer = ("gated_linear_attention", dict(
            hidden_size=cfg.width, n_heads=m["heads"], dim=m["dim"], value_dim=m["vdim"],
            decay_rank=m.get("decay_rank", DEFAULT_DECAY_RANK), tau=float(m["tau"]),
            q_scale=float(m["dim"]) ** -0.5,            # the design scales queries by dim^(-1/2)
            norm_eps=cfg.norm_eps,
            names={"q": mix + "q", "k": mix + "k", "v": mix + "v", "g": mix + "g", "a1": mix + "a1", "a2": mix + "a2",
                   "a2_bias": mix + "a2.b", "gain": mix + "norm", "o": mix + "o"}))
    else:
        own_kv = m.get("kv_from") is None
        names = {"q": mix + "q", "q_norm": mix + "q.norm", "g": mix + "g", "o": mix + "o"}
        if own_kv:
            names.update({"k": mix + "k", "v": mix + "v", "k_norm": mix + "k.norm"})
        temp = m.get("q_temp")
        mixer = ("gqa_attention", dict(
            hidden_size=cfg.width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
            value_dim=m["vdim"], scale=float(m["scale"]), position=("none", {}), qk_norm="per_layer",
            qk_norm_eps=cfg.norm_eps, names=names, own_kv=own_kv, float32_output=True,
            q_temperature=None if temp is None else (float(temp["coef"]), int(temp["every"]))))
    params = dict(hidden_size=cfg.width, streams=max(cfg.streams, 1), mixer=mixer, mixer_norm=norm("norm1"),
                  residual_mult=cfg.residual_mult)
    if cfg.streams:
        params["names"] = {f"{k}{q}": f"{p}hc{q}.{k}" for q in ("1", "2") for k in ("in", "mix", "out")}
    if layer.mlp is not None:
        mlp = p + "mlp."
        if layer.mlp["kind"] == "dense":
            ff = ("ungated_dense", dict(hidden_size=cfg.width, inner_size=int(layer.mlp["ff"]),
                                        names={"up": mlp + "up", "down": mlp + "down"}, activation="relu_squared"))
        else:
            ff = ("softmax_topk_experts", dict(
                hidden_size=cfg.width, expert_size=int(layer.mlp["expert"]["ff"]),
                n_experts=int(layer.mlp["router"]["experts"]), top_k=int(layer.mlp["router"]["top"]), use_bias=True,
                names={"gate": mlp + "router", "bias": mlp + "router.b", "up": mlp + "e{e}.up", "down": mlp + "e{e}.down"}))
        params.update(feed_forward=ff, feed_forward_norm=norm("norm2"))
    return ("hyper_connected", params)


def build_spec(cfg: TirizenConfig) -> ModelSpec:
    if cfg.max_positions <= 0:
        raise ValueError("Tirizen: max_positions is unknown (neither config.json nor a checkpoint gave it)")
    schedule = []
    for i, layer in enumerate(cfg.layers):
        src = layer.mixer.get("kv_from") if layer.type == "attention" else None
        # every layer runs once, so a layer's index is also its position in the run order
        schedule.append(ScheduleEntry(i, read_cache_of=None if src is None else int(src)))
    final_norm = ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="final.norm"))
    return ModelSpec(
        name="Tirizen", vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
        layers=[layer_choice(cfg, i) for i in range(len(cfg.layers))],
        final_norm=final_norm, head_name=None, tied_head=True,
        embedding=("token_table", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="embed",
                                       scale=cfg.embedding_scale, positions_name="pos",
                                       max_positions=cfg.max_positions, streams=max(cfg.streams, 1))),
        head=("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, norm=final_norm, weight_name=None,
                             tied_to="embed", logit_scale=cfg.logit_scale)),
        schedule=schedule,
    )


ARCHITECTURE = register_architecture(["Tirizen", "tirizen"], TirizenConfig, build_spec)
