"""Typed configuration of the Tirizen decoder, from config.json.

The file is nested: ``layers`` lists the layers in order, each with its ``type`` (which mixer: ``attention`` or
``gla``), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense`` with ``ff``, or ``moe``
with ``expert.ff`` and ``router.experts`` / ``router.top``; null for a layer with a mixer only).  ``streams`` is
the number of residual streams the layers are connected to (absent: one stream and the plain pre-norm residual,
without connection weights); ``residual_mult`` multiplies every sublayer's output; ``embedding.scale`` multiplies
the embedded tokens; ``max_positions`` is the length of the table of learned positions; ``logit_scale``
multiplies the logits; ``norm.eps`` is the epsilon of every RMS norm.  Sizes that the file does not carry (the
inner rank of the recurrence's decay) come from the checkpoint's tensor shapes and are filled in by
``with_tensor_shapes`` when a model folder is opened.

Every size and constant the layers use is read here; what the layers cannot run is refused.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .minimax_m3 import ConfigError

MIXER_TYPES = ("attention", "gla")
_MIXER_KEYS = {
    "attention": ("dim", "heads", "kv_heads", "vdim", "scale"),
    "gla": ("dim", "heads", "vdim", "tau"),
}
MAX_STREAMS = 16
MAX_HEAD_SIZE = 256
DEFAULT_DECAY_RANK = 16           # inner rank of the decay when no checkpoint says otherwise (random models)


@dataclass(frozen=True)
class TirizenLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class TirizenConfig:
    vocab: int
    width: int
    layers: tuple[TirizenLayer, ...]
    norm_eps: float
    max_positions: int
    streams: int = 0                  # 0: one stream, plain residual (no connection tensors)
    residual_mult: float = 1.0
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    eos_token_ids: tuple = ()
    architecture: str = "Tirizen"
    extra: dict = field(default_factory=dict, compare=False)

    # ---- reading ---------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, generation: dict | None = None) -> "TirizenConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            if "type" not in entry or "mixer" not in entry:
                raise ConfigError(f"layers[{i}] needs 'type' and 'mixer'")
            mlp = entry.get("mlp")
            layers.append(TirizenLayer(str(entry["type"]), copy.deepcopy(dict(entry["mixer"])),
                                       None if mlp is None else copy.deepcopy(dict(mlp))))
        eos = (generation or {}).get("eos_token_id", raw.get("eos_token_id"))
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        known = {"architecture", "architectures", "model_type", "vocab", "width", "layers", "norm", "embedding",
                 "streams", "residual_mult", "logit_scale", "max_positions", "eos_token_id"}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                  norm_eps=float(raw["norm"]["eps"]), max_positions=int(raw.get("max_positions") or 0),
                  streams=int(raw.get("streams") or 0), residual_mult=float(raw.get("residual_mult", 1.0)),
                  embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                  logit_scale=float(raw.get("logit_scale", 1.0)), eos_token_ids=eos,
                  architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Tirizen"])[0]),
                  extra={k: v for k, v in raw.items() if k not in known})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not 0 <= self.streams <= MAX_STREAMS:
            raise ConfigError(f"streams {self.streams}: the connection kernel takes at most {MAX_STREAMS}")
        if self.max_positions < 0:
            raise ConfigError(f"max_positions {self.max_positions} must be positive")
        for i, layer in enumerate(self.layers):
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"layers[{i}].type {layer.type!r} is not one of {MIXER_TYPES}")
            m = layer.mixer
            missing = [k for k in _MIXER_KEYS[layer.type] if k not in m]
            if missing:
                raise ConfigError(f"layers[{i}].mixer lacks {missing}")
            if m["heads"] <= 0 or not 0 < m["dim"] <= MAX_HEAD_SIZE or not 0 < m["vdim"] <= MAX_HEAD_SIZE:
                raise ConfigError(f"layers[{i}]: heads must be positive and dim, vdim between 1 and {MAX_HEAD_SIZE}")
            if layer.type == "gla":
                if float(m["tau"]) <= 0:
                    raise ConfigError(f"layers[{i}].mixer.tau must be positive")
            else:
                if m["kv_heads"] <= 0 or m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"layers[{i}]: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                temp = m.get("q_temp")
                if temp is not None and ("coef" not in temp or int(temp.get("every", 0)) <= 0):
                    raise ConfigError(f"layers[{i}].mixer.q_temp needs 'coef' and a positive 'every'")
                src = m.get("kv_from")
                if src is not None:
                    if not 0 <= int(src) < i or self.layers[int(src)].type != "attention" \
                            or self.layers[int(src)].mixer.get("kv_from") is not None:
                        raise ConfigError(f"layers[{i}].mixer.kv_from {src}: not an earlier attention layer with keys "
                                          f"and values of its own")
                    other = self.layers[int(src)].mixer
                    if any(other[k] != m[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"layers[{i}] reads the keys and values of layer {src}, whose kv_heads, dim "
                                          f"or vdim differ")
            mlp = layer.mlp
            if mlp is not None:
                kind = mlp.get("kind")
                if kind == "dense":
                    if int(mlp.get("ff", 0)) <= 0:
                        raise ConfigError(f"layers[{i}].mlp.ff must be positive")
                elif kind == "moe":
                    router, expert = mlp.get("router") or {}, mlp.get("expert") or {}
                    E, top = int(router.get("experts", 0)), int(router.get("top", 0))
                    if not 0 < top <= E or E > 1024 or int(expert.get("ff", 0)) <= 0:
                        raise ConfigError(f"layers[{i}].mlp: needs expert.ff > 0 and 0 < router.top <= router.experts "
                                          f"<= 1024")
                else:
                    raise ConfigError(f"layers[{i}].mlp.kind {kind!r} is not 'dense' or 'moe'")

    # ---- sizes that only the checkpoint knows --------------------------------------------------------
    def with_tensor_shapes(self, shape_of) -> "TirizenConfig":
        """``shape_of(name) -> shape or None``: fill in sizes that are no keys of the file: the inner rank of a
        recurrence's decay (``mixer.decay_rank``, the row count of ``l<i>.mix.a1``) and, if the file does not say,
        the number of learned positions (the row count of ``pos``)."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = dict(layer.mixer)
            if layer.type == "gla" and "decay_rank" not in m:
                shape = shape_of(f"l{i}.mix.a1")
                if shape is None:
                    raise ConfigError(f"layers[{i}]: the checkpoint has no l{i}.mix.a1 to take the decay's inner rank from")
                m["decay_rank"] = int(shape[0])
            layers.append(TirizenLayer(layer.type, m, layer.mlp))
        max_positions = self.max_positions
        if max_positions <= 0:
            shape = shape_of("pos")
            if shape is None:
                raise ConfigError("neither max_positions nor a tensor 'pos' says how many positions are learned")
            max_positions = int(shape[0])
        return TirizenConfig(**{**self.__dict__, "layers": tuple(layers), "max_positions": max_positions})

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update({
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "max_positions": self.max_positions, "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
        })
        if self.streams:
            d["streams"] = self.streams
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
