"""Typed configuration of the Guravik decoder, from config.json.

The file is nested: ``layers`` lists the layers in order, each with its ``type`` (which mixer), the
mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for a layer with a mixer only);
``loop`` names a range of layers that runs several times in a row; ``canon.taps`` is the length of the
short convolution in front of every mixer; ``embedding.scale`` multiplies the embedded tokens;
``norm.eps`` is the epsilon of every RMS norm.  Sizes that the file does not carry (the inner rank of
the delta-rule decay) come from the checkpoint's tensor shapes and are filled in by
``with_tensor_shapes`` when a model folder is opened.

Every size and constant the layers use is read here; what the layers cannot run is refused.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .minimax_m3 import ConfigError

MIXER_TYPES = ("general_delta", "latent_attention")
_MIXER_KEYS = {
    "general_delta": ("dim", "heads"),
    "latent_attention": ("dim", "heads", "kv_rank", "q_rank", "rot_dim", "scale", "vdim", "rot"),
}


@dataclass(frozen=True)
class GuravikLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class GuravikConfig:
    vocab: int
    width: int
    layers: tuple[GuravikLayer, ...]
    norm_eps: float
    embedding_scale: float = 1.0
    canon_taps: int = 1
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: tuple = ()
    architecture: str = "Guravik"
    extra: dict = field(default_factory=dict, compare=False)

    # ---- reading ---------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict, generation: dict | None = None) -> "GuravikConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"config.json lacks {key!r}")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            if "type" not in entry or "mixer" not in entry:
                raise ConfigError(f"layers[{i}] needs 'type' and 'mixer'")
            mlp = entry.get("mlp")
            layers.append(GuravikLayer(str(entry["type"]), copy.deepcopy(dict(entry["mixer"])),
                                       None if mlp is None else copy.deepcopy(dict(mlp))))
        loop = raw.get("loop") or {}
        eos = (generation or {}).get("eos_token_id", raw.get("eos_token_id"))
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        known = {"architecture", "architectures", "model_type", "vocab", "width", "layers", "norm", "embedding", "canon",
                 "loop", "eos_token_id"}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                  norm_eps=float(raw["norm"]["eps"]),
                  embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                  canon_taps=int((raw.get("canon") or {}).get("taps", 1)),
                  loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                  loop_times=int(loop.get("times", 1)), eos_token_ids=eos,
                  architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Guravik"])[0]),
                  extra={k: v for k, v in raw.items() if k not in known})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if self.canon_taps < 1:
            raise ConfigError(f"canon.taps {self.canon_taps}: a convolution has at least one tap")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError(f"loop {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit {n} layers")
        for i, layer in enumerate(self.layers):
            if layer.type not in MIXER_TYPES:
                raise ConfigError(f"layers[{i}].type {layer.type!r} is not one of {MIXER_TYPES}")
            missing = [k for k in _MIXER_KEYS[layer.type] if k not in layer.mixer]
            if missing:
                raise ConfigError(f"layers[{i}].mixer lacks {missing}")
            m = layer.mixer
            if m["heads"] <= 0 or m["dim"] <= 0:
                raise ConfigError(f"layers[{i}]: heads and dim must be positive")
            if layer.type == "latent_attention":
                rot = m["rot"]
                if "base" not in rot or "dims" not in rot:
                    raise ConfigError(f"layers[{i}].mixer.rot needs 'base' and 'dims'")
                if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["rot_dim"]:
                    raise ConfigError(f"layers[{i}]: rot.dims {rot['dims']} must be even and at most rot_dim {m['rot_dim']}")
                if m["kv_rank"] > 512:
                    raise ConfigError(f"layers[{i}]: kv_rank {m['kv_rank']} above 512, the attention kernel's limit")
            if layer.type == "general_delta" and m["dim"] > 256:
                raise ConfigError(f"layers[{i}]: dim {m['dim']} above 256, the recurrence kernel's limit")
            if layer.mlp is not None:
                if layer.mlp.get("kind") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind {layer.mlp.get('kind')!r}: only 'dense' is built")
                if int(layer.mlp.get("ff", 0)) <= 0:
                    raise ConfigError(f"layers[{i}].mlp.ff must be positive")

    # ---- sizes that only the checkpoint knows --------------------------------------------------------
    def with_tensor_shapes(self, shape_of) -> "GuravikConfig":
        """``shape_of(name) -> shape or None``: fill in sizes that are no keys of the file (the inner rank of
        the delta-rule decay, ``mixer.decay_rank``, is the row count of ``l<i>.mix.w1``)."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = dict(layer.mixer)
            if layer.type == "general_delta" and "decay_rank" not in m:
                shape = shape_of(f"l{i}.mix.w1")
                if shape is None:
                    raise ConfigError(f"layers[{i}]: the checkpoint has no l{i}.mix.w1 to take the decay's inner rank from")
                m["decay_rank"] = int(shape[0])
            layers.append(GuravikLayer(layer.type, m, layer.mlp))
        return GuravikConfig(**{**self.__dict__, "layers": tuple(layers)})

    # ---- the run order ------------------------------------------------------------------------------
    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding output is added first) in the order the layers run: the layers
        before the loop, the looped range ``times`` times (each pass but the first starts with the
        embedding output added), the rest."""
        order = [(i, False) for i in range(self.loop_start)]
        if self.loop_stop > self.loop_start:
            for rep in range(self.loop_times):
                order += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        order += [(i, False) for i in range(self.loop_stop, len(self.layers))]
        return order

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update({
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "canon": {"taps": self.canon_taps},
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
        })
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
