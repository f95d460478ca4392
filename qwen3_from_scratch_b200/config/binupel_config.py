"""Configuration of the Binupel architecture: a decoder whose layers choose their mixer one by one.

config.json names the model with ``"architecture": "Binupel"`` and carries::

    vocab, width                 sizes of the embedding and of the residual stream
    norm: {eps}                  epsilon of every RMSNorm (the layers', the heads', the last one)
    postln_alpha                 x <- norm(alpha * x + sublayer(x))
    layers: [ {type, mixer: {...}, mlp: {kind, ff} | null, weights_of: j (optional)} ]

``type`` is ``attention`` (mixer: heads, kv_heads, dim, vdim, scale, q_temp: {coef, every}), ``rglru`` (width,
blocks, conv) or ``mamba1`` (inner, state, dt_rank, conv).  A layer with ``weights_of: j`` runs layer j's
tensors on a cache and state of its own; its sizes are read from layer j's entry (from the entry that j's own
``weights_of`` leads to, if j has one).  Every number comes from the file; nothing is assumed about the
order or the count of the layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, ModelConfig

ARCHITECTURE = "Binupel"
MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim"),
    "rglru": ("width", "blocks", "conv"),
    "mamba1": ("inner", "state", "dt_rank", "conv"),
}


def _int(where: str, data: Mapping[str, Any], key: str) -> int:
    if key not in data:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {where}: '{key}' must be a positive integer, got {value!r}")
    return value


def _number(where: str, data: Mapping[str, Any], key: str) -> float:
    if key not in data:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}: '{key}' must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class BinupelLayer:
    """One entry of ``layers``.  ``mixer`` holds the mixer's sizes and constants as read (a tuple of pairs, so
    that the configuration stays hashable); ``ff`` is the feed-forward's inner width or None for no
    feed-forward; ``weights_of`` the layer whose tensors this one runs, or None for its own."""

    type: str
    mixer: Tuple[Tuple[str, Any], ...]
    ff: Optional[int]
    weights_of: Optional[int] = None

    def sizes(self) -> dict:
        return dict(self.mixer)


@dataclass(frozen=True)
class BinupelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    postln_alpha: float = 1.0
    layers: Tuple[BinupelLayer, ...] = field(default_factory=tuple)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BinupelConfig":
        vocab, width = _int("model", data, "vocab"), _int("model", data, "width")
        norm = data.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _number("norm", norm, "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        alpha = _number("model", data, "postln_alpha")
        entries = data.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, entry in enumerate(entries):
            if not isinstance(entry, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
        # whose tensors each entry runs: its own, or those of the entry that `weights_of` leads to
        owner_of = []
        for i, entry in enumerate(entries):
            j, seen = i, set()
            while entries[j].get("weights_of") is not None:
                nxt = entries[j]["weights_of"]
                if isinstance(nxt, bool) or not isinstance(nxt, int) or not 0 <= nxt < len(entries) or nxt == j or j in seen:
                    raise ConfigError(f"config.json: layers[{i}]: weights_of must lead to a layer with tensors of its own, "
                                      f"got {entries[i]['weights_of']!r}")
                seen.add(j)
                j = nxt
            owner_of.append(j)
        layers = []
        for i, shown in enumerate(entries):
            where = f"layers[{i}]"
            entry = entries[owner_of[i]]  # a sharing entry equals its owner's in everything but `weights_of`
            if shown.get("type", entry.get("type")) != entry.get("type"):
                raise ConfigError(f"config.json: {where}: a layer that runs layer {owner_of[i]}'s weights must be of its type")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind = entry.get("type")
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not built (built: {', '.join(MIXER_KEYS)})")
            m = entry["mixer"]
            if kind == "attention" and "vdim" not in m:
                m = dict(m, vdim=m.get("dim"))  # the values are the keys
            sizes = {key: _int(where, m, key) for key in MIXER_KEYS[kind]}
            if kind == "attention":
                if sizes["heads"] % sizes["kv_heads"]:
                    raise ConfigError(f"config.json: {where}: {sizes['heads']} heads are not a multiple of "
                                      f"{sizes['kv_heads']} kv_heads")
                if sizes["vdim"] != sizes["dim"]:
                    raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {sizes['vdim']} must "
                                      f"equal dim {sizes['dim']}")
                sizes["scale"] = _number(where, m, "scale")
                temp = m.get("q_temp")
                if temp is not None:
                    if not isinstance(temp, Mapping):
                        raise ConfigError(f"config.json: {where}: 'q_temp' must be an object with 'coef' and 'every'")
                    sizes["q_temp_coef"] = _number(f"{where}.q_temp", temp, "coef")
                    sizes["q_temp_every"] = _int(f"{where}.q_temp", temp, "every")
            elif kind == "rglru":
                if sizes["width"] % sizes["blocks"]:
                    raise ConfigError(f"config.json: {where}: width {sizes['width']} is not a multiple of "
                                      f"{sizes['blocks']} blocks")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}: mlp must be null or of kind 'dense', got {mlp!r}")
                ff = _int(f"{where}.mlp", mlp, "ff")
            layers.append(BinupelLayer(kind, tuple(sorted(sizes.items())), ff, None if owner_of[i] == i else owner_of[i]))
        eos = data.get("eos_token_id")
        return cls(architecture=ARCHITECTURE, vocab=vocab, width=width, norm_eps=eps, postln_alpha=alpha,
                   layers=tuple(layers), eos_token_id=eos if isinstance(eos, int) else None)

    def to_dict(self) -> dict:
        entries = []
        for layer in self.layers:
            m = layer.sizes()
            if layer.type == "attention" and "q_temp_coef" in m:
                m["q_temp"] = {"coef": m.pop("q_temp_coef"), "every": m.pop("q_temp_every")}
            entry = {"type": layer.type, "mixer": m, "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            entries.append(entry)
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "postln_alpha": self.postln_alpha, "layers": entries}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
