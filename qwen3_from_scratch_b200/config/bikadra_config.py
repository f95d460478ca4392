"""Configuration of the Bikadra architecture: a pre-norm decoder over several residual streams whose layers choose
between attention through a latent and a state-space mixer, with a span of layers that may run several times.

config.json names the model with ``"architecture": "Bikadra"`` and carries::

    vocab, width                 sizes of the embedding and of a residual stream
    embedding: {scale}           what the looked-up rows are multiplied by
    streams                      how many residual streams a token has
    norm: {eps}                  epsilon of every RMS norm
    logit_softcap                logits <- cap * tanh(logits / cap)
    loop: {start, stop, times}   layers start .. stop - 1 run ``times`` times in a row on the same tensors, each pass
                                 with a cache or state of its own (optional: without it every layer runs once)
    layers: [ {type, mixer: {...}, mlp: {kind: "dense", ff} | null} ]

``type`` is ``latent_attention`` (mixer: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims,
scaling: {factor, original, fast, slow} | absent}) or ``mamba2`` (heads, vdim, state, groups, norm_groups, conv).
Every number comes from the file; nothing is assumed about the order or the count of the layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .binupel_config import _int, _number
from .model_config import ConfigError, ModelConfig

ARCHITECTURE = "Bikadra"
MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"),
    "mamba2": ("heads", "vdim", "state", "groups", "norm_groups", "conv"),
}


@dataclass(frozen=True)
class RotaryScaling:
    """Frequencies stretched by ``factor`` where a pair turns fewer than ``slow`` times in ``original`` positions,
    kept where it turns more than ``fast`` times, a linear ramp between."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class BikadraLayer:
    """One entry of ``layers``: ``mixer`` holds the sizes and constants as read (pairs, so that the configuration
    stays hashable), ``rot`` the rotation of an attention layer, ``ff`` the feed-forward's inner width or None."""

    type: str
    mixer: Tuple[Tuple[str, Any], ...]
    ff: Optional[int]
    rot_base: float = 0.0
    rot_dims: int = 0
    rot_scaling: Optional[RotaryScaling] = None

    def sizes(self) -> dict:
        return dict(self.mixer)


@dataclass(frozen=True)
class BikadraConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    streams: int = 1
    norm_eps: float = 0.0
    logit_softcap: Optional[float] = None
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    layers: Tuple[BikadraLayer, ...] = field(default_factory=tuple)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BikadraConfig":
        vocab, width = _int("model", data, "vocab"), _int("model", data, "width")
        norm = data.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _number("norm", norm, "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        emb = data.get("embedding")
        if not isinstance(emb, Mapping):
            raise ConfigError("config.json: 'embedding' must be an object with 'scale'")
        scale = _number("embedding", emb, "scale")
        streams = _int("model", data, "streams")
        cap = data.get("logit_softcap")
        if cap is not None:
            cap = _number("model", data, "logit_softcap")
            if cap <= 0:
                raise ConfigError(f"config.json: logit_softcap must be positive, got {cap!r}")
        entries = data.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind, m = entry.get("type"), entry["mixer"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not built (built: {', '.join(MIXER_KEYS)})")
            sizes = {key: _int(where, m, key) for key in MIXER_KEYS[kind]}
            rot_base, rot_dims, rot_scaling = 0.0, 0, None
            if kind == "latent_attention":
                sizes["scale"] = _number(where, m, "scale")
                rot = m.get("rot")
                if not isinstance(rot, Mapping):
                    raise ConfigError(f"config.json: {where}: 'rot' must be an object with 'base' and 'dims'")
                rot_base, rot_dims = _number(f"{where}.rot", rot, "base"), _int(f"{where}.rot", rot, "dims")
                if rot_base <= 1 or rot_dims % 2 or rot_dims > sizes["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.rot: base {rot_base!r} must exceed 1 and dims {rot_dims} be "
                                      f"even and at most rot_dim {sizes['rot_dim']}")
                sc = rot.get("scaling")
                if sc is not None:
                    if not isinstance(sc, Mapping):
                        raise ConfigError(f"config.json: {where}.rot.scaling must be an object")
                    rot_scaling = RotaryScaling(*(_number(f"{where}.rot.scaling", sc, k)
                                                  for k in ("factor", "original", "fast", "slow")))
                    if min(rot_scaling.factor, rot_scaling.original, rot_scaling.fast, rot_scaling.slow) <= 0:
                        raise ConfigError(f"config.json: {where}.rot.scaling: every value must be positive")
            else:
                if sizes["heads"] % sizes["groups"]:
                    raise ConfigError(f"config.json: {where}: {sizes['heads']} heads are not a multiple of "
                                      f"{sizes['groups']} groups")
                if (sizes["heads"] * sizes["vdim"]) % sizes["norm_groups"]:
                    raise ConfigError(f"config.json: {where}: {sizes['heads'] * sizes['vdim']} channels are not a multiple "
                                      f"of {sizes['norm_groups']} norm_groups")
            mlp, ff = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}: mlp must be null or of kind 'dense', got {mlp!r}")
                ff = _int(f"{where}.mlp", mlp, "ff")
            layers.append(BikadraLayer(kind, tuple(sorted(sizes.items())), ff, rot_base, rot_dims, rot_scaling))
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            for key in ("start", "stop", "times"):
                v = loop.get(key)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"config.json: loop.{key} must be a non-negative integer, got {v!r}")
            loop = (loop["start"], loop["stop"], loop["times"])
            if not 0 <= loop[0] <= loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(layers)} layers")
        eos = data.get("eos_token_id")
        return cls(architecture=ARCHITECTURE, vocab=vocab, width=width, embedding_scale=scale, streams=streams,
                   norm_eps=eps, logit_softcap=cap, loop=loop, layers=tuple(layers),
                   eos_token_id=eos if isinstance(eos, int) else None)

    def run_order(self):
        """The layer index of every layer run: the looped span as often as it says, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        entries = []
        for layer in self.layers:
            m = layer.sizes()
            if layer.type == "latent_attention":
                rot = {"base": layer.rot_base, "dims": layer.rot_dims}
                if layer.rot_scaling is not None:
                    s = layer.rot_scaling
                    rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                m["rot"] = rot
            entries.append({"type": layer.type, "mixer": m,
                            "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "streams": self.streams, "norm": {"eps": self.norm_eps},
             "layers": entries}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
