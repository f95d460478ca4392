"""Binupel as a model specification: post-norm blocks with a token shift, each with the mixer its entry of
``layers`` names (sigmoid attention whose values are its keys, the RG-LRU recurrent block, or a selective
scan) and a gated feed-forward with a ReLU gate, or none.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``,
``final.norm``, ``head``.  An entry with ``weights_of: j`` runs layer j's parts on a cache and state of its own:
it becomes one more entry of the run order, not one more layer.
"""

from __future__ import annotations

from ..config.binupel_config import ARCHITECTURE, BinupelConfig
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..registry import register_architecture

RGLRU_DECAY = 8.0  # log a = -8 * r * softplus(lam): a constant of the design
_BLOCK_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp", "shift": "shift"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _mixer(kind: str, m: dict, cfg: BinupelConfig) -> PartSpec:
    if kind == "attention":
        return PartSpec("sigmoid_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "scale": m["scale"], "qk_norm_eps": cfg.norm_eps, "temp_coef": m.get("q_temp_coef", 0.0),
            "temp_every": m.get("q_temp_every", 0)})
    if kind == "rglru":
        return PartSpec("rglru", {"hidden_size": cfg.width, "width": m["width"], "blocks": m["blocks"],
                                  "conv": m["conv"], "decay": RGLRU_DECAY})
    if kind == "mamba1":
        return PartSpec("selective_scan", {"hidden_size": cfg.width, "inner": m["inner"], "state": m["state"],
                                           "dt_rank": m["dt_rank"], "conv": m["conv"]})
    raise ValueError(f"mixer type '{kind}' is not built")


@register_architecture(ARCHITECTURE, BinupelConfig)
def binupel_spec(cfg: BinupelConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "suffix": ""})
    layers, order, index_of = [], [], {}
    for i, layer in enumerate(cfg.layers):  # first the layers with tensors of their own, whichever entries run them
        if layer.weights_of is None:
            ff = None if layer.ff is None else PartSpec("gated_mlp", {
                "hidden_size": cfg.width, "intermediate_size": layer.ff, "activation": "relu", "names": _MLP_NAMES})
            block = PartSpec("post_norm", {
                "norm1": norm, "mixer": _mixer(layer.type, layer.sizes(), cfg), "norm2": norm if ff else None,
                "feed_forward": ff, "alpha": cfg.postln_alpha, "token_shift": True, "width": cfg.width,
                "names": _BLOCK_NAMES})
            index_of[i] = len(layers)
            layers.append((f"l{i}", block))
    for i, layer in enumerate(cfg.layers):
        order.append(LayerCall(layer=index_of[i if layer.weights_of is None else layer.weights_of], cache=i))
    return ModelSpec(
        embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                                         "suffix": ""})),
        layers=layers, order=order,
        final_norm=("final.norm", norm),
        head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "suffix": ""})),
        vocab_size=cfg.vocab,
        max_positions=1 << 30,  # nothing in the design depends on a longest position
        eos_token_id=cfg.eos_token_id,
    )
