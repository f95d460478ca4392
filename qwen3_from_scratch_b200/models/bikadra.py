"""Bikadra as a model specification: pre-norm blocks over several residual streams (hyper-connections), each with
the mixer its entry of ``layers`` names (attention through a latent with a rotated key part shared by the heads, or
a state-space mixer with one decay per head) and a dense feed-forward with the tanh form of GELU, or none.  The
embedding is scaled and tied to the head, whose logits are capped by a tanh.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.{in,out,mix}``, ``l<i>.hc2.{in,out,mix}``,
``l<i>.mix.*``, ``l<i>.mlp.{up,down}``, ``final.norm``.  A looped span of layers becomes further entries of the run
order on the same layers, each with a cache id (pages, state slots) of its own.
"""

from __future__ import annotations

from ..config.bikadra_config import ARCHITECTURE, BikadraConfig, BikadraLayer
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..registry import register_architecture

# constants of the design (what config.json cannot change)
YARN_MAGNITUDE = (0.1, 1.0)  # sines and cosines are multiplied by 0.1 * ln(factor) + 1
_BLOCK_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp", "hc1": "hc1", "hc2": "hc2"}


def _mixer(layer: BikadraLayer, cfg: BikadraConfig) -> PartSpec:
    m = layer.sizes()
    if layer.type == "latent_attention":
        scaling = None
        if layer.rot_scaling is not None:
            s = layer.rot_scaling
            scaling = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow,
                       "magnitude": YARN_MAGNITUDE}
        position = PartSpec("rotary_stretched", {"dims": layer.rot_dims, "base": layer.rot_base, "scaling": scaling})
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
            "vdim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
            "norm_eps": cfg.norm_eps, "position": position})
    if layer.type == "mamba2":
        return PartSpec("ssd", {"hidden_size": cfg.width, "num_heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                                "groups": m["groups"], "norm_groups": m["norm_groups"], "conv": m["conv"],
                                "norm_eps": cfg.norm_eps})
    raise ValueError(f"mixer type '{layer.type}' is not built")


@register_architecture(ARCHITECTURE, BikadraConfig)
def bikadra_spec(cfg: BikadraConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "suffix": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ff = None if layer.ff is None else PartSpec("dense_mlp", {
            "hidden_size": cfg.width, "intermediate_size": layer.ff, "activation": "gelu_tanh",
            "names": {"up": "up", "down": "down"}})
        layers.append((f"l{i}", PartSpec("hyper_pre_norm", {
            "norm1": norm, "mixer": _mixer(layer, cfg), "norm2": norm if ff else None, "feed_forward": ff,
            "streams": cfg.streams, "width": cfg.width, "names": _BLOCK_NAMES})))
    order = [LayerCall(layer=i, cache=run) for run, i in enumerate(cfg.run_order())]
    return ModelSpec(
        embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "suffix": "",
                                                         "scale": cfg.embedding_scale, "copies": cfg.streams})),
        layers=layers, order=order,
        final_norm=("final.norm", PartSpec("stream_sum_rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "suffix": "",
                                                                   "streams": cfg.streams})),
        head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed",
                                           "softcap": cfg.logit_softcap})),
        vocab_size=cfg.vocab,
        max_positions=1 << 30,  # nothing in the design depends on a longest position
        eos_token_id=cfg.eos_token_id,
    )
