"""Small Bikadra configurations and model folders for the tests: the configuration dicts, the tensors the design
names for them (names and shapes restated here from the design, not asked of the engine) and random weights strong
enough that every mechanism moves the logits."""

from __future__ import annotations

import json
import os
from typing import Dict

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims=None, scaling=None, ff=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale, "rot": rot}
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mamba2(heads, vdim, state, groups, norm_groups, conv, ff=None):
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}
    return {"type": "mamba2", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# X: three streams; a loop of three passes that starts after the first layer; every head size different from the
# others, a latent that is no multiple of 32, stretched frequencies whose ramp lies inside the pairs, layers
# without feed-forward, states of 24 and 40 (no multiples of the lanes' 16), one and three groups, norm parts
# that differ from the groups, two and four taps.
BIKADRA_X = {
    "architecture": "Bikadra", "vocab": 211, "width": 64, "embedding": {"scale": 4.0}, "streams": 3,
    "norm": {"eps": 1e-5}, "logit_softcap": 20.0, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [latent(4, 24, 16, 40, 40, 24, 0.2, 10000.0, scaling=(4.0, 64, 8.0, 1.0), ff=72),
               mamba2(6, 16, 24, 3, 2, 4, ff=80),
               latent(3, 16, 8, 8, 48, 56, 0.3, 500.0, ff=None),
               mamba2(4, 8, 40, 1, 4, 2, ff=None)]}
# Y: a single stream (the coefficients still apply), no loop, no cap on the logits, a state-space layer first, a
# single tap (no tail to keep), one norm part, a rotation over fewer dimensions than the rotated part has, one head.
BIKADRA_Y = {
    "architecture": "Bikadra", "vocab": 173, "width": 48, "embedding": {"scale": 1.0}, "streams": 1,
    "norm": {"eps": 1e-6},
    "layers": [mamba2(3, 16, 16, 3, 1, 1, ff=88),
               latent(1, 32, 16, 24, 64, 32, 0.18, 10000.0, dims=8, scaling=(16.0, 32, 4.0, 0.5), ff=40),
               latent(5, 8, 24, 16, 24, 40, 0.25, 200000.0, ff=56)]}
# Z: sizes in the manner of the serving kernels, small: sixteen heads over a latent of 128 with a rotated part
# of 64, a state of 64 with heads of 64 channels, widths in multiples of 128; four streams; the loop is the whole
# model.
BIKADRA_Z = {
    "architecture": "Bikadra", "vocab": 300, "width": 128, "embedding": {"scale": 8.0}, "streams": 4,
    "norm": {"eps": 1e-6}, "logit_softcap": 50.0, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [latent(16, 32, 64, 32, 128, 96, 0.1, 1000000.0, scaling=(8.0, 256, 16.0, 2.0), ff=256),
               mamba2(4, 64, 64, 2, 4, 4, ff=256)]}
CONFIGS = {"x": (BIKADRA_X, 3), "y": (BIKADRA_Y, 4), "z": (BIKADRA_Z, 5)}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V, S = config["width"], config["vocab"], config["streams"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    for i, entry in enumerate(config["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        shapes.update({p + "norm1": (W,), p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        if entry["type"] == "latent_attention":
            H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({p + "mix.dq": (rq, W), p + "mix.dq.norm": (rq,), p + "mix.uq": (H * (dn + dr), rq),
                           p + "mix.dkv": (rk + dr, W), p + "mix.dkv.norm": (rk,), p + "mix.uk": (H * dn, rk),
                           p + "mix.uv": (H * dv, rk), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        else:
            H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * P, H * P + 2 * G * N
            shapes.update({p + "mix.in": (inner + C + H, W), p + "mix.conv": (C, K), p + "mix.conv.b": (C,),
                           p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,),
                           p + "mix.o": (W, inner)})
        if entry["mlp"] is not None:
            F = entry["mlp"]["ff"]
            shapes.update({p + "norm2": (W,), p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S),
                           p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return shapes


def random_tensor(name: str, shape: tuple, g: torch.Generator) -> torch.Tensor:
    leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
    r = lambda: torch.randn(shape, generator=g)  # noqa: E731
    if leaf in ("norm1", "norm2") or name == "final.norm" or leaf.endswith("norm"):
        t = 1.0 + 0.2 * r()
    elif leaf.endswith(".in"):  # how a sub-layer reads the streams
        t = 0.7 + 0.3 * r() if leaf.startswith("hc") else r() * (1.3 / shape[-1] ** 0.5)
    elif leaf.startswith("hc") and leaf.endswith(".out"):
        t = 0.8 + 0.3 * r()
    elif leaf.startswith("hc") and leaf.endswith(".mix"):  # near the identity, every stream leaking into the others
        t = 0.8 * torch.eye(shape[0]) + 0.15 * r()
    elif leaf.endswith("A_log"):
        t = torch.log(0.2 + 2.0 * torch.rand(shape, generator=g))
    elif leaf.endswith(".D"):
        t = 1.0 + 0.3 * r()
    elif leaf.endswith("dt_bias"):
        t = -1.0 + 0.7 * r()
    elif leaf.endswith(".b"):
        t = 0.4 * r()
    elif leaf.endswith("conv"):
        t = 0.6 * r()
    elif name == "embed":
        t = 0.5 * r()
    else:  # a matrix [out, in]: outputs of order one for inputs of order one
        t = r() * (1.3 / shape[-1] ** 0.5)
    return t.to(torch.bfloat16)


def make_folder(folder: str, config: dict, seed: int, tweak=None) -> str:
    """config.json and model.safetensors (bfloat16) in ``folder``.  ``tweak(tensors)`` may change them first."""
    os.makedirs(folder, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    tensors = {name: random_tensor(name, shape, g) for name, shape in sorted(tensor_shapes(config).items())}
    if tweak is not None:
        tweak(tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
