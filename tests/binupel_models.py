"""Small Binupel configurations and model folders for the tests: the configuration dicts, the tensors the
design names for them (names and shapes restated here from the design, not asked of the engine) and random
weights strong enough that every mechanism moves the logits."""

from __future__ import annotations

import json
import os
from typing import Dict

import torch
from safetensors.torch import save_file


def attention(heads, kv_heads, dim, scale, q_temp=None, ff=None, **more):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return dict({"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}, **more)


def rglru(width, blocks, conv, ff=None, **more):
    return dict({"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv},
                 "mlp": None if ff is None else {"kind": "dense", "ff": ff}}, **more)


def mamba1(inner, state, dt_rank, conv, ff=None, **more):
    return dict({"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
                 "mlp": None if ff is None else {"kind": "dense", "ff": ff}}, **more)


def shared(entry, owner):
    return dict(entry, weights_of=owner)


# P: every mixer once and again with shared weights, in another order than "scan, recurrence, attention"; two kv
# heads, a head size that is no power of two, four taps, a layer without feed-forward, a temperature that changes
# every 7 positions.
_P = [attention(4, 2, 48, 0.21, q_temp=(0.4, 7), ff=72), rglru(96, 3, 4, ff=None), mamba1(80, 8, 5, 2, ff=56)]
BINUPEL_P = {"architecture": "Binupel", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
             "layers": _P + [shared(_P[1], 1), shared(_P[0], 0), shared(_P[2], 2)]}
# Q: starts with a scan, one block in the gates, as many kv heads as heads, no temperature, a head size that the
# tensor-core kernels refuse (20), alpha 1, a state size beyond 16.
_Q = [mamba1(96, 20, 8, 4, ff=None), attention(3, 3, 20, 0.3, ff=40), rglru(64, 1, 3, ff=88),
      attention(6, 1, 32, 0.17, q_temp=(1.5, 3), ff=None)]
BINUPEL_Q = {"architecture": "Binupel", "vocab": 173, "width": 48, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
             "layers": _Q + [shared(_Q[0], 0)]}
# R: the serving kernels' sizes in small: heads of 64 and 128, groups of 4 and 8, widths in multiples of 128.
_R = [attention(8, 2, 64, 0.125, q_temp=(0.3, 50), ff=256), mamba1(256, 16, 16, 4, ff=256), rglru(256, 2, 4, ff=256),
      attention(8, 1, 128, 0.09, ff=256)]
BINUPEL_R = {"architecture": "Binupel", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "postln_alpha": 3.0,
             "layers": _R + [shared(_R[0], 0)]}
CONFIGS = {"p": (BINUPEL_P, 3), "q": (BINUPEL_Q, 4), "r": (BINUPEL_R, 5)}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, entry in enumerate(config["layers"]):
        if "weights_of" in entry:
            continue
        p, m = f"l{i}.", entry["mixer"]
        shapes[p + "norm1"] = (W,)
        shapes[p + "shift"] = (W,)
        if entry["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.q.norm": (d,),
                           p + "mix.k.norm": (d,), p + "mix.pb": (H,), p + "mix.g": (H, W), p + "mix.o": (W, H * d)})
        elif entry["type"] == "rglru":
            C, nb, K = m["width"], m["blocks"], m["conv"]
            shapes.update({p + "mix.y": (C, W), p + "mix.y.b": (C,), p + "mix.x": (C, W), p + "mix.x.b": (C,),
                           p + "mix.conv": (C, K), p + "mix.conv.b": (C,), p + "mix.ra": (nb, C // nb, C // nb),
                           p + "mix.ra.b": (nb, C // nb), p + "mix.ri": (nb, C // nb, C // nb),
                           p + "mix.ri.b": (nb, C // nb), p + "mix.lam": (C,), p + "mix.o": (W, C)})
        else:
            I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            shapes.update({p + "mix.in": (2 * I, W), p + "mix.conv": (I, K), p + "mix.conv.b": (I,),
                           p + "mix.x": (R + 2 * N, I), p + "mix.dt": (I, R), p + "mix.dt.b": (I,),
                           p + "mix.A_log": (I, N), p + "mix.D": (I,), p + "mix.o": (W, I)})
        if entry["mlp"] is not None:
            F = entry["mlp"]["ff"]
            shapes.update({p + "norm2": (W,), p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return shapes


def random_tensor(name: str, shape: tuple, g: torch.Generator) -> torch.Tensor:
    leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
    r = lambda: torch.randn(shape, generator=g)  # noqa: E731
    if leaf in ("norm1", "norm2") or name == "final.norm" or leaf.endswith(".norm"):
        t = 1.0 + 0.2 * r()
    elif leaf == "shift":
        t = torch.rand(shape, generator=g)
    elif leaf.endswith("A_log"):
        t = torch.log(0.3 + 3.0 * torch.rand(shape, generator=g))
    elif leaf.endswith(".D"):
        t = 1.0 + 0.3 * r()
    elif leaf.endswith("dt.b"):
        t = -1.0 + 0.7 * r()
    elif leaf.endswith("lam"):
        t = 0.8 * r()
    elif leaf.endswith("pb"):
        t = -0.7 + 0.8 * r()
    elif leaf.endswith(".b"):
        t = 0.4 * r()
    elif leaf.endswith("conv"):
        t = 0.6 * r()
    elif name in ("embed",):
        t = r()
    else:  # a matrix [.., out, in]: outputs of order one for inputs of order one
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
