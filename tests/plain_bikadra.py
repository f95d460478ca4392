"""A plain, slow statement of the Bikadra design in float64 on the CPU: one function per mechanism, written
from the mechanism's equations, sharing no code with the engine.  Whatever is carried from token to token
(the latent cache of an attention layer, the state and the convolution tail of a state-space layer) is taken
and returned explicitly, so that a prompt can run whole, in portions or token by token through the same
functions.

Notation: T tokens, W the stream's width, S the number of residual streams.  ``w`` maps tensor names to
float64 tensors.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

F64 = torch.float64

# What a projection does to its operand and its result: nothing, or (inside ``bfloat16_projections()``) rounding
# both to bfloat16, which is where a bfloat16 run rounds.
_round = [lambda t: t]


class bfloat16_projections:
    def __enter__(self):
        _round.append(lambda t: t.to(torch.bfloat16).to(F64))

    def __exit__(self, *exc):
        _round.pop()


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x W^T for a weight stored [out, in]."""
    r = _round[-1]
    return r(r(x) @ weight.t())


def read_model_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            w[name] = t.to(F64) if t.is_floating_point() else t
    return config, w


# ---------------------------------------------------------------------- small functions
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------------- rotation with stretched frequencies
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair [dims / 2], factor on sines and cosines).  Without ``scaling`` the plain
    frequencies base^(-2i / dims) and 1.  With it, pairs that turn slowly are slowed by ``factor``, pairs
    that turn fast are kept, with a linear ramp between the pair indices at which ``fast`` and ``slow``
    turns fit into ``original`` positions."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(half, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """x [..., T, heads, dims]: dimension i is paired with i + dims / 2."""
    half = freq.numel()
    a = positions.to(F64)[:, None] * freq[None, :]  # [T, half]
    cos, sin = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], dim=-1)


# ---------------------------------------------------------------------- attention through a latent
def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, cache=None):
    """h [T, W] at positions len(cache) ...; ``cache`` = (latents [n, kv_rank], rotated key parts [n, rot_dim])
    of the n tokens before.  Returns (output [T, W], new cache)."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    freq, mag = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    before = 0 if cache is None else cache[0].shape[0]
    pos = torch.arange(before, before + T)

    cq = rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = linear(cq, w[p + "uq"]).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_half(q[..., dn:], pos, freq, mag)

    down = linear(h, w[p + "dkv"])
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_half(down[:, None, rank:], pos, freq, mag)[:, 0]
    if cache is not None:
        c, k_rot = torch.cat([cache[0], c]), torch.cat([cache[1], k_rot])
    n = c.shape[0]
    k_plain = linear(c, w[p + "uk"]).view(n, H, dn)
    v = linear(c, w[p + "uv"]).view(n, H, dv)

    scores = (torch.einsum("thd,nhd->htn", q_plain, k_plain) + torch.einsum("thd,nd->htn", q_rot, k_rot)) * m["scale"]
    visible = torch.arange(n)[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    out = torch.einsum("htn,nhd->thd", torch.softmax(scores, dim=-1), v)
    gate = sigmoid(linear(h, w[p + "g"]))  # [T, H]
    out = (out * gate[:, :, None]).reshape(T, H * dv)
    return linear(out, w[p + "o"]), (c, k_rot)


# ---------------------------------------------------------------------- state-space mixer
def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, tail: Optional[torch.Tensor]):
    """x [T, C]; weight [C, taps], the last column multiplies the current token.  ``tail``: the taps - 1 inputs
    before x (zeros at the start of a sequence).  Returns (output [T, C], new tail)."""
    taps = weight.shape[1]
    if tail is None:
        tail = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype)
    full = torch.cat([tail, x])
    out = torch.zeros_like(x) + bias
    for j in range(taps):
        out = out + full[j:j + x.shape[0]] * weight[:, j]
    return out, full[full.shape[0] - (taps - 1):]


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, state=None):
    """state = (S [heads, N, vdim], convolution tail [taps - 1, channels]) or None at a sequence's start."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = linear(h, w[p + "in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    S, tail = state if state is not None else (torch.zeros(H, N, P, dtype=F64), None)
    conv, tail = causal_conv(xbc, w[p + "conv"], w[p + "conv.b"], tail)
    xbc = _round[-1](silu(conv))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    step = softplus(dt + w[p + "dt_bias"])  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * step)
    per_group = H // G
    y = torch.zeros(T, H, P, dtype=F64)
    S = S.clone()
    group_of = torch.arange(H) // per_group
    for t in range(T):  # all heads at once: S_h = decay_h S_h + step_h B_g(h) x_h^T, y_h = S_h^T C_g(h) + D_h x_h
        Bh, Ch = B[t, group_of], C[t, group_of]  # [H, N]
        S = decay[t, :, None, None] * S + step[t, :, None, None] * Bh[:, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ch) + w[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return linear(y, w[p + "o"]), (S, tail)


# ---------------------------------------------------------------------- feed-forward
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return linear(_round[-1](gelu_tanh(linear(h, w[p + "up"]))), w[p + "down"])


# ---------------------------------------------------------------------- several residual streams
def streams_read(xs: torch.Tensor, read: torch.Tensor) -> torch.Tensor:
    """xs [S, T, W] -> the sub-layer's input sum_s read[s] xs[s]."""
    return torch.einsum("s,stw->tw", read, xs)


def streams_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, write: torch.Tensor) -> torch.Tensor:
    """New stream t = sum_s mix[s, t] xs[s] + write[t] y, all from the old streams."""
    return torch.einsum("st,sxw->txw", mix, xs) + write[:, None, None] * y[None]


# ---------------------------------------------------------------------- the model
def run_mixer(kind: str, h, w, p: str, m: dict, eps: float, state):
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps, state)
    if kind == "mamba2":
        return mamba2(h, w, p, m, eps, state)
    raise ValueError(f"mixer {kind!r}")


def layer(xs: torch.Tensor, w, config: dict, i: int, state):
    """One run of layer i on the streams xs [S, T, W]."""
    entry, eps, p = config["layers"][i], config["norm"]["eps"], f"l{i}."
    u = streams_read(xs, w[p + "hc1.in"])
    y, state = run_mixer(entry["type"], rms_norm(u, w[p + "norm1"], eps), w, p + "mix.", entry["mixer"], eps, state)
    xs = streams_write(xs, y, w[p + "hc1.mix"], w[p + "hc1.out"])
    if entry.get("mlp") is not None:
        u = streams_read(xs, w[p + "hc2.in"])
        y = dense_ff(rms_norm(u, w[p + "norm2"], eps), w, p + "mlp.")
        xs = streams_write(xs, y, w[p + "hc2.mix"], w[p + "hc2.out"])
    return xs, state


def run_order(config: dict) -> List[int]:
    """The layer index of every layer run: the looped span repeated, then the rest."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def forward(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], states: Optional[List] = None,
            per_layer: Optional[list] = None):
    """Logits [T, vocab] of the tokens ``ids`` that follow what ``states`` (one per layer run) has seen.
    ``per_layer``: a list that receives the sum of the streams after every layer run."""
    x = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * config["embedding"]["scale"]
    xs = x[None].repeat(config["streams"], 1, 1)
    order = run_order(config)
    states = [None] * len(order) if states is None else list(states)
    for r, i in enumerate(order):
        xs, states[r] = layer(xs, w, config, i, states[r])
        if per_layer is not None:
            per_layer.append(xs.sum(dim=0))
    x = rms_norm(xs.sum(dim=0), w["final.norm"], config["norm"]["eps"])
    logits = linear(x, w["embed"])
    cap = config.get("logit_softcap")
    return (logits if cap is None else cap * torch.tanh(logits / cap)), states


def forward_logits(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    return forward(config, w, ids)[0]


def rounding_error(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> float:
    """The largest difference that rounding every projection's operand and result to bfloat16 makes to a
    logit of this prompt, relative to the largest logit."""
    exact = forward_logits(config, w, ids)
    with bfloat16_projections():
        rounded = forward_logits(config, w, ids)
    return float((rounded - exact).abs().max()) / float(exact.abs().max())


def greedy(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int):
    """(generated ids, gap between the two largest logits at every step), token by token through the states."""
    logits, states = forward(config, w, prompt)
    out, margins = [], []
    for _ in range(new_tokens):
        top = torch.topk(logits[-1], 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(torch.argmax(logits[-1])))
        logits, states = forward(config, w, [out[-1]], states)
    return out, margins
