"""A plain, slow statement of the Binupel design in float64 on the CPU: one function per mechanism, each
written from the mechanism's equations and none of them sharing code with the engine.  Every function that
carries something from token to token takes and returns that state explicitly, so that the tests can run a
prompt whole or token by token through the same function and see that both agree before they compare the
engine with either.

Notation: T tokens, W the stream's width.  ``w`` maps tensor names to float64 tensors.
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
# both to bfloat16, which is where a bfloat16 run rounds.  The difference between the two is the size of the
# error that rounding alone causes, and the tests bound a bfloat16 run's error by a multiple of it.
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
    """x divided by its root mean square over the last axis, eps inside the root."""
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


# ---------------------------------------------------------------------- token shift
def token_shift(x: torch.Tensor, mu: torch.Tensor, before: Optional[torch.Tensor]):
    """h_t = x_t + (x_{t-1} - x_t) * mu.  ``before``: the x of the token ahead of x[0] (None: zeros).
    Returns (h, the last x)."""
    prev = torch.zeros(1, x.shape[1], dtype=x.dtype) if before is None else before.reshape(1, -1)
    shifted = torch.cat([prev, x[:-1]], dim=0)
    return x + (shifted - x) * mu, x[-1].clone()


# ---------------------------------------------------------------------- short convolution
def causal_conv(v: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor, tail: Optional[torch.Tensor]):
    """out[t, c] = bias[c] + sum_j taps[c, j] * v[t - (K - 1 - j), c]; the last column of ``taps`` meets the
    current token.  ``tail``: the K - 1 inputs ahead of v[0] (None: zeros).  Returns (out, new tail)."""
    T, C = v.shape
    K = taps.shape[1]
    tail = torch.zeros(K - 1, C, dtype=v.dtype) if tail is None else tail
    padded = torch.cat([tail, v], dim=0)
    out = torch.zeros(T, C, dtype=v.dtype)
    for t in range(T):
        window = padded[t:t + K]  # inputs t - (K - 1) .. t
        out[t] = (window * taps.t()).sum(dim=0) + bias
    return out, padded[padded.shape[0] - (K - 1):].clone()


# ---------------------------------------------------------------------- RG-LRU block
def rglru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, blocks: int, state=None):
    """``state``: None or (S [C], conv tail [K - 1, C]).  Returns (out [T, W], state)."""
    S, tail = state if state is not None else (None, None)
    y = gelu_tanh(linear(h, w[p + "y"]) + w[p + "y.b"])
    u, tail = causal_conv(linear(h, w[p + "x"]) + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"], tail)
    T, C = u.shape
    bw = C // blocks
    S = torch.zeros(C, dtype=h.dtype) if S is None else S
    lam = softplus(w[p + "lam"])
    rows = []
    for t in range(T):
        r = torch.empty(C, dtype=h.dtype)
        i = torch.empty(C, dtype=h.dtype)
        for b in range(blocks):
            part = u[t, b * bw:(b + 1) * bw]
            r[b * bw:(b + 1) * bw] = sigmoid(w[p + "ra"][b] @ part + w[p + "ra.b"][b])
            i[b * bw:(b + 1) * bw] = sigmoid(w[p + "ri"][b] @ part + w[p + "ri.b"][b])
        a = torch.exp(-8.0 * r * lam)
        S = a * S + torch.sqrt(1.0 - a * a) * (i * u[t])
        rows.append(S * y[t])
    return linear(torch.stack(rows), w[p + "o"]), (S, tail)


# ---------------------------------------------------------------------- selective scan
def selective_scan(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, dt_rank: int, state=None):
    """``state``: None or (S [I, N], conv tail [K - 1, I]).  Returns (out [T, W], state)."""
    S, tail = state if state is not None else (None, None)
    both = linear(h, w[p + "in"])
    inner = both.shape[1] // 2
    x, z = both[:, :inner], both[:, inner:]
    x, tail = causal_conv(x, w[p + "conv"], w[p + "conv.b"], tail)
    x = silu(x)
    low = linear(x, w[p + "x"])
    n = (low.shape[1] - dt_rank) // 2
    step = softplus(linear(low[:, :dt_rank], w[p + "dt"]) + w[p + "dt.b"])
    Bm, Cm = low[:, dt_rank:dt_rank + n], low[:, dt_rank + n:]
    A = -torch.exp(w[p + "A_log"])
    S = torch.zeros(inner, n, dtype=h.dtype) if S is None else S
    rows = []
    for t in range(h.shape[0]):
        S = torch.exp(step[t].unsqueeze(1) * A) * S + (step[t] * x[t]).unsqueeze(1) * Bm[t].unsqueeze(0)
        rows.append(S @ Cm[t] + w[p + "D"] * x[t])
    y = torch.stack(rows) * silu(z)
    return linear(y, w[p + "o"]), (S, tail)


# ---------------------------------------------------------------------- attention
def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def sigmoid_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, state=None):
    """``state``: None or (normed keys [n, G, d], raw keys [n, G, d]) of the tokens before h[0].
    Returns (out [T, W], state)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = linear(h, w[p + "q"]).view(T, H, d)
    k = linear(h, w[p + "k"]).view(T, G, d)
    kn = unit_rms(k, eps) * w[p + "k.norm"]
    keys, values = (kn, k) if state is None else (torch.cat([state[0], kn]), torch.cat([state[1], k]))
    past = keys.shape[0] - T
    positions = past + torch.arange(T)
    qn = unit_rms(q, eps) * w[p + "q.norm"]
    if m.get("q_temp") is not None:
        qn = qn * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"]).view(T, 1, 1)
    gate = sigmoid(linear(h, w[p + "g"]))
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        visible = int(positions[t]) + 1
        for head in range(H):
            kv = head // (H // G)
            score = keys[:visible, kv] @ qn[t, head] * m["scale"] + w[p + "pb"][head]
            out[t, head] = gate[t, head] * (sigmoid(score).unsqueeze(1) * values[:visible, kv]).sum(dim=0)
    return linear(out.reshape(T, H * d), w[p + "o"]), (keys, values)


# ---------------------------------------------------------------------- feed-forward
def relu_glu(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return linear(torch.relu(linear(x, w[p + "gate"])) * linear(x, w[p + "up"]), w[p + "down"])


# ---------------------------------------------------------------------- layer and model
def run_mixer(kind: str, h, w, p, m, eps, state):
    if kind == "attention":
        return sigmoid_attention(h, w, p, m, eps, state)
    if kind == "rglru":
        return rglru(h, w, p, m["blocks"], state)
    if kind == "mamba1":
        return selective_scan(h, w, p, m["dt_rank"], state)
    raise ValueError(kind)


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], config: dict, index: int, state=None):
    """One entry of ``layers`` on the tokens x [T, W].  ``state``: None or (last x, mixer state)."""
    entry = config["layers"][index]
    p = f"l{entry.get('weights_of', index)}."
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    before, mixer_state = state if state is not None else (None, None)
    h, last = token_shift(x, w[p + "shift"], before)
    mixed, mixer_state = run_mixer(entry["type"], h, w, p + "mix.", entry["mixer"], eps, mixer_state)
    x = rms_norm(alpha * x + mixed, w[p + "norm1"], eps)
    if entry.get("mlp") is not None:
        x = rms_norm(alpha * x + relu_glu(x, w, p + "mlp."), w[p + "norm2"], eps)
    return x, (last, mixer_state)


def forward(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], states: Optional[List] = None):
    """Logits [T, vocab] of the tokens ``ids`` that follow what ``states`` has seen.  Returns (logits, states)."""
    x = w["embed"][torch.tensor(list(ids), dtype=torch.long)]
    states = [None] * len(config["layers"]) if states is None else list(states)
    for i in range(len(config["layers"])):
        x, states[i] = layer(x, w, config, i, states[i])
    return linear(rms_norm(x, w["final.norm"], config["norm"]["eps"]), w["head"]), states


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
