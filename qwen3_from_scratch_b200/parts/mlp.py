"""Gated feed-forward: y = (up(x) * act(gate(x))) W_down^T, no biases.  ``swiglu`` is the form with the SiLU
gate and the checkpoint's ``gate_proj`` / ``up_proj`` / ``down_proj`` names; ``gated_mlp`` takes the gate's
activation (``silu``, ``relu``, ``gelu_tanh``) and the tensors' names as parameters.

Reference: models/feedback.py:14-34.  The gate and up weights are merged into one [2I, H] weight at load, so
one product feeds the gate kernel.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import FeedForward, Runtime, StreamNorm, WeightSpec
from .linear import Linear

_DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_capturable = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: Optional[Dict[str, str]] = None):
        """``names``: what follows the part's name (and a dot) in the names of its gate, up and down tensors."""
        super().__init__(name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        ops.activation_code(activation, gate=True)
        self.activation = activation
        n = dict(_DEFAULT_NAMES)
        n.update(names or {})
        self.tensors = {k: f"{name}.{v}" for k, v in n.items()}

    def weight_specs(self) -> List[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.tensors["gate"], (i, h)),
                WeightSpec(self.tensors["up"], (i, h)),
                WeightSpec(self.tensors["down"], (h, i))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        gate = weights.pop(self.tensors["gate"])
        up = weights.pop(self.tensors["up"])
        dtype = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        h, i = self.hidden_size, self.intermediate_size
        # bfloat16: gate and up rows alternate in blocks of eight, so that the decode kernel has a
        # gate value and its up value in one thread and applies the activation before storing
        self.blocks_of_eight = dtype == torch.bfloat16 and i % 8 == 0
        if self.blocks_of_eight:
            merged = torch.cat([gate.view(i // 8, 8, h), up.view(i // 8, 8, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            merged = torch.cat([gate.to(dtype), up.to(dtype)], dim=0)
        del gate, up
        self.gate_up = Linear(merged, rt, tag="ffn.gate_up")
        self.down = Linear(weights.pop(self.tensors["down"]), rt, tag="ffn.down")
        self._act = rt.shared("ffn.act", rt.max_tokens, self.intermediate_size)
        # the few-rows product applies any gate in its epilogue, the tcgen05 product those of ops.GEMM_TC_GATES; the
        # product that also applies a norm that was never computed is built for the SiLU gate
        self.fused_gate = self.blocks_of_eight

    fuses_stream = True

    def can_fuse_stream(self, rows: int) -> bool:
        return (self.fused_gate and self.activation == "silu" and self.gate_up.takes_stream_norm(rows)
                and self.down.can_add_into_stream(rows))

    def forward(self, x, into_stream=None, next_norm_weight=None):
        act = self._act[: x.shape[0]]
        rows = x.shape[0]
        if isinstance(x, StreamNorm):
            # decoding without norm kernels: the norm is applied inside the gate/up product
            ops.gemm_skinny_normed(x.scaled, x.sumsq, x.parts, x.eps, self.gate_up.weight, act, swiglu_blocks=True)
        elif self.fused_gate and ops.gemm_skinny_takes(rows, self.gate_up.weight):
            # decoding: stream the weight once, activation applied before the store
            ops.gemm_skinny(x, self.gate_up.weight, act, swiglu_blocks=True, activation=self.activation)
        elif (self.fused_gate and self.activation in ops.GEMM_TC_GATES
              and ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight) and ops.gemm_tc_takes(x, self.gate_up.weight)):
            # prompt portions: the engine's tcgen05 product with the activation in its epilogue, so the
            # [T, 2I] gate/up product never goes to memory
            ops.gemm_tc(x, self.gate_up.weight, act, self.rt.status, swiglu_blocks=True,
                        pair=ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight) == "pair", activation=self.activation)
        else:
            ops.gated_act(self.gate_up(x), act, interleave8=self.blocks_of_eight, activation=self.activation)
        if into_stream is not None:
            return self.down.into_stream(act, into_stream, next_norm_weight)
        return self.down(act)


@register_part("feed_forward", "swiglu")
class SwiGLU(GatedMLP):
    def __init__(self, name: str, hidden_size: int, intermediate_size: int):
        super().__init__(name, hidden_size, intermediate_size, activation="silu")


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """Feed-forward without a gate: y = W_down act(W_up x), no biases.  ``names``: what follows the part's name (and
    a dot) in the names of its up and down tensors."""

    graph_capturable = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh",
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        ops.activation_code(activation, gate=True)
        self.activation = activation
        n = {"up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.tensors = {k: f"{name}.{v}" for k, v in n.items()}

    def weight_specs(self) -> List[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.tensors["up"], (i, h)), WeightSpec(self.tensors["down"], (h, i))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.up = Linear(weights.pop(self.tensors["up"]), rt, tag="ffn.up")
        self.down = Linear(weights.pop(self.tensors["down"]), rt, tag="ffn.down")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        if (ops.gemm_skinny_takes(rows, self.up.weight) and x.dtype == torch.bfloat16
                and self.up.out_dtype == torch.bfloat16):
            # decoding: the weight is streamed once and the activation applied before the store
            h = self.up._buffer("_out", rows, self.up.out_dtype)
            ops.gemm_skinny(x, self.up.weight, h, plain_activation=self.activation)
            return self.down(h)
        h = self.up(x)
        ops.act(h, h, self.activation)
        return self.down(h)
