"""Feed-forward without a gate: y = W_down act(W_up h), act one of `kernels.ops.ACTIVATIONS`
(relu2: the square of relu; gelu_tanh; gelu, the erf form; silu; relu)."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import FeedForward, Runtime, StepContext
from .registry import register_part

DEFAULT_NAMES = {"up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("ffn", "dense_mlp")
class DenseMLP(FeedForward):
    graph_safe = True

    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 names: dict | None = None):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_mlp: activation {activation!r} is not one of {', '.join(ops.ACTIVATIONS)}")
        self.runtime, self.D, self.F, self.activation = runtime, hidden_size, intermediate_size, activation
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.w_up: linear.LinearWeight | None = None
        self.w_down: linear.LinearWeight | None = None

    def weights(self):
        n = self.names
        return {n["up"]: WeightSpec((self.F, self.D)), n["down"]: WeightSpec((self.D, self.F))}

    def load(self, tensors):
        self.w_up = linear.LinearWeight(tensors[self.names["up"]])
        self.w_down = linear.LinearWeight(tensors[self.names["down"]])

    def forward(self, h, ctx: StepContext, residual):
        """With `residual` None the output comes back as float32 [T, D] instead of being added."""
        act = linear.linear_act(h, self.w_up, self.activation, self.runtime.act_dtype)
        if residual is None:
            return linear.linear(act, self.w_down, torch.float32)
        linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual)
        return None
