"""Gated feed-forward in its general form: W_down (act(W_gate h + b_gate) * (W_up h + b_up)) + b_down, with act
"silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) and optional biases. Gate and up are
stacked so that one product yields both; they stay 32-bit until act(g) * u is formed."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import FeedForward, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import register_feed_forward

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


class GatedMLP(FeedForward):
    graph_safe = True

    """params: hidden_size, ff_dim, activation, bias. weights: gate, up [ff, H]; down [H, ff];
    gate_bias, up_bias [ff], down_bias [H] if bias."""

    @classmethod
    def weight_specs(cls, params):
        H, ff = params["hidden_size"], params["ff_dim"]
        specs = {"gate": TensorSpec((ff, H), "linear"), "up": TensorSpec((ff, H), "linear"), "down": TensorSpec((H, ff), "linear")}
        if params.get("bias"):
            specs.update(gate_bias=TensorSpec((ff,), "bias"), up_bias=TensorSpec((ff,), "bias"), down_bias=TensorSpec((H,), "bias"))
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.ff, self.dtype = int(params["hidden_size"]), int(params["ff_dim"]), dtype
        self.activation = params.get("activation", "silu")
        if self.activation not in ACTIVATIONS:
            raise ConfigError(f"gated_mlp: activation {self.activation!r}; known: {sorted(ACTIVATIONS)}")
        self.gate_up = Linear(stack_rows(weights["gate"], weights["up"]), dtype)
        self.down = Linear(weights["down"], dtype)
        self.bg = self.bu = self.bd = None
        if params.get("bias"):
            self.bg = weights["gate_bias"].contiguous()
            self.bu = weights["up_bias"].to(self.bg.dtype).contiguous()
            self.bd = weights["down_bias"].to(self.bg.dtype).contiguous()
        self.extra = 0
        self._record = None

    def stack_behind_input(self, weight: torch.Tensor) -> bool:
        if self._record is not None or self.extra or weight.dtype != self.gate_up.weight.dtype or weight.shape[1] != self.H:
            return False
        self.gate_up = Linear(stack_rows(self.gate_up.weight, weight), self.dtype)
        self.extra = int(weight.shape[0])
        return True

    def stacked_rows(self) -> torch.Tensor:
        return self.gate_up.weight[self.gate_up.weight.shape[0] - self.extra:]

    def record(self):
        from ..ops._lib import tag
        from ..runtime import records as R
        if self._record is None and self.gate_up.weight.dtype == self.dtype == self.down.weight.dtype:
            p = R.GatedMlpParams(R.linear(self.gate_up.weight), R.linear(self.down.weight), R.ptr(self.bg), R.ptr(self.bu),
                                 R.ptr(self.bd), tag(self.bg) if self.bg is not None else tag(self.dtype), self.ff,
                                 ACTIVATIONS[self.activation], self.extra)
            self._record = R.Record(R.GATED_MLP, p, part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            return super().emit(emitter)
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from .. import ops
        from ..runtime.program import part_program
        rec = self.record()
        if rec is not None:
            return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx)
        gu = self.gate_up(x, out_dtype=torch.float32)[:, :2 * self.ff]
        y = self.down(ops.gated_act(gu, self.bg, self.bu, self.activation, self.dtype), out_dtype=torch.float32)
        if self.bd is not None:
            y = y + self.bd.to(torch.float32)
        return y.to(self.dtype)


register_feed_forward("gated_mlp", GatedMLP)
