"""A routed feed-forward: many small experts, of which every token runs a few, and optionally one shared expert
that every token runs.

    z = R h (32-bit);  s = sigmoid(z);  c = s + correction
    the experts lie in `groups` equal runs of neighbours; a run's score is the sum of its two largest c; only
    experts of the `keep_groups` best runs can be chosen
    the `top` experts with the largest c are chosen; weight_k = s_k / (sum of the chosen s + 1e-20) * route_scale
    out = sum_k weight_k * D_k act(U_k h)  +  sigmoid(g . h) * D_s act(U_s h)

The experts' matrices are kept one below the other, so that a kernel reaches expert e by an offset. The router's
rows and the shared expert's gate row form one matrix."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import FeedForward, StepContext, TensorSpec
from .linear import stack_rows
from .registry import register_feed_forward

ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


class RoutedExperts(FeedForward):
    graph_safe = True

    """params: hidden_size, experts, top, ff_dim, activation ("gelu": the exact form), route_scale, groups (default 1),
    keep_groups (default groups), correction (default True), shared_ff (default 0: no shared expert), shared_gate
    (default True). weights: router [experts, H], correction [experts], up_<e> [ff, H] and down_<e> [H, ff] for every
    expert e, shared_up [shared_ff, H], shared_down [H, shared_ff], shared_gate [1, H]."""

    @classmethod
    def weight_specs(cls, params):
        H, E, ff = params["hidden_size"], params["experts"], params["ff_dim"]
        specs = {"router": TensorSpec((E, H), "linear")}
        if params.get("correction", True):
            specs["correction"] = TensorSpec((E,), "bias")
        for e in range(E):
            specs[f"up_{e}"] = TensorSpec((ff, H), "linear")
            specs[f"down_{e}"] = TensorSpec((H, ff), "linear")
        sff = params.get("shared_ff", 0)
        if sff:
            specs["shared_up"] = TensorSpec((sff, H), "linear")
            specs["shared_down"] = TensorSpec((H, sff), "linear")
            if params.get("shared_gate", True):
                specs["shared_gate"] = TensorSpec((1, H), "linear")
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.E, self.top, self.ff = (int(params[k]) for k in ("hidden_size", "experts", "top", "ff_dim"))
        self.dtype = dtype
        self.groups = int(params.get("groups", 1))
        self.keep = int(params.get("keep_groups", self.groups))
        self.route_scale = float(params.get("route_scale", 1.0))
        self.activation = params.get("activation", "gelu")
        if self.activation not in ACTIVATIONS:
            raise ConfigError(f"routed_experts: activation {self.activation!r}; known: {sorted(ACTIVATIONS)}")
        if not 1 <= self.top <= self.E:
            raise ConfigError(f"routed_experts: top {self.top} of {self.E} experts")
        if self.groups < 1 or self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ConfigError(f"routed_experts: {self.E} experts in {self.groups} groups of which {self.keep} are kept")
        if self.keep * (self.E // self.groups) < self.top:
            raise ConfigError(f"routed_experts: {self.keep} groups of {self.E // self.groups} experts cannot give {self.top} choices")
        self.up = stack_rows(*[weights[f"up_{e}"] for e in range(self.E)])
        self.down = stack_rows(*[weights[f"down_{e}"] for e in range(self.E)])
        dev = self.up.device
        self.shared_ff = int(params.get("shared_ff", 0))
        self.has_gate = bool(self.shared_ff and params.get("shared_gate", True))
        self.router = stack_rows(weights["router"], weights["shared_gate"]) if self.has_gate else weights["router"].contiguous()
        self.correction = (weights["correction"].contiguous() if params.get("correction", True)
                           else torch.zeros(self.E, dtype=torch.float32, device=dev))
        self.shared_up = weights["shared_up"].contiguous() if self.shared_ff else None
        self.shared_down = weights["shared_down"].contiguous() if self.shared_ff else None
        self._record = None

    def record(self):
        from ..ops._lib import tag
        from ..runtime import records as R
        mats = [self.up, self.down, self.router] + ([self.shared_up, self.shared_down] if self.shared_ff else [])
        if self._record is None and all(m.dtype == self.dtype for m in mats):
            p = R.RoutedMlpParams()
            p.up, p.down, p.router = R.linear(self.up), R.linear(self.down), R.linear(self.router)
            p.correction, p.c_dtype = self.correction.data_ptr(), tag(self.correction)
            p.experts, p.top, p.n_groups, p.keep, p.scale = self.E, self.top, self.groups, self.keep, self.route_scale
            p.ff, p.act = self.ff, ACTIVATIONS[self.activation]
            if self.shared_ff:
                p.shared_up, p.shared_down = R.linear(self.shared_up), R.linear(self.shared_down)
            p.shared_ff, p.shared_gate = self.shared_ff, int(self.has_gate)
            self._record = R.Record(R.ROUTED_MLP, p, part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            raise ConfigError("routed_experts: matrices kept in another element type than the activations")
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from ..runtime.program import part_program
        rec = self.record()
        if rec is None:
            raise ConfigError("routed_experts: matrices kept in another element type than the activations")
        return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx)


register_feed_forward("routed_experts", RoutedExperts)
