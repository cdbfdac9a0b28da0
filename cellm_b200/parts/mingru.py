"""minGRU mixer: a gated recurrence whose gates read only the current token.

    z = sigmoid(W_z h + b_z)        u = W_x h + b_x        c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z) S_(t-1) + z c     output = W_o (S_t * silu(W_g h))

The state S (`width` floats per request, zero at its start) lives in the request's slot. The three input matrices
are stacked so that one product yields z, u and the output gate side by side; gates, candidate and state are 32-bit
whatever the activations are."""
from __future__ import annotations

import torch

from .base import CacheBinding, FixedState, Mixer, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import register_mixer


class MinGRUMixer(Mixer):
    graph_safe = True

    """params: hidden_size, width, bias (default True: z and the candidate have biases).
    weights: z, x, g [width, H]; o [H, width]; z_bias, x_bias [width] if bias."""

    @classmethod
    def weight_specs(cls, params):
        H, W = params["hidden_size"], params["width"]
        specs = {"z": TensorSpec((W, H), "linear"), "x": TensorSpec((W, H), "linear"), "g": TensorSpec((W, H), "linear"),
                 "o": TensorSpec((H, W), "linear")}
        if params.get("bias", True):
            specs["z_bias"] = TensorSpec((W,), "bias")
            specs["x_bias"] = TensorSpec((W,), "bias")
        return specs

    @classmethod
    def cache_need(cls, params):
        return FixedState((int(params["width"]),), torch.float32)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.W, self.dtype = int(params["hidden_size"]), int(params["width"]), dtype
        self.in_proj = Linear(stack_rows(weights["z"], weights["x"], weights["g"]), dtype)
        self.out_proj = Linear(weights["o"], dtype)
        self.bz = self.bx = None
        if params.get("bias", True):
            self.bz = weights["z_bias"].contiguous()
            self.bx = weights["x_bias"].to(self.bz.dtype).contiguous()
        self.extra = 0
        self._record = None

    def stack_behind_input(self, weight: torch.Tensor) -> bool:
        if self._record is not None or self.extra or weight.dtype != self.in_proj.weight.dtype or weight.shape[1] != self.H:
            return False
        self.in_proj = Linear(stack_rows(self.in_proj.weight, weight), self.dtype)
        self.extra = int(weight.shape[0])
        return True

    def stacked_rows(self) -> torch.Tensor:
        return self.in_proj.weight[self.in_proj.weight.shape[0] - self.extra:]

    def record(self):
        from ..ops._lib import tag
        from ..runtime import records as R
        if self._record is None and self.in_proj.weight.dtype == self.dtype == self.out_proj.weight.dtype:
            p = R.MinGruParams(R.linear(self.in_proj.weight), R.linear(self.out_proj.weight), R.ptr(self.bz), R.ptr(self.bx),
                               tag(self.bz) if self.bz is not None else tag(self.dtype), self.W, self.extra)
            self._record = R.Record(R.MINGRU, p, part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            return super().emit(emitter)
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        from ..runtime.program import part_program
        rec = self.record()
        if rec is not None:
            return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx, cache)
        proj = self.in_proj(x, out_dtype=torch.float32)[:, :3 * self.W]
        y = ops.mingru_scan(proj, self.bz, self.bx, cache.state, ctx.slot_ids, ctx.cu_seqlens, self.dtype, ctx.err, ctx.max_q_len)
        return self.out_proj(y)


register_mixer("mingru", MinGRUMixer)
