"""A selective state-space mixer (Mamba, first form): an input product into a convolved branch x and a gate z, a short
causal convolution per channel with SiLU, products that give each token its step size dt and its input and output
vectors B and C, the recurrence S <- exp(dt A) S + dt x B, y = S C + D x per channel, the gate y * silu(z), and an
output product.  The products run on the engine's matrix kernels; convolution, recurrence and gate are the kernels of
csrc/selective_scan.cu.  Each request keeps, in its state slot, S (FP32 [inner, state]) and the convolution's last
taps - 1 inputs, so a prompt may be cut anywhere and a decoded token costs one step of the recurrence."""
from __future__ import annotations

import torch

from .. import ops
from ..spec import TensorSpec
from . import linear
from .base import Mixer, register_mixer, to_f32, to_operand

_NAMES = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "x": "x_proj.weight", "dt": "dt_proj.weight",
          "dt_bias": "dt_proj.bias", "A_log": "A_log", "D": "D", "out": "out_proj.weight"}


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, inner: int, state: int, conv: int, dt_rank: int, names=None):
        if conv < 1 or conv > 16:
            raise ValueError(f"{conv} convolution taps: the kernel takes 1 to 16")
        if state < 1 or state > 256:
            raise ValueError(f"{state} states per channel: the kernel takes 1 to 256")
        self.D, self.inner, self.N, self.taps, self.R = hidden_size, inner, state, conv, dt_rank
        self.names = {**_NAMES, **(names or {})}

    def tensors(self):
        n, C = self.names, self.inner
        return [TensorSpec(n["in"], (2 * C, self.D)),
                TensorSpec(n["conv"], (C, self.taps), "f32", ("normal", 0.4)), TensorSpec(n["conv_bias"], (C,), "f32", ("normal", 0.1)),
                TensorSpec(n["x"], (self.R + 2 * self.N, C)),
                TensorSpec(n["dt"], (C, self.R), "matrix", ("normal", 0.3)), TensorSpec(n["dt_bias"], (C,), "f32", ("normal", 0.5)),
                TensorSpec(n["A_log"], (C, self.N), "f32", ("normal", 0.5)), TensorSpec(n["D"], (C,), "f32", ("ones_plus", 0.1)),
                TensorSpec(n["out"], (self.D, C))]

    def bind(self, get, rt):
        self.rt = rt
        n = self.names
        self.w_in, self.w_x = to_operand(get(n["in"]), rt), to_operand(get(n["x"]), rt)
        self.w_dt, self.w_o = to_operand(get(n["dt"]), rt), to_operand(get(n["out"]), rt)
        self.conv_w, self.conv_b = to_f32(get(n["conv"]), rt), to_f32(get(n["conv_bias"]), rt)
        self.dt_b, self.skip = to_f32(get(n["dt_bias"]), rt), to_f32(get(n["D"]), rt)
        self.A = (-torch.exp(to_f32(get(n["A_log"]), rt))).contiguous()          # FP32: the decay is exp(dt * A)

    def state_shape(self):
        return {"ssm": ((self.inner, self.N), torch.float32), "conv": ((self.taps - 1, self.inner), torch.float32)}

    def forward(self, xn, ctx, cache, state, out):
        rt, C, N, R = self.rt, self.inner, self.N, self.R
        ops.current_tag = "scan.in"
        xz = linear.matmul(xn, self.w_in, rt)                                   # FP32 [T, x | z]
        ops.current_tag = "scan.conv"
        u = ops.conv_silu(xz, C, self.conv_w, self.conv_b, state["conv"], ctx.req_of_token, ctx.q_start, ctx.slot_ids, rt.dtype)
        ops.current_tag = "scan.x"
        proj = linear.matmul(u, self.w_x, rt)                                   # FP32 [T, dt | B | C]
        ops.current_tag = "scan.dt"
        dt_raw = linear.matmul(ops.cast_columns(proj, 0, R, rt.dtype), self.w_dt, rt)     # FP32 [T, inner]; bias and softplus in the scan
        ops.current_tag = "scan.recurrence"
        key = ("scan_segments",)
        if key not in ctx.plans:                # long portions are walked in segments by several blocks: the same plan for every layer
            ctx.plans[key] = ops.selective_scan_segments(ctx.q_lens, rt.device)
        y = ops.selective_scan(u, dt_raw, self.dt_b, proj, R, R + N, self.A, self.skip, xz, C, state["ssm"], state["conv"],
                               ctx.q_start, ctx.slot_ids, ctx.R, segments=ctx.plans[key])
        ops.current_tag = "scan.out"
        return linear.matmul(y, self.w_o, rt, partials_ok=True)
