"""A gated delta rule mixer: per head a matrix-valued state S [dk, dv] that every token first decays, then corrects along
its key towards its value, and reads with its query:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

q and k come from `num_kv_heads` projected heads (query head h uses head h // (heads / kv_heads)), v from `num_heads`.
Each of q, k and v passes a short causal convolution over time per channel and SiLU; q and k are then made unit
vectors per head (q also times dk^-1/2); beta = sigmoid(W_b x) and g = exp(-exp(A_log) softplus(W_a x + dt_bias)) are one
number per head and token.  Each head's o is divided by its root mean square, multiplied by a weight shared by the
heads and by silu(W_g x), and leaves through the output product.

The products run on the engine's matrix kernels (q, k, v, the gate and the two per-head projections as one stacked
product); convolution, recurrence and output norm are the kernels of csrc/gated_delta.cu.  Everything between the
projection and the output product is FP32.  Each request keeps, in its state slot, S (FP32) and the convolution's
last taps - 1 projected values, so a prompt may be cut anywhere and a decoded token costs one step of the recurrence.
"""
from __future__ import annotations

import torch

from .. import ops
from ..spec import TensorSpec
from . import linear
from .base import Mixer, register_mixer, to_f32

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight",
          "v_conv": "v_conv.weight", "beta": "b_proj.weight", "decay": "a_proj.weight", "A_log": "A_log", "dt_bias": "dt_bias",
          "gate": "g_proj.weight", "norm": "norm.weight", "o": "o_proj.weight"}


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    graph_safe = True
    prepare_beyond = 16          # steps whose longest portion has more tokens make the recurrence's per-token inputs in a kernel of their own

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, conv: int, eps: float, names=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key heads")
        if conv < 1 or conv > 16:
            raise ValueError(f"{conv} convolution taps: the kernel takes 1 to 16")
        self.D, self.H, self.G, self.dk, self.dv, self.taps, self.eps = hidden_size, num_heads, num_kv_heads, head_dim, v_dim, conv, float(eps)
        self.names = {**_NAMES, **(names or {})}
        # columns of the stacked product: [q | k | v | gate | beta | decay], padded to a multiple of 8 rows
        self.C = 2 * self.G * self.dk + self.H * self.dv
        self.g_col, self.b_col, self.a_col = self.C, self.C + self.H * self.dv, self.C + self.H * self.dv + self.H
        self.N = (self.a_col + self.H + 7) // 8 * 8

    def tensors(self):
        n, D, H, G, dk, dv = self.names, self.D, self.H, self.G, self.dk, self.dv
        return [TensorSpec(n["q"], (G * dk, D)), TensorSpec(n["q_conv"], (G * dk, self.taps), "f32", ("normal", 0.5)),
                TensorSpec(n["k"], (G * dk, D)), TensorSpec(n["k_conv"], (G * dk, self.taps), "f32", ("normal", 0.5)),
                TensorSpec(n["v"], (H * dv, D)), TensorSpec(n["v_conv"], (H * dv, self.taps), "f32", ("normal", 0.5)),
                TensorSpec(n["beta"], (H, D)), TensorSpec(n["A_log"], (H,), "f32", ("normal", 0.5)),
                TensorSpec(n["norm"], (dv,), "f32", ("ones_plus", 0.1)), TensorSpec(n["decay"], (H, D)),
                TensorSpec(n["dt_bias"], (H,), "f32", ("normal", 0.5)), TensorSpec(n["gate"], (H * dv, D)),
                TensorSpec(n["o"], (D, H * dv))]

    def bind(self, get, rt):
        if self.dk > ops.gated_delta_max_dim():
            raise ValueError(f"keys of {self.dk} entries: the recurrence kernel takes up to {ops.gated_delta_max_dim()}")
        self.rt = rt
        n = self.names
        self.w_in = torch.zeros((self.N, self.D), dtype=rt.dtype, device=rt.device)
        at = 0
        for name in ("q", "k", "v", "gate", "beta", "decay"):
            w = get(n[name])
            self.w_in[at:at + w.shape[0]].copy_(w)
            at += w.shape[0]
        self.conv_w = torch.cat([to_f32(get(n[x + "_conv"]), rt) for x in "qkv"]).contiguous()
        self.A_log, self.dt_bias, self.norm_w = to_f32(get(n["A_log"]), rt), to_f32(get(n["dt_bias"]), rt), to_f32(get(n["norm"]), rt)
        self.w_o = torch.empty((self.D, self.H * self.dv), dtype=rt.dtype, device=rt.device)
        self.w_o.copy_(get(n["o"]))

    def state_shape(self):
        # the state is kept column-major: a column's rows lie together
        return {"S": ((self.H, self.dv, self.dk), torch.float32), "conv": ((self.taps - 1, self.C), torch.float32)}

    def forward(self, xn, ctx, cache, state, out):
        rt = self.rt
        ops.current_tag = "delta.in"
        p = linear.matmul(xn, self.w_in, rt)                                      # FP32 [T, q | k | v | gate | beta | decay]
        ops.current_tag = "delta.conv"
        u = ops.short_conv(p, self.C, self.conv_w, None, state["conv"], ctx.req_of_token, ctx.q_start, ctx.slot_ids, ctx.R, act="silu")
        ops.current_tag = "delta.recurrence"
        o = ops.gated_delta(u, p, self.b_col, self.a_col, self.A_log, self.dt_bias, state["S"], ctx.q_start, ctx.slot_ids, ctx.R,
                            self.H, self.G, self.dk, self.dv, prepare=ctx.max_q_len > self.prepare_beyond)
        ops.current_tag = "delta.out"
        y = ops.delta_out(o, p, self.g_col, self.norm_w, self.eps, self.H, self.dv, rt.dtype)
        ops.current_tag = "delta.o"
        return linear.matmul(y, self.w_o, rt, partials_ok=not ctx.hold_results)
