"""The recurrent block with a real-gated linear recurrent unit (RG-LRU), as in the Griffin architecture.

Two branches of size ``width`` from the block's input ``h``: ``y = gelu_tanh(W_y h + b_y)`` and
``u = conv(W_x h + b_x)``, a short convolution along time with ``taps`` weights per channel: weight ``taps - 1`` multiplies
the current token's input, weight ``k`` the input ``taps - 1 - k`` tokens back, and a new sequence has only zeros behind it.
The channels of ``u`` fall into ``blocks`` consecutive slices of equal size; slice ``b`` has two square matrices that give its
gates, ``r_t = sigmoid(A_b u_b + a_b)`` (recurrence) and ``i_t = sigmoid(I_b u_b + i_b)`` (input).  With
``a_t = exp(-decay * softplus(lam) * r_t)`` the state moves as ``S_t = a_t * S_{t-1} + sqrt(1 - a_t^2) * (i_t * u_t)``; a new
sequence has ``S = 0`` and its first token runs this same update.  The block returns ``W_o (S * y)``.

Per request the state slot holds ``[taps, width]`` 32-bit values: the recurrent state and the convolution's last
``taps - 1`` inputs, so a sequence may be cut into steps anywhere.  Gates, decay and the recurrence are 32-bit in every
run; the two input projections are one product, the block-diagonal gate products one batched product.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, FixedStateNeed, FixedStateView, StepContext
from ..registry import register_part


@register_part("mixer", "rglru")
class RGLRU(Mixer):
    def __init__(self, prefix: str, d_model: int, width: int, blocks: int, taps: int, decay: float = 8.0,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        if width % blocks:
            raise ValueError(f"width {width} is not a multiple of {blocks} blocks")
        if taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {taps}")
        self.d_model, self.width, self.blocks, self.taps, self.decay = int(d_model), int(width), int(blocks), int(taps), float(decay)
        self.bs = self.width // self.blocks
        self.names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                      "gate_a": "ra", "gate_a_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "o": "o"}
        if names:
            self.names.update(names)

    def param_specs(self):
        n, d, W, B, bs = self.names, self.d_model, self.width, self.blocks, self.bs
        return {n["y"]: ParamSpec((W, d)), n["y_bias"]: ParamSpec((W,), init="zeros"),
                n["x"]: ParamSpec((W, d)), n["x_bias"]: ParamSpec((W,), init="zeros"),
                n["conv"]: ParamSpec((W, self.taps), storage="vector", init="normal", std=0.3),
                n["conv_bias"]: ParamSpec((W,), storage="vector", init="zeros"),
                n["gate_a"]: ParamSpec((B, bs, bs), std=0.1), n["gate_a_bias"]: ParamSpec((B, bs), storage="vector", init="zeros"),
                n["gate_i"]: ParamSpec((B, bs, bs), std=0.1), n["gate_i_bias"]: ParamSpec((B, bs), storage="vector", init="zeros"),
                n["lam"]: ParamSpec((W,), storage="vector", init="normal", std=1.0),
                n["o"]: ParamSpec((d, W))}

    def load(self, params):
        n = self.names
        self.w_in = torch.cat([params[n["y"]], params[n["x"]]], dim=0).contiguous()             # [2W, d]: y first
        self.b_in = torch.cat([params[n["y_bias"]], params[n["x_bias"]]], dim=0).contiguous()
        vec = params[n["lam"]].dtype
        self.conv_w = params[n["conv"]].to(vec).t().contiguous()                               # tap-major [taps, W]: a tap's weights lie side by side
        self.conv_b = params[n["conv_bias"]].to(vec).contiguous()
        self.w_gates = torch.cat([params[n["gate_a"]], params[n["gate_i"]]], dim=1).contiguous()   # [B, 2*bs, bs]: r rows, then i rows
        self.gate_a_bias = params[n["gate_a_bias"]].to(vec).reshape(-1).contiguous()
        self.gate_i_bias = params[n["gate_i_bias"]].to(vec).reshape(-1).contiguous()
        self.lam = params[n["lam"]].contiguous()
        self.w_out = params[n["o"]].contiguous()

    def product_weights(self):
        return [self.w_in, self.w_out]

    def cache_need(self):
        return FixedStateNeed((self.taps, self.width), "float32")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: FixedStateView) -> torch.Tensor:
        ops, W = self.ops, self.width
        proj = ops.linear(x, self.w_in, self.b_in)                   # [T, 2W] = [y pre-activation | convolution input]
        T = proj.shape[0]
        lowp = x.dtype != torch.float32
        u32, u_c = ops.causal_conv(proj, W, W, self.taps, self.conv_w, self.conv_b, cache.state, ctx.token_seq,
                                   ctx.query_start_loc, ctx.slot_ids, lowp)
        ub = (u_c if lowp else u32).view(T, self.blocks, self.bs).transpose(0, 1)               # [B, T, bs], a view
        pre = ops.batched_linear(ub, self.w_gates, out_dtype=torch.float32)                      # [B, T, 2*bs] float32
        gated = ops.rglru_scan(pre, self.gate_a_bias, self.gate_i_bias, self.lam, u32, proj, W, proj, 0, cache.state,
                               ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs, W, self.taps, self.bs, self.decay,
                               ctx.max_q_len, ctx.num_tokens)
        return ops.linear(gated, self.w_out, None, partial_ok=True)
