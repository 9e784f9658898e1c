"""The matrix memory of xLSTM (mLSTM): a matrix state per head with exponential gating and a running maximum.

With ``h`` the mixer's input: ``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim); per head
a log input gate ``i = cap * tanh((W_i h + b_i) / cap)`` and a log forget gate
``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``.  S, n and the running maximum m start at zero (m at 0, not at minus
infinity):

    m_t = max(f + m_(t-1), i)      S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T      n_t likewise with k alone
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Each head's ``o`` is divided by its root mean square (``x / sqrt(mean(x^2) + eps)``), the heads are concatenated, multiplied
by ``norm`` and by ``sigmoid(W_g h)``, and projected by ``W_o``.

Per request three state rows, all 32-bit: S ``[heads, vdim, padded dim]``, n ``[heads, padded dim]`` and m ``[heads]``.
Gates, exponentials, state and read-out are 32-bit in every run; the gate pre-activations leave their (small) product in
32-bit; q, k, v and the output gate are one product.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, FixedStateNeed, StepContext
from .wkv import padded_keys, MAX_KEYS
from ..registry import register_part

DENOMINATOR_FLOOR = 1e-6        # added to the read-out's denominator (the scan kernel carries the same constant)


@register_part("mixer", "mlstm")
class MLSTM(Mixer):
    def __init__(self, prefix: str, d_model: int, num_heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.d_model, self.num_heads, self.dim, self.vdim = int(d_model), int(num_heads), int(dim), int(vdim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        if self.dim > MAX_KEYS:
            raise ValueError(f"mlstm: {dim} key channels per head (at most {MAX_KEYS})")
        if not self.gate_cap > 0:
            raise ValueError(f"mlstm: gate_cap must be positive, got {gate_cap}")
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b",
                      "norm": "norm", "o": "o"}
        if names:
            self.names.update(names)

    def param_specs(self):
        n, d, H, D, Dv = self.names, self.d_model, self.num_heads, self.dim, self.vdim
        return {n["q"]: ParamSpec((H * D, d)), n["k"]: ParamSpec((H * D, d)), n["v"]: ParamSpec((H * Dv, d)),
                n["g"]: ParamSpec((H * Dv, d)), n["i"]: ParamSpec((H, d)), n["f"]: ParamSpec((H, d)),
                n["i_bias"]: ParamSpec((H,), storage="vector", init="normal", std=1.0),
                n["f_bias"]: ParamSpec((H,), storage="vector", init="normal", std=1.0),
                n["norm"]: ParamSpec((H * Dv,), storage="vector", init="ones"), n["o"]: ParamSpec((d, H * Dv))}

    def load(self, params):
        n = self.names
        self.w_in = torch.cat([params[n[s]] for s in ("q", "k", "v", "g")], dim=0).contiguous()       # [2*H*dim + 2*H*vdim, d]
        self.w_gates = torch.cat([params[n["i"]], params[n["f"]]], dim=0).contiguous()                  # [2H, d]: input gate rows, then forget
        self.b_gates = torch.cat([params[n["i_bias"]], params[n["f_bias"]]], dim=0).to(self.w_gates.dtype).contiguous()
        self.norm_w = params[n["norm"]].float().contiguous()
        self.w_out = params[n["o"]].contiguous()

    def product_weights(self):
        return [self.w_in, self.w_out]

    def cache_needs(self):
        P = padded_keys(self.dim)
        return [FixedStateNeed((self.num_heads, self.vdim, P), "float32"), FixedStateNeed((self.num_heads, P), "float32"),
                FixedStateNeed((self.num_heads,), "float32")]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        ops, H, D, Dv = self.ops, self.num_heads, self.dim, self.vdim
        S, nrm, mx = cache
        proj = ops.linear(x, self.w_in, None)                                                  # [T, q | k | v | g]
        gates = ops.linear(x, self.w_gates, self.b_gates, out_dtype=torch.float32)             # [T, 2H] float32
        q, k, v, g = proj[:, :H * D], proj[:, H * D:2 * H * D], proj[:, 2 * H * D:2 * H * D + H * Dv], proj[:, 2 * H * D + H * Dv:]
        weights, n_before = ops.mlstm_gates(gates, mx.state, nrm.state, ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs, H, self.gate_cap)
        o = ops.mlstm_scan(q, k, v, weights, S.state, nrm.state, n_before, ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs,
                           H, D, Dv, D ** -0.5)
        y = ops.head_norm_gate(o, g, self.norm_w, H, Dv, self.eps, "sigmoid")
        return ops.linear(y, self.w_out, None, partial_ok=True)
