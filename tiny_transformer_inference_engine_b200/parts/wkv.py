"""RWKV-style time mixing with a decay that depends on the token (a matrix state per head).

With ``h`` the mixer's input and ``h'`` the previous token's input (zeros before a sequence's first token), each of the five
branches r, k, v, g, w reads its own mix ``h + (h' - h) * mu_s``.  ``r, k, v`` are projections of their mixes into
``heads x dim``; the gate is ``silu(W_g mix_g)``; the decay is ``w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))`` per head and key
channel (a low-rank path of width ``W_w1.shape[0]``).  Per head, with the state S [dim x dim] starting at zero,

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          S_t = diag(w_t) S_(t-1) + k_t v_t^T

(the bonus ``u`` acts on the current token only).  Each head's ``o`` is divided by its root mean square
(``x / sqrt(mean(x^2) + eps)``), the heads are concatenated, multiplied by ``norm`` and by the gate, and projected by ``W_o``.

Per request two state rows, both 32-bit: S as ``[heads, dim, padded dim]`` (value column major, see the scan kernel) and
the last token's ``h``; a sequence may therefore be cut into steps anywhere.  Decay, exponentials, state and read-out
are 32-bit in every run; the four equal-shaped projections are one batched product.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Mixer, ParamSpec, FixedStateNeed, StepContext
from ..registry import register_part

MAX_KEYS = 512                  # key channels per head the scan kernels take (csrc/matrix_memory.cu)


def padded_keys(dim: int) -> int:
    """Key channels of a matrix-state row as the scan kernels lay it out: a power-of-two number of slices of 4 channels
    (heads of up to 128 key channels), 8 (up to 256) or 16."""
    per_thread = 4 if dim <= 128 else 8 if dim <= 256 else 16
    slices = 1
    while slices * per_thread < dim:
        slices *= 2
    return slices * per_thread


@register_part("mixer", "wkv")
class WKV(Mixer):
    BRANCHES = ("r", "k", "v", "g", "w")

    def __init__(self, prefix: str, d_model: int, num_heads: int, dim: int, eps: float, decay_rank: Optional[int] = None,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(prefix)
        self.d_model, self.num_heads, self.dim, self.eps = int(d_model), int(num_heads), int(dim), float(eps)
        self.decay_rank = -1 if decay_rank is None else int(decay_rank)      # -1: the width of the decay's low-rank path is the weight file's
        if self.dim > MAX_KEYS:
            raise ValueError(f"wkv: {dim} key channels per head (at most {MAX_KEYS})")
        self.names = {"mu": "mu", "r": "r", "k": "k", "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u",
                      "norm": "norm", "o": "o"}
        if names:
            self.names.update(names)

    def param_specs(self):
        n, d, HD = self.names, self.d_model, self.num_heads * self.dim
        specs = {f"{n['mu']}.{s}": ParamSpec((d,), storage="vector", init="normal", std=0.3) for s in self.BRANCHES}
        for s in ("r", "k", "v", "g"):
            specs[n[s]] = ParamSpec((HD, d))
        specs.update({n["w1"]: ParamSpec((self.decay_rank, d)), n["w2"]: ParamSpec((HD, self.decay_rank)),
                      n["w0"]: ParamSpec((HD,), storage="vector", init="normal", std=0.5),
                      n["u"]: ParamSpec((self.num_heads, self.dim), storage="vector", init="normal", std=0.5),
                      n["norm"]: ParamSpec((HD,), storage="vector", init="ones"), n["o"]: ParamSpec((d, HD))})
        return specs

    def load(self, params):
        n = self.names
        self.mu = torch.stack([params[f"{n['mu']}.{s}"].float() for s in self.BRANCHES]).contiguous()     # [5, d] in branch order
        self.w_rkvg = torch.stack([params[n[s]] for s in ("r", "k", "v", "g")]).contiguous()              # [4, H*dim, d]
        self.w1, self.w2 = params[n["w1"]].contiguous(), params[n["w2"]].contiguous()
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"{self.prefix}: the decay's two matrices disagree on the width between them "
                             f"({self.w1.shape[0]} and {self.w2.shape[1]})")
        self.w0 = params[n["w0"]].float().contiguous()
        self.u = params[n["u"]].float().reshape(-1).contiguous()
        self.norm_w = params[n["norm"]].float().contiguous()
        self.w_out = params[n["o"]].contiguous()

    def product_weights(self):
        return [self.w_out]

    def cache_needs(self):
        return [FixedStateNeed((self.num_heads, self.dim, padded_keys(self.dim)), "float32"),
                FixedStateNeed((self.d_model,), "float32")]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        ops, H, D = self.ops, self.num_heads, self.dim
        S, prev = cache
        mixes = ops.token_shift_mix(x, self.mu, prev.state, ctx.token_seq, ctx.query_start_loc, ctx.slot_ids)      # [5, T, d]
        rkvg = ops.batched_linear(mixes[:4], self.w_rkvg)                                                         # [4, T, H*dim]
        lora = ops.activation(ops.linear(mixes[4], self.w1, None, out_dtype=torch.float32), "tanh", out_dtype=x.dtype)
        wlog = ops.linear(lora, self.w2, None, out_dtype=torch.float32)                                           # [T, H*dim] float32
        o = ops.wkv_scan(rkvg[0], rkvg[1], rkvg[2], ops.wkv_decay(wlog, self.w0), self.u, S.state, x, prev.state,
                         ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs, H, D)
        y = ops.head_norm_gate(o, rkvg[3], self.norm_w, H, D, self.eps, "silu")
        return ops.linear(y, self.w_out, None, partial_ok=True)
