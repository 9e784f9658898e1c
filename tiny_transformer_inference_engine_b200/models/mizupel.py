"""The Mizupel design as data: a pre-norm decoder that mixes windowed attention with two kinds of matrix-state recurrence.

Token embedding; pre-norm layers (``x += mixer(rms_norm(x))`` and, where the layer has one, ``x += ff(rms_norm(x))``); the
model's RMS norm; logits from an untied head, soft-capped.  The mixer of a layer is

* ``attention``: grouped-query attention with biases on q, k and v, a short causal convolution over time on their channels,
  a rotation of the first ``rot.dims`` values of every head (pairs ``(i, i + dims/2)``, frequencies optionally rescaled by
  wavelength), soft-capped scores, a sliding window, one output gate per head, a value size of its own;
* ``wkv``: RWKV-style time mixing with a token-dependent decay (``parts/wkv.py``);
* ``mlstm``: xLSTM's matrix memory (``parts/mlstm.py``).

The feed-forward is ``W_down relu(W_up h)^2`` or absent.  A layer entry with ``weights_of: j`` owns no tensors: its run entry
runs layer j's parts again with a cache or state of its own.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.up`` / ``.down``, ``final.norm``, ``head``.

Constants the design fixes (not in config.json): the feed-forward's activation, the pairing of rotated values, the mLSTM
denominator's floor (in its part), silu / sigmoid as the recurrent mixers' gates.
"""
from __future__ import annotations

from ..config.mizupel_config import MizupelConfig
from ..parts.base import PartSpec, LayerSpec, RunEntry, ModelSpec
from ..registry import register_model

FF_ACTIVATION = "relu2"
ROTARY_STYLE = "half"


def _norm(prefix: str, name: str, d: int, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", prefix, {"dim": d, "eps": eps, "name": name})


def _mixer(L: dict, p: str, d: int, eps: float) -> PartSpec:
    m = L["mixer"]
    if L["type"] == "attention":
        rot = m.get("rot")
        if rot is not None and rot["dims"] > 0:
            position = PartSpec("rope", "", {"dim": rot["dims"], "base": rot["base"], "style": ROTARY_STYLE,
                                             "scaling": rot.get("scaling")})
        else:
            position = PartSpec("none", "", {})
        mask = m.get("mask")
        return PartSpec("attention", f"{p}.mix", {
            "d_model": d, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
            "v_head_dim": m.get("vdim", m["dim"]),
            "position": position, "window": None if mask is None else mask["size"], "scale": m["scale"],
            "softcap": m.get("softcap"), "conv_taps": m.get("conv"), "gated": True, "qkv_bias": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}, "weight_suffix": "", "bias_suffix": ".b",
            "conv_suffix": ".conv"})
    if L["type"] == "wkv":
        return PartSpec("wkv", f"{p}.mix", {"d_model": d, "num_heads": m["heads"], "dim": m["dim"], "eps": eps,
                                            "decay_rank": m.get("decay_rank")})
    return PartSpec("mlstm", f"{p}.mix", {"d_model": d, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                          "gate_cap": m["gate_cap"], "eps": eps})


@register_model("Mizupel")
def mizupel(config: MizupelConfig) -> ModelSpec:
    d, eps = config.width, config.norm_eps
    layers, run_order, index_of = [], [], {}
    for i, L in enumerate(config.layers):                            # layers that own tensors, under their own names l<i>
        if L.get("weights_of") is not None:
            continue
        p, f = f"l{i}", L.get("mlp")
        ffn = None if f is None else PartSpec("mlp", f"{p}.mlp", {"d_model": d, "hidden": f["ff"], "act": FF_ACTIVATION})
        block = PartSpec("pre_norm", p, {
            "mixer_norm": _norm(p, "norm1", d, eps), "mixer": _mixer(L, p, d, eps),
            "ffn_norm": None if ffn is None else _norm(p, "norm2", d, eps), "ffn": ffn})
        index_of[i] = len(layers)
        layers.append(LayerSpec(block))
    for i, L in enumerate(config.layers):                            # every entry runs once, in the file's order
        j = L.get("weights_of")
        run_order.append(RunEntry(index_of[i if j is None else j]))
    return ModelSpec(
        d_model=d, vocab_size=config.vocab, max_seq_len=config.max_seq_len,
        embedding=PartSpec("token", "", {"vocab_size": config.vocab, "dim": d, "name": "embed"}),
        layers=tuple(layers), run_order=tuple(run_order),
        final_norm=_norm("final", "norm", d, eps),
        head=PartSpec("linear", "", {"dim": d, "vocab_size": config.vocab, "name": "head", "softcap": config.logit_softcap}),
        eos_token_id=config.eos_token_id,
    )
