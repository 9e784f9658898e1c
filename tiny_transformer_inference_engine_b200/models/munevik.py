"""The Munevik design as data: a post-norm decoder of latent-attention and recurrent layers.

Token embedding; post-norm layers (``x = LN(alpha * x + sublayer(x))`` for the mixer and, where the layer has one, for the
feed-forward; LayerNorm with weight and bias); the model's LayerNorm; logits from the embedding table.
The mixer is latent attention (sliding window, gated heads, rotated key part shared by all heads; a layer may read an
earlier layer's latent cache instead of keeping one) or the RG-LRU recurrent block; the feed-forward is a clamped gated
linear unit or a grouped top-k mixture of SwiGLU experts with a shared expert.  Tensor names: ``embed``,
``l<i>.norm1``/``.b``, ``l<i>.norm2``/``.b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``/``.b``.

Constants the design fixes (not in config.json): the recurrence's decay factor 8, the dense unit's ``sigmoid(1.702 g)``
and ``u + 1``, a group's score from its two best experts, expert weights not renormalised.
"""
from __future__ import annotations

from ..config.munevik_config import MunevikConfig
from ..parts.base import PartSpec, LayerSpec, RunEntry, ModelSpec
from ..registry import register_model

RGLRU_DECAY = 8.0
DENSE_ALPHA, DENSE_SHIFT = 1.702, 1.0
GROUP_TOP = 2


def _norm(prefix: str, name: str, d: int, eps: float) -> PartSpec:
    return PartSpec("layernorm", prefix, {"dim": d, "eps": eps, "names": {"weight": name, "bias": f"{name}.b"}})


@register_model("Munevik")
def munevik(config: MunevikConfig) -> ModelSpec:
    d, eps = config.width, config.norm_eps
    layers, run_order = [], []
    # a latent cache is read by its own layer and by the layers that name it: its pages must outlast the widest window
    widest = {}
    for i, L in enumerate(config.layers):
        if L["type"] == "latent_attention":
            owner = L["mixer"].get("kv_from")
            owner = i if owner is None else owner
            widest[owner] = max(widest.get(owner, 0), L["mixer"]["mask"]["size"])
    for i, L in enumerate(config.layers):
        p, m = f"l{i}", L["mixer"]
        cache_from = None
        if L["type"] == "latent_attention":
            owner = m.get("kv_from")
            cache_from = owner
            mixer = PartSpec("latent_attention", f"{p}.mix", {
                "d_model": d, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "window": m["mask"]["size"],
                "cache_window": widest[i if owner is None else owner], "shares_kv": owner is not None, "gated": True,
                "position": PartSpec("rope", "", {"dim": m["rot"]["dims"], "base": m["rot"]["base"], "style": "interleaved"})})
        else:
            mixer = PartSpec("rglru", f"{p}.mix", {"d_model": d, "width": m["width"], "blocks": m["blocks"], "taps": m["conv"],
                                                   "decay": RGLRU_DECAY})
        f = L.get("mlp")
        if f is None:
            ffn = None
        elif f["kind"] == "dense":
            ffn = PartSpec("glu", f"{p}.mlp", {"d_model": d, "hidden": f["ff"], "alpha": DENSE_ALPHA, "limit": f["limit"],
                                               "shift": DENSE_SHIFT})
        else:
            r = f["router"]
            shared = f.get("shared")
            ffn = PartSpec("grouped_moe", f"{p}.mlp", {
                "d_model": d, "hidden": f["expert"]["ff"], "experts": r["experts"], "top": r["top"],
                "groups": r["groups"]["count"], "keep": r["groups"]["keep"], "group_top": GROUP_TOP, "scale": r["scale"],
                "renorm": False,
                "shared": None if shared is None else PartSpec("glu", f"{p}.mlp.shared", {"d_model": d, "hidden": shared["ff"]})})
        block = PartSpec("post_norm", p, {
            "alpha": config.postln_alpha, "mixer": mixer, "mixer_norm": _norm(p, "norm1", d, eps),
            "ffn": ffn, "ffn_norm": None if ffn is None else _norm(p, "norm2", d, eps)})
        layers.append(LayerSpec(block))
        run_order.append(RunEntry(i, cache_from))
    return ModelSpec(
        d_model=d, vocab_size=config.vocab, max_seq_len=config.max_seq_len,
        embedding=PartSpec("token", "", {"vocab_size": config.vocab, "dim": d, "name": "embed"}),
        layers=tuple(layers), run_order=tuple(run_order),
        final_norm=_norm("final", "norm", d, eps),
        head=PartSpec("tied", "", {"dim": d, "vocab_size": config.vocab}),
        eos_token_id=config.eos_token_id,
    )
