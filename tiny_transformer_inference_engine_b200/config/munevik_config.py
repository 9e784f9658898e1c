"""Configuration of the Munevik design: a post-norm decoder whose layers are listed one by one.

config.json keys: ``architecture`` ("Munevik"), ``vocab``, ``width``, ``norm.eps``, ``postln_alpha`` and ``layers``, a list
with one entry per layer: ``type`` (the mixer: ``latent_attention`` or ``rglru``), ``mixer`` (its sizes and constants) and
``mlp`` (``kind`` ``dense`` or ``moe`` with its sizes, or null for a layer without a feed-forward).  Every size and every
constant that can differ between models is read from there; nothing has a default in code.  The design names no longest
sequence; ``max_seq_len`` is this engine's own bound on positions (an optional key, else ``DEFAULT_MAX_SEQ_LEN``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, register_config

DEFAULT_MAX_SEQ_LEN = 131072
MIXERS = ("latent_attention", "rglru")
MLPS = ("dense", "moe")


def _need(d: dict, keys, where: str):
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{where} lacks key(s) {missing}")


def _pos_int(v, where: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{where} must be a positive integer, got {v!r}")
    return v


@register_config("Munevik")
@dataclass(frozen=True)
class MunevikConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    postln_alpha: float
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    eos_token_id: Optional[int] = None
    architecture: str = "Munevik"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self):
        _pos_int(self.vocab, "vocab"); _pos_int(self.width, "width"); _pos_int(self.max_seq_len, "max_seq_len")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(L, ("type", "mixer"), where)                       # ("mlp" absent reads like null: no feed-forward)
            m = L["mixer"]
            if L["type"] == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask", "rot"), f"{where}.mixer")
                _need(m["mask"], ("size",), f"{where}.mixer.mask")
                _need(m["rot"], ("base", "dims"), f"{where}.mixer.rot")
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                _pos_int(m["mask"]["size"], f"{where}.mixer.mask.size")
                if m["rot"]["dims"] != m["rot_dim"]:
                    raise ConfigError(f"{where}.mixer: rot.dims={m['rot']['dims']} differs from rot_dim={m['rot_dim']} "
                                      "(the whole rotated part is rotated in this design)")
                if m["rot_dim"] % 2:
                    raise ConfigError(f"{where}.mixer.rot_dim must be even")
                j = m.get("kv_from")
                if j is not None:
                    if not isinstance(j, int) or not 0 <= j < i:
                        raise ConfigError(f"{where}.mixer.kv_from={j!r} must name an earlier layer")
                    o = self.layers[j]
                    if o["type"] != "latent_attention" or o["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from={j}: that layer keeps no latent cache of its own")
                    om = o["mixer"]
                    if (om["kv_rank"], om["rot_dim"], om["rot"]["base"], om["rot"]["dims"]) != \
                            (m["kv_rank"], m["rot_dim"], m["rot"]["base"], m["rot"]["dims"]):
                        raise ConfigError(f"{where}.mixer: kv_rank, rot_dim and rot must equal those of layer {j}")
            elif L["type"] == "rglru":
                _need(m, ("width", "blocks", "conv"), f"{where}.mixer")
                for k in ("width", "blocks", "conv"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                if m["width"] % m["blocks"]:
                    raise ConfigError(f"{where}.mixer: width {m['width']} is not a multiple of {m['blocks']} blocks")
            else:
                raise ConfigError(f"{where}.type {L['type']!r} unknown; known: {MIXERS}")
            f = L.get("mlp")
            if f is None:
                continue
            _need(f, ("kind",), f"{where}.mlp")
            if f["kind"] == "dense":
                _need(f, ("ff", "limit"), f"{where}.mlp")
                _pos_int(f["ff"], f"{where}.mlp.ff")
            elif f["kind"] == "moe":
                _need(f, ("expert", "router"), f"{where}.mlp")
                _need(f["expert"], ("ff",), f"{where}.mlp.expert")
                r = f["router"]
                _need(r, ("experts", "top", "groups", "scale"), f"{where}.mlp.router")
                _need(r["groups"], ("count", "keep"), f"{where}.mlp.router.groups")
                if r["experts"] % r["groups"]["count"]:
                    raise ConfigError(f"{where}.mlp.router: {r['experts']} experts do not form {r['groups']['count']} equal groups")
                if f.get("shared") is not None:
                    _need(f["shared"], ("ff",), f"{where}.mlp.shared")
            else:
                raise ConfigError(f"{where}.mlp.kind {f['kind']!r} unknown; known: {MLPS}")

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def d_model(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MunevikConfig":
        raw = dict(raw)
        _need(raw, ("vocab", "width", "layers", "norm", "postln_alpha"), "config.json")
        _need(raw["norm"], ("eps",), "config.json 'norm'")
        raw.pop("architecture", None)
        kw = dict(vocab=raw.pop("vocab"), width=raw.pop("width"), layers=tuple(raw.pop("layers")),
                  norm_eps=float(raw.pop("norm")["eps"]), postln_alpha=float(raw.pop("postln_alpha")))
        if "max_seq_len" in raw:
            kw["max_seq_len"] = raw.pop("max_seq_len")
        if "eos_token_id" in raw:
            kw["eos_token_id"] = raw.pop("eos_token_id")
        return cls(extra=raw, **kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": list(self.layers),
             "norm": {"eps": self.norm_eps}, "postln_alpha": self.postln_alpha}
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            d["max_seq_len"] = self.max_seq_len
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        d.update({k: v for k, v in self.extra.items() if k not in d})
        return d

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
        return path
