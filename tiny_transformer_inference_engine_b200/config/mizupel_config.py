"""Configuration of the Mizupel design: a pre-norm decoder whose layers are listed one by one.

config.json keys: ``architecture`` ("Mizupel"), ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (optional or null:
none) and ``layers``, a list with one entry per layer: ``type`` (the mixer: ``attention``, ``wkv`` or ``mlstm``), ``mixer``
(its sizes and constants), ``mlp`` (``kind`` ``dense`` with ``ff``, or null / absent for a layer without a feed-forward) and
optionally ``weights_of``: j, a layer that owns no tensors and runs layer j's (mixer, feed-forward and norms) with a cache or
state of its own; such an entry is of layer j's type and layer j's sizes and constants are the ones that run.  Every size and every constant that can differ between
models is read from there; nothing has a default in code.  The design names no longest sequence; ``max_seq_len`` is this
engine's own bound on positions (an optional key, else ``DEFAULT_MAX_SEQ_LEN``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .model_config import ConfigError, register_config
from .munevik_config import _need, _pos_int, DEFAULT_MAX_SEQ_LEN

MIXERS = ("attention", "wkv", "mlstm")
MLPS = ("dense",)


def _pos_num(v, where: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"{where} must be a positive number, got {v!r}")
    return float(v)


@register_config("Mizupel")
@dataclass(frozen=True)
class MizupelConfig:
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    logit_softcap: Optional[float] = None
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    eos_token_id: Optional[int] = None
    architecture: str = "Mizupel"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self):
        _pos_int(self.vocab, "vocab"); _pos_int(self.width, "width"); _pos_int(self.max_seq_len, "max_seq_len")
        if self.logit_softcap is not None:
            _pos_num(self.logit_softcap, "logit_softcap")
        if not self.layers:
            raise ConfigError("'layers' must list at least one layer")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(L, ("type", "mixer"), where)
            m = L["mixer"]
            if L["type"] == "attention":
                _need(m, ("heads", "dim", "scale"), f"{where}.mixer")          # (kv_heads absent: one per head; vdim absent: dim)
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if k in m:
                        _pos_int(m[k], f"{where}.mixer.{k}")
                if m["heads"] % m.get("kv_heads", m["heads"]):
                    raise ConfigError(f"{where}.mixer: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
                _pos_num(m["scale"], f"{where}.mixer.scale")
                if m.get("conv") is not None:
                    _pos_int(m["conv"], f"{where}.mixer.conv")
                if m.get("softcap") is not None:
                    _pos_num(m["softcap"], f"{where}.mixer.softcap")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), f"{where}.mixer.mask")
                    _pos_int(m["mask"]["size"], f"{where}.mixer.mask.size")
                if m.get("rot") is not None:
                    _need(m["rot"], ("base", "dims"), f"{where}.mixer.rot")
                    dims = m["rot"]["dims"]
                    if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims={dims!r} must be even and at most dim={m['dim']}")
                    _pos_num(m["rot"]["base"], f"{where}.mixer.rot.base")
                    sc = m["rot"].get("scaling")
                    if sc is not None:
                        _need(sc, ("factor", "low", "high", "original"), f"{where}.mixer.rot.scaling")
                        for k in ("factor", "low", "high", "original"):
                            _pos_num(sc[k], f"{where}.mixer.rot.scaling.{k}")
                        if not sc["high"] > sc["low"]:
                            raise ConfigError(f"{where}.mixer.rot.scaling: high must exceed low")
            elif L["type"] == "wkv":
                _need(m, ("heads", "dim"), f"{where}.mixer")
                for k in ("heads", "dim"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                if m.get("decay_rank") is not None:
                    _pos_int(m["decay_rank"], f"{where}.mixer.decay_rank")
            elif L["type"] == "mlstm":
                _need(m, ("heads", "dim", "vdim", "gate_cap"), f"{where}.mixer")
                for k in ("heads", "dim", "vdim"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                _pos_num(m["gate_cap"], f"{where}.mixer.gate_cap")
            else:
                raise ConfigError(f"{where}.type {L['type']!r} unknown; known: {MIXERS}")
            f = L.get("mlp")
            if f is not None:
                _need(f, ("kind",), f"{where}.mlp")
                if f["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp.kind {f['kind']!r} unknown; known: {MLPS}")
                _need(f, ("ff",), f"{where}.mlp")
                _pos_int(f["ff"], f"{where}.mlp.ff")
            j = L.get("weights_of")
            if j is not None:
                if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(self.layers) or j == i:
                    raise ConfigError(f"{where}.weights_of={j!r} must name another layer")
                o = self.layers[j]
                if o.get("weights_of") is not None:
                    raise ConfigError(f"{where}.weights_of={j}: that layer owns no tensors itself")
                if o["type"] != L["type"]:
                    raise ConfigError(f"{where}: an entry with weights_of must have layer {j}'s type")

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def d_model(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MizupelConfig":
        raw = dict(raw)
        _need(raw, ("vocab", "width", "layers", "norm"), "config.json")
        _need(raw["norm"], ("eps",), "config.json 'norm'")
        raw.pop("architecture", None)
        kw = dict(vocab=raw.pop("vocab"), width=raw.pop("width"), layers=tuple(raw.pop("layers")),
                  norm_eps=float(raw.pop("norm")["eps"]), logit_softcap=raw.pop("logit_softcap", None))
        if "max_seq_len" in raw:
            kw["max_seq_len"] = raw.pop("max_seq_len")
        if "eos_token_id" in raw:
            kw["eos_token_id"] = raw.pop("eos_token_id")
        return cls(extra=raw, **kw)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": list(self.layers),
             "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap}
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
