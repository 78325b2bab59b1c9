"""Typed configuration of the Bivizen decoder, read from config.json's own keys.

config.json names the design under "architecture" and gives: "vocab", "width", "norm" {"eps"}, and "layers", a
list in which every entry has a "type" (which mixer the layer has: "attention", "delta" or "gla"), the mixer's
sizes and constants under "mixer", and its feed-forward under "mlp" (null: the layer has none).  Every size and
every constant that may differ between two models of the design is read from there; nothing has a default in code,
except keys that only some models have (a rotation, a soft cap, value mixing).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("attention", "delta", "gla")
# No key of config.json bounds a request's length; the block tables need a width, and this is it.
POSITIONS = 1 << 20


def _get(d: Mapping[str, Any], key: str, typ, where: str, default=None, required=True):
    if not isinstance(d, Mapping) or d.get(key) is None:
        if required:
            raise ConfigError("data_error", f"config.json lacks '{key}' in {where}")
        return default
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError("data_error", f"config.json '{key}' in {where} must be an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError("data_error", f"config.json '{key}' in {where} must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class BivizenFeedForward:
    kind: str
    ff: int
    limit: float


@dataclass(frozen=True)
class BivizenLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0            # attention, delta
    scale: float = 0.0           # attention
    softcap: float = 0.0         # attention (0: none)
    rot_dims: int = 0            # attention (0: no rotation)
    rot_base: float = 1.0
    v_mix: bool = False          # attention
    conv: int = 0                # delta
    tau: float = 0.0             # gla
    rank: int = 0                # gla: the narrow middle of the decay's projection
    mlp: Optional[BivizenFeedForward] = None


@dataclass(frozen=True)
class BivizenConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[BivizenLayer, ...]
    max_positions: int = POSITIONS
    eos_token_id: Optional[int] = None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # Sizes that config.json does not give are taken from the shapes of the model file's tensors: load_config hands
    # them to from_dict when it reads a folder.
    reads_shapes = True

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "BivizenConfig":
        arch = d.get("architecture") or (d.get("architectures") or [None])[0]
        if arch is None:
            raise ConfigError("data_error", "config.json lacks 'architecture'")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("data_error", "config.json lacks 'layers'")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            if kind not in MIXER_TYPES:
                raise ConfigError("unsupported", f"{where}: mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError("data_error", f"config.json lacks 'mixer' in {where}")
            where_m = where + ".mixer"
            kw = dict(type=kind, heads=_get(m, "heads", int, where_m), dim=_get(m, "dim", int, where_m),
                      vdim=_get(m, "vdim", int, where_m))
            if kind == "attention":
                rot = m.get("rot") or {}
                kw.update(kv_heads=_get(m, "kv_heads", int, where_m), scale=_get(m, "scale", float, where_m),
                          softcap=_get(m, "softcap", float, where_m, 0.0, required=False),
                          rot_dims=_get(rot, "dims", int, where_m + ".rot", 0, required=False),
                          rot_base=_get(rot, "base", float, where_m + ".rot", 1.0, required=bool(rot)),
                          v_mix=bool(m.get("v_mix", False)))
            elif kind == "delta":
                kw.update(kv_heads=_get(m, "kv_heads", int, where_m), conv=_get(m, "conv", int, where_m))
            else:
                rank = _get(m, "rank", int, where_m, 0, required=False)
                if not rank and shapes is not None and f"l{i}.mix.a1" in shapes:
                    rank = int(shapes[f"l{i}.mix.a1"][0])
                if rank <= 0:
                    raise ConfigError("data_error", f"{where_m}: the rank of the decay's projection is neither under "
                                                    f"'rank' nor given by the shape of a tensor l{i}.mix.a1")
                kw.update(tau=_get(m, "tau", float, where_m), rank=rank)
            f = entry.get("mlp")
            if f is not None:
                where_f = where + ".mlp"
                fkind = _get(f, "kind", str, where_f)
                if fkind != "dense":
                    raise ConfigError("unsupported", f"{where_f}: feed-forward kind {fkind!r} (known: dense)")
                kw["mlp"] = BivizenFeedForward(fkind, _get(f, "ff", int, where_f), _get(f, "limit", float, where_f))
            layers.append(BivizenLayer(**kw))
        eos = d.get("eos_token_id")
        cfg = cls(architecture=arch, vocab=_get(d, "vocab", int, "config.json"),
                  width=_get(d, "width", int, "config.json"),
                  eps=_get(d.get("norm"), "eps", float, "norm"), layers=tuple(layers),
                  max_positions=_get(d, "max_positions", int, "config.json", POSITIONS, required=False),
                  eos_token_id=eos if isinstance(eos, int) else None, raw=dict(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
            if l.type == "attention":
                m.update(kv_heads=l.kv_heads, scale=l.scale, softcap=l.softcap, v_mix=l.v_mix)
                if l.rot_dims:
                    m["rot"] = {"dims": l.rot_dims, "base": l.rot_base}
            elif l.type == "delta":
                m.update(kv_heads=l.kv_heads, conv=l.conv)
            else:
                m.update(tau=l.tau, rank=l.rank)
            layers.append({"type": l.type, "mixer": m,
                           "mlp": None if l.mlp is None else {"kind": l.mlp.kind, "ff": l.mlp.ff, "limit": l.mlp.limit}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": layers}
        if self.max_positions != POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("data_error", "Bivizen geometry is incomplete: vocab and width must be positive")
        if not (self.eps > 0.0):
            raise ConfigError("data_error", "Bivizen norm eps is missing or invalid")
        for i, l in enumerate(self.layers):
            if min(l.heads, l.dim, l.vdim) <= 0:
                raise ConfigError("data_error", f"layers[{i}]: heads, dim and vdim must be positive")
            if l.type in ("attention", "delta") and (l.kv_heads <= 0 or l.heads % l.kv_heads):
                raise ConfigError("data_error", f"layers[{i}]: heads must be a multiple of kv_heads")
            if l.type == "attention" and (l.rot_dims % 2 or l.rot_dims > l.dim or l.rot_dims < 0):
                raise ConfigError("data_error", f"layers[{i}]: rot.dims must be even and at most dim")
            if l.type == "delta" and l.conv < 1:
                raise ConfigError("data_error", f"layers[{i}]: conv must be at least 1")
            if l.type == "gla" and not (l.tau > 0.0):
                raise ConfigError("data_error", f"layers[{i}]: tau must be positive")
            if l.mlp is not None and (l.mlp.ff <= 0 or not (l.mlp.limit > 0.0)):
                raise ConfigError("data_error", f"layers[{i}].mlp: ff and limit must be positive")
