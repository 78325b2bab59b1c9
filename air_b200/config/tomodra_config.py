"""Typed configuration of the Tomodra decoder, read from config.json's own keys.

config.json names the design under "architecture" and gives "vocab", "width", "norm" {"eps"}, "postln_alpha" (what
the stream is multiplied by before a sub-layer's output is added and the sum normalised) and "layers": every entry
has a "type" ("latent_attention" or "attention"), the mixer's sizes and constants under "mixer" and its feed-forward
under "mlp" (null: none).  Every size and constant that may differ between two models of the design is read from
there; nothing has a default in code except keys that only some models have (a frequency scaling, a shared expert,
the layer whose latent a layer reads).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .bivizen_config import _get
from .model_config import ConfigError

MIXER_TYPES = ("latent_attention", "attention")
# No key of config.json bounds a request's length; the block tables need a width, and this is it.
POSITIONS = 1 << 20


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class TomodraMixture:
    """The feed-forward: `experts` gated experts of width `ff`, of which a token takes `top`; a shared expert of width
    shared_ff (0: none) beside them."""
    experts: int
    top: int
    ff: int
    shared_ff: int = 0


@dataclass(frozen=True)
class TomodraLayer:
    type: str
    heads: int
    dim: int                     # query/key size per head (latent attention: the part that is not rotated)
    vdim: int
    scale: float
    mask_size: int               # latent attention: the window; attention: the chunk
    rot_dims: int
    rot_base: float
    kv_heads: int = 0            # attention
    scaling: Optional[RotationScaling] = None      # attention
    rot_dim: int = 0             # latent attention: the rotated part of a head and of the shared key
    kv_rank: int = 0             # latent attention
    kv_from: Optional[int] = None                  # latent attention: the layer whose latent this one reads
    mlp: Optional[TomodraMixture] = None
    second_norm: bool = True     # a layer without feed-forward has a second norm only if the model file has its weight


@dataclass(frozen=True)
class TomodraConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    alpha: float
    layers: Tuple[TomodraLayer, ...]
    max_positions: int = POSITIONS
    eos_token_id: Optional[int] = None
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False)

    reads_shapes = True      # whether a layer without feed-forward has a second norm shows in the model file only

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes=None) -> "TomodraConfig":
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
            wm = where + ".mixer"
            rot = m.get("rot")
            if not isinstance(rot, Mapping):
                raise ConfigError("data_error", f"config.json lacks 'rot' in {wm}")
            kw = dict(type=kind, heads=_get(m, "heads", int, wm), dim=_get(m, "dim", int, wm),
                      vdim=_get(m, "vdim", int, wm), scale=_get(m, "scale", float, wm),
                      mask_size=_get(m.get("mask"), "size", int, wm + ".mask"),
                      rot_dims=_get(rot, "dims", int, wm + ".rot"), rot_base=_get(rot, "base", float, wm + ".rot"))
            if kind == "attention":
                kw.update(kv_heads=_get(m, "kv_heads", int, wm))
                sc = rot.get("scaling")
                if sc is not None:
                    ws = wm + ".rot.scaling"
                    kw["scaling"] = RotationScaling(*(_get(sc, k, float, ws) for k in ("factor", "original", "fast",
                                                                                       "slow")))
            else:
                kw.update(rot_dim=_get(m, "rot_dim", int, wm), kv_rank=_get(m, "kv_rank", int, wm))
                src = m.get("kv_from")
                if src is not None:
                    kw["kv_from"] = _get(m, "kv_from", int, wm)
            f = entry.get("mlp")
            if f is not None:
                wf = where + ".mlp"
                fkind = _get(f, "kind", str, wf)
                if fkind != "moe":
                    raise ConfigError("unsupported", f"{wf}: feed-forward kind {fkind!r} (known: moe)")
                shared = f.get("shared")
                kw["mlp"] = TomodraMixture(
                    experts=_get(f.get("router"), "experts", int, wf + ".router"),
                    top=_get(f.get("router"), "top", int, wf + ".router"),
                    ff=_get(f.get("expert"), "ff", int, wf + ".expert"),
                    shared_ff=_get(shared, "ff", int, wf + ".shared") if shared is not None else 0)
            elif shapes is not None:
                kw["second_norm"] = f"l{i}.norm2" in shapes
            else:
                kw["second_norm"] = bool(entry.get("second_norm", False))
            layers.append(TomodraLayer(**kw))
        eos = d.get("eos_token_id")
        cfg = cls(architecture=arch, vocab=_get(d, "vocab", int, "config.json"),
                  width=_get(d, "width", int, "config.json"), eps=_get(d.get("norm"), "eps", float, "norm"),
                  alpha=_get(d, "postln_alpha", float, "config.json"), layers=tuple(layers),
                  max_positions=_get(d, "max_positions", int, "config.json", POSITIONS, required=False),
                  eos_token_id=eos if isinstance(eos, int) else None, raw=dict(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale, "mask": {"size": l.mask_size},
                 "rot": {"dims": l.rot_dims, "base": l.rot_base}}
            if l.type == "attention":
                m["kv_heads"] = l.kv_heads
                if l.scaling is not None:
                    m["rot"]["scaling"] = l.scaling.to_dict()
            else:
                m.update(rot_dim=l.rot_dim, kv_rank=l.kv_rank)
                if l.kv_from is not None:
                    m["kv_from"] = l.kv_from
            f = None
            if l.mlp is not None:
                f = {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
                if l.mlp.shared_ff:
                    f["shared"] = {"ff": l.mlp.shared_ff}
            entry = {"type": l.type, "mixer": m, "mlp": f}
            if l.mlp is None and l.second_norm:
                entry["second_norm"] = True
            layers.append(entry)
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "postln_alpha": self.alpha, "layers": layers}
        if self.max_positions != POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("data_error", "Tomodra geometry is incomplete: vocab and width must be positive")
        if not (self.eps > 0.0):
            raise ConfigError("data_error", "Tomodra norm eps is missing or invalid")
        for i, l in enumerate(self.layers):
            if min(l.heads, l.dim, l.vdim, l.mask_size) <= 0:
                raise ConfigError("data_error", f"layers[{i}]: heads, dim, vdim and mask.size must be positive")
            if l.rot_dims % 2 or l.rot_dims < 0:
                raise ConfigError("data_error", f"layers[{i}]: rot.dims must be even")
            if l.type == "attention":
                if l.kv_heads <= 0 or l.heads % l.kv_heads:
                    raise ConfigError("data_error", f"layers[{i}]: heads must be a multiple of kv_heads")
                if l.rot_dims > l.dim:
                    raise ConfigError("data_error", f"layers[{i}]: rot.dims must be at most dim")
                if l.scaling is not None and not (l.scaling.factor > 0 and l.scaling.original > 0
                                                  and l.scaling.fast > 0 and l.scaling.slow > 0 and l.rot_base > 1):
                    raise ConfigError("data_error", f"layers[{i}]: rot.scaling needs positive numbers and a base above 1")
            else:
                if l.kv_rank <= 0 or l.rot_dim < 0 or l.rot_dims != l.rot_dim:
                    raise ConfigError("data_error", f"layers[{i}]: kv_rank must be positive and rot.dims equal rot_dim")
                if l.kv_from is not None:
                    j = l.kv_from
                    if not (0 <= j < i) or self.layers[j].type != "latent_attention" or self.layers[j].kv_from is not None:
                        raise ConfigError("data_error", f"layers[{i}]: kv_from must name an earlier latent_attention "
                                                        "layer that has a latent of its own")
                    o = self.layers[j]
                    if (o.kv_rank, o.rot_dim, o.rot_base) != (l.kv_rank, l.rot_dim, l.rot_base):
                        raise ConfigError("data_error", f"layers[{i}]: kv_rank, rot_dim and rot.base must equal those "
                                                        f"of layer {j}, whose latent it reads")
            f = l.mlp
            if f is not None and (f.experts <= 0 or not (0 < f.top <= f.experts) or f.ff <= 0 or f.shared_ff < 0):
                raise ConfigError("data_error", f"layers[{i}].mlp: experts, top (at most experts) and ff must be positive")
