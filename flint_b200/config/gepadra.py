"""Typed configuration of Gepadra, read from the keys of its own config.json.

The file is nested: ``vocab``, ``width``, ``norm`` (eps) and ``layers``, a list with one entry per layer that
gives the mixer's ``type`` (``attention`` or ``mlstm``), the mixer's sizes and constants (``mixer``) and the
feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).  Nothing is assumed about the number or
the order of the layers, and every size and constant comes from the file.  The design gives no limit on
positions; ``DEFAULT_MAX_POSITIONS`` bounds what an engine may be built for.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from . import fields as F
from .puledra import _section

DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class SinkAttention:
    heads: int
    kv_heads: int
    dim: int                # query/key dims per head
    vdim: int               # value dims per head
    scale: float
    window: int             # 0: every earlier key is seen
    keep_first: int         # the first tokens of a sequence that stay visible behind the window
    rot_dims: int           # leading dims of every head that rotate (0: none)
    rot_base: float
    v_mix: bool             # values are blended with those of the first such layer


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float


@dataclass(frozen=True)
class ExpertMlp:
    ff: int
    experts: int
    top: int
    shared_ff: int          # 0: no shared expert


@dataclass(frozen=True)
class GepadraLayer:
    type: str
    mixer: object
    mlp: object


def _attention(m, where):
    heads, kv = F.get_int(m, "heads", minimum=1), F.get_int(m, "kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = F.get_int(m, "dim", minimum=1)
    rot = _section(m, "rot", optional=True)
    rot_dims = F.get_int(rot, "dims", 0, minimum=0) if rot is not None else 0
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}.rot.dims must be even and at most dim {dim}, got {rot_dims}")
    mask = _section(m, "mask", optional=True)
    window = F.get_int(mask, "size", 0, minimum=0) if mask is not None else 0
    keep = F.get_int(mask, "keep_first", 0, minimum=0) if mask is not None else 0
    return SinkAttention(heads=heads, kv_heads=kv, dim=dim, vdim=F.get_int(m, "vdim", minimum=1),
                         scale=F.get_float(m, "scale"), window=window, keep_first=keep if window else 0,
                         rot_dims=rot_dims, rot_base=F.get_float(rot, "base") if rot_dims else 1.0,
                         v_mix=F.get_bool(m, "v_mix", False))


def _mlp(f, where):
    kind = F.get_str(f, "kind")
    if kind == "dense":
        return DenseMlp(ff=F.get_int(f, "ff", minimum=1), limit=F.get_float(f, "limit"))
    if kind == "moe":
        r = _section(f, "router")
        shared = _section(f, "shared", optional=True)
        out = ExpertMlp(ff=F.get_int(_section(f, "expert"), "ff", minimum=1), experts=F.get_int(r, "experts", minimum=1),
                        top=F.get_int(r, "top", minimum=1), shared_ff=F.get_int(shared, "ff", minimum=1) if shared else 0)
        if out.top > out.experts:
            raise ConfigError(f"{where}.router.top {out.top} exceeds the {out.experts} experts")
        return out
    raise ConfigError(f"{where}: unknown kind {kind!r} (known: dense, moe)")


@dataclass(frozen=True)
class GepadraConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    architecture: str = "Gepadra"

    @classmethod
    def from_dict(cls, d: dict) -> "GepadraConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty list")
        out = []
        mix_width = None
        for i, entry in enumerate(layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = F.get_str(entry, "type")
            m = _section(entry, "mixer")
            if kind == "attention":
                mixer = _attention(m, f"layers[{i}].mixer")
                if mixer.v_mix:
                    if mix_width is not None and mix_width != (mixer.kv_heads, mixer.vdim):
                        raise ConfigError(f"layers[{i}].mixer: layers that blend values must agree in kv_heads and vdim")
                    mix_width = (mixer.kv_heads, mixer.vdim)
            elif kind == "mlstm":
                mixer = MatrixMemory(heads=F.get_int(m, "heads", minimum=1), dim=F.get_int(m, "dim", minimum=1),
                                     vdim=F.get_int(m, "vdim", minimum=1), gate_cap=F.get_float(m, "gate_cap"))
                if mixer.gate_cap <= 0:
                    raise ConfigError(f"layers[{i}].mixer.gate_cap must be positive, got {mixer.gate_cap}")
            else:
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (known: attention, mlstm)")
            f = _section(entry, "mlp", optional=True)
            out.append(GepadraLayer(kind, mixer, _mlp(f, f"layers[{i}].mlp") if f is not None else None))
        return cls(vocab=F.get_int(d, "vocab", minimum=1), width=F.get_int(d, "width", minimum=1),
                   eps=F.get_float(_section(d, "norm"), "eps"), layers=tuple(out))
