"""Typed configuration of Puledra, read from the keys of its own config.json.

Puledra's config.json is nested: ``embedding`` (scale and the hashed pair table), ``norm`` (eps), and
``layers``, a list with one entry per layer giving the mixer's type and sizes and the feed-forward (or null).
Nothing is assumed about the order or number of layers, and every size comes from the file.  The design
gives no limit on positions; ``DEFAULT_MAX_POSITIONS`` bounds what an engine may be built for.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from . import fields as F

DEFAULT_MAX_POSITIONS = 1 << 20


def _section(d, key, optional=False):
    v = d.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"missing config section {key!r}")
    if not isinstance(v, dict):
        raise ConfigError(f"config section {key!r} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int                # unrotated query/key dims per head
    rot_dim: int            # rotated query/key dims per head
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int           # how many of the rot_dim dims rotate
    kv_from: int | None     # the layer whose cached latent this one reads, or None


@dataclass(frozen=True)
class MoE:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    scale: float


@dataclass(frozen=True)
class PuledraLayer:
    type: str
    mixer: LatentMixer
    mlp: MoE | None


@dataclass(frozen=True)
class PuledraConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    pair_table: PairTable | None
    layers: tuple
    architecture: str = "Puledra"

    @classmethod
    def from_dict(cls, d: dict) -> "PuledraConfig":
        emb = _section(d, "embedding")
        pt = _section(emb, "bigram", optional=True)
        pair = None
        if pt is not None:
            pair = PairTable(F.get_int(pt, "buckets", minimum=1), F.get_int(pt, "mul_prev", minimum=0),
                             F.get_int(pt, "mul_cur", minimum=0))
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            if not isinstance(entry, dict):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = F.get_str(entry, "type")
            if kind != "latent_attention":
                raise ConfigError(f"layers[{i}]: unknown layer type {kind!r} (known: latent_attention)")
            m = _section(entry, "mixer")
            rot = _section(m, "rot")
            rot_dim = F.get_int(m, "rot_dim", minimum=0)
            rot_dims = F.get_int(rot, "dims", minimum=0)
            if rot_dims % 2 or rot_dims > rot_dim:
                raise ConfigError(f"layers[{i}].mixer.rot.dims must be even and at most rot_dim {rot_dim}, got {rot_dims}")
            kv_from = m.get("kv_from")
            if kv_from is not None:
                kv_from = F.get_int(m, "kv_from", minimum=0)
                if kv_from >= i:
                    raise ConfigError(f"layers[{i}].mixer.kv_from must name an earlier layer, got {kv_from}")
            mixer = LatentMixer(heads=F.get_int(m, "heads", minimum=1), dim=F.get_int(m, "dim", minimum=0), rot_dim=rot_dim,
                                vdim=F.get_int(m, "vdim", minimum=1), kv_rank=F.get_int(m, "kv_rank", minimum=1),
                                scale=F.get_float(m, "scale"), rot_base=F.get_float(rot, "base"), rot_dims=rot_dims,
                                kv_from=kv_from)
            if kv_from is not None:
                src = out[kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"layers[{i}].mixer.kv_from names layer {kv_from}, which has no latent of its own")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                    raise ConfigError(f"layers[{i}].mixer: latent size and rotation must equal those of layer {kv_from}")
            mlp = None
            f = _section(entry, "mlp", optional=True)
            if f is not None:
                kind = F.get_str(f, "kind")
                if kind != "moe":
                    raise ConfigError(f"layers[{i}].mlp: unknown kind {kind!r} (known: moe)")
                r = _section(f, "router")
                g = _section(r, "groups", optional=True) or {}
                mlp = MoE(ff=F.get_int(_section(f, "expert"), "ff", minimum=1), experts=F.get_int(r, "experts", minimum=1),
                          top=F.get_int(r, "top", minimum=1), groups=F.get_int(g, "count", 1, minimum=1),
                          keep=F.get_int(g, "keep", 1, minimum=1), scale=F.get_float(r, "scale", 1.0))
                if not g:
                    mlp = MoE(mlp.ff, mlp.experts, mlp.top, 1, 1, mlp.scale)
            out.append(PuledraLayer(kind, mixer, mlp))
        return cls(vocab=F.get_int(d, "vocab", minimum=1), width=F.get_int(d, "width", minimum=1),
                   eps=F.get_float(_section(d, "norm"), "eps"), embed_scale=F.get_float(emb, "scale", 1.0),
                   pair_table=pair, layers=tuple(out))
