"""Tiny Puledra configurations that differ in every size and option, and a writer of model folders whose
random weights are large enough that every mechanism shows in the logits (attention is peaked, router
scores are spread, the pair table matters)."""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


def _mixer(heads, dim, rot_dim, rot_dims, vdim, kv_rank, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dims}, "scale": 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, count, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# P1: sizes that are multiples of 8 beside sizes that are not (latent rows padded, products on the float32 pipes),
# a partly rotated key part, a layer without a feed-forward, two layers reading another's latent, one expert a
# token, one group, a router scale of 1.
P1 = {
    "architecture": "Puledra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.5, "bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 5}},
    "layers": [
        _layer(_mixer(3, 16, 8, 8, 24, 40, 10000.0), _moe(32, 8, 2, 4, 2, 1.5)),
        _layer(_mixer(2, 8, 8, 8, 16, 40, 10000.0, kv_from=0), None),
        _layer(_mixer(5, 10, 6, 4, 12, 20, 300.0), _moe(24, 6, 1, 1, 1, 1.0)),
        _layer(_mixer(1, 12, 6, 4, 20, 20, 300.0, kv_from=2), _moe(16, 4, 4, 2, 2, 0.5)),
    ],
}

# P2: no pair table, no rotation limit below rot_dim, two layers with equal cache needs (one page group, two
# caches), three experts of twelve from two of three groups, every product on the tensor cores in bfloat16.
P2 = {
    "architecture": "Puledra", "vocab": 160, "width": 64, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0},
    "layers": [
        _layer(_mixer(4, 32, 16, 16, 32, 48, 500000.0), _moe(48, 12, 3, 3, 2, 2.0)),
        _layer(_mixer(4, 32, 16, 16, 32, 48, 500000.0), _moe(48, 12, 3, 3, 2, 2.0)),
        _layer(_mixer(8, 16, 16, 16, 8, 48, 500000.0, kv_from=1), _moe(32, 4, 2, 1, 1, 1.0)),
    ],
}

CONFIGS = {"P1": P1, "P2": P2}


def tensor_shapes(cfg):
    """Every tensor of a checkpoint by name, written down here independently of the package."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W)}
    pair = cfg["embedding"].get("bigram")
    if pair:
        out["bigram"] = (pair["buckets"] + 1, W)
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out[f"l{i}.norm1"] = (W,)
        out[f"l{i}.mix.q"] = (H * (D + R), W)
        if m.get("kv_from") is None:
            out[f"l{i}.mix.dkv"] = (C + R, W)
            out[f"l{i}.mix.dkv.norm"] = (C,)
        out[f"l{i}.mix.uk"] = (H * D, C)
        out[f"l{i}.mix.uv"] = (H * V, C)
        out[f"l{i}.mix.o"] = (W, H * V)
        f = layer.get("mlp")
        if f:
            out[f"l{i}.mlp.router"] = (f["router"]["experts"], W)
            for e in range(f["router"]["experts"]):
                out[f"l{i}.mlp.e{e}.gate"] = (f["expert"]["ff"], W)
                out[f"l{i}.mlp.e{e}.up"] = (f["expert"]["ff"], W)
                out[f"l{i}.mlp.e{e}.down"] = (W, f["expert"]["ff"])
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, seed=0):
    """bfloat16 tensors: matrices N(0, g^2 / fan_in) with g = 2 for queries, latents and routers (peaked attention,
    spread router scores), norm scales 1 + N(0, 0.1), tables N(0, 1) and N(0, 0.5)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name == "bigram":
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            gain = 2.0 if name.endswith((".q", ".dkv", ".router")) else 1.0
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[1])
        w[name] = t.to(torch.bfloat16)
    return w


def write_safetensors(path, tensors):
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        code = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}[t.dtype]
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    Path(path).write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def write_model(folder, cfg, seed=0, weights=None):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    w = weights if weights is not None else random_weights(cfg, seed)
    write_safetensors(folder / "model.safetensors", w)
    return folder, {k: v.double() for k, v in w.items()}
