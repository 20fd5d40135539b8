"""Tiny Gepadra configurations that differ in every size and option, and a writer of model folders whose random
weights are large enough that every mechanism shows in the logits (attention is peaked, sinks take a real share,
the forget gates keep memory over many tokens, router scores are spread, the clamps of the gated unit bite)."""
from __future__ import annotations

import math

import torch

from tiny_puledra import write_model as _write_folder


def _attn(heads, kv, dim, vdim, scale=None, window=None, keep=0, rot=None, base=10000.0, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return m


def _mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


# G1: sizes that are not multiples of 8 or of 32 (rows read element by element, products on the float32 pipes),
# three query heads to a key head, values wider and narrower than keys, a window shorter than a page with kept
# first tokens, a window that keeps none, an attention layer that sees everything and rotates nothing, a partly and
# a fully rotated head, a layer without a feed-forward, two and three experts a token, a mixture without a shared
# expert, a one-headed matrix memory wider than a warp, an attention layer that blends values and one that does not.
G1 = {
    "architecture": "Gepadra", "vocab": 91, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(6, 2, 24, 10, window=9, keep=3, rot=12, v_mix=True), "mlp": _dense(56, 1.0)},
        {"type": "mlstm", "mixer": _mlstm(3, 20, 12, 6.0), "mlp": _moe(24, 5, 2, shared=16)},
        {"type": "attention", "mixer": _attn(4, 2, 16, 10, scale=0.3, window=17, keep=0, rot=16, base=300.0, v_mix=True), "mlp": None},
        {"type": "mlstm", "mixer": _mlstm(1, 40, 6, 9.0), "mlp": _moe(16, 3, 1)},
        {"type": "attention", "mixer": _attn(2, 1, 8, 18), "mlp": _moe(8, 4, 3, shared=24)},
        {"type": "attention", "mixer": _attn(2, 2, 12, 10, window=30, keep=20, rot=4, v_mix=True), "mlp": _dense(24, 2.5)},
    ],
}

# G2: sizes in multiples of 16 (every product on the tensor cores in bfloat16), the matrix memory first, kept
# first tokens that reach into a second page of 16, one query head a key head and two, a dense unit beside attention,
# experts beside both kinds of mixer.
G2 = {
    "architecture": "Gepadra", "vocab": 160, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": _mlstm(4, 32, 32, 15.0), "mlp": _moe(32, 8, 2, shared=64)},
        {"type": "attention", "mixer": _attn(8, 8, 32, 16, window=24, keep=19, rot=16, base=500000.0, v_mix=True), "mlp": _dense(96, 7.0)},
        {"type": "attention", "mixer": _attn(16, 8, 16, 16, scale=0.2, window=40, keep=2, rot=8, v_mix=True), "mlp": _moe(48, 6, 1, shared=32)},
        {"type": "mlstm", "mixer": _mlstm(2, 64, 48, 10.0), "mlp": _dense(64, 1.5)},
    ],
}

CONFIGS = {"G1": G1, "G2": G2}


def tensor_shapes(cfg):
    """Every tensor of a checkpoint by name, written down here independently of the package."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                        p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.sink": (H,), p + "mix.o": (W, H * dv)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                        p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        f = layer.get("mlp")
        if f:
            out[p + "norm2"] = (W,)
            if f["kind"] == "dense":
                out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
            else:
                out[p + "mlp.router"] = (f["router"]["experts"], W)
                for e in range(f["router"]["experts"]):
                    out[p + f"mlp.e{e}.up"] = (f["expert"]["ff"], W)
                    out[p + f"mlp.e{e}.down"] = (W, f["expert"]["ff"])
                if f.get("shared"):
                    out.update({p + "mlp.shared.up": (f["shared"]["ff"], W), p + "mlp.shared.down": (W, f["shared"]["ff"]),
                                p + "mlp.shared.sg": (1, W)})
    out["final.norm"] = (W,)
    return out


def random_weights(cfg, seed=0):
    """bfloat16 tensors: matrices N(0, g^2 / fan_in) with g = 2.5 for queries, keys, routers and the gated unit
    (peaked attention, spread scores, clamps that bite), norm offsets N(0, 0.1), the matrix memory's scale
    1 + N(0, 0.1), sinks N(1, 1), blend weights in (0.2, 0.8), forget-gate biases N(3, 1), input-gate biases N(0, 1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".vmix"):
            t = 0.2 + 0.6 * torch.rand((), generator=g)
        elif name.endswith(".sink"):
            t = 1.0 + torch.randn(shape, generator=g)
        elif name.endswith(".f.b"):
            t = 3.0 + torch.randn(shape, generator=g)
        elif name.endswith(".mix.norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith((".norm1", ".norm2", "final.norm")):
            t = 0.1 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = torch.randn(shape, generator=g)            # projection and gate biases
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            gain = 2.5 if name.endswith((".q", ".k", ".router", ".gate", ".up", ".i", ".f", ".sg")) else 1.0
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[1])
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(folder, cfg, seed=0, weights=None):
    return _write_folder(folder, cfg, seed, weights if weights is not None else random_weights(cfg, seed))
