"""Plain, slow Puledra forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Puledra tests.  It shares no code with ``flint_b200``: the configuration is a
dictionary, the weights a dictionary of dense CPU tensors (float64 by default), and every
mechanism is a dense torch expression over a whole sequence.

Puledra is a decoder of parallel layers, x <- x + (mixer(n) + ff(n)) with n = rmsnorm(x):
  * the embedding is the token's row times a constant plus a hashed row for the pair
    (previous token, token);
  * the mixer is attention over a low-rank latent: each token stores one normed latent vector c and
    one rotated key part shared by all heads; a head's key is [W_uk c, rotated part], its value
    W_uv c; a layer may read the latents that an earlier layer stored instead of making its own;
  * the feed-forward is a mixture of SiLU-gated experts chosen by a softmax router whose choice is
    limited to the best groups of neighbouring experts.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64,
       "F64": torch.float64}


def read_safetensors(path):
    """8-byte little-endian header length, JSON header, raw tensor bytes."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    out = {}
    for name, info in json.loads(raw[8:8 + n]).items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=_ST[info["dtype"]]) if hi > lo else \
            torch.empty(0, dtype=_ST[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir, dtype=torch.float64):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    w = {n: (t.to(dtype) if t.is_floating_point() else t)
         for n, t in read_safetensors(model_dir / "model.safetensors").items()}
    return cfg, w


# ----------------------------------------------------------------------------- mechanisms

def rms_norm(x, weight, eps):
    """y = x / sqrt(mean(x^2) + eps) * weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every place: (prev * mul_prev + cur * mul_cur) mod buckets, and the extra last
    row (number ``buckets``) for the first token of a sequence."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (int(tokens[i - 1]) * mul_prev + int(t) * mul_cur) % buckets)
    return rows


def embed(tokens, table, scale, pair_table=None, pair=None):
    x = table[torch.as_tensor(list(tokens), dtype=torch.long)] * scale
    if pair_table is not None:
        rows = bigram_rows(tokens, int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"]))
        x = x + pair_table[torch.as_tensor(rows, dtype=torch.long)]
    return x


def rotate_pairs(x, positions, base, dims):
    """Rotary encoding of the first ``dims`` numbers of the last axis, neighbours (2i, 2i+1) as a pair:
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims).  x: [T, ..., D]."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=x.dtype)[:, None] * freq[None, :]       # [T, dims/2]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_of(n, w_dkv, w_norm, eps, kv_rank, rot_dim, rot, positions):
    """What a layer stores per token: the normed latent c [T, kv_rank] and the rotated shared key part
    [T, rot_dim]."""
    d = n @ w_dkv.T
    c = rms_norm(d[:, :kv_rank], w_norm, eps)
    kr = rotate_pairs(d[:, kv_rank:kv_rank + rot_dim], positions, float(rot["base"]), int(rot["dims"]))
    return c, kr


def latent_attention(n, w, m, eps, positions, stored=None):
    """The mixer on normed rows n [T, width].  ``w``: the mixer's tensors by short name (q, dkv, dkv.norm, uk,
    uv, o).  ``stored``: (c, rotated key part) of the layer this one reads from, or None to make its own.
    Returns (output [T, width], (c, rotated key part))."""
    T = n.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (n @ w["q"].T).view(T, H, D + R)
    q_plain = q[..., :D]
    q_rot = rotate_pairs(q[..., D:].contiguous(), positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    if stored is None:
        stored = latent_of(n, w["dkv"], w["dkv.norm"], eps, C, R, m["rot"], positions)
    c, kr = stored
    k_plain = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, V)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, kr)) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    p = torch.softmax(scores, -1)
    o = torch.einsum("hts,shv->thv", p, v).reshape(T, H * V)
    return o @ w["o"].T, stored


def route(z, top, n_groups, keep, scale):
    """Router logits z [E] -> (chosen experts, weights).  s = softmax(z); a group of E / n_groups neighbours
    scores as its best member; only members of the ``keep`` best groups may be chosen; the ``top`` best of
    those are chosen; weights s_e / (sum of chosen s + 1e-20) * scale."""
    E = z.numel()
    s = torch.softmax(z, -1)
    per = E // n_groups
    gs = s.view(n_groups, per).max(-1).values
    kept = torch.topk(gs, keep).indices.tolist()
    allowed = torch.zeros(E, dtype=torch.bool)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    cand = s.masked_fill(~allowed, -1.0)
    ids = torch.topk(cand, top).indices
    ws = s[ids]
    return ids.tolist(), (ws / (ws.sum() + 1e-20) * scale).tolist()


def expert(x, gate, up, down):
    g = x @ gate.T
    return ((g * torch.sigmoid(g)) * (x @ up.T)) @ down.T


def moe(n, w, f, router_dtype=None):
    """Mixture of experts on normed rows n.  ``w``: the feed-forward's tensors by short name (router,
    e<i>.gate/up/down).  Returns (output, chosen experts per row)."""
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    z = n @ w["router"].T
    out = torch.zeros_like(n)
    chosen = []
    for t in range(n.shape[0]):
        ids, ws = route(z[t], top, int(r["groups"]["count"]), int(r["groups"]["keep"]), float(r["scale"]))
        chosen.append(ids)
        for e, g in zip(ids, ws):
            out[t] += g * expert(n[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    return out, chosen


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg, w, tokens, return_layers=False, return_experts=False, follow=None):
    """Logits [T, vocab] of a whole sequence.  ``return_layers``: also the residual stream after every layer.
    ``follow``: per layer, per row, the experts to use instead of the router's own choice (weights are still
    the router's scores of those experts)."""
    eps = float(cfg["norm"]["eps"])
    emb = cfg["embedding"]
    pair = emb.get("bigram")
    x = embed(tokens, w["embed"], float(emb["scale"]), w.get("bigram") if pair else None, pair)
    positions = list(range(len(tokens)))
    stored, layers, experts = {}, [], []
    for i, layer in enumerate(cfg["layers"]):
        n = rms_norm(x, w[f"l{i}.norm1"], eps)
        m = layer["mixer"]
        src = m.get("kv_from")
        a, st = latent_attention(n, sub(w, f"l{i}.mix."), m, eps, positions, stored[src] if src is not None else None)
        if src is None:
            stored[i] = st
        y = a
        if layer.get("mlp") is not None:
            f = layer["mlp"]
            fw = sub(w, f"l{i}.mlp.")
            if follow is not None:
                y_ff = torch.zeros_like(n)
                z = n @ fw["router"].T
                r = f["router"]
                for t in range(n.shape[0]):
                    ids = list(follow[i][t])
                    s = torch.softmax(z[t], -1)[ids]
                    g = s / (s.sum() + 1e-20) * float(r["scale"])
                    for e, ge in zip(ids, g.tolist()):
                        y_ff[t] += ge * expert(n[t:t + 1], fw[f"e{e}.gate"], fw[f"e{e}.up"], fw[f"e{e}.down"])[0]
                experts.append([list(v) for v in follow[i]])
            else:
                y_ff, ch = moe(n, fw, f)
                experts.append(ch)
            y = y + y_ff
        else:
            experts.append(None)
        x = x + y
        layers.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    out = (logits,)
    if return_layers:
        out += (torch.stack(layers),)
    if return_experts:
        out += (experts,)
    return out if len(out) > 1 else logits
