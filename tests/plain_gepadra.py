"""Plain, slow implementation of Gepadra, one function per mechanism, in float64 torch on the CPU.

It shares no code with the package: weights come in as a dictionary of tensors by their stored names,
the configuration as the dictionary that ``config.json`` holds.  A whole sequence is run at once (or, for
the recurrent mixer, token by token from a given state), and the package's results under every way of
cutting a prompt are compared with that.

Notation: x the residual stream [T, W]; h a normalised copy of it; positions p count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, w, eps):
    """RMS norm whose stored scale is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate_leading_dims(x, pos, base, dims):
    """x [T, heads, d]: dims i and i + dims/2 (i < dims/2) of every head turn by the angle
    pos * base^(-2i/dims); dims from ``dims`` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = pos.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def visible(pos_q, pos_k, size, keep_first):
    """[Tq, Tk] bool: key j is seen from i if it is not later and either near (i - j < size) or one of the
    first ``keep_first`` of the sequence."""
    i, j = pos_q[:, None], pos_k[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def sink_softmax_mix(scores, sink, values, mask):
    """scores [H, Tq, Tk], sink [H], values [H, Tk, dv]: softmax over the seen keys and one more logit per head
    that has no value."""
    scores = scores.masked_fill(~mask[None], -math.inf)
    top = torch.maximum(scores.max(-1).values, sink[:, None])
    e = torch.exp(scores - top[..., None])
    denom = e.sum(-1) + torch.exp(sink[:, None] - top)
    return (e / denom[..., None]) @ values


def attention_mixer(h, w, pre, m, pos, v_first, is_first):
    """The attention mixer on a whole sequence.  Returns (output [T, W], the values of this layer before mixing
    if it is the first that mixes, else None)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, d)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_leading_dims(q, pos, float(rot["base"]), int(rot["dims"]))
    k = rotate_leading_dims(k, pos, float(rot["base"]), int(rot["dims"]))
    own_v = None
    if m.get("v_mix"):
        if is_first:
            own_v = v
        else:
            lam = w[pre + "vmix"]
            v = (1.0 - lam) * v + lam * v_first
    per = H // G
    kk = k.repeat_interleave(per, 1).transpose(0, 1)            # [H, T, d]
    vv = v.repeat_interleave(per, 1).transpose(0, 1)
    scores = (q.transpose(0, 1) @ kk.transpose(1, 2)) * float(m["scale"])
    mask_cfg = m.get("mask") or {}
    size = int(mask_cfg.get("size", 1 << 40))
    mask = visible(pos, pos, size, int(mask_cfg.get("keep_first", 0)))
    o = sink_softmax_mix(scores, w[pre + "sink"], vv, mask)     # [H, T, dv]
    return o.transpose(0, 1).reshape(T, H * dv) @ w[pre + "o"].T, own_v


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def mlstm_gates(h, w, pre, cap):
    """Log input gate and log forget gate per head, [T, heads] each."""
    i = capped(h @ w[pre + "i"].T + w[pre + "i.b"], cap)
    f = torch.nn.functional.logsigmoid(capped(h @ w[pre + "f"].T + w[pre + "f.b"], cap))
    return i, f


def mlstm_step(state, q, k, v, i, f):
    """One token of one head.  state = (S [d, dv], n [d], m scalar); q, k [d], v [dv]; i, f scalars (logs)."""
    S, n, m = state
    m_new = torch.maximum(f + m, i)
    keep, take = torch.exp(f + m - m_new), torch.exp(i - m_new)
    S = keep * S + take * torch.outer(k, v)
    n = keep * n + take * k
    o = (S.T @ q) / (torch.maximum(torch.abs(n @ q), torch.exp(-m_new)) + 1e-6)
    return (S, n, m_new), o


def mlstm_zero_state(heads, d, dv):
    return [(torch.zeros(d, dv, dtype=F64), torch.zeros(d, dtype=F64), torch.zeros((), dtype=F64)) for _ in range(heads)]


def mlstm_mixer(h, w, pre, m, eps, state=None):
    """The matrix-memory mixer on consecutive tokens of one sequence, from ``state`` (None: a new sequence).
    Returns (output [T, W], state after the last token)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    i, f = mlstm_gates(h, w, pre, float(m["gate_cap"]))
    state = list(state) if state is not None else mlstm_zero_state(H, d, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for a in range(H):
            state[a], o[t, a] = mlstm_step(state[a], q[t, a], k[t, a], v[t, a], i[t, a], f[t, a])
    o = unit_rms(o, eps).reshape(T, H * dv) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, state


def clamped_glu(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def small_expert(x, w, pre):
    return gelu_erf(x @ w[pre + "up"].T) @ w[pre + "down"].T


def sigmoid_router(h, w, pre, top):
    """(chosen experts [T, top], their scores [T, top], logits [T, E]): the largest sigmoid scores, as they are."""
    z = h @ w[pre + "router"].T
    s = torch.sigmoid(z)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val, z


def expert_mixture(h, w, pre, f, forced=None):
    """Each token's chosen experts run on the token's row times the expert's score; a shared expert runs on
    every row and is weighted by a sigmoid gate.  ``forced`` [T, top]: experts to use instead of the router's
    choice (their scores still come from the router)."""
    top = int(f["router"]["top"])
    idx, val, z = sigmoid_router(h, w, pre, top)
    if forced is not None:
        idx = forced.long()
        val = torch.sigmoid(z).gather(1, idx)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += small_expert(val[t, c] * h[t], w, f"{pre}e{e}.")
    if f.get("shared") is not None:
        gate = torch.sigmoid(h @ w[pre + "shared.sg"].T)            # [T, 1]
        out = out + gate * small_expert(h, w, pre + "shared.")
    return out, idx, z


def widen(weights):
    return {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}


def forward(cfg, weights, tokens, forced_experts=None, keep=None):
    """Logits [T, vocab] of one whole sequence.  ``forced_experts``: {layer: [T, top]}.  ``keep``: a dict that
    receives the residual stream after every layer ("layers"), the experts chosen ("experts") and the router
    logits ("router_logits") by layer."""
    w = widen(weights)
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    v_first, seen_mix = None, False
    for li, layer in enumerate(cfg["layers"]):
        pre = f"l{li}."
        h1 = offset_rms_norm(x, w[pre + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            first = bool(m.get("v_mix")) and not seen_mix
            mixed, own_v = attention_mixer(h1, w, pre + "mix.", m, pos, v_first, first)
            if first:
                v_first, seen_mix = own_v, True
        elif layer["type"] == "mlstm":
            mixed, _ = mlstm_mixer(h1, w, pre + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        fed = 0.0
        f = layer.get("mlp")
        if f is not None:
            h2 = offset_rms_norm(x, w[pre + "norm2"], eps)
            if f["kind"] == "dense":
                fed = clamped_glu(h2, w, pre + "mlp.", float(f["limit"]))
            else:
                fed, idx, z = expert_mixture(h2, w, pre + "mlp.", f, None if forced_experts is None else forced_experts.get(li))
                if keep is not None:
                    keep.setdefault("experts", {})[li] = idx
                    keep.setdefault("router_logits", {})[li] = z
        x = x + (mixed + fed)
        if keep is not None:
            keep.setdefault("layers", []).append(x.clone())
    return offset_rms_norm(x, w["final.norm"], eps) @ w["embed"].T
