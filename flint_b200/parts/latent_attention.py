"""The latent-attention mixer: attention whose keys and values are up-projections of one cached
low-rank latent per token.

Per token the layer stores c = rmsnorm(first C rows of W_dkv x) and r = rotate(last R rows of W_dkv x),
one vector each, shared by all heads.  Head h has the key [W_uk_h c | r] and the value W_uv_h c; its query
is [q_plain_h | rotate(q_rot_h)] (D + R numbers).  Because the key's up-projection is linear, the score

    q_plain_h . (W_uk_h c_j) + q_rot_h . r_j  =  [W_uk_h^T q_plain_h | q_rot_h] . [c_j | r_j]

is a dot product with the cached row itself, and the head's output W_uv_h (sum_j p_j c_j) needs the
probability-weighted sum of the latents only.  So the mixer runs as attention of H query heads over ONE
cached row per token whose first C numbers double as the value, with two small per-head products around
it (W_uk folded into the query, W_uv applied to the result); keys and values are never materialised.
A layer with ``own_cache`` False makes no latent: it reads the rows another layer call cached, with its
own W_uk, W_uv, queries and output projection.

The reference's attention is grouped-query over cached keys and values
(crates/thuban_architectures/src/transformer/forward.rs:114-365); it has no latent form.
"""
from __future__ import annotations

import torch

from ..cache.manager import KVSpec
from ..errors import ConfigError, ModelError
from ..registry import MIXERS
from .attention import shared_position_encoding
from .base import Mixer, Pending, mat, matmul_dtype, vec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, dim (unrotated q/k dims per head), rot_dim (rotated dims per head, one
    rotated key part for all heads), value_dim, kv_rank (latent size), scale, norm_eps (of the latent's RMS norm),
    window (0 = none), own_cache (False: reads another call's cache and has no down-projection),
    position (PartSpec; its rotary_dim of the rot_dim dims rotate).
    tensors: q [H (dim + rot_dim), hidden], dkv [kv_rank + rot_dim, hidden], dkv.norm [kv_rank],
    uk [H dim, kv_rank], uv [H value_dim, kv_rank], o [hidden, H value_dim]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.D, self.R = int(p["num_heads"]), int(p["dim"]), int(p["rot_dim"])
        self.V, self.C = int(p["value_dim"]), int(p["kv_rank"])
        if min(self.H, self.V, self.C) < 1 or self.D < 0 or self.R < 0 or self.D + self.R < 1:
            raise ConfigError("latent attention: heads, value size and latent size must be positive")
        if self.C > 512:
            raise ConfigError(f"latent attention: latent size {self.C} is not supported (up to 512)")
        self.scale = float(p["scale"])
        self.eps = float(p["norm_eps"])
        self.window = int(p.get("window", 0) or 0)
        self.own_cache = bool(p.get("own_cache", True))
        self.position = shared_position_encoding(p["position"], ctx) if p.get("position") is not None else None
        self.rot = self.position.rotary_dim if self.position is not None else 0
        self.rot_style = self.position.style if self.position is not None else "half"
        if self.rot > self.R:
            raise ConfigError(f"latent attention: {self.rot} rotating dims exceed rot_dim {self.R}")
        self.Dk = self.C + self.R
        self.row_w = -(-self.Dk // 8) * 8          # cached rows are padded with zeros to whole 16-byte units

    def weights(self):
        H, D, R, V, C, W = self.H, self.D, self.R, self.V, self.C, self.hidden
        w = {"q": mat(H * (D + R), W), "uk": mat(H * D, C), "uv": mat(H * V, C), "o": mat(W, H * V)}
        if self.own_cache:
            w["dkv"] = mat(C + R, W)
            w["dkv.norm"] = vec(C, init="gamma")
        return w

    def load(self, t):
        H, D, V, C = self.H, self.D, self.V, self.C
        dt = matmul_dtype(*(v for k, v in t.items() if k != "dkv.norm"))
        # q and the latent's down-projection are one product
        self.w_in = torch.cat([t["q"].to(dt)] + ([t["dkv"].to(dt)] if self.own_cache else []), 0).contiguous()
        self.w_norm = t.get("dkv.norm")
        # W_uk per head, transposed: the product that folds it into the query takes [C, D] per head
        self.w_ukT = t["uk"].to(dt).view(H, D, C).transpose(1, 2).contiguous()
        self.w_uv = t["uv"].to(dt).view(H, V, C).contiguous()
        self.w_o = t["o"].to(dt)
        if self.position is not None:
            self.cos, self.sin = self.position.tables()
        else:
            self.cos = self.sin = torch.zeros((1, 1), dtype=torch.float32, device=self.ctx.device)

    def input_dtypes(self):
        return (self.w_in.dtype,)

    def cache_spec(self):
        # one row per token for all heads, no separate values: the latent is the start of the row
        return KVSpec(1, self.row_w, self.window, value_dim=0) if self.own_cache else None

    def plan_step(self, step, captured):
        """A batch of decoded tokens that is captured as a CUDA graph has its key ranges cut for a bucketed
        context length (four buckets per doubling, at least 256 apart), so that the graph serves every step up
        to that length; the bucket is part of the graph's key."""
        if not captured or step.n_tokens != len(step.entries):
            return None
        kv = max(step.max_kv_len, 1)
        gran = max(256, 1 << max(kv.bit_length() - 3, 0))
        step.max_kv_len = -(-kv // gran) * gran
        return (step.max_kv_len,)

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        if cache is None:
            raise ModelError("latent attention needs a cache")
        if writes_cache != self.own_cache:
            raise ModelError("latent attention: a layer with a down-projection writes its own cache, one without reads another's")
        ops, H, D, R, V, C = self.ops, self.H, self.D, self.R, self.V, self.C
        xin = x[self.w_in.dtype]
        T, dev = xin.shape[0], xin.device
        act = self.ctx.act_dtype if self.w_in.dtype == torch.bfloat16 else torch.float32
        proj = ops.gemm_partials(xin, self.w_in)                 # [S, T, H (D + R) (+ C + R)] partial sums
        q_plain = torch.empty((T, H, D), dtype=act, device=dev)
        qa = torch.empty((T, H, self.Dk), dtype=act, device=dev)
        ops.latent_prepare(proj, step.pos, step.slot, self.cos, self.sin, self.rot, self.rot_style, self.w_norm, self.eps,
                           q_plain, qa, cache, H, D, R, C, writes_cache, step.status)
        if D:
            ops.head_products(q_plain, self.w_ukT, qa[:, :, :C])     # qa[t, h, :C] = W_uk_h^T q_plain[t, h]
        else:
            qa[:, :, :C].zero_()
        o_lat = torch.empty((T, H, C), dtype=act, device=dev)
        ops.latent_attention(qa, cache, step, o_lat, H, C, self.window, self.scale)
        attn = torch.empty((T, H, V), dtype=act, device=dev)
        ops.head_products(o_lat, self.w_uv, attn)                    # attn[t, h] = W_uv_h o_lat[t, h]
        # the output projection is handed on as partial sums
        return Pending(partials=ops.gemm_partials(attn.view(T, H * V), self.w_o))
