"""The mLSTM mixer: a matrix memory per head with exponential gating (the mLSTM cell of xLSTM), run as a
recurrence over the tokens a step brings, from the state the request's earlier steps left.

Per head, with q scaled by dim^(-1/2), log gates i = cap tanh(z_i / cap) and f = logsigmoid(cap tanh(z_f / cap))
(z the gate projections with their biases), a running maximum m (from 0) and S [dim, vdim], n [dim] (from 0):

    m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' likewise with k alone;
    o  = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)

Each head's o is divided by its root mean square, the heads side by side are scaled by ``norm``, gated by
sigmoid(W_g x) and projected by W_o.  The state (S, n, m of every head, float32) is a slab of the cache manager,
one row per request slot, zeroed on admission; the recurrence is evaluated strictly token by token in float32, so
its result does not depend on how a prompt was cut into steps.  The reference keeps recurrent state outside its
paged pool in the same way (crates/thuban_architectures/src/qwen35/state.rs:5-55); it has no mLSTM.
"""
from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..errors import ConfigError, ModelError
from ..registry import MIXERS
from .base import Mixer, Pending, mat, matmul_dtype, vec


@MIXERS.register("mlstm")
class MatrixLSTM(Mixer):
    """params: hidden_size, num_heads, dim (query/key dims per head), value_dim, gate_cap, norm_eps.
    tensors: q, k [H dim, hidden]; v, g [H value_dim, hidden]; i, f [H, hidden] with i.b, f.b [H];
    norm [H value_dim]; o [hidden, H value_dim]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.D, self.V = int(p["num_heads"]), int(p["dim"]), int(p["value_dim"])
        if min(self.H, self.D, self.V) < 1:
            raise ConfigError("mlstm: heads and head sizes must be positive")
        if self.D > 256:
            raise ConfigError(f"mlstm: {self.D} query/key dims per head are not supported (up to 256)")
        self.cap = float(p["gate_cap"])
        self.eps = float(p["norm_eps"])

    def weights(self):
        H, D, V, W = self.H, self.D, self.V, self.hidden
        return {"q": mat(H * D, W), "k": mat(H * D, W), "v": mat(H * V, W), "g": mat(H * V, W), "o": mat(W, H * V),
                "norm": vec(H * V, init="gamma"), "i": mat(H, W), "i.b": vec(H), "f": mat(H, W), "f.b": vec(H)}

    def load(self, t):
        names = ("q", "k", "v", "g", "i", "f")
        dt = matmul_dtype(*(t[n] for n in names), t["o"])
        # one product gives q, k, v, the output gate and the two recurrence gates of every head
        self.w_in = torch.cat([t[n].to(dt) for n in names], 0).contiguous()
        self.b_gates = torch.cat([t["i.b"], t["f.b"]], 0).contiguous()
        self.w_norm = t["norm"]
        self.w_o = t["o"].to(dt)

    def input_dtypes(self):
        return (self.w_in.dtype,)

    def state_spec(self):
        H, D, V = self.H, self.D, self.V
        return StateSpec((H * (D * V + D + 1),), torch.float32)      # per head: S transposed [V, D], then n [D], then m

    def plan_step(self, step, captured):
        """Where each request's rows start, for the recurrence (one request after the other in the flattened
        batch).  A batch of single decoded tokens needs no list: row r is request r."""
        if step.n_tokens != len(step.entries):
            starts = torch.tensor(list(step.entry_start) + [step.n_tokens], dtype=torch.int32)
            step.plans["mlstm.seq_start"] = starts.to(step.pos.device)
        return None

    def forward(self, x, residual, step, cache, state, writes_cache=True):
        if state is None:
            raise ModelError("mlstm needs a state slab")
        ops, H, D, V = self.ops, self.H, self.D, self.V
        xin = x[self.w_in.dtype]
        T, dev = xin.shape[0], xin.device
        act = self.ctx.act_dtype if self.w_in.dtype == torch.bfloat16 else torch.float32
        proj = ops.gemm_partials(xin, self.w_in)                  # [S, T, 2 H D + 2 H V + 2 H] partial sums
        o = torch.empty((T, H * V), dtype=torch.float32, device=dev)
        seq_start = None if T == len(step.entries) else step.plans["mlstm.seq_start"]
        gate = ops.mlstm_scan(proj, self.b_gates, step.slot, seq_start, len(step.entries), state, o, H, D, V, self.cap)
        a = torch.empty((T, H * V), dtype=act, device=dev)
        ops.mlstm_finish(o, gate, self.w_norm, self.eps, a, H, V)
        return Pending(partials=ops.gemm_partials(a, self.w_o))
