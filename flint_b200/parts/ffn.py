"""Feed-forward parts: a dense gated MLP, a top-2 sparsemixer mixture of experts, and a mixture whose softmax
router chooses the top k experts among the best groups of neighbouring experts.

Dense: h += (act(x Wg^T) * (x Wu^T)) Wd^T, as the reference's feed-forward
(crates/thuban_model/src/ops/mlp.rs:24-79).  Mixture of experts (no counterpart in
the reference): float32 router logits, sparsemixer top-2 selection, rows sorted by
expert, two grouped products, and the gated sum of the two experts' outputs added to
the residual stream in a fixed order.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..registry import FEED_FORWARDS
from .base import FeedForward, Pending, RouterRequest, mat, matmul_dtype


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """params: hidden_size, intermediate_size, act; tensors gate_proj/up_proj [I,H], down_proj [H,I]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.act = params.get("act", "silu")

    def weights(self):
        return {"gate_proj.weight": mat(self.inter, self.hidden), "up_proj.weight": mat(self.inter, self.hidden),
                "down_proj.weight": mat(self.hidden, self.inter)}

    def fused(self):
        return {"gate_up_proj.weight": ["gate_proj.weight", "up_proj.weight"]}

    def load(self, t):
        dt = matmul_dtype(*t.values())
        # gate and up rows in the layout the kernels want: one product gives both
        self.w_gate_up = self.ops.pair_gate_up(t["gate_proj.weight"].to(dt), t["up_proj.weight"].to(dt)).contiguous()
        self.w_down = t["down_proj.weight"].to(dt)

    def input_dtypes(self):
        return (self.w_gate_up.dtype,)

    def forward(self, x, residual, step):
        xin = x[self.w_gate_up.dtype]
        a = torch.empty((xin.shape[0], self.inter), dtype=self.w_gate_up.dtype, device=xin.device)
        self.ops.gated_gemm(xin, self.w_gate_up, a, self.act)
        self.ops.gemm(a, self.w_down, residual, accumulate=True)


@FEED_FORWARDS.register("sparsemixer_moe")
class SparseMixerMoE(FeedForward):
    """params: hidden_size, intermediate_size, num_experts, jitter_eps, act.
    tensors: gate.weight [E,H]; experts.{e}.w1 / w3 [I,H] (gate / up), w2 [H,I] (down)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.E = int(params["num_experts"])
        if not 2 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (2..256)")
        self.eps = float(params["jitter_eps"])
        self.act = params.get("act", "silu")

    def weights(self):
        w = {"gate.weight": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"experts.{e}.w1.weight"] = mat(self.inter, self.hidden)
            w[f"experts.{e}.w2.weight"] = mat(self.hidden, self.inter)
            w[f"experts.{e}.w3.weight"] = mat(self.inter, self.hidden)
        return w

    def load(self, t):
        self.w_router = t["gate.weight"]
        dt = matmul_dtype(*(t[k] for k in t if k.startswith("experts.")))
        # per expert the gate rows (w1) and the up rows (w3) in the layout the kernels want: [E, rows, H]
        self.w13 = torch.stack([self.ops.pair_gate_up(t[f"experts.{e}.w1.weight"].to(dt), t[f"experts.{e}.w3.weight"].to(dt))
                                for e in range(self.E)], 0).contiguous()
        self.w2 = torch.stack([t[f"experts.{e}.w2.weight"].to(dt) for e in range(self.E)], 0).contiguous()

    def input_dtypes(self):
        return (torch.float32, self.w13.dtype)

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        dev = self.w_router.device
        return RouterRequest(self.w_router, self.eps, torch.empty((n_rows, 2), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, 2), dtype=torch.float32, device=dev))

    def input_dtypes_when_routed(self):
        return (self.w13.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w13.dtype]
        T = xa.shape[0]
        dev = xa.device
        if routed is not None:
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, 2), dtype=torch.int32, device=dev)
            gates = torch.empty((T, 2), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_sparsemixer(x[torch.float32], self.w_router, self.eps, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w13.dtype), xa)
        a = torch.empty((2 * T, self.inter), dtype=self.w13.dtype, device=dev)
        ops.gated_gemm(xs, self.w13, a, self.act, plan)
        y = torch.empty((2 * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w2, y, plan, plan_ready=True)     # the gate/up product ran over the same plan
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            if logits is not None:
                step.record.setdefault("router_logits", []).append(logits)
        # the gated sum of the two experts' rows is added by the next norm's kernel
        return Pending(y=y, row_of=plan.row_of, gates=gates)


@FEED_FORWARDS.register("grouped_topk_moe")
class GroupedTopKMoE(FeedForward):
    """A mixture of gated experts with a softmax router: scores s = softmax(W_router x) in float32; the experts
    form ``groups`` equal groups of neighbours, a group scores as its best member, only members of the
    ``keep_groups`` best groups may be chosen, and the ``top`` best of those are; an expert's weight is its score
    over the sum of the chosen scores (+ 1e-20), times ``router_scale``.  The output is the weighted sum of the
    chosen experts' down(act(gate x) * (up x)).  (No counterpart in the reference, whose feed-forward is dense:
    crates/thuban_model/src/ops/mlp.rs:24-79.)

    params: hidden_size, intermediate_size, num_experts, top, groups, keep_groups, router_scale, act.
    tensors: router [E, H]; e{i}.gate / e{i}.up [I, H], e{i}.down [H, I]."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.E, self.top = int(p["num_experts"]), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep_groups", 1))
        self.router_scale = float(p.get("router_scale", 1.0))
        self.act = p.get("act", "silu")
        if not 1 <= self.E <= 256:
            raise ConfigError(f"num_experts {self.E} is not supported (1..256)")
        if not 1 <= self.top <= min(self.E, 16):
            raise ConfigError(f"{self.top} experts a token of {self.E} is not supported (1..16)")
        if self.groups < 1 or self.groups > 64 or self.E % self.groups:
            raise ConfigError(f"{self.E} experts do not form {self.groups} equal groups (up to 64)")
        if not 1 <= self.keep <= self.groups or self.keep * (self.E // self.groups) < self.top:
            raise ConfigError(f"{self.keep} of {self.groups} groups cannot give {self.top} experts a token")

    def weights(self):
        w = {"router": mat(self.E, self.hidden)}
        for e in range(self.E):
            w[f"e{e}.gate"] = mat(self.inter, self.hidden)
            w[f"e{e}.up"] = mat(self.inter, self.hidden)
            w[f"e{e}.down"] = mat(self.hidden, self.inter)
        return w

    def load(self, t):
        self.w_router = t["router"]
        dt = matmul_dtype(*(v for k, v in t.items() if k != "router"))
        self.w13 = torch.stack([self.ops.pair_gate_up(t[f"e{e}.gate"].to(dt), t[f"e{e}.up"].to(dt))
                                for e in range(self.E)], 0).contiguous()
        self.w2 = torch.stack([t[f"e{e}.down"].to(dt) for e in range(self.E)], 0).contiguous()

    def input_dtypes(self):
        return (torch.float32, self.w13.dtype)       # the router reads the float32 rows

    def router_request(self, n_rows):
        """Routing can ride on the norm before this part (the normalised row is in registers there)."""
        dev = self.w_router.device
        return RouterRequest(self.w_router, 0.0, torch.empty((n_rows, self.top), dtype=torch.int32, device=dev),
                             torch.empty((n_rows, self.top), dtype=torch.float32, device=dev), top=self.top,
                             groups=self.groups, keep=self.keep, scale=self.router_scale)

    def input_dtypes_when_routed(self):
        return (self.w13.dtype,)

    def forward(self, x, residual, step, routed=None):
        ops = self.ops
        xa = x[self.w13.dtype]
        T, dev, k = xa.shape[0], xa.device, self.top
        if routed is not None:
            ids, gates, logits = routed.expert_ids, routed.gates, routed.logits
        else:
            ids = torch.empty((T, k), dtype=torch.int32, device=dev)
            gates = torch.empty((T, k), dtype=torch.float32, device=dev)
            logits = torch.empty((T, self.E), dtype=torch.float32, device=dev) if step.record is not None else None
            ops.router_topk(x[torch.float32], self.w_router, k, self.groups, self.keep, self.router_scale, ids, gates, logits)
        plan, xs = ops.moe_dispatch(ids, self.E, ops.moe_tile_rows(T, self.E, self.w13.dtype, k), xa)
        a = torch.empty((k * T, self.inter), dtype=self.w13.dtype, device=dev)
        ops.gated_gemm(xs, self.w13, a, self.act, plan)
        y = torch.empty((k * T, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(a, self.w2, y, plan, plan_ready=True)
        if step.record is not None:
            step.record.setdefault("experts", []).append(ids)
            step.record.setdefault("gates", []).append(gates)
            if logits is not None:
                step.record.setdefault("router_logits", []).append(logits)
        # the weighted sum of the chosen experts' rows is added by the next norm's kernel
        return Pending(y=y, row_of=plan.row_of, gates=gates)
