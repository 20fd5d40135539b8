"""Gepadra on the GPU: each new kernel beside the plain function of its mechanism (planted keys far back, among a
window's kept first tokens and just past them, at a window's two edges and at page borders, in prompts and in
decoding, with forced splits; the matrix memory cut anywhere; the sigmoid router; the clamped gated unit), and the
whole model under every cut, in long decoding and in generation, beside the plain implementation."""
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_gepadra as P
import tiny_gepadra as tiny
import traces
from flint_b200.cache.manager import CacheView, KVSpec
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.sampling.params import SamplingParams

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = (1, 2, 9, 37, 70, 130)


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def paged_kv(keys, values, P_, dtype, seed=0):
    """keys / values: per slot [n, G, d] / [n, G, dv] float64.  A cache whose pages lie in a shuffled order, and
    the dense rows as the cache's type rounds them."""
    rnd = random.Random(seed)
    G, d, dv = keys[0].shape[1], keys[0].shape[2], values[0].shape[2]
    n_pages = sum(-(-len(k) // P_) for k in keys) + 3
    order = list(range(n_pages))
    rnd.shuffle(order)
    kc, vc = torch.zeros(n_pages, G, P_, d, dtype=dtype), torch.zeros(n_pages, G, P_, dv, dtype=dtype)
    bt = torch.full((len(keys), max(-(-len(k) // P_) for k in keys) + 1), -1, dtype=torch.int32)
    for s, (k, v) in enumerate(zip(keys, values)):
        for j in range(len(k)):
            if j % P_ == 0:
                bt[s, j // P_] = order.pop()
            kc[bt[s, j // P_], :, j % P_] = k[j].to(dtype)
            vc[bt[s, j // P_], :, j % P_] = v[j].to(dtype)
    dense = [(k.to(dtype).double(), v.to(dtype).double()) for k, v in zip(keys, values)]
    return CacheView(kc.to(DEV), vc.to(DEV), bt.to(DEV), P_, KVSpec(G, d, 0, dv)), dense


def dense_attention(q, dense, pos, slot, H, G, scale, window, keep, sinks):
    """The plain mechanism row by row: visibility, sink softmax, value mix."""
    out = []
    for t in range(q.shape[0]):
        p = int(pos[t])
        k, v = dense[int(slot[t])]
        k, v = k[:p + 1].repeat_interleave(H // G, 1).transpose(0, 1), v[:p + 1].repeat_interleave(H // G, 1).transpose(0, 1)
        scores = (q[t].double()[:, None, :] @ k.transpose(1, 2)) * scale                   # [H, 1, n]
        mask = P.visible(torch.tensor([p]), torch.arange(p + 1), window if window else 1 << 40, keep)
        out.append(P.sink_softmax_mix(scores, sinks.double() if sinks is not None else torch.full((H,), -math.inf, dtype=F64), v, mask)[:, 0])
    return torch.stack(out)


def step_of(pos, slot, n_entries):
    pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
    return SimpleNamespace(pos=pos, slot=torch.tensor(slot, dtype=torch.int32, device=DEV), max_kv_len=int(pos.max()) + 1,
                           entries=[None] * n_entries)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(6, 2, 24, 10), (8, 8, 32, 16), (5, 1, 7, 33), (16, 2, 128, 64)])
@pytest.mark.parametrize("window,keep", [(40, 4), (9, 3), (0, 0), (64, 19), (33, 0)])
def test_sink_attention_finds_planted_keys(ops, dtype, H, G, d, dv, window, keep):
    """One key a row is made to stand out (its score far above the rest): the first token, the last kept one, the
    first one that is not kept, the one just outside the window, the one just inside it, keys on both sides of
    page borders, the row's own.  Rows of a prompt's portion and single decoded rows, two requests."""
    g = torch.Generator().manual_seed(H * 1000 + d + window)
    n = [333, 150]
    P_ = 16
    keys = [torch.randn(m, G, d, generator=g, dtype=F64) for m in n]
    values = [torch.randn(m, G, dv, generator=g, dtype=F64) for m in n]
    rows = []          # (slot, position, planted key)
    for s, m in enumerate(n):
        for p in (m - 1, m - 2, m - 30, 70, 17, 16, 15, 1, 0):
            for j in {0, max(keep - 1, 0), keep, p - window, p - window + 1, p - 1, p, (p // P_) * P_, (p // P_) * P_ - 1, 31, 32}:
                if 0 <= j <= p:
                    rows.append((s, p, j))
    unit = torch.nn.functional.normalize(torch.randn(len(rows), d, generator=g, dtype=F64), dim=-1)
    q = torch.randn(len(rows), H, d, generator=g, dtype=F64)
    for r, (s, p, j) in enumerate(rows):          # the planted pair: a long query along a direction, and that key along it too
        q[r, r % H] = 8.0 * unit[r] * math.sqrt(d)
    # keys are shared by rows, so a planted key is written for one row at a time: group rows by planted key
    by_key = {}
    for r, (s, p, j) in enumerate(rows):
        by_key.setdefault((s, j), []).append(r)
    sinks = torch.randn(H, generator=g) + 1.0
    scale = d ** -0.5
    for (s, j), rs in by_key.items():
        kk = [k.clone() for k in keys]
        kk[s][j, (rs[0] % H) // (H // G)] = 3.0 * unit[rs[0]] * math.sqrt(d)
        view, dense = paged_kv(kk, values, P_, dtype, seed=j)
        qs = q[rs].to(dtype)
        pos, slot = [rows[r][1] for r in rs], [rows[r][0] for r in rs]
        want = dense_attention(qs, dense, pos, slot, H, G, scale, window, keep, sinks)
        for splits in (None, (32, -(-(max(pos) + 1) // 32))):
            out = torch.zeros(len(rs), H * dv, dtype=dtype, device=DEV)
            ops.sink_attention(qs.reshape(len(rs), H * d).to(DEV), view, step_of(pos, slot, len(rs)), out, H, G, d, dv, window, keep,
                               sinks.to(DEV), scale, splits=splits)
            err = (out.cpu().double().view(len(rs), H, dv) - want).abs().max().item()
            assert err < (2e-5 if dtype == torch.float32 else 3e-2), (s, j, splits, err)
    # without a sink the weights sum to one
    view, dense = paged_kv(keys, values, P_, dtype)
    pos, slot = [n[0] - 1, 5], [0, 1]
    qs = q[:2].to(dtype)
    out = torch.zeros(2, H * dv, dtype=dtype, device=DEV)
    ops.sink_attention(qs.reshape(2, H * d).to(DEV), view, step_of(pos, slot, 2), out, H, G, d, dv, window, keep, None, scale)
    want = dense_attention(qs, dense, pos, slot, H, G, scale, window, keep, None)
    assert (out.cpu().double().view(2, H, dv) - want).abs().max().item() < (2e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 32, 16), (8, 8, 128, 48), (6, 2, 64, 128), (2, 1, 16, 64)])
@pytest.mark.parametrize("window,keep", [(40, 4), (9, 3), (0, 0), (100, 70), (33, 0)])
def test_sink_attention_tiles_on_the_tensor_cores(ops, H, G, d, dv, window, keep):
    """Portions of prompts as tiles of up to 64 rows (whole tiles, a ragged last one, a portion that starts in the
    middle of a request and of a page, a portion just past the kept tokens) beside single rows, two requests: the
    tensor-core kernel and the row kernel together against the plain mechanism, with peaked scores."""
    from flint_b200.engine.step import Tiling
    g = torch.Generator().manual_seed(H + d + window)
    n, P_ = [333, 150], 16
    keys = [2.0 * torch.randn(m, G, d, generator=g, dtype=F64) for m in n]
    values = [torch.randn(m, G, dv, generator=g, dtype=F64) for m in n]
    view, dense = paged_kv(keys, values, P_, torch.bfloat16, seed=3)
    portions = [(0, 0, 150), (1, 0, 64), (0, 150, 17), (1, 64, 3), (0, 167, 166), (1, 67, 1), (1, 68, 82)]    # (slot, first position, count)
    pos = [p0 + i for s_, p0, c in portions for i in range(c)]
    slot = [s_ for s_, p0, c in portions for i in range(c)]
    T = len(pos)
    q = (2.0 * torch.randn(T, H, d, generator=g, dtype=F64)).to(torch.bfloat16)
    sinks = torch.randn(H, generator=g) + 1.0
    scale = d ** -0.5
    tiles, others, row = [], [], 0
    for s_, p0, c in portions:
        if c < 16:
            others += range(row, row + c)
        else:
            for r in range(0, c, 64):
                tiles.append([row + r, min(64, c - r), s_, p0 + r])
        row += c
    tiles.sort(key=lambda t: -(t[3] + t[1]))
    tiling = Tiling(torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles), torch.tensor(others, dtype=torch.int32, device=DEV), len(others))
    want = dense_attention(q, dense, pos, slot, H, G, scale, window, keep, sinks)
    out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
    ops.sink_attention(q.reshape(T, H * d).to(DEV), view, step_of(pos, slot, len(portions)), out, H, G, d, dv, window, keep,
                       sinks.to(DEV), scale, tiling=tiling)
    err = (out.cpu().double().view(T, H, dv) - want).abs()
    assert err.max().item() < 4e-2, (int(err.view(T, -1).max(-1).values.argmax()), err.max().item())
    plain = torch.zeros_like(out)
    ops.sink_attention(q.reshape(T, H * d).to(DEV), view, step_of(pos, slot, len(portions)), plain, H, G, d, dv, window, keep, sinks.to(DEV), scale)
    assert (plain.float() - out.float()).abs().max().item() < 4e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style,rot", [("half", 12), ("half", 24), ("interleaved", 8), ("half", 0)])
def test_qkv_write_rotates_blends_and_fills_the_pages(ops, dtype, style, rot):
    H, G, d, dv, P_, T = 6, 2, 24, 10, 16, 37
    g = torch.Generator().manual_seed(rot + 1)
    W = (H + G) * d + G * dv
    parts = torch.randn(3, T, W, generator=g)
    bias = torch.randn(W, generator=g)
    pos = torch.tensor([(5 * t) % 61 for t in range(T)], dtype=torch.int32)
    slot = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    pos[1::2] += 64          # no two rows of a slot share a position
    base = 300.0
    half = max(rot // 2, 1)
    ang = pos.double()[:, None] * base ** (-2.0 * torch.arange(half, dtype=F64) / max(rot, 1))[None, :]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    table = torch.zeros(int(pos.max()) + 1, half)
    ct, st = table.clone(), table.clone()
    ct[pos.long()], st[pos.long()] = cos.cpu(), sin.cpu()
    n_pages = 2 * 9
    view = CacheView(torch.zeros(n_pages, G, P_, d, dtype=dtype, device=DEV), torch.zeros(n_pages, G, P_, dv, dtype=dtype, device=DEV),
                     torch.arange(n_pages, dtype=torch.int32).view(2, 9).to(DEV), P_, KVSpec(G, d, 0, dv))
    x = parts.double().sum(0) + bias.double()
    qw = x[:, :H * d].view(T, H, d)
    kw = x[:, H * d:(H + G) * d].view(T, G, d)
    vw = x[:, (H + G) * d:].view(T, G, dv)
    if style == "half":
        qw, kw = P.rotate_leading_dims(qw, pos, base, rot), P.rotate_leading_dims(kw, pos, base, rot)
    elif rot:                      # pairs (2i, 2i + 1): the plain rotation on a permuted copy
        perm = list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, d))
        inv = [perm.index(i) for i in range(d)]
        qw = P.rotate_leading_dims(qw[..., perm], pos, base, rot)[..., inv]
        kw = P.rotate_leading_dims(kw[..., perm], pos, base, rot)[..., inv]
    v_from = torch.randn(T, G * dv, generator=g)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for blend in (None, 0.35):
        q_out = torch.zeros(T, H * d, dtype=dtype, device=DEV)
        v_keep = torch.zeros(T, G * dv, device=DEV)
        ops.qkv_write(parts.to(DEV), bias.to(DEV), pos.to(DEV), slot.to(DEV), ct.to(DEV), st.to(DEV), rot, style, q_out, view,
                      H, G, d, dv, status, v_keep=v_keep, v_from=v_from.to(DEV) if blend else None, blend=blend or 0.0)
        assert (q_out.cpu().double().view(T, H, d) - qw).abs().max() < tol * 4
        assert (v_keep.cpu().double().view(T, G, dv) - vw).abs().max() < 1e-5
        vv = vw if blend is None else (1 - blend) * vw + blend * v_from.double().view(T, G, dv)
        page = view.block_table.cpu()[slot.long(), (pos // P_).long()].long()
        assert (view.k.cpu()[page, :, (pos % P_).long()].double() - kw).abs().max() < tol * 4
        assert (view.v.cpu()[page, :, (pos % P_).long()].double() - vv).abs().max() < tol * 4
    assert int(status.item()) == 0


@pytest.mark.parametrize("H,D,V", [(3, 20, 12), (1, 40, 6), (2, 64, 48), (2, 130, 33), (4, 32, 32)])
def test_matrix_memory_kernels_follow_the_recurrence_however_the_tokens_are_cut(ops, H, D, V):
    """Three requests of unequal length in one batch against the plain step function; then the same tokens in
    portions, single tokens and a decode batch from the carried state: the same numbers to float32 rounding."""
    g = torch.Generator().manual_seed(H + D + V)
    cap, lens = 7.0, [23, 1, 40]
    T, N = sum(lens), 2 * H * D + 2 * H * V + 2 * H
    proj = torch.randn(2, T, N, generator=g) * 0.7
    proj[..., -2 * H:] *= 3.0                        # gates over their whole range, the caps included
    bg = torch.randn(2 * H, generator=g)
    bg[H:] += 2.0
    x = proj.double().sum(0)
    o_k, o_v, o_g, o_i = H * D, 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V
    gi = P.capped(x[:, o_i:o_i + H] + bg[:H].double(), cap)
    gf = torch.nn.functional.logsigmoid(P.capped(x[:, o_i + H:] + bg[H:].double(), cap))
    want = torch.zeros(T, H, V, dtype=F64)
    t0 = 0
    for n in lens:
        st = P.mlstm_zero_state(H, D, V)
        for t in range(t0, t0 + n):
            for h in range(H):
                st[h], want[t, h] = P.mlstm_step(st[h], x[t, h * D:(h + 1) * D] * D ** -0.5, x[t, o_k + h * D:o_k + (h + 1) * D],
                                                 x[t, o_v + h * V:o_v + (h + 1) * V], gi[t, h], gf[t, h])
        t0 += n
    size = H * (D * V + D + 1)
    scale = float(want.abs().max())

    def run(pieces, slots_of):
        """pieces: list of batches, a batch a list of (request, first token, count)."""
        state = torch.full((5, size), 7.0, device=DEV)
        for s in slots_of:
            state[s].zero_()
        out = torch.zeros(T, H, V, dtype=F64)
        starts = [0, lens[0], lens[0] + lens[1]]
        for batch in pieces:
            rows = [starts[r] + a + i for r, a, c in batch for i in range(c)]
            seq = [0]
            for r, a, c in batch:
                seq.append(seq[-1] + c)
            slot = torch.tensor([slots_of[r] for r, a, c in batch for _ in range(c)], dtype=torch.int32, device=DEV)
            o = torch.zeros(len(rows), H * V, device=DEV)
            single = all(c == 1 for _, _, c in batch)
            gate = ops.mlstm_scan(proj[:, rows].contiguous().to(DEV), bg.to(DEV), slot,
                                  None if single else torch.tensor(seq, dtype=torch.int32, device=DEV), len(batch), state, o, H, D, V, cap)
            assert torch.equal(gate.cpu(), proj[:, rows].sum(0)[:, o_g:o_i]) or (gate.cpu() - proj[:, rows].sum(0)[:, o_g:o_i]).abs().max() < 1e-5
            out[rows] = o.cpu().double().view(len(rows), H, V)
        assert float(state[4].min()) == 7.0          # a slot nobody used is untouched
        return out
    slots = [3, 0, 2]
    whole = run([[(0, 0, 23), (1, 0, 1), (2, 0, 40)]], slots)
    assert (whole - want).abs().max() < 2e-5 * max(scale, 1.0)
    cut = run([[(0, 0, 2), (2, 0, 17)], [(2, 17, 1), (0, 2, 1), (1, 0, 1)], [(0, 3, 20), (2, 18, 2)], [(2, 20, 19)], [(2, 39, 1)]], slots)
    assert (cut - want).abs().max() < 2e-5 * max(scale, 1.0)
    ones = run([[(0, i, 1), (2, i, 1)] + ([(1, 0, 1)] if i == 0 else []) for i in range(23)] + [[(2, i, 1)] for i in range(23, 40)], slots)
    assert (ones - want).abs().max() < 2e-5 * max(scale, 1.0)
    # the norm, the scale and the output gate
    nw = torch.randn(H * V, generator=g)
    gate = torch.randn(T, H * V + 5, generator=g)[:, 2:2 + H * V]
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        out = torch.zeros(T, H * V, dtype=dt, device=DEV)
        ops.mlstm_finish(want.float().reshape(T, H * V).to(DEV), gate.to(DEV), nw.to(DEV), 1e-5, out, H, V)
        y = P.unit_rms(want.float().double(), 1e-5).reshape(T, H * V) * nw.double() * torch.sigmoid(gate.double())
        assert (out.cpu().double() - y).abs().max() < tol * float(y.abs().max())


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,extra", [(16, 1, 1), (5, 2, 1), (3, 1, 0), (4, 3, 1), (64, 6, 0), (200, 16, 1)])
def test_sigmoid_router(ops, wdtype, E, top, extra):
    g = torch.Generator().manual_seed(E + top)
    T, Hd = 45, 72
    x = torch.randn(T, Hd, generator=g)
    w = (torch.randn(E + extra, Hd, generator=g) * 0.4).to(wdtype)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    scores, weights = torch.zeros(T, top, device=DEV), torch.zeros(T, top + extra, device=DEV)
    logits = torch.zeros(T, E + extra, device=DEV)
    ops.router_sigmoid(x.to(DEV), w.to(DEV), E, top, ids, scores, weights, logits)
    wd = {"r.router": w[:E].double()}
    idx, val, z = P.sigmoid_router(x.double(), wd, "r.", top)
    assert (logits.cpu().double()[:, :E] - z).abs().max() < 1e-4
    assert torch.equal(ids.cpu().long(), idx)
    assert (scores.cpu().double() - val).abs().max() < 1e-5
    assert torch.all(weights.cpu()[:, :top] == 1.0)
    if extra:
        assert (weights.cpu().double()[:, top] - torch.sigmoid(x.double() @ w[E].double())).abs().max() < 1e-5


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H", [(41, 72), (5, 2048), (300, 2048)])     # a block a row; a cluster of blocks a row; many rows
@pytest.mark.parametrize("E,top,extra", [(16, 1, 1), (5, 2, 0), (64, 6, 1)])
def test_sigmoid_router_rides_on_the_norm(ops, wdtype, T, H, E, top, extra):
    """The norm's kernel fills a routing request for the sigmoid rule: the same experts, scores and gate as the plain
    rule on the plain norm (scale stored as an offset from one) of the rows."""
    from flint_b200.parts.base import RouterRequest
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=g)
    offset = 0.1 * torch.randn(H, generator=g)
    wr = (torch.randn(E + extra, H, generator=g) * (3.0 / math.sqrt(H))).to(wdtype)
    req = RouterRequest(wr.to(DEV), 0.0, torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV),
                        logits=torch.zeros(T, E + extra, device=DEV), top=top, rule="sigmoid", extra=extra,
                        weights=torch.zeros(T, top + extra, device=DEV))
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    ops.row_norm(x.clone().to(DEV), (1.0 + offset).to(DEV), None, 1e-5, "rms", out_bf16=out, router=req)
    n = P.offset_rms_norm(x.double(), offset.double(), 1e-5)
    assert (out.cpu().double() - n).abs().max() < 3e-2
    idx, val, z = P.sigmoid_router(n, {"r.router": wr[:E].double()}, "r.", top)
    assert (req.logits.cpu().double()[:, :E] - z).abs().max() < 2e-4
    same = int((req.expert_ids.cpu().long() == idx).all(-1).sum())
    assert same >= T - 2                        # elsewhere two scores are within rounding of each other
    rows = (req.expert_ids.cpu().long() == idx).all(-1)
    assert (req.gates.cpu().double()[rows] - val[rows]).abs().max() < 1e-4
    assert torch.all(req.weights.cpu()[:, :top] == 1.0)
    if extra:
        assert (req.weights.cpu().double()[:, top] - torch.sigmoid(n @ wr[E].double())).abs().max() < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_activation_with_scores_and_the_clamped_gated_unit(ops, dtype):
    g = torch.Generator().manual_seed(5)
    T, top, N = 19, 2, 24
    parts = torch.randn(3, T * top, N, generator=g)
    row_of = torch.randperm(T * top, generator=g).to(torch.int32).view(T, top)
    scale = torch.rand(T, top + 1, generator=g)
    out = torch.zeros(T * top, N, dtype=dtype, device=DEV)
    ops.row_act(parts.to(DEV), out, "gelu", row_of=row_of.to(DEV), row_scale=scale.to(DEV))
    s = torch.zeros(T * top, dtype=F64)
    s[row_of.view(-1).long()] = scale[:, :top].reshape(-1).double()
    want = P.gelu_erf(parts.double().sum(0) * s[:, None])
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (out.cpu().double() - want).abs().max() < tol * 4
    ops.row_act(parts.to(DEV), out, "gelu")
    assert (out.cpu().double() - P.gelu_erf(parts.double().sum(0))).abs().max() < tol * 4
    # the clamped unit through the product: weights large enough that both clamps bite
    K, I = 40, 24
    x = torch.randn(T, K, generator=g).to(dtype)
    wg, wu, wd = (torch.randn(I, K, generator=g) * 0.5).to(dtype), (torch.randn(I, K, generator=g) * 0.5).to(dtype), torch.eye(I, dtype=F64)
    a = torch.zeros(T, I, dtype=dtype, device=DEV)
    ops.gated_gemm(x.to(DEV), ops.pair_gate_up(wg, wu).contiguous().to(DEV), a, "swish_clamped", act_params=(1.702, 1.5))
    want = P.clamped_glu(x.double(), {"m.gate": wg.double(), "m.up": wu.double(), "m.down": wd}, "m.", 1.5)
    assert float((x.double() @ wg.double().T).max()) > 1.5 and float((x.double() @ wu.double().T).min()) < -1.5
    assert (a.cpu().double() - want).abs().max() < tol * 8


# ------------------------------------------------------------------------------------------------ the whole model

@pytest.fixture(scope="module", params=["G1", "G2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("gepadra") / which, cfg, seed=3)
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, dtype, page_size=64, record=False):
    rp = Replayer(folder, dtype=dtype, max_tokens=traces.max_tokens_needed(steps), page_size=page_size, max_requests=4, device=DEV)
    out, recs = {}, {}
    for s in steps:
        rec = {} if record else None
        lg = rp.run_step(s["entries"], s["end"], record=rec)
        if lg is not None:
            out[s["step"]] = lg
        if record:
            recs[s["step"]] = {k: [t.cpu() for t in v] for k, v in rec.items()}
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, recs, rp


def followed(cfg, w, reqs, folder, dtype):
    """The plain implementation run with the experts the engine chose for the whole prompts (in bfloat16 a
    near-tie of two router scores may fall the other way).  Also returns how many (row, layer) choices differ
    from what the plain router would choose on the same rows, and the largest gap in score that such a
    difference bridges."""
    steps = traces.whole(reqs)
    _, recs, _ = replay(folder, steps, dtype, record=True)
    routed = [i for i, l in enumerate(cfg["layers"]) if l.get("mlp") and l["mlp"]["kind"] == "moe"]
    out, flips, gap = {}, 0, 0.0
    for s in steps:
        rid = s["entries"][0]["id"]
        ex = recs[s["step"]]["experts"]
        keep = {}
        out[rid] = P.forward(cfg, w, reqs[rid], forced_experts={i: ex[k] for k, i in enumerate(routed)}, keep=keep)
        for k, i in enumerate(routed):
            score = torch.sigmoid(keep["router_logits"][i])
            top = ex[k].shape[1]
            own = torch.topk(score, top, dim=-1)
            for t in range(score.shape[0]):
                if set(own.indices[t].tolist()) != set(ex[k][t].tolist()):
                    flips += 1
                    gap = max(gap, float(own.values[t].min() - score[t][ex[k][t].long()].min()))
    return out, flips, gap


def rel_err(got, want):
    d = got.double() - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp(min=1e-6))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain_under_every_cut(setup, dtype):
    which, cfg, folder, w, reqs, plain = setup
    if dtype == "bfloat16":
        base, flips, gap = followed(cfg, w, reqs, folder, dtype)
        assert flips <= 0.03 * sum(LENGTHS) * len(cfg["layers"]) and gap < 0.03, \
            f"the engine's experts differ from the plain choice at {flips} places, by up to {gap:.3g} in score"
    else:
        base = plain
    limit = 1e-4 if dtype == "float32" else 5e-2
    cuts = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=24), "portions": traces.portions,
            "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128)), "mixed": lambda r: traces.mixed(r, seed=3)}
    for name, cut in cuts.items():
        steps = cut(reqs)
        out, _, rp = replay(folder, steps, dtype, page_size=16 if name == "mixed" else 64)
        exp = traces.expected_rows(steps, base)
        assert set(out) == set(exp)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        bad = int((errs > limit).sum())
        assert bad <= (0 if dtype == "float32" else 0.03 * len(errs)), f"{name}: {bad} of {len(errs)} rows, worst {float(errs.max()):.3g}"
        if name == "mixed":
            assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


def test_long_decoding_token_by_token(setup):
    """Two requests decoded side by side, one token a step each, over several pages and past every window, after
    prompts of unequal length: the captured decode step is replayed many times and the matrix memory is carried
    through all of them."""
    which, cfg, folder, w, reqs, plain = setup
    a, b = reqs["r5"], reqs["r4"]
    rp = Replayer(folder, dtype="float32", max_tokens=512, page_size=16, max_requests=2, device=DEV)
    rp.run_step([{"id": "a", "tokens": a[:40], "want": []}, {"id": "b", "tokens": b[:3], "want": []}])
    worst = 0.0
    for i in range(66):
        out = rp.run_step([{"id": "a", "tokens": [a[40 + i]], "want": [0]}, {"id": "b", "tokens": [b[3 + i]], "want": [0]}])
        worst = max(worst, float(rel_err(out, torch.stack([plain["r5"][40 + i], plain["r4"][3 + i]])).max()))
    assert worst < 1e-4
    assert len(rp.model._graphs) >= 1


def test_greedy_generation_through_the_entry_point(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(12):
            lg = P.forward(cfg, w, toks)[-1]
            t = int(torch.argmax(lg))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages in (16, 3):
        m = load_model(folder, dtype="float32", device=DEV, page_size=16, n_pages=n_pages, max_slots=4, max_step_tokens=24,
                       max_context=256)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        assert eng.generate(prompts, 12) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(setup, tmp_path, dtype):
    """bin/trace_run in a process of its own, fed a mixed trace over standard input."""
    which, cfg, folder, w, reqs, plain = setup
    steps = traces.mixed(reqs, seed=5)
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, f"{REPO}/bin/trace_run", "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(traces.max_tokens_needed(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l] == [f"done {s['step']}" for s in steps]
    exp = traces.expected_rows(steps, plain)
    errs = []
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        n = sum(len(e["want"]) for e in s["entries"])
        assert f.exists() == (n > 0)
        if n:
            got = torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(n, cfg["vocab"]))
            errs.append(rel_err(got, torch.stack(exp[s["step"]])))
    errs = torch.cat(errs)
    if dtype == "float32":
        assert float(errs.max()) < 1e-4
    else:       # a near-tie of two router scores may fall the other way at a few rows
        assert int((errs > 5e-2).sum()) <= 0.08 * len(errs) and float(errs.median()) < 2.5e-2


def test_chat_program_with_random_weights(tmp_path):
    """bin/flint_chat with ``--random-config FILE --seed N``, token ids in and out, greedy: the tokens of the folder
    that the random-weights mode writes for that configuration and seed, under the plain implementation."""
    from flint_b200.engine.loading import write_random_model
    from flint_b200.weights.safetensors_io import SafetensorsFile
    seed, cfg = 4, tiny.G1
    folder = write_random_model(tmp_path / "model", cfg, seed=seed)
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.read(n).double() for n in f.names()}
    prompt = [3, 50, 50, 7, 90, 0, 12, 13, 14, 15, 16]
    cfg_file = tmp_path / "only_config.json"
    cfg_file.write_text(json.dumps(cfg))
    proc = subprocess.run([sys.executable, f"{REPO}/bin/flint_chat", "--random-config", str(cfg_file), "--prompt", " ".join(map(str, prompt)),
                           "--max-tokens", "8", "--temperature", "0", "--seed", str(seed), "--dtype", "float32", "--ctx-size", "128"],
                          capture_output=True, text=True, timeout=600, env={**os.environ, "VERIFY_IDS": "1"})
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(x) for x in proc.stdout.split()]
    toks, want = list(prompt), []
    for _ in range(8):
        t = int(torch.argmax(P.forward(cfg, w, toks)[-1]))
        want.append(t)
        toks.append(t)
    assert got == want
