"""Puledra on the GPU: each new kernel beside the plain function of its mechanism (planted keys far away, at
page borders and at a window's edges; router groups; pair-table state), and the whole model under every cut,
in long decoding and in generation, beside the plain implementation."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_puledra as P
import tiny_puledra as tiny
import traces
from flint_b200.cache.manager import CacheView, KVSpec
from flint_b200.engine.engine import Engine
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.parts.base import Pending
from flint_b200.sampling.params import SamplingParams

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from flint_b200.csrc.ops import get_ops
    return get_ops(DEV)


def paged_rows(rows_by_slot, row_w, P_, dtype, seed=0):
    """A latent cache whose pages lie in a shuffled order: (view, dense rows per slot as float64)."""
    rnd = random.Random(seed)
    n_pages = sum(-(-len(r) // P_) for r in rows_by_slot) + 3
    order = list(range(n_pages))
    rnd.shuffle(order)
    k = torch.zeros(n_pages, 1, P_, row_w, dtype=dtype)
    bt = torch.full((len(rows_by_slot), max(-(-len(r) // P_) for r in rows_by_slot) + 1), -1, dtype=torch.int32)
    for s, rows in enumerate(rows_by_slot):
        for j in range(len(rows)):
            if j % P_ == 0:
                bt[s, j // P_] = order.pop()
            k[bt[s, j // P_], 0, j % P_, :rows.shape[1]] = rows[j].to(dtype)
    dense = [k[bt[s, torch.arange(len(r)) // P_].long(), 0, torch.arange(len(r)) % P_].double() for s, r in enumerate(rows_by_slot)]
    view = CacheView(k.to(DEV), torch.zeros(n_pages, 1, P_, 0, dtype=dtype, device=DEV), bt.to(DEV), P_, KVSpec(1, row_w, 0, 0))
    return view, dense


def dense_latent_attention(qa, dense, pos, slot, C, Dk, scale, window=0):
    out = torch.zeros(qa.shape[0], qa.shape[1], C, dtype=torch.float64)
    for t in range(qa.shape[0]):
        p = int(pos[t])
        lo = max(0, p + 1 - window) if window else 0
        k = dense[int(slot[t])][lo:p + 1]
        s = (qa[t].double() @ k[:, :Dk].T) * scale
        out[t] = torch.softmax(s, -1) @ k[:, :C]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,R,H", [(40, 8, 5), (20, 6, 1), (128, 32, 9)])
def test_latent_attention_finds_planted_keys(ops, dtype, C, R, H):
    """Every query is aimed at one key (its score stands out by far): keys far back, on both sides of page
    borders, the first tokens, the query's own position.  The output must be that key's latent."""
    P_, Dk = 16, C + R
    row_w = -(-Dk // 8) * 8
    lens = (300, 50)
    rows = [torch.randn(n, Dk) for n in lens]
    view, dense = paged_rows(rows, row_w, P_, dtype)
    cases = [(0, 299, 3), (0, 299, 0), (0, 299, 15), (0, 299, 16), (0, 299, 255), (0, 299, 256), (0, 299, 299),
             (0, 16, 16), (0, 16, 15), (0, 15, 0), (0, 0, 0), (0, 17, 1), (1, 49, 2), (1, 49, 48), (1, 32, 31), (0, 256, 17)]
    pos = torch.tensor([c[1] for c in cases], dtype=torch.int32)
    slot = torch.tensor([c[0] for c in cases], dtype=torch.int32)
    qa = torch.randn(len(cases), H, Dk) * 0.1
    for t, (s, p, j) in enumerate(cases):
        aim = dense[s][j, :Dk].float()
        qa[t] += 40.0 * aim / (aim.norm() ** 2)            # the planted key's score is about 40 above the rest
    qa = qa.to(dtype)
    step = SimpleNamespace(pos=pos.to(DEV), slot=slot.to(DEV), max_kv_len=300)
    exp = dense_latent_attention(qa.cpu(), dense, pos, slot, C, Dk, 1.0)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    kernels = ("simt",) if dtype == torch.float32 else ("simt", "mma")
    for kernel in kernels:
        for splits in (None, (64, 5), (304, 1), (32, 10)):
            out = torch.zeros(len(cases), H, C, dtype=dtype, device=DEV)
            ops.latent_attention(qa.to(DEV), view, step, out, H, C, 0, 1.0, splits=splits, kernel=kernel)
            assert (out.double().cpu() - exp).abs().max() < tol, (kernel, splits)
            for t, (s, p, j) in enumerate(cases):                # and it is the planted key's latent, not a neighbour's
                assert (out[t].double().cpu() - dense[s][j, :C]).abs().max() < 5e-2 + tol
    # a list of rows: the others stay as they were
    out = torch.full((len(cases), H, C), 7.0, dtype=dtype, device=DEV)
    some = torch.tensor([1, 4, 12], dtype=torch.int32, device=DEV)
    ops.latent_attention(qa.to(DEV), view, step, out, H, C, 0, 1.0, rows=some)
    keep = torch.ones(len(cases), dtype=torch.bool)
    keep[some.cpu().long()] = False
    assert (out.cpu()[keep] == 7.0).all() and (out.double().cpu()[~keep] - exp[~keep]).abs().max() < tol


@pytest.mark.parametrize("C,R,H", [(40, 8, 5), (64, 32, 6), (256, 64, 40), (512, 64, 16)])
def test_latent_attention_tiles_of_consecutive_tokens(ops, C, R, H):
    """The tensor-core kernel on portions of prompts: blocks hold several tokens of one request (each with its
    own causal limit), the last tokens of one request beside the first of the next, and decoded tokens."""
    P_, Dk = 16, C + R
    row_w = -(-Dk // 8) * 8
    lens = (150, 90, 40)
    rows = [torch.randn(n, Dk) for n in lens]
    view, dense = paged_rows(rows, row_w, P_, torch.bfloat16, seed=2)
    # portions: slot 0 positions 100..149, slot 1 positions 0..89, slot 2 position 39 alone
    pos = torch.tensor(list(range(100, 150)) + list(range(0, 90)) + [39], dtype=torch.int32)
    slot = torch.tensor([0] * 50 + [1] * 90 + [2], dtype=torch.int32)
    T = len(pos)
    qa = (torch.randn(T, H, Dk) * (2.0 / math.sqrt(Dk))).to(torch.bfloat16)
    exp = dense_latent_attention(qa, dense, pos, slot, C, Dk, 1.0)
    step = SimpleNamespace(pos=pos.to(DEV), slot=slot.to(DEV), max_kv_len=150, entries=[0, 1, 2])
    for splits in (None, (64, 3), (192, 1)):
        out = torch.zeros(T, H, C, dtype=torch.bfloat16, device=DEV)
        ops.latent_attention(qa.to(DEV), view, step, out, H, C, 0, 1.0, splits=splits, kernel="mma")
        assert (out.double().cpu() - exp).abs().max() < 3e-2, splits
    ref = torch.zeros(T, H, C, dtype=torch.bfloat16, device=DEV)
    ops.latent_attention(qa.to(DEV), view, step, ref, H, C, 0, 1.0, kernel="simt")
    assert (ref.double().cpu() - exp).abs().max() < 3e-2
    # decoded tokens: one token a request
    pos1 = torch.tensor([149, 89, 39], dtype=torch.int32)
    slot1 = torch.tensor([0, 1, 2], dtype=torch.int32)
    q1 = qa[[49, 139, 140]].contiguous()
    step1 = SimpleNamespace(pos=pos1.to(DEV), slot=slot1.to(DEV), max_kv_len=150, entries=[0, 1, 2])
    out = torch.zeros(3, H, C, dtype=torch.bfloat16, device=DEV)
    ops.latent_attention(q1.to(DEV), view, step1, out, H, C, 0, 1.0, kernel="mma")
    assert (out.double().cpu() - exp[[49, 139, 140]]).abs().max() < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_window_edges(ops, dtype):
    """With a window the key just inside is seen and the key just outside is not (the mixer's window is a
    parameter; Puledra's layers use none)."""
    C, R, H, P_, W = 24, 8, 3, 16, 20
    Dk = C + R
    rows = [torch.randn(100, Dk)]
    view, dense = paged_rows(rows, Dk, P_, dtype)
    pos = torch.tensor([99, 99, 40, 40, 19, 20], dtype=torch.int32)
    aims = [99 - W + 1, 99 - W, 40 - W + 1, 40 - W, 0, 0]            # inside, outside, inside, outside, inside, outside
    slot = torch.zeros(6, dtype=torch.int32)
    qa = torch.zeros(6, H, Dk)
    for t, j in enumerate(aims):
        aim = dense[0][j, :Dk].float()
        qa[t] = 40.0 * aim / (aim.norm() ** 2)
    qa = qa.to(dtype)
    step = SimpleNamespace(pos=pos.to(DEV), slot=slot.to(DEV), max_kv_len=100)
    exp = dense_latent_attention(qa.cpu(), dense, pos, slot, C, Dk, 1.0, window=W)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for kernel in (("simt",) if dtype == torch.float32 else ("simt", "mma")):
        out = torch.zeros(6, H, C, dtype=dtype, device=DEV)
        ops.latent_attention(qa.to(DEV), view, step, out, H, C, W, 1.0, kernel=kernel)
        assert (out.double().cpu() - exp).abs().max() < tol
        for t, j in enumerate(aims):
            hit = (out[t].double().cpu() - dense[0][j, :C]).abs().max() < 5e-2 + tol
            assert bool(hit) == (t % 2 == 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style,rot_dims", [("interleaved", 8), ("interleaved", 4), ("half", 8), ("interleaved", 0)])
def test_latent_prepare(ops, dtype, style, rot_dims):
    H, D, R, C, T, P_, S = 3, 10, 8, 20, 37, 16, 3
    row_w = 32
    W = H * (D + R) + C + R
    proj = torch.randn(S, T, W)
    total = proj.double().sum(0)
    pos = torch.tensor([(5 * t + 3) % 64 for t in range(T)], dtype=torch.int32)
    pos[0] = 0
    slot = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    pos = pos + 0
    # distinct (slot, position) pairs so that every row has a cache row of its own
    seen = set()
    for t in range(T):
        while (int(slot[t]), int(pos[t])) in seen:
            pos[t] = (int(pos[t]) + 1) % 64
        seen.add((int(slot[t]), int(pos[t])))
    half = max(rot_dims // 2, 1)
    i = torch.arange(half, dtype=torch.float64)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * (300.0 ** (-2.0 * i / max(rot_dims, 1)))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    norm_w = 1.0 + 0.1 * torch.randn(C)
    view, _ = paged_rows([torch.zeros(64, row_w), torch.zeros(64, row_w)], row_w, P_, dtype)
    q_plain = torch.zeros(T, H, D, dtype=dtype, device=DEV)
    qa = torch.zeros(T, H, C + R, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.latent_prepare(proj.to(DEV), pos.to(DEV), slot.to(DEV), cos.to(DEV), sin.to(DEV), rot_dims, style, norm_w.to(DEV),
                       1e-5, q_plain, qa, view, H, D, R, C, True, status)
    assert int(status.item()) == 0

    def rotate(v):
        if rot_dims == 0:
            return v
        if style == "interleaved":
            return P.rotate_pairs(v, pos.tolist(), 300.0, rot_dims)
        c = torch.cos(ang)[pos.long()].view([T] + [1] * (v.dim() - 2) + [half])
        s = torch.sin(ang)[pos.long()].view([T] + [1] * (v.dim() - 2) + [half])
        a, b = v[..., :half], v[..., half:rot_dims]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., rot_dims:]], -1)
    q = total[:, :H * (D + R)].view(T, H, D + R)
    tol = 1e-5 if dtype == torch.float32 else 4e-2
    assert (q_plain.double().cpu() - q[..., :D]).abs().max() < tol
    assert (qa.double().cpu()[..., C:] - rotate(q[..., D:].contiguous())).abs().max() < tol
    lat = total[:, H * (D + R):]
    c_exp = P.rms_norm(lat[:, :C], norm_w.double(), 1e-5)
    r_exp = rotate(lat[:, C:].contiguous())
    bt = view.block_table.cpu()
    got = view.k.cpu()[bt[slot.long(), (pos // P_).long()].long(), 0, (pos % P_).long()].double()
    assert (got[:, :C] - c_exp).abs().max() < tol and (got[:, C:C + R] - r_exp).abs().max() < tol
    assert (got[:, C + R:] == 0).all()
    # a layer that reads another's latent: only the queries, nothing written
    before = view.k.clone()
    ops.latent_prepare(proj[:, :, :H * (D + R)].contiguous().to(DEV), pos.to(DEV), slot.to(DEV), cos.to(DEV), sin.to(DEV),
                       rot_dims, style, None, 1e-5, q_plain, qa, None, H, D, R, C, False, status)
    assert torch.equal(before, view.k)


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 3, 2), (8, 2, 4, 2), (6, 1, 1, 1), (16, 4, 2, 1), (4, 4, 2, 2), (64, 6, 8, 3)])
def test_router_topk(ops, wdtype, E, top, groups, keep):
    T, H = 41, 72
    x = torch.randn(T, H)
    wr = (torch.randn(E, H) * 0.3).to(wdtype)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    gates = torch.zeros(T, top, dtype=torch.float32, device=DEV)
    logits = torch.zeros(T, E, dtype=torch.float32, device=DEV)
    ops.router_topk(x.to(DEV), wr.to(DEV), top, groups, keep, 1.7, ids, gates, logits)
    z = x.double() @ wr.double().T
    assert (logits.double().cpu() - z).abs().max() < 1e-4
    for t in range(T):
        e_ids, e_w = P.route(z[t], top, groups, keep, 1.7)
        assert ids[t].tolist() == e_ids
        assert (gates[t].double().cpu() - torch.tensor(e_w)).abs().max() < 1e-5


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H", [(41, 72), (5, 2048), (300, 2048)])     # a block a row; a cluster of blocks a row; many rows
@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 3, 2), (64, 6, 8, 3), (6, 1, 1, 1)])
def test_router_rides_on_the_norm(ops, wdtype, T, H, E, top, groups, keep):
    """The norm's kernel fills a routing request for the grouped softmax rule: the same experts and gates as the
    plain rule on the plain norm of the rows."""
    from flint_b200.parts.base import RouterRequest
    x = torch.randn(T, H)
    gamma = 1.0 + 0.1 * torch.randn(H)
    wr = (torch.randn(E, H) * (3.0 / math.sqrt(H))).to(wdtype)
    req = RouterRequest(wr.to(DEV), 0.0, torch.zeros(T, top, dtype=torch.int32, device=DEV),
                        torch.zeros(T, top, dtype=torch.float32, device=DEV),
                        logits=torch.zeros(T, E, dtype=torch.float32, device=DEV), top=top, groups=groups, keep=keep, scale=2.5)
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    ops.row_norm(x.clone().to(DEV), gamma.to(DEV), None, 1e-5, "rms", out_bf16=out, router=req)
    n = P.rms_norm(x.double(), gamma.double(), 1e-5)
    z = n @ wr.double().T
    assert (req.logits.double().cpu() - z).abs().max() < 2e-4
    same = 0
    for t in range(T):
        e_ids, e_w = P.route(z[t], top, groups, keep, 2.5)
        if req.expert_ids[t].tolist() == e_ids:
            same += 1
            assert (req.gates[t].double().cpu() - torch.tensor(e_w)).abs().max() < 1e-4
        else:       # only where two scores are within rounding of each other
            e2, _ = P.route(req.logits[t].double().cpu(), top, groups, keep, 2.5)
            assert req.expert_ids[t].tolist() == e2
    assert same >= T - 2


@pytest.mark.parametrize("H", [64, 50, 4096])
def test_pending_rows_of_three_experts_join_the_norm(ops, H):
    T, k, S = 19, 3, 2
    x = torch.randn(T, H)
    y = torch.randn(k * T, H)
    row_of = torch.randperm(k * T).to(torch.int32).view(T, k)
    gates = torch.rand(T, k)
    parts = torch.randn(S, T, H)
    gamma = 1.0 + 0.1 * torch.randn(H)
    xd = x.clone().to(DEV)
    out = torch.zeros(T, H, device=DEV)
    pend = Pending(partials=parts.to(DEV), y=y.to(DEV), row_of=row_of.to(DEV), gates=gates.to(DEV))
    ops.row_norm(xd, gamma.to(DEV), None, 1e-5, "rms", out_f32=out, pending=pend)
    exp_x = x.double() + parts.double().sum(0) + sum(gates[:, i:i + 1].double() * y.double()[row_of[:, i].long()] for i in range(k))
    assert (xd.double().cpu() - exp_x).abs().max() < 1e-4
    assert (out.double().cpu() - P.rms_norm(exp_x, gamma.double(), 1e-5)).abs().max() < 1e-4


def test_pair_table_kernel_keeps_each_request_s_newest_token(ops):
    H, buckets, mp, mc = 24, 53, 31, 5
    table = torch.randn(buckets + 1, H)
    last = torch.full((4,), 12345, dtype=torch.int32, device=DEV)        # stale state must not matter at position 0
    seqs = {2: [4, 9, 9, 50, 1, 7], 0: [3, 3, 8], 3: [60, 2, 11, 5]}

    def run(entries, fed=None):
        ids = torch.tensor([t for _, _, toks in entries for t in toks], dtype=torch.int32, device=DEV)
        pos = torch.tensor([p0 + i for _, p0, toks in entries for i in range(len(toks))], dtype=torch.int32, device=DEV)
        slot = torch.tensor([s for s, _, toks in entries for _ in toks], dtype=torch.int32, device=DEV)
        out = torch.zeros(len(ids), H, device=DEV)
        kw = {}
        if fed is not None:
            kw = {"fed_rows": torch.tensor(fed[0], dtype=torch.int32, device=DEV),
                  "fed_from": torch.tensor(fed[1], dtype=torch.int32, device=DEV)}
        ops.pair_embed_add(ids, pos, slot, last, table.to(DEV), out, mp, mc, **kw)
        return out.cpu()
    exp = {s: table[torch.tensor(P.bigram_rows(t, buckets, mp, mc))] for s, t in seqs.items()}
    out = run([(2, 0, seqs[2][:3]), (0, 0, seqs[0][:1])])
    assert torch.equal(out[:3], exp[2][:3]) and torch.equal(out[3:], exp[0][:1])
    out = run([(0, 1, seqs[0][1:2]), (3, 0, seqs[3][:2]), (2, 3, seqs[2][3:4])])
    assert torch.equal(out[0:1], exp[0][1:2]) and torch.equal(out[1:3], exp[3][:2]) and torch.equal(out[3:], exp[2][3:4])
    # tokens that are still on the device (sampled, not read): row 0 takes its token from place 1 of the feed
    out = run([(2, 4, [0]), (0, 2, seqs[0][2:3])], fed=([1, -1], [99, seqs[2][4]]))
    assert torch.equal(out[0:1], exp[2][4:5]) and torch.equal(out[1:2], exp[0][2:3])
    out = run([(2, 5, seqs[2][5:6])])
    assert torch.equal(out, exp[2][5:6])
    assert last.tolist()[2] == 7 and last.tolist()[0] == 8 and last.tolist()[3] == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [21, 5, 1, 70])            # many tokens, and the few of a decode step
def test_head_products(ops, dtype, T):
    H, K, N = 5, 24, 40
    wide = torch.randn(T, H, K + 8).to(dtype)
    w = torch.randn(H, N, K).to(dtype)
    out_wide = torch.zeros(T, H, N + 16, dtype=dtype, device=DEV)
    ops.head_products(wide.to(DEV)[:, :, :K], w.to(DEV), out_wide[:, :, :N])
    exp = torch.einsum("thk,hnk->thn", wide[:, :, :K].double(), w.double())
    tol = 1e-4 if dtype == torch.float32 else 0.15
    assert (out_wide[:, :, :N].double().cpu() - exp).abs().max() < tol and (out_wide[:, :, N:] == 0).all()


# ------------------------------------------------------------------------------------------------ whole model

LENGTHS = (1, 2, 9, 37, 70, 130, 333)


@pytest.fixture(scope="module", params=["P1", "P2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("puledra") / which, cfg, seed=3)
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
    near-tie of two router scores may fall the other way)."""
    steps = traces.whole(reqs)
    _, recs, _ = replay(folder, steps, dtype, record=True)
    with_ffn = [i for i, l in enumerate(cfg["layers"]) if l.get("mlp")]
    out = {}
    for s in steps:
        rid = s["entries"][0]["id"]
        ex = recs[s["step"]]["experts"]
        follow = {i: ex[k].tolist() for k, i in enumerate(with_ffn)}
        out[rid] = P.forward(cfg, w, reqs[rid], follow=follow)
    return out


def rel_err(got, want):
    d = got.double() - want
    d = d - d.mean(-1, keepdim=True)
    c = want - want.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / c.pow(2).mean(-1).sqrt().clamp(min=1e-6))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain_under_every_cut(setup, dtype):
    which, cfg, folder, w, reqs, plain = setup
    if dtype == "bfloat16":
        base = followed(cfg, w, reqs, folder, dtype)
        differ = sum(int((rel_err(base[r], plain[r]) > 1e-6).sum()) for r in reqs)
        assert differ <= 0.05 * sum(LENGTHS), "the engine's experts differ from the plain choice at too many rows"
    else:
        base = plain
    limit = 1e-4 if dtype == "float32" else 4e-2
    cuts = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=24), "portions": traces.portions,
            "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3, 128)), "mixed": lambda r: traces.mixed(r, seed=3)}
    for name, cut in cuts.items():
        steps = cut(reqs)
        out, _, rp = replay(folder, steps, dtype, page_size=16 if name == "mixed" else 64)
        exp = traces.expected_rows(steps, base)
        assert set(out) == set(exp)
        errs = torch.cat([rel_err(out[k], torch.stack(rows)) for k, rows in exp.items()])
        bad = int((errs > limit).sum())
        assert bad <= (0 if dtype == "float32" else 0.02 * len(errs)), f"{name}: {bad} of {len(errs)} rows, worst {float(errs.max()):.3g}"
        if name == "mixed":
            assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


def test_long_decoding_token_by_token(setup):
    """Two requests decoded side by side, one token a step each, over several pages, after prompts of unequal
    length: the captured decode step is replayed hundreds of times."""
    which, cfg, folder, w, reqs, plain = setup
    a, b = reqs["r6"], reqs["r5"]
    rp = Replayer(folder, dtype="float32", max_tokens=512, page_size=16, max_requests=2, device=DEV)
    rp.run_step([{"id": "a", "tokens": a[:40], "want": []}, {"id": "b", "tokens": b[:3], "want": []}])
    worst = 0.0
    for i in range(127):
        out = rp.run_step([{"id": "a", "tokens": [a[40 + i]], "want": [0]}, {"id": "b", "tokens": [b[3 + i]], "want": [0]}])
        worst = max(worst, float(rel_err(out, torch.stack([plain["r6"][40 + i], plain["r5"][3 + i]])).max()))
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
            top2 = torch.topk(lg, 2).values
            assert float(top2[0] - top2[1]) > 1e-3, "the test's own choice is a near-tie"
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


# ------------------------------------------------------------------------------------------------ the programs

REPO = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(setup, tmp_path, dtype):
    """bin/trace_run in a process of its own, fed a mixed trace over standard input."""
    import json
    import subprocess
    import sys
    import numpy as np
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
        assert int((errs > 4e-2).sum()) <= 0.05 * len(errs) and float(errs.median()) < 2e-2


@pytest.mark.parametrize("source", ["folder", "random-config"])
def test_chat_program_prints_the_plain_arg_max_tokens(tmp_path, source):
    """bin/flint_chat, token ids in and out, greedy: from a model folder, and with ``--random-config FILE --seed N``,
    which must give the tokens of the folder that the random-weights mode writes for that configuration and seed."""
    import json
    import os
    import subprocess
    import sys
    from flint_b200.engine.loading import write_random_model
    seed = 4
    cfg = tiny.P1
    folder = write_random_model(tmp_path / "model", cfg, seed=seed)
    prompt = [3, 50, 50, 7, 96, 0, 12, 13, 14, 15, 16]
    if source == "folder":
        where = ["--model", str(folder)]
    else:
        cfg_file = tmp_path / "only_config.json"
        cfg_file.write_text(json.dumps(cfg))
        where = ["--random-config", str(cfg_file)]
    proc = subprocess.run([sys.executable, f"{REPO}/bin/flint_chat", *where, "--prompt", " ".join(map(str, prompt)), "--max-tokens", "8",
                           "--temperature", "0", "--seed", str(seed), "--dtype", "float32", "--ctx-size", "128"],
                          capture_output=True, text=True, timeout=600, env={**os.environ, "VERIFY_IDS": "1"})
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(x) for x in proc.stdout.split()]
    assert "prefill: 11 tok" in proc.stderr and "decode:" in proc.stderr
    pcfg, w = P.load_model_dir(folder)
    toks, want = list(prompt), []
    for _ in range(8):
        t = int(torch.argmax(P.forward(pcfg, w, toks)[-1]))
        want.append(t)
        toks.append(t)
    assert got == want
