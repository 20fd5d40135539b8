"""Gepadra through the engine's plumbing on the CPU (the kernels replaced by their plain references): the
configuration reader, tensor names, the two-norm block, pages that a window keeps for a request's first tokens,
the matrix memory's state across steps and slots, and replay under every cut against the plain implementation."""
import copy

import pytest
import torch

import plain_gepadra as P
import tiny_gepadra as tiny
import traces
from flint_b200.cache.manager import CacheManager, KVSpec
from flint_b200.engine.engine import Engine
from flint_b200.engine.loading import expected_from_config, write_random_model
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.errors import ConfigError, WeightError
from flint_b200.sampling.params import SamplingParams
from kernel_refs import RefOps

LENGTHS = (1, 2, 9, 37, 70, 130)


@pytest.fixture(scope="module", params=["G1", "G2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("gepadra") / which, cfg, seed=3)
    reqs = traces.make_requests(cfg["vocab"], LENGTHS, seed=7)
    plain = {rid: P.forward(cfg, w, t) for rid, t in reqs.items()}
    return which, cfg, folder, w, reqs, plain


def replay(folder, steps, page_size=16):
    n = traces.max_tokens_needed(steps)
    rp = Replayer(folder, dtype="float32", max_tokens=n, page_size=page_size, max_requests=4, device="cpu", ops=RefOps())
    out = {}
    for s in steps:
        lg = rp.run_step(s["entries"], s["end"])
        if lg is not None:
            out[s["step"]] = lg
        rp.model.cache.check()
    assert all(g.pages.pool.used_pages == 0 for g in rp.model.cache.groups)
    return out, rp


def compare(out, steps, plain, tol=3e-4):
    exp = traces.expected_rows(steps, plain)
    assert set(out) == set(exp)
    for k, rows in exp.items():
        want = torch.stack(rows)
        err = (out[k].double() - want).abs().max().item()
        assert err < tol * max(1.0, float(want.abs().max())), f"step {k}: max error {err:.2e}"


def test_the_plain_mechanisms_hold_their_invariants():
    pos = torch.arange(12)
    seen = P.visible(pos, pos, size=4, keep_first=2)
    assert seen[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]          # the first two and the last four
    assert seen[3].nonzero().flatten().tolist() == [0, 1, 2, 3] and not seen[3, 4]
    assert P.visible(pos, pos, size=4, keep_first=0)[9].nonzero().flatten().tolist() == [6, 7, 8, 9]
    # a sink takes its share of the weights and gives nothing
    s = torch.zeros(1, 1, 3, dtype=torch.float64)
    v = torch.ones(1, 3, 2, dtype=torch.float64)
    full = torch.ones(1, 3, dtype=torch.bool)
    assert torch.allclose(P.sink_softmax_mix(s, torch.tensor([0.0], dtype=torch.float64), v, full), torch.full((1, 1, 2), 0.75, dtype=torch.float64))
    assert torch.allclose(P.sink_softmax_mix(s, torch.tensor([-1e9], dtype=torch.float64), v, full), torch.ones(1, 1, 2, dtype=torch.float64))
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    y = P.rotate_leading_dims(x, torch.arange(5), 100.0, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    assert torch.allclose(y[2, 1, 0] ** 2 + y[2, 1, 4] ** 2, x[2, 1, 0] ** 2 + x[2, 1, 4] ** 2)     # dim i turns with i + dims/2
    # the matrix memory: with the forget gate open and the input gate at its running maximum, one step stores k v^T
    st = P.mlstm_zero_state(1, 3, 2)[0]
    k, v, q = torch.tensor([1.0, 2.0, 0.0], dtype=torch.float64), torch.tensor([3.0, -1.0], dtype=torch.float64), torch.tensor([0.5, 0.5, 1.0], dtype=torch.float64)
    (S, n, m), o = P.mlstm_step(st, q, k, v, torch.tensor(2.0, dtype=torch.float64), torch.tensor(-0.1, dtype=torch.float64))
    assert float(m) == 2.0 and torch.allclose(S, torch.outer(k, v)) and torch.allclose(n, k)
    assert torch.allclose(o, (torch.outer(k, v).T @ q) / (1.5 + 1e-6))
    # a router score scales the expert's input, not its output
    w = {"m.router": torch.tensor([[4.0, 0.0], [0.0, 1.0]], dtype=torch.float64), "m.e0.up": torch.eye(2, dtype=torch.float64),
         "m.e0.down": torch.eye(2, dtype=torch.float64), "m.e1.up": torch.eye(2, dtype=torch.float64), "m.e1.down": torch.eye(2, dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.5]], dtype=torch.float64)
    out, idx, z = P.expert_mixture(h, w, "m.", {"router": {"top": 1}, "expert": {"ff": 2}})
    s0 = torch.sigmoid(torch.tensor(4.0, dtype=torch.float64))
    assert idx.tolist() == [[0]] and torch.allclose(out, P.gelu_erf(s0 * h))
    # the clamped gated unit
    wd = {"d.gate": torch.tensor([[10.0]], dtype=torch.float64), "d.up": torch.tensor([[-10.0]], dtype=torch.float64),
          "d.down": torch.tensor([[1.0]], dtype=torch.float64)}
    got = P.clamped_glu(torch.tensor([[1.0]], dtype=torch.float64), wd, "d.", 2.0)
    assert torch.allclose(got, torch.tensor([[2.0 * torch.sigmoid(torch.tensor(3.404)).item() * (-2.0 + 1.0)]], dtype=torch.float64))


def test_config_names_every_size_and_refuses_what_it_cannot_read():
    for which, cfg in tiny.CONFIGS.items():
        spec, expected = expected_from_config(cfg)
        stored = {spec.stored_names.get(n, n): tuple(ws.shape) for n, ws in expected.items()}
        assert stored == tiny.tensor_shapes(cfg)
        assert spec.tie_word_embeddings and [c.layer for c in spec.order] == list(range(len(cfg["layers"])))
    spec, _ = expected_from_config(tiny.G1)
    roles = [l.parts["mixer"].params.get("value_mix") for l in spec.layers]
    assert roles == ["source", None, "blend", None, None, "blend"]
    assert "norm2" not in spec.layers[2].parts and "ffn" not in spec.layers[2].parts
    for key, value, message in ((("layers", 0, "type"), "conv", "unknown layer type"),
                                (("layers", 0, "mixer", "kv_heads"), 4, "multiple of kv_heads"),
                                (("layers", 0, "mixer", "rot", "dims"), 26, "at most dim"),
                                (("layers", 1, "mixer", "gate_cap"), 0.0, "gate_cap"),
                                (("layers", 1, "mlp", "router", "top"), 6, "exceeds"),
                                (("layers", 5, "mixer", "vdim"), 12, "agree in kv_heads and vdim"),
                                (("layers", 0, "mlp", "kind"), "conv", "unknown kind")):
        bad = copy.deepcopy(tiny.G1)
        d = bad
        for k in key[:-1]:
            d = d[k]
        d[key[-1]] = value
        with pytest.raises(ConfigError, match=message):
            expected_from_config(bad)
    bad = copy.deepcopy(tiny.G1)
    del bad["layers"][3]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match="vdim"):
        expected_from_config(bad)


def test_a_missing_or_misshaped_tensor_is_named(tmp_path):
    w = tiny.random_weights(tiny.G1, 1)
    del w["l1.mix.f.b"]
    w["l0.mix.sink"] = w["l0.mix.sink"][:3]
    folder, _ = tiny.write_model(tmp_path / "m", tiny.G1, weights=w)
    with pytest.raises(WeightError) as e:
        load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=4, max_slots=2, max_context=64)
    assert "l1.mix.f.b" in str(e.value) and "l0.mix.sink" in str(e.value)


def test_pages_of_the_kept_first_tokens_stay_while_the_window_moves_on():
    """A group whose window keeps the first 20 positions holds the two pages of 16 that carry them until the
    request ends; the pages between them and the window go back as the window passes."""
    spec = KVSpec(2, 8, window=10, value_dim=4, keep_first=20)
    cm = CacheManager({0: spec}, {}, page_size=16, n_pages=8, max_slots=2, max_context=16 * 12, dtype=torch.float32, device="cpu")
    g = cm.groups[0]
    s = cm.admit()
    for start in range(0, 150, 7):
        end = min(start + 7, 150)
        assert cm.can_run(s, start, end)
        cm.ensure(s, start, end)
        cm.advance(s, end)
        cm.check()
        pages = g.pages.tables[s].pages
        assert pages[0] >= 0 and (len(pages) < 2 or pages[1] >= 0)
        first = max(0, end + 1 - 10) // 16
        assert all(p < 0 for p in pages[2:first]) and all(p >= 0 for p in pages[max(first, 2):])
        assert g.pages.pool.used_pages <= 4
    assert tuple(g.values.shape[-2:]) == (16, 4) and tuple(g.keys.shape[-2:]) == (16, 8)
    # a request admitted far behind its start (recomputed after preemption) still gets its kept pages
    t = cm.admit()
    assert cm.pages_needed(t, 100, 104) == 2 + 2
    cm.ensure(t, 100, 104)
    pages = g.pages.tables[t].pages
    assert pages[0] >= 0 and pages[1] >= 0 and all(p < 0 for p in pages[2:5]) and pages[5] >= 0 and pages[6] >= 0
    cm.release(s)
    cm.release(t)
    cm.check()
    assert g.pages.pool.used_pages == 0


def test_replay_matches_plain_whole_and_cut(setup):
    which, cfg, folder, w, reqs, plain = setup
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs, tail=24), traces.portions(reqs),
                  traces.portions(reqs, sizes=(2, 2, 1, 2, 3, 128))):
        out, _ = replay(folder, steps)
        compare(out, steps, plain)


def test_replay_matches_plain_in_mixed_batches_with_slots_and_pages_used_again(setup):
    which, cfg, folder, w, reqs, plain = setup
    more = dict(reqs)
    more.update({f"s{i}": t for i, t in enumerate(traces.make_requests(cfg["vocab"], (5, 33, 18), seed=11).values())})
    plain = dict(plain)
    for rid in ("s0", "s1", "s2"):
        plain[rid] = P.forward(cfg, w, more[rid])
    for seed in (0, 3):
        steps = traces.mixed(more, seed=seed)
        out, rp = replay(folder, steps)
        compare(out, steps, plain)
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2


def test_the_matrix_memory_starts_from_zero_in_a_slot_that_was_used(setup):
    """One slot, three requests one after the other: each must see the state of a new sequence."""
    which, cfg, folder, w, reqs, plain = setup
    rp = Replayer(folder, dtype="float32", max_tokens=192, page_size=16, max_requests=1, device="cpu", ops=RefOps())
    for rid in ("r3", "r2", "r3"):
        t = reqs[rid]
        a = rp.run_step([{"id": rid, "tokens": t[:5], "want": [4]}])
        b = rp.run_step([{"id": rid, "tokens": t[5:], "want": [len(t) - 6]}], end=[rid])
        got = torch.cat([a, b]).double()
        want = torch.stack([plain[rid][4], plain[rid][-1]])
        assert (got - want).abs().max() < 3e-4 * float(want.abs().max())


def test_random_weights_mode_writes_the_design_s_own_names(tmp_path):
    folder = write_random_model(tmp_path / "m", tiny.G2, seed=5)
    from flint_b200.weights.safetensors_io import SafetensorsFile
    names = set(SafetensorsFile(folder / "model.safetensors").names())
    assert names == set(tiny.tensor_shapes(tiny.G2))
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2, max_context=128)
    assert m.spec.architecture == "Gepadra" and len(m.cache.groups) == 2 and len(m.cache.state) == 2


def test_greedy_generation_through_the_engine_with_preemption(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(10):
            t = int(torch.argmax(P.forward(cfg, w, toks)[-1]))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages, ahead in ((16, True), (16, False), (3, True)):
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=n_pages, max_slots=4,
                       max_step_tokens=24, max_context=256, use_graphs=False)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=ahead) if "run_ahead" in Engine.__init__.__code__.co_varnames \
            else Engine(m, SamplingParams.greedy(), prefill_chunk=16)
        assert eng.generate(prompts, 10) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0
