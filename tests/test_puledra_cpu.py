"""Puledra through the engine's plumbing on the CPU (the kernels replaced by their plain references): the
configuration reader, tensor names, the cache shared between layers, the pair table's per-request state, and
replay under every cut against the plain implementation."""
import copy

import pytest
import torch

import plain_puledra as P
import tiny_puledra as tiny
import traces
from flint_b200.engine.engine import Engine
from flint_b200.engine.loading import expected_from_config, write_random_model
from flint_b200.engine.model import load_model
from flint_b200.engine.replay import Replayer
from flint_b200.errors import ConfigError, WeightError
from flint_b200.sampling.params import SamplingParams
from kernel_refs import RefOps

LENGTHS = (1, 2, 9, 37, 70, 130)


@pytest.fixture(scope="module", params=["P1", "P2"])
def setup(request, tmp_path_factory):
    which = request.param
    cfg = tiny.CONFIGS[which]
    folder, w = tiny.write_model(tmp_path_factory.mktemp("puledra") / which, cfg, seed=3)
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
    z = torch.tensor([0.1, 2.0, 1.9, -1.0, 0.5, 0.4, 3.0, -2.0], dtype=torch.float64)
    # four groups of two: the best groups are {6,7} and {1,0}... group scores 2.0 (g0), 1.9 (g1), 0.5 (g2), 3.0 (g3)
    ids, ws = P.route(z, top=2, n_groups=4, keep=2, scale=1.5)
    assert ids == [6, 1] and abs(sum(ws) - 1.5) < 1e-12
    ids, _ = P.route(z, top=3, n_groups=4, keep=2, scale=1.0)
    assert ids == [6, 1, 0]                          # expert 2 (1.9) is in a group that was not kept
    ids, _ = P.route(z, top=3, n_groups=1, keep=1, scale=1.0)
    assert ids == [6, 1, 2]
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    y = P.rotate_pairs(x, range(5), 100.0, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])           # position 0, unrotated dims
    assert torch.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    assert P.bigram_rows([4, 9, 9], 53, 31, 5) == [53, (4 * 31 + 9 * 5) % 53, (9 * 31 + 9 * 5) % 53]


def test_config_names_every_size_and_refuses_what_it_cannot_read():
    for which, cfg in tiny.CONFIGS.items():
        spec, expected = expected_from_config(cfg)
        stored = {spec.stored_names.get(n, n): tuple(ws.shape) for n, ws in expected.items()}
        assert stored == tiny.tensor_shapes(cfg)
        assert [c.cache_of for c in spec.order] == [l["mixer"].get("kv_from") for l in cfg["layers"]]
    bad = copy.deepcopy(tiny.P1)
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="earlier layer"):
        expected_from_config(bad)
    bad = copy.deepcopy(tiny.P1)
    bad["layers"][3]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="no latent of its own"):
        expected_from_config(bad)
    bad = copy.deepcopy(tiny.P1)
    bad["layers"][1]["mixer"]["kv_rank"] = 24
    with pytest.raises(ConfigError, match="must equal"):
        expected_from_config(bad)
    bad = copy.deepcopy(tiny.P1)
    del bad["layers"][0]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match="vdim"):
        expected_from_config(bad)
    bad = copy.deepcopy(tiny.P1)
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 3
    with pytest.raises(ConfigError, match="equal groups"):
        expected_from_config(bad)
    bad = copy.deepcopy(tiny.P1)
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ConfigError, match="unknown layer type"):
        expected_from_config(bad)


def test_a_checkpoint_with_a_missing_tensor_is_refused_by_name(tmp_path):
    w = tiny.random_weights(tiny.P1, 1)
    del w["l2.mix.dkv.norm"]
    w["l1.mix.dkv"] = torch.zeros(48, 48, dtype=torch.bfloat16)        # a layer that reads another's latent has none
    folder, _ = tiny.write_model(tmp_path / "m", tiny.P1, weights=w)
    with pytest.raises(WeightError) as e:
        load_model(folder, dtype="float32", device="cpu", ops=RefOps(), max_context=64)
    assert "l2.mix.dkv.norm" in str(e.value) and "l1.mix.dkv" in str(e.value)


def test_random_weights_mode_writes_the_design_s_own_names(tmp_path):
    folder = write_random_model(tmp_path / "r", tiny.P2, seed=5)
    assert set(P.read_safetensors(folder / "model.safetensors")) == set(tiny.tensor_shapes(tiny.P2))
    load_model(folder, dtype="float32", device="cpu", ops=RefOps(), max_context=64, n_pages=4, max_slots=1)


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "twos", "mixed"])
@pytest.mark.parametrize("page_size", [16, 64])
def test_replay_matches_plain_under_every_cut(setup, cut, page_size):
    which, cfg, folder, w, reqs, plain = setup
    steps = {"whole": traces.whole, "tail": lambda r: traces.tail_decoded(r, tail=20), "portions": traces.portions,
             "twos": lambda r: traces.portions(r, sizes=(2, 2, 1, 2, 3)),
             "mixed": lambda r: traces.mixed(r, seed=3)}[cut](reqs)
    out, rp = replay(folder, steps, page_size)
    compare(out, steps, plain)
    if cut == "mixed" and page_size == 16:
        assert max(max(g.pages.pool.served) for g in rp.model.cache.groups) >= 2, "no page was used again"
        assert len(reqs) > rp.model.cache.max_slots, "no slot was used again"


def test_layers_with_equal_needs_share_a_page_group_and_readers_own_no_cache(setup):
    which, cfg, folder, w, reqs, plain = setup
    m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=8, max_slots=2, max_context=128)
    owners = [i for i, l in enumerate(cfg["layers"]) if l["mixer"].get("kv_from") is None]
    assert sorted(c for g in m.cache.groups for c in g.calls) == owners
    for g in m.cache.groups:
        assert g.values.shape[-1] == 0                     # the latent is the start of the key row: no values kept
        mixer = m.layers[g.calls[0]].parts["mixer"]
        assert g.keys.shape[-1] == -(-(mixer.C + mixer.R) // 8) * 8
    if which == "P2":
        assert len(m.cache.groups) == 1 and len(m.cache.groups[0].calls) == 2


def test_the_pair_table_s_predecessor_survives_steps_and_slots(setup):
    """Single-token steps of two interleaved requests, one of which ends and gives its slot to a third."""
    which, cfg, folder, w, reqs, plain = setup
    a, b, c = reqs["r2"], reqs["r3"][:12], reqs["r4"][:7]
    steps = []
    for i in range(9):
        entries = [{"id": "a", "tokens": [a[i]], "want": [0]}]
        if i < 12:
            entries.append({"id": "b", "tokens": [b[i]], "want": [0]})
        steps.append({"step": len(steps), "entries": entries, "end": ["a"] if i == 8 else []})
    steps.append({"step": len(steps), "entries": [{"id": "c", "tokens": c[:3], "want": [0, 2]},
                                                   {"id": "b", "tokens": b[9:12], "want": [0, 1, 2]}], "end": ["b"]})
    steps.append({"step": len(steps), "entries": [{"id": "c", "tokens": c[3:], "want": [0, 3]}], "end": ["c"]})
    rp = Replayer(folder, dtype="float32", max_tokens=128, page_size=16, max_requests=2, device="cpu", ops=RefOps())
    pl = {"a": plain["r2"], "b": P.forward(cfg, w, b), "c": P.forward(cfg, w, c)}
    done = {}
    for s in steps:
        out = rp.run_step(s["entries"], s["end"])
        r = 0
        for e in s["entries"]:
            base = done.get(e["id"], 0)
            for k in e["want"]:
                assert (out[r].double() - pl[e["id"]][base + k]).abs().max() < 3e-4
                r += 1
            done[e["id"]] = base + len(e["tokens"])


def test_greedy_generation_through_the_entry_point(setup):
    which, cfg, folder, w, reqs, plain = setup
    prompts = [reqs["r2"], reqs["r3"][:14], reqs["r0"]]
    expected = []
    for p in prompts:
        toks, out = list(p), []
        for _ in range(8):
            t = int(torch.argmax(P.forward(cfg, w, toks)[-1]))
            out.append(t)
            toks.append(t)
        expected.append(out)
    for n_pages, run_ahead in ((16, True), (16, False), (3, True)):      # three pages: requests are preempted and recomputed
        m = load_model(folder, dtype="float32", device="cpu", ops=RefOps(), page_size=16, n_pages=n_pages, max_slots=4,
                       max_step_tokens=24, max_context=256)
        eng = Engine(m, SamplingParams.greedy(), prefill_chunk=16, run_ahead=run_ahead)
        assert eng.generate(prompts, 8) == expected
        assert all(g.pages.pool.used_pages == 0 for g in m.cache.groups) and m.cache.free_slots == 4
    assert eng.scheduler.preemptions > 0
