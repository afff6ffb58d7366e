"""The Bolovik decoder without a GPU: its configuration, its model description,
its tensors, the page bookkeeping of a window that keeps the first tokens, and
the plain implementation's own pieces."""
import copy
import json

import pytest
import torch

import plain_bolovik as pb
from bolovik_cases import CASES, DENSE, attention, delta, moe, rot
from infernum_b200.cache import CacheManager
from infernum_b200.config.bolovik import BolovikConfig
from infernum_b200.errors import ConfigError
from infernum_b200.models.model import CacheNeed
from infernum_b200.parts.base import PagedCacheSpec
from infernum_b200.registry import resolve_config, supported_architectures
from infernum_b200.weights.random_init import model_specs_for


def test_the_registry_knows_the_architecture():
    assert "Bolovik" in supported_architectures()
    arch, cfg = resolve_config(CASES["A"])
    assert isinstance(cfg, BolovikConfig) and arch.name == "Bolovik"


def test_every_size_and_constant_is_read():
    cfg = BolovikConfig.from_dict(CASES["A"])
    assert (cfg.vocab, cfg.width, cfg.norm_groups, cfg.norm_eps) == (211, 96, 3, 1e-5)
    d, a = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 16, 24, 4)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first) == (6, 2, 16, 8, 0.35, 21, 5)
    assert (a.rot.dims, a.rot.base, a.rot.scaling) == (8, 10000.0, (8.0, 1.0, 4.0, 64.0))
    m = cfg.layers[1].mlp
    assert (m.kind, m.ff, m.experts, m.top, m.group_count, m.group_keep) == ("moe", 40, 8, 3, 4, 2)
    assert cfg.layers[0].mlp.kind == "dense" and cfg.layers[0].mlp.ff == 72
    assert cfg.layers[2].mlp is None


def test_keys_left_out_mean_what_their_absence_says():
    cfg = BolovikConfig.from_dict(CASES["B"])
    assert cfg.norm_groups == 1
    full = cfg.layers[2].mixer
    assert full.window == 0 and full.keep_first == 0 and full.rot is None
    bare = cfg.layers[3].mixer
    assert (bare.kv_heads, bare.vdim, bare.conv) == (2, 12, 0)
    assert cfg.layers[5].mixer.keep_first == 0
    one = cfg.layers[1].mlp
    assert (one.experts, one.top, one.group_count, one.group_keep) == (1, 1, 1, 1)
    no_scale = copy.deepcopy(CASES["D"])
    del no_scale["layers"][1]["mixer"]["scale"]
    assert BolovikConfig.from_dict(no_scale).layers[1].mixer.scale == 16 ** -0.5


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "cannot give"),
    (lambda c: c["norm"].update(groups=5), "does not split"),
    (lambda c: c.pop("layers"), "non-empty list"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "not supported"),
])
def test_bad_configurations_are_refused_by_name(change, message):
    cfg = copy.deepcopy(CASES["A"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        BolovikConfig.from_dict(cfg)


def test_the_tensors_of_a_model_are_those_of_its_layers():
    _, spec, specs = model_specs_for(CASES["A"])
    assert specs["embed"].shape == (211, 96) and specs["head"].shape == (211, 96)
    assert specs["l0.mix.q"].shape == (32, 96) and specs["l0.mix.v"].shape == (96, 96)
    assert specs["l0.mix.q.conv"].shape == (32, 4) and specs["l0.mix.v.conv"].shape == (96, 4)
    assert specs["l0.mix.b"].shape == (4, 96) and specs["l0.mix.A_log"].shape == (4,)
    assert specs["l0.mix.norm"].shape == (24,) and specs["l0.mix.o"].shape == (96, 96)
    assert specs["l1.mix.q"].shape == (96, 96) and specs["l1.mix.q.b"].shape == (96,)
    assert specs["l1.mix.v"].shape == (16, 96) and specs["l1.mix.v.b"].shape == (16,)
    assert specs["l1.mix.o"].shape == (96, 48)
    assert specs["l1.mlp.router"].shape == (8, 96) and specs["l1.mlp.e7.down"].shape == (96, 40)
    assert "l1.mlp.router.b" not in specs and "l2.norm2" not in specs
    for i in range(5):
        assert specs[f"l{i}.dwa"].shape == (i + 2,)
    _, _, bare = model_specs_for(CASES["B"])
    assert "l3.mix.q.conv" not in bare and bare["l1.mix.q.conv"].shape == (28, 1)
    assert spec.embedding.params["result_slots"] == 6


def _manager(window, keep_first, page_size=4, pages=64):
    need = CacheNeed(0, PagedCacheSpec(1, 8, window, v_head_dim=4, keep_first=keep_first), None, None)
    return CacheManager([need], page_size=page_size, num_pages=pages, max_requests=2)


def test_pages_of_kept_first_tokens_stay_and_the_rest_go_back_behind_the_window():
    cm = _manager(window=10, keep_first=5)
    rc = cm.admit("a")
    for n in (7, 30, 1, 1, 26):
        cm.extend(rc, n)
        cm.commit(rc, n)
        cm.check_invariants()
        table = rc.tables[0]
        first_needed = rc.num_tokens - 10 + 1
        for i, page in enumerate(table):
            holds_kept = i * 4 < 5
            out_of_reach = (i + 1) * 4 <= first_needed
            assert (page >= 0) == (holds_kept or not out_of_reach), (rc.num_tokens, i, table)
    held = sum(p >= 0 for p in rc.tables[0])
    assert held <= 2 + 4
    cm.release(rc)
    assert cm.free_pages() == [64]
    # without kept tokens the first pages go back too
    cm = _manager(window=10, keep_first=0)
    rc = cm.admit("b")
    cm.extend(rc, 40)
    cm.commit(rc, 40)
    assert rc.tables[0][0] == -1 and rc.tables[0][-1] >= 0
    assert _manager(10, 5).peak_pages(1000, 8)[0] == 5 + 1 + 2


def test_groups_of_specs_tell_kept_tokens_and_value_sizes_apart():
    needs = [CacheNeed(0, PagedCacheSpec(1, 8, 10, v_head_dim=4, keep_first=5), None, None),
             CacheNeed(1, PagedCacheSpec(1, 8, 10, v_head_dim=4, keep_first=5), None, None),
             CacheNeed(2, PagedCacheSpec(1, 8, 10, v_head_dim=4, keep_first=0), None, None),
             CacheNeed(3, PagedCacheSpec(1, 8, 10, v_head_dim=8), None, None)]
    cm = CacheManager(needs, page_size=4, num_pages=8, max_requests=1)
    assert [g.positions for g in cm.groups] == [[0, 1], [2], [3]]


# ---- the plain implementation's own pieces ------------------------------------------
def test_plain_visibility():
    see = pb.visible(12, 4, 2)
    assert see[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert see[3].tolist() == [True] * 4 + [False] * 8
    assert pb.visible(5, 1, 0).sum().item() == 5


def test_plain_routing_stays_inside_the_best_groups():
    torch.manual_seed(3)
    h = torch.randn(50, 16, dtype=torch.float64)
    w = torch.randn(12, 16, dtype=torch.float64)
    ids, wts = pb.route(h, w, {"experts": 12, "top": 3, "groups": {"count": 3, "keep": 1}})
    s = torch.sigmoid(h @ w.t())
    for t in range(50):
        groups = {int(e) // 4 for e in ids[t]}
        assert len(groups) == 1
        g = groups.pop()
        score = lambda j: s[t, 4 * j: 4 * j + 4].topk(2).values.sum()  # noqa: E731
        assert all(score(g) >= score(j) for j in range(3))
        assert torch.equal(wts[t], s[t, ids[t]])


def test_plain_delta_rule_against_its_closed_form_for_two_tokens():
    torch.manual_seed(5)
    q, k = torch.randn(2, 6, dtype=torch.float64), torch.randn(2, 6, dtype=torch.float64)
    v = torch.randn(2, 4, dtype=torch.float64)
    beta, g = torch.tensor([0.3, 0.8], dtype=torch.float64), torch.tensor([0.9, 0.5], dtype=torch.float64)
    out = pb.delta_rule(q, k, v, beta, g)
    S1 = torch.outer(k[0], beta[0] * v[0])
    assert torch.allclose(out[0], S1.t() @ q[0])
    S2 = g[1] * S1
    S2 = S2 + torch.outer(k[1], beta[1] * (v[1] - S2.t() @ k[1]))
    assert torch.allclose(out[1], S2.t() @ q[1])


def test_plain_convolution_starts_from_zeros_and_ends_on_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert pb.causal_conv(x, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_a_model_folder_round_trips_through_the_writer(tmp_path):
    from bolovik_cases import make_folder
    folder = make_folder(str(tmp_path / "m"), CASES["D"], seed=4)
    assert json.load(open(folder + "/config.json"))["architecture"] == "Bolovik"
    plain = pb.Plain(folder)
    logits = plain.logits([1, 5, 9, 2, 7, 7, 3])
    assert logits.shape == (7, 97) and torch.isfinite(logits).all()
