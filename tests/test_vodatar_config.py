"""The Vodatar decoder without a GPU: its configuration reader, its model description (the
order of runs, tensor names, what every run needs from the cache manager) and pieces of the
plain implementation that the GPU tests rest on."""
import copy
import math

import pytest
import torch

import plain_vodatar as pv
from vodatar_cases import CASES, random_case

from infernum_b200.config.vodatar import VodatarConfig
from infernum_b200.errors import ConfigError
from infernum_b200.models.model import Model
from infernum_b200.parts.base import Runtime
from infernum_b200.registry import resolve_config, supported_architectures


def build(cfg_dict):
    arch, cfg = resolve_config(cfg_dict)
    spec = arch.build_spec(cfg)
    return cfg, spec, Model(spec, Runtime(torch.device("cpu"), torch.bfloat16))


def test_the_architecture_is_registered():
    assert "Vodatar" in supported_architectures()


@pytest.mark.parametrize("name", sorted(CASES))
def test_every_case_reads_and_describes_a_model(name):
    cfg, spec, model = build(CASES[name])
    assert isinstance(cfg, VodatarConfig)
    order = pv.run_order(CASES[name])
    assert [(i.layer, i.enter) for i in spec.schedule] == order
    assert (spec.pass_entry is not None) == ("loop" in CASES[name])
    names = set(model.weight_specs())
    assert {"embed", "embed.norm", "final.norm", "head"} <= names
    assert ("loop.in" in names) == ("loop" in CASES[name])
    for i, layer in enumerate(CASES[name]["layers"]):
        assert f"l{i}.norm1" in names and f"l{i}.norm1b" in names and f"l{i}.rg1" in names and f"l{i}.rg1.b" in names
        assert (f"l{i}.canon1" in names) == ("canon" in CASES[name])
        assert (f"l{i}.norm2" in names) == (layer["mlp"] is not None) == (f"l{i}.rg2" in names)
        if layer["type"] == "attention":
            assert (f"l{i}.mix.q.conv" in names) == bool(layer["mixer"].get("conv"))
            assert f"l{i}.mix.lq1" in names
        else:
            assert f"l{i}.mix.dkv.norm" in names and f"l{i}.mix.uk" in names
        if layer["mlp"] is not None:
            r = layer["mlp"]["router"]
            ws = model.weight_specs()
            assert ws[f"l{i}.mlp.router"].shape == (r["experts"] + r.get("identity", 0), CASES[name]["width"])
            assert f"l{i}.mlp.e{r['experts'] - 1}.down" in names and f"l{i}.mlp.e{r['experts']}.down" not in names
            assert (f"l{i}.mlp.shared.sg" in names) == ("shared" in layer["mlp"])


def test_every_run_has_a_cache_and_states_of_its_own():
    cfg, spec, model = build(CASES["A"])
    needs = model.cache_needs()
    assert len(needs) == len(spec.schedule) == 1 + 2 * 3 + 1
    taps, width = CASES["A"]["canon"]["taps"], CASES["A"]["width"]
    for need, item in zip(needs, spec.schedule):
        layer = CASES["A"]["layers"][item.layer]
        m = layer["mixer"]
        assert need.block_state.shape == (2 * (taps - 1) * width,)
        if layer["type"] == "attention":
            assert (need.paged.kv_heads, need.paged.head_dim, need.paged.value_dim) == (m["kv_heads"], 2 * m["dim"], m["vdim"])
            channels = (m["heads"] + m["kv_heads"]) * 2 * m["dim"] + m["kv_heads"] * m["vdim"]
            assert need.state.shape == ((m["conv"] - 1) * channels,)
        else:
            assert (need.paged.kv_heads, need.paged.head_dim, need.paged.value_dim) == (1, m["kv_rank"] + m["rot_dim"], 0)
            assert need.state is None
    # no convolution anywhere: nothing but pages
    _, _, model = build(CASES["B"])
    assert all(n.block_state is None for n in model.cache_needs())
    assert [n.state for n in model.cache_needs()] == [None] * 4


def test_the_cache_manager_gives_every_run_its_states():
    from infernum_b200.cache import CacheManager
    _, spec, model = build(CASES["E"])
    cache = CacheManager(model.cache_needs(), page_size=4, num_pages=8, max_requests=2, device=None)
    assert len(cache.layer_caches) == len(spec.schedule)
    assert len(cache.groups) == 2


def test_keys_left_out_mean_what_their_absence_says():
    cfg = VodatarConfig.from_dict(CASES["B"])
    assert cfg.loop is None and cfg.canon_taps == 0 and cfg.residual_mult == 1.0 and cfg.norm_groups == 1
    a = cfg.layers[0].mixer
    assert (a.softcap, a.conv, a.rot.dims, a.diff) == (0.0, 0, 0, 0.0)
    assert cfg.layers[1].mlp.identity == 1 and cfg.layers[1].mlp.shared_ff == 0
    assert cfg.layers[0].mlp.identity == 0
    d = copy.deepcopy(CASES["B"])
    del d["layers"][0]["mixer"]["kv_heads"], d["layers"][0]["mixer"]["vdim"], d["layers"][0]["mixer"]["scale"]
    m = VodatarConfig.from_dict(d).layers[0].mixer
    assert (m.kv_heads, m.vdim) == (1, 12) and math.isclose(m.scale, 12 ** -0.5)


@pytest.mark.parametrize("edit,what", [
    (lambda d: d["layers"][0].__setitem__("type", "delta"), "type"),
    (lambda d: d["loop"].__setitem__("stop", 9), "loop"),
    (lambda d: d["loop"].__setitem__("start", 3), "loop"),
    (lambda d: d["norm"].__setitem__("groups", 5), "norm groups"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 64), "dims"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda d: d["canon"].__setitem__("taps", 40), "taps"),
    (lambda d: d.__delitem__("width"), "width"),
])
def test_a_configuration_that_cannot_be_is_refused(edit, what):
    d = copy.deepcopy(CASES["A"])
    edit(d)
    with pytest.raises(ConfigError):
        VodatarConfig.from_dict(d)


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random_describe_models(seed):
    cfg_dict = random_case(seed)
    _, spec, model = build(cfg_dict)
    assert [(i.layer, i.enter) for i in spec.schedule] == pv.run_order(cfg_dict)
    assert model.weight_specs()


def test_frequencies_on_a_ramp_and_their_magnitude():
    from infernum_b200.parts.rope import rotary_inv_freq, rotary_magnitude
    for dims, base, sc in [(32, 10000.0, (2.0, 512, 32.0, 1.0)), (8, 100.0, (4.0, 64, 8.0, 1.0)),
                           (16, 500.0, (2.0, 32, 4.0, 2.0)), (2, 20.0, (8.0, 16, 2.0, 1.0)), (64, 250000.0, None)]:
        rot = {"dims": dims, "base": base}
        scaling = None
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
            scaling = {"rope_type": "ramp", **rot["scaling"]}
        want, mag = pv.rotary_frequencies(rot)
        got = rotary_inv_freq(dims, base, scaling)
        assert max(abs(a - b) / b for a, b in zip(got, want)) < 1e-12
        assert math.isclose(rotary_magnitude(scaling), mag)
    # the ramp's ends: pairs before it keep their frequency, pairs behind it are divided by the factor
    freqs, _ = pv.rotary_frequencies({"dims": 32, "base": 10000.0,
                                      "scaling": {"factor": 2.0, "original": 512, "fast": 32.0, "slow": 1.0}})
    plain = [10000.0 ** (-2.0 * i / 32) for i in range(16)]
    assert freqs[0] == plain[0] and math.isclose(freqs[-1], plain[-1] / 2.0)
    assert any(plain[i] / 2.0 < freqs[i] < plain[i] for i in range(16))


def test_the_plain_pieces_agree_with_themselves():
    """A convolution over a whole sequence equals the same over portions that carry the last
    inputs along; a rotation of neighbouring pairs keeps lengths and depends on position
    differences only; a difference of two equal maps with weight 1 is zero."""
    g = torch.Generator().manual_seed(1)
    u, w = torch.randn(20, 6, generator=g, dtype=torch.float64), torch.randn(6, 4, generator=g, dtype=torch.float64)
    whole = pv.causal_conv(u, w)
    tail = pv.causal_conv(torch.cat([u[4:7], u[7:]]), w)[3:]
    assert torch.allclose(whole[7:], tail)
    x = torch.randn(5, 3, 8, generator=g, dtype=torch.float64)
    freqs = [0.5, 0.1, 0.02]
    r = pv.rotate_pairs(x, torch.arange(5), freqs, 1.0)
    assert torch.allclose(r.norm(dim=-1), x.norm(dim=-1)) and torch.equal(r[..., 6:], x[..., 6:])
    a, b = pv.rotate_pairs(x[:1], torch.tensor([7]), freqs), pv.rotate_pairs(x[1:2], torch.tensor([4]), freqs)
    a2, b2 = pv.rotate_pairs(x[:1], torch.tensor([13]), freqs), pv.rotate_pairs(x[1:2], torch.tensor([10]), freqs)
    assert torch.allclose((a * b).sum(), (a2 * b2).sum())
    ids, wts = pv.route(torch.randn(9, 5, generator=g, dtype=torch.float64), {"top": 3},
                        {"r.router": torch.eye(5, dtype=torch.float64)}, "r.")
    assert torch.allclose(wts.sum(-1), torch.ones(9, dtype=torch.float64)) and ids.shape == (9, 3)
