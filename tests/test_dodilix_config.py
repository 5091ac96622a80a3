"""Dodilix on the CPU: configuration keys and errors, the model as data, declared tensors, cache needs, the oracle's own
properties, and the engine's host side with every launcher replaced by its plain statement."""
import copy
import tempfile

import pytest
import torch

import dodilix_models as dm
import kernel_refs
import plain_dodilix as plain
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.cache.manager import PagedNeed, SlotNeed
from neurogrid_b200.config import config_from_dict
from neurogrid_b200.config.lfm2 import ConfigError
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.models.decoder import Decoder


def test_spec_of_every_option():
    spec = config_from_dict(dm.DODI_A).model_spec()
    assert spec.architecture == "Dodilix" and spec.streams == 3 and spec.logit_scale == 0.6 and spec.embed_scale == 1.7
    assert [l.block for l in spec.layers] == ["hyper"] * 4
    assert [(e.layer, e.cache, e.writes) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    lat, par = spec.layers[0].mixer, spec.layers[1].mixer
    assert (lat.kind, lat.rope_dim, lat.gate, lat.window, lat.position.pairing) == ("latent_attention", 4, "element", None, "adjacent")
    assert par.kind == "side_by_side" and par.combine == "weighted" and (par.left_scale, par.right_scale) == (0.7, 1.3)
    left, right = par.left, par.right
    assert (left.chunk, left.cache_window, left.window, left.sink, left.out_gate, left.norm_weight) == (13, 13, None, True, True, False)
    assert (left.position.pairing, left.position.rotary_dims, left.position.theta) == ("half", 8, 1000.0)
    assert (right.kind, right.decay_rank, right.tau) == ("gated_linear_attention", 5, 7.0)
    moe = spec.layers[0].ffn
    assert (moe.scoring, moe.group_score, moe.route_scale, moe.n_groups, moe.keep_groups, moe.shared_gate) == \
        ("softmax_all", "max", 1.7, 3, 1, True)
    assert spec.layers[2].ffn is None and spec.layers[1].ffn.kind == "swiglu"
    plain_spec = config_from_dict(dm.DODI_B0).model_spec()
    assert plain_spec.streams == 0 and all(l.block == "prenorm" for l in plain_spec.layers)
    b = config_from_dict(dm.DODI_B).model_spec()
    assert b.layers[0].mixer.left.position.kind == "none" and b.layers[2].mixer.left.chunk is None
    assert b.layers[1].mixer.rope_dim == 0 and b.layers[1].mixer.position is None


def test_declared_tensors():
    names = declare_tensors(config_from_dict(dm.DODI_A).model_spec())
    for n, shape in {"embed": (131, 56), "head": (131, 56), "final.norm": (56,), "l0.hc1.mix": (3, 3), "l0.hc2.in": (3,),
                     "l0.mix.dkv": (28, 56), "l0.mix.dkv.norm": (24,), "l0.mix.uq": (36, 20), "l0.mix.g": (18, 56),
                     "l0.mlp.shared.sg": (1, 56), "l0.mlp.e5.down": (56, 16), "l1.mix.left.g": (48, 56),
                     "l1.mix.left.sink": (4,), "l1.mix.right.a1": (5, 56), "l1.mix.right.a2": (24, 5),
                     "l1.mix.right.a2.b": (24,), "l1.mix.right.norm": (10,), "l1.mlp.gate": (40, 56), "l2.hc1.out": (3,),
                     "l2.mix.uk": (24, 24)}.items():
        assert names[n].shape == shape, n
    assert not any(n.startswith(("l2.mix.dkv", "l2.hc2", "l2.norm2", "l2.mlp")) for n in names)
    assert not any(".hc" in n for n in declare_tensors(config_from_dict(dm.DODI_B0).model_spec()))


def test_decay_rank_comes_from_the_shapes():
    cfg = config_from_dict({k: v for k, v in copy.deepcopy(dm.DODI_A).items()})
    for layer in cfg.layers:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank")
    assert cfg.model_spec().layers[1].mixer.right.decay_rank == 16           # nothing said: the default
    seen = cfg.with_shapes({"l1.mix.right.a1": (7, 56), "l3.mix.right.a1": (3, 56)}).model_spec()
    assert [seen.layers[i].mixer.right.decay_rank for i in (1, 3)] == [7, 3]


def _broken(path, value):
    cfg = copy.deepcopy(dm.DODI_A)
    node = cfg
    for k in path[:-1]:
        node = node[k]
    if value is None:
        node.pop(path[-1])
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 1, "mixer", "left", "heads"), 5, "kv_heads"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "rot.dims"),
    (("layers", 1, "mixer", "right", "tau"), None, "tau"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 2, "mixer", "kv_from"), 3, "kv_from"),
    (("layers", 2, "mixer", "kv_rank"), 32, "kv_from"),
    (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("layers", 0, "mlp", "router", "top"), 5, "router"),
    (("layers", 0, "mlp", "kind"), "gated", "kind"),
    (("streams",), 40, "streams"),
    (("norm",), None, "norm.eps"),
])
def test_config_errors_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(path, value))
    assert word in str(e.value)


def test_cache_needs():
    needs = Decoder(config_from_dict(dm.DODI_A).model_spec(), dtype=torch.float32, device="cpu").cache_needs()
    assert set(needs) == {0, 1, 3}                                           # layer 2 reads layer 0's pages
    assert needs[0] == PagedNeed(1, 32, None, values=False)                  # 24 latent + 4 rotated columns, in sixteens
    paged, state = needs[1]
    assert paged == PagedNeed(2, 16, 13, True, v_heads=2, v_dim=12) and state == SlotNeed((3, 8, 10))


LENS = {"A": [1, 9, 40, 67, 23], "B": [3, 50, 30], "B0": [2, 41], "C": [2, 17, 90, 33], "D": [1, 30, 12]}


@pytest.mark.parametrize("name", ["A", "B", "B0", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_against_plain(dodilix_dirs, monkeypatch, name, cut):
    """The step function, cache manager and parts on the CPU, every launcher replaced by its plain statement: the
    states, pages and slots reach the right layer of the right request however the work is cut."""
    kernel_refs.install(monkeypatch)
    cfg, w = dm.load_plain(dodilix_dirs[name])
    reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=17)
    ps = dm.PAGE_SIZE[name]
    cap = 128 if cut == "mixed" else 256
    runner = make_runner(dodilix_dirs[name], dtype=torch.float32, device="cpu", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": lambda r: scenarios.tail_decode(r, 12), "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = []
    for s in steps:
        got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
        for r in s["end"]:
            runner.finish(r)
        runner.cache.check()
    got = scenarios.collect(steps, lambda i: got[i])
    for r, t in reqs.items():
        assert rel_err(got[r], plain.forward(cfg, w, t)) < 2e-5, (r, len(t))
    assert all(f == cap // ps for f in runner.cache.pages_free()) and runner.cache.slots_free() == 4


def test_oracle_is_causal_and_its_mechanisms_bite():
    cfg, w = dm.load_plain(dm.write_model(dm.DODI_A, 5, tempfile.mkdtemp()))
    toks = scenarios.make_requests([48], cfg["vocab"], seed=2)["r0"]
    a = plain.forward(cfg, w, toks)
    assert rel_err(a[:30], plain.forward(cfg, w, toks[:30])) < 1e-12
    # the recurrent state carries the first token beyond every chunk
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert rel_err(plain.forward(cfg, w, other)[40:], a[40:]) > 1e-6

    def changed(edit):
        c2, w2 = copy.deepcopy(cfg), dict(w)
        edit(c2, w2)
        return rel_err(plain.forward(c2, w2, toks), a)

    def scale(name, f):
        return lambda c, ww: ww.__setitem__(name, ww[name] * f)

    assert changed(lambda c, ww: c["layers"][1]["mixer"]["left"]["mask"].__setitem__("size", 14)) > 1e-4
    assert changed(lambda c, ww: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 6)) > 1e-4
    assert changed(scale("l1.mix.left.sink", 0.0)) > 1e-4
    assert changed(scale("l1.mix.left.g", 0.0)) > 1e-4
    assert changed(lambda c, ww: c["layers"][1]["mixer"]["right"].__setitem__("tau", 3.0)) > 1e-4
    assert changed(lambda c, ww: c["layers"][1]["mixer"].__setitem__("left_scale", 0.75)) > 1e-4
    assert changed(lambda c, ww: c["layers"][0]["mixer"]["rot"].__setitem__("base", 30.0)) > 1e-4
    assert changed(lambda c, ww: c["layers"][2]["mixer"].pop("kv_from") or ww.update(
        {"l2.mix.dkv": ww["l0.mix.dkv"] * 0.5, "l2.mix.dkv.norm": ww["l0.mix.dkv.norm"]})) > 1e-4
    assert changed(lambda c, ww: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 2)) > 1e-5
    assert changed(lambda c, ww: c["layers"][0]["mlp"]["router"].__setitem__("scale", 1.0)) > 1e-4
    assert changed(scale("l0.mlp.shared.sg", 0.0)) > 1e-4
    assert changed(scale("l3.hc2.mix", 0.9)) > 1e-4
    assert changed(lambda c, ww: c.__setitem__("logit_scale", 1.0)) > 1e-2
