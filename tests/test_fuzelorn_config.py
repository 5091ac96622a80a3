"""Fuzelorn without a GPU: configuration, declared tensors, cache needs, the plain statement's own properties, and the
engine's host side (step function, cache manager, parts) with every launcher replaced by its plain statement."""
import copy

import pytest
import torch

import fuzelorn_models as fm
import kernel_refs
import plain_fuzelorn as plain
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.cache.manager import PagedNeed, SlotNeed
from neurogrid_b200.config import ConfigError, config_from_dict
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.models import Decoder, declare_tensors


def test_spec_and_declared_tensors():
    cfg = config_from_dict(fm.FUZE_S)
    spec = cfg.model_spec()
    assert spec.architecture == "Fuzelorn" and len(spec.layers) == 4
    # layers 1 and 2 run twice in a row, every run with a cache id of its own
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (3, 5)]
    assert cfg.layer_runs() == tuple(plain.layer_runs(fm.FUZE_S))
    d = declare_tensors(spec)
    assert d["bigram"].shape == (54, 72) and d["embed"].shape == (151, 72) and d["final.norm"].shape == (72,)
    assert d["l0.mix.left.q.norm"].shape == (64,) and d["l0.mix.left.k.norm"].shape == (32,) and d["l0.mix.left.sink"].shape == (4,)
    assert d["l1.mix.right.q"].shape == (24, 72) and d["l1.mix.right.v.conv"].shape == (40, 4) and d["l1.mix.right.b"].shape == (2, 72)
    assert d["l1.mix.right.norm"].shape == (20,) and d["l1.mix.right.o"].shape == (72, 40) and d["l1.mix.left.out"].shape == (72,)
    assert d["l0.mlp.up.b"].shape == (40,) and d["l0.mlp.down.b"].shape == (72,)
    assert d["l1.mlp.e5.down"].shape == (72, 24) and d["l1.mlp.shared.sg"].shape == (1, 72) and d["l1.mlp.correction"].shape == (6,)
    assert not any(k.startswith("l2.mlp") or k.startswith("l2.norm2") for k in d)
    assert "l1.mlp.router.b" not in d
    u = declare_tensors(config_from_dict(fm.FUZE_U).model_spec())
    assert "bigram" not in u and "l1.mlp.shared.gate" not in u and u["l0.mix.right.q.conv"].shape == (8, 1)


def _broken(path, value, base=fm.FUZE_S):
    cfg = copy.deepcopy(base)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "serial", "type"),
    (("layers", 0, "mixer", "left", "heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "right", "conv"), 9, "conv"),
    (("layers", 1, "mixer", "right", "dim"), None, "mixer.right.dim"),
    (("layers", 1, "mlp", "router", "top"), 5, "router"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "router"),
    (("layers", 3, "mlp", "expert", "limit"), None, "expert.limit"),
    (("layers", 0, "mlp", "kind"), "gated", "kind"),
    (("loop", "stop"), 7, "loop"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("norm",), None, "norm.eps"),
    (("layers", 0, "mixer", "left", "q_temp", "every"), 0, "every"),
])
def test_config_errors_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(path, value))
    assert word in str(e.value)


def test_cache_needs_per_run():
    spec = config_from_dict(fm.FUZE_S).model_spec()
    needs = Decoder(spec, dtype=torch.float32, device="cpu").cache_needs()
    assert set(needs) == {-1, 0, 1, 2, 3, 4, 5}
    assert needs[-1] == SlotNeed((), "int32", -1)                       # the model's own state: the previous token
    assert needs[1] == needs[3] and needs[2] == needs[4] and needs[1] != needs[2]
    paged, state, conv = needs[1]
    assert paged == PagedNeed(2, 8, 13, True, v_heads=2, v_dim=12)
    assert state == SlotNeed((2, 24, 20)) and conv == SlotNeed((3, 2 * 24 + 40))
    u = Decoder(config_from_dict(fm.FUZE_U).model_spec(), dtype=torch.float32, device="cpu").cache_needs()
    assert -1 not in u and u[1][0].window is None and u[0][2] == SlotNeed((1, 24))     # one tap runs as two


LENS = {"S": [1, 9, 40, 67, 23], "U": [3, 50, 30], "W": [2, 17, 90, 33]}


@pytest.mark.parametrize("name", ["S", "U", "W"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_against_plain(fuzelorn_dirs, monkeypatch, name, cut):
    """The step function, cache manager and parts on the CPU, every launcher replaced by its plain statement: the
    states, pages and slots reach the right layer run of the right request however the work is cut."""
    kernel_refs.install(monkeypatch)
    cfg, w = fm.load_plain(fuzelorn_dirs[name])
    reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=17)
    ps = fm.PAGE_SIZE[name]
    cap = 128 if cut == "mixed" else 256
    runner = make_runner(fuzelorn_dirs[name], dtype=torch.float32, device="cpu", page_size=ps, num_pages=cap // ps,
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
    cfg, w = fm.load_plain(fm.write_model(fm.FUZE_S, 5, __import__("tempfile").mkdtemp()))
    toks = scenarios.make_requests([48], cfg["vocab"], seed=2)["r0"]
    a = plain.forward(cfg, w, toks)
    assert rel_err(a[:30], plain.forward(cfg, w, toks[:30])) < 1e-12
    # the recurrent state carries the first token far beyond every window; the pair embedding one token only
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert rel_err(plain.forward(cfg, w, other)[-1], a[-1]) > 1e-6
    wide = copy.deepcopy(cfg)
    wide["layers"][0]["mixer"]["left"]["mask"]["size"] += 1
    b = plain.forward(wide, w, toks)
    assert rel_err(b[:9], a[:9]) < 1e-12 and rel_err(b, a) > 1e-4
    for change in (lambda c: c["layers"][0]["mixer"]["left"]["q_temp"].update(every=6),
                   lambda c: c["loop"].update(times=1), lambda c: c.update(logit_softcap=8.0),
                   lambda c: c["embedding"]["bigram"].update(mul_prev=8),
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=3),
                   lambda c: c["layers"][1]["mlp"]["shared"].update(limit=0.7),
                   lambda c: c["layers"][3]["mlp"]["expert"].update(limit=0.8)):
        c = copy.deepcopy(cfg)
        change(c)
        assert rel_err(plain.forward(c, w, toks), a) > 1e-5
    for name in ("l0.mix.left.sink", "l1.mlp.correction", "l2.mix.right.A_log", "l1.mix.right.k.conv"):
        w2 = dict(w)
        w2[name] = w[name] + torch.linspace(-1.0, 1.0, w[name].shape[-1], dtype=torch.float64)      # not the same for all
        assert rel_err(plain.forward(cfg, w2, toks), a) > 1e-5, name
    assert plain.bigram_rows([3, 4, 4], {"buckets": 5, "mul_prev": 2, "mul_cur": 3}).tolist() == [5, (6 + 12) % 5, (8 + 12) % 5]
    assert plain.window_visible(6, {"size": 2}).tolist()[5] == [False, False, False, False, True, True]
    # choice by score plus correction among the kept groups; weights from the scores alone; a negative choice score wins over an excluded one
    z = torch.tensor([[2.0, 1.9, -9.0, -9.0, 0.1, 0.0]], dtype=torch.float64)
    corr = torch.tensor([0.0, 0.0, -0.9, -0.9, 0.5, 0.6], dtype=torch.float64)
    wts = plain.route(z, corr, {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}})
    s = torch.sigmoid(z[0])
    assert (wts[0] > 0).nonzero().flatten().tolist() == [0, 4, 5]        # the corrections lift 4 and 5 over 1
    assert abs(float(wts[0, 0]) - float(s[0] / (s[0] + s[4] + s[5]))) < 1e-12 and float(wts[0, 0]) > float(wts[0, 5])
    wts = plain.route(z, corr, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert (wts[0] > 0).nonzero().flatten().tolist() == [4, 5]           # a group's score is the sum of its two largest
    wts = plain.route(z, corr, {"experts": 6, "top": 2, "groups": {"count": 6, "keep": 1}} | {"top": 1})
    assert (wts[0] > 0).nonzero().flatten().tolist() == [5] and float(wts[0, 5]) == pytest.approx(1.0)
    lone = plain.route(torch.tensor([[-3.0, -2.0, 5.0, 5.0]], dtype=torch.float64), torch.tensor([0.0, 0.0, -2.0, -2.0], dtype=torch.float64),
                       {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert (lone[0] > 0).nonzero().flatten().tolist() == [0, 1]       # group 0 wins on corrected scores; its raw scores are small
