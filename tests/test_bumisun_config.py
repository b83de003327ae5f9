"""Bumisun without a GPU: the configuration reader, the description as parts, the tensors it asks for, the cache
manager's kept pages, and the plain implementation against itself."""

import copy

import pytest
import torch

import plain_bumisun as P
from bumisun_models import CONFIGS, ODD, SMALL, random_weights, tensor_shapes

from paged_llm_rs_b200.cache.manager import CacheManager
from paged_llm_rs_b200.config.registry import resolve_architecture
from paged_llm_rs_b200.errors import ConfigError, UnsupportedModelError
from paged_llm_rs_b200.parts.base import JoinedKVNeed, StateNeed
from paged_llm_rs_b200.parts.decoder import DecoderModel, Runtime, tensor_specs_of


def describe(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.describe(arch.parse(cfg))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_parts_ask_for_exactly_the_files_tensors(name):
    cfg = CONFIGS[name]
    arch, spec = describe(cfg)
    assert arch.name == "Bumisun"
    asked = {s.name: tuple(s.shape) for s in tensor_specs_of(spec)}
    assert asked == {n: tuple(shape) for n, (shape, _) in tensor_shapes(cfg).items()}


def test_every_constant_comes_from_the_configuration():
    cfg = copy.deepcopy(SMALL)
    cfg["residual_mult"], cfg["logit_scale"], cfg["norm"]["eps"] = 0.3, 2.0, 1e-3
    cfg["layers"][0]["mixer"].update(scale=0.7, softcap=5.0)
    cfg["layers"][0]["mixer"]["mask"] = dict(size=11, keep_first=6)
    cfg["layers"][0]["mixer"]["rot"] = dict(dims=4, base=77.0)
    cfg["layers"][0]["mlp"]["expert"]["limit"] = 0.25
    cfg["layers"][0]["mlp"]["shared"]["limit"] = 9.0
    _, spec = describe(cfg)
    a, f = spec.layers[0].mixer.params, spec.layers[0].feed_forward.params
    assert (a["scale"], a["softcap"], a["window"], a["keep_first"], a["rot_dims"], a["rot_base"]) == (0.7, 5.0, 11, 6, 4, 77.0)
    assert (f["limit"], f["shared_limit"], f["activation"]) == (0.25, 9.0, "clamped")
    assert spec.final_norm.params["mult"] == 0.3 and spec.final_norm.params["eps"] == 1e-3 and spec.head.params["scale"] == 2.0
    assert spec.layers[1].mixer.params["eps"] == 1e-3


def test_the_first_mixing_layer_is_the_source():
    _, spec = describe(SMALL)
    assert [L.mixer.params.get("value_mix") for L in spec.layers] == ["source", None, "mixed", None, "mixed"]
    assert spec.layers[2].feed_forward is None and "feed_forward" not in spec.layers[2].norms


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="ring"), UnsupportedModelError),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), ConfigError),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), ConfigError),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), ConfigError),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), ConfigError),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), UnsupportedModelError),
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), ConfigError),          # value-mixing layers of two shapes
    (lambda c: c["norm"].update(eps=0.0), ConfigError),
    (lambda c: c.pop("layers"), ConfigError)])
def test_bad_configurations_are_refused(change, error):
    cfg = copy.deepcopy(SMALL)
    change(cfg)
    with pytest.raises(error):
        describe(cfg)


def test_cache_needs_and_groups():
    _, spec = describe(SMALL)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    needs = model.cache_needs()
    assert isinstance(needs[1], StateNeed) and needs[1].shape == (4 * 16 * 8 + 3 * (32 + 32),)
    assert isinstance(needs[0], JoinedKVNeed) and (needs[0].window, needs[0].keep_first) == (20, 3)
    cm = CacheManager(needs, 8, 16, 4, torch.float32, "cpu", allocate_device=False)
    assert [len(g.entries) for g in cm.groups] == [3, 1]       # the three alike share pages and tables
    assert cm.prefix_cache is False


def test_a_window_group_keeps_the_pages_of_the_first_tokens():
    need = JoinedKVNeed("window", 2, 16, 8, window=20, keep_first=9, group_size=3)
    cm = CacheManager([need], 8, 12, 2, torch.float32, "cpu", allocate_device=False)
    cm.open("a")
    for n in (30, 1, 1, 40, 1):
        assert cm.reserve("a", n)
        cm.commit("a", n)
    t = cm.get("a").tables[0]
    # 73 tokens: the next query sees from 73 - 20 + 1 = 54 on (page 6 on) and the first 9 (pages 0 and 1)
    assert [b >= 0 for b in t.blocks] == [True, True, False, False, False, False, True, True, True, True]
    cm.check_invariants()
    assert cm.groups[0].allocator.available() == 12 - 6
    cm.close("a")
    assert cm.groups[0].allocator.available() == 12
    assert cm.pages_for(1000, step_tokens=16) == 5 + 1 + 2


def test_plain_token_by_token_equals_whole():
    """The plain implementation keeps nothing between calls: a prefix's logits are the whole's."""
    for cfg in (SMALL, ODD):
        w = {k: v.double() for k, v in random_weights(cfg, 3).items()}
        toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
        whole = P.forward(cfg, w, toks)
        assert torch.allclose(P.forward(cfg, w, toks[:17]), whole[:17], atol=1e-9)


def test_plain_mechanisms_alone():
    # the window and the kept first tokens
    assert [j for j in range(12) if P.visible(10, j, 3, 2)] == [0, 1, 8, 9, 10]
    # a sink of minus infinity is no sink; a huge one silences the head
    q, k, v = torch.randn(1, 1, 4, dtype=P.F64), torch.randn(3, 1, 4, dtype=P.F64), torch.randn(3, 1, 2, dtype=P.F64)
    none = P.sink_window_attention(q, k, v, [2], 0.5, 0.0, 10, 0, torch.tensor([-1e30], dtype=P.F64))
    assert torch.allclose(none[0, 0], torch.softmax((k[:, 0] @ q[0, 0]) * 0.5, 0) @ v[:, 0])
    assert float(P.sink_window_attention(q, k, v, [2], 0.5, 0.0, 10, 0, torch.tensor([50.0], dtype=P.F64)).abs().max()) < 1e-15
    # rotation turns pairs (i, i + dims / 2) and leaves the rest
    x = torch.arange(8, dtype=P.F64).view(1, 1, 8)
    r = P.rotate(x, [3], 4, 10.0)
    assert torch.equal(r[..., 4:], x[..., 4:]) and abs(float(r[0, 0, 0]) - (0 * torch.cos(torch.tensor(3.0)) - 2 * torch.sin(torch.tensor(3.0)))) < 1e-6
    # the router: the largest logits, softmax over them alone
    ids, wt = P.route(torch.eye(3, dtype=P.F64)[:1], torch.tensor([[1.0, 0, 0], [3.0, 0, 0], [2.0, 0, 0]], dtype=P.F64),
                      torch.tensor([0.0, 0.0, 5.0], dtype=P.F64), 2)
    assert ids.tolist() == [[2, 1]] and torch.allclose(wt, torch.softmax(torch.tensor([[7.0, 3.0]], dtype=P.F64), -1))
    # the clamped activation
    w = {"e.gate": torch.ones(1, 1, dtype=P.F64), "e.up": torch.ones(1, 1, dtype=P.F64), "e.down": torch.ones(1, 1, dtype=P.F64)}
    y = P.clamped_expert(torch.tensor([[5.0]], dtype=P.F64), w, "e", 2.0)
    assert abs(float(y) - 2.0 * float(torch.sigmoid(torch.tensor(1.702 * 2.0, dtype=P.F64))) * 3.0) < 1e-9
