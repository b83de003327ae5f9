"""Surelorn without a GPU: reading its configuration, describing it as parts, the tensors it asks for,
a random model folder, and the plain implementation's own consistency."""

import copy
import json
import os

import pytest
import torch

import plain_surelorn as P
from surelorn_models import CONFIGS, ODD, SMALL, WIDE, random_weights, tensor_shapes, write_model

from paged_llm_rs_b200.config.registry import load_config, resolve_architecture
from paged_llm_rs_b200.errors import ConfigError, UnsupportedModelError
from paged_llm_rs_b200.parts.decoder import tensor_specs_of
from paged_llm_rs_b200.weights.loader import check_tensors
from paged_llm_rs_b200.weights.random_init import write_random_model
from paged_llm_rs_b200.weights.safetensors_io import open_model_files


def test_the_architecture_is_found_by_its_single_name():
    arch = resolve_architecture(SMALL)
    assert arch.name == "Surelorn"
    cfg = arch.parse(SMALL)
    assert cfg.width == 64 and cfg.vocab == 200 and cfg.embedding_scale == 4.0 and cfg.norm_eps == 1e-6
    assert [L.weights_of for L in cfg.layers] == [None, None, None, 1, 0]
    assert cfg.layers[2].mlp_kind is None and cfg.layers[1].routed.group_keep == 2 and cfg.layers[1].routed.shared_ff == 32


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_described_model_asks_for_exactly_the_tensors_of_the_file(name):
    cfg = CONFIGS[name]
    arch = resolve_architecture(cfg)
    spec = arch.describe(arch.parse(cfg))
    asked = {t.name: tuple(t.shape) for t in tensor_specs_of(spec)}
    assert asked == {k: tuple(s) for k, (s, _) in tensor_shapes(cfg).items()}
    check_tensors(tensor_specs_of(spec), asked)


def test_layers_that_borrow_tensors_are_further_runs_of_the_lender():
    arch = resolve_architecture(SMALL)
    spec = arch.describe(arch.parse(SMALL))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2, 1, 0]
    assert spec.layers[2].feed_forward is None and "feed_forward" not in spec.layers[2].norms
    assert all(e.reads_cache_of is None for e in spec.schedule)        # every run keeps a cache of its own


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), UnsupportedModelError),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "maxout"), UnsupportedModelError),
    (lambda c: c["layers"][3].__setitem__("weights_of", 3), ConfigError),
    (lambda c: c["layers"][4].__setitem__("weights_of", 3), ConfigError),          # a borrower lends nothing
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), ConfigError),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), ConfigError),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), ConfigError),
    (lambda c: c.__setitem__("width", 63), ConfigError),
    (lambda c: c["norm"].__setitem__("eps", 0.0), ConfigError),
    (lambda c: c.pop("layers"), ConfigError),
])
def test_what_the_configuration_refuses(change, error):
    c = copy.deepcopy(SMALL)
    change(c)
    arch = resolve_architecture(c)
    with pytest.raises(error):
        arch.parse(c)


def test_random_model_folder_round_trip(tmp_path):
    d = write_random_model(str(tmp_path / "m"), ODD, seed=3)
    arch, cfg = load_config(d)
    assert arch.name == "Surelorn" and cfg.layers[0].routed.identity == 3
    files = open_model_files(d)
    names = {n for f in files for n in f.names()}
    assert names == set(tensor_shapes(ODD))
    assert files[0].tensor("l0.mlp.correction").float().abs().max() > 0     # a correction that steers something


def test_plain_pieces_agree_with_themselves():
    """The plain implementation's prefix property (causality) and its router's invariants."""
    cfg = SMALL
    w = {k: v.double() for k, v in random_weights(cfg, 1).items()}
    toks = [5, 9, 150, 3, 77, 12, 199, 0, 42]
    full = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:5])
    assert torch.allclose(full[:5], part, atol=1e-10)
    x = torch.randn(7, cfg["width"], dtype=torch.float64)
    r = cfg["layers"][1]["mlp"]["router"]
    picks, weights = P.route(w, "l1.mlp", r, x)
    per = (r["experts"] + r.get("identity", 0)) // r["groups"]["count"]
    for chosen, ws in zip(picks, weights):
        assert len(set(chosen)) == r["top"] and abs(sum(ws) - 1) < 1e-12
        assert len({j // per for j in chosen}) <= r["groups"]["keep"]
    pv = P.position_vectors([0, 3], 8)
    assert torch.allclose(pv[0], torch.tensor([0., 1.] * 4, dtype=torch.float64))
    assert abs(float(pv[1, 0]) - 0.1411200080598672) < 1e-12 and abs(float(pv[1, 2]) - 0.29552020666133955) < 1e-12
