"""Kolorax without a device: configuration and registry, the spec's tensors and schedule, sizes taken from
tensor shapes, and the plain implementation against itself (whole sequences against token-by-token runs
with carried state)."""
import json

import pytest
import torch

import plain_kolorax as P
from test_kolorax_gpu import CONFIGS


def test_the_design_is_chosen_by_its_name_and_its_tensors_are_the_plain_model_s():
    from firefly_b200.models import config_from_dict, expected_weights, known_architectures, spec_for
    assert "Kolorax" in known_architectures() and "Qwen3ForCausalLM" in known_architectures()
    for name, cfg in CONFIGS.items():
        conf = config_from_dict(cfg)
        assert type(conf).__name__ == "KoloraxConfig" and conf.vocab_size == cfg["vocab"]
        spec = spec_for(conf)
        got = {w.name: tuple(w.shape) for w in expected_weights(spec)}
        assert got == P.tensor_shapes(cfg), name
        runs = [(layer, j) for (layer, _, _), j in zip(spec.resolved_schedule(), spec.resolved_junctions())]
        assert [(layer, None if j is None else j[1]) for layer, j in runs] == P.layer_runs(cfg), name
        slots = [slot for _, slot, _ in spec.resolved_schedule()]
        assert len(set(slots)) == len(slots)                       # every run of a looped layer has a cache of its own
        assert config_from_dict(conf.to_dict()) == conf


def test_sizes_that_only_tensor_shapes_give_are_read_from_them():
    from firefly_b200.models import config_from_dict, spec_for
    from firefly_b200.models.registry import apply_file_hints
    cfg = json.loads(json.dumps(CONFIGS["looped"]))
    for L in cfg["layers"]:
        L["mixer"].pop("decay_rank", None)
    shapes = {"l0.mix.w1": (12, 40), "l2.mix.w1": (5, 40), "l1.mix.q": (72, 40)}
    spec = spec_for(config_from_dict(apply_file_hints(cfg, shapes)))
    assert spec.layers[0].mixer.params["decay_rank"] == 12 and spec.layers[2].mixer.params["decay_rank"] == 5


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_wrong_configuration_is_told_by_name(edit, word):
    from firefly_b200.config import ConfigError
    from firefly_b200.models import config_from_dict
    cfg = json.loads(json.dumps(CONFIGS["looped"]))
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_experts_that_cannot_be_chosen_are_refused():
    from firefly_b200.config import PartSpec
    from firefly_b200.parts import Runtime, build_part
    rt = Runtime(torch.device("cpu"), torch.float32)
    good = dict(hidden_size=8, experts=6, top=2, groups=3, keep=2, ff=4, limit=1.0)
    build_part("feed_forward", PartSpec("grouped_experts", good, "m"), rt)
    for bad in (dict(good, groups=4), dict(good, keep=4), dict(good, top=5)):
        with pytest.raises(ValueError):
            build_part("feed_forward", PartSpec("grouped_experts", bad, "m"), rt)


def test_plain_mixers_carry_their_state():
    cfg = CONFIGS["looped"]
    w = P.random_weights(cfg, 3)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(23, 40, generator=g, dtype=torch.float64)
    whole, _ = P.wkv_mixer(x, w, "l0.mix", 2, 24, 1e-5)
    state, rows = None, []
    for a, b in ((0, 7), (7, 8), (8, 23)):
        out, state = P.wkv_mixer(x[a:b], w, "l0.mix", 2, 24, 1e-5, state)
        rows.append(out)
    assert torch.allclose(torch.cat(rows), whole, atol=1e-12)
    mx = cfg["layers"][1]["mixer"]
    kw = dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=32, scale=mx["scale"], base=mx["rot"]["base"], eps=1e-5)
    whole, _ = P.latent_attention_mixer(x, w, "l1.mix", torch.arange(23), **kw)
    cached, rows = None, []
    for a, b in ((0, 5), (5, 6), (6, 23)):
        out, cached = P.latent_attention_mixer(x[a:b], w, "l1.mix", torch.arange(a, b), cached=cached, **kw)
        rows.append(out)
    assert torch.allclose(torch.cat(rows), whole, atol=1e-12)


def test_plain_router_keeps_to_the_best_groups():
    z = torch.tensor([5.0, 0.0, 0.1, 0.2, 4.0, 3.9], dtype=torch.float64)     # groups (0,1) (2,3) (4,5)
    chosen, wts = P.route(z, top=2, group_count=3, group_keep=1)
    assert chosen == [0, 1] and abs(float(wts.sum()) - 1) < 1e-12             # 4 and 5 score higher than 1 but lie outside
    chosen, _ = P.route(z, top=2, group_count=3, group_keep=2)
    assert chosen == [0, 4]


def test_a_cache_group_of_one_plane_keeps_one_vector_a_token():
    from firefly_b200.cache import CacheManager, PagedKVSpec
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import Runtime
    model = DecoderModel(spec_for(config_from_dict(CONFIGS["looped"])), Runtime(torch.device("cpu"), torch.float32))
    specs = model.cache_slot_specs()
    paged = {s: sp for s, sp in specs.items() if isinstance(sp, PagedKVSpec)}
    assert len(paged) == 3 and all(sp.planes == 1 and sp.num_kv_heads == 1 and sp.head_dim == 40 for sp in paged.values())
    cm = CacheManager(specs, block_size=8, num_blocks=5, max_requests=2)
    cm.allocate_storage(torch.float32, "cpu")
    (g,) = cm.groups
    assert tuple(g.storage.shape) == (3, 6, 1, 1, 8, 40) and g.bytes_per_token(torch.float32) == 3 * 40 * 4
    two = CacheManager({0: PagedKVSpec(1, 40)}, block_size=8, num_blocks=5, max_requests=2)
    assert two.groups[0].bytes_per_token(torch.float32) == 2 * 40 * 4
    # the recurrent runs hold state slots: every head's state in the kernel's size, and the last input row
    states = {s: sp for s, sp in specs.items() if not isinstance(sp, PagedKVSpec)}
    assert sorted(sp.shape[0] for sp in states.values()) == sorted([2 * 32 * 32 + 40] * 3 + [3 * 32 * 32 + 40])
