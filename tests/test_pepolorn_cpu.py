"""Pepolorn without a device: its configuration, its spec (parts, schedule, cache slots, tensor names) and the plain
implementation's own consistency (the recurrences carried over a cut, the chunk mask)."""
import copy

import pytest
import torch

import plain_pepolorn as P
from firefly_b200.cache.spec import PagedKVSpec, StateSpec, sub_slot
from firefly_b200.config.base import ConfigError
from firefly_b200.models import config_from_dict, expected_weights, spec_for
from firefly_b200.models.decoder import DecoderModel
from firefly_b200.parts import Runtime

ATT = {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "scale": 0.4, "mask": {"size": 10},
       "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}}
LIN = {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.99]}
SSM = {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "conv": 3, "norm_groups": 2}
MOE = {"kind": "moe", "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}, "expert": {"ff": 16}}
CFG = {"architecture": "Pepolorn", "vocab": 60, "width": 32, "norm": {"eps": 1e-5}, "layers": [
    {"type": "mamba2", "mixer": SSM, "mlp": {"kind": "dense", "ff": 40}},
    {"type": "parallel", "mixer": {"left": ATT, "right": LIN, "left_scale": 1.2, "right_scale": 0.5}, "mlp": MOE},
    {"type": "mamba2", "mixer": SSM, "mlp": None},
    {"type": "parallel", "mixer": {"left": ATT, "right": LIN, "left_scale": 1.2, "right_scale": 0.5}, "mlp": MOE, "weights_of": 1},
]}


def test_the_spec_names_every_tensor_and_runs_a_shared_layer_twice():
    cfg = config_from_dict(CFG)
    spec = spec_for(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2, 1]
    names = {w.name: tuple(w.shape) for w in expected_weights(spec) if not w.optional}
    want = {k: tuple(v.shape) for k, v in P.random_weights(CFG, 0).items()}
    assert names == want
    assert not any(n.startswith("l3.") for n in names)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    slots = model.cache_slot_specs()
    # a cache or state per run: two state-space runs, and for each parallel run pages and a state
    assert sorted(slots) == [0, 2, sub_slot(1, 0), sub_slot(3, 0), sub_slot(1, 1), sub_slot(3, 1)]
    assert isinstance(slots[0], StateSpec) and isinstance(slots[sub_slot(3, 1)], StateSpec)
    kv = slots[sub_slot(1, 0)]
    assert isinstance(kv, PagedKVSpec) and (kv.num_kv_heads, kv.head_dim, kv.window) == (2, 24, None)
    assert slots[sub_slot(3, 0)] == kv


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "cannot be chosen"),
    (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][3].update(mlp=None), "differently"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_a_wrong_configuration_is_told_by_name(edit, word):
    raw = copy.deepcopy(CFG)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_optional_entries_may_be_absent():
    raw = copy.deepcopy(CFG)
    raw["layers"][1]["mixer"]["left"]["rot"]["scaling"] = None
    raw["layers"][3]["mixer"]["left"]["rot"]["scaling"] = None
    raw["layers"][1]["mlp"]["router"].pop("groups")
    raw["layers"][3]["mlp"]["router"].pop("groups", None)      # (the two layers may share one object)
    spec = spec_for(config_from_dict(raw))
    assert spec.layers[1].feed_forward.params["groups"] == 1 and spec.layers[1].feed_forward.params["keep"] == 1
    assert spec.layers[1].mixer.params["positions"][0].params["scaling"] is None


def test_rescaled_frequencies_of_the_position_part_are_the_plain_ones():
    from firefly_b200.config.base import PartSpec
    from firefly_b200.parts import build_part
    for rot in (ATT["rot"], {"base": 5000.0, "dims": 48, "scaling": {"factor": 16.0, "original": 512, "fast": 24.0, "slow": 2.0}},
                {"base": 50.0, "dims": 6, "scaling": None}):
        part = build_part("position", PartSpec("rotary", dict(head_dim=64, rotary_dim=rot["dims"], theta=rot["base"],
                                                             max_positions=0, scaling=rot["scaling"])),
                          Runtime(torch.device("cpu"), torch.float32))
        f, mag = P.rotary_frequencies(rot)
        assert torch.allclose(part.frequencies(), f, rtol=1e-14, atol=0) and abs(part.magnitude - mag) < 1e-15
    f, _ = P.rotary_frequencies(ATT["rot"])
    plain, _ = P.rotary_frequencies(dict(ATT["rot"], scaling=None))
    assert float(f[0]) == float(plain[0]) and abs(float(f[-1]) - float(plain[-1]) / 4.0) < 1e-12   # fast ones kept, slow ones stretched


def test_the_plain_recurrences_carry_over_a_cut_and_the_mask_is_by_chunks():
    w = P.random_weights(CFG, 3)
    x = torch.randn(23, 32, generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    whole, _ = P.lightning_attention(x, w, "l1.mix.right", LIN, 1e-5)
    a, S = P.lightning_attention(x[:9], w, "l1.mix.right", LIN, 1e-5)
    b, _ = P.lightning_attention(x[9:], w, "l1.mix.right", LIN, 1e-5, state=S)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
    # a row of the chunked attention depends on the rows of its own chunk only
    out = P.chunked_attention(x, w, "l1.mix.left", ATT, 1e-5)
    y = x.clone()
    y[:10] = torch.randn(10, 32, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    moved = P.chunked_attention(y, w, "l1.mix.left", ATT, 1e-5)
    assert torch.allclose(moved[10:], out[10:], atol=1e-12) and not torch.allclose(moved[9], out[9], atol=1e-6)
    # the whole model is causal and a request does not depend on the length it is run to
    toks = [5, 9, 2, 33, 8, 1, 0, 59, 17, 4, 4, 21, 6]
    full = P.forward(CFG, w, toks)
    assert torch.allclose(P.forward(CFG, w, toks[:7]), full[:7], atol=1e-9)


def test_the_router_keeps_to_open_groups_and_weights_by_the_plain_score():
    w = {"r.router": torch.zeros(6, 4, dtype=torch.float64), "r.correction": torch.tensor([0.0, -0.1, -0.9, -0.9, 0.3, -2.0], dtype=torch.float64)}
    ids, wts = P.route(torch.zeros(1, 4, dtype=torch.float64), w, "r", MOE["router"])
    # scores are all 0.5; group sums of the two best: (0.9, -0.8, -0.7): groups 0 and 2 are open, expert 4 and 0 chosen
    assert ids.tolist() == [[4, 0]] and wts.tolist() == [[0.5, 0.5]]
