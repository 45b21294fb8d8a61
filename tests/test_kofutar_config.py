"""Kofutar without a GPU: the configuration and its errors, the model as data (the loop's schedule, caches,
tensor names), the cache table that keys and values share, and the plain rules on hand cases."""
import copy

import numpy as np
import pytest

import plain_kofutar as PK
from kapel_b200.config import ConfigError, config_from_json

RAW = {"architecture": "Kofutar", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "conv": 3}, "mlp": {"kind": "dense", "ff": 16}},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 0.3,
                                    "rot": {"base": 1000.0, "dims": 4, "scaling": {"factor": 2.0}}}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 8, "q_rank": 10, "kv_rank": 12, "scale": 0.25,
                                           "rot": {"base": 50.0, "dims": 4}}, "mlp": {"kind": "dense", "ff": 20}},
]}


def test_round_trip_and_schedule():
    c = config_from_json(RAW)
    assert type(c).__name__ == "KofutarConfig" and config_from_json(c.to_json()) == c
    spec = c.to_spec()
    assert [(e.layer, e.replica, e.before is not None) for e in spec.schedule] == \
        [(0, 0, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False)]
    assert spec.layers[1].ffn is None and set(spec.layers[1].norms) == {"pre_mixer", "post_mixer"}
    assert all(n.kind == "layer" for l in spec.layers for n in l.norms.values()) and spec.final_norm.kind == "layer"
    assert spec.layers[1].mixer.position.divisor == 2.0 and spec.layers[1].mixer.position.rotary_dim == 4
    assert spec.layers[2].mixer.position.divisor == 1.0 and spec.head.weight == "head" and spec.embed.scale == 1.0
    no_loop = copy.deepcopy(RAW)
    del no_loop["loop"]
    assert [(e.layer, e.replica, e.before) for e in config_from_json(no_loop).to_spec().schedule] == [(0, 0, None), (1, 0, None), (2, 0, None)]
    whole = dict(copy.deepcopy(RAW), loop={"start": 0, "stop": 3, "times": 1})
    assert [e.before is not None for e in config_from_json(whole).to_spec().schedule] == [True, False, False]
    empty = dict(copy.deepcopy(RAW), loop={"start": 2, "stop": 2, "times": 5})           # no layer in the loop: nothing runs twice
    assert len(config_from_json(empty).to_spec().schedule) == 3


def test_tensor_names_and_shapes():
    from kapel_b200.parts import expected_tensors

    t = expected_tensors(config_from_json(RAW).to_spec())
    assert t["embed"] == (50, 24) and t["head"] == (50, 24) and t["loop.in"] == (24, 48) and t["final.norm"] == (24,)
    assert t["l0.mix.q"] == (8, 24) and t["l0.mix.v.conv"] == (24, 3) and t["l0.mix.A_log"] == (2,) and t["l0.mix.norm"] == (12,)
    assert t["l1.mix.q.norm"] == (8,) and t["l1.mix.v"] == (8, 24) and t["l1.mix.o"] == (24, 16) and "l1.norm2" not in t and "l1.mlp.up" not in t
    assert t["l2.mix.dkv"] == (16, 24) and t["l2.mix.uq"] == (20, 10) and t["l2.mix.uk"] == (12, 12) and t["l2.mix.uv"] == (16, 12)
    assert t["l2.mix.sink"] == (2,) and t["l2.mix.g"] == (16, 24) and t["l2.norm2b"] == (24,)


@pytest.mark.parametrize("edit,words", [
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=5), "even"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10), "more than"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][0]["mixer"].update(conv=0), "conv"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda r: r["loop"].update(stop=4), "loop.stop"),
    (lambda r: r["loop"].update(times=0), "loop.times"),
    (lambda r: r.pop("width"), "width"),
])
def test_errors_name_the_key(edit, words):
    raw = copy.deepcopy(RAW)
    edit(raw)
    with pytest.raises(ConfigError, match=words):
        config_from_json(raw)


def test_every_pass_of_the_loop_has_a_cache_and_latent_layers_one_table():
    import torch

    from kapel_b200.cache import CacheManager
    from kapel_b200.engine.model import ModelParts
    from kapel_b200.parts import BuildContext

    spec = config_from_json(RAW).to_spec()
    model = ModelParts(spec, BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 2, 4, 5]                                              # layers 1 and 2 once more, beyond the three layers
    assert needs[0].state is not None and needs[0].paged is None and needs[4].paged == needs[1].paged
    made = []
    cache = CacheManager(needs, 16, 4, 2, allocate=lambda shape, dtype: made.append(shape) or object(), dtype="float32")
    k, v = cache.tables(5)
    assert k is v and cache.tables(1)[0] is not cache.tables(1)[1]
    assert (4, 1, 16, 16) in made and (4, 2, 16, 8) in made and (4, 2, 16, 4) in made and len(cache.states) == 1


def test_plain_rules_on_hand_cases():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    y = PK.layer_norm(x, np.ones(4), 0.0)
    assert abs(y.mean()) < 1e-12 and abs((y * y).mean() - 1.0) < 1e-12
    # a filter of three taps: the last weighs the row itself, zeros before the start
    got = PK.short_conv(np.array([[1.0], [2.0], [4.0]]), np.array([[100.0, 10.0, 1.0]]))
    assert got[:, 0].tolist() == [1.0, 12.0, 124.0]
    # a quarter turn of the pair (0, 2); component 1 of `dims`' second half is 3; the rest passes
    r = PK.rotate(np.array([[[1.0, 0.0, 0.0, 0.0, 7.0]]]), [1], {"base": 1.0, "dims": 4, "scaling": {"factor": 2.0 / np.pi}})
    assert np.allclose(r[0, 0], [0.0, 0.0, 1.0, 0.0, 7.0])
    # a sink as large as the only score takes half
    w = PK.causal_softmax(np.array([[2.0]]), sink=2.0)
    assert np.allclose(w, [[0.5]])
    assert PK.layer_runs({"layers": [0, 1, 2], "loop": {"start": 1, "stop": 2, "times": 3}}) == [(0, False), (1, True), (1, True), (1, True), (2, False)]
