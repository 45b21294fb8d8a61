"""Fusitar without a GPU: its configuration, its specs and tensor names, the cache's kept first
pages, and the plain implementation's own rules on hand cases."""
import math

import numpy as np
import pytest

import plain_fusitar as PF
from kapel_b200.cache import CacheManager, CacheNeeds, PagedKV
from kapel_b200.config import ConfigError, FusitarConfig, config_from_json
from kapel_b200.parts import expected_tensors
from plain_cache import PlainCacheManager

RAW = {"architecture": "Fusitar", "vocab": 50, "width": 24, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "layers": [
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 6, "vdim": 4, "gate_cap": 9.0}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.3, "mask": {"size": 9, "keep_first": 2}},
     "mlp": {"kind": "moe", "expert": {"ff": 14}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
]}


def test_config_is_read_registered_and_written_back():
    c = config_from_json(RAW)
    assert isinstance(c, FusitarConfig) and c.vocab == 50 and len(c.layers) == 2
    assert FusitarConfig.from_json(c.to_json()) == c
    spec = c.to_spec()
    assert [b.kind for b in spec.layers] == ["postnorm", "postnorm"] and spec.layers[0].ffn is None
    att = spec.layers[1].mixer
    assert (att.window, att.keep_first, att.v_head_dim, att.gated, att.position.kind) == (9, 2, 10, True, "none")
    assert att.q_norm.width == 24 and att.k_norm.width == 12 and att.q_norm.offset == 0.0
    moe = spec.layers[1].ffn
    assert (moe.experts, moe.top, moe.groups, moe.keep_groups, moe.group_top, moe.scoring, moe.renormalize) == (6, 2, 3, 2, 2, "sigmoid", False)
    names = expected_tensors(spec)
    assert names["l0.mix.i"] == (2, 24) and names["l0.mix.f.b"] == (2,) and names["l0.mix.norm"] == (8,)
    assert names["l1.mix.v"] == (20, 24) and names["l1.mix.g"] == (40, 24) and names["l1.mix.o"] == (24, 40)
    assert names["l1.mlp.e5.down"] == (24, 14) and names["l1.mlp.correction"] == (6,) and "l0.norm2" not in names
    assert names["embed"] == (50, 24) and "final.norm" in names


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 1, "mlp", "router", "groups", "count"), 4),
    (("layers", 1, "mlp", "router", "top"), 5), (("layers", 0, "mixer", "gate_cap"), None), (("width",), 0), (("layers",), []),
])
def test_config_errors_name_the_key(path, value):
    import copy

    raw = copy.deepcopy(RAW)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        config_from_json(raw)


def test_a_windowed_group_keeps_the_pages_of_its_first_positions():
    needs = {0: CacheNeeds(paged=PagedKV(1, 8, window=20, keep_first=18)), 1: CacheNeeds(paged=PagedKV(1, 8, window=20))}
    m = CacheManager(needs, 16, 32, 2)
    p = PlainCacheManager([(20, 32, 18), (20, 32)], 16, 2)
    for c in (m, p):
        c.add_sequence("s")
        for n in (50, 1, 1, 70, 3):
            c.commit(c.plan([("s", n)]))
    for g in (0, 1):
        assert m.page_list("s", g) == [int(x) for x in p._sequences["s"].pages[g]]
    kept, plain_window = m.page_list("s", 0), m.page_list("s", 1)
    assert kept[0] >= 0 and kept[1] >= 0 and kept[2] == -1, "positions 0..17 lie on the first two pages"
    assert plain_window[0] == -1 and plain_window[1] == -1
    m.remove_sequence("s")
    m.check()
    assert m.free_pages() == m.total_pages()


def test_visibility_rule():
    assert PF.visible(10, 10, 3, 0) and PF.visible(10, 8, 3, 0) and not PF.visible(10, 7, 3, 0)
    assert PF.visible(10, 1, 3, 2) and not PF.visible(10, 2, 3, 2) and not PF.visible(3, 4, 3, 2)


def test_recurrence_is_the_plain_gated_sum_when_nothing_overflows():
    """With small gates the running maximum only rescales: S_t = sum_s exp(gi_s + sum_{s<u<=t} gf_u) k_s v_s^T."""
    rng = np.random.default_rng(0)
    T, d, e = 9, 3, 2
    q, k, v = rng.standard_normal((T, d)), rng.standard_normal((T, d)), rng.standard_normal((T, e))
    gi, gf = 0.3 * rng.standard_normal(T), -np.abs(rng.standard_normal(T))
    got = PF.mlstm_recurrence(q, k, v, gi, gf)
    for t in range(T):
        S, n = np.zeros((d, e)), np.zeros(d)
        for s in range(t + 1):
            w = math.exp(gi[s] + gf[s + 1 : t + 1].sum())
            S += w * np.outer(k[s], v[s])
            n += w * k[s]
        m = 0.0
        for s in range(t + 1):
            m = max(gf[s] + m, gi[s])
        want = (S.T @ q[t]) / (max(abs(n @ q[t]), 1.0) * math.exp(-m) + 1e-6) * math.exp(-m)
        assert np.allclose(got[t], want, rtol=1e-9, atol=1e-12)


def test_routing_by_hand():
    # groups (0,1) (2,3) (4,5): choice scores below; the best two groups are the first and the last
    z = np.log(np.array([0.6, 0.5, 0.9, 0.1, 0.55, 0.58]) / (1 - np.array([0.6, 0.5, 0.9, 0.1, 0.55, 0.58])))
    corr = np.array([0.0, 0.0, -0.5, 0.0, 0.0, 0.0])
    chosen, weights = PF.route(z, corr, top=2, groups=3, keep=2)
    assert chosen == [0, 5] and np.allclose(weights, [0.6, 0.58])
    # negative choice scores everywhere: the dropped group's experts must not win as zeros would
    corr = np.full(6, -2.0)
    chosen, _ = PF.route(z, corr, top=3, groups=3, keep=2)
    assert chosen == [0, 5, 4]
