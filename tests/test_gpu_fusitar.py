"""Fusitar on the GPU: each mechanism's kernels against the plain functions of `plain_fusitar`, and
the engine (step function, cache, scheduler, entry point) against the plain forward pass, on two
small configurations that differ in every size, constant and in the order of their layers."""
import json

import numpy as np
import pytest
import torch

import plain_fusitar as PF
from helpers import TraceBuilder, compare_trace, random_tokens, rel_err, run_trace_engine

pytestmark = pytest.mark.gpu


def attention_layer(heads, kv_heads, dim, vdim, scale, size, keep_first, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                      "mask": {"size": size, "keep_first": keep_first}}}


def mlstm_layer(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def moe(experts, top, count, keep, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


# A: values of another size than keys, a layer without a feed-forward, a window shorter than a page
# and one longer, groups of which half are kept. B: starts with two recurrent layers, one key/value
# head, a single group, one expert a token, other eps and scales.
FUSITAR_A = {"architecture": "Fusitar", "vocab": 211, "width": 64, "embedding": {"scale": 6.5}, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(4, 2, 16, 24, 0.21, 20, 3, moe(8, 3, 4, 2, 40)),
    mlstm_layer(2, 24, 16, 8.0, moe(8, 3, 4, 2, 40)),
    attention_layer(2, 2, 8, 6, 0.4, 7, 0, None),
    mlstm_layer(4, 8, 8, 12.0, moe(4, 2, 2, 2, 20)),
]}
FUSITAR_B = {"architecture": "Fusitar", "vocab": 97, "width": 96, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "layers": [
    mlstm_layer(3, 16, 32, 15.0, moe(6, 1, 1, 1, 24)),
    mlstm_layer(1, 40, 20, 5.0, None),
    attention_layer(6, 1, 32, 32, 0.125, 33, 5, moe(6, 2, 3, 2, 56)),
]}
CONFIGS = {"A": (FUSITAR_A, 11), "B": (FUSITAR_B, 12)}
# Largest difference of logits over the largest plain logit. In 32-bit the runs see 2e-5; in bfloat16 (products
# and caches in bfloat16 under 32-bit norms, scores and recurrences) these small models, whose logits are a few tenths, see up to 8e-2 (the kernels alone are held to 2e-2 and 3e-2 above).
TOL = {"float32": 1e-4, "bfloat16": 1e-1}


def make_folder(raw, seed, tmp):
    from kapel_b200.config import config_from_json
    from kapel_b200.weights import write_random_model

    return write_random_model(tmp, config_from_json(raw), seed)


def read_tensors(folder):
    """{name: float64 array} of a folder's model.safetensors, read with this file's own few lines."""
    blob = (folder / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8 : 8 + n])
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = np.frombuffer(blob[8 + n + a : 8 + n + b], dtype="<u2" if rec["dtype"] == "BF16" else "<f4")
        if rec["dtype"] == "BF16":
            raw = (raw.astype(np.uint32) << 16).view(np.float32)
        out[name] = raw.reshape(rec["shape"]).astype(np.float64)
    return out


def far_apart(experts, groups, seed):
    """Corrections (exact in bfloat16) such that any two experts' values, and any two groups' sums
    of their two largest, differ by at least 0.25."""
    rng = np.random.default_rng(seed)
    per = experts // groups
    while True:
        c = rng.integers(-24, 25, size=experts) / 8.0
        sums = [np.sort(c[g * per : (g + 1) * per])[::-1][:2].sum() for g in range(groups)]
        gap = lambda v: np.diff(np.sort(np.asarray(v))).min() if len(v) > 1 else 1.0
        if gap(c) >= 0.25 and gap(sums) >= 0.25:
            return c


def make_routers_decisive(folder):
    """Rewrites a folder's routers so that no choice of experts is a close call: the scores move
    little from token to token and the corrections (and the groups' sums of them) lie far apart. A bfloat16
    run then chooses the experts the 64-bit plain implementation chooses; the weights still
    follow the scores. (Random routers are what the 32-bit runs and the router's own test use.)"""
    from kapel_b200.config import config_from_dir
    from kapel_b200.parts import expected_tensors
    from kapel_b200.weights import load_tensors, write_safetensors

    tensors = load_tensors(folder, expected_tensors(config_from_dir(folder)[0].to_spec()), "cpu")
    tensors = {name: t.clone() for name, t in tensors.items()}       # the loader's tensors are views of the file about to be rewritten
    raw = json.loads((folder / "config.json").read_text())
    for i, layer in enumerate(raw["layers"]):
        if layer["mlp"] is None:
            continue
        r = layer["mlp"]["router"]
        tensors[f"l{i}.mlp.router"] = (tensors[f"l{i}.mlp.router"].float() * 0.02).to(torch.bfloat16)
        tensors[f"l{i}.mlp.correction"] = torch.tensor(far_apart(r["experts"], r["groups"]["count"], seed=i), dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per configuration: random weights (for the 32-bit runs), and the same with decisive routers
    (for the bfloat16 runs), each as (folder, config.json's dict, tensors in 64-bit)."""
    out = {}
    for name, (raw, seed) in CONFIGS.items():
        for variant in ("", "_decisive"):
            folder = make_folder(raw, seed, tmp_path_factory.mktemp(f"fusitar_{name}{variant}"))
            if variant:
                make_routers_decisive(folder)
            out[name + variant] = (folder, raw, read_tensors(folder))
    return out


def variant_for(name, dtype):
    return name + ("_decisive" if dtype == "bfloat16" else "")


_PLAIN = {}


def plain(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        _, raw, t = models[name]
        _PLAIN[key] = PF.forward(raw, t, list(tokens))
    return _PLAIN[key]


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda").contiguous()


# --------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,dv,size,keep", [(4, 2, 16, 24, 20, 3), (3, 1, 40, 10, 300, 270), (2, 2, 12, 7, 5, 0), (8, 1, 64, 64, 64, 17),
                                                   (4, 2, 48, 48, 90, 130), (6, 3, 128, 128, 200, 1)])
def test_attention_with_kept_first_keys_against_plain(dtype, hq, hkv, d, dv, size, keep):
    """The norm over the whole projections, the append and the attention kernel over shuffled pages,
    in two portions, against the plain mixer's pieces; lengths cross pages, the window and the chunk."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(hq * 100 + d)
    T, page = 600, 16
    eps, scale = 1e-5, 0.3
    q = rng.standard_normal((T, hq * d))
    k = rng.standard_normal((T, hkv * d))
    v = rng.standard_normal((T, hkv * dv))
    wq, wk = rng.standard_normal(hq * d), rng.standard_normal(hkv * d)
    if dtype == torch.bfloat16:
        r = lambda a: torch.tensor(a, dtype=torch.bfloat16).double().numpy()
        wq, wk = r(wq), r(wk)
    qn = PF.rms_norm(q, wq, eps).reshape(T, hq, d)
    kn = PF.rms_norm(k, wk, eps).reshape(T, hkv, d)
    vv = v.reshape(T, hkv, dv)
    want = np.zeros((T, hq, dv))
    for h in range(hq):
        g = h // (hq // hkv)
        want[:, h] = PF.attention_scores(qn[:, h], kn[:, g], scale, size, keep) @ vv[:, g]

    n_pages = -(-T // page) + 3
    pages = rng.permutation(n_pages)[: -(-T // page)]
    k_table = torch.zeros((n_pages, hkv, page, d), dtype=dtype, device="cuda")
    v_table = torch.zeros((n_pages, hkv, page, dv), dtype=dtype, device="cuda")
    table = dev(pages[None, :], torch.int32)
    stacked = dev(np.concatenate([q, k, v], axis=1))
    got = []
    for a, b in ((0, 333), (333, T)):
        pos = np.arange(a, b)
        lines = dev(pages[pos // page] * page + pos % page, torch.int32)
        part = stacked[a:b].contiguous()
        if a:                                                # the second portion comes as split-K partial sums: two slices that add up to it
            noise = torch.randn_like(part)
            part = K.SplitSum(torch.stack([noise, part - noise]).contiguous())
        qq = K.proj_norm_append(part, 0, hq * d, hq * d + hkv * d, (dev(wq, dtype), eps, 0.0), (dev(wk, dtype), eps, 0.0),
                                lines, k_table, v_table, hq, hkv, d, dv, True, dtype)
        slots = min(-(-b // K.attention_chunk()), (size - 1) // K.attention_chunk() + 2) + K.attention_keep_slots(size, keep)
        y = K.paged_attention_rows(qq, k_table, v_table, table, dev(np.zeros(b - a), torch.int32), dev(pos + 1, torch.int32),
                                   page, size, scale, None, slots, keep)
        got.append(y.float().cpu().numpy())
        if dtype == torch.bfloat16 and d == dv and K.attention_mma_takes(dtype, d, hq // hkv):
            # the same portion through the tensor-core kernel for prompt portions
            from kapel_b200.engine.batch import cut_tiles

            tiles = tuple(dev(t, torch.int32) for t in cut_tiles(np.asarray([0]), np.asarray([b - a]), K.attention_mma_rows(False) // (hq // hkv)))
            z = K.paged_attention_mma(qq, k_table, v_table, table, dev(pos + 1, torch.int32), tiles, page, size, scale, None, 0, 0, 1,
                                      keep_first=keep)
            assert rel_err(z.float().cpu().numpy(), want[a:b]) < 3e-2
    err = rel_err(np.concatenate(got), want)
    assert err < (2e-5 if dtype == torch.float32 else 3e-2), err


@pytest.mark.parametrize("dtype,dv", [(torch.float32, 8), (torch.bfloat16, 8), (torch.bfloat16, 16)])
def test_a_window_and_its_kept_keys_are_exact_to_the_token(dtype, dv):
    """One key's score is made to stand out: the output is that key's value exactly when the plain
    rule says the query sees it. Keys just inside and just outside the window and the kept first
    tokens, at page borders and far back, for a prompt's rows and for a single decoded token."""
    from kapel_b200 import kernels as K

    hq = hkv = 1
    d, page, size, keep, T = 16, 16, 37, 5, 420
    rng = np.random.default_rng(5)
    n_pages = -(-T // page)
    pages = rng.permutation(n_pages)
    table = dev(pages[None, :], torch.int32)
    pos = np.arange(T)
    lines = dev(pages[pos // page] * page + pos % page, torch.int32)
    v = rng.standard_normal((T, dv))
    for target in (0, 4, 5, 6, 15, 16, 100, 255, 256, 300):
        k = 0.01 * rng.standard_normal((T, d))
        k[target, 0] = 30.0                                 # with q = (1, 0, ...) this key's score is 30, all others near 0
        stacked = dev(np.concatenate([np.tile(np.eye(1, d), (T, 1)), k, v], axis=1))
        k_table = torch.zeros((n_pages, hkv, page, d), dtype=dtype, device="cuda")
        v_table = torch.zeros((n_pages, hkv, page, dv), dtype=dtype, device="cuda")
        q = K.proj_norm_append(stacked, 0, d, 2 * d, None, None, lines, k_table, v_table, hq, hkv, d, dv, True, dtype)
        queries = sorted({i for i in (target, target + 1, target + size - 1, target + size, target + size + 1, T - 1) if target <= i < T})
        slots = (size - 1) // K.attention_chunk() + 2 + K.attention_keep_slots(size, keep)
        # as a prompt's rows, all at once
        rows = K.paged_attention_rows(q, k_table, v_table, table, dev(np.zeros(T), torch.int32), dev(pos + 1, torch.int32),
                                      page, size, 1.0, None, slots + T // K.attention_chunk(), keep).float().cpu().numpy()
        ways = [rows]
        if dtype == torch.bfloat16 and d == dv:               # and through the tensor-core kernel for prompt portions
            from kapel_b200.engine.batch import cut_tiles

            tiles = tuple(dev(t, torch.int32) for t in cut_tiles(np.asarray([0]), np.asarray([T]), K.attention_mma_rows(False)))
            ways.append(K.paged_attention_mma(q, k_table, v_table, table, dev(pos + 1, torch.int32), tiles, page, size, 1.0, None, 0, 0, 1,
                                              keep_first=keep).float().cpu().numpy())
        vt = v_table.float().cpu().numpy()
        stored = vt[pages[target // page], 0, target % page]
        for i in queries:
            # and as one decoded token
            one = K.paged_attention_rows(q[i : i + 1].contiguous(), k_table, v_table, table, dev([0], torch.int32), dev([i + 1], torch.int32),
                                         page, size, 1.0, None, slots, keep).float().cpu().numpy()[0, 0]
            sees = PF.visible(i, target, size, keep)
            for got in [w[i, 0] for w in ways] + [one]:
                hit = np.abs(got - stored).max() < 1e-3
                assert hit == sees, f"query {i}, key {target}: visible {sees}, output follows the key {hit}"


@pytest.mark.parametrize("unit", [False, True])
def test_head_gate_against_plain(unit):
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(3)
    rows, heads, e = 37, 3, 20
    y, g, w = rng.standard_normal((rows, heads, e)), 3 * rng.standard_normal((rows, 7 + heads * e)), rng.standard_normal(heads * e)
    want = (PF.rms_unit(y, 1e-4) if unit else y).reshape(rows, -1) * (w if unit else 1.0) * PF.sigmoid(g[:, 7:])
    got = K.head_gate(dev(y), dev(g), 7, dev(w) if unit else None, unit, 1e-4, torch.float32)
    assert rel_err(got.cpu().numpy().reshape(rows, -1), want) < 1e-5
    wide = K.head_gate(dev(y), dev(g), 7, dev(w) if unit else None, unit, 1e-4, torch.float32, pad_to=64).cpu().numpy()
    assert wide.shape == (rows, 64) and np.array_equal(wide[:, :60], got.cpu().numpy().reshape(rows, -1)) and not wide[:, 60:].any()
    # the gate as split-K partial sums (what a product of a few rows leaves): three slices that add up to it
    parts = rng.standard_normal((3, rows, g.shape[1]))
    parts[2] = g - parts[0] - parts[1]
    split = K.head_gate(dev(y), K.SplitSum(dev(parts)), 7, dev(w) if unit else None, unit, 1e-4, torch.float32)
    assert rel_err(split.cpu().numpy().reshape(rows, -1), want) < 1e-5


@pytest.mark.parametrize("heads,d,e,cap", [(2, 24, 16, 8.0), (3, 9, 33, 15.0), (1, 130, 20, 2.0)])
def test_mlstm_scan_in_portions_and_token_by_token_against_plain(heads, d, e, cap):
    """Three requests of unequal length: whole, then in portions down to two tokens beside each
    other's single tokens, through slots that are used again; the state carries across steps."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(d)
    lengths = {"a": 150, "b": 37, "c": 64}
    width = 2 * heads * d + heads * e + 2 * heads
    data, want = {}, {}
    bi, bf = rng.standard_normal(heads), 2 + rng.standard_normal(heads)
    for name, T in lengths.items():
        x = rng.standard_normal((T, width))
        x[:, -2 * heads :] *= 4.0                           # gates that swing, so that the running maximum moves both ways
        data[name] = x
        q = x[:, : heads * d].reshape(T, heads, d) * d ** -0.5
        k = x[:, heads * d : 2 * heads * d].reshape(T, heads, d)
        v = x[:, 2 * heads * d : 2 * heads * d + heads * e].reshape(T, heads, e)
        gi = cap * np.tanh((x[:, -2 * heads : -heads] + bi) / cap)
        gf = PF.log_sigmoid(cap * np.tanh((x[:, -heads:] + bf) / cap))
        want[name] = np.stack([PF.mlstm_recurrence(q[:, h], k[:, h], v[:, h], gi[:, h], gf[:, h]) for h in range(heads)], axis=1)
    state = torch.zeros((3, heads, K.mlstm_state_floats(d, e)), dtype=torch.float32, device="cuda")

    def run(step):                                           # step: [(name, slot, a, b)]
        rows = np.concatenate([data[n][a:b] for n, _, a, b in step])
        entry = np.concatenate([np.full(b - a, i) for i, (_, _, a, b) in enumerate(step)])
        ranges = K.entry_ranges(dev(entry, torch.int32), len(step))
        rows = dev(rows)
        if len(rows) <= 4:                                   # a few rows come as split-K partial sums, as a small product leaves them
            # slices whose sum is the row exactly: its upper bits, the rest, and zeros (random slices left a
            # rounding error that the gates' exponentials magnified differently from run to run)
            upper = (rows.view(torch.int32) & -4096).view(torch.float32)
            rows = K.SplitSum(torch.stack([upper, rows - upper, torch.zeros_like(rows)]).contiguous())
        out = K.mlstm_scan(rows, 0, heads * d, 2 * heads * d, width - 2 * heads, width - heads, dev(bi), dev(bf), state, ranges,
                           dev([s for _, s, _, _ in step], torch.int32), len(step), heads, d, e, cap, d ** -0.5, 1e-6).cpu().numpy()
        at = 0
        for n, _, a, b in step:
            err = float(np.abs(out[at : at + b - a] - want[n][a:b]).max() / np.abs(want[n]).max())      # against the request's largest value
            assert err < 5e-5, f"{n}[{a}:{b}]: {err:.2e}"
            at += b - a

    run([("a", 1, 0, 150), ("b", 2, 0, 37)])                 # whole
    state.zero_()
    run([("a", 1, 0, 2), ("b", 2, 0, 30)])                   # portions, a's first of two tokens
    run([("b", 2, 30, 31), ("a", 1, 2, 99)])
    for i in range(6):                                       # b token by token beside a's portions of two
        run([("a", 1, 99 + 2 * i, 101 + 2 * i), ("b", 2, 31 + i, 32 + i)])
    state[2].zero_()                                         # b is finished; c takes its slot
    run([("c", 2, 0, 3), ("a", 1, 111, 150)])
    for i in range(3, 64):
        run([("c", 2, i, i + 1)])
    # rows of no request (slot 0) give zeros and leave every state alone
    before = state.clone()
    out = K.mlstm_scan(dev(data["a"][:4]), 0, heads * d, 2 * heads * d, width - 2 * heads, width - heads, dev(bi), dev(bf), state,
                       K.entry_ranges(dev([0, 1, 2, 3], torch.int32), 4), dev([0, 0, 0, 0], torch.int32), 4, heads, d, e, cap, 1.0, 1e-6)
    assert float(out.abs().max()) == 0.0 and torch.equal(before, state)


@pytest.mark.parametrize("experts,top,count,keep", [(8, 3, 4, 2), (6, 1, 1, 1), (12, 4, 3, 3), (16, 2, 8, 1), (4, 4, 2, 2)])
def test_router_against_plain(experts, top, count, keep):
    """Choice scores with negative corrections (a dropped group must lose to a negative score, not to
    zero), weights without the correction, ties between equal scores."""
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(experts)
    rows, width = 300, 24
    h = rng.standard_normal((rows, width)).astype(np.float32)
    router = rng.standard_normal((experts, width)).astype(np.float32)
    router[1] = router[0]                                    # two experts always tie
    h[:5] = 0.0                                              # and whole rows of equal scores
    corr = (rng.standard_normal(experts) - 1.5).astype(np.float32)
    corr[1] = corr[0]
    got_e, got_w = K.moe_route(dev(h), dev(router), dev(corr), top, count, keep, 2, "sigmoid", False)
    got_e, got_w = got_e.cpu().numpy(), got_w.cpu().numpy()
    z = h.astype(np.float64) @ router.astype(np.float64).T
    close = 0
    for r in range(rows):
        chosen, weights = PF.route(z[r], corr.astype(np.float64), top, count, keep)
        if list(got_e[r]) != chosen:                         # a 32-bit sum may turn a near tie; then the scores must be near
            s = PF.sigmoid(z[r]) + corr
            assert np.abs(np.sort(s[got_e[r]]) - np.sort(s[chosen])).max() < 1e-5, f"row {r}: {got_e[r]} != {chosen}"
            close += 1
            continue
        assert np.abs(got_w[r] - np.asarray(weights)).max() < 1e-5
    assert close <= rows // 50


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rows,width,ff,experts,top", [(70, 40, 24, 6, 2), (1, 64, 100, 5, 5), (200, 24, 9, 3, 1), (700, 72, 136, 4, 2), (900, 40, 130, 3, 1)])
def test_experts_against_plain(dtype, tol, rows, width, ff, experts, top):
    from kapel_b200 import kernels as K

    rng = np.random.default_rng(rows)
    r = (lambda a: torch.tensor(a, dtype=torch.bfloat16).double().numpy()) if dtype == torch.bfloat16 else (lambda a: a)
    h = r(rng.standard_normal((rows, width)))
    up = r(rng.standard_normal((experts, ff, width)) / width ** 0.5)
    down = r(rng.standard_normal((experts, width, ff)) / ff ** 0.5)
    chosen = np.stack([rng.permutation(experts)[:top] for _ in range(rows)])
    weights = rng.random((rows, top))
    want = np.zeros((rows, width))
    for i in range(rows):
        for x, w in zip(chosen[i], weights[i]):
            want[i] += w * (down[x] @ (np.maximum(up[x] @ h[i], 0.0) ** 2))
    lists = K.moe_sort(dev(chosen, torch.int32), experts, dtype)
    inner = K.moe_grouped(dev(h, dtype), dev(up, dtype), lists, "relu2", True, False, dtype)
    y = K.moe_grouped(inner, dev(down, dtype), lists, "none", False, True, torch.float32)
    got = K.moe_combine(y, dev(weights), torch.float32).cpu().numpy()
    assert rel_err(got, want) < tol


# -------------------------------------------------------------------------------------- the engine
def engine_for(models, name, dtype, **kw):
    from kapel_b200.engine import Engine

    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_sequences", 4)
    return Engine.from_dir(models[name][0], dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts_portions_and_decoding_against_plain(models, name, dtype):
    """A prompt whole; the same prompt in portions of changing size down to two tokens and then
    token by token (a long decoding that passes the windows); logits at every position."""
    name = variant_for(name, dtype)
    raw = models[name][1]
    rng = np.random.default_rng(7)
    tokens = random_tokens(rng, 150, raw["vocab"])
    want = {"w": plain(models, name, tokens), "p": plain(models, name, tokens)}
    eng = engine_for(models, name, dtype)
    tb = TraceBuilder()
    tb.step([("w", tokens, range(len(tokens)))], end=["w"])
    at = 0
    for n in (2, 17, 3, 2, 40, 5):
        tb.step([("p", tokens[at : at + n], range(n))])
        at += n
    while at < len(tokens):
        tb.step([("p", tokens[at : at + 1], [0])], end=(["p"] if at + 1 == len(tokens) else []))
        at += 1
    worst = compare_trace(run_trace_engine(eng, tb.steps), tb, want, TOL[dtype], f"{name} {dtype}")
    print(f"fusitar {name} {dtype}: worst {worst:.2e}")
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_and_reused_slots_against_each_alone(models, name, dtype):
    """Up to four unequal requests a step, portions beside single tokens, a request left out of a
    step, requests that end and whose pages and slots the next ones take; a pool of few pages."""
    name = variant_for(name, dtype)
    raw = models[name][1]
    rng = np.random.default_rng(8)
    reqs = {k: random_tokens(rng, n, raw["vocab"]) for k, n in dict(a=90, b=41, c=23, d=70, e=33, f=18).items()}
    want = {k: plain(models, name, v) for k, v in reqs.items()}
    eng = engine_for(models, name, dtype, max_tokens=64 * 2 + 128 * 2)
    tb = TraceBuilder()
    fed = {k: 0 for k in reqs}

    def take(k, n, want_all=True):
        a = fed[k]
        n = min(n, len(reqs[k]) - a)
        fed[k] += n
        return (k, reqs[k][a : a + n], list(range(n)) if want_all else [n - 1])

    done = lambda k: fed[k] == len(reqs[k])
    tb.step([take("a", 30), take("b", 2), take("c", 23)], end=["c"])
    tb.step([take("a", 1), take("b", 20), take("d", 17)])
    tb.step([take("b", 1), take("d", 2), take("e", 33, False)], end=["e"])            # a is left out of this step
    tb.step([take("a", 40), take("b", 1), take("d", 1), take("f", 5)])
    while not all(done(k) for k in "abdf"):
        entries = [take(k, 1) for k in "abdf" if not done(k)]
        tb.step(entries, end=[k for k, _, _ in entries if done(k)])
    worst = compare_trace(run_trace_engine(eng, tb.steps), tb, want, TOL[dtype], f"{name} {dtype}")
    print(f"fusitar mixed {name} {dtype}: worst {worst:.2e}")
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages() and eng.cache.free_slots() == 4


def test_recorded_passes_leave_the_state_as_eager_ones_do(models):
    """A prompt pass of a shape seen before and a decoding pass go through recordings, whose first
    eager run must not advance the recurrent state a second time: the logits are those of an engine
    without recordings (up to the order in which a recorded pass, cut for its bucket, adds up)."""
    raw = models["B"][1]
    rng = np.random.default_rng(9)
    outs = []
    for graphs in (False, True):
        eng = engine_for(models, "B", "float32", graphs=graphs)
        tb = TraceBuilder()
        for k in ("x", "y", "z"):                            # the same shape three times: eager, recorded, replayed
            tokens = random_tokens(np.random.default_rng(ord(k)), 80, raw["vocab"])
            tb.step([(k, tokens[:70], [69])])
            for i in range(70, 80):
                tb.step([(k, tokens[i : i + 1], [0])], end=([k] if i == 79 else []))
        outs.append(run_trace_engine(eng, tb.steps))
        if graphs:
            assert eng.recorded_passes > 0
    for step in outs[0]:
        assert rel_err(outs[1][step], outs[0][step]) < 2e-6, f"step {step}"


ONE_KIND = {
    "recurrent": {"architecture": "Fusitar", "vocab": 60, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6}, "layers": [
        mlstm_layer(2, 8, 12, 6.0, moe(4, 2, 1, 1, 16)), mlstm_layer(1, 24, 8, 10.0, None)]},
    "attending": {"architecture": "Fusitar", "vocab": 60, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6}, "layers": [
        attention_layer(2, 1, 16, 16, 0.25, 12, 2, moe(4, 2, 2, 1, 16)), attention_layer(4, 4, 8, 4, 0.3, 100, 0, None)]},
}


@pytest.mark.parametrize("kind", sorted(ONE_KIND))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_one_kind_of_mixer(kind, dtype, tmp_path):
    """No paged group at all, or no state at all (then a prompt alone in its pass is recorded at a rounded
    length, with rows that are no token's): prompts of one length three times over, then token by token."""
    from kapel_b200.engine import Engine

    raw = ONE_KIND[kind]
    folder = make_folder(raw, 5, tmp_path)
    if dtype == "bfloat16":
        make_routers_decisive(folder)
    t = read_tensors(folder)
    eng = Engine.from_dir(folder, dtype=dtype, max_tokens=512, max_sequences=4)
    assert (len(eng.cache.groups) == 0) == (kind == "recurrent") and (len(eng.cache.states) == 0) == (kind == "attending")
    tb, want = TraceBuilder(), {}
    for n, k in enumerate("xyz"):
        tokens = random_tokens(np.random.default_rng(n), 83, raw["vocab"])
        want[k] = PF.forward(raw, t, tokens)
        tb.step([(k, tokens[:70], [69])])
        for i in range(70, 83):
            tb.step([(k, tokens[i : i + 1], [0])], end=([k] if i == 82 else []))
    compare_trace(run_trace_engine(eng, tb.steps), tb, want, TOL[dtype], f"{kind} {dtype}")
    assert eng.recorded_passes > 0


ODD = {"architecture": "Fusitar", "vocab": 77, "width": 52, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(3, 1, 12, 10, 0.3, 19, 1, moe(5, 2, 1, 1, 13)), mlstm_layer(2, 10, 6, 7.0, moe(3, 1, 3, 2, 11)),
    attention_layer(3, 3, 20, 20, 0.2, 40, 3, None)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_eight(dtype, tmp_path):
    """A width, head sizes, value sizes and expert sizes that fit no 16-byte piece: the bfloat16 products run
    on zero-padded rows, the other kernels value by value."""
    from kapel_b200.engine import Engine

    folder = make_folder(ODD, 6, tmp_path)
    if dtype == "bfloat16":
        make_routers_decisive(folder)
    t = read_tensors(folder)
    eng = Engine.from_dir(folder, dtype=dtype, max_tokens=512, max_sequences=4)
    tokens = random_tokens(np.random.default_rng(3), 95, ODD["vocab"])
    want = {"a": PF.forward(ODD, t, tokens)}
    tb = TraceBuilder()
    tb.step([("a", tokens[:70], range(70))])
    tb.step([("a", tokens[70:73], range(3))])
    for i in range(73, 95):
        tb.step([("a", tokens[i : i + 1], [0])], end=(["a"] if i == 94 else []))
    compare_trace(run_trace_engine(eng, tb.steps), tb, want, TOL[dtype], f"odd {dtype}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point_and_scheduler(models, name):
    """`Model.generate` and `generate_batch` (prompt portions under a token budget, decoding passes
    staged and recorded) give the plain implementation's greedy tokens."""
    import kapel_b200

    folder, raw, t = models[name]
    rng = np.random.default_rng(10)
    prompts = [random_tokens(rng, n, raw["vocab"]) for n in (3, 29, 75)]

    def plain_greedy(prompt, n):
        seq, margins = list(prompt), []
        for _ in range(n):
            row = PF.forward(raw, t, seq)[-1]
            order = np.argsort(row)
            margins.append(float(row[order[-1]] - row[order[-2]]))
            seq.append(int(order[-1]))
        return seq[len(prompt):], margins

    want = [plain_greedy(p, 12) for p in prompts]
    model = kapel_b200.Model(str(folder), dtype="f32", max_tokens_cached=1024, max_sequences=4, max_pass_tokens=32)
    for p, (tokens, margins) in zip(prompts, want):
        safe = next((i for i, m in enumerate(margins) if m < 1e-3), len(margins))
        assert model.generate(p, max_tokens=12)[:safe] == tokens[:safe]
    together = model.generate_batch(prompts, max_tokens=12)
    for got, (tokens, margins) in zip(together, want):
        safe = next((i for i, m in enumerate(margins) if m < 1e-3), len(margins))
        assert got[:safe] == tokens[:safe]
    assert model.engine.cache.free_pages() == model.engine.cache.total_pages()


def test_replay_program_and_command_line(models, tmp_path):
    """`bin/trace_run` and `python -m kapel_b200 run` take a Fusitar folder as they take any other: the
    program's logits are the plain ones, the command's greedy tokens are the entry point's."""
    import subprocess
    import sys

    import kapel_b200
    from helpers import ROOT

    folder, raw, _ = models["A"]
    tokens = random_tokens(np.random.default_rng(4), 40, raw["vocab"])
    want = plain(models, "A", tokens)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": tokens[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": tokens[33:35], "want": []}], "end": []},
             {"step": 5, "entries": [{"id": "q", "tokens": tokens[35:], "want": [4]}], "end": ["q"]}]
    out = tmp_path / "logits"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 5"]
    assert sorted(f.name for f in out.iterdir()) == ["0.f32", "5.f32"]
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, raw["vocab"])
    last = np.fromfile(out / "5.f32", dtype="<f4").reshape(1, raw["vocab"])
    assert rel_err(first, want[[0, 32]]) < TOL["float32"] and rel_err(last, want[[39]]) < TOL["float32"]

    model = kapel_b200.Model(str(folder), dtype="f32", max_tokens_cached=256, max_sequences=2)
    expect = model.generate(tokens[:9], max_tokens=6)
    r = subprocess.run([sys.executable, "-m", "kapel_b200", "run", str(folder), "--tokens", ",".join(map(str, tokens[:9])), "--max-tokens", "6",
                        "--greedy", "--dtype", "f32"], capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.strip().splitlines()[0].split(",")] == expect
