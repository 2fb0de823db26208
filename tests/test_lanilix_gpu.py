"""The Lanilix decoder on the device against the plain implementation (tests/plain/lanilix_plain.py):
each mechanism alone, then whole models through the replay program (whole prompts, token-by-token
decoding, prompts cut into portions, batches of unequal requests, slots and pages used again), the
edges of the window and of the kept first positions with inputs made so that one key decides the
output, and greedy generation through the library's entry point."""

import os

import numpy as np
import pytest
import torch

import harness
import lanilix_tiny as tiny
from plain import lanilix_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lanilix_models")
    return {name: tiny.write_model(str(root / name), name) for name in tiny.CONFIGS}


# ----------------------------------------------------------------------------- comparison

_oracle = {}


def oracle(folder, tokens, precision):
    key = (folder, tuple(tokens), precision)
    if key not in _oracle:
        _oracle[key] = plain.model_logits(folder, list(tokens), precision).numpy()
    return _oracle[key]


def position_error(got, want):
    """Per position: root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want.astype(np.float64)
    d = d - d.mean(axis=1, keepdims=True)
    return np.sqrt((d * d).mean(axis=1))


def check_logits(got, folder, tokens, dtype, what, places=None):
    """float32: within a few float32 roundings of the plain float32 result.  bfloat16, against
    exact arithmetic and measured by the plain implementation's own bfloat16 emulation: the worst
    place no worse than twice the emulation's worst place (single places flip roundings by
    chance), and the mean over the places no more than one and a half times the emulation's
    mean (a fault that touches most places moves the mean)."""
    places = list(range(len(tokens))) if places is None else places
    assert got.shape[0] == len(places), f"{what}: {got.shape[0]} rows for {len(places)} places"
    exact = oracle(folder, tokens, torch.float64)[places]
    spread = max(1.0, float(np.abs(exact).max()))
    if dtype == "float32":
        err = position_error(got, oracle(folder, tokens, torch.float32)[places])
        assert err.max() <= 2e-5 * spread, f"{what}: float32 logits differ by {err.max():.3e} at place {places[int(err.argmax())]}"
    else:
        noise = position_error(oracle(folder, tokens, torch.bfloat16)[places], exact)
        err = position_error(got, exact)
        worst = int(err.argmax())
        assert err.max() <= 2.0 * noise.max() + 2e-3 * spread, (
            f"{what}: bfloat16 logits are {err[worst]:.3e} from exact at place {places[worst]}, the emulation's worst "
            f"{noise.max():.3e}")
        assert err.mean() <= 1.5 * noise.mean() + 1e-3 * spread, (
            f"{what}: bfloat16 logits are {err.mean():.3e} from exact on average, the emulation {noise.mean():.3e}")


def run_trace(folder, dtype, records, tmp_path, requests, what, max_tokens=None):
    out = harness.replay(folder, dtype, records, str(tmp_path / what.replace(" ", "_")), max_tokens)
    for name, toks in requests.items():
        check_logits(out[name], folder, toks, dtype, f"{what} {name}")
    return out


def trace_portions(requests, sizes):
    """Each request alone, its tokens brought in portions of the given sizes (the last size
    repeats), logits at every place."""
    records, step = [], 0
    for name, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[min(k, len(sizes) - 1)], len(toks) - at)
            records.append({"step": step, "entries": [{"id": name, "tokens": toks[at:at + n], "want": list(range(n))}],
                            "end": [name] if at + n == len(toks) else []})
            at, k, step = at + n, k + 1, step + 1
    return records


# ----------------------------------------------------------------------------- mechanisms alone


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what, exact=None):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err <= 2e-5 * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > 2e-2 + want.abs() / 32
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 200, 5000])
def test_norms_around_a_float32_stream(dtype, width):
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    d = rand((5, width), 1, 3.0).to(t)
    h0 = rand((5, width), 2, 2.0)
    wp, wn = rand((width,), 3, 0.2), rand((width,), 4, 0.2)
    post, gain = ops.Gain(wp.to(DEV), 1.0, 1e-5), ops.Gain(wn.to(DEV), 1.0, 1e-5)
    # a stream that starts from the rows
    h, y = ops.residual_norm(None, d.to(DEV), None, gain, t)
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), d.float())
    close(y, plain.norm_one_plus(d.float(), wn, 1e-5), dtype, "first norm")
    # norm of the branch, add, norm of the sum
    h = h0.clone().to(DEV)
    _, y = ops.residual_norm(h, d.to(DEV), post, gain, t)
    want_h = h0 + plain.norm_one_plus(d.float(), wp, 1e-5)
    assert (h.cpu() - want_h).abs().max() <= 1e-5 * want_h.abs().max(), "the float32 sum"
    close(y, plain.norm_one_plus(want_h, wn, 1e-5), dtype, "norm of the sum")
    # plain gains (offset 0), no branch norm, no second norm
    h = h0.clone().to(DEV)
    _, none = ops.residual_norm(h, d.to(DEV), None, None, t)
    assert none is None and torch.equal(h.cpu(), h0 + d.float())
    _, y = ops.residual_norm(h, None, None, ops.Gain(wn.to(DEV), 0.0, 1e-3), t)
    close(y, plain.norm_plain_weight(h0 + d.float(), wn, 1e-3), dtype, "plain gain")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, size, offset, tail", [(3, 40, 11, 3), (3, 40, 12, 0), (2, 128, 64, 4), (1, 320, 0, 0), (4, 9, 5, 1)])
def test_gated_head_norm(dtype, heads, size, offset, tail):
    """Sizes and gate offsets that take the 16-byte kernel and ones that do not."""
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    rows = 7
    o = rand((rows, heads, size), 5, 4.0)
    gate = rand((rows, offset + heads * size + tail), 6).to(t)
    w = 1 + rand((size,), 7, 0.2)
    got = ops.gated_head_norm(o.to(DEV), gate.to(DEV), offset, w.to(DEV), 1e-5, heads, size, t)
    z = gate[:, offset:offset + heads * size].float().reshape(rows, heads, size)
    want = plain.norm_plain_weight(o, w, 1e-5) * plain.silu(z)
    close(got, want.reshape(rows, -1), dtype, "gated head norm")


def rotate_reference(x, positions, dims, base, layout):
    """x [T, heads, d]; the first ``dims`` entries of each head rotated by position * base^(-2i/dims),
    entry i paired with entry i + dims / 2 ("half") or entry 2i with 2i + 1 ("interleaved")."""
    if layout == "interleaved":
        return plain.rotate_pairs(x, positions, dims, base)
    i = torch.arange(dims // 2, dtype=torch.float64)
    angle = positions.to(torch.float32)[:, None] * (base ** (-2.0 * i / dims)).to(torch.float32)[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    lo, hi = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.clone()
    out[..., :dims // 2] = lo * c - hi * s
    out[..., dims // 2:dims] = hi * c + lo * s
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scope", [None, "head", "projection"])
@pytest.mark.parametrize("layout", ["half", "interleaved"])
@pytest.mark.parametrize("n_q, n_kv, d, dims, own_values", [(4, 2, 64, 32, False), (3, 1, 48, 48, True), (2, 2, 40, 12, False),
                                                           (5, 5, 9, 4, True), (2, 1, 128, 6, False)])
def test_query_and_key_preparation_alone(dtype, scope, layout, n_q, n_kv, d, dims, own_values):
    """`ops.qk_prepare`: norm per head, over the whole projection or none; rotation of the first
    `dims` entries with either pairing; the values from the row or from the keys as projected;
    head sizes that are even (two entries per thread) and odd (one), rotations whose half is odd."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    t = TORCH[dtype]
    T, eps, base = 70, 1e-5, 777.0
    width = (n_q + (2 if own_values else 1) * n_kv) * d + (0 if (n_q + n_kv) % 2 else 2)    # also rows longer than needed
    proj = rand((T, width), 31 + d).to(t)
    gq = 1 + rand((n_q * d if scope == "projection" else d,), 32, 0.2)
    gk = 1 + rand((n_kv * d if scope == "projection" else d,), 33, 0.2)
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv_freq = (base ** (-2.0 * i / dims)).to(torch.float32).to(DEV)
    cos, sin = torch.empty((128, dims // 2), device=DEV), torch.empty((128, dims // 2), device=DEV)
    ops.rope_table(cos, sin, inv_freq, 0, 128)
    tables = ops.RotaryTables(cos, sin, dims, layout)
    cache = SequenceCache([KVSpec(n_kv, d)], max_tokens=128, dtype=t, device=DEV, max_slots=2)
    (slot,) = cache.open(1)
    cache.prepare([slot], [T])
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    rows = ops.step_rows(cu, torch.tensor([slot], dtype=torch.int32, device=DEV), cache.seq_lens, T, T)
    err = ops.new_error_word(DEV)
    q = ops.qk_prepare(proj.to(DEV), gq.to(DEV) if scope else None, gk.to(DEV) if scope else None, scope, eps, tables,
                       rows, cache.kv_view(0), n_q, not own_values, True, err)
    assert int(err.item()) == 0
    x = proj.float()
    q_raw, k_raw = x[:, :n_q * d], x[:, n_q * d:(n_q + n_kv) * d]
    v_raw = x[:, (n_q + n_kv) * d:(n_q + 2 * n_kv) * d] if own_values else k_raw
    if scope == "projection":
        q_n, k_n = plain.norm_plain_weight(q_raw, gq, eps), plain.norm_plain_weight(k_raw, gk, eps)
    elif scope == "head":
        q_n = plain.norm_plain_weight(q_raw.reshape(T, n_q, d), gq, eps).reshape(T, -1)
        k_n = plain.norm_plain_weight(k_raw.reshape(T, n_kv, d), gk, eps).reshape(T, -1)
    else:
        q_n, k_n = q_raw, k_raw
    positions = torch.arange(T)
    want_q = rotate_reference(q_n.reshape(T, n_q, d), positions, dims, base, layout).reshape(T, -1)
    want_k = rotate_reference(k_n.reshape(T, n_kv, d), positions, dims, base, layout)
    close(q, want_q, dtype, "queries")
    pages = cache.book.pages_of(0, slot)
    storage = cache.kv_view(0).storage.float().cpu()                  # [pages, 2, n_kv, 64, d]
    got_k = torch.cat([storage[pages[p], 0] for p in sorted(pages)], dim=1)[:, :T].transpose(0, 1)
    got_v = torch.cat([storage[pages[p], 1] for p in sorted(pages)], dim=1)[:, :T].transpose(0, 1)
    close(got_k, want_k, dtype, "keys in the cache")
    assert torch.equal(got_v, v_raw.to(t).float().reshape(T, n_kv, d)), "values are copied untouched"


def part_of(folder, layer_index, member, dtype):
    """One member part of a layer of a written model, built as the model builds it, with the
    checkpoint's tensors and the layer's own config entry."""
    from thing_htn_2026_b200.config import load_config
    from thing_htn_2026_b200.parts import Runtime, part_class
    from thing_htn_2026_b200.weights.loader import load_tensors
    config = load_config(folder)
    plan = config.plan()
    block = plan.layers[plan.schedule[layer_index].layer].block
    spec = block.params[member]
    family = {"mixer": "mixer", "ffn": "ffn"}[member]
    cls = part_class(family, spec.kind)
    tensors = load_tensors(folder, cls.tensor_specs(spec), TORCH[dtype], torch.device(DEV), ignored=("*",))
    runtime = Runtime(TORCH[dtype], torch.device(DEV), tensors)
    part = cls(spec, runtime)
    for shared in runtime.shared.values():
        shared.ensure(4096)
    return part, config


class Stepper:
    """Feeds rows to one mixer part through a cache of its own, as the step function would."""

    def __init__(self, part, dtype, n_slots=3):
        from thing_htn_2026_b200 import ops
        from thing_htn_2026_b200.cache import SequenceCache
        self.ops, self.part = ops, part
        self.cache = SequenceCache([part.cache_need()], max_tokens=64 * 40, dtype=TORCH[dtype], device=DEV,
                                   max_slots=n_slots)
        self.err = ops.new_error_word(DEV)
        self.entry = None

    def step(self, slots, xs):
        """xs[i]: rows [n_i, width] that slot i brings; returns the mixer's rows per slot."""
        from thing_htn_2026_b200.config.base import ScheduleEntry
        from thing_htn_2026_b200.parts import HostBatch, StepContext
        ops, cache = self.ops, self.cache
        counts = [x.shape[0] for x in xs]
        cache.prepare(slots, counts)
        held = [cache.length(s) for s in slots]
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
        slots_dev = torch.tensor(slots, dtype=torch.int32, device=DEV)
        rows = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts))
        asked = {}
        if hasattr(self.part, "step_inputs"):
            self.part.step_inputs(HostBatch(slots, counts, held, cache.page_size), asked)
        inputs = {k: torch.tensor(v, dtype=torch.int32, device=DEV) for k, v in asked.items()}
        ctx = StepContext(rows=rows, cache=cache, err=self.err, inputs=inputs)
        y = self.part.forward(torch.cat(xs).to(DEV).contiguous(), ctx, ScheduleEntry(0, 0))
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(slots, counts)
        assert int(self.err.item()) == 0
        return [y[a:b] for a, b in zip(cu[:-1], cu[1:])]


MIXERS = [("p", 0), ("p", 1), ("q", 0), ("q", 1), ("q", 2), ("q", 3), ("r", 0), ("r", 1), ("r", 2), ("s", 0), ("s", 1),
          ("s", 2), ("t", 0), ("t", 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, layer", MIXERS)
def test_mixer_alone_whole_in_portions_and_token_by_token(models, dtype, name, layer):
    """One mixer of every kind and size against the plain mechanism, for a sequence brought
    whole, in portions of unequal sizes down to two and one, and beside another sequence."""
    folder = models[name]
    part, config = part_of(folder, layer, "mixer", dtype)
    data = tiny.config_json(name)["layers"][layer]
    _, w = plain.read_model(folder)
    T = 150
    x = rand((T, config.width), 100 + layer).to(TORCH[dtype])
    other = rand((31, config.width), 200 + layer).to(TORCH[dtype])
    fn = plain.delta_mixer if data["type"] == "delta" else plain.windowed_attention
    precision = torch.float32 if dtype == "float32" else torch.bfloat16
    want = fn(x.float(), w, f"l{layer}.mix.", data["mixer"], config.norm_eps, plain.Arithmetic(precision))
    want_other = fn(other.float(), w, f"l{layer}.mix.", data["mixer"], config.norm_eps, plain.Arithmetic(precision))

    stepper = Stepper(part, dtype)
    a, b, c = stepper.cache.open(3)
    (whole,) = stepper.step([a], [x])
    close(whole, want, dtype, "whole")
    # portions, the other sequence in the same steps while it lasts
    cuts = [0, 3, 5, 69, 71, 72, 130, 132, 133, 134, T]
    got, got_other, at = [], [], 0
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        if at < other.shape[0]:
            n = min(hi - lo + 1, other.shape[0] - at)
            ys = stepper.step([c, b], [other[at:at + n], x[lo:hi]])
            got_other.append(ys[0])
            got.append(ys[1])
            at += n
        else:
            got.append(stepper.step([b], [x[lo:hi]])[0])
    close(torch.cat(got), want, dtype, "in portions")
    close(torch.cat(got_other), want_other, dtype, "the sequence beside it")
    if dtype == "float32":
        # what a position gets must not depend on the cut beyond rounding
        assert (torch.cat(got).float() - whole.float()).abs().max() <= 2e-5 * max(1.0, whole.abs().max().item())
    # a slot given back and taken again starts from nothing
    stepper.cache.close([a])
    (again,) = stepper.cache.open(1)
    assert again == a
    close(stepper.step([again], [other])[0], want_other, dtype, "a slot used again")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lanes", [8, 32])
@pytest.mark.parametrize("name, layer", [m for m in MIXERS if tiny.CONFIGS[m[0]]["layers"][m[1]]["type"] == "delta"])
def test_recurrence_with_either_lane_layout(models, monkeypatch, dtype, lanes, name, layer):
    """The prompt kernel of the delta rule holds a column of the state in 8 or in 32 lanes,
    chosen by the step's size; both are run here on the same rows, two sequences of unequal
    lengths in one step, the longer one continued in a second step."""
    from thing_htn_2026_b200 import ops
    monkeypatch.setattr(ops, "DELTA_LANES", lanes)
    folder = models[name]
    part, config = part_of(folder, layer, "mixer", dtype)
    data = tiny.config_json(name)["layers"][layer]
    _, w = plain.read_model(folder)
    xs = [rand((n, config.width), 300 + n).to(TORCH[dtype]) for n in (77, 18)]
    ar = plain.Arithmetic(torch.float32 if dtype == "float32" else torch.bfloat16)
    want = [plain.delta_mixer(x.float(), w, f"l{layer}.mix.", data["mixer"], config.norm_eps, ar) for x in xs]
    stepper = Stepper(part, dtype)
    a, b = stepper.cache.open(2)
    first = stepper.step([a, b], [xs[0][:40], xs[1]])
    (rest,) = stepper.step([a], [xs[0][40:]])
    close(torch.cat([first[0], rest]), want[0], dtype, f"{lanes} lanes, two steps")
    close(first[1], want[1], dtype, f"{lanes} lanes, beside it")


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_alone(models, dtype):
    folder = models["q"]
    part, config = part_of(folder, 2, "ffn", dtype)
    _, w = plain.read_model(folder)
    x = rand((9, config.width), 8, 4.0).to(TORCH[dtype])      # products beyond the limit of 0.7 on both sides
    precision = torch.float32 if dtype == "float32" else torch.bfloat16
    ar = plain.Arithmetic(precision)
    want = plain.clamped_glu(x.float(), w, "l2.mlp.", {"limit": 0.7}, ar)
    raw = ar.linear(x.float(), w["l2.mlp.up"])
    assert (raw > 0.7).any() and (raw < -0.7).any()
    close(part.forward(x.to(DEV), None), want, dtype, "clamped gated unit")


# ----------------------------------------------------------------------------- edges, made to show


def attend(dtype, n_q, n_kv, d, scale, window, keep_first, q_rows, k_rows, prompt_len):
    """q_rows [T, n_q * d], k_rows [T, n_kv * d] as projected (no norm, no rotation; the values
    are the keys): the first prompt_len positions (or all, if fewer) as one step, the rest one
    by one.  Returns the attention output [T, n_q * d]."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    t = TORCH[dtype]
    T = q_rows.shape[0]
    cache = SequenceCache([KVSpec(n_kv, d, window, keep_first)], max_tokens=64 * 12, dtype=t, device=DEV, max_slots=2)
    err = ops.new_error_word(DEV)
    (slot,) = cache.open(1)
    proj = torch.cat([q_rows, k_rows], dim=1).to(t).to(DEV).contiguous()
    outs, at = [], 0
    for n in [min(prompt_len, T)] + [1] * max(0, T - prompt_len):
        cache.prepare([slot], [n])
        cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot], dtype=torch.int32, device=DEV)
        rows = ops.step_rows(cu, slots, cache.seq_lens, n, n)
        kv = cache.kv_view(0)
        q = ops.qk_prepare(proj[at:at + n].contiguous(), None, None, None, 1.0, None, rows, kv, n_q, True, True, err)
        tiles = None
        size = ops.prompt_attention_tile(t, d, kv.page_size, n_q, n_kv) if n > 1 else 0
        if size:
            r0, rn = ops.row_tiles_of([n], [cache.length(slot)], size)
            tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=DEV),
                                 torch.tensor(rn, dtype=torch.int32, device=DEV), len(r0), size)
        outs.append(ops.attention(q, rows, kv, n_q, scale, window, err, tiles, keep_first))
        ops.advance(cache.seq_lens, slots, cu)
        cache.commit([slot], [n])
        at += n
    assert int(err.item()) == 0
    return torch.cat(outs).float().cpu()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, n_q, n_kv", [(64, 4, 2), (16, 2, 2), (128, 2, 1)])
@pytest.mark.parametrize("window, keep_first", [(40, 5), (70, 0), (64, 64), (100, 70), (None, 0)])
def test_one_key_decides_at_every_edge(dtype, d, n_q, n_kv, window, keep_first):
    """For a handful of queries, one key is made to stand out (a long vector along the query)
    and every other key is small: the output is that key if the design lets the query see it,
    and small if not.  Keys just inside and just outside the window, the last kept position
    and the first that is not kept, the sequence's first key, a key a page border away, a
    far key; queries inside the prompt and decoded one by one."""
    T, prompt_len = 230, 170
    big = 8.0
    size = window if window is not None else T + 1
    cases = []                      # (query position, key position)
    for i in (100, 128, 169, 170, 192, 193, 229):
        for j in (i, i - 1, i - size + 1, i - size, keep_first - 1, keep_first, 0, i - 64, i - 63, 2):
            if 0 <= j <= i:
                cases.append((i, j))
    g = torch.Generator().manual_seed(d + (window or 0))
    for i, j in cases:
        q = torch.randn(T, n_q * d, generator=g) * 0.05
        k = torch.randn(T, n_kv * d, generator=g) * 0.05
        direction = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
        q[i] = (direction * big).repeat(n_q)
        k[j] = (direction * big).repeat(n_kv)
        out = attend(dtype, n_q, n_kv, d, 1.0, window, keep_first, q[:i + 1], k[:i + 1], prompt_len)[i].reshape(n_q, d)
        sees = plain.visible(i, j, size, keep_first)
        along = (out @ direction)
        if sees:
            assert (along > 0.9 * big).all(), f"query {i} should see key {j} (window {window}, kept {keep_first}): {along}"
        else:
            assert (along.abs() < 0.1 * big).all(), f"query {i} should not see key {j} (window {window}, kept {keep_first}): {along}"


# ----------------------------------------------------------------------------- whole models


def requests_for(name, lengths, seed=0, tag=""):
    return {f"{name}{tag}{i}": tiny.tokens(name, n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_whole_prompts_and_their_first_tokens(models, tmp_path, dtype, name):
    requests = requests_for(name, [1, 2, 3, 70, 211])
    run_trace(models[name], dtype, harness.trace_whole(requests), tmp_path, requests, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_decoding_token_by_token_long(models, tmp_path, dtype, name):
    """A short prompt and then 190 tokens one by one: past page borders, past the window and
    the kept positions of every configuration, with the state carried all the way."""
    requests = requests_for(name, [200, 96], seed=10)
    run_trace(models[name], dtype, harness.trace_tail(requests, tail=190), tmp_path, requests, "decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_prompts_in_portions(models, tmp_path, dtype, name):
    requests = requests_for(name, [180, 67], seed=20)
    for sizes in ([2], [63, 2, 1, 64, 3], [5, 100, 2, 2, 7]):
        run_trace(models[name], dtype, trace_portions(requests, sizes), tmp_path, requests, f"portions {sizes[0]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_batches_of_unequal_requests(models, tmp_path, dtype, name):
    """Requests of very different lengths start together and go on together; the shorter end
    earlier; a second batch then takes the slots and pages the first gave back, with a cache
    that holds no more than one batch."""
    first = requests_for(name, [1, 140, 33, 75], seed=30)
    second = requests_for(name, [90, 2, 129], seed=40, tag="x")
    prompt_lens = {n: max(1, len(t) - k) for k, (n, t) in zip([0, 40, 9, 70, 12, 1, 64], {**first, **second}.items())}
    records = harness.trace_batches([first, second], prompt_lens)
    requests = {**first, **second}
    out = run_trace(models[name], dtype, records, tmp_path, requests, "batches",
                    max_tokens=max(harness.max_tokens_of(harness.trace_batches([b], prompt_lens)) for b in (first, second)))
    if dtype == "float32":
        alone = harness.replay(models[name], dtype, harness.trace_whole(requests), str(tmp_path / "alone"))
        for n in requests:
            err = position_error(out[n], alone[n]).max()
            assert err <= 2e-5 * max(1.0, np.abs(alone[n]).max()), f"{n}: in a batch and alone differ by {err:.3e}"


def test_a_state_that_is_lost_would_show(models, tmp_path):
    """The tests above can only catch a lost state if the state matters: at the end of a long
    sequence the logits must differ from those of its last tokens alone by far more than the
    tolerance."""
    toks = tiny.tokens("p", 211, 4)
    whole = oracle(models["p"], toks, torch.float32)[-1]
    tail = plain.model_logits(models["p"], toks[-30:], torch.float32).numpy()[-1]
    assert np.abs(whole - tail).max() > 1e-2


# ----------------------------------------------------------------------------- generation


def greedy_by_plain(folder, prompt, n):
    tokens = list(prompt)
    margins = []
    for _ in range(n):
        logits = plain.model_logits(folder, tokens, torch.float32)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(logits.argmax()))
    return tokens[len(prompt):], margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["p", "q"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """Engine.generate: the library's own entry point, scheduler, captured decode step and token
    choice, on prompts of unequal lengths, against greedy continuation by the plain
    implementation (up to the first step whose two best logits are closer than rounding)."""
    from thing_htn_2026_b200 import Engine
    prompts = [tiny.tokens(name, n, 50 + n) for n in (5, 70, 23)]
    new = 24
    engine = Engine(models[name], dtype="float32", graphs=graphs)
    got = [[] for _ in prompts]
    for step in engine.generate(prompts, new):
        for i, token in enumerate(step):
            got[i].append(token)
    for i, prompt in enumerate(prompts):
        want, margins = greedy_by_plain(models[name], prompt, new)
        sure = next((k for k, m in enumerate(margins) if m < 1e-3), new)
        assert got[i][:sure] == want[:sure], f"prompt {i}: {got[i]} against {want} (sure of the first {sure})"
        assert sure >= 8
    # the same engine again: slots and state of the first call are gone
    again = [[] for _ in prompts]
    for step in engine.generate(prompts, 6):
        for i, token in enumerate(step):
            again[i].append(token)
    assert [a[:6] for a in again] == [g[:6] for g in got]


def test_generation_in_bfloat16_runs_and_stays_in_the_vocabulary(models):
    from thing_htn_2026_b200 import Engine
    engine = Engine(models["r"], dtype="bfloat16")
    prompts = [tiny.tokens("r", n, 60 + n) for n in (3, 40)]
    steps = list(engine.generate(prompts, 12, temperature=[0.0, 0.8], seed=3))
    assert len(steps) == 12 and all(0 <= t < 128 for step in steps for t in step)
