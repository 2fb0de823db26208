"""The Bunudra decoder on the device against the plain implementation (tests/plain/bunudra_plain.py):
each mechanism alone, then whole models through the replay program (whole prompts, token-by-token
decoding, prompts cut into portions, batches of unequal requests, slots and pages used again), the
edges of chunks and windows with inputs made so that one key decides the output, and greedy
generation through the library's entry point."""

import numpy as np
import pytest
import torch

import bunudra_tiny as tiny
import harness
from plain import bunudra_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("bunudra_models")
    return {name: tiny.write_model(str(root / name), name) for name in tiny.CONFIGS}


# ----------------------------------------------------------------------------- comparison

_oracle, _read = {}, {}


def read(folder):
    if folder not in _read:
        _read[folder] = plain.read_model(folder)
    return _read[folder]


def oracle(folder, tokens, precision):
    key = (folder, tuple(tokens), precision)
    if key not in _oracle:
        config, tensors = read(folder)
        _oracle[key] = plain.forward(config, tensors, list(tokens), precision).to(torch.float64).numpy()
    return _oracle[key]


def position_error(got, want):
    """Per position: root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want.astype(np.float64)
    d = d - d.mean(axis=1, keepdims=True)
    return np.sqrt((d * d).mean(axis=1))


def check_logits(got, folder, tokens, dtype, what, places=None):
    """float32: within a few float32 roundings of the plain float32 result.  bfloat16, against
    exact arithmetic and measured by the plain implementation's own bfloat16 emulation.  A
    router's close call, decided the other way by one rounding, moves a single place by far more
    than rounding does, in the emulation as here, so the measures are the median and the ninth
    decile over the places, and the number of places far out."""
    places = list(range(len(tokens))) if places is None else places
    assert got.shape[0] == len(places), f"{what}: {got.shape[0]} rows for {len(places)} places"
    exact = oracle(folder, tokens, torch.float64)
    spread = max(1.0, float(np.abs(exact).max()))
    if dtype == "float32":
        err = position_error(got, oracle(folder, tokens, torch.float32)[places])
        far = err > 3e-5 * spread
        assert far.sum() <= max(1, len(places) // 50), (
            f"{what}: float32 logits differ by {err.max():.3e} at place {places[int(err.argmax())]}, {int(far.sum())} places out")
    else:
        noise = position_error(oracle(folder, tokens, torch.bfloat16), exact)      # over all places of the sequence
        err = position_error(got, exact[places])
        if len(places) >= 32:       # a close call early in a short sequence moves most of its places
            assert np.median(err) <= 2.0 * np.median(noise) + 2e-3 * spread, (
                f"{what}: bfloat16 median distance {np.median(err):.3e}, the emulation's {np.median(noise):.3e}")
        limit = 3.0 * np.percentile(noise, 90) + 2e-3 * spread
        out = int((err > limit).sum())
        assert out <= max(1, len(places) // 10), (
            f"{what}: {out} of {len(places)} places are more than {limit:.3e} from exact; worst {err.max():.3e} at place "
            f"{places[int(err.argmax())]}")


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


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err <= 2e-5 * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > 2e-2 * max(1.0, want.abs().max().item()) + want.abs() / 32
        assert bad.sum() <= bad.numel() // 200, f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


# ----------------------------------------------------------------------------- small mechanisms


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 100, 5000])
def test_layer_norm_on_a_branch_and_the_stream_as_it_is(dtype, width):
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    d = (rand((5, width), 1, 3.0) + 0.7).to(t)             # a mean that is not zero
    h0 = rand((5, width), 2, 2.0)
    w1, b1, w2, b2 = 1 + rand((width,), 3, 0.2), rand((width,), 4, 0.3), 1 + rand((width,), 5, 0.2), rand((width,), 6, 0.3)
    post = ops.Gain(w1.to(DEV), 0.0, 1e-5, b1.to(DEV), "layer")
    final = ops.Gain(w2.to(DEV), 0.0, 1e-5, b2.to(DEV), "layer")
    # norm of the branch, add, the sum itself rounded
    h = h0.clone().to(DEV)
    _, y = ops.residual_norm(h, d.to(DEV), post, ops.STREAM_AS_IS, t)
    want_h = h0 + plain.layer_norm(d.float(), w1, b1, 1e-5)
    assert (h.cpu() - want_h).abs().max() <= 2e-5 * want_h.abs().max(), "the float32 sum"
    assert torch.equal(y.cpu(), h.cpu().to(t)), "the stream as a sublayer reads it is the sum, rounded once"
    # norm of the branch, add, another layer norm of the sum (the model's last norm)
    h = h0.clone().to(DEV)
    _, y = ops.residual_norm(h, d.to(DEV), post, final, t)
    close(y, plain.layer_norm(want_h, w2, b2, 1e-5), dtype, "layer norm of the sum")
    # no bias; the stream alone
    _, y = ops.residual_norm(h0.clone().to(DEV), None, None, ops.Gain(w2.to(DEV), 0.0, 1e-3, None, "layer"), t)
    close(y, plain.layer_norm(h0, w2, torch.zeros(width), 1e-3), dtype, "layer norm without bias")
    _, y = ops.residual_norm(h0.clone().to(DEV), None, None, ops.STREAM_AS_IS, t)
    assert torch.equal(y.cpu(), h0.to(t))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_rows_are_scaled_in_float32(dtype):
    from thing_htn_2026_b200 import ops
    table = rand((50, 36), 8).to(TORCH[dtype])
    index = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    err = ops.new_error_word(DEV)
    got = ops.gather_rows_scaled(table.to(DEV), index.to(DEV), 12.0, err)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), table.float()[index.long()] * 12.0)
    assert int(err.item()) == 0
    ops.gather_rows_scaled(table.to(DEV), torch.tensor([50], dtype=torch.int32, device=DEV), 1.0, err)
    assert int(err.item()) == ops.ERR_TOKEN_RANGE


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, size, offset", [(3, 40, 11), (2, 128, 64), (5, 17, 0), (1, 9, 4)])
def test_read_out_norm_with_a_gain_over_all_heads_and_a_logistic_gate(dtype, heads, size, offset):
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    rows = 7
    o = rand((rows, heads, size), 5, 4.0)
    gate = rand((rows, offset + heads * size + 3), 6).to(t)
    w = 1 + rand((heads * size,), 7, 0.2)
    got = ops.gated_head_norm(o.to(DEV), gate.to(DEV), offset, w.to(DEV), 1e-5, heads, size, t, gate_kind="logistic")
    z = gate[:, offset:offset + heads * size].float()
    want = plain.over_rms(o, 1e-5).reshape(rows, -1) * w * torch.sigmoid(z)
    close(got, want, dtype, "read-out norm")


@pytest.mark.parametrize("experts, groups, keep, top, scale", [(8, 4, 3, 4, 2.0), (6, 3, 2, 2, 1.5), (4, 1, 1, 1, 1.0), (9, 3, 2, 4, 2.5),
                                                               (4, 2, 2, 4, 0.5), (64, 8, 4, 6, 1.0), (5, 5, 1, 1, 3.0)])
def test_routing_alone(experts, groups, keep, top, scale):
    """Scores, the best groups, the best allowed experts and their weights, on logits without
    close calls; also with one more column in the row (the shared expert's gate logit)."""
    from thing_htn_2026_b200 import ops
    rows = 97
    z = rand((rows, experts + 1), 40 + experts, 2.0)
    got = ops.moe_route(z.to(DEV), experts, groups, keep, top, scale)
    router = {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    chosen, weights = plain.route(z[:, :experts].double(), router)
    dense = torch.zeros(rows, experts, dtype=torch.float64)
    dense.scatter_(1, chosen, weights)
    assert torch.equal(got.chosen.cpu().long().sort(dim=1).values, chosen.sort(dim=1).values), "the chosen experts"
    assert (got.dense.cpu().double() - dense).abs().max() <= 1e-6 * scale
    assert (got.chosen_weight.cpu().double() - dense.gather(1, got.chosen.cpu().long())).abs().max() <= 1e-6 * scale
    if keep < groups:      # an expert with a high score in a group that is not kept is not chosen
        per = experts // groups
        s = torch.softmax(z[:, :experts].double(), dim=-1)
        best_groups = s.view(rows, groups, per).max(-1).values.topk(keep, dim=-1).indices
        assert all(int(e) // per in set(best_groups[r].tolist()) for r in range(rows) for e in got.chosen[r].cpu())


# ----------------------------------------------------------------------------- one part at a time


def part_of(folder, layer_index, member, dtype):
    """One member part of a layer of a written model, built as the model builds it."""
    from thing_htn_2026_b200.config import load_config
    from thing_htn_2026_b200.parts import Runtime, part_class
    from thing_htn_2026_b200.weights.loader import load_tensors
    config = load_config(folder)
    plan = config.plan()
    spec = plan.layers[plan.schedule[layer_index].layer].block.params[member]
    cls = part_class(member if member == "mixer" else "ffn", spec.kind)
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

    def step(self, slots, xs):
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


MIXERS = [(name, i) for name in tiny.CONFIGS for i in range(len(tiny.CONFIGS[name]["layers"]))]


def plain_mixer(data, x, w, prefix, eps, precision):
    ar = plain.Arithmetic(precision)
    x = x.to(ar.work)
    w = {k: v.to(ar.work) if v.is_floating_point() else v for k, v in w.items()}
    if data["type"] == "mlstm":
        return plain.mlstm_mixer(x, w, prefix, data["mixer"], eps, ar)[0]
    return plain.MIXERS[data["type"]](x, w, prefix, data["mixer"], eps, ar)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, layer", MIXERS)
def test_mixer_alone_whole_in_portions_and_token_by_token(models, dtype, name, layer):
    """One mixer of every kind and size against the plain mechanism, for a sequence brought
    whole, in portions of unequal sizes down to two and one, and beside another sequence."""
    folder = models[name]
    part, config = part_of(folder, layer, "mixer", dtype)
    data = tiny.config_json(name)["layers"][layer]
    _, w = read(folder)
    T = 150
    x = rand((T, config.width), 100 + layer).to(TORCH[dtype])
    other = rand((31, config.width), 200 + layer).to(TORCH[dtype])
    precision = torch.float32 if dtype == "float32" else torch.bfloat16
    want = plain_mixer(data, x.float(), w, f"l{layer}.mix.", config.norm_eps, precision)
    want_other = plain_mixer(data, other.float(), w, f"l{layer}.mix.", config.norm_eps, precision)

    stepper = Stepper(part, dtype)
    a, b, c = stepper.cache.open(3)
    (whole,) = stepper.step([a], [x])
    close(whole, want, dtype, "whole")
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
        assert (torch.cat(got).float() - whole.float()).abs().max() <= 2e-5 * max(1.0, whole.abs().max().item())
    # a slot given back and taken again starts from nothing
    stepper.cache.close([a])
    (again,) = stepper.cache.open(1)
    assert again == a
    close(stepper.step([again], [other])[0], want_other, dtype, "a slot used again")
    # token by token from the start
    stepper.cache.close([again])
    (slot,) = stepper.cache.open(1)
    single = torch.cat([stepper.step([slot], [other[i:i + 1]])[0] for i in range(other.shape[0])])
    close(single, want_other, dtype, "token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("staged, lanes", [(False, 0), (True, 8), (True, 16), (True, 32)])
@pytest.mark.parametrize("name, layer", [m for m in MIXERS if tiny.CONFIGS[m[0]]["layers"][m[1]]["type"] == "mlstm"])
def test_matrix_memory_with_every_prompt_kernel(models, dtype, staged, lanes, name, layer):
    """The recurrence over a prompt with the plain kernel, with tokens staged in shared memory at 8,
    16 and 32 lanes per column (sizes whose rows are not aligned fall back to the plain kernel by
    themselves): a prompt longer than several stages, cut so that a stage is left partly filled,
    then continued token by token from the state the prompt left."""
    from thing_htn_2026_b200 import ops
    folder = models[name]
    part, config = part_of(folder, layer, "mixer", dtype)
    data = tiny.config_json(name)["layers"][layer]
    _, w = read(folder)
    x = rand((83, config.width), 400 + layer).to(TORCH[dtype])
    precision = torch.float32 if dtype == "float32" else torch.bfloat16
    want = plain_mixer(data, x.float(), w, f"l{layer}.mix.", config.norm_eps, precision)
    ops.set_mlstm_kernel(staged, lanes)
    try:
        stepper = Stepper(part, dtype)
        (a,) = stepper.cache.open(1)
        got = [stepper.step([a], [x[:37]])[0], stepper.step([a], [x[37:70]])[0]]
        got += [stepper.step([a], [x[i:i + 1]])[0] for i in range(70, 83)]
    finally:
        ops.set_mlstm_kernel()
    close(torch.cat(got), want, dtype, f"staged={staged}, {lanes} lanes")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, layer", [("a", 0), ("a", 3), ("b", 0), ("c", 1)])
def test_feed_forward_alone(models, dtype, name, layer):
    """Routed experts with groups, a shared expert with its gate, one expert per token without a
    shared one; a row's result does not depend on the rows beside it."""
    folder = models[name]
    part, config = part_of(folder, layer, "ffn", dtype)
    data = tiny.config_json(name)["layers"][layer]
    _, w = read(folder)
    x = rand((83, config.width), 300 + layer, 1.5).to(TORCH[dtype])
    precision = torch.float32 if dtype == "float32" else torch.bfloat16
    ar = plain.Arithmetic(precision)
    wt = {k: v.to(ar.work) if v.is_floating_point() else v for k, v in w.items()}
    want = plain.moe(x.float().to(ar.work), wt, f"l{layer}.mlp.", data["mlp"], ar)

    class Ctx:
        err = None
    got = part.forward(x.to(DEV), Ctx())
    close(got, want, dtype, "feed-forward")
    alone = torch.cat([part.forward(x[i:i + 1].to(DEV), Ctx()) for i in (0, 41, 82)])
    if dtype == "float32":
        assert (alone.cpu() - got.cpu()[[0, 41, 82]]).abs().max() <= 1e-5 * max(1.0, float(got.abs().max()))
    else:
        close(alone, want[[0, 41, 82]], dtype, "rows alone")


# ----------------------------------------------------------------------------- edges made to show


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv, n_q, n_kv", [(16, 16, 2, 1), (64, 64, 4, 2), (48, 32, 3, 3), (20, 36, 2, 1), (128, 128, 2, 1)])
@pytest.mark.parametrize("mask, size", [("chunk", 64), ("chunk", 24), ("chunk", 70), ("window", 72), ("window", 5), ("window", 64)])
def test_one_key_decides_at_every_edge(dtype, d, dv, n_q, n_kv, mask, size):
    """Keys and values are written as they are (no norm, no rotation).  All keys of a sequence are
    tiny but one, whose score stands out by far, and every value row is its own position: the
    output of a query names the key that decided it, or, where the loud key is hidden, the mean
    position of the keys it does see.  Several sequences, each with its loud key elsewhere (the
    first key of a chunk or window, the key before it, page borders, far back), run as one batch:
    as a whole prompt, and with the second half decoded one token a step.  Head sizes that take the
    warp-per-row kernel and the tensor-core kernels, values of another size than the keys."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    t = TORCH[dtype]
    L = 300
    louds = sorted({x for x in (0, size - 1, size, 2 * size - 1, 2 * size, 63, 64, 128, 192 - size, 200) if 0 <= x < L})
    S = len(louds)
    cache = SequenceCache([KVSpec(n_kv, d, value_dim=dv)], max_tokens=64 * 5 * S, dtype=t, device=DEV, max_slots=S)
    kv = cache.kv_view(0)
    err = ops.new_error_word(DEV)
    k = torch.full((S, L, n_kv, d), 0.01)
    for s, loud in enumerate(louds):
        k[s, loud] = 1.0
    v = (torch.arange(L, dtype=torch.float32) / 64.0)[None, :, None, None].expand(S, L, n_kv, dv)
    proj = torch.cat([torch.ones(S, L, n_q * d), k.reshape(S, L, -1), v.reshape(S, L, -1)], dim=2).to(t)
    chunk, window = (size, None) if mask == "chunk" else (None, size)
    tile = ops.prompt_attention_tile(t, d, cache.page_size, n_q, n_kv, dv, chunk)
    i = np.arange(L)
    first = i // size * size if mask == "chunk" else np.maximum(0, i - size + 1)

    for prompt_len in (L, 150):
        slots = cache.open(S)
        outs, at = [[] for _ in range(S)], 0
        for n in [prompt_len] + [1] * (L - prompt_len):
            cache.prepare(slots, [n] * S)
            cu = torch.tensor([n * j for j in range(S + 1)], dtype=torch.int32, device=DEV)
            sl = torch.tensor(slots, dtype=torch.int32, device=DEV)
            rows = ops.step_rows(cu, sl, cache.seq_lens, n * S, n, max_context=L)
            x = proj[:, at:at + n].reshape(S * n, -1).to(DEV).contiguous()
            q = ops.qk_prepare(x, None, None, None, 1.0, None, rows, kv, n_q, False, True, err)
            tiles = None
            if n > 1 and tile:
                r0, rr = ops.row_tiles_of([n] * S, [at] * S, tile)
                tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=DEV),
                                     torch.tensor(rr, dtype=torch.int32, device=DEV), len(r0), tile)
            a = ops.attention(q, rows, kv, n_q, 30.0 / d, window, err, tiles, chunk=chunk).float().cpu().reshape(S, n, n_q, dv)
            for s in range(S):
                outs[s].append(a[s])
            ops.advance(cache.seq_lens, sl, cu)
            cache.commit(slots, [n] * S)
            at += n
        assert int(err.item()) == 0
        for s, loud in enumerate(louds):
            out = torch.cat(outs[s]).numpy()                         # [L, n_q, dv]
            sees = (loud <= i) & (loud >= first)
            want = np.where(sees, loud, (first + i) / 2.0) / 64.0
            tolerance = (1e-4 if dtype == "float32" else 6e-3) * np.maximum(1.0, want) + (1e-4 if dtype == "float32" else 4e-3)
            wrong = np.abs(out - want[:, None, None]).max(axis=(1, 2)) > tolerance
            assert not wrong.any(), (
                f"loud key {loud}, prompt of {prompt_len}: queries {i[wrong][:8].tolist()} got "
                f"{(out[wrong][:8, 0, 0] * 64).round(2).tolist()}, expected {(want[wrong][:8] * 64).round(2).tolist()}")
        cache.close(slots)


# ----------------------------------------------------------------------------- whole models


def requests_of(name, lengths, seed):
    return {f"r{n}": tiny.tokens(name, n, seed + n) for n in lengths}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_prompts_and_their_first_tokens(models, tmp_path, dtype, name):
    requests = requests_of(name, [1, 2, 3, 64, 65, 211], 10)
    run_trace(models[name], dtype, harness.trace_whole(requests), tmp_path, requests, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_decoding_token_by_token_long(models, tmp_path, dtype, name):
    """A prompt of 40 and 190 tokens decoded one by one: every window and chunk passes over
    decoded tokens, pages of windowed layers are given back and others taken on the way."""
    requests = requests_of(name, [230], 20)
    run_trace(models[name], dtype, harness.trace_tail(requests, tail=190), tmp_path, requests, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_prompts_in_portions(models, tmp_path, dtype, name):
    requests = requests_of(name, [150], 30)
    for sizes in ([2], [63, 2, 1, 64, 3], [5, 100, 2, 2, 7]):
        run_trace(models[name], dtype, trace_portions(requests, sizes), tmp_path, requests, f"portions {sizes[0]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_batches_of_unequal_requests(models, tmp_path, dtype, name):
    """Two batches, one after the other, in a cache that holds one of them: the second batch
    takes the slots and pages that the first gave back.  Every request also alone."""
    first = requests_of(name, [1, 70, 135, 23], 40)
    second = {k + "x": v for k, v in requests_of(name, [90, 2, 140], 50).items()}
    prompt_lens = {"r1": 1, "r70": 50, "r135": 100, "r23": 23, "r90x": 64, "r2x": 1, "r140x": 128}
    records = harness.trace_batches([first, second], prompt_lens)
    together = run_trace(models[name], dtype, records, tmp_path, {**first, **second}, "batches",
                         max_tokens=harness.max_tokens_of(records))
    alone = harness.replay(models[name], dtype, harness.trace_whole({**first, **second}), str(tmp_path / "alone"))
    if dtype == "float32":
        for key in together:
            err = position_error(together[key], alone[key])
            assert err.max() <= 3e-5 * max(1.0, np.abs(alone[key]).max()), f"{key}: a batch and the request alone differ by {err.max():.3e}"


def test_a_state_that_is_lost_would_show(models, tmp_path):
    """The plain implementation with the matrix memory reset in mid-sequence is far from the
    library's result: the comparison above would notice a state that is not carried."""
    name = "c"
    config, tensors = read(models[name])
    toks = tiny.tokens(name, 80, 77)
    whole = plain.forward(config, tensors, toks, torch.float64).numpy()
    tail_alone = plain.forward(config, tensors, toks[40:], torch.float64).numpy()
    assert position_error(whole[40:], tail_alone).min() > 1e-2


def greedy_by_plain(folder, prompt, n_new):
    config, tensors = read(folder)
    seq, margins = list(prompt), []
    for _ in range(n_new):
        logits = plain.forward(config, tensors, seq, torch.float64)[-1]
        top = logits.topk(2).values
        margins.append(float(top[0] - top[1]))
        seq.append(int(logits.argmax()))
    return seq[len(prompt):], margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """Engine.generate: the library's own entry point, scheduler, captured decode step and token
    choice, on prompts of unequal lengths, against greedy continuation by the plain
    implementation (up to the first step whose two best logits are closer than rounding)."""
    from thing_htn_2026_b200 import Engine
    prompts = [tiny.tokens(name, n, 50 + n) for n in (5, 70, 23)]
    new = 20
    engine = Engine(models[name], dtype="float32", graphs=graphs)
    got = [[] for _ in prompts]
    for step in engine.generate(prompts, new):
        for i, token in enumerate(step):
            got[i].append(token)
    for i, prompt in enumerate(prompts):
        want, margins = greedy_by_plain(models[name], prompt, new)
        sure = next((k for k, m in enumerate(margins) if m < 1e-3), new)
        assert got[i][:sure] == want[:sure], f"prompt {i}: {got[i]} against {want} (sure of the first {sure})"
        assert sure >= 6
    again = [[] for _ in prompts]
    for step in engine.generate(prompts, 6):
        for i, token in enumerate(step):
            again[i].append(token)
    assert [a[:6] for a in again] == [g[:6] for g in got]


def test_generation_in_bfloat16_runs_and_stays_in_the_vocabulary(models):
    from thing_htn_2026_b200 import Engine
    engine = Engine(models["b"], dtype="bfloat16")
    prompts = [tiny.tokens("b", n, 60 + n) for n in (3, 40)]
    steps = list(engine.generate(prompts, 12, temperature=[0.0, 0.8], seed=3))
    assert len(steps) == 12 and all(0 <= t < 300 for step in steps for t in step)
