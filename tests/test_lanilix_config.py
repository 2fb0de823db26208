"""The Lanilix configuration: reading, refusing, the plan it makes; the cache's books for a
window that keeps first positions; the plain implementation's own mechanisms against closed
forms.  No device."""

import copy
import math

import pytest
import torch

import lanilix_tiny as tiny
from plain import lanilix_plain as plain
from thing_htn_2026_b200.cache import CacheBook, GroupBook
from thing_htn_2026_b200.config import ConfigError, LanilixConfig, config_from_dict, known_architectures
from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
from thing_htn_2026_b200.weights.loader import merge_specs


def test_architecture_is_registered_and_chosen_by_its_key():
    assert "Lanilix" in known_architectures()
    config = config_from_dict(tiny.config_json("p"))
    assert isinstance(config, LanilixConfig)
    assert config.to_dict()["layers"][1]["mixer"]["mask"] == {"size": 24, "keep_first": 3}
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_plan_follows_the_layer_list(name):
    data = tiny.config_json(name)
    plan = config_from_dict(data).plan()
    owners = [layer.get("weights_of") for layer in data["layers"]]
    assert len(plan.schedule) == len(data["layers"])
    assert len(plan.layers) == sum(o is None for o in owners)
    assert [e.cache for e in plan.schedule] == list(range(len(owners)))        # a cache or state of its own each
    for i, (entry, owner) in enumerate(zip(plan.schedule, owners)):
        twin = plan.schedule[owner if owner is not None else i]
        assert entry.layer == twin.layer
    for entry, layer in zip(plan.schedule, data["layers"]):
        block = plan.layers[entry.layer].block
        assert block.kind == "sandwich_norm"
        assert block.params["mixer"].kind == {"delta": "gated_delta", "attention": "attention"}[layer["type"]]
        assert ("ffn" in block.params) == (layer["mlp"] is not None)
        assert ("post_norm_ffn" in block.params) == (layer["mlp"] is not None)


def test_every_size_and_constant_of_the_file_reaches_a_part():
    data = tiny.config_json("q")
    plan = config_from_dict(data).plan()
    attn = plan.layers[0].block.params["mixer"].params
    assert (attn["n_heads"], attn["n_kv_heads"], attn["head_dim"]) == (4, 2, 64)
    assert (attn["scale"], attn["window"], attn["keep_first"]) == (0.125, 70, 66)
    assert attn["qk_norm_scope"] == "projection" and attn["values"] == "keys"
    rope = attn["position"].params
    assert (rope["rotary_dim"], rope["theta"], rope["layout"]) == (64, 500000.0, "interleaved")
    delta = plan.layers[1].block.params["mixer"].params
    assert (delta["n_heads"], delta["n_kv_heads"], delta["key_dim"], delta["value_dim"], delta["conv_taps"]) == (3, 3, 10, 16, 2)
    assert delta["norm_eps"] == 3e-6
    ffn = plan.layers[1].block.params["ffn"].params
    assert (ffn["intermediate_size"], ffn["limit"]) == (100, 3.0)
    free = plan.layers[2].block.params["mixer"].params
    assert free["window"] is None and free["position"] is None and free["keep_first"] == 0
    norm = plan.final_norm.params
    assert (norm["eps"], norm["gain_offset"], norm["residual"]) == (3e-6, 1.0, "float32")


def test_tensor_names_and_shapes():
    specs = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("p")).plan()))
    shapes = {name: tuple(s.shape) for name, s in specs.items()}
    assert shapes["embed"] == (200, 48) and shapes["head"] == (200, 48) and shapes["final.norm"] == (48,)
    assert shapes["l0.mix.q"] == (48, 48) and shapes["l0.mix.v"] == (160, 48) and shapes["l0.mix.q.conv"] == (48, 3)
    assert shapes["l0.mix.v.conv"] == (160, 3) and shapes["l0.mix.b"] == (4, 48) and shapes["l0.mix.A_log"] == (4,)
    assert shapes["l0.mix.norm"] == (40,) and shapes["l0.mix.o"] == (48, 160)
    assert shapes["l1.mix.q"] == (96, 48) and shapes["l1.mix.k"] == (48, 48) and shapes["l1.mix.q.norm"] == (96,)
    assert shapes["l1.mix.k.norm"] == (48,) and "l1.mix.v" not in shapes
    assert shapes["l1.mlp.gate"] == (80, 48) and shapes["l1.mlp.down"] == (48, 80)
    assert not any(name.startswith(("l2.", "l3.")) for name in shapes)          # borrowed weights
    no_ffn = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("q")).plan()))
    assert "l0.norm1b" in no_ffn and "l0.norm2" not in no_ffn and "l0.mlp.gate" not in no_ffn


def broken(name, change):
    data = copy.deepcopy(tiny.config_json(name))
    change(data)
    return data


@pytest.mark.parametrize("change, word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d.__setitem__("layers", []), "layers"),
    (lambda d: d["norm"].__setitem__("eps", 0), "eps"),
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("vdim", 20), "vdim"),
    (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "routed"), "kind"),
    (lambda d: d["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda d: d["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda d: d["layers"][2].__setitem__("weights_of", 1), "another type"),
    (lambda d: d["layers"][3].__setitem__("weights_of", 2), "no tensors of its own"),
])
def test_bad_files_are_refused_with_the_key_named(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(broken("p", change))


# ----------------------------------------------------------------------------- the cache's books


def test_a_window_gives_pages_back_but_never_those_of_the_kept_positions():
    page = 8
    book = CacheBook([GroupBook(window=12, n_pages=40, keep_first=10), GroupBook(window=12, n_pages=40),
                      GroupBook(window=None, n_pages=40)], page, max_slots=2, max_pages_per_seq=40)
    slot = book.open()
    book.prepare([slot], [70])
    book.commit([slot], [70])
    # a query at position 70 sees keys 59..70: pages 7 and 8; the kept positions 0..9: pages 0 and 1
    assert sorted(book.pages_of(0, slot)) == [0, 1, 7, 8]
    assert sorted(book.pages_of(1, slot)) == [7, 8]
    assert sorted(book.pages_of(2, slot)) == list(range(9))
    for _ in range(30):
        book.prepare([slot], [1])
        book.commit([slot], [1])
    assert sorted(book.pages_of(0, slot))[:2] == [0, 1] and min(sorted(book.pages_of(0, slot))[2:]) == (100 - 11) // page
    book.check()
    book.close(slot)
    assert all(alloc.n_held == 0 for alloc in book.pages)
    book.check()


def test_kept_positions_inside_the_window_cost_nothing_extra():
    book = CacheBook([GroupBook(window=64, n_pages=8, keep_first=4)], 16, max_slots=1, max_pages_per_seq=8)
    slot = book.open()
    book.prepare([slot], [40])
    book.commit([slot], [40])
    assert sorted(book.pages_of(0, slot)) == [0, 1, 2]


# ----------------------------------------------------------------------------- the plain implementation


def test_plain_visibility():
    seen = [j for j in range(12) if plain.visible(11, j, 4, 2)]
    assert seen == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(5) if plain.visible(3, j, 4, 2)] == [0, 1, 2, 3]
    assert [j for j in range(12) if plain.visible(11, j, 100, 0)] == list(range(12))


def test_plain_recurrence_against_its_closed_form():
    """With one fixed unit key, S^T k after t writes is a scalar recursion per value entry:
    y <- g y + b (v - g y)."""
    torch.manual_seed(0)
    T, dk, dv = 9, 6, 4
    k = torch.zeros(T, dk, dtype=torch.float64)
    k[:, 2] = 1.0
    v = torch.randn(T, dv, dtype=torch.float64)
    beta, decay = torch.rand(T, dtype=torch.float64), torch.rand(T, dtype=torch.float64)
    out = plain.delta_recurrence(k.clone(), k, v, beta, decay)
    y = torch.zeros(dv, dtype=torch.float64)
    for t in range(T):
        y = decay[t] * y + beta[t] * (v[t] - decay[t] * y)
        assert torch.allclose(out[t], y, atol=1e-12)


def test_plain_convolution_and_rotation():
    x = torch.arange(10, dtype=torch.float64).reshape(5, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = plain.causal_conv(x, w)
    assert y[:, 1].tolist() == x[:, 1].tolist()
    assert y[0, 0] == 0.0 and y[1, 0] == 200.0 and y[2, 0] == 1.0 * 0 + 10.0 * 2 + 100.0 * 4
    q = torch.randn(3, 2, 6, dtype=torch.float64)
    r = plain.rotate_pairs(q, torch.tensor([0, 5, 9]), 4, 50.0)
    assert torch.equal(r[0], q[0]) and torch.equal(r[..., 4:], q[..., 4:])
    a = 9 * 50.0 ** (-2.0 / 4)
    assert math.isclose(r[2, 1, 2], q[2, 1, 2] * math.cos(a) - q[2, 1, 3] * math.sin(a), rel_tol=1e-12)
    assert math.isclose(r[2, 1, 3], q[2, 1, 3] * math.cos(a) + q[2, 1, 2] * math.sin(a), rel_tol=1e-12)
    assert torch.allclose((r * r).sum(-1), (q * q).sum(-1))


def test_written_folders_load_by_name(tmp_path):
    folder = tiny.write_model(str(tmp_path / "p"), "p")
    config, tensors = plain.read_model(folder)
    assert config["architecture"] == "Lanilix" and tensors["l0.mix.A_log"].shape == (4,)
    assert math.isclose(float(tensors["l0.mix.A_log"][2]), math.log(0.012), rel_tol=1e-6)
    logits = plain.model_logits(folder, tiny.tokens("p", 7, 0))
    assert logits.shape == (7, 200) and torch.isfinite(logits).all()
