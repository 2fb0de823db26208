"""The Bunudra configuration: reading, refusing, the plan it makes; the cache's books for chunks;
the plain implementation's own mechanisms against closed forms.  No device."""

import copy
import math

import pytest
import torch

import bunudra_tiny as tiny
from plain import bunudra_plain as plain
from thing_htn_2026_b200.cache import CacheBook, GroupBook
from thing_htn_2026_b200.config import BunudraConfig, ConfigError, config_from_dict, known_architectures
from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
from thing_htn_2026_b200.weights.loader import merge_specs


def test_architecture_is_registered_and_chosen_by_its_key():
    assert "Bunudra" in known_architectures()
    config = config_from_dict(tiny.config_json("a"))
    assert isinstance(config, BunudraConfig)
    assert config.to_dict()["layers"][2]["mixer"]["mask"] == {"size": 24}
    assert config.to_dict()["embedding"] == {"scale": 3.0}
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_plan_follows_the_layer_list(name):
    data = tiny.config_json(name)
    plan = config_from_dict(data).plan()
    assert len(plan.schedule) == len(plan.layers) == len(data["layers"])
    assert [e.cache for e in plan.schedule] == list(range(len(data["layers"])))
    assert plan.embedding.params["scale"] == data["embedding"]["scale"] and plan.embedding.params["stream"] == "float32"
    assert plan.final_norm.kind == "layernorm" and plan.final_norm.tensors == {"weight": "final.norm", "bias": "final.norm.b"}
    for entry, layer in zip(plan.schedule, data["layers"]):
        block = plan.layers[entry.layer].block
        assert block.kind == "branch_norm"
        assert block.params["mixer"].kind == layer["type"]
        assert ("ffn" in block.params) == (layer["mlp"] is not None) == ("norm_ffn" in block.params)
        assert block.params["norm_mixer"].params["eps"] == data["norm"]["eps"]


def test_every_size_and_constant_of_the_file_reaches_a_part():
    data = tiny.config_json("a")
    plan = config_from_dict(data).plan()
    lat = plan.layers[0].block.params["mixer"].params
    assert (lat["n_heads"], lat["plain_dim"], lat["rot_dim"], lat["value_dim"], lat["latent_rank"]) == (3, 20, 6, 12, 24)
    assert (lat["scale"], lat["window"], lat["norm_eps"]) == (0.21, 5, 1e-5)
    rope = lat["position"].params
    assert (rope["rotary_dim"], rope["theta"], rope["layout"]) == (6, 1000.0, "interleaved")
    assert dict(rope["scaling"]) == {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    mem = plan.layers[1].block.params["mixer"].params
    assert (mem["n_heads"], mem["key_dim"], mem["value_dim"], mem["gate_cap"]) == (2, 24, 40, 8.0)
    att = plan.layers[2].block.params["mixer"].params
    assert (att["n_heads"], att["n_kv_heads"], att["head_dim"], att["value_dim"], att["chunk"], att["window"]) == (6, 3, 16, 24, 24, None)
    assert (att["position"].params["rotary_dim"], att["position"].params["layout"]) == (8, "half")
    ffn = plan.layers[0].block.params["ffn"].params
    assert (ffn["n_experts"], ffn["top"], ffn["groups"], ffn["keep"], ffn["scale"], ffn["expert_ff"], ffn["shared_ff"]) == \
        (6, 2, 3, 2, 1.5, 40, 24)
    plain_ffn = config_from_dict(tiny.config_json("b")).plan().layers[0].block.params["ffn"].params
    assert (plain_ffn["groups"], plain_ffn["keep"], plain_ffn["shared_ff"], plain_ffn["scale"]) == (1, 1, 0, 1.0)
    assert config_from_dict(tiny.config_json("c")).plan().layers[3].block.params["mixer"].params["chunk"] is None


def test_tensor_names_and_shapes():
    specs = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("a")).plan()))
    shape = {name: tuple(spec.shape) for name, spec in specs.items()}
    assert shape["embed"] == (200, 48) and shape["head"] == (200, 48) and shape["final.norm.b"] == (48,)
    assert shape["l0.mix.q"] == (3 * 26, 48) and shape["l0.mix.dkv"] == (30, 48) and shape["l0.mix.dkv.norm"] == (24,)
    assert shape["l0.mix.uk"] == (60, 24) and shape["l0.mix.uv"] == (36, 24) and shape["l0.mix.g"] == (36, 48)
    assert shape["l0.mix.o"] == (48, 36)
    assert shape["l1.mix.i"] == (2, 48) and shape["l1.mix.f.b"] == (2,) and shape["l1.mix.norm"] == (80,)
    assert shape["l1.mix.k"] == (48, 48) and shape["l1.mix.v"] == (80, 48) and shape["l1.mix.o"] == (48, 80)
    assert shape["l2.mix.k"] == (48, 48) and shape["l2.mix.v"] == (72, 48) and shape["l2.mix.o"] == (48, 144)
    assert shape["l2.mix.q.norm"] == (16,) and shape["l2.norm2.b"] == (48,)
    assert shape["l0.mlp.e5.up"] == (40, 48) and shape["l0.mlp.e5.down"] == (48, 40) and shape["l0.mlp.router"] == (6, 48)
    assert shape["l0.mlp.shared.sg"] == (1, 48) and shape["l0.mlp.shared.down"] == (48, 24)
    assert not any(name.startswith("l1.mlp") or name.startswith("l1.norm2") for name in shape)
    assert "l0.mlp.shared.up" not in merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("b")).plan()))


def broken(change):
    data = copy.deepcopy(tiny.config_json("a"))
    change(data)
    return data


@pytest.mark.parametrize("change, key", [
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda d: d["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(scaling={"factor": 2.0}), "scaling"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_what_cannot_run_is_refused_with_its_key(change, key):
    with pytest.raises(ConfigError) as error:
        config_from_dict(broken(change))
    assert key in str(error.value)


def test_chunked_groups_give_back_the_pages_behind_the_current_chunk():
    book = CacheBook([GroupBook(None, 40), GroupBook(None, 40, 0, 100)], page_size=64, max_slots=2, max_pages_per_seq=20)
    slot = book.open()
    book.prepare([slot], [250])
    book.commit([slot], [250])             # the next position, 250, lies in chunk [200, 300): pages 0..2 hold nothing of it
    assert sorted(book.pages_of(0, slot)) == [0, 1, 2, 3]
    assert sorted(book.pages_of(1, slot)) == [3]
    for _ in range(50):
        book.prepare([slot], [1])
        book.commit([slot], [1])
    assert sorted(book.pages_of(1, slot)) == [4]          # position 300 starts a chunk at 300, page 4
    book.prepare([slot], [100])
    book.commit([slot], [100])
    assert sorted(book.pages_of(1, slot)) == [6]
    book.close(slot)
    book.check()
    assert book.pages[1].n_free == 40


# ----------------------------------------------------------------------------- the plain mechanisms


def test_masks():
    m = plain.chunk_mask(10, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert m[4].tolist() == [False] * 4 + [True] + [False] * 5 and m[3].tolist() == [True] * 4 + [False] * 6
    w = plain.window_mask(10, 3)
    assert w[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4 and w[1].tolist() == [True, True] + [False] * 8


def test_rotation_frequencies_with_and_without_scaling():
    f, magnitude = plain.rotary_frequencies(8, 10000.0)
    assert magnitude == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64))
    scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    g, magnitude = plain.rotary_frequencies(8, 10000.0, scaling)
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    turn = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(turn(8.0)), 0), min(math.ceil(turn(1.0)), 7)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert float(g[i]) == pytest.approx(float(f[i]) * (ramp / 4.0 + 1.0 - ramp))
    assert float(g[0]) == float(f[0]) and float(g[3]) == pytest.approx(float(f[3]) / 4.0)      # fast pairs stay, slow ones stretch


def test_rotation_layouts():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 1, 12) + 1
    pos = torch.tensor([3])
    half = plain.rotate(x, pos, 4, 100.0, "half", None, torch.float64)[0, 0]
    inter = plain.rotate(x, pos, 4, 100.0, "interleaved", None, torch.float64)[0, 0]
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert half[0].item() == pytest.approx(1 * math.cos(a0) - 3 * math.sin(a0)) and half[2].item() == pytest.approx(3 * math.cos(a0) + 1 * math.sin(a0))
    assert half[1].item() == pytest.approx(2 * math.cos(a1) - 4 * math.sin(a1))
    assert inter[0].item() == pytest.approx(1 * math.cos(a0) - 2 * math.sin(a0)) and inter[1].item() == pytest.approx(2 * math.cos(a0) + 1 * math.sin(a0))
    assert inter[3].item() == pytest.approx(4 * math.cos(a1) + 3 * math.sin(a1))
    assert torch.equal(half[4:], x[0, 0, 4:]) and torch.equal(inter[4:], x[0, 0, 4:])


def test_matrix_memory_first_tokens_by_hand():
    """Two tokens of one head, by hand: the running maximum starts at 0, not at minus infinity."""
    W, D, E, cap = 3, 2, 2, 4.0
    g = torch.Generator().manual_seed(5)
    t = {"q": torch.randn(D, W, generator=g), "k": torch.randn(D, W, generator=g), "v": torch.randn(E, W, generator=g),
         "g": torch.randn(E, W, generator=g), "o": torch.eye(W, E), "norm": torch.ones(E), "i": torch.randn(1, W, generator=g),
         "f": torch.randn(1, W, generator=g), "i.b": torch.tensor([-3.0]), "f.b": torch.tensor([1.0])}
    t = {k: v.double() for k, v in t.items()}
    x = torch.randn(2, W, generator=g).double()
    y, (S, n, m) = plain.mlstm_mixer(x, t, "", {"heads": 1, "dim": D, "vdim": E, "gate_cap": cap}, 1e-6, plain.Arithmetic(torch.float64))
    li = [cap * math.tanh((float(t["i"][0] @ x[s]) - 3.0) / cap) for s in range(2)]
    lf = [math.log(1 / (1 + math.exp(-cap * math.tanh((float(t["f"][0] @ x[s]) + 1.0) / cap)))) for s in range(2)]
    m1 = max(lf[0] + 0.0, li[0])
    m2 = max(lf[1] + m1, li[1])
    assert float(m[0]) == pytest.approx(m2)
    k = [t["k"] @ x[s] for s in range(2)]
    n2 = math.exp(lf[1] + m1 - m2) * math.exp(li[0] - m1) * k[0] + math.exp(li[1] - m2) * k[1]
    assert torch.allclose(n[0], n2)
    q2 = (t["q"] @ x[1]) * D ** -0.5
    v = [t["v"] @ x[s] for s in range(2)]
    S2 = math.exp(lf[1] + m1 - m2) * math.exp(li[0] - m1) * torch.outer(k[0], v[0]) + math.exp(li[1] - m2) * torch.outer(k[1], v[1])
    o = (S2.t() @ q2) / (max(abs(float(n2 @ q2)), math.exp(-m2)) + 1e-6)
    want = o / torch.sqrt((o * o).mean() + 1e-6) * torch.sigmoid(t["g"] @ x[1])
    assert torch.allclose(y[1, :E], want)


def test_routing_by_hand():
    z = torch.log(torch.tensor([[0.30, 0.05, 0.02, 0.28, 0.20, 0.15]], dtype=torch.float64))      # scores are these numbers
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    chosen, weights = plain.route(z, router)
    # groups (0,1), (2,3), (4,5) score 0.30, 0.28, 0.20: the last group is out, so 0.20 is not chosen
    assert sorted(chosen[0].tolist()) == [0, 3]
    assert sorted(weights[0].tolist()) == pytest.approx([0.56, 0.60])
    chosen, _ = plain.route(z, {"experts": 6, "top": 3, "scale": 1.0})
    assert sorted(chosen[0].tolist()) == [0, 3, 4]


def test_layer_norm_is_the_textbook_one():
    x = torch.randn(4, 9, dtype=torch.float64)
    w, b = torch.randn(9, dtype=torch.float64), torch.randn(9, dtype=torch.float64)
    want = torch.nn.functional.layer_norm(x, (9,), w, b, 1e-5)
    assert torch.allclose(plain.layer_norm(x, w, b, 1e-5), want)
    assert torch.allclose(plain.gelu_erf(x), torch.nn.functional.gelu(x))
