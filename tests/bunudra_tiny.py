"""Small Bunudra configurations of the tests' own, each unlike the others in every size and
option, and model folders with random weights for them.  Sizes visit the corners: values larger
and smaller than keys, key sizes that are no multiple of 8 or 16, one kv head for many heads and
one per head, chunks and windows shorter and longer than a cache page, partial and full rotation,
rotation with and without frequency scaling, one expert per token and several, one group and
several, a layer without a feed-forward, a feed-forward without a shared expert, every order of
the three mixers."""

import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, scale, rot=None, chunk=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def latent(heads, dim, rot_dim, vdim, rank, scale, base, window=None, scaling=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    # latent attention first, a window of five; values larger than keys in the attention layer; a
    # layer without a feed-forward; a window that crosses a page border, on keys of 32 with values of
    # 16 (in bfloat16 the cache pads such values to the keys' size for the tensor-core kernels)
    "a": dict(vocab=200, width=48, eps=1e-5, emb=3.0, seed=21, layers=[
        {"type": "latent_attention", "mixer": latent(3, 20, 6, 12, 24, 0.21, 1000.0, window=5, scaling=(4.0, 64, 8.0, 1.0)),
         "mlp": moe(6, 2, 40, groups=(3, 2), scale=1.5, shared=24)},
        {"type": "mlstm", "mixer": mlstm(2, 24, 40, 8.0), "mlp": None},
        {"type": "attention", "mixer": attention(6, 3, 16, 24, 0.3, rot=(8, 10000.0), chunk=24),
         "mlp": moe(6, 2, 40, groups=(3, 2), scale=1.5, shared=24)},
        {"type": "latent_attention", "mixer": latent(2, 24, 8, 16, 16, 0.3, 300.0, window=70),
         "mlp": moe(4, 4, 16, groups=(2, 2), scale=0.5, shared=8)},
    ]),
    # tensor-core sizes: heads of 64 with values of 64 in both attentions, chunks and a window longer
    # than a page; one head of 128 x 20 in the matrix memory; one expert per token, one group, no
    # shared expert; no frequency scaling
    "b": dict(vocab=300, width=72, eps=3e-6, emb=1.0, seed=22, layers=[
        {"type": "attention", "mixer": attention(4, 4, 64, 64, 0.125, rot=(64, 500000.0), chunk=70), "mlp": moe(4, 1, 48)},
        {"type": "mlstm", "mixer": mlstm(1, 128, 20, 15.0), "mlp": moe(4, 1, 48)},
        {"type": "latent_attention", "mixer": latent(2, 48, 16, 64, 40, 0.11, 20000.0, window=130), "mlp": moe(4, 1, 48)},
        {"type": "attention", "mixer": attention(8, 1, 32, 32, 0.18, rot=(2, 100.0), chunk=64), "mlp": None},
    ]),
    # nothing a multiple of eight: width 100, heads of 9 with values of 5, five heads of 10 x 17, a
    # latent of 11; chunks of seven and a window of three; nine experts in three groups, four per
    # token; all keys visible in the last layer (no mask)
    "c": dict(vocab=333, width=100, eps=2e-5, emb=0.5, seed=23, layers=[
        {"type": "mlstm", "mixer": mlstm(5, 10, 17, 5.0), "mlp": moe(9, 4, 30, groups=(3, 2), scale=2.5, shared=50)},
        {"type": "attention", "mixer": attention(3, 1, 9, 5, 0.4, rot=(4, 50.0), chunk=7),
         "mlp": moe(9, 4, 30, groups=(3, 2), scale=2.5, shared=50)},
        {"type": "latent_attention", "mixer": latent(2, 7, 2, 9, 11, 0.35, 77.0, window=3, scaling=(2.0, 16, 4.0, 0.5)),
         "mlp": moe(9, 4, 30, groups=(3, 2), scale=2.5, shared=50)},
        {"type": "attention", "mixer": attention(2, 2, 12, 20, 0.25), "mlp": None},
    ]),
    # what a file may leave out, and the largest sizes: chunks of exactly a page with full rotation; a
    # latent attention without a window on keys of 64 with values of 48 (padded for the tensor-core
    # kernels in bfloat16); one head with a key of 264 (64 state registers per lane); an attention
    # without rotation and without a mask on one kv head for four heads; every expert chosen, no groups,
    # no shared expert; one kept group whose experts are all chosen
    "d": dict(vocab=97, width=40, eps=1e-6, emb=7.0, seed=24, layers=[
        {"type": "attention", "mixer": attention(2, 2, 48, 48, 0.15, rot=(48, 1000000.0), chunk=64), "mlp": moe(5, 5, 24)},
        {"type": "latent_attention", "mixer": latent(3, 48, 16, 48, 24, 0.14, 500000.0, scaling=(8.0, 32, 16.0, 2.0)),
         "mlp": moe(6, 3, 16, groups=(2, 1), scale=1.0, shared=16)},
        {"type": "mlstm", "mixer": mlstm(1, 264, 8, 10.0), "mlp": moe(5, 5, 24)},
        {"type": "attention", "mixer": attention(4, 1, 32, 32, 0.2), "mlp": moe(6, 3, 16, groups=(2, 1), scale=1.0, shared=16)},
    ]),
}


def config_json(name):
    c = CONFIGS[name]
    return {"architecture": "Bunudra", "vocab": c["vocab"], "width": c["width"], "embedding": {"scale": c["emb"]},
            "norm": {"eps": c["eps"]}, "layers": c["layers"]}


def write_model(folder, name, dtype=torch.bfloat16):
    """Random weights through the library's random-weights mode (stored in bfloat16, as served
    models are), with matrices wide enough that attention weights are far from uniform.  Router
    matrices are six times wider still: the scores of the experts lie far apart, so that a
    rounding seldom decides which expert is chosen (such a flip, carried on by a recurrent layer,
    would move every later place of a sequence)."""
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import random_tensors_cpu
    from thing_htn_2026_b200.weights.safetensors_io import write_safetensors
    config = config_from_dict(config_json(name))
    tensors = random_tensors_cpu(config, CONFIGS[name]["seed"], dtype, matrix_std=0.12, gain_std=0.1)
    for key in tensors:
        if key.endswith(".mlp.router"):
            tensors[key] = (tensors[key].float() * 6.0).to(dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json(name), handle, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return folder


def tokens(name, length, seed):
    g = torch.Generator().manual_seed(9000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (length,), generator=g).tolist()
