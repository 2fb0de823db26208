"""Small Lanilix configurations of the tests' own, each unlike the others in every size and
option, and model folders with random weights for them.  Sizes are chosen to visit the corners:
key sizes that are no multiple of 4 or 32, value sizes that are no multiple of 16, one, two and
five convolution taps, layers without a feed-forward, layers that borrow another layer's
weights, attention first or last, windows shorter and longer than a cache page, kept first
positions within one page and across two, no window, no rotation, partial and full rotation,
one kv head for many heads and one per head."""

import json
import math
import os

import torch


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def attention(heads, kv_heads, dim, scale, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    return m


def mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


CONFIGS = {
    # delta and attention in turn, the second pair on the first pair's weights; small heads
    "p": dict(vocab=200, width=48, eps=1e-5, stored="float32", seed=11, layers=[
        {"type": "delta", "mixer": delta(4, 2, 24, 40, 3), "mlp": mlp(80, 1.5)},
        {"type": "attention", "mixer": attention(6, 3, 16, 0.3, rot=(8, 10000.0), mask=(24, 3)), "mlp": mlp(80, 1.5)},
        {"type": "delta", "mixer": delta(4, 2, 24, 40, 3), "mlp": mlp(80, 1.5), "weights_of": 0},
        {"type": "attention", "mixer": attention(6, 3, 16, 0.3, rot=(8, 10000.0), mask=(24, 3)), "mlp": mlp(80, 1.5),
         "weights_of": 1},
    ]),
    # attention first; head size 64; the kept positions reach into a second page; a key size of 10;
    # an attention over all keys without rotation; layers without a feed-forward
    "q": dict(vocab=300, width=72, eps=3e-6, stored="bfloat16", seed=12, layers=[
        {"type": "attention", "mixer": attention(4, 2, 64, 0.125, rot=(64, 500000.0), mask=(70, 66)), "mlp": None},
        {"type": "delta", "mixer": delta(3, 3, 10, 16, 2), "mlp": mlp(100, 3.0)},
        {"type": "attention", "mixer": attention(2, 1, 32, 0.18), "mlp": mlp(64, 0.7)},
        {"type": "delta", "mixer": delta(2, 1, 64, 24, 5), "mlp": None},
    ]),
    # one head of 128 x 128; a convolution of one tap; eight heads on one kv head, a window of five
    "r": dict(vocab=128, width=64, eps=1e-6, stored="bfloat16", seed=13, layers=[
        {"type": "delta", "mixer": delta(1, 1, 128, 128, 4), "mlp": mlp(96, 2.5)},
        {"type": "delta", "mixer": delta(2, 1, 40, 8, 1), "mlp": mlp(32, 1.0)},
        {"type": "attention", "mixer": attention(8, 1, 32, 0.25, rot=(2, 100.0), mask=(5, 0)), "mlp": mlp(96, 2.5)},
    ]),
    # nothing a multiple of eight: width 100, key size 20 with six taps, five heads; a head size of
    # 48 with three heads on one kv head and full rotation; a head size of 40 (no tensor-core
    # kernel takes it) with more kept positions than the window holds
    "s": dict(vocab=333, width=100, eps=2e-5, stored="bfloat16", seed=14, layers=[
        {"type": "delta", "mixer": delta(5, 5, 20, 12, 6), "mlp": mlp(70, 1.2)},
        {"type": "attention", "mixer": attention(3, 1, 48, 0.2, rot=(48, 20000.0), mask=(130, 1)), "mlp": mlp(70, 5.0)},
        {"type": "attention", "mixer": attention(2, 2, 40, 0.22, rot=(6, 300.0), mask=(7, 9)), "mlp": None},
        {"type": "delta", "mixer": delta(5, 5, 20, 12, 6), "mlp": mlp(70, 1.2), "weights_of": 0},
    ]),
    # a key size above 256 (64 registers of state per lane), with and without 16-byte accesses
    "t": dict(vocab=64, width=32, eps=1e-5, stored="float32", seed=15, layers=[
        {"type": "delta", "mixer": delta(2, 1, 264, 8, 2), "mlp": None},
        {"type": "delta", "mixer": delta(1, 1, 259, 20, 3), "mlp": mlp(48, 2.0)},
    ]),
}


def config_json(name):
    c = CONFIGS[name]
    return {"architecture": "Lanilix", "vocab": c["vocab"], "width": c["width"], "norm": {"eps": c["eps"]},
            "layers": c["layers"]}


def write_model(folder, name, slow_decay=True):
    """Random weights through the library's random-weights mode, then, so that what a sequence
    wrote long ago still counts at the tests' tolerances, slow decays on every other head of the
    delta layers (``A_log`` set by hand)."""
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import random_tensors_cpu
    from thing_htn_2026_b200.weights.safetensors_io import write_safetensors
    c = CONFIGS[name]
    config = config_from_dict(config_json(name))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[c["stored"]]
    tensors = random_tensors_cpu(config, c["seed"], dtype, matrix_std=0.08, gain_std=0.1)
    if slow_decay:
        for key, t in tensors.items():
            if key.endswith(".A_log"):
                for h in range(0, t.shape[0], 2):
                    t[h] = math.log(0.004 * (h + 1))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json(name), handle, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return folder


def tokens(name, length, seed):
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (length,), generator=g).tolist()
