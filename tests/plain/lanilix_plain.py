"""A plain, slow implementation of the Lanilix decoder, one function per mechanism, written
from the design's equations with torch on the CPU.  It shares no code with the library:
it reads a model folder with the tests' own safetensors reader below, walks a sequence
token by token where the design has a recurrence, and keeps no cache.

Notation.  ``x[t]`` is the residual stream at token t (width ``W``).  A layer is

    x <- x + N1b(mix(N1(x)))        x <- x + N2b(ff(N2(x)))      (the second only with a feed-forward)

with ``N(x) = x / sqrt(mean(x^2) + eps) * (1 + w)``.  ``precision`` is ``torch.float32`` or
``torch.float64`` for exact arithmetic, or ``torch.bfloat16`` for an emulation of serving
precision: operands and results of matrix products are rounded to bfloat16, everything
else stays in float32.
"""

import json
import math
import os
import struct

import numpy as np
import torch


# ----------------------------------------------------------------------------- reading


def read_safetensors(path):
    with open(path, "rb") as handle:
        (n,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(n).decode("utf-8"))
        data = handle.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8)
        if meta["dtype"] == "BF16":
            wide = raw.view("<u2").astype(np.uint32) << 16
            t = torch.from_numpy(wide.view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(raw.view("<f4").copy())
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(raw.view("<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(meta["shape"])
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


# ----------------------------------------------------------------------------- precision


class Arithmetic:
    """``work``: the type everything is computed in; ``round_products``: whether operands and
    results of matrix products pass through bfloat16."""

    def __init__(self, precision):
        self.round_products = precision == torch.bfloat16
        self.work = torch.float32 if self.round_products else precision

    def rb(self, t):
        return t.to(torch.bfloat16).to(self.work) if self.round_products else t

    def linear(self, x, w):
        """w is stored [out, in] and applied as w x."""
        return self.rb(self.rb(x) @ self.rb(w.to(self.work)).t())


# ----------------------------------------------------------------------------- mechanisms


def norm_one_plus(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w), over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w.to(x.dtype))


def norm_plain_weight(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w, over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(x.dtype)


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x, taps_w):
    """x [T, C]; taps_w [C, K], last column multiplies the current token, zeros before the
    start: y[t, c] = sum_j taps_w[c, j] * x[t - (K - 1) + j, c]."""
    T, C = x.shape
    K = taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + T] * taps_w[:, j].to(x.dtype)
    return y


def delta_recurrence(q, k, v, beta, decay):
    """One head, token by token.  q, k [T, dk] (already unit vectors, q scaled), v [T, dv],
    beta, decay [T].  S [dk, dv] starts at zero:
        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    out = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.t() @ q[t]
    return out


def delta_mixer(h, w, prefix, sizes, eps, ar):
    """h [T, W] -> [T, W].  ``sizes``: the layer's 'mixer' entry."""
    T = h.shape[0]
    heads, kv_heads, dk, dv = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    per = heads // kv_heads
    q = silu(causal_conv(ar.linear(h, w[prefix + "q"]), w[prefix + "q.conv"].to(ar.work)))
    k = silu(causal_conv(ar.linear(h, w[prefix + "k"]), w[prefix + "k.conv"].to(ar.work)))
    v = silu(causal_conv(ar.linear(h, w[prefix + "v"]), w[prefix + "v.conv"].to(ar.work)))
    q = q.reshape(T, kv_heads, dk)
    k = k.reshape(T, kv_heads, dk)
    v = v.reshape(T, heads, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(ar.linear(h, w[prefix + "b"]))                                   # [T, heads]
    rate = torch.exp(w[prefix + "A_log"].to(ar.work))
    step = torch.nn.functional.softplus(ar.linear(h, w[prefix + "a"]) + w[prefix + "dt_bias"].to(ar.work))
    decay = torch.exp(-rate * step)                                                       # [T, heads]
    gate = silu(ar.linear(h, w[prefix + "g"])).reshape(T, heads, dv)
    out = torch.zeros(T, heads, dv, dtype=ar.work)
    for head in range(heads):
        o = delta_recurrence(q[:, head // per], k[:, head // per], v[:, head], beta[:, head], decay[:, head])
        out[:, head] = norm_plain_weight(o, w[prefix + "norm"], eps) * gate[:, head]
    return ar.linear(out.reshape(T, heads * dv), w[prefix + "o"])


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, d]: the first ``dims`` entries of each head are rotated, entry 2i with
    entry 2i + 1, by the angle position * base^(-2i / dims); the rest pass."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (base ** (-2.0 * i / dims)).to(x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                                # [T, dims / 2]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def windowed_attention(h, w, prefix, sizes, eps, ar):
    """h [T, W] -> [T, W].  The values are the keys as projected."""
    T = h.shape[0]
    heads, kv_heads, d = sizes["heads"], sizes["kv_heads"], sizes["dim"]
    per = heads // kv_heads
    q_flat = ar.linear(h, w[prefix + "q"])
    k_flat = ar.linear(h, w[prefix + "k"])
    values = k_flat.reshape(T, kv_heads, d)
    q = norm_plain_weight(q_flat, w[prefix + "q.norm"], eps).reshape(T, heads, d)
    k = norm_plain_weight(k_flat, w[prefix + "k.norm"], eps).reshape(T, kv_heads, d)
    positions = torch.arange(T)
    rot = sizes.get("rot") or {}
    q = rotate_pairs(q, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_pairs(k, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    mask = sizes.get("mask") or {}
    size, keep_first = int(mask.get("size", T + 1)), int(mask.get("keep_first", 0))
    out = torch.zeros(T, heads, values.shape[-1], dtype=ar.work)
    for t in range(T):
        seen = [j for j in range(t + 1) if visible(t, j, size, keep_first)]
        for head in range(heads):
            g = head // per
            scores = (k[seen, g] @ q[t, head]) * sizes["scale"]
            weights = torch.softmax(scores, dim=0)
            out[t, head] = weights @ values[seen, g]
    return ar.linear(out.reshape(T, -1), w[prefix + "o"])


def clamped_glu(h, w, prefix, sizes, ar):
    """g = min(gate h, limit); u = clamp(up h, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    limit = float(sizes["limit"])
    g = torch.clamp(ar.linear(h, w[prefix + "gate"]), max=limit)
    u = torch.clamp(ar.linear(h, w[prefix + "up"]), min=-limit, max=limit)
    return ar.linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[prefix + "down"])


# ----------------------------------------------------------------------------- the model


def residual_streams(config, w, tokens, precision=torch.float32):
    """[layers run + 1, T, W]: the stream after the embedding and after every layer."""
    ar = Arithmetic(precision)
    eps = float(config["norm"]["eps"])
    x = ar.rb(w["embed"].to(ar.work))[torch.tensor(tokens, dtype=torch.long)]
    streams = [x]
    for index, layer in enumerate(config["layers"]):
        owner = layer.get("weights_of", index)
        p = f"l{owner}."
        n = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "delta":
            branch = delta_mixer(n, w, p + "mix.", layer["mixer"], eps, ar)
        elif layer["type"] == "attention":
            branch = windowed_attention(n, w, p + "mix.", layer["mixer"], eps, ar)
        else:
            raise ValueError(f"layer {index}: unknown type {layer['type']}")
        x = x + norm_one_plus(branch, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            n = norm_one_plus(x, w[p + "norm2"], eps)
            x = x + norm_one_plus(clamped_glu(n, w, p + "mlp.", layer["mlp"], ar), w[p + "norm2b"], eps)
        streams.append(x)
    return torch.stack(streams)


def logits_of_stream(config, w, x, precision=torch.float32):
    ar = Arithmetic(precision)
    n = norm_one_plus(x, w["final.norm"], float(config["norm"]["eps"]))
    if ar.round_products:
        return ar.rb(n) @ ar.rb(w["head"].to(ar.work)).t()        # logits keep the accumulator's precision
    return n @ w["head"].to(ar.work).t()


def model_logits(folder, tokens, precision=torch.float32):
    """Logits [T, vocab] at every place of one sequence."""
    config, w = read_model(folder)
    with torch.no_grad():
        x = residual_streams(config, w, tokens, precision)[-1]
        return logits_of_stream(config, w, x, precision).to(torch.float32)
