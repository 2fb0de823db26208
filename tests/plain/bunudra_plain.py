"""A plain, slow implementation of the Bunudra decoder, one function per mechanism, written
from the design's equations with torch on the CPU.  It shares no code with the library: it
reads a model folder with its own safetensors reader, walks a sequence token by token where
the design has a recurrence, builds every mask as a full matrix and keeps no cache.

Notation.  ``x[t]`` is the residual stream at token t (width ``W``); a layer is

    x <- x + LN1(mix(x))        x <- x + LN2(ff(x))          (the second only with a feed-forward)

with ``LN(y) = (y - mean y) / sqrt(var y + eps) * w + b``: the norm stands on a sublayer's
output, the sublayers read the stream itself.  ``precision`` is ``torch.float32`` or
``torch.float64`` for exact arithmetic, or ``torch.bfloat16`` for an emulation of serving
precision: operands and results of matrix products are rounded to bfloat16, everything else
stays in float32.
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
            t = torch.from_numpy((raw.view("<u2").astype(np.uint32) << 16).view(np.float32).copy())
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

    def linear(self, x, w, keep=False):
        """``x @ w.T`` for a weight matrix of shape [outputs, inputs]; ``keep``: the result is not rounded."""
        y = self.rb(x) @ self.rb(w.to(self.work)).t()
        return y if keep else self.rb(y)


# ----------------------------------------------------------------------------- small pieces


def layer_norm(y, w, b, eps):
    mean = y.mean(-1, keepdim=True)
    var = ((y - mean) ** 2).mean(-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * w + b


def over_rms(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotary_frequencies(dims, base, scaling=None):
    """(frequencies [dims / 2] in float64, magnitude of cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn(t):      # the (fractional) pair index whose wavelength fits `original` t times
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, base, layout, scaling, work):
    """x [T, heads, D]: the first ``dims`` entries of every head are rotated by the token's
    position; ``layout`` "half" pairs entry i with i + dims/2, "interleaved" 2i with 2i+1."""
    if not dims:
        return x
    f, magnitude = rotary_frequencies(dims, base, scaling)
    angle = positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]      # 32-bit angles
    if work == torch.float64:
        angle = positions.to(torch.float64)[:, None] * f[None, :]
    cos = (torch.cos(angle) * magnitude).to(work)[:, None, :]
    sin = (torch.sin(angle) * magnitude).to(work)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_attention(q, k, v, scale, visible):
    """q [T, H, D], k [T, G, D], v [T, G, E], visible [T, T] bool -> [T, H, E]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def chunk_mask(T, size):
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def window_mask(T, size):
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


# ----------------------------------------------------------------------------- mixers


def attention_mixer(h, t, prefix, m, eps, ar):
    """Grouped-query attention, q/k norm per head, partial rotate-half rotation, chunked mask."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = ar.linear(h, t[prefix + "q"]).view(T, H, D)
    k = ar.linear(h, t[prefix + "k"]).view(T, G, D)
    v = ar.linear(h, t[prefix + "v"]).view(T, G, E)
    q = over_rms(q, eps) * t[prefix + "q.norm"].to(ar.work)
    k = over_rms(k, eps) * t[prefix + "k.norm"].to(ar.work)
    rot = m.get("rot")
    pos = torch.arange(T)
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], "half", rot.get("scaling"), ar.work)
        k = rotate(k, pos, rot["dims"], rot["base"], "half", rot.get("scaling"), ar.work)
    mask = m.get("mask")
    visible = chunk_mask(T, mask["size"]) if mask else window_mask(T, T)
    a = softmax_attention(ar.rb(q), ar.rb(k), v, float(m["scale"]), visible)
    return ar.linear(a.reshape(T, H * E), t[prefix + "o"])


def latent_attention_mixer(h, t, prefix, m, eps, ar):
    """Attention whose keys and values are read out of one low-rank latent per token, with a
    rotated key part shared by the heads, a sliding window and an output gate."""
    T = h.shape[0]
    H, D, R, E, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    q = ar.linear(h, t[prefix + "q"]).view(T, H, D + R)
    down = ar.linear(h, t[prefix + "dkv"])
    c = over_rms(down[:, :C], eps) * t[prefix + "dkv.norm"].to(ar.work)
    k_rot = down[:, C:].view(T, 1, R)
    k_plain = ar.linear(c, t[prefix + "uk"]).view(T, H, D)
    v = ar.linear(c, t[prefix + "uv"]).view(T, H, E)
    pos = torch.arange(T)
    q_rot = rotate(q[..., D:], pos, R, rot["base"], "interleaved", rot.get("scaling"), ar.work)
    k_rot = rotate(k_rot, pos, R, rot["base"], "interleaved", rot.get("scaling"), ar.work)
    q_all = torch.cat([q[..., :D], q_rot], dim=-1)
    k_all = torch.cat([k_plain, k_rot.expand(T, H, R)], dim=-1)
    mask = m.get("mask")
    visible = window_mask(T, mask["size"] if mask else T)
    a = softmax_attention(ar.rb(q_all), ar.rb(k_all), v, float(m["scale"]), visible).reshape(T, H * E)
    gate = torch.sigmoid(ar.linear(h, t[prefix + "g"]))
    return ar.linear(a * gate, t[prefix + "o"])


def mlstm_mixer(h, t, prefix, m, eps, ar, state=None):
    """Matrix memory with exponential gating, token by token.  ``state`` (S, n, m) may carry
    a sequence on; the new state is returned beside the output."""
    T = h.shape[0]
    H, D, E, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    w = ar.work
    q = ar.linear(h, t[prefix + "q"]).view(T, H, D) * D ** -0.5
    k = ar.linear(h, t[prefix + "k"]).view(T, H, D)
    v = ar.linear(h, t[prefix + "v"]).view(T, H, E)
    gi = ar.linear(h, t[prefix + "i"], keep=True) + t[prefix + "i.b"].to(w)
    gf = ar.linear(h, t[prefix + "f"], keep=True) + t[prefix + "f.b"].to(w)
    gi = cap * torch.tanh(gi / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(gf / cap))
    if state is None:
        state = (torch.zeros(H, D, E, dtype=w), torch.zeros(H, D, dtype=w), torch.zeros(H, dtype=w))
    S, n, mx = (s.clone() for s in state)
    out = torch.zeros(T, H, E, dtype=w)
    for s in range(T):
        m_new = torch.maximum(gf[s] + mx, gi[s])
        keep, take = torch.exp(gf[s] + mx - m_new), torch.exp(gi[s] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[s]
        mx = m_new
        top = torch.einsum("hde,hd->he", S, q[s])
        bottom = torch.maximum((n * q[s]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[s] = top / bottom[:, None]
    y = over_rms(out, eps).reshape(T, H * E) * t[prefix + "norm"].to(w)
    y = y * torch.sigmoid(ar.linear(h, t[prefix + "g"]))
    return ar.linear(y, t[prefix + "o"]), (S, n, mx)


# ----------------------------------------------------------------------------- feed-forward


def route(z, router):
    """z [T, experts] router logits -> (chosen [T, top], weights [T, top])."""
    s = torch.softmax(z, dim=-1)
    T, n = s.shape
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = router.get("groups")
    if groups:
        per = n // groups["count"]
        best = s.view(T, groups["count"], per).max(-1).values.topk(groups["keep"], dim=-1).indices
        on = torch.zeros(T, groups["count"], dtype=torch.bool)
        on[torch.arange(T)[:, None], best] = True
        allowed = on[:, :, None].expand(T, groups["count"], per).reshape(T, n)
    chosen = s.masked_fill(~allowed, -1.0).topk(router["top"], dim=-1).indices
    return chosen, s.gather(-1, chosen) * float(router.get("scale", 1.0))


def expert(h, t, prefix, ar):
    return ar.linear(gelu_erf(ar.linear(h, t[prefix + "up"])), t[prefix + "down"])


def moe(h, t, prefix, mlp, ar):
    router = mlp["router"]
    z = ar.linear(h, t[prefix + "router"], keep=True)
    chosen, weights = route(z, router)
    out = torch.zeros_like(h)
    for e in range(router["experts"]):
        for slot in range(router["top"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += weights[rows, slot, None] * expert(h[rows], t, f"{prefix}e{e}.", ar)
    if mlp.get("shared"):
        gate = torch.sigmoid(ar.linear(h, t[prefix + "shared.sg"], keep=True))
        out = out + gate * expert(h, t, prefix + "shared.", ar)
    return out


# ----------------------------------------------------------------------------- the model


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer}


def forward(config, tensors, tokens, precision=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after
    every layer."""
    ar = Arithmetic(precision)
    w = ar.work
    t = {k: v.to(w) if v.is_floating_point() else v for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] == "mlstm":
            y, _ = mlstm_mixer(x, t, p + "mix.", layer["mixer"], eps, ar)
        else:
            y = MIXERS[layer["type"]](x, t, p + "mix.", layer["mixer"], eps, ar)
        x = x + layer_norm(y, t[p + "norm1"], t[p + "norm1.b"], eps)
        if layer.get("mlp"):
            y = moe(x, t, p + "mlp.", layer["mlp"], ar)
            x = x + layer_norm(y, t[p + "norm2"], t[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    return ar.linear(x, t["head"], keep=True)


def greedy(config, tensors, prompt, n_new, precision=torch.float64):
    out = list(prompt)
    for _ in range(n_new):
        out.append(int(forward(config, tensors, out, precision)[-1].argmax()))
    return out[len(prompt):]
