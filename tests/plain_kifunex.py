"""Plain, slow implementation of the Kifunex decoder: whole sequences, no cache, one function per mechanism,
float64 arithmetic on bfloat16-rounded weight values.  It shares no code with the package: it reads the
configuration as a dict, makes and writes its own weights, and loops over heads and tokens.

Notation.  The model keeps ``n`` copies of the residual stream, ``X[t, c]`` (token t, copy c), all equal to the
token's embedding row at the start.  A sublayer F (mixer, then feed-forward) with its three small tensors
``r`` (read, [n]), ``M`` (carry, [n, n], indexed [from, to]) and ``w`` (write, [n]) does

    u = sum_c r[c] X[:, c];   y = F(dyt(u));   X'[:, d] = sum_c M[c, d] X[:, c] + w[d] y

with ``dyt(u) = tanh(a u) * g + b`` (a scalar ``a``, vectors ``g`` and ``b``).  After the last layer the copies are
summed, ``dyt`` is applied once more, and the logits are ``cap * tanh(s * (head x) / cap)``.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ small functions
def dyt(u, a, g, b):
    return torch.tanh(a * u) * g + b


def silu(z):
    return z * torch.sigmoid(z)


def norm_of(W, name):
    return W[name + ".alpha"], W[name], W[name + ".b"]


# ------------------------------------------------------------------------------ rotation of pairs
def rotary_frequencies(rot):
    """f_i = base^(-2i / dims), then stretched by wavelength: short waves stay, long waves are divided by
    ``factor``, and between the two bounds the two are blended linearly in ``original / wavelength``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, lo, hi, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        for i, fi in enumerate(f):
            wave = 2.0 * math.pi / fi
            if wave < orig / hi:
                continue
            if wave > orig / lo:
                f[i] = fi / factor
            else:
                s = (orig / wave - lo) / (hi - lo)
                f[i] = (1.0 - s) * fi / factor + s * fi
    return torch.tensor(f, dtype=F64)


def rotate_halves(x, positions, rot):
    """x [T, heads, dim]: element i is paired with element i + dims / 2, i < dims / 2; the pair at position p is
    turned by p * f_i.  Elements from ``dims`` on pass unchanged."""
    if not rot or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f = rotary_frequencies(rot)
    ang = torch.tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ------------------------------------------------------------------------------ attention whose values are its keys
def window_attention(h, W, p, m, positions=None):
    """Grouped-query softmax attention over the last ``mask.size`` positions (the row's own among them).  There is
    no value projection: a key head as projected, before its rotation, is also the value head."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    positions = list(range(T)) if positions is None else positions
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = k.clone()
    q, k = rotate_halves(q, positions, m.get("rot")), rotate_halves(k, positions, m.get("rot"))
    size = int(m["mask"]["size"]) if m.get("mask") else 0
    scale = float(m["scale"])
    out = torch.zeros(T, H, D, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            lo = max(0, t + 1 - size) if size > 0 else 0
            s = (k[lo:t + 1, g] @ q[t, hd]) * scale
            w = torch.softmax(s, dim=0)
            out[t, hd] = w @ v[lo:t + 1, g]
    return out.reshape(T, H * D) @ W[p + "o"].T


# ------------------------------------------------------------------------------ mixture of experts
def expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, r):
    """Per token: s = sigmoid(router h); the ``top`` experts by s + correction (the lower index on a tie); their
    weights are s * scale."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    E, K = int(r["experts"]), int(r["top"])
    picks = []
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:K]
        picks.append([(e, float(s[t, e]) * float(r["scale"])) for e in order])
    return picks, choice


def choice_margins(choice, K):
    """Per token: how far the last chosen expert's choice score lies above the first one left out (inf if none is)."""
    if K >= choice.shape[1]:
        return torch.full((choice.shape[0],), float("inf"), dtype=F64)
    top = torch.sort(choice, dim=1, descending=True).values
    return top[:, K - 1] - top[:, K]


def mixture(h, W, p, mlp, margins=None):
    picks, choice = route(h, W, p, mlp["router"])
    if margins is not None:
        margins.append(choice_margins(choice, int(mlp["router"]["top"])))
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t, chosen in enumerate(picks):
        for e, w in chosen:
            out[t] += w * expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, W, p + "shared.")
    return out


# ------------------------------------------------------------------------------ the copies of the stream
def connected(X, W, p, norm, F):
    """One sublayer around the copies X [T, n, width]; ``p`` names its read / carry / write tensors."""
    r, M, w = W[p + "in"], W[p + "mix"], W[p + "out"]
    u = torch.einsum("c,tcw->tw", r, X)
    y = F(dyt(u, *norm_of(W, norm)))
    return torch.einsum("cd,tcw->tdw", M, X) + w[None, :, None] * y[:, None, :]


def weight_owner(cfg, i):
    while cfg["layers"][i].get("weights_of") is not None:
        i = int(cfg["layers"][i]["weights_of"])
    return i


# ------------------------------------------------------------------------------ the whole model
def forward(cfg, W, tokens, layer_sums=None, margins=None):
    """Logits [T, vocab] of a whole sequence.  ``layer_sums``: a list that receives the sum of the copies after
    every layer; ``margins``: a list that receives every router's ``choice_margins``."""
    T = len(tokens)
    n = int(cfg.get("streams", 1))
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    X = x[:, None, :].repeat(1, n, 1)
    for i, L in enumerate(cfg["layers"]):
        lp = f"l{weight_owner(cfg, i)}."
        X = connected(X, W, lp + "hc1.", lp + "norm1", lambda h: window_attention(h, W, lp + "mix.", L["mixer"]))
        if L.get("mlp"):
            X = connected(X, W, lp + "hc2.", lp + "norm2", lambda h: mixture(h, W, lp + "mlp.", L["mlp"], margins))
        if layer_sums is not None:
            layer_sums.append(X.sum(dim=1))
    x = dyt(X.sum(dim=1), *norm_of(W, "final.norm"))
    z = (x @ W["head"].T) * float(cfg.get("logit_scale", 1.0))
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0 else z


# ------------------------------------------------------------------------------ weights
def tensor_table(cfg):
    """name -> (shape, kind) of every tensor the model has; kinds: matrix, gain (around one), shift (around zero),
    alpha (a scalar around one), read / carry / write (the copies' small tensors), correction."""
    Wd, V, n = int(cfg["width"]), int(cfg["vocab"]), int(cfg.get("streams", 1))
    out = {"embed": ((V, Wd), "embed"), "head": ((V, Wd), "matrix")}

    def norm(name):
        out[name] = ((Wd,), "gain")
        out[name + ".b"] = ((Wd,), "shift")
        out[name + ".alpha"] = ((), "alpha")

    def hc(p):
        out[p + "in"] = ((n,), "read")
        out[p + "out"] = ((n,), "write")
        out[p + "mix"] = ((n, n), "carry")

    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        hc(p + "hc1.")
        H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
        out[p + "mix.q"] = ((H * D, Wd), "matrix")
        out[p + "mix.k"] = ((G * D, Wd), "matrix")
        out[p + "mix.o"] = ((Wd, H * D), "matrix")
        mlp = L.get("mlp")
        if mlp:
            norm(p + "norm2")
            hc(p + "hc2.")
            E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"] = ((ff, Wd), "matrix")
                out[f"{p}mlp.e{e}.up"] = ((ff, Wd), "matrix")
                out[f"{p}mlp.e{e}.down"] = ((Wd, ff), "matrix")
            out[p + "mlp.router"] = ((E, Wd), "router")
            out[p + "mlp.correction"] = ((E,), "correction")
            if mlp.get("shared"):
                sf = int(mlp["shared"]["ff"])
                out[p + "mlp.shared.gate"] = ((sf, Wd), "matrix")
                out[p + "mlp.shared.up"] = ((sf, Wd), "matrix")
                out[p + "mlp.shared.down"] = ((Wd, sf), "matrix")
    norm("final.norm")
    return out


def make_weights(cfg, seed, scale=1.0):
    """Random weights as float64 tensors holding bfloat16 values.  Sizes of the draws are chosen so that every
    sublayer's output weighs about as much as the stream it is added to."""
    g = torch.Generator().manual_seed(seed)
    n = int(cfg.get("streams", 1))
    W = {}
    for name, (shape, kind) in tensor_table(cfg).items():
        if kind in ("matrix", "router"):
            fan = shape[1]
            t = torch.randn(shape, generator=g, dtype=F64) * (scale * (2.5 if kind == "router" else 1.3) / math.sqrt(fan))
        elif kind == "embed":
            t = torch.randn(shape, generator=g, dtype=F64)
        elif kind == "gain":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g, dtype=F64)
        elif kind == "shift":
            t = 0.1 * torch.randn(shape, generator=g, dtype=F64)
        elif kind == "alpha":
            t = 0.6 + 0.4 * torch.rand(shape, generator=g, dtype=F64)
        elif kind == "read":
            t = (1.0 + 0.5 * torch.randn(shape, generator=g, dtype=F64)) / n
        elif kind == "write":
            t = 1.0 + 0.5 * torch.randn(shape, generator=g, dtype=F64)
        elif kind == "carry":
            t = torch.eye(n, dtype=F64) + 0.2 * torch.randn(shape, generator=g, dtype=F64)
        elif kind == "correction":
            t = 0.3 * torch.randn(shape, generator=g, dtype=F64)
        else:
            raise AssertionError(kind)
        W[name] = t.to(torch.bfloat16).to(F64)
    return W


def write_folder(cfg, W, folder):
    """config.json and model.safetensors (bfloat16) of a model."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name in sorted(W):
        t = W[name].to(torch.bfloat16).contiguous()
        raw = t.view(torch.int16).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
    return folder


def greedy_generate(cfg, W, prompt, n):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(torch.argmax(forward(cfg, W, seq)[-1])))
    return seq[len(prompt):]


def attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, base=10000.0, scaling=None, scale=None,
                    mlp=None, weights_of=None):
    """A layer entry of config.json."""
    L = {"type": "attention",
         "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
                   "rot": {"base": base, "dims": rot_dims, "scaling": scaling},
                   "scale": scale if scale is not None else dim ** -0.5},
         "mlp": mlp}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def moe(experts=6, top=2, ff=24, shared_ff=24, scale=1.25):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale},
            "shared": {"ff": shared_ff} if shared_ff else None}


def model_config(layers, width=64, vocab=160, streams=2, logit_scale=1.5, logit_softcap=12.0, eps=1e-6):
    return {"architecture": "Kifunex", "layers": layers, "width": width, "vocab": vocab, "streams": streams,
            "logit_scale": logit_scale, "logit_softcap": logit_softcap, "norm": {"eps": eps}}
