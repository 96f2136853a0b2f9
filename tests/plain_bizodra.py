"""Plain, slow implementation of the Bizodra decoder: whole sequences, no cache, one function per mechanism,
float64 arithmetic on bfloat16-rounded weight values.  It shares no code with the package: it reads the
configuration as a dict, makes and writes its own weights, and loops over tokens where the model is recurrent.

Notation.  ``rms(x) = x / sqrt(mean(x^2) + eps)`` over the last axis.  A layer is
``x += rms(mixer(x)) (1 + w1)``, then ``x += rms(mlp(x)) (1 + w2)`` if it has an MLP, then the token input
``x += rms(P (gelu_tanh(G x) * e_token)) w3`` if the model has one.  The sublayers read ``x`` itself.
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
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z * torch.sigmoid(z)


def log_sigmoid(z):
    return -torch.log1p(torch.exp(-z.abs())) + torch.minimum(z, torch.zeros_like(z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.maximum(z, torch.zeros_like(z))


# ------------------------------------------------------------------------------ matrix LSTM
def matrix_lstm(h, W, p, m, eps, trace=None):
    """h [T, width] -> [T, width].  Per head, token by token:
    m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' likewise with k;
    o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6), where q is scaled by dim^(-1/2)."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[p + "q"].T).view(T, H, dk) / math.sqrt(dk)
    k = (h @ W[p + "k"].T).view(T, H, dk)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    gf = log_sigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        n = torch.zeros(dk, dtype=F64)
        mx = torch.zeros((), dtype=F64)
        for t in range(T):
            m_new = torch.maximum(gf[t, hd] + mx, gi[t, hd])
            keep, take = torch.exp(gf[t, hd] + mx - m_new), torch.exp(gi[t, hd] - m_new)
            S = keep * S + take * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + take * k[t, hd]
            mx = m_new
            den = torch.maximum((n @ q[t, hd]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
        if trace is not None:
            trace.append((S, n, mx))
    y = rms(out, eps).reshape(T, H * dv) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


# ------------------------------------------------------------------------------ rotation of pairs
def rotary_frequencies(rot):
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def where(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(float(sc["fast"]))), 0)
        hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
        for i in range(len(f)):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=F64), amp


def rotate_interleaved(x, positions, rot):
    """x [T, heads, dim]: elements (2i, 2i + 1), i < dims / 2, are turned by positions * f_i."""
    f, amp = rotary_frequencies(rot)
    dims = rot["dims"]
    if dims == 0:
        return x
    ang = torch.tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ------------------------------------------------------------------------------ attention with a sink
def sink_attention(h, W, p, m, eps, positions=None):
    """Causal attention over all earlier keys with p_j = e^(s_j) / (1 + sum_i e^(s_i))."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, Dv)
    q = rotate_interleaved(rms(q, eps) * W[p + "q.norm"], positions, m["rot"])
    k = rotate_interleaved(rms(k, eps) * W[p + "k.norm"], positions, m["rot"])
    out = torch.zeros(T, H, Dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * float(m["scale"])
            e = torch.exp(s)
            out[t, hd] = (e / (1.0 + e.sum())) @ v[:t + 1, g]
    return out.reshape(T, H * Dv) @ W[p + "o"].T + W[p + "o.b"]


# ------------------------------------------------------------------------------ gated delta rule
def short_conv(x, w):
    """x [T, C], w [C, taps], last column the current token's, zeros before the start; then silu."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                y[t] += w[:, j] * x[src]
    return silu(y)


def gated_delta(h, W, p, m, eps, trace=None):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, dk)
    k = short_conv(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, dk)
    v = short_conv(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
        if trace is not None:
            trace.append(S)
    y = (rms(out, eps) * W[p + "norm"]).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


def side_by_side(h, W, p, m, eps):
    a = sink_attention(h, W, p + "left.", m["left"], eps)
    b = gated_delta(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms(a, eps) * W[p + "left.out"] + rms(b, eps) * W[p + "right.out"])


# ------------------------------------------------------------------------------ the rest of a layer
def dense_mlp(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def token_input(h, ids, W, p, layer, dim):
    e = W["side.embed"][ids][:, layer * dim:(layer + 1) * dim]
    return (gelu_tanh(h @ W[p + "gate"].T) * e) @ W[p + "proj"].T


def forward(cfg, W, ids, layers_out=None):
    """float64 logits [T, vocab] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.tensor(list(ids), dtype=torch.long)
    x = W["embed"][ids]
    side = (cfg.get("token_side") or {}).get("dim", 0)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] in ("mlstm", "mlstm_2"):
            y = matrix_lstm(x, W, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = side_by_side(x, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + rms(y, eps) * (1.0 + W[p + "norm1"])
        if L.get("mlp"):
            x = x + rms(dense_mlp(x, W, p + "mlp."), eps) * (1.0 + W[p + "norm2"])
        if side:
            x = x + rms(token_input(x, ids, W, p + "side.", i, side), eps) * W[p + "side.norm"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * (1.0 + W["final.norm"])) @ W["head"].T


def greedy_generate(cfg, W, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]


# ------------------------------------------------------------------------------ weights of our own
def tensor_shapes(cfg):
    """name -> (shape, kind); kind: 'w' matrix, 'z' vector around zero, 'o' vector around one, 'c' conv taps,
    'a' decay rate, 'd' decay bias."""
    Wd, V = cfg["width"], cfg["vocab"]
    side = (cfg.get("token_side") or {}).get("dim", 0)
    out = {"embed": ((V, Wd), "e"), "head": ((V, Wd), "w"), "final.norm": ((Wd,), "z")}
    if side:
        out["side.embed"] = ((V, side * len(cfg["layers"])), "e")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = ((Wd,), "z")
        m = L["mixer"]
        if L["type"] in ("mlstm", "mlstm_2"):
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": ((H * dk, Wd), "w"), p + "mix.k": ((H * dk, Wd), "w"), p + "mix.v": ((H * dv, Wd), "w"),
                        p + "mix.g": ((H * dv, Wd), "w"), p + "mix.o": ((Wd, H * dv), "w"), p + "mix.norm": ((H * dv,), "o"),
                        p + "mix.i": ((H, Wd), "w"), p + "mix.i.b": ((H,), "z"), p + "mix.f": ((H, Wd), "w"),
                        p + "mix.f.b": ((H,), "f")})
        else:
            a, r = m["left"], m["right"]
            l, rr = p + "mix.left.", p + "mix.right."
            out.update({l + "q": ((a["heads"] * a["dim"], Wd), "w"), l + "q.b": ((a["heads"] * a["dim"],), "z"),
                        l + "k": ((a["kv_heads"] * a["dim"], Wd), "w"), l + "k.b": ((a["kv_heads"] * a["dim"],), "z"),
                        l + "v": ((a["kv_heads"] * a["vdim"], Wd), "w"), l + "v.b": ((a["kv_heads"] * a["vdim"],), "z"),
                        l + "q.norm": ((a["dim"],), "o"), l + "k.norm": ((a["dim"],), "o"),
                        l + "o": ((Wd, a["heads"] * a["vdim"]), "w"), l + "o.b": ((Wd,), "z"),
                        rr + "q": ((r["kv_heads"] * r["dim"], Wd), "w"), rr + "q.conv": ((r["kv_heads"] * r["dim"], r["conv"]), "c"),
                        rr + "k": ((r["kv_heads"] * r["dim"], Wd), "w"), rr + "k.conv": ((r["kv_heads"] * r["dim"], r["conv"]), "c"),
                        rr + "v": ((r["heads"] * r["vdim"], Wd), "w"), rr + "v.conv": ((r["heads"] * r["vdim"], r["conv"]), "c"),
                        rr + "b": ((r["heads"], Wd), "w"), rr + "a": ((r["heads"], Wd), "w"),
                        rr + "A_log": ((r["heads"],), "a"), rr + "dt_bias": ((r["heads"],), "d"),
                        rr + "norm": ((r["vdim"],), "o"), rr + "g": ((r["heads"] * r["vdim"], Wd), "w"),
                        rr + "o": ((Wd, r["heads"] * r["vdim"]), "w"),
                        p + "mix.left.out": ((Wd,), "o"), p + "mix.right.out": ((Wd,), "o")})
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out.update({p + "norm2": ((Wd,), "z"), p + "mlp.up": ((ff, Wd), "w"), p + "mlp.down": ((Wd, ff), "w")})
        if side:
            out.update({p + "side.gate": ((side, Wd), "w"), p + "side.proj": ((Wd, side), "w"), p + "side.norm": ((Wd,), "o")})
    return out


def to_bf16(t):
    return t.to(torch.float32).to(torch.bfloat16).to(F64)


def random_weights(cfg, seed, std=None):
    """float64 tensors whose values are bfloat16 numbers.  Matrices N(0, 1/sqrt(fan_in)) so that activations keep
    their size; embeddings N(0, 1); norm weights around 0 or 1; gates' biases so that the memories neither forget
    at once nor never."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g, dtype=F64)
        if kind == "w":
            t = r * (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        elif kind == "e":
            t = r
        elif kind == "z":
            t = 0.2 * r
        elif kind == "o":
            t = 1.0 + 0.2 * r
        elif kind == "c":
            t = 0.5 * r
        elif kind == "f":
            t = 2.0 + r
        elif kind == "a":
            t = -1.0 + 0.5 * r
        else:
            t = 0.5 * r
        W[name] = to_bf16(t)
    return W


def _bf16_bits(t):
    u = t.to(torch.float32).contiguous().numpy().view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write_folder(cfg, W, out_dir):
    """config.json and model.safetensors (BF16): 8 bytes of header length, the JSON header, the data."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name in sorted(W):
        raw = _bf16_bits(W[name]).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(W[name].shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return out_dir
