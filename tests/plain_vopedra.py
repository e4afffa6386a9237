"""A plain, slow implementation of the Vopedra design on the CPU.

Whole sequences, no cache, no batching, one function per mechanism, written
from the design's equations.  It imports nothing from gopherllm_b200.
Arithmetic is float64 unless ``dtype`` says otherwise.

Notation: h is a mixer's input [T, width]; W x means x @ W.T (weights are
stored [out, in]); every recurrence runs token by token from a zero state.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


def read_folder(folder, dtype=torch.float64):
    """config.json and every tensor of model.safetensors, widened to ``dtype`` (integer tables stay
    integers).  Own small reader of the container: 8-byte length, JSON table, raw data."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        table = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
             "I32": torch.int32}
    out = {}
    for name, info in table.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t if info["dtype"] == "I32" else t.to(dtype)
    return cfg, out


# --------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis; w None leaves the unit-RMS vector."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


def gated_feed_forward(h, w_gate, w_up, w_down):
    """W_down (gelu_tanh(W_gate h) * (W_up h))."""
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------
def mlstm_mixer(h, t, pre, m, eps):
    """Matrix memory with exponential gates held stable by a running maximum that starts at 0.
    t: tensors, pre: name prefix ("l0.mix."), m: the mixer's sizes."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ t[pre + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ t[pre + "k"].T).view(T, H, D)
    v = (h @ t[pre + "v"].T).view(T, H, V)
    gi = cap * torch.tanh((h @ t[pre + "i"].T + t[pre + "i.b"]) / cap)                   # [T, H] log input gate
    gf = log_sigmoid(cap * torch.tanh((h @ t[pre + "f"].T + t[pre + "f.b"]) / cap))      # [T, H] log forget gate
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        n = torch.zeros(D, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for s in range(T):
            m_new = torch.maximum(gf[s, a] + mx, gi[s, a])
            keep, take = torch.exp(gf[s, a] + mx - m_new), torch.exp(gi[s, a] - m_new)
            S = keep * S + take * torch.outer(k[s, a], v[s, a])
            n = keep * n + take * k[s, a]
            mx = m_new
            den = torch.maximum(torch.abs(n @ q[s, a]), torch.exp(-mx)) + 1e-6
            out[s, a] = (S.T @ q[s, a]) / den
    out = rms_norm(out, None, eps).reshape(T, H * V) * t[pre + "norm"]
    out = out * torch.sigmoid(h @ t[pre + "g"].T)
    return out @ t[pre + "o"].T


def mamba1_mixer(h, t, pre, m):
    """Selective state-space scan with a short causal convolution in front."""
    T = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ t[pre + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    w, b = t[pre + "conv"], t[pre + "conv.b"]                         # [inner, taps], [inner]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], 0)
    xc = torch.stack([(padded[s:s + taps].T * w).sum(-1) + b for s in range(T)], 0)
    xc = silu(xc)
    proj = xc @ t[pre + "x"].T
    dt, Bm, Cm = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(dt @ t[pre + "dt"].T + t[pre + "dt.b"])             # [T, inner]
    A = -torch.exp(t[pre + "A_log"])                                  # [inner, N]
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for s in range(T):
        S = torch.exp(dt[s][:, None] * A) * S + (dt[s] * xc[s])[:, None] * Bm[s][None, :]
        y[s] = S @ Cm[s] + t[pre + "D"] * xc[s]
    return (y * silu(z)) @ t[pre + "o"].T


def rotate_half_pairs(x, positions, dims, base):
    """x [T, heads, dim]: dimension i of the first ``dims`` is paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    ang = (positions.to(torch.float64)[:, None] * freq[None, :]).to(x.dtype)      # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def talking_attention(h, t, pre, m, eps, positions):
    """Grouped-query softmax attention; queries and keys normalised over the whole projection, partly
    rotated; the softmax weights of the heads are mixed by a square table before they meet the values."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ t[pre + "q"].T, t[pre + "q.norm"], eps).view(T, H, D)
    k = rms_norm(h @ t[pre + "k"].T, t[pre + "k.norm"], eps).view(T, G, D)
    v = (h @ t[pre + "v"].T).view(T, G, V)
    q = rotate_half_pairs(q, positions, m["rot"]["dims"], float(m["rot"]["base"]))
    k = rotate_half_pairs(k, positions, m["rot"]["dims"], float(m["rot"]["base"]))
    per = H // G
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    weights = []
    for a in range(H):
        s = (q[:, a] @ k[:, a // per].T) * float(m["scale"])
        s = s.masked_fill(~causal, float("-inf"))
        weights.append(torch.softmax(s, -1))
    weights = torch.stack(weights, 0)                                   # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", t[pre + "talk"], weights)
    out = torch.stack([mixed[a] @ v[:, a // per] for a in range(H)], 1)   # [T, H, V]
    return out.reshape(T, H * V) @ t[pre + "o"].T


def hgrn2_mixer(h, t, pre, m, eps):
    """Linear attention whose forget gate, bounded from below, also says what is written."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ t[pre + "q"].T).view(T, H, D)
    v = (h @ t[pre + "v"].T).view(T, H, V)
    low = t[pre + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ t[pre + "f"].T + t[pre + "f.b"])).view(T, H, D)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for s in range(T):
            S = f[s, a][:, None] * S + torch.outer(1.0 - f[s, a], v[s, a])
            out[s, a] = S.T @ q[s, a]
    out = rms_norm(out, t[pre + "norm"], eps).reshape(T, H * V)
    return out @ t[pre + "o"].T


def parallel_mixer(h, t, pre, m, eps, positions):
    """Half the sum of two mixers' outputs, each normalised over the model width first."""
    left = talking_attention(h, t, pre + "left.", m["left"], eps, positions)
    right = hgrn2_mixer(h, t, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, t[pre + "left.out"], eps) + rms_norm(right, t[pre + "right.out"], eps))


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def layer_order(cfg):
    """[(layer index, number of the pass or None, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or None
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(a)]
    for p in range(times):
        order += [(i, p, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def forward(cfg, t, tokens, dtype=torch.float64, want_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = rms_norm(t["embed"][tokens].to(dtype), t["embed.norm"], eps)
    x0 = x.clone()
    trail = []
    for i, p, first in layer_order(cfg):
        if first:
            if p > 0:
                x = x + x0
            x = x + t["loop.step"][p]
        L = cfg["layers"][i]
        pre = f"l{i}."
        hn = rms_norm(x, t[pre + "norm1"], eps)
        if L["type"] == "mlstm":
            mix = mlstm_mixer(hn, t, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "mamba1":
            mix = mamba1_mixer(hn, t, pre + "mix.", L["mixer"])
        elif L["type"] == "parallel":
            mix = parallel_mixer(hn, t, pre + "mix.", L["mixer"], eps, positions)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            h2 = rms_norm(x, t[pre + "norm2"], eps)
            mix = mix + gated_feed_forward(h2, t[pre + "mlp.gate"], t[pre + "mlp.up"], t[pre + "mlp.down"])
        x = x + mix
        trail.append(x.clone())
    logits = rms_norm(x, t["final.norm"], eps) @ t["head"].T
    return (logits, torch.stack(trail, 0)) if want_layers else logits
