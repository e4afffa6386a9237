"""A plain, slow statement of the Gozolix design in 64-bit torch on the CPU: one function per mechanism,
whole sequences only, no cache.  The tests compare the library with it; it shares no code with the library.

Notation: h [T, W] is a sublayer's input, ``w`` a dict from tensor name (as the model file spells it) to a
64-bit tensor, ``cfg`` the config.json dict.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def embedding(tokens, w, cfg):
    """Token rows times the embedding scale, plus a row of the bigram table chosen by a hash of the token
    before and the token; a sequence's first token takes the table's last row."""
    e = cfg["embedding"]
    x = w["embed"][tokens] * e["scale"]
    bg = e.get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = [n]
        for prev, cur in zip(tokens[:-1], tokens[1:]):
            rows.append((int(prev) * int(bg["mul_prev"]) + int(cur) * int(bg["mul_cur"])) % n)
        x = x + w["bigram"][torch.tensor(rows)]
    return x


def short_conv_silu(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y * torch.sigmoid(y)


def delta_mixer(h, w, pre, m, eps):
    """The gated delta rule.  Per head a memory S [dim, vdim]:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[pre + "q"].T, w[pre + "q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ w[pre + "k"].T, w[pre + "k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ w[pre + "v"].T, w[pre + "v.conv"]).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                                   # [T, H]
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) * torch.nn.functional.softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[pre + "norm"]
    gate = (h @ w[pre + "g"].T).view(T, H, V)
    out = out * (gate * torch.sigmoid(gate))
    return out.reshape(T, H * V) @ w[pre + "o"].T


def attention_keys_values(h, w, pre, m):
    T = h.shape[0]
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, m["kv_heads"], m["dim"])
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(h, w, pre, m, k, v):
    """Softmax attention without rotation: a query temperature that grows with the position, soft-capped
    scores and a penalty on distance with a slope per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    pos = torch.arange(T)
    qt = m.get("q_temp")
    if qt:
        temp = 1.0 + qt["coef"] * torch.log(torch.floor((pos + 1).to(h.dtype) / qt["every"]) + 1.0)
        q = q * temp[:, None, None]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)
    visible = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        cap = m.get("softcap")
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s - 2.0 ** (-8.0 * (head + 1) / H) * dist
        s = s.masked_fill(~visible, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    z = torch.relu(h @ w[pre + "up"].T)
    return (z * z) @ w[pre + "down"].T


def expert_ff(h, w, pre):
    g = h @ w[pre + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """Chosen experts [T, top] and their weights [T, top]."""
    s = torch.sigmoid(h @ w[pre + "router"].T)                                # [T, E]
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        sg = s.view(T, n, per)
        score = sg.topk(min(2, per), -1).values.sum(-1)                      # [T, n]
        best = score.topk(keep, -1).indices
        allowed = torch.zeros(T, n, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, 1)
    chosen = s.masked_fill(~allowed, -1.0).topk(int(r["top"]), -1).indices
    weights = s.gather(1, chosen)
    weights = weights / (weights.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return chosen, weights


def moe_ff(h, w, pre, mlp):
    chosen, weights = route(h, w, pre, mlp["router"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            out[t] += wt * expert_ff(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert_ff(h, w, pre + "shared.")
    return out


def forward(tokens, w, cfg, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = embedding(tokens, w, cfg)
    held = {}
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "delta":
            mixed = delta_mixer(h, w, pre + "mix.", m, eps)
        else:
            if m.get("kv_from") is not None:
                k, v = held[int(m["kv_from"])]
            else:
                k, v = held[i] = attention_keys_values(h, w, pre + "mix.", m)
            mixed = attention_mixer(h, w, pre + "mix.", m, k, v)
        mlp = layer.get("mlp")
        if mlp is not None:
            mixed = mixed + (dense_ff(h, w, pre + "mlp.") if mlp.get("kind", "dense") == "dense"
                             else moe_ff(h, w, pre + "mlp.", mlp))
        x = x + mixed
        if keep_layers:
            layers.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, layers) if keep_layers else logits
