"""Porovik written out plainly and slowly in 64-bit, one function per mechanism, token loops where the design has a
recurrence.  It shares no code with the package.  Every function takes the rows of one request (whole, or a piece
with the state an earlier piece left) and the tensors by their names in the weight file.

    embed               token row + hashed bigram row + position row
    weight_norm         x / sqrt(mean(x^2) + eps) * (1 + w)
    gate_write          S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;  o_t = S_t^T q_t
    general_delta       S_t = diag(w_t) S_(t-1) - (a_t u_t) (u_t^T S_(t-1)) + k_t v_t^T;  o_t = S_t^T r_t
    biased_attention    softmax(q k^T scale - slope_h (i - j)) v with a query temperature, mixed values, a gate
    dense_ff, expert_ff the two feed-forwards
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weight_norm(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w.double())


def lin(x, w):
    return x @ w.double().T


def embed(tokens: List[int], W, cfg, state) -> torch.Tensor:
    """state: {"before": the request's last token or None, "pos": tokens so far}."""
    rows = []
    bg = (cfg.get("embedding") or {}).get("bigram")
    for t in tokens:
        x = W["embed"][t].double()
        if bg:
            b = state["before"]
            row = bg["buckets"] if b is None else (b * bg["mul_prev"] + t * bg["mul_cur"]) % bg["buckets"]
            x = x + W["bigram"][row].double()
        x = x + W["pos"][state["pos"]].double()
        state["before"], state["pos"] = t, state["pos"] + 1
        rows.append(x)
    return torch.stack(rows)


def gate_write(h, W, m, state, eps, at="mix."):
    """state: {"S": [heads, dim, vdim]}."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = silu(lin(h, W[at + "q"])).reshape(T, H, dk)
    v = lin(h, W[at + "v"]).reshape(T, H, dv)
    low = W[at + "lower"].double()
    f = (low + (1.0 - low) * sigmoid(lin(h, W[at + "f"]) + W[at + "f.b"].double())).reshape(T, H, dk)
    S = state["S"]
    out = []
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    state["S"] = S
    o = unit_rms(torch.stack(out), eps) * W[at + "norm"].double()
    return lin(o.reshape(T, H * dv), W[at + "o"])


def general_delta(h, W, m, state, eps, at="mix.", decay_scale=math.exp(-0.5)):
    """state: {"S": [heads, dim, vdim]}."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m.get("vdim", m["dim"])
    r = lin(h, W[at + "r"]).reshape(T, H, dk)
    k = lin(h, W[at + "k"]).reshape(T, H, dk)
    v = lin(h, W[at + "v"]).reshape(T, H, dv)
    w = torch.exp(-decay_scale * sigmoid(lin(torch.tanh(lin(h, W[at + "w1"])), W[at + "w2"]) + W[at + "w0"].double()))
    w = w.reshape(T, H, dk)
    a = sigmoid(lin(h, W[at + "a"]) + W[at + "a.b"].double()).reshape(T, H, dk)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    S = state["S"]
    out = []
    for t in range(T):
        seen = torch.einsum("hkv,hk->hv", S, u[t])                       # u^T S of the old state
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, r[t]))
    state["S"] = S
    o = unit_rms(torch.stack(out), eps).reshape(T, H * dv) * W[at + "norm"].double() * sigmoid(lin(h, W[at + "g"]))
    return lin(o, W[at + "o"])


def biased_attention(h, W, m, state, at="mix.", v_first: Optional[torch.Tensor] = None, slopes=None):
    """state: {"k": [tokens so far, kv_heads, dim], "v": [.., kv_heads, vdim]} (the cached, mixed values).  Returns
    (output rows, this layer's own values of the piece's tokens before any mixing)."""
    T = h.shape[0]
    H, G = m["heads"], m.get("kv_heads", m["heads"])
    dk, dv = m["dim"], m.get("vdim", m["dim"])
    start = state["k"].shape[0]
    pos = torch.arange(start, start + T, dtype=F64)
    q = lin(h, W[at + "q"]).reshape(T, H, dk)
    k = lin(h, W[at + "k"]).reshape(T, G, dk)
    v_own = lin(h, W[at + "v"]).reshape(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos + 1.0) / qt["every"]) + 1.0))[:, None, None]
    v = v_own
    if v_first is not None:
        lam = W[at + "vmix"].double()
        v = (1.0 - lam) * v_own + lam * v_first
    K = state["k"] = torch.cat([state["k"], k])
    V = state["v"] = torch.cat([state["v"], v])
    keys = torch.arange(K.shape[0], dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H) if slopes is None else slopes[hd]
        s = q[:, hd] @ K[:, g].T * m["scale"] - slope * (pos[:, None] - keys[None, :])
        s = s.masked_fill(keys[None, :] > pos[:, None], float("-inf"))
        out[:, hd] = torch.softmax(s, dim=-1) @ V[:, g]
    y = out.reshape(T, H * dv) * sigmoid(lin(h, W[at + "g"]))
    return lin(y, W[at + "o"]), v_own


def dense_ff(h, W, at="mlp."):
    return lin(gelu_tanh(lin(h, W[at + "gate"])) * lin(h, W[at + "up"]), W[at + "down"])


def expert_ff(h, W, f, at="mlp."):
    """Sigmoid scores, the ``top`` largest chosen, each chosen score multiplying the expert's input."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = sigmoid(lin(h, W[at + "router"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            x = s[t, e] * h[t]
            e_at = f"{at}e{e}."
            out[t] += lin(silu(lin(x, W[e_at + "gate"])) * lin(x, W[e_at + "up"]), W[e_at + "down"])
    return out


def new_state(cfg) -> Dict:
    layers = []
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] == "attention":
            G = m.get("kv_heads", m["heads"])
            layers.append({"k": torch.zeros(0, G, m["dim"], dtype=F64), "v": torch.zeros(0, G, m.get("vdim", m["dim"]), dtype=F64)})
        else:
            layers.append({"S": torch.zeros(m["heads"], m["dim"], m.get("vdim", m["dim"]), dtype=F64)})
    return {"before": None, "pos": 0, "layers": layers}


def forward(cfg, W, tokens: List[int], state, residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of the next piece of one request; ``state`` carries everything between pieces."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, W, cfg, state)
    v_first = None
    have_first = False
    for i, (l, st) in enumerate(zip(cfg["layers"], state["layers"])):
        p = f"l{i}."
        Wl = {k[len(p):]: v for k, v in W.items() if k.startswith(p)}
        h = weight_norm(x, Wl["norm1"], eps)
        if l["type"] == "hgrn2":
            y = gate_write(h, Wl, l["mixer"], st, eps)
        elif l["type"] == "general_delta":
            y = general_delta(h, Wl, l["mixer"], st, eps)
        else:
            mix = bool(l["mixer"].get("v_mix"))
            y, v_own = biased_attention(h, Wl, l["mixer"], st, v_first=v_first if (mix and have_first) else None)
            if mix and not have_first:
                v_first, have_first = v_own, True
        x = x + weight_norm(y, Wl["norm1b"], eps)
        f = l.get("mlp")
        if f:
            h = weight_norm(x, Wl["norm2"], eps)
            y = dense_ff(h, Wl) if f["kind"] == "dense" else expert_ff(h, Wl, f)
            x = x + weight_norm(y, Wl["norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return lin(weight_norm(x, W["final.norm"], eps), W["embed"])
