"""A plain, slow Sobivik in 64-bit on the CPU: one function per mechanism, written from the design's equations.
It shares no code with the package.  A sequence may be fed in pieces: ``new_state`` makes what a sequence keeps
(per layer the last inputs of the short convolution and the mixer's memory), every function takes the position of
the piece's first token from it.

Notation: ``x`` [T, width] is the stream, ``h`` a sublayer's input, ``W[name]`` the tensors of one layer with the
layer's prefix taken off (``mix.q`` and so on), ``p`` the mixer's sizes as ``config.json`` gives them.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gain_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is one number."""
    return unit_rms(x, eps) * g.to(F).reshape(())


def weight_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w.to(F)


def short_conv_input(h: torch.Tensor, w: torch.Tensor, hist: torch.Tensor):
    """h + causal convolution of h per channel; ``w`` [C, taps], ``hist`` [taps - 1, C] the inputs before this
    piece (zeros at a sequence's start).  Returns (result, new history)."""
    taps = w.shape[1]
    full = torch.cat([hist, h], dim=0)                      # row (taps - 1 + t) is h_t
    out = h.clone()
    T = h.shape[0]
    for j in range(taps):
        out += w[:, j].to(F)[None, :] * full[j:j + T]
    return out, full[full.shape[0] - (taps - 1):].clone() if taps > 1 else hist


def retention(h, W, p, mem, eps):
    """Linear attention with a fixed decay a head.  ``mem['S']`` [H, dk, dv]."""
    H, dk, dv = p["heads"], p["dim"], p["vdim"]
    T = h.shape[0]
    q = (h @ W["mix.q"].to(F).T).view(T, H, dk)
    k = (h @ W["mix.k"].to(F).T).view(T, H, dk) * dk ** -0.5
    v = (h @ W["mix.v"].to(F).T).view(T, H, dv)
    decay = torch.tensor(p["decay"], dtype=F)
    S = mem["S"]
    o = torch.empty(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    mem["S"] = S
    o = unit_rms(o, eps).reshape(T, H * dv)
    gate = h @ W["mix.g"].to(F).T
    return (o * gate * torch.sigmoid(gate)) @ W["mix.o"].to(F).T


def yarn_angles(rot: Dict, positions: torch.Tensor):
    """(cos, sin) [T, dims / 2] of a rotation whose frequencies are stretched by the ramp of the scaling section."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        def turn(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(turn(sc["fast"])), 0)
        hi = min(math.ceil(turn(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(sc["factor"]) + 1.0
    a = positions.to(F)[:, None] * f[None, :]
    return a.cos() * mult, a.sin() * mult


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, ..., D]: element i < dims / 2 turns with element i + dims / 2; from ``dims`` on nothing changes."""
    half = dims // 2
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = cos.view(shape), sin.view(shape)
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


def latent_attention(h, W, p, mem, eps):
    """``mem['c']`` [n, kv_rank] latents and ``mem['kr']`` [n, rot_dim] rotated shared key parts of the tokens so far."""
    H, D, P, V, R = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    T = h.shape[0]
    start = mem["c"].shape[0]
    pos = torch.arange(start, start + T)
    cos, sin = yarn_angles(p["rot"], pos)
    cq = weight_norm(h @ W["mix.dq"].to(F).T, W["mix.dq.norm"], eps)
    q = (cq @ W["mix.uq"].to(F).T).view(T, H, D + P)
    q_flat, q_rot = q[..., :D], rotate_half(q[..., D:], cos, sin, p["rot"]["dims"])
    low = h @ W["mix.dkv"].to(F).T
    c = weight_norm(low[:, :R], W["mix.dkv.norm"], eps)
    kr = rotate_half(low[:, R:], cos, sin, p["rot"]["dims"])
    mem["c"], mem["kr"] = torch.cat([mem["c"], c]), torch.cat([mem["kr"], kr])
    n = start + T
    k_flat = (mem["c"] @ W["mix.uk"].to(F).T).view(n, H, D)
    val = (mem["c"] @ W["mix.uv"].to(F).T).view(n, H, V)
    s = (torch.einsum("thd,jhd->htj", q_flat, k_flat) + torch.einsum("thd,jd->htj", q_rot, mem["kr"])) * p["scale"]
    j = torch.arange(n)[None, :]
    seen = (j <= pos[:, None]) & (pos[:, None] - j < p["mask"]["size"])
    s = s.masked_fill(~seen[None], -math.inf)
    sink = W["mix.sink"].to(F)[:, None, None].expand(H, T, 1)
    w = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :n]
    o = torch.einsum("htj,jhv->thv", w, val).reshape(T, H * V)
    return (o * torch.sigmoid(h @ W["mix.g"].to(F).T)) @ W["mix.o"].to(F).T


def differential_attention(h, W, p, mem, eps):
    """Two softmax maps per head over the same values, the second taken off the first.  ``mem['k']`` [n, G, 2, D],
    ``mem['v']`` [n, G, V]."""
    H, G, D, V = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    T = h.shape[0]
    start = mem["k"].shape[0]
    pos = torch.arange(start, start + T)
    q = (h @ W["mix.q"].to(F).T).view(T, H, 2, D)
    mem["k"] = torch.cat([mem["k"], (h @ W["mix.k"].to(F).T).view(T, G, 2, D)])
    mem["v"] = torch.cat([mem["v"], (h @ W["mix.v"].to(F).T).view(T, G, V)])
    n = start + T
    kk = mem["k"].repeat_interleave(H // G, dim=1)           # query head a reads key head a // (H / G)
    vv = mem["v"].repeat_interleave(H // G, dim=1)
    s = torch.einsum("thmd,jhmd->hmtj", q, kk) * p["scale"]
    j = torch.arange(n)[None, :]
    seen = (j <= pos[:, None]) & ((pos[:, None] - j < p["mask"]["size"]) | (j < p["mask"].get("keep_first", 0)))
    w = torch.softmax(s.masked_fill(~seen[None, None], -math.inf), dim=-1)
    a = torch.einsum("hmtj,jhv->mthv", w, vv)
    lam = (torch.exp((W["mix.lq1"].to(F) * W["mix.lk1"].to(F)).sum())
           - torch.exp((W["mix.lq2"].to(F) * W["mix.lk2"].to(F)).sum()) + p["diff"])
    o = unit_rms(a[0] - lam * a[1], eps) * (1.0 - p["diff"])
    o = o * torch.sigmoid(h @ W["mix.g"].to(F).T)[:, :, None]
    return o.reshape(T, H * V) @ W["mix.o"].to(F).T


def gated_ff(h, W):
    g = h @ W["mlp.gate"].to(F).T
    return (g * torch.sigmoid(g) * (h @ W["mlp.up"].to(F).T)) @ W["mlp.down"].to(F).T


MIXERS = {"retention": retention, "latent_attention": latent_attention, "attention": differential_attention}


def new_state(cfg: Dict) -> List[Dict]:
    out = []
    for l in cfg["layers"]:
        p = l["mixer"]
        mem = {"hist": torch.zeros(cfg["canon"]["taps"] - 1, cfg["width"], dtype=F)}
        if l["type"] == "retention":
            mem["S"] = torch.zeros(p["heads"], p["dim"], p["vdim"], dtype=F)
        elif l["type"] == "latent_attention":
            mem["c"], mem["kr"] = torch.zeros(0, p["kv_rank"], dtype=F), torch.zeros(0, p["rot_dim"], dtype=F)
        else:
            mem["k"], mem["v"] = torch.zeros(0, p["kv_heads"], 2, p["dim"], dtype=F), torch.zeros(0, p["kv_heads"], p["vdim"], dtype=F)
        out.append(mem)
    return out


def layer_tensors(tensors: Dict[str, torch.Tensor], i: int) -> Dict[str, torch.Tensor]:
    pre = f"l{i}."
    return {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}


def forward(cfg: Dict, tensors: Dict[str, torch.Tensor], tokens, state: List[Dict], streams: Optional[list] = None):
    """Logits [T, vocab] of a piece of a sequence whose earlier pieces left ``state``.  ``streams``: a list that
    receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = tensors["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    results = [x]                                           # what the embedding gave, then every layer's result
    for i, l in enumerate(cfg["layers"]):
        W = layer_tensors(tensors, i)
        mem = state[i]
        h = gain_norm(x, W["norm1"], eps)
        h, mem["hist"] = short_conv_input(h, W["canon1"], mem["hist"])
        x = x + gain_norm(MIXERS[l["type"]](h, W, l["mixer"], mem, eps), W["norm1b"], eps)
        if l.get("mlp"):
            x = x + gain_norm(gated_ff(gain_norm(x, W["norm2"], eps), W), W["norm2b"], eps)
        results.append(x)
        x = sum(W["dwa"].to(F)[j] * r for j, r in enumerate(results))
        if streams is not None:
            streams.append(x)
    return gain_norm(x, tensors["final.norm"], eps) @ tensors["head"].to(F).T * cfg["logit_scale"]
