"""Tiny Porovik configurations for the tests.  They differ from one another in every size and option and use values
that are easy to confuse when they happen to be equal or 1: key size against value size, heads against key heads, one
head, one expert chosen and several, a layer without feed-forward, a model without any attention layer, attention as
the first layer, a query temperature that changes at every position and none at all, mixed values in two, one or no
layer, hash multipliers whose products pass 2^31, sizes no vector load or tensor-core tile divides, and sizes the
tensor-core attention takes."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def hgrn2(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def general_delta(heads, dim, rank, vdim=None):
    m = {"heads": heads, "dim": dim, "decay_rank": rank}
    if vdim:
        m["vdim"] = vdim
    return {"type": "general_delta", "mixer": m}


def attention(heads, kv_heads, dim, vdim, scale=None, temp=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
         "v_mix": v_mix}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def model(vocab, width, eps, max_positions, bigram, layers):
    d = {"architecture": "Porovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_positions": max_positions,
         "layers": layers}
    if bigram:
        d["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    return d


# attention first; two layers that mix values and one that does not; two of four experts; a key size of 12
POROVIK_A = model(300, 64, 1e-5, 400, (101, 7, 13), [
    layer(attention(4, 2, 8, 16, scale=0.6, temp=(0.7, 5), v_mix=True), dense(48)),
    layer(hgrn2(2, 16, 24), moe(4, 2, 24)),
    layer(general_delta(3, 12, 6), dense(40)),
    layer(attention(6, 2, 12, 16, scale=0.4, temp=(0.3, 1), v_mix=True), None),
    layer(attention(2, 1, 16, 8, scale=0.5), moe(3, 1, 16))])
# heads the tensor-core attention takes (keys as wide as values); one key head; a state of 128 key channels; one of
# three experts; multipliers whose products pass 2^31
POROVIK_B = model(515, 128, 3e-6, 512, (257, 1000003, 65537), [
    layer(general_delta(2, 64, 8, vdim=40), moe(3, 1, 32)),
    layer(attention(4, 1, 64, 64, scale=0.2, temp=(0.5, 16), v_mix=True), dense(96)),
    layer(hgrn2(3, 128, 40), dense(72)),
    layer(attention(2, 2, 32, 32, scale=0.3), None)])
# sizes nothing divides; one head; no temperature, no mixed values; every expert chosen
POROVIK_C = model(331, 72, 1e-6, 300, (50, 3, 0), [
    layer(hgrn2(1, 12, 20), dense(28)),
    layer(general_delta(5, 33, 3, vdim=7), moe(2, 2, 20)),
    layer(attention(3, 3, 10, 6, scale=1.1), None),
    layer(hgrn2(5, 6, 10), moe(5, 3, 12))])
# no attention layer at all (the engine then has no paged cache) and no bigram table
POROVIK_D = model(257, 100, 2e-6, 260, None, [
    layer(general_delta(5, 20, 4), dense(36)),
    layer(hgrn2(2, 40, 36), None),
    layer(general_delta(1, 16, 1, vdim=48), moe(6, 2, 20))])
# sizes of real layers in small: heads of 128 and 64, a delta rule of 128 key channels, eight and six experts
POROVIK_E = model(400, 384, 5e-6, 640, (997, 29, 19), [
    layer(hgrn2(3, 64, 128), dense(448)),
    layer(attention(4, 2, 128, 128, scale=0.09, temp=(0.6, 48), v_mix=True), moe(8, 2, 64)),
    layer(general_delta(2, 128, 16), dense(256)),
    layer(attention(8, 2, 64, 128, scale=0.12, v_mix=True), moe(6, 1, 48))])
CONFIGS = {"A": POROVIK_A, "B": POROVIK_B, "C": POROVIK_C, "D": POROVIK_D, "E": POROVIK_E}


def write_model(path: str, cfg: dict, seed: int, dtype: torch.dtype, sharp: float = 4.0, std: float = 0.08) -> str:
    """Random weights shaped so that faults show: attention queries scaled by ``sharp`` (a token's attention then
    rests on few keys, often old ones, against the distance bias: a key lost or one too many moves the logits); forget
    gates and decays pushed towards one in half of the channels, so that the states remember far tokens; the lower
    bounds spread over (0, 1); removal rates, gates and the value mix large enough to matter; norm weights spread
    around zero; the routers sharp enough that the chosen scores differ."""
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    from dinfer_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = []
    for d in model_declarations(cfg):
        t = random_tensor(d, seed, std, 0.3, torch.float32)
        n = d.name
        kind = cfg["layers"][int(n[1:n.index(".")])]["type"] if n.startswith("l") and "." in n and n[1:n.index(".")].isdigit() else ""
        if n.endswith("mix.q") and kind == "attention":
            t = t * sharp
        elif n.endswith("mix.lower"):
            t = torch.sigmoid(t * 25.0) * 0.9 + 0.05
        elif n.endswith("mix.f.b"):
            t = t * 20.0 + torch.where(torch.arange(t.numel()) % 2 == 0, 3.0, 0.0)
        elif n.endswith("mix.w0"):
            t = t * 20.0 - torch.where(torch.arange(t.numel()) % 2 == 0, 4.0, 0.0)
        elif n.endswith(("mix.w2", "mix.a.b")):
            t = t * 10.0
        elif n.endswith("mix.vmix"):
            t = torch.tensor(0.35)
        elif n.endswith(("norm1", "norm2", "norm1b", "norm2b", "final.norm")):
            t = t * 3.0
        elif n.endswith("mlp.router"):
            t = t * 6.0
        tensors.append((n, t.to(torch.bfloat16).to(dtype)))     # the same values in every dtype
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path


def load_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))
