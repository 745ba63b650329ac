"""Tiny Sobivik configurations for the tests.  They differ from one another in every size and option and use values
that are easy to confuse when they happen to be equal or 1: key size against value size, heads against key heads, a
window shorter than a page and one of a single token, more kept first tokens than the window holds, none kept at all,
a convolution of one tap (no history), a layer without feed-forward, a model without any attention layer, a rotation
with and without stretched frequencies, sizes no vector load or tensor-core tile divides."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def retention(heads, dim, vdim, decay):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=10000.0, scale=None, scaling=None, rot_dims=None):
    rot = {"base": base, "dims": rot_dims or rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": rot, "mask": {"size": window}}}


def differential(heads, kv_heads, dim, vdim, window, keep_first, diff, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
                      "scale": scale if scale is not None else dim ** -0.5,
                      "mask": {"size": window, "keep_first": keep_first}}}


def layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


def model(vocab, width, eps, emb, logit, taps, layers):
    return {"architecture": "Sobivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb},
            "logit_scale": logit, "canon": {"taps": taps}, "layers": layers}


# an attention layer first; fewer key heads than query heads; a stretched rotation; a layer without feed-forward
SOBIVIK_A = model(300, 64, 1e-5, 3.0, 0.5, 4, [
    layer(differential(4, 2, 8, 16, 9, 3, 0.3, scale=0.6), 48),
    layer(retention(2, 16, 24, (0.9, 0.995)), 40),
    layer(latent(3, 8, 8, 12, 24, 20, 20, base=500.0, scale=0.5, scaling=(4.0, 64, 8.0, 2.0)), None),
    layer(retention(4, 8, 8, (0.5, 0.97, 0.999, 1.0)), 24)])
# a window shorter than a page; one key head for six query heads; no kept tokens; a state of 128 key channels; a
# latent the tensor-core kernel takes; a convolution of two taps
SOBIVIK_B = model(515, 128, 3e-6, 1.0, 2.5, 2, [
    layer(latent(4, 16, 16, 40, 32, 48, 50, base=1e6, scale=0.2), 96),
    layer(differential(6, 1, 24, 40, 7, 0, 0.8, scale=0.3), 64),
    layer(retention(3, 128, 40, (0.98, 0.9995, 0.93)), 72)])
# sizes nothing divides; a convolution of one tap; a window of one token with more kept tokens than that; a rotation
# over part of the rotated elements
SOBIVIK_C = model(331, 72, 1e-6, 0.7, 1.0, 1, [
    layer(retention(1, 12, 20, (0.99,)), 28),
    layer(latent(5, 6, 10, 14, 18, 7, 33, base=100.0, scaling=(2.5, 40, 16.0, 1.0), rot_dims=6), 20),
    layer(differential(3, 3, 10, 6, 1, 5, 0.1), None),
    layer(differential(9, 3, 6, 14, 40, 17, 0.5), 36)])
# no attention layer at all (the engine then has no paged cache), a width of 100, five taps
SOBIVIK_D = model(257, 100, 2e-6, 8.0, 0.25, 5, [
    layer(retention(5, 12, 12, (0.9, 0.95, 0.99, 0.999, 0.9999)), 36),
    layer(retention(2, 40, 36, (0.999, 0.8)), None)])
# sizes of real layers in small: heads of 64 and 128, a latent of 128, six taps
SOBIVIK_E = model(400, 384, 5e-6, 12.0, 1.5, 6, [
    layer(retention(3, 64, 128, (0.97, 0.99, 0.9995)), 448),
    layer(differential(4, 2, 64, 128, 64, 4, 0.25), 256),
    layer(latent(8, 64, 64, 64, 128, 96, 100, base=5000.0, scaling=(2.0, 128, 32.0, 1.0)), 128)])
CONFIGS = {"A": SOBIVIK_A, "B": SOBIVIK_B, "C": SOBIVIK_C, "D": SOBIVIK_D, "E": SOBIVIK_E}


def write_model(path: str, cfg: dict, seed: int, dtype: torch.dtype, sharp: float = 4.0, std: float = 0.08) -> str:
    """Random weights shaped so that faults show: attention queries scaled by ``sharp`` (a token's attention then
    rests on few keys, often old or kept ones: a key lost or one too many moves the logits); convolution taps large
    enough that every tap matters; sinks and the lambda vectors large enough to matter; the weights of the average over
    the layers' results spread between -1 and 1."""
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    from dinfer_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    tensors = []
    for d in model_declarations(cfg):
        t = random_tensor(d, seed, std, 0.3, torch.float32)
        if d.name.endswith(("mix.q", "mix.uq")):
            t = t * sharp
        elif d.name.endswith("canon1"):
            t = t * 6.0
        elif d.name.endswith("mix.sink"):
            t = t * 20.0
        elif d.name.endswith(("lq1", "lk1", "lq2", "lk2")):
            t = t * 8.0
        elif d.name.endswith(".dwa"):
            t = (t - 1.0) * 3.0 + 0.5
        tensors.append((d.name, t.to(torch.bfloat16).to(dtype)))     # the same values in every dtype
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path


def load_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return load_file(os.path.join(model_dir, "model.safetensors"))
