"""Porovik without a device: the configuration reader and its refusals, the declared tensors, and the plain
implementation against itself (pieces against whole, each mechanism against a second way of writing it)."""
import copy
import math
import random

import pytest
import torch

import helpers as H  # noqa: F401  (puts the repository on the path)
import plain_porovik as P
import porovik_cases as C
from dinfer_b200.config.model_config import ConfigError, PorovikConfig
from dinfer_b200.config.registry import resolve_architecture


def test_config_round_trip_and_spec():
    for name, d in C.CONFIGS.items():
        arch = resolve_architecture(d)
        cfg = arch.parse_config(d)
        assert isinstance(cfg, PorovikConfig) and cfg.to_dict() == PorovikConfig.from_dict(cfg.to_dict()).to_dict()
        spec = arch.build_spec(cfg)
        spec.check()
        assert spec.tie_word_embeddings and spec.embedding.kind == "hashed_bigram"
        assert len(spec.layers) == len(d["layers"]) and all(l.block == "sandwich_residual" for l in spec.layers)
        want = {"hgrn2": "gate_write", "general_delta": "general_delta", "attention": "gqa_attention"}
        assert [l.mixer.kind for l in spec.layers] == [want[l["type"]] for l in d["layers"]]
        ff = {None: "none", "dense": "gated_mlp", "moe": "moe"}
        assert [l.feed_forward.kind for l in spec.layers] == [ff[(l["mlp"] or {}).get("kind")] for l in d["layers"]]


def test_config_defaults():
    """Keys a mixer may leave out: key heads (as many as heads), the values' width (the keys'), the temperature."""
    d = copy.deepcopy(C.POROVIK_C)
    m = d["layers"][2]["mixer"]
    del m["kv_heads"], m["vdim"], m["v_mix"]
    a = PorovikConfig.from_dict(d).layers[2].mixer
    assert (a.kv_heads, a.vdim, a.v_mix, a.temp_coef) == (3, 10, False, 0.0)
    assert PorovikConfig.from_dict(C.POROVIK_D).bigram is None


@pytest.mark.parametrize("path, value", [
    (("norm", "eps"), 0.0), (("layers", 0, "type"), "mamba"), (("layers", 0, "mixer", "kv_heads"), 3),
    (("layers", 0, "mixer", "heads"), 0), (("layers", 0, "mixer", "scale"), None), (("layers", 0, "mixer", "q_temp", "every"), 0),
    (("layers", 1, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "kind"), "sparse"), (("layers", 2, "mixer", "dim"), -4),
    (("layers", 2, "mixer", "decay_rank"), 0), (("layers", 3, "mixer", "vdim"), 8), (("max_positions",), None),
    (("embedding", "bigram", "buckets"), 0), (("vocab",), None), (("layers",), [])])
def test_config_refusals(path, value):
    d = copy.deepcopy(C.POROVIK_A)
    at = d
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError):
        PorovikConfig.from_dict(d)


def test_declared_tensors():
    from dinfer_b200.weights.random_init import model_declarations
    decls = {x.name: tuple(x.shape) for x in model_declarations(C.POROVIK_A)}
    w = C.POROVIK_A["width"]
    assert decls["embed"] == (300, w) and decls["bigram"] == (102, w) and decls["pos"] == (400, w) and "head" not in decls
    assert decls["l0.norm1"] == (w,) and decls["l3.norm1b"] == (w,) and decls["final.norm"] == (w,)
    assert "l3.norm2" not in decls and "l3.mlp.gate" not in decls            # a layer without feed-forward
    assert decls["l0.mix.q"] == (32, w) and decls["l0.mix.k"] == (16, w) and decls["l0.mix.v"] == (32, w)
    assert decls["l0.mix.g"] == (64, w) and decls["l0.mix.o"] == (w, 64) and decls["l0.mix.vmix"] == ()
    assert decls["l3.mix.vmix"] == () and "l4.mix.vmix" not in decls
    assert decls["l1.mix.f"] == (32, w) and decls["l1.mix.f.b"] == (32,) and decls["l1.mix.lower"] == (32,)
    assert decls["l1.mix.norm"] == (24,) and decls["l1.mix.o"] == (w, 48)
    assert decls["l1.mlp.router"] == (4, w) and decls["l1.mlp.e3.gate"] == (24, w) and decls["l1.mlp.e0.down"] == (w, 24)
    assert decls["l2.mix.w1"] == (6, w) and decls["l2.mix.w2"] == (36, 6) and decls["l2.mix.w0"] == (36,)
    assert decls["l2.mix.a.b"] == (36,) and decls["l2.mix.norm"] == (36,) and decls["l2.mix.r"] == (36, w)
    no_bigram = {x.name for x in model_declarations(C.POROVIK_D)}
    assert "bigram" not in no_bigram and "pos" in no_bigram
    # a file decides the thin middle of the decay's projection where the configuration does not name it
    d = copy.deepcopy(C.POROVIK_D)
    del d["layers"][0]["mixer"]["decay_rank"]
    arch = resolve_architecture(d)
    from dinfer_b200.models.decoder import DecoderModel
    from dinfer_b200.parts.base import BuildEnv
    spec = arch.build_spec(arch.parse_config(d))
    shapes = {x.name: tuple(x.shape) for x in DecoderModel(spec, BuildEnv(torch.device("cpu"), torch.float32, 100, 260)).declarations()}
    assert shapes["l0.mix.w1"] == (-1, 100) and shapes["l0.mix.w2"] == (100, -1)


def _weights(cfg, seed=3):
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    return {d.name: random_tensor(d, seed, 0.2, 0.3, torch.float32).double() for d in model_declarations(cfg)}


def test_plain_in_pieces_is_plain_whole():
    for name in ("A", "C", "D"):
        cfg = C.CONFIGS[name]
        W = _weights(cfg)
        ids = H.random_tokens(random.Random(1), 60, cfg["vocab"])
        whole = P.forward(cfg, W, ids, P.new_state(cfg))
        state, parts, at = P.new_state(cfg), [], 0
        for n in (1, 2, 30, 1, 26):
            parts.append(P.forward(cfg, W, ids[at:at + n], state))
            at += n
        assert torch.allclose(torch.cat(parts), whole, atol=1e-9, rtol=1e-9)


def test_plain_recurrences_against_sums():
    """The gate-write recurrence unrolled: o_t = sum_s (prod_(s<r<=t) f_r) (1 - f_s) (q_t . ) v_s per channel; the
    general delta rule with a removal rate of zero is the same sum with k in place of 1 - f."""
    g = torch.Generator().manual_seed(0)
    T, dk, dv = 9, 5, 3
    f = torch.rand(T, dk, generator=g).double()
    q, v = torch.randn(T, dk, generator=g).double(), torch.randn(T, dv, generator=g).double()
    S = torch.zeros(dk, dv).double()
    for t in range(T):
        S = f[t][:, None] * S + (1 - f[t])[:, None] * v[t][None, :]
        want = torch.zeros(dv).double()
        for s in range(t + 1):
            keep = torch.ones(dk).double()
            for r in range(s + 1, t + 1):
                keep = keep * f[r]
            want += ((q[t] * keep * (1 - f[s])).sum()) * v[s]
        assert torch.allclose(S.T @ q[t], want, atol=1e-12)
    # the hash of the embedding: big multipliers stay exact in Python integers
    bg = C.POROVIK_B["embedding"]["bigram"]
    assert (514 * bg["mul_prev"] + 514 * bg["mul_cur"]) > 2 ** 28
    # slopes of the distance bias: a geometric row that ends at 2^-8
    H_ = 6
    assert math.isclose(2.0 ** (-8.0 * H_ / H_), 1 / 256)
