"""Sobivik without a device: the configuration reader and its refusals, the declared tensors, the plain implementation
against itself, and the cache managers' first tokens that stay behind a window."""
import copy
import random

import pytest
import torch

import helpers as H  # noqa: F401  (puts the repository on the path)
import plain_sobivik as P
import sobivik_cases as C
from dinfer_b200.config.model_config import ConfigError, SobivikConfig
from dinfer_b200.config.registry import resolve_architecture


def test_config_round_trip_and_spec():
    for name, d in C.CONFIGS.items():
        arch = resolve_architecture(d)
        cfg = arch.parse_config(d)
        assert isinstance(cfg, SobivikConfig) and cfg.to_dict() == SobivikConfig.from_dict(cfg.to_dict()).to_dict()
        spec = arch.build_spec(cfg)
        spec.check()
        assert spec.embedding_scale == d["embedding"]["scale"] and spec.logit_scale == d["logit_scale"]
        assert len(spec.layers) == len(d["layers"]) and all(l.block == "sandwich_residual" for l in spec.layers)
        kinds = [l.mixer.params["inner"].kind for l in spec.layers]
        want = {"retention": "retention", "latent_attention": "latent_attention", "attention": "differential_attention"}
        assert kinds == [want[l["type"]] for l in d["layers"]]


@pytest.mark.parametrize("path, value", [
    (("canon", "taps"), 0), (("norm", "eps"), 0.0), (("layers", 0, "type"), "mamba"), (("layers", 1, "mixer", "decay"), [0.5]),
    (("layers", 1, "mixer", "decay"), [0.5, 1.5]), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "mask", "size"), 0),
    (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 2, "mixer", "rot", "scaling", "factor"), -1.0),
    (("layers", 0, "mlp", "kind"), "moe"), (("embedding",), None), (("logit_scale",), None), (("layers", 0, "mixer", "diff"), None)])
def test_config_refusals(path, value):
    d = copy.deepcopy(C.SOBIVIK_A)
    at = d
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError):
        SobivikConfig.from_dict(d)


def test_declared_tensors():
    from dinfer_b200.weights.random_init import model_declarations
    decls = {x.name: tuple(x.shape) for x in model_declarations(C.SOBIVIK_C)}
    w = C.SOBIVIK_C["width"]
    assert decls["l0.norm1"] == () and decls["l2.norm1b"] == () and decls["final.norm"] == ()
    assert decls["l0.canon1"] == (w, 1) and decls["l0.dwa"] == (2,) and decls["l3.dwa"] == (5,)
    assert "l2.norm2" not in decls and "l2.mlp.gate" not in decls            # a layer without feed-forward
    assert decls["l1.mix.dkv"] == (18 + 10, w) and decls["l1.mix.uq"] == (5 * 16, 7) and decls["l1.mix.sink"] == (5,)
    assert decls["l1.mix.g"] == (5 * 14, w) and decls["l2.mix.g"] == (3, w) and decls["l3.mix.q"] == (9 * 2 * 6, w)
    assert decls["l3.mix.k"] == (3 * 2 * 6, w) and decls["l3.mix.v"] == (3 * 14, w) and decls["l3.mix.lq2"] == (6,)
    assert decls["l0.mix.g"] == (20, w) and decls["l0.mix.o"] == (w, 20)


def test_plain_mechanisms_in_pieces():
    """Every plain mixer fed in pieces gives what it gives whole; the rotation keeps lengths up to its factor."""
    g = torch.Generator().manual_seed(0)
    cfg = C.SOBIVIK_A
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    W = {d.name: random_tensor(d, 3, 0.2, 0.3, torch.float32).double() for d in model_declarations(cfg)}
    for i, l in enumerate(cfg["layers"]):
        Wl = P.layer_tensors(W, i)
        x = torch.randn(50, cfg["width"], generator=g).double()
        whole = P.MIXERS[l["type"]](x, Wl, l["mixer"], P.new_state(cfg)[i], 1e-5)
        mem, parts, at = P.new_state(cfg)[i], [], 0
        for n in (1, 2, 20, 1, 26):
            parts.append(P.MIXERS[l["type"]](x[at:at + n], Wl, l["mixer"], mem, 1e-5))
            at += n
        assert torch.allclose(torch.cat(parts), whole, atol=1e-10, rtol=1e-10)
    rot = cfg["layers"][2]["mixer"]["rot"]
    cos, sin = P.yarn_angles(rot, torch.arange(40))
    v = torch.randn(40, 3, 8, generator=g).double()
    mult = 0.1 * torch.log(torch.tensor(rot["scaling"]["factor"])).item() + 1.0
    assert torch.allclose(P.rotate_half(v, cos, sin, 8).norm(dim=-1), v.norm(dim=-1) * mult)


@pytest.mark.parametrize("native", [False, True])
def test_first_tokens_stay_behind_the_window(native):
    """A group with a window and kept first tokens gives back the pages the window has passed, except those that
    hold the kept tokens; without kept tokens they go as before."""
    from dinfer_b200.cache.manager import CacheManager, GroupSpec
    if native:
        from dinfer_b200.cache.native import NativeCacheManager as Manager
    else:
        Manager = CacheManager
    m = Manager([GroupSpec(window=6, keep_first=5), GroupSpec(window=6)], 4, [32, 32], 2)
    assert m.allocate("r", 40)
    m.advance("r", 40)
    kept, plain = m.block_table("r", 0), m.block_table("r", 1)
    first_needed = (40 - 6 + 1) // 4
    assert [i for i, b in enumerate(kept) if b < 0] == list(range(2, first_needed))          # tokens 0..4 lie on pages 0 and 1
    assert [i for i, b in enumerate(plain) if b < 0] == list(range(first_needed))
    m.check_invariants()
    m.free("r")
    assert m.num_free_blocks(0) == 32 and m.num_free_blocks(1) == 32
