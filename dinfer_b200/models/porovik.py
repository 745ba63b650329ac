"""Porovik as a list of parts.

The embedding adds to a token's row a row of a second table picked by a hash of (the token before, the token) and a
learned position vector.  Every sublayer has an RMS norm on its input and one on its output, each with a weight stored
around zero (the norm multiplies by ``1 + w``): ``x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))``.  The mixer
is one of: ``hgrn2`` (linear attention whose forget gate also says what is written), ``general_delta`` (the generalized
delta rule with a decay and a removal rate per key channel), ``attention`` (grouped heads without a rotation: a query
temperature that grows with the position, a distance bias per head, values that may be mixed with those of the first
such layer, a sigmoid gate on the heads).  The feed-forward is a dense gated one (tanh gelu), a mixture of gated silu
experts (sigmoid scores, the chosen scores multiply the experts' inputs, not renormalized), or absent.  The head is the
embedding table.  Tensor names: ``embed``, ``bigram``, ``pos``, ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.model_config import PorovikConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(l, cfg: PorovikConfig) -> PartSpec:
    m = l.mixer
    if l.type == "hgrn2":
        return PartSpec("gate_write", {"num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "eps": cfg.norm_eps,
                                       "out_float32": True, "q_proj": "mix.q", "f_proj": "mix.f", "f_bias": "mix.f.b",
                                       "lower": "mix.lower", "v_proj": "mix.v", "norm": "mix.norm", "o_proj": "mix.o"})
    if l.type == "general_delta":
        return PartSpec("general_delta", {
            "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "eps": cfg.norm_eps, "out_float32": True,
            "decay_rank": m.decay_rank, "r_proj": "mix.r", "k_proj": "mix.k", "v_proj": "mix.v", "a_proj": "mix.a",
            "a_bias": "mix.a.b", "decay_proj": ("mix.w1", "mix.w2"), "decay_bias": "mix.w0", "gate_proj": "mix.g",
            "norm": "mix.norm", "o_proj": "mix.o"})
    p = {"num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
         "eps": cfg.norm_eps, "distance_slopes": "geometric", "gate_proj": "mix.g", "out_float32": True,
         "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "o_proj": "mix.o"}
    if m.temp_coef != 0.0:
        p["q_temperature"] = (m.temp_coef, m.temp_every)
    if m.v_mix:
        p["value_mix"] = {"weight": "mix.vmix", "key": "v_mix"}
    return PartSpec("gqa_attention", p)


def porovik_spec(cfg: PorovikConfig) -> ModelSpec:
    def norm(name: str, optional: bool = False) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name, "offset": 1.0,
                                    "optional": optional})

    layers = []
    for i, l in enumerate(cfg.layers):
        f = l.mlp
        if f is None:
            ff = PartSpec("none")
        elif f.kind == "dense":
            ff = PartSpec("gated_mlp", {"intermediate_size": f.ff, "activation": "gelu_tanh", "gate_proj": "mlp.gate",
                                        "up_proj": "mlp.up", "down_proj": "mlp.down", "out_float32": True})
        else:
            ff = PartSpec("moe", {"num_experts": f.experts, "top_k": f.top, "expert_size": f.ff, "activation": "silu",
                                  "gated": True, "scoring": "sigmoid", "renormalize": False, "weight_on": "input",
                                  "router": "mlp.router", "expert_gate": "mlp.e{e}.gate", "expert_up": "mlp.e{e}.up",
                                  "expert_down": "mlp.e{e}.down"})
        none = f is None
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="sandwich_residual", mixer=_mixer(l, cfg), mixer_norm=norm("norm1"), feed_forward=ff,
            feed_forward_norm=norm("norm2", optional=none),
            extras={"mixer_norm_out": norm("norm1b"), "feed_forward_norm_out": norm("norm2b", optional=none)}))
    emb = {"tensor": "embed", "vocab_size": cfg.vocab, "positions": "pos", "max_positions": cfg.max_positions}
    if cfg.bigram is not None:
        emb.update(bigram="bigram", buckets=cfg.bigram.buckets, mul_prev=cfg.bigram.mul_prev, mul_cur=cfg.bigram.mul_cur)
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_tensor="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(cfg.layers))),
        final_norm=norm("final.norm"), lm_head_tensor="head", tie_word_embeddings=True,
        eos_token_ids=cfg.eos_token_ids, embedding=PartSpec("hashed_bigram", emb))


register_architecture("Porovik", PorovikConfig.from_dict, porovik_spec)
