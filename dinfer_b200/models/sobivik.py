"""Sobivik as a list of parts.

Every sublayer has a norm on its input and one on its output, each an RMS norm whose weight is one number:
``x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))``.  What a mixer reads first goes through a short causal
convolution per channel that is added to it (``canon1``, history in the request's state).  The mixer is retention (a
linear-attention recurrence with a fixed decay per head), latent attention over a sliding window (a learned sink per
head in the softmax, a sigmoid output gate, a rotation in halves whose frequencies may be stretched by a ramp), or
differential attention (two softmax maps per head over the same values, a window behind which the first tokens stay
visible, one gate per head).  The feed-forward is a dense gated one (silu) or absent.  What leaves layer i is a weighted
sum of the embedding's output and the results of all layers up to i (``dwa``).  The embedding's rows and the logits
each carry a fixed factor.  Tensor names: ``embed``, ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.canon1``, ``l<i>.dwa``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.model_config import SobivikConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(l, cfg: SobivikConfig) -> PartSpec:
    m = l.mixer
    if l.type == "retention":
        return PartSpec("retention", {"num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": m.decay,
                                      "eps": cfg.norm_eps, "out_float32": True, "q_proj": "mix.q", "k_proj": "mix.k",
                                      "v_proj": "mix.v", "gate_proj": "mix.g", "o_proj": "mix.o"})
    if l.type == "latent_attention":
        a = m.latent
        rope = {"head_dim": a.rot_dim, "rotary_dim": a.rot_dims, "theta": a.rot_base,
                "max_positions": cfg.max_positions, "style": "neox"}
        if m.scaling:
            rope["ramp"] = m.scaling.to_dict()
        return PartSpec("latent_attention", {
            "num_heads": a.heads, "nope_dim": a.dim, "rope_dim": a.rot_dim, "v_dim": a.vdim, "kv_rank": a.kv_rank,
            "q_rank": a.q_rank, "scale": a.scale, "eps": cfg.norm_eps, "position": PartSpec("rope", rope),
            "window": m.window, "sink": "mix.sink", "gate_proj": "mix.g", "out_float32": True,
            "q_down": "mix.dq", "q_norm": "mix.dq.norm", "q_up": "mix.uq", "kv_down": "mix.dkv",
            "kv_norm": "mix.dkv.norm", "k_up": "mix.uk", "v_up": "mix.uv", "o_proj": "mix.o"})
    return PartSpec("differential_attention", {
        "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
        "diff": m.diff, "eps": cfg.norm_eps, "window": m.window, "keep_first": m.keep_first, "out_float32": True,
        "q_proj": "mix.q", "k_proj": "mix.k", "v_proj": "mix.v", "gate_proj": "mix.g", "o_proj": "mix.o",
        "lambda_q1": "mix.lq1", "lambda_k1": "mix.lk1", "lambda_q2": "mix.lq2", "lambda_k2": "mix.lk2"})


def sobivik_spec(cfg: SobivikConfig) -> ModelSpec:
    def gain(name: str, optional: bool = False) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name, "scalar": True,
                                    "optional": optional})

    layers = []
    for i, l in enumerate(cfg.layers):
        mixer = PartSpec("short_conv_input", {"inner": _mixer(l, cfg), "taps": cfg.conv_taps, "weight": "canon1"})
        none = l.mlp is None
        ff = PartSpec("none") if none else PartSpec("gated_mlp", {
            "intermediate_size": l.mlp.ff, "activation": "silu", "gate_proj": "mlp.gate", "up_proj": "mlp.up",
            "down_proj": "mlp.down", "out_float32": True})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="sandwich_residual", mixer=mixer, mixer_norm=gain("norm1"), feed_forward=ff,
            feed_forward_norm=gain("norm2", optional=none),
            extras={"mixer_norm_out": gain("norm1b"), "feed_forward_norm_out": gain("norm2b", optional=none),
                    "depth_average": "dwa", "depth_index": i, "depth_layers": len(cfg.layers)}))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding_tensor="embed", layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(cfg.layers))),
        final_norm=gain("final.norm"), lm_head_tensor="head", tie_word_embeddings=False,
        eos_token_ids=cfg.eos_token_ids, embedding_scale=cfg.embedding_scale, logit_scale=cfg.logit_scale)


register_architecture("Sobivik", SobivikConfig.from_dict, sobivik_spec)
