"""Ladedra: configuration -> model description.

A pre-norm decoder over a 32-bit stream whose layers are listed one by one.  Every sublayer's result is weighted by a
learned scale per feature and by a sigmoid gate that reads the sublayer's input (``gated_pre_norm`` block with
``scaled_sigmoid_gate``).  Two mixers: ``latent_attention`` (causal; keys and values from one latent vector per token, a
rotated key part shared by all heads, pair rotation with stretched frequencies, an output gate), and ``parallel_mixers``
of ``normed_attention`` (biases, rotate-half rotation, unit-norm queries and keys, capped scores, a sliding window with
averaged blocks in front of it, a learned sink per head) beside ``lightning`` in its retention form (rotated queries and
keys, scaled keys, a norm per head, a SiLU gate).  The feed-forward is ``plain_mlp`` (squared ReLU), ``routed_experts``
(softmax over all experts, groups of experts, gated SiLU experts, a shared expert) or absent.  The embedding is scaled;
the head is a matrix of its own.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1/2``,
``l<i>.ls1/2``, ``l<i>.rg1/2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..parts.parallel_mixers import ParallelMixers
from .ladedra_config import (LadedraConfig, LadedraDense, LadedraExperts, LadedraLatentAttention, LadedraParallel)

STREAM = "float32"       # the residual sum is 32-bit in every run dtype


def _position(kind: str, rotation, head_dim: int):
    if rotation is None or not rotation.dims:
        return {}
    return {"position": PartSpec.make(kind, {"head_dim": head_dim, "dims": rotation.dims, "base": rotation.base,
                                             "scaling": rotation.scaling})}


def _latent(cfg: LadedraConfig, m: LadedraLatentAttention, mix: str) -> PartSpec:
    return PartSpec.make(
        "latent_attention",
        {"hidden_size": cfg.width, "num_heads": m.heads, "key_dim": m.dim, "rot_width": m.rot_dim, "value_dim": m.vdim,
         "rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "mask": (("kind", "causal"),), "gate": True,
         "stream": STREAM},
        {"q": mix + "q", "down": mix + "dkv", "down_norm": mix + "dkv.norm", "up_k": mix + "uk", "up_v": mix + "uv",
         "g": mix + "g", "o": mix + "o"},
        _position("rotary_pairs", m.rotation, m.rot_dim))


def _parallel(cfg: LadedraConfig, m: LadedraParallel, mix: str) -> PartSpec:
    left, right, a, b = m.left, m.right, mix + "left.", mix + "right."
    children = {
        "left": PartSpec.make(
            "normed_attention",
            {"hidden_size": cfg.width, "num_heads": left.heads, "num_kv_heads": left.kv_heads, "key_dim": left.dim,
             "value_dim": left.vdim, "scale": left.scale, "qk_norm_eps": cfg.norm_eps, "softcap": left.softcap,
             "mask": (("kind", "window_pooled"), ("pool", left.pool), ("size", left.window)), "sink": True, "bias": True,
             "stream": STREAM},
            {"q": a + "q", "k": a + "k", "v": a + "v", "o": a + "o", "q_bias": a + "q.b", "k_bias": a + "k.b",
             "v_bias": a + "v.b", "sink": a + "sink"},
            _position("rotary_blend", left.rotation, left.dim)),
        "right": PartSpec.make(
            "lightning",
            {"hidden_size": cfg.width, "num_heads": right.heads, "key_dim": right.dim, "value_dim": right.vdim,
             "decay": right.decay, "eps": cfg.norm_eps, "activation": "none", "key_scale": right.dim ** -0.5,
             "norm": "per_head", "gate": "silu", "stream": STREAM},
            {"q": b + "q", "k": b + "k", "v": b + "v", "g": b + "g", "o": b + "o"},
            _position("rotary_blend", right.rotation, right.dim)),
    }
    return PartSpec.make("parallel_mixers", {"hidden_size": cfg.width, "left_scale": m.left_scale, "right_scale": m.right_scale},
                         ParallelMixers.lifted_weights(children), children)


def _feed_forward(cfg: LadedraConfig, mlp, prefix: str):
    if isinstance(mlp, LadedraDense):
        return PartSpec.make("plain_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                           "activation": "squared_relu", "stream": STREAM},
                             {"up": prefix + "up", "down": prefix + "down"})
    assert isinstance(mlp, LadedraExperts)
    weights = {"router": prefix + "router"}
    for e in range(mlp.experts):
        weights.update({f"gate.{e}": f"{prefix}e{e}.gate", f"up.{e}": f"{prefix}e{e}.up", f"down.{e}": f"{prefix}e{e}.down"})
    if mlp.shared_ff:
        weights.update({"shared_gate": prefix + "shared.gate", "shared_up": prefix + "shared.up",
                        "shared_down": prefix + "shared.down"})
    return PartSpec.make(
        "routed_experts",
        {"hidden_size": cfg.width, "num_experts": mlp.experts, "top_k": mlp.top, "expert_size": mlp.ff,
         "shared_size": mlp.shared_ff, "scoring": "softmax_all", "groups": mlp.groups, "keep_groups": mlp.keep,
         "weight_scale": mlp.scale, "expert_form": "gated_silu", "stream": STREAM},
        weights)


def ladedra_spec(cfg: LadedraConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec.make("grouped_rms_norm", {"size": cfg.width, "groups": 1, "eps": cfg.norm_eps}, {"weight": name})

    layers = []
    for index, layer in enumerate(cfg.layers):
        prefix = f"l{index}."
        if isinstance(layer.mixer, LadedraLatentAttention):
            mixer = _latent(cfg, layer.mixer, prefix + "mix.")
        else:
            mixer = _parallel(cfg, layer.mixer, prefix + "mix.")
        norms = {"input": norm(prefix + "norm1")}
        gates = {"mixer_scale": prefix + "ls1", "mixer_gate": prefix + "rg1", "mixer_gate_bias": prefix + "rg1.b"}
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = _feed_forward(cfg, layer.mlp, prefix + "mlp.")
            norms["post_mixer"] = norm(prefix + "norm2")
            gates.update({"feed_forward_scale": prefix + "ls2", "feed_forward_gate": prefix + "rg2",
                          "feed_forward_gate_bias": prefix + "rg2.b"})
        residual_gates = PartSpec.make("scaled_sigmoid_gate", {"hidden_size": cfg.width,
                                                               "feed_forward": layer.mlp is not None}, gates)
        layers.append(LayerSpec.make("gated_pre_norm", mixer, feed_forward, norms, residual_gates=residual_gates))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": cfg.width}
    return ModelSpec(
        architecture=LadedraConfig.ARCHITECTURE,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=1 << 30,           # the design sets no limit; positions are 32-bit
        embedding=PartSpec.make("token_embedding", dict(sizes, stream=STREAM, scale=cfg.embedding_scale), {"table": "embed"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(index) for index in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec.make("lm_head", sizes, {"weight": "head"}),
    )


def ladedra_ignorable_tensors(cfg: LadedraConfig):
    """Tensors a checkpoint may hold that this model does not read: what belongs to the feed-forward of a layer
    without one."""
    names = []
    for index, layer in enumerate(cfg.layers):
        if layer.mlp is None:
            names += [f"l{index}.norm2", f"l{index}.ls2", f"l{index}.rg2", f"l{index}.rg2.b"]
    return names


def ladedra_kernel_libraries(cfg: LadedraConfig, dtype: str):
    """The kernel files a Ladedra model of this run dtype calls: a first call compiles these and no others."""
    shared = ["elementwise", "norm", "pointwise", "gated_residual", "sampling"]
    kinds = {type(layer.mixer) for layer in cfg.layers}
    if LadedraLatentAttention in kinds:
        shared += ["latent_rope_cache", "attention_masked"]
    if LadedraParallel in kinds:
        shared += ["rope_norm_cache", "attention_masked", "lightning"]
    if any(isinstance(layer.mlp, LadedraExperts) for layer in cfg.layers):
        shared.append("experts")
    if dtype != "float32":
        import torch

        from .. import kernels

        if any(isinstance(layer.mixer, LadedraParallel)
               and kernels.attention_prompt_mma_supported(torch.bfloat16, layer.mixer.left.dim, layer.mixer.left.vdim)
               for layer in cfg.layers):
            shared.append("attention_prompt_mma")     # (head sizes the tensor-core attention takes)
        if any(isinstance(layer.mixer, LadedraLatentAttention)
               and kernels.attention_latent_mma_supported(torch.bfloat16, layer.mixer.kv_rank + layer.mixer.rot_dim,
                                                          layer.mixer.kv_rank) for layer in cfg.layers):
            shared.append("attention_latent_mma")     # (latent sizes the tensor-core attention takes)
    shared = list(dict.fromkeys(shared))
    return shared + (["gemm_f32"] if dtype == "float32" else ["decode_linear", "skinny_tcgen05"])


register_architecture(Architecture(
    name=LadedraConfig.ARCHITECTURE,
    read_config=LadedraConfig.from_dict,
    build_spec=ladedra_spec,
    ignorable_tensors=ladedra_ignorable_tensors,
    kernel_libraries=ladedra_kernel_libraries,
))
