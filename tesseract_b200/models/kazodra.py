"""Kazodra: configuration -> model description.

A decoder whose layers are listed one by one.  Every sublayer is normed on both sides (``sandwich`` block over layer
norms with weight and bias): ``x += post(sub(pre(x)))`` for the mixer and then for the gated SiLU feed-forward
(``gated_mlp``), if the layer has one.  Behind its sublayers a layer adds a term for the token itself
(``gated_token_slice``: the layer's slice of a second embedding table, gated by a projection of the stream).  Three
mixers: ``latent_attention`` (keys and values from one latent vector per token, a rotated key part shared by all heads,
sliding window), ``lightning`` (linear attention with a fixed decay per head, a state per request) and
``differential_attention`` (two score maps per head over the same values, subtracted, normed per head, gated).  A run
of layers may be walked several times with the same weights and a cache or state of its own per walk; every walk starts
with ``stream_bias``, which adds the walk's own vector to the stream.  The logits come from the embedding table; the
residual stream is 32-bit in every run dtype.  Tensor names: ``embed``, ``side.embed``, ``loop.step``, ``final.norm[.b]``
and per layer ``l<i>.norm{1,1b,2,2b}[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``l<i>.side.{gate,proj,norm}``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .kazodra_config import KazodraAttention, KazodraConfig, KazodraLatentAttention, KazodraLightning

STREAM = "float32"       # the residual sum is 32-bit in every run dtype


def _mask(window):
    return (("kind", "window"), ("size", window)) if window else (("kind", "causal"),)


def _position(rotation, head_dim: int):
    if rotation is None or not rotation.dims:
        return {}
    return {"position": PartSpec.make("rotary_pairs", {"head_dim": head_dim, "dims": rotation.dims, "base": rotation.base,
                                                       "scaling": rotation.scaling})}


def _mixer(cfg: KazodraConfig, index: int) -> PartSpec:
    m, mix = cfg.layers[index].mixer, f"l{index}.mix."
    if isinstance(m, KazodraLatentAttention):
        return PartSpec.make(
            "latent_attention",
            {"hidden_size": cfg.width, "num_heads": m.heads, "key_dim": m.dim, "rot_width": m.rot_dim, "value_dim": m.vdim,
             "rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "mask": _mask(m.window), "stream": STREAM},
            {"q": mix + "q", "down": mix + "dkv", "down_norm": mix + "dkv.norm", "up_k": mix + "uk", "up_v": mix + "uv",
             "o": mix + "o"},
            _position(m.rotation, m.rot_dim))
    if isinstance(m, KazodraLightning):
        return PartSpec.make(
            "lightning",
            {"hidden_size": cfg.width, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": m.decay,
             "eps": cfg.norm_eps, "stream": STREAM},
            {"q": mix + "q", "k": mix + "k", "v": mix + "v", "g": mix + "g", "o": mix + "o", "norm": mix + "norm"})
    assert isinstance(m, KazodraAttention)
    return PartSpec.make(
        "differential_attention",
        {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
         "scale": m.scale, "lambda_offset": m.diff, "post_scale": 1.0 - m.diff, "eps": cfg.norm_eps,
         "mask": _mask(m.window), "gate": True, "stream": STREAM},
        {"q": mix + "q", "k": mix + "k", "v": mix + "v", "g": mix + "g", "o": mix + "o", "lq1": mix + "lq1",
         "lk1": mix + "lk1", "lq2": mix + "lq2", "lk2": mix + "lk2"},
        _position(m.rotation, m.dim))


def kazodra_spec(cfg: KazodraConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec.make("layer_norm", {"size": cfg.width, "eps": cfg.norm_eps}, {"weight": name, "bias": name + ".b"})

    layers = []
    for index, layer in enumerate(cfg.layers):
        prefix = f"l{index}."
        norms = {"pre_mixer": norm(prefix + "norm1"), "post_mixer": norm(prefix + "norm1b")}
        feed_forward = None
        if layer.ff is not None:
            feed_forward = PartSpec.make(
                "gated_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.ff, "activation": "silu", "bias": False,
                              "stream": STREAM},
                {"gate": prefix + "mlp.gate", "up": prefix + "mlp.up", "down": prefix + "mlp.down"})
            norms.update({"pre_feed_forward": norm(prefix + "norm2"), "post_feed_forward": norm(prefix + "norm2b")})
        token_input = None
        if cfg.side_dim is not None:
            token_input = PartSpec.make(
                "gated_token_slice",
                {"hidden_size": cfg.width, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "slices": len(cfg.layers),
                 "slice": index, "activation": "gelu_tanh", "eps": cfg.norm_eps},
                {"table": "side.embed", "gate": prefix + "side.gate", "proj": prefix + "side.proj",
                 "norm": prefix + "side.norm"})
        layers.append(LayerSpec.make("sandwich", _mixer(cfg, index), feed_forward, norms, token_input))
    injections = ()
    if cfg.loops:
        # one vector per walk, all rows of one tensor
        injections = tuple(PartSpec.make("stream_bias", {"hidden_size": cfg.width, "rows": cfg.loop.times, "row": walk},
                                         {"table": "loop.step"}) for walk in range(cfg.loop.times))
    sizes = {"vocab_size": cfg.vocab, "hidden_size": cfg.width}
    return ModelSpec(
        architecture=KazodraConfig.ARCHITECTURE,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=1 << 30,           # the design sets no limit; positions are 32-bit
        embedding=PartSpec.make("token_embedding", dict(sizes, stream=STREAM), {"table": "embed"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer, inject=walk) for layer, walk in cfg.run_order()),
        final_norm=norm("final.norm"),
        head=PartSpec.make("lm_head", sizes, {"weight": "embed"}),
        injections=injections,
    )


def kazodra_ignorable_tensors(cfg: KazodraConfig):
    """Tensors a checkpoint may hold that this model does not read: the feed-forward's norms of a layer without one,
    the walks' vectors of a model that walks nothing twice, the second table of a model without token inputs."""
    names = []
    for index, layer in enumerate(cfg.layers):
        if layer.ff is None:
            names += [f"l{index}.norm2", f"l{index}.norm2.b", f"l{index}.norm2b", f"l{index}.norm2b.b"]
    if not cfg.loops:
        names.append("loop.step")
    if cfg.side_dim is None:
        names.append("side.embed")
    return names


def kazodra_kernel_libraries(cfg: KazodraConfig, dtype: str):
    """The kernel files a Kazodra model of this run dtype calls: a first call compiles these and no others."""
    shared = ["elementwise", "sandwich_norm", "pointwise", "sampling"]
    kinds = {type(layer.mixer) for layer in cfg.layers}
    if KazodraLightning in kinds:
        shared.append("lightning")
    if KazodraAttention in kinds:
        shared += ["differential", "attention_masked"]
    if KazodraLatentAttention in kinds:
        shared += ["latent_rope_cache", "attention_masked"]
    if dtype != "float32":
        import torch

        from .. import kernels

        if any(isinstance(layer.mixer, KazodraAttention)
               and kernels.attention_prompt_mma_supported(torch.bfloat16, layer.mixer.dim, layer.mixer.vdim)
               for layer in cfg.layers):
            shared.append("attention_prompt_mma")     # (head sizes the tensor-core attention takes)
        if any(isinstance(layer.mixer, KazodraLatentAttention)
               and kernels.attention_latent_mma_supported(torch.bfloat16, layer.mixer.kv_rank + layer.mixer.rot_dim,
                                                          layer.mixer.kv_rank) for layer in cfg.layers):
            shared.append("attention_latent_mma")     # (latent sizes the tensor-core attention takes)
    shared = list(dict.fromkeys(shared))
    return shared + (["gemm_f32"] if dtype == "float32" else ["decode_linear", "skinny_tcgen05"])


register_architecture(Architecture(
    name=KazodraConfig.ARCHITECTURE,
    read_config=KazodraConfig.from_dict,
    build_spec=kazodra_spec,
    ignorable_tensors=kazodra_ignorable_tensors,
    kernel_libraries=kazodra_kernel_libraries,
))
