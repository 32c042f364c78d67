"""The Sozarax architecture as a ``ModelSpec``: a decoder whose layers are either a
recurrent mixer (``wkv``) or causal attention without rotation, each with a norm before
and after every sublayer, a dense or routed feed-forward or none, and a run of layers
that may repeat with the same weights.

This file holds no sizes and no kernels: it translates ``SozaraxConfig`` into part
descriptions.  What the design fixes is written here as parameters of general parts:
the attention layer is the paged attention mixer with an RMS norm over the whole q and k
projections and a position-dependent temperature on the queries (``whole_rmsnorm``),
no position part, geometric slopes of a bias that grows with the distance, float32
softmax weights, and values of their own head size; the dense feed-forward is the plain
MLP with the square of relu; the experts are routed by sigmoid scores that are used as
they are and multiply the expert's input.  A layer that runs several times gets a cache
slot (pages or state) per run.  Tensor names: ``embed``, ``head``, ``final.norm``, and
``l<i>.{norm1,norm1b,norm2,norm2b}``, ``l<i>.mix.*``, ``l<i>.mlp.*`` for layer i.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.sozarax import SozaraxConfig
from ..parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec

MAX_POSITION = 1 << 24          # no table depends on the position: the cache's size is the only bound


def build_sozarax_spec(cfg: SozaraxConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", "", {"width": d, "eps": cfg.norm_eps, "tensor": name})

    blocks = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        if L.type == "wkv":
            mixer = PartSpec("wkv", p + ".mix", {"hidden": d, "heads": m.heads, "size": m.dim, "eps": cfg.norm_eps})
        else:
            mixer = PartSpec("paged_attention", p + ".mix", {
                "hidden": d, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "window": None, "scale": m.scale, "position": None, "score_slopes": "geometric", "exact_weights": True,
                "tensors": {k: f"{p}.mix.{k}" for k in "qkvo"},
                "qk_transform": PartSpec("whole_rmsnorm", "", {
                    "q_dim": m.heads * m.dim, "k_dim": m.kv_heads * m.dim, "eps": cfg.norm_eps,
                    "q_gain": p + ".mix.q.norm", "k_gain": p + ".mix.k.norm",
                    "temp_coef": m.q_temp_coef, "temp_every": m.q_temp_every})})
        ff = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ff = PartSpec("plain_mlp", p + ".mlp", {"hidden": d, "intermediate": L.mlp.ff, "activation": "relu2"})
        elif L.mlp is not None:
            ff = PartSpec("routed_experts", p + ".mlp", {
                "hidden": d, "experts": L.mlp.experts, "top": L.mlp.top, "expert_ff": L.mlp.ff,
                "score": "sigmoid", "renormalize": False, "weight_on": "input"})
        blocks.append(BlockSpec(
            kind="sandwich_norm", prefix=p, mixer=mixer, feed_forward=ff,
            mixer_norm=norm(p + ".norm1"), ff_norm=norm(p + ".norm2") if ff else None,
            params={"mixer_post_norm": norm(p + ".norm1b"), "ff_post_norm": norm(p + ".norm2b") if ff else None}))
    return ModelSpec(
        hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", "", {"vocab": cfg.vocab, "width": d, "scale": cfg.embedding_scale,
                                                   "tensor": "embed"}),
        blocks=blocks,
        schedule=[LayerCall(block=b, cache=run) for run, b in enumerate(cfg.layer_order())],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "", {"vocab": cfg.vocab, "width": d, "tied_to": None, "tensor": "head"}),
        eos_token_ids=())


register_architecture("Sozarax", SozaraxConfig, build_sozarax_spec)
