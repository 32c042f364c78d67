"""The Nutizen architecture as a ``ModelSpec``: a decoder whose layers attend through cached
low-rank latents inside a sliding window, with a learned sink per head and no position
encoding, over several residual streams; the feed-forward is a dense gated MLP, or experts
that a table assigns to token ids plus an expert that every token runs, or absent.

This file holds no sizes and no kernels: it translates ``NutizenConfig`` into part
descriptions.  What the design fixes is written here as parameters of general parts: the
experts' activation is the clamped one with slope 1.702, each table-chosen expert weighs
1 / top on its output, the shared expert is gated by the sigmoid of a logit, every head has a
sink.  A layer with ``kv_from`` reads the cache slot of the layer it names; that slot keeps
as many keys as the widest window among its readers needs.  Without ``streams`` the layers are
plain pre-norm layers.  Tensor names: ``embed``, ``head``, ``final.norm``, and
``l<i>.{norm1,norm2}``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc{1,2}.{in,out,mix}`` for layer i.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.nutizen import NutizenConfig
from ..parts.spec import BlockSpec, LayerCall, ModelSpec, PartSpec

MAX_POSITION = 1 << 24          # no table depends on the position: the cache's size is the only bound
EXPERT_SLOPE = 1.702            # of the experts' sigmoid


def build_nutizen_spec(cfg: NutizenConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", "", {"width": d, "eps": cfg.norm_eps, "tensor": name})

    # what each cache must keep: the widest window among the layer that writes it and its readers
    keep = {}
    for i, L in enumerate(cfg.layers):
        owner = i if L.mixer.kv_from is None else L.mixer.kv_from
        w = L.mixer.window
        if owner not in keep:
            keep[owner] = w
        elif keep[owner] is not None:
            keep[owner] = None if w is None else max(keep[owner], w)
    slot_of = {owner: n for n, owner in enumerate(sorted(keep))}

    blocks, schedule = [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        own = m.kv_from is None
        owner = i if own else m.kv_from
        mixer = PartSpec("latent_attention", p + ".mix", {
            "hidden": d, "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "q_rank": m.q_rank,
            "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": m.window,
            "cache_window": keep[owner], "sinks": True, "own_latent": own,
            "tensors": {"dq_norm": p + ".mix.dq.norm", "dkv_norm": p + ".mix.dkv.norm"}})
        ff = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ff = PartSpec("gated_mlp", p + ".mlp", {"hidden": d, "intermediate": L.mlp.ff, "activation": "silu",
                                                    "tensors": {k: f"{p}.mlp.{k}" for k in ("gate", "up", "down")}})
        elif L.mlp is not None:
            shared = None
            if L.mlp.shared_ff:
                shared = {"ff": L.mlp.shared_ff, "activation": "clamped", "limit": L.mlp.shared_limit,
                          "alpha": EXPERT_SLOPE,
                          "tensors": {"gate": p + ".mlp.shared.gate", "up": p + ".mlp.shared.up",
                                      "down": p + ".mlp.shared.down", "gate_logit": p + ".mlp.shared.sg"}}
            ff = PartSpec("routed_experts", p + ".mlp", {
                "hidden": d, "experts": L.mlp.experts, "top": L.mlp.top, "expert_ff": L.mlp.ff,
                "routing": "table", "table_tensor": p + ".mlp.table", "vocab": cfg.vocab,
                "table_weight": 1.0 / L.mlp.top, "weight_on": "output",
                "activation": "clamped", "limit": L.mlp.limit, "alpha": EXPERT_SLOPE, "shared": shared})
        params = {}
        if cfg.streams:
            params = {"streams": cfg.streams, "read1": p + ".hc1.in", "write1": p + ".hc1.out", "mix1": p + ".hc1.mix",
                      "read2": p + ".hc2.in", "write2": p + ".hc2.out", "mix2": p + ".hc2.mix"}
        blocks.append(BlockSpec(kind="residual_streams" if cfg.streams else "pre_norm", prefix=p, mixer=mixer,
                                feed_forward=ff, mixer_norm=norm(p + ".norm1"),
                                ff_norm=norm(p + ".norm2") if ff else None, params=params))
        schedule.append(LayerCall(block=i, cache=slot_of[owner], writes_cache=own))
    return ModelSpec(
        hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", "", {"vocab": cfg.vocab, "width": d, "scale": cfg.embedding_scale,
                                                   "tensor": "embed"}),
        blocks=blocks, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "", {"vocab": cfg.vocab, "width": d, "tied_to": None, "tensor": "head"}),
        eos_token_ids=())


register_architecture("Nutizen", NutizenConfig, build_nutizen_spec)
