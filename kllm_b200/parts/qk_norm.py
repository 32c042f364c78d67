"""RMS norm of queries and keys over the WHOLE projection (all heads at once, before
they are split), with a temperature on the queries that grows with the position:
a ``qk_transform`` of the attention mixer for layers without rotation.

    q <- q / sqrt(mean(q^2 over H * dk) + eps) * g_q * (1 + coef * ln(floor((p + 1) / every) + 1))
    k <- k / sqrt(mean(k^2 over G * dk) + eps) * g_k

params: ``q_dim`` (H * dk), ``k_dim`` (G * dk), ``eps``, ``q_gain`` / ``k_gain`` (full tensor
names, plain gains, float32), ``temp_coef`` (0 or absent: no temperature), ``temp_every``.
It offers ``prepare`` (see ``parts/attention.py``): it takes the projection's float32
result, so sums, scales and the temperature are float32 in both dtypes, returns the queries
in the model dtype and writes keys and values (of their own head size) into the layer's
pages, all in one kernel (csrc/qknorm_append.cu).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class WholeProjectionNorm:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.q_dim, self.k_dim = int(p["q_dim"]), int(p["k_dim"])
        self.eps = float(p["eps"])
        self.q_name, self.k_name = p["q_gain"], p["k_gain"]
        self.coef = float(p.get("temp_coef") or 0.0)
        self.every = int(p.get("temp_every") or 1)
        if self.coef != 0.0 and self.every < 1:
            raise ValueError(f"query temperature: period {self.every} must be positive")
        self.dtype = env.dtype
        self.q_gain = self.k_gain = None

    def tensor_specs(self):
        return [TensorSpec(self.q_name, (self.q_dim,), store="float32", init="gain"),
                TensorSpec(self.k_name, (self.k_dim,), store="float32", init="gain")]

    def bind(self, tensors):
        self.q_gain, self.k_gain = tensors[self.q_name], tensors[self.k_name]

    def prepare(self, qkv, ctx, cache, attn):
        q = torch.empty((qkv.shape[0], self.q_dim), dtype=self.dtype, device=qkv.device)
        writes = cache.writes
        kernels.qknorm_append(q, qkv, self.q_gain, self.k_gain if writes else None, self.eps, self.coef, self.every,
                              ctx.positions, ctx.token_req, cache.block_table if writes else None,
                              cache.k if writes else None, cache.v if writes else None,
                              attn.n_heads, attn.n_kv, attn.head_dim, attn.v_head_dim)
        return q


register_part("qk_transform", "whole_rmsnorm", WholeProjectionNorm)
