"""A recurrent mixer in the manner of RWKV's time mixing: a linear-attention state per
head with a data-dependent decay per key channel and a bonus for the current token.

With h the mixer's input, h' the row before it in the same sequence (zeros before the
first token) and m_s = h + (h' - h) * mu_s for s in r, k, v, g, w:

    r, k, v = W_r m_r, W_k m_k, W_v m_v          [heads * size]
    gate    = silu(W_g m_g)
    w       = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))   per head and key channel, in (0, 1)
    o_t     = (S_(t-1) + diag(u) k_t v_t^T)^T r_t ;  S_t = diag(w_t) S_(t-1) + k_t v_t^T   per head
    y       = W_o (concat_heads(o / rms(o)) * gain * gate)

params: ``hidden``, ``heads``, ``size`` (key and value channels of a head), ``eps`` (of the
heads' unit norm), ``decay_rank`` (rows of W_w1 for random weights; a file's own rank is
taken from its tensor), optional ``tensors`` (name -> full tensor name for mu.r .. mu.w, r,
k, v, g, w1, w2, w0, u, norm, o; default ``<prefix>.<name>``).

State (``StateNeed``): per request one float32 vector, [heads][value channel][key channel] for
S followed by [hidden] for the last row of h that the request has seen (rounded up to a
multiple of four floats), zero when the request opens.
Decay, state, sums, unit norm and gate are float32 in both dtypes; the projections take
inputs in the model dtype and hand their results on unrounded (float32); the decay's inner
product goes through tanh and its outer matrix in one float32 kernel.  Kernels: csrc/wkv.cu
(token shift, decay, recurrence, unit norm and gate); the projections are library products,
or the weight-streaming product for steps of a few rows.  A position's result does not depend on how its prompt was cut: the recurrence
visits a request's rows one by one in order, whatever the batch.
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, StateNeed, TensorSpec, register_part

_MIX = ("r", "k", "v", "g", "w")


class WkvMixer:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.size = int(p["size"])
        if not (0 < self.size <= 128):
            raise ValueError(f"wkv: a head of {self.size} channels (the recurrence kernel holds up to 128)")
        self.eps = float(p["eps"])
        self.rank = int(p.get("decay_rank") or 16)
        self.inner = self.heads * self.size
        self.dtype = env.dtype
        names = dict(p.get("tensors") or {})
        self.n = {k: names.get(k) or f"{spec.prefix}.{k}" for k in
                  [f"mu.{s}" for s in _MIX] + ["r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o"]}
        self.state_size = -(-(self.inner * self.size + self.hidden) // 4) * 4    # whole 16-byte units per slot

    def tensor_specs(self):
        n, d, A = self.n, self.hidden, self.inner
        return [TensorSpec(n[f"mu.{s}"], (d,), store="float32", init="uniform:0:1") for s in _MIX] + \
            [TensorSpec(n[s], (A, d)) for s in ("r", "k", "v", "g")] + \
            [TensorSpec(n["w1"], (self.rank, d), free=(0,)), TensorSpec(n["w2"], (A, self.rank), free=(1,)),
             TensorSpec(n["w0"], (A,), store="float32", init="uniform:-6:0"),
             TensorSpec(n["u"], (self.heads, self.size), store="float32"),
             TensorSpec(n["norm"], (A,), store="float32", init="gain"), TensorSpec(n["o"], (d, A))]

    def bind(self, tensors):
        n = self.n
        self.mu = torch.stack([tensors[n[f"mu.{s}"]] for s in _MIX]).contiguous()
        # the four projections read four inputs: one batched product over the stacked matrices
        self.w_rkvg = torch.stack([tensors[n[s]] for s in ("r", "k", "v", "g")]).contiguous()
        self.w1, self.w2 = tensors[n["w1"]], tensors[n["w2"]].contiguous()
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"wkv: the decay's two matrices disagree on its rank ({tuple(self.w1.shape)}, "
                             f"{tuple(self.w2.shape)})")
        self.w0 = tensors[n["w0"]].reshape(-1).contiguous()
        self.u = tensors[n["u"]].reshape(-1).contiguous()
        self.gain = tensors[n["norm"]]
        self.w_o = tensors[n["o"]]

    def cache_need(self):
        return StateNeed((self.state_size,), "float32")

    def forward(self, xn, ctx, cache):
        f32 = torch.float32
        state = cache.state
        mix = kernels.wkv_shift_mix(xn, self.mu, state, self.inner * self.size, ctx)
        if kernels.skinny_fits(xn.shape[0], self.hidden, self.dtype):
            # a few rows: four weight-streaming products instead of one batched library product
            r, k, v, g = (kernels.linear(mix[i], self.w_rkvg[i], out_dtype=f32, small_ok=True) for i in range(4))
        else:
            r, k, v, g = kernels.linear_batched(mix[:4], self.w_rkvg)
        low = kernels.linear(mix[4], self.w1, out_dtype=f32, small_ok=True)
        if self.w2.shape[1] <= 256:
            z = kernels.wkv_decay_outer(low, self.w2)           # tanh and the outer matrix in one kernel
        else:
            z = kernels.linear(kernels.unary(low, "tanh", self.dtype), self.w2, out_dtype=f32)
        o = kernels.wkv_scan(r, k, v, z, self.w0, self.u, state, ctx, self.heads, self.size)
        y = kernels.wkv_gate_norm(o, g, self.gain, self.eps, self.heads, self.size, self.dtype)
        return kernels.linear(y, self.w_o, out_dtype=f32, small_ok=True)


register_part("mixer", "wkv", WkvMixer)
