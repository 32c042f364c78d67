"""Several residual streams in place of one: the ``residual_streams`` arrangement of a layer.

A model of this kind keeps S copies x_1 .. x_S of the residual stream, all equal to the
embedding's output at the start.  Sublayer q of a layer (1: the mixer, 2: the feed-forward)
has three small tensors, ``in`` [S], ``out`` [S] and ``mix`` [S, S] (indexed [from, to]):

    u   = sum_s in[s] x_s
    y   = sublayer(norm(u))
    x_t <- sum_s mix[s, t] x_s + out[t] y          every t at once, from the old streams

and the model's output stream is the sum of the streams.  The streams are float32 [S, n, d]
and live for one step; a sublayer's write, the next sublayer's read and its RMS norm are one
kernel (csrc/streams.cu), also across layers: the block hands on a ``ResidualStreams`` as its
``pending`` with the last write still owed, and the next block of this kind (or ``settle``, which
leaves the sum of the streams in the model's single stream x) performs it.

params of the block: ``streams`` (S), ``read1`` / ``write1`` / ``mix1`` and ``read2`` / ``write2`` /
``mix2`` (full tensor names, float32).  ``feed_forward`` may be None.  The norms must be RMS
norms that a kernel can apply itself (``fusable_rmsnorm``: ``gain``, ``eps``).
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BlockSpec, BuildEnv, TensorSpec, part_factory, register_part


class ResidualStreams:
    """The S streams of a step and the write that is still owed to them."""

    accepted_by = "accepts_streams"

    def __init__(self, xs, y, mix, out_w):
        self.xs, self.y, self.mix, self.out_w = xs, y, mix, out_w

    def settle(self, x):
        """Perform the owed write and leave the sum of the streams in x."""
        kernels.streams_step(self.xs, y=self.y, mix=self.mix, out_w=self.out_w, total=x)
        self.y = None
        return None

    def peek(self, x):
        """What ``settle`` would leave in x, computed on a copy."""
        total = torch.empty_like(x)
        kernels.streams_step(self.xs.clone(), y=self.y, mix=self.mix, out_w=self.out_w, total=total)
        return total


class ResidualStreamsBlock:
    accepts_streams = True

    def __init__(self, spec: BlockSpec, env: BuildEnv):
        p = spec.params
        self.S = int(p["streams"])
        if not 1 <= self.S <= 16:
            raise ValueError(f"residual streams: {self.S} streams (1 to 16)")
        self.dtype = env.dtype
        self.mixer = part_factory("mixer", spec.mixer.kind)(spec.mixer, env)
        self.mixer_norm = part_factory("norm", spec.mixer_norm.kind)(spec.mixer_norm, env)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = part_factory("feed_forward", spec.feed_forward.kind)(spec.feed_forward, env)
            self.ff_norm = part_factory("norm", spec.ff_norm.kind)(spec.ff_norm, env)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not getattr(norm, "fusable_rmsnorm", False):
                raise ValueError("residual streams: the norms must be RMS norms with a gain and an eps")
        self.names = {k: p[k] for k in ("read1", "write1", "mix1")}
        if self.feed_forward is not None:
            self.names.update({k: p[k] for k in ("read2", "write2", "mix2")})
        self.w = {}

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        S = self.S
        own = [TensorSpec(name, (S, S) if key.startswith("mix") else (S,), store="float32",
                          init="eye" if key.startswith("mix") else ("mean" if key.startswith("read") else "gain"))
               for key, name in self.names.items()]
        return own + [s for p in self.parts() for s in p.tensor_specs()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors):
        for p in self.parts():
            p.bind(tensors)
        self.w = {key: tensors[name].contiguous() for key, name in self.names.items()}

    def forward(self, x, pending, ctx, cache):
        w, norm1 = self.w, self.mixer_norm
        normed = torch.empty(x.shape, dtype=self.dtype, device=x.device)
        if isinstance(pending, ResidualStreams) and pending.xs.shape[0] == self.S:
            xs = pending.xs
            kernels.streams_step(xs, y=pending.y, mix=pending.mix, out_w=pending.out_w, in_w=w["read1"],
                                 gain=norm1.gain, eps=norm1.eps, normed=normed)
        else:
            if hasattr(pending, "settle"):
                pending = pending.settle(x)
            if pending is not None:
                x.add_(pending.to(torch.float32))
            xs = torch.empty((self.S,) + tuple(x.shape), dtype=torch.float32, device=x.device)
            kernels.streams_step(xs, init=x, in_w=w["read1"], gain=norm1.gain, eps=norm1.eps, normed=normed)
        y = self._f32(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return ResidualStreams(xs, y, w["mix1"], w["write1"])
        norm2 = self.ff_norm
        normed = torch.empty(x.shape, dtype=self.dtype, device=x.device)
        kernels.streams_step(xs, y=y, mix=w["mix1"], out_w=w["write1"], in_w=w["read2"], gain=norm2.gain,
                             eps=norm2.eps, normed=normed)
        y = self._f32(self.feed_forward.forward(normed, ctx))
        return ResidualStreams(xs, y, w["mix2"], w["write2"])

    @staticmethod
    def _f32(y):
        return y if y.dtype == torch.float32 and y.is_contiguous() else y.to(torch.float32).contiguous()


register_part("block", "residual_streams", ResidualStreamsBlock)
