"""Routed experts: a feed-forward in which every token runs ``top`` of ``experts`` small
gated feed-forwards, chosen by a router.

    z = W_router h (float32);  s = sigmoid(z) or softmax(z);  the ``top`` largest s are chosen
    expert_e(x) = W_down,e (silu(W_gate,e x) * (W_up,e x))
    y = sum over the chosen e of  expert_e(s_e h)        (``weight_on`` "input")
     or sum over the chosen e of  s_e expert_e(h)        (``weight_on`` "output")

params: ``hidden``, ``experts``, ``top``, ``expert_ff``, ``score`` ("sigmoid" | "softmax"),
``renormalize`` (divide the chosen scores by their sum), ``weight_on`` ("input" | "output"),
optional ``router_tensor`` and ``expert_tensors`` (a format string with ``{e}`` and ``{m}``
for the expert's number and matrix gate/up/down; default ``<prefix>.e{e}.{m}``).
The router table stays float32 in both dtypes.  At bind time the experts' matrices are
stacked into [E, 2f, d] (gate rows, then up rows) and [E, d, f].

A step sorts its (token, choice) pairs by expert on the device and runs two grouped
products over the sorted rows (csrc/moe.cu); shapes and launch sizes depend on the number
of tokens alone, never on the routing, so decode steps can be replayed as CUDA graphs.
The result is float32 [n, hidden].
"""
from __future__ import annotations

import torch

from .. import kernels
from .spec import BuildEnv, PartSpec, TensorSpec, register_part


class RoutedExperts:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        p = spec.params
        self.hidden = int(p["hidden"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_ff"])
        if not (1 <= self.top <= self.experts <= 1024):
            raise ValueError(f"routed experts: {self.top} of {self.experts} (at most 1024 experts)")
        self.score = p.get("score", "sigmoid")
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on = p.get("weight_on", "input")
        if self.score not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: score {self.score!r}, weight on {self.weight_on!r}")
        self.router_name = p.get("router_tensor") or f"{spec.prefix}.router"
        self.fmt = p.get("expert_tensors") or (spec.prefix + ".e{e}.{m}")
        self.dtype = env.dtype

    def _name(self, e, m):
        return self.fmt.format(e=e, m=m)

    def tensor_specs(self):
        out = [TensorSpec(self.router_name, (self.experts, self.hidden), store="float32")]
        for e in range(self.experts):
            out += [TensorSpec(self._name(e, "gate"), (self.ff, self.hidden)),
                    TensorSpec(self._name(e, "up"), (self.ff, self.hidden)),
                    TensorSpec(self._name(e, "down"), (self.hidden, self.ff))]
        return out

    def bind(self, tensors):
        self.router = tensors[self.router_name]
        self.w_gate_up = torch.stack([torch.cat([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.experts)]).contiguous()

    def forward(self, xn, ctx):
        idx, wt = kernels.moe_route(xn, self.router, self.top, self.score, self.renormalize)
        offsets, perm = kernels.moe_sort(idx, self.experts)
        on_input = self.weight_on == "input"
        act = kernels.moe_gemm(xn, self.w_gate_up, offsets, perm, wt, self.top, gated=True, scale_in=on_input)
        parts = kernels.moe_gemm(act, self.w_down, offsets, perm, wt, self.top, gated=False, scale_out=not on_input)
        return kernels.moe_combine(parts, self.top)


register_part("feed_forward", "routed_experts", RoutedExperts)
