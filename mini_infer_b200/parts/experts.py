"""Routed experts: a feed-forward of which every token uses a few experts out of many, chosen by a
router, and optionally one shared expert that every token uses.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, ParamDecl, register_feed_forward
from .builtin import Linear, _as_compute


class RoutedExperts(FeedForward):
    """Router logits ``z = W_r h`` in fp32; a token's ``top`` experts are those with the largest
    logits and their weights the softmax over those logits alone; the output is the weighted sum of
    their outputs, plus the shared expert's where there is one.  An expert is
    ``W_down (g' * sigmoid(alpha g') * (u' + 1))`` with ``g' = min(W_gate h, limit)`` and
    ``u' = clamp(W_up h, -limit, limit)``, no biases.

    params: ``hidden_size``, ``experts``, ``top``, ``expert_ff``, ``limit``, optional ``alpha``
    (default 1.702), ``shared_ff`` (0 or absent: no shared expert), ``shared_limit``.
    tensors: ``router``, ``e{i}.gate``, ``e{i}.up``, ``e{i}.down`` and, with a shared expert,
    ``shared.gate``, ``shared.up``, ``shared.down``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.experts, self.top = int(self.param("experts")), int(self.param("top"))
        self.ff = int(self.param("expert_ff"))
        self.limit = float(self.param("limit"))
        self.alpha = float(g("alpha", 1.702))
        self.shared_ff = int(g("shared_ff") or 0)
        self.shared_limit = float(g("shared_limit", self.limit))
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{self.top} of {self.experts} experts per token")

    def param_decls(self):
        H, ff = self.hidden, self.ff
        decls = {"router": ParamDecl((self.experts, H))}
        for e in range(self.experts):
            decls[f"e{e}.gate"] = ParamDecl((ff, H))
            decls[f"e{e}.up"] = ParamDecl((ff, H))
            decls[f"e{e}.down"] = ParamDecl((H, ff))
        if self.shared_ff:
            decls["shared.gate"] = ParamDecl((self.shared_ff, H))
            decls["shared.up"] = ParamDecl((self.shared_ff, H))
            decls["shared.down"] = ParamDecl((H, self.shared_ff))
        return decls

    def bind(self, tensors, dtype, device):
        E = range(self.experts)
        self.router = _as_compute(tensors["router"], dtype).contiguous()
        # per expert its gate rows, then its up rows: one operand for a grouped product, two for the own kernels
        self.w_gate_up = torch.stack([torch.cat([_as_compute(tensors[f"e{e}.gate"], dtype),
                                                 _as_compute(tensors[f"e{e}.up"], dtype)]) for e in E]).contiguous()
        self.w_down = torch.stack([_as_compute(tensors[f"e{e}.down"], dtype) for e in E]).contiguous()
        self.shared_in = self.shared_out = None
        if self.shared_ff:
            self.shared_in = Linear(torch.cat([_as_compute(tensors["shared.gate"], dtype),
                                               _as_compute(tensors["shared.up"], dtype)], dim=0).contiguous())
            self.shared_out = Linear(_as_compute(tensors["shared.down"], dtype).contiguous())

    def forward(self, x, ctx):
        shared = None
        if self.shared_in is not None:
            shared = self.shared_out(ops.clamped_glu(self.shared_in(x), self.shared_limit, self.alpha))
        ids, weights = ops.moe_route(x, self.router, self.top)
        return ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit, self.alpha, shared)


register_feed_forward("routed_experts", RoutedExperts, replace=True)
