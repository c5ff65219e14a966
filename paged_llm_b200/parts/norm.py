"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, eps inside the
root, the weight multiplied before the down-cast (reference:
pagedllm/model/llama.py:74-83).  With `unit_offset` the checkpoint stores the
weight around zero and the factor is 1 + w; it is formed once, in float32, when
the weights are taken."""

from __future__ import annotations

from .base import LazyLinear, Norm, TensorSpec, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, weights: dict[str, str], dim: int, eps: float, unit_offset: bool = False):
        self.dim, self.eps, self.unit_offset = dim, float(eps), bool(unit_offset)
        self.name = weights["weight"]
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.dim,), role="vector", init="norm_zero" if self.unit_offset else "norm")}

    def load(self, tensors):
        w = tensors[self.name]
        self.weight = (w.float() + 1.0).contiguous() if self.unit_offset else w.contiguous()

    def bytes_read_per_step(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, ctx):
        return ctx.ops.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, branch, ctx):
        if branch is None:
            return ctx.ops.rms_norm(x, self.weight, self.eps)
        if isinstance(branch, LazyLinear):
            return ctx.ops.linear_add_rms_norm(branch.input, branch.weight, x, self.weight, self.eps)
        return ctx.ops.add_rms_norm(x, branch, self.weight, self.eps)
