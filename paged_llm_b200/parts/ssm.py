"""A selective state-space mixer with a scalar decay per head (the state-space duality form).

    [z | x | B | C | dt] = W_in h             z, x: heads * head_dim; B, C: groups * state; dt: heads
    [x | B | C] <- silu(conv(.) + bias)        causal convolution per channel, `taps` wide
    dt <- softplus(dt + dt_bias)
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T     per head (its group's B and C), S: [state, head_dim]
    y_t = S_t^T C_t + D x_t
    out = W_o (norm_in_parts(y * silu(z)) * w)               `norm_groups` equal parts, each by its own RMS

The state per request is of fixed size and float32: the last taps-1 inputs of the convolution and S.  It
starts at zero and is carried from token to token, so a request's tokens may arrive in portions of any size.
dt, the decay, the recurrence, the gate and the norm are float32 in both precisions.
"""

from __future__ import annotations

from .base import FixedState, LazyLinear, Mixer, TensorSpec, register_mixer


@register_mixer("state_space")
class StateSpaceMixer(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, head_dim: int, state_size: int,
                 groups: int, conv_taps: int, norm_groups: int, eps: float):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads do not divide into {groups} groups")
        self.inner = num_heads * head_dim
        if self.inner % norm_groups:
            raise ValueError(f"{self.inner} channels do not divide into {norm_groups} parts for the norm")
        if conv_taps < 1:
            raise ValueError(f"conv_taps={conv_taps}")
        self.hidden_size, self.num_heads, self.head_dim, self.state_size = hidden_size, num_heads, head_dim, state_size
        self.groups, self.conv_taps, self.norm_groups, self.eps = groups, conv_taps, norm_groups, float(eps)
        self.channels = self.inner + 2 * groups * state_size
        self.names = weights
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def cache_requirement(self):
        return FixedState(((self.conv_taps - 1) * self.channels + self.num_heads * self.head_dim * self.state_size,))

    def tensor_specs(self):
        n = self.names
        return {
            n["in_proj"]: TensorSpec((2 * self.inner + 2 * self.groups * self.state_size + self.num_heads, self.hidden_size)),
            n["conv"]: TensorSpec((self.channels, self.conv_taps), role="vector"),
            n["conv_bias"]: TensorSpec((self.channels,), role="vector"),
            n["dt_bias"]: TensorSpec((self.num_heads,), role="vector"),
            n["a_log"]: TensorSpec((self.num_heads,), role="vector"),
            n["d_skip"]: TensorSpec((self.num_heads,), role="vector", init="norm"),
            n["norm"]: TensorSpec((self.inner,), role="vector", init="norm"),
            n["o_proj"]: TensorSpec((self.hidden_size, self.inner)),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = tensors[n["in_proj"]].contiguous()
        self.w_o = tensors[n["o_proj"]].contiguous()
        f32 = lambda k: tensors[n[k]].float().contiguous()      # noqa: E731
        self.conv_w, self.conv_b, self.dt_bias = f32("conv"), f32("conv_bias"), f32("dt_bias")
        self.a_log, self.d_skip, self.norm_w = f32("a_log"), f32("d_skip"), f32("norm")

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        if any(slot < 0 for slot in ctx.host.state_slots):
            raise RuntimeError("a request of a model with per-request state runs without a state slot "
                               "(CacheManager.acquire_state_slot at its admission)")
        zx = ops.linear(h, self.w_in)
        y = ops.ssm_mix(zx, self.inner, self.groups, self.state_size, self.num_heads, self.head_dim, self.conv_w,
                        self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w, self.norm_groups, self.eps,
                        cache.state, ctx)
        return LazyLinear(y, self.w_o)
