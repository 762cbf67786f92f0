"""A selective state-space mixer ("state-space duality" form): one input projection gives a gate z, the
recurrence's input x, its input and output maps B and C (shared by the heads of a group) and a raw step size a
head; x | B | C pass a short causal convolution per channel and silu; per head

    dt_t = softplus(raw_t + dt_bias),  S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t

with S [state, head_dim] float32; y * silu(z) is divided, in `norm_groups` equal parts, by each part's root mean
square, multiplied by a weight, and projected back to the model width.

A request's state (S of every head, and the convolution's last taps - 1 inputs) lives in its state slot, as one
float32 vector; it counts as zero where a sequence starts at position 0.  Step sizes, decays, the recurrence and
the norm are float32; the two projections are products in the engine's dtype with float32 sums."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import MIXERS, Mixer, StateNeed
from .linear import linear


@MIXERS.register("mamba2")
class StateSpaceMixer(Mixer):
    replayable = True      # the step's facts are read from device tensors only

    def __init__(self, prefix: str, width: int, heads: int, head_dim: int, state: int, groups: int, conv: int,
                 norm_groups: int, eps: float, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.heads, self.p, self.n = int(width), int(heads), int(head_dim), int(state)
        self.groups, self.taps, self.norm_groups, self.eps = int(groups), int(conv), int(norm_groups), float(eps)
        if self.heads % self.groups:
            raise InvalidRequest("heads must be a multiple of groups")
        self.inner = self.heads * self.p
        if self.inner % self.norm_groups:
            raise InvalidRequest("the recurrence's output is no multiple of the norm's parts")
        if not 1 <= self.taps <= 16 or self.n > 512 or self.p > 256:
            raise InvalidRequest("convolutions of 1 to 16 taps, states up to 512 and heads up to 256 elements are built")
        self.channels = self.inner + 2 * self.groups * self.n           # x | B | C
        self.leaf = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias",
                     "a_log": "A_log", "d": "D", "norm": "norm.weight", "out": "out_proj.weight"}
        self.leaf.update(names or {})
        self.conv_floats = (self.taps - 1) * self.channels
        self.w_in = self.w_out = None

    def weight_specs(self):
        n = self.leaf
        return [WeightSpec(self.name(n["in"]), (2 * self.inner + 2 * self.groups * self.n + self.heads, self.width)),
                WeightSpec(self.name(n["conv"]), (self.channels, self.taps), "bias"),
                WeightSpec(self.name(n["conv_bias"]), (self.channels,), "bias"),
                WeightSpec(self.name(n["dt_bias"]), (self.heads,), "bias"),
                WeightSpec(self.name(n["a_log"]), (self.heads,), "bias"),
                WeightSpec(self.name(n["d"]), (self.heads,), "bias"),
                WeightSpec(self.name(n["norm"]), (self.inner,), "vector"),
                WeightSpec(self.name(n["out"]), (self.width, self.inner))]

    def state_need(self):
        return StateNeed((self.conv_floats + self.heads * self.n * self.p,), torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        self.w_in = tensors[self.name(n["in"])].contiguous()
        self.w_out = tensors[self.name(n["out"])].contiguous()
        self.conv_w = tensors[self.name(n["conv"])].float().contiguous()
        self.conv_b = tensors[self.name(n["conv_bias"])].float().contiguous()
        self.dt_bias = tensors[self.name(n["dt_bias"])].float().contiguous()
        self.a_log = tensors[self.name(n["a_log"])].float().contiguous()
        self.d_skip = tensors[self.name(n["d"])].float().contiguous()
        self.norm_w = tensors[self.name(n["norm"])].float().contiguous()

    def forward(self, h, ctx, cache, write_cache=True):
        tokens = h.shape[0]
        device = self.w_out.device
        proj = linear(h, self.w_in, out_dtype=torch.float32)            # z | x | B | C | dt
        slots = cache.state.shape[0]
        conv_state = cache.state[:, :self.conv_floats].view(slots, self.taps - 1, self.channels)
        ssm_state = cache.state[:, self.conv_floats:].view(slots, self.heads, self.n, self.p)
        xbc = torch.empty((tokens, self.channels), dtype=torch.float32, device=device)
        kernels.causal_conv_silu(proj, self.inner, self.conv_w, self.conv_b, conv_state, ctx.positions, ctx.seq_of_token,
                                 ctx.q_start, ctx.state_slots, xbc, update_state=write_cache)
        y = torch.zeros((tokens, self.inner), dtype=torch.float32, device=device)
        kernels.ssm_scan(xbc, proj[:, self.inner + self.channels:], self.dt_bias, self.a_log, self.d_skip, ssm_state,
                         ctx.positions, ctx.q_start, ctx.state_slots, y, self.heads, self.groups, self.n, self.p,
                         write_state=write_cache)
        normed = torch.empty((tokens, self.inner), dtype=self.runtime.dtype, device=device)
        kernels.gated_part_norm(y, proj[:, :self.inner], self.norm_w, self.eps, normed, self.norm_groups)
        return linear(normed, self.w_out, out_dtype=torch.float32)
