"""A selective state-space mixer with one scalar decay per head (Mamba-2, state-space duality),
in its recurrent form.

With ``inner = heads * value_dim``, ``N = state_size`` and ``G = groups``, the input projection
of a row splits into ``z`` (inner), ``x`` (inner), ``B`` (G*N), ``C`` (G*N) and ``dt`` (heads), in
this order.  The ``x | B | C`` columns go through a depthwise convolution along the sequence,
``u_t[c] = b[c] + sum_j w[c, j] * in_{t - (taps-1) + j}[c]`` with inputs of negative positions
taken as zero (so ``w[c, taps-1]`` weighs the row itself), followed by SiLU.  The step size is
``dt = softplus(dt + dt_bias)``; head ``h`` reads ``B`` and ``C`` of group ``h // (heads / G)`` and
keeps a state ``S`` of ``N x value_dim``: ``S_t = exp(-exp(A_log[h]) dt) S_{t-1} + dt B_t x_t^T``,
``y_t = S_t^T C_t + D[h] x_t``.  The gated output ``y * silu(z)`` is cut into ``norm_groups``
slices of equal length, each slice rescaled to unit mean square on its own, multiplied by the
weight ``norm`` and projected out.

What a request carries between steps is a state of fixed size: ``S`` of every head and the last
``conv_taps - 1`` inputs of the convolution, both 32-bit, in the request's state slot.  A portion
that starts at position 0 starts from zeros.  Everything that enters the recurrence is 32-bit;
the projections give 32-bit sums.  The kernels read only the step's device tensors.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, LayerCache, Mixer, PartError, WeightSpec, register
from .linear import Linear


@register("mixer", "mamba2")
class Mamba2(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``value_dim``, ``state_size``, ``groups``,
    ``conv_taps``, ``norm_groups``, ``norm_eps``; tensors ``in``, ``conv``, ``conv.b``,
    ``dt_bias``, ``A_log``, ``D``, ``norm``, ``o``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "heads", "value_dim", "state_size", "groups", "conv_taps", "norm_groups",
                     "norm_eps")
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.vd, self.N = int(p["heads"]), int(p["value_dim"]), int(p["state_size"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["conv_taps"]), int(p["norm_groups"])
        self.eps = float(p["norm_eps"])
        self.inner = self.heads * self.vd
        if self.groups <= 0 or self.heads % self.groups:
            raise PartError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise PartError(f"a row of {self.inner} does not fall into {self.norm_groups} equal parts")
        if self.taps < 1 or self.N < 1 or self.N > 512:
            raise PartError(f"conv_taps {self.taps} / state_size {self.N} are not ones the kernels take")
        self.conv_channels = self.inner + 2 * self.groups * self.N
        self.proj_size = self.inner + self.conv_channels + self.heads
        self.in_proj = Linear(env, self.proj_size, self.hidden)
        self.out_proj = Linear(env, self.hidden, self.inner)
        self.ssm_floats = self.heads * self.N * self.vd
        self.conv_floats = (self.taps - 1) * self.conv_channels

    def weights(self) -> Dict[str, WeightSpec]:
        return {"in": WeightSpec((self.proj_size, self.hidden)),
                "conv": WeightSpec((self.conv_channels, self.taps), "bias"),
                "conv.b": WeightSpec((self.conv_channels,), "bias"),
                "dt_bias": WeightSpec((self.heads,), "bias"), "A_log": WeightSpec((self.heads,), "bias"),
                "D": WeightSpec((self.heads,), "bias"), "norm": WeightSpec((self.inner,), "norm"),
                "o": WeightSpec((self.hidden, self.inner))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.in_proj.load(tensors["in"])
        self.out_proj.load(tensors["o"])
        # what enters the recurrence is 32-bit whatever the engine's type
        self.conv_w = tensors["conv"].float().contiguous()
        self.conv_b = tensors["conv.b"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.a_log = tensors["A_log"].float().contiguous()
        self.d_skip = tensors["D"].float().contiguous()
        self.norm_w = tensors["norm"].contiguous()

    def state_bytes(self) -> int:
        return 4 * (self.ssm_floats + self.conv_floats)

    def forward(self, h: torch.Tensor, step, cache: LayerCache) -> torch.Tensor:
        T, S = h.shape[0], step.num_seqs
        ws = self.env.workspace
        proj = self.in_proj.forward(h, "mamba.proj", "float32")              # [T, z | x B C | dt]
        rows = cache.state.view(torch.float32)                               # [slots, ssm | conv]
        ssm_state = rows[:, :self.ssm_floats].unflatten(1, (self.heads, self.N, self.vd))
        conv_state = rows[:, self.ssm_floats:].unflatten(1, (self.taps - 1, self.conv_channels)) \
            if self.taps > 1 else None
        xbc = ws.get("mamba.xbc", (T, self.conv_channels), torch.float32)
        ops.causal_conv_silu(proj, self.inner, self.conv_w, self.conv_b, conv_state, step.token_seq, step.seq_start,
                             step.positions, step.state_slots, xbc, S)
        y = ws.get("mamba.y", (T, self.inner), torch.float32)
        ops.ssm_scan(xbc, proj[:, self.inner + self.conv_channels:], self.dt_bias, self.a_log, self.d_skip,
                     ssm_state, step.seq_start, step.positions, step.state_slots, y, S, self.heads, self.groups,
                     self.N, self.vd)
        gated = ws.get("mamba.gated", (T, self.inner), self.env.dtype)
        ops.gated_group_rmsnorm(y, proj[:, :self.inner], self.norm_w, self.eps, gated, self.norm_groups)
        return self.out_proj.forward(gated, "mamba.o", "delta")
