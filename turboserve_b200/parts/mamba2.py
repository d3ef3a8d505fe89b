"""The Mamba-2 mixer: a state-space recurrence with one scalar decay per head.

With ``inner = heads * vdim``, ``N = state`` and ``G = groups`` the input projection gives, per
token, ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``. ``x``, ``B`` and ``C`` together
pass a short causal convolution per channel (``taps`` taps, with a bias) and silu. Then per head
``h`` (group ``h // (heads / G)``), in float32:

    dt  = softplus(dt + dt_bias)
    S_t = exp(-exp(A_log) dt) S_{t-1} + dt B_t x_t^T          (S is N x vdim, zero at the start)
    y_t = S_t^T C_t + D x_t

``y`` (the heads side by side) is multiplied by ``silu(z)``, divided part by part (``norm_groups``
equal parts of a row) by its root mean square with ``eps`` inside the root, multiplied by a weight
and projected back. A request keeps two states between steps: ``S`` of every head in float32 and
the last ``taps - 1`` inputs of the convolution.

Sizes and constants are parameters: ``heads``, ``vdim``, ``state``, ``groups``, ``norm_groups``,
``taps``, ``eps``; ``names`` maps the roles ``in conv conv_bias dt_bias a_log d norm out`` to the
checkpoint's local tensor names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, ParamSpec, StateNeed, register_mixer

DEFAULT_NAMES = {
    "in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias",
    "a_log": "A_log", "d": "D", "norm": "norm.weight", "out": "out_proj.weight",
}


class Mamba2Mixer(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("a state-space mixer has no pages another run could share")
        self.hidden_size = int(hidden_size)
        self.heads, self.vdim, self.state = int(spec["heads"]), int(spec["vdim"]), int(spec["state"])
        self.groups, self.norm_groups = int(spec.get("groups", 1)), int(spec.get("norm_groups", 1))
        self.taps = int(spec.get("taps", 4))
        self.eps = float(spec["eps"])
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        self.inner = self.heads * self.vdim
        if self.heads % self.groups:
            raise ValueError(f"heads ({self.heads}) must be a multiple of groups ({self.groups})")
        if self.inner % self.norm_groups:
            raise ValueError(f"heads * vdim ({self.inner}) must be a multiple of norm_groups ({self.norm_groups})")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"taps must be between 1 and 16, got {self.taps}")
        if not 1 <= self.state <= 512:
            raise ValueError(f"state must be between 1 and 512, got {self.state}")
        self.conv_width = self.inner + 2 * self.groups * self.state
        self.proj_width = self.inner + self.conv_width + self.heads
        for name in ("in_w", "conv_w", "conv_b", "dt_bias", "a_log", "d_skip", "norm_w", "out_w"):
            setattr(self, name, None)

    def cache_need(self):
        recurrent = StateNeed((self.heads, self.vdim, self.state), torch.float32)
        if self.taps == 1:
            return recurrent
        return recurrent, StateNeed((self.taps - 1, self.conv_width), None)

    def scratch_per_token(self) -> int:
        # the projection, the convolved channels, y in float32 (two elements' worth), the normed rows, the output
        return self.proj_width + self.conv_width + 3 * self.inner + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        return [
            ParamSpec(n["in"], (self.proj_width, h)),
            ParamSpec(n["conv"], (self.conv_width, self.taps), role="gain", init="bias_normal"),
            ParamSpec(n["conv_bias"], (self.conv_width,), role="bias", init="bias_normal"),
            ParamSpec(n["dt_bias"], (self.heads,), role="bias", init="bias_normal"),
            ParamSpec(n["a_log"], (self.heads,), role="gain", init="bias_normal"),
            ParamSpec(n["d"], (self.heads,), role="gain", init="one_plus_normal"),
            ParamSpec(n["norm"], (self.inner,), role="gain", init="one_plus_normal"),
            ParamSpec(n["out"], (h, self.inner)),
        ]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.in_w = tensors[n["in"]].contiguous()
        self.conv_w = tensors[n["conv"]].contiguous()
        self.conv_b = tensors[n["conv_bias"]].contiguous()
        self.dt_bias = tensors[n["dt_bias"]].contiguous()
        self.a_log = tensors[n["a_log"]].contiguous()
        self.d_skip = tensors[n["d"]].contiguous()
        self.norm_w = tensors[n["norm"]].contiguous()
        self.out_w = tensors[n["out"]].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        projected = ctx.buffer("mamba2.in", (n, self.proj_width))
        linear(x, self.in_w, projected, None, n, ctx)
        convolved = ctx.buffer("mamba2.conv", (n, self.conv_width))
        tail = cache.states[1] if self.taps > 1 else projected.new_empty((1, 0, self.conv_width))
        kernels.causal_conv(projected, self.inner, self.conv_w, self.conv_b, tail, convolved, batch.seq_of_token,
                            batch.query_start_loc, batch.state_slots, n, batch.num_seqs, silu=True, status=ctx.status)
        y = ctx.buffer("mamba2.y", (n, self.inner), torch.float32)
        kernels.ssd_scan(convolved, projected[:, self.inner + self.conv_width:], self.dt_bias, self.a_log, self.d_skip,
                         cache.states[0], y, batch.query_start_loc, batch.state_slots, batch.num_seqs, self.heads,
                         self.groups, self.vdim, self.state, num_tokens=n)
        normed = ctx.buffer("mamba2.normed", (n, self.inner))
        kernels.gated_group_norm(y, projected[:, :self.inner], self.norm_w, normed, n, self.norm_groups, self.eps)
        out = ctx.buffer("mamba2.out", (n, self.hidden_size))
        linear(normed, self.out_w, out, None, n, ctx)
        return out


register_mixer("mamba2", Mamba2Mixer)
