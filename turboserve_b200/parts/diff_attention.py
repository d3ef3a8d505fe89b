"""Differential attention over a paged cache, with a short causal convolution after the projections.

Per token ``q, k, v = x Wq^T, x Wk^T, x Wv^T`` (one fused product, no biases); each channel of
``q``, ``k`` and ``v`` then passes a short causal convolution over time (``taps`` taps, no bias, no
activation; the last ``taps - 1`` projected rows of a request are kept as state between steps).
A query head has two query vectors of ``dim`` elements and its key head two key vectors: two
score maps ``scale * <q_m, k_m>`` over the same ``vdim`` values, each with its own softmax over
the keys the query sees (the last ``window`` positions, itself included; ``None``: all),

    o = a_1 - lam * a_2,   lam = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff,

then ``o`` is divided by its root mean square over the head (``eps`` inside the root, no weight)
and multiplied by ``1 - diff``; the output projection follows. Positions do not enter the scores.

A step in which every request brings one token, float32, and sizes the tensor-core kernel does not
take run the kernel for every size (``diff_attention.cu``); bfloat16 steps with portions of prompts
run the tiled tensor-core kernel (``diff_attention_mma.cu``).

The cache holds, per page slot and key head, a key row of ``2 * dim`` elements (both maps) and a
value row of ``vdim``; the convolution kernel appends them while it writes its outputs.

Sizes and constants are parameters: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``taps``, ``scale``,
``diff``, ``window``, ``eps``; ``names`` maps the roles ``q k v o q_conv k_conv v_conv lq1 lk1 lq2
lk2`` to the checkpoint's local tensor names.
"""

from __future__ import annotations

import math

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, PagedKVNeed, ParamSpec, StateNeed, register_mixer

DEFAULT_NAMES = {
    "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
    "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight",
    "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2", "lk2": "lambda_k2",
}


class DifferentialAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("differential attention keeps convolution state and cannot read another run's cache")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads = int(spec["heads"]), int(spec["kv_heads"])
        self.dim, self.vdim = int(spec["dim"]), int(spec["vdim"])
        self.taps = int(spec.get("taps", 1))
        self.scale = float(spec.get("scale", self.dim ** -0.5))
        self.diff = float(spec["diff"])
        self.eps = float(spec["eps"])
        window = spec.get("window")
        self.window = int(window) if window else None
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        if self.heads < 1 or self.kv_heads < 1 or self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"taps must be between 1 and 16, got {self.taps}")
        if not 1 <= self.vdim <= 256:
            raise ValueError(f"vdim must be between 1 and 256, got {self.vdim}")
        self.q_width = self.heads * 2 * self.dim
        self.k_width = self.kv_heads * 2 * self.dim
        self.v_width = self.kv_heads * self.vdim
        self.width = self.q_width + self.k_width + self.v_width
        self.lam = 0.0
        self.qkv: torch.Tensor | None = None
        self.conv: torch.Tensor | None = None
        self.out_w: torch.Tensor | None = None

    def cache_need(self):
        pages = PagedKVNeed(self.kv_heads, 2 * self.dim, self.window, value_dim=self.vdim)
        if self.taps == 1:
            return pages
        return pages, StateNeed((self.taps - 1, self.width), None)

    def scratch_per_token(self) -> int:
        return 2 * self.width + self.heads * self.vdim + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["q"], (self.q_width, h)), ParamSpec(n["k"], (self.k_width, h)), ParamSpec(n["v"], (self.v_width, h))]
        specs += [ParamSpec(n[role], (width, self.taps), role="gain", init="bias_normal")
                  for role, width in (("q_conv", self.q_width), ("k_conv", self.k_width), ("v_conv", self.v_width))]
        specs += [ParamSpec(n[role], (self.dim,), role="gain", init="bias_normal") for role in ("lq1", "lk1", "lq2", "lk2")]
        specs.append(ParamSpec(n["o"], (h, self.heads * self.vdim)))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.conv = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        self.out_w = tensors[n["o"]].contiguous()
        first = float((tensors[n["lq1"]].double() * tensors[n["lk1"]].double()).sum())
        second = float((tensors[n["lq2"]].double() * tensors[n["lk2"]].double()).sum())
        self.lam = math.exp(first) - math.exp(second) + self.diff

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        projected = ctx.buffer("diff_attn.qkv", (n, self.width))
        linear(x, self.qkv, projected, None, n, ctx)
        mixed = ctx.buffer("diff_attn.conv", (n, self.width))
        table = batch.block_tables[cache.group]
        append = dict(k_pages=cache.k_pages, v_pages=cache.v_pages, block_table=table, positions=batch.positions,
                      k_first=self.q_width, k_width=self.k_width, v_first=self.q_width + self.k_width, v_width=self.v_width)
        tail = cache.states[0] if self.taps > 1 else projected.new_empty((1, 0, self.width))
        kernels.causal_conv(projected, 0, self.conv, None, tail, mixed, batch.seq_of_token, batch.query_start_loc,
                            batch.state_slots, n, batch.num_seqs, silu=False, append=append, status=ctx.status)
        attended = ctx.buffer("diff_attn.attended", (n, self.heads * self.vdim))
        if batch.max_query_len > 1 and kernels.diff_attention_mma_takes(mixed.dtype, self.dim, self.vdim, self.scale):
            # portions of prompts in bfloat16: tiles of 64 positions on tensor cores
            kernels.diff_attention_mma(mixed, attended, cache.k_pages, cache.v_pages, table, batch.query_start_loc,
                                       batch.context_lens, n, batch.num_seqs, self.heads, self.kv_heads, self.dim, self.vdim,
                                       self.window, self.scale, self.lam, self.eps, 1.0 - self.diff, ctx.status)
        else:
            kernels.diff_attention(mixed, attended, cache.k_pages, cache.v_pages, table, batch.seq_of_token, batch.positions,
                                   n, self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.scale, self.lam,
                                   self.eps, 1.0 - self.diff, ctx.status)
        out = ctx.buffer("diff_attn.out", (n, self.hidden_size))
        linear(attended, self.out_w, out, None, n, ctx)
        return out


register_mixer("diff_attention", DifferentialAttention)
