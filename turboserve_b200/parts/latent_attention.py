"""Latent attention: keys and values of all heads are made from one small latent per position.

Per token, with ``h`` the mixer's input: ``q = Wq h`` holds, head by head, ``dim`` plain and ``rot_dim``
rotated query elements. ``Wdkv h`` gives ``kv_rank + rot_dim`` numbers: the first ``kv_rank``, RMS-normed
with a weight, are the latent ``c``; the last ``rot_dim`` are one rotated key part ``r`` that all heads
share. A head's key is ``[Wuk_h c | r]``, its value ``Wuv_h c``; the score of key ``j`` is
``(q_plain . Wuk_h c_j + q_rot . r_j) * scale`` over the last ``window`` positions (itself included;
``None``: all), softmax, then the output projection on the heads' values side by side. Only ``c`` and ``r``
(after rotation) are cached: a page row is ``[c | r]``.

Keys and values are never formed. The query is carried into the latent space instead,
``q~ = Wuk_h^T q_plain``, so that a score is ``q~ . c_j + q_rot . r_j``, the softmax-weighted sum is taken
over the latents themselves and ``Wuv_h`` is applied to that sum: the attention kernel reads ``kv_rank +
rot_dim`` numbers per key for all heads together, in prompts and in decoding alike.

The rotation acts on pairs ``(i, i + rot_dim / 2)`` with frequencies from ``rot`` (``base``, ``dims``, optional
``scaling``: see :func:`~turboserve_b200.parts.rope.scaled_rotary_frequencies`); ``scale`` is used as given.

With ``shares_cache`` the mixer has no ``Wdkv`` and attends over the rows another run writes, with its own
queries, ``Wuk``, ``Wuv`` and window; ``cache_window`` is then the window the shared pages are kept for (the
largest of the runs that read them; ``None`` keeps everything).

Sizes and constants are parameters: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``window``,
``cache_window``, ``eps``, ``rot``; ``names`` maps the roles ``q dkv dkv_norm uk uv o`` to the checkpoint's names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, PagedKVNeed, ParamSpec, register_mixer
from .rope import scaled_rotary_frequencies

DEFAULT_NAMES = {"q": "q_proj.weight", "dkv": "kv_down_proj.weight", "dkv_norm": "kv_norm.weight",
                 "uk": "k_up_proj.weight", "uv": "v_up_proj.weight", "o": "o_proj.weight"}
_UNSET = object()


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        self.hidden_size = int(hidden_size)
        self.heads, self.dim, self.rot_dim = int(spec["heads"]), int(spec["dim"]), int(spec["rot_dim"])
        self.vdim, self.rank = int(spec["vdim"]), int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        window = spec.get("window")
        self.window = int(window) if window else None
        kept = spec.get("cache_window", _UNSET)
        self.cache_window = self.window if kept is _UNSET else (int(kept) if kept else None)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError("the window of a latent attention reaches beyond what its cache keeps")
        self.shares_cache = bool(shares_cache)
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        rot = dict(spec.get("rot") or {})
        if self.heads < 1 or self.dim < 1 or self.vdim < 1 or not 1 <= self.rank <= 512:
            raise ValueError("latent attention needs heads, dim, vdim >= 1 and a kv_rank between 1 and 512")
        if self.rot_dim % 2 or self.rot_dim < 0 or (self.rot_dim and int(rot.get("dims", self.rot_dim)) != self.rot_dim):
            raise ValueError("rot_dim must be even and the rotation must cover all of it")
        if self.rot_dim:
            freq, self.amplitude = scaled_rotary_frequencies(self.rot_dim, float(rot["base"]), rot.get("scaling"))
            self.inv_freq = freq.to(device)
        else:
            self.inv_freq, self.amplitude = torch.zeros(0, dtype=torch.float32, device=device), 1.0
        self.q_head = self.dim + self.rot_dim
        self.q_width = self.heads * self.q_head
        self.row = self.rank + self.rot_dim
        self.proj_width = self.q_width + (0 if self.shares_cache else self.row)
        for name in ("proj", "norm_w", "uk_t", "uv", "out_w"):
            setattr(self, name, None)

    def cache_need(self) -> PagedKVNeed:
        # one row [c | r] per position, shared by all heads; the value of a key is the row's first kv_rank elements
        return PagedKVNeed(1, self.row, self.cache_window, value_dim=0)

    def scratch_per_token(self) -> int:
        return self.proj_width + 2 * self.heads * self.rank + self.heads * self.vdim + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["q"], (self.q_width, h))]
        if not self.shares_cache:
            specs += [ParamSpec(n["dkv"], (self.row, h)), ParamSpec(n["dkv_norm"], (self.rank,), role="gain", init="one_plus_normal")]
        specs += [ParamSpec(n["uk"], (self.heads * self.dim, self.rank)), ParamSpec(n["uv"], (self.heads * self.vdim, self.rank)),
                  ParamSpec(n["o"], (h, self.heads * self.vdim))]
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        if self.shares_cache:
            self.proj = tensors[n["q"]].contiguous()
        else:
            self.proj = torch.cat([tensors[n["q"]], tensors[n["dkv"]]], dim=0).contiguous()
            self.norm_w = tensors[n["dkv_norm"]].contiguous()
        # [heads, rank, dim]: a head's rows are the columns of its Wuk, so that q~ = Wuk^T q_plain is a product by rows
        self.uk_t = tensors[n["uk"]].reshape(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].reshape(self.heads, self.vdim, self.rank).contiguous()
        self.out_w = tensors[n["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        table = batch.block_tables[cache.group]
        projected = ctx.buffer("latent_attn.proj", (n, self.proj_width))
        linear(x, self.proj, projected, None, n, ctx)
        down = None if self.shares_cache else projected[:, self.q_width:]
        kernels.latent_prepare(projected, down, self.norm_w, self.inv_freq, self.amplitude, batch.positions,
                               batch.seq_of_token, table, cache.k_pages, n, self.heads, self.dim, self.rot_dim, self.rank,
                               self.eps, ctx.status)
        carried = ctx.buffer("latent_attn.q", (n, self.heads * self.rank))
        kernels.head_linear(projected, self.q_head, self.uk_t, carried, self.rank, n)
        mixed = ctx.buffer("latent_attn.mixed", (n, self.heads * self.rank))
        kernels.latent_attention(carried, projected[:, self.dim:], self.q_head, mixed, cache.k_pages, table,
                                 batch.seq_of_token, batch.positions, n, self.heads, self.rank, self.rot_dim, self.window,
                                 self.scale, ctx.status)
        values = ctx.buffer("latent_attn.values", (n, self.heads * self.vdim))
        kernels.head_linear(mixed, self.rank, self.uv, values, self.vdim, n)
        out = ctx.buffer("latent_attn.out", (n, self.hidden_size))
        linear(values, self.out_w, out, None, n, ctx)
        return out


register_mixer("latent_attention", LatentAttention)
