"""The Filezen design in float64, written from its equations alone: one function per mechanism.

Nothing here is shared with the package: no kernels, no parts, no cache. A sequence is computed
whole, position by position where the design is a recurrence, so it is slow and plain.

Notation: ``h`` [T, width] is a sublayer's input, ``p`` the positions 0..T-1, weights are stored
``[out, in]`` and applied as ``h @ W.T``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotary_constants(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies of the pairs (i, i + dims / 2) and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    index = torch.arange(half, dtype=F64)
    freq = base ** (-2.0 * index / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = ((index - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    freq = freq / factor * ramp + freq * (1.0 - ramp)
    return freq, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """``x`` [T, heads, d]: the first ``dims`` of every head are rotated in pairs (i, i + dims / 2)."""
    dims = int(rot["dims"])
    half = dims // 2
    freq, factor = rotary_constants(rot)
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = (torch.cos(angle) * factor)[:, None, :], (torch.sin(angle) * factor)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def latent_cache(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """What a latent-attention layer with a down projection keeps per position: the normed latent
    and the rotated shared key part."""
    rank, rot_dim = int(sizes["kv_rank"]), int(sizes["rot_dim"])
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    positions = torch.arange(h.shape[0])
    shared = rotate(down[:, None, rank:rank + rot_dim], positions, sizes["rot"])[:, 0]
    return latent, shared


def window_softmax(scores: torch.Tensor, window: int | None) -> torch.Tensor:
    """``scores`` [..., T, T] (query, key): softmax over the keys a query sees, itself and the ``window - 1`` before it."""
    tokens = scores.shape[-1]
    positions = torch.arange(tokens)
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    if window:
        seen = seen & (distance < int(window))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)


def latent_attention(h: torch.Tensor, w: dict, sizes: dict, eps: float, kept: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    heads, dim, rot_dim, vdim = int(sizes["heads"]), int(sizes["dim"]), int(sizes["rot_dim"]), int(sizes["vdim"])
    latent, shared = kept
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    q = (h @ w["q"].T).reshape(tokens, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, sizes["rot"])
    keys = (latent @ w["uk"].T).reshape(tokens, heads, dim)
    values = (latent @ w["uv"].T).reshape(tokens, heads, vdim)
    scores = torch.einsum("thd,shd->hts", q_plain, keys) + torch.einsum("thr,sr->hts", q_rot, shared)
    weights = window_softmax(scores * float(sizes["scale"]), (sizes.get("mask") or {}).get("size"))
    mixed = torch.einsum("hts,shv->thv", weights, values).reshape(tokens, heads * vdim)
    return mixed @ w["o"].T


def decayed_sums(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """``S_t = decay S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head; q, k [T, heads, dim], v [T, heads, vdim]."""
    tokens, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F64)
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F64)
    for t in range(tokens):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    return out


def retention(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    heads, dim, vdim = int(sizes["heads"]), int(sizes["dim"]), int(sizes["vdim"])
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    q = rotate((h @ w["q"].T).reshape(tokens, heads, dim), positions, sizes["rot"])
    k = rotate((h @ w["k"].T).reshape(tokens, heads, dim), positions, sizes["rot"]) * dim ** -0.5
    v = (h @ w["v"].T).reshape(tokens, heads, vdim)
    out = decayed_sums(q, k, v, torch.tensor([float(d) for d in sizes["decay"]], dtype=F64))
    out = rms_norm(out, None, eps).reshape(tokens, heads * vdim)
    return (out * silu(h @ w["g"].T)) @ w["o"].T


def gated_expert(h: torch.Tensor, w: dict, prefix: str = "") -> torch.Tensor:
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h: torch.Tensor, router: torch.Tensor, sizes: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [T, top] and their weights."""
    experts, top = int(sizes["experts"]), int(sizes["top"])
    scores = torch.softmax(h @ router.T, dim=-1)
    allowed = scores.clone()
    groups = sizes.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = experts // count
        best = scores.reshape(-1, count, per).max(dim=-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = allowed.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    chosen = allowed.topk(top, dim=-1).indices
    picked = scores.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def mixture(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    chosen, weights = route(h, w["router"], mlp["router"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] += g * gated_expert(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, "shared.")
    return out


def feed_forward(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    return gated_expert(h, w) if mlp["kind"] == "dense" else mixture(h, w, mlp)


def part(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t.to(F64) for name, t in weights.items() if name.startswith(prefix)}


def forward(config: dict, weights: dict, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [T, vocab] and the stream after every layer [layers, T, width]."""
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    embed = weights["embed"].to(F64)
    x = embed[torch.tensor(tokens)] * float(config["embedding"]["scale"])
    kept: dict[int, tuple] = {}
    after = []
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        w, sizes = part(weights, name + "mix."), layer["mixer"]
        if layer["type"] == "latent_attention":
            source = sizes.get("kv_from")
            if source is None:
                kept[index] = latent_cache(x, w, sizes, eps)
                source = index
            mixed = latent_attention(x, w, sizes, eps, kept[int(source)])
        elif layer["type"] == "retention":
            mixed = retention(x, w, sizes, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(mixed, weights[name + "norm1"].to(F64), eps)
        if layer.get("mlp"):
            moved = feed_forward(x, part(weights, name + "mlp."), layer["mlp"])
            x = x + mult * rms_norm(moved, weights[name + "norm2"].to(F64), eps)
        after.append(x)
    final = rms_norm(x, weights["final.norm"].to(F64), eps)
    return final @ embed.T, torch.stack(after)


def logits_of(config: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    return forward(config, weights, tokens)[0]


def greedy(config: dict, weights: dict, prompt: list[int], count: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(logits_of(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


def read_model_folder(folder):
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))
