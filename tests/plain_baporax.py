"""A plain, slow Baporax: every mechanism of the design as one small function, in float64 on the CPU.

It reads the same ``config.json`` mapping and the same tensor names as the engine, and shares no
code with it. Sequences are whole: ``forward(config, weights, ids)`` returns the logits of every
position and, if asked, the residual stream after every layer run.

Mechanisms (``h`` is a layer's input, rows are positions ``0 .. T-1``):

* ``zero_centred_rms_norm``: ``h / sqrt(mean(h^2) + eps) * (1 + w)``.
* ``causal_taps``: ``y[t, c] = sum_j w[c, j] * u[t - (J - 1) + j, c]`` with ``u`` zero before the
  sequence starts (``J`` taps, the last tap is the current position's), plus a bias if given.
* ``squared_relu_ff``: ``W_down max(W_up h, 0)^2``.
* ``differential_window_attention``: two score maps per head over the same values, softmax each
  over the last ``window`` positions, ``a1 - lam * a2``, unit RMS per head, times ``1 - diff``.
* ``ssd_recurrence``: the scalar-decay state space recurrence per head,
  ``S <- exp(-exp(A) dt) S + dt B x^T``, ``y = S^T C + D x``, followed by the gate, the grouped RMS
  norm and the output projection in ``state_space_mixer``.
* ``layer``: both branches read the same input, ``h + mixer(norm1 h) + ff(norm2 h)``.
* ``forward``: embedding, the looped stretch of layers (a learned vector added before each pass),
  the rest, the final norm, and the tied head times ``logit_scale``.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def zero_centred_rms_norm(h, w, eps):
    return h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * (1.0 + w)


def causal_taps(u, w, bias=None):
    """``u`` [T, C], ``w`` [C, J]; the last column of ``w`` multiplies the current position."""
    T, C = u.shape
    J = w.shape[1]
    padded = torch.cat([torch.zeros(J - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros(T, C, dtype=u.dtype)
    for j in range(J):
        y = y + padded[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def squared_relu_ff(h, up, down):
    a = torch.clamp(h @ up.T, min=0.0)
    return (a * a) @ down.T


def differential_maps(q, k, v, scale, window, lam, diff, eps):
    """``q`` [T, H, 2, d], ``k`` [T, G, 2, d], ``v`` [T, G, dv] of one whole sequence -> [T, H, dv]."""
    T, H = q.shape[0], q.shape[1]
    G, dv = k.shape[1], v.shape[-1]
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for m in range(2):
            s = (q[:, head, m] @ k[:, g, m].T) * scale
            s = s.masked_fill(~seen, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
        out[:, head] = o * (1.0 - diff)
    return out


def differential_lambda(w, diff):
    return math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff


def differential_window_attention(h, p, w, eps):
    """``p``: the mixer's mapping of the configuration; ``w``: its tensors by local name."""
    T = h.shape[0]
    H, G, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    window = (p.get("mask") or {}).get("size")
    q = causal_taps(h @ w["q"].T, w["q.conv"]).view(T, H, 2, d)
    k = causal_taps(h @ w["k"].T, w["k.conv"]).view(T, G, 2, d)
    v = causal_taps(h @ w["v"].T, w["v.conv"]).view(T, G, dv)
    out = differential_maps(q, k, v, p["scale"], window, differential_lambda(w, p["diff"]), p["diff"], eps)
    return out.reshape(T, H * dv) @ w["o"].T


def ssd_recurrence(x, B, C, dt, A_log, D, groups):
    """``x`` [T, heads, P], ``B``/``C`` [T, groups, N], ``dt`` [T, heads] (already positive)."""
    T, heads, P = x.shape
    N = B.shape[-1]
    y = torch.zeros(T, heads, P, dtype=x.dtype)
    for head in range(heads):
        g = head // (heads // groups)
        S = torch.zeros(N, P, dtype=x.dtype)
        rate = torch.exp(A_log[head])
        for t in range(T):
            S = torch.exp(-rate * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + D[head] * x[t, head]
    return y


def state_space_mixer(h, p, w, eps):
    T = h.shape[0]
    heads, P, N, G = p["heads"], p["vdim"], p["state"], p["groups"]
    inner = heads * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_taps(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = ssd_recurrence(x, B, C, dt, w["A_log"], w["D"], G).reshape(T, inner)
    y = y * silu(z)
    parts = p["norm_groups"]
    y = y.view(T, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (y.reshape(T, inner) * w["norm"]) @ w["o"].T


MIXERS = {"attention": differential_window_attention, "mamba2": state_space_mixer}


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(h, spec, weights, index, eps):
    mixed = MIXERS[spec["type"]](zero_centred_rms_norm(h, weights[f"l{index}.norm1"], eps), spec["mixer"],
                                 sub(weights, f"l{index}.mix."), eps)
    out = h + mixed
    if spec.get("mlp"):
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        out = out + squared_relu_ff(zero_centred_rms_norm(h, weights[f"l{index}.norm2"], eps),
                                    weights[f"l{index}.mlp.up"], weights[f"l{index}.mlp.down"])
    return out


def run_order(config):
    """(layer index, pass number or None): which layers run in which order."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["times"] < 1 or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    order += [(i, None) for i in range(loop["stop"], n)]
    return order


def read_model_folder(folder):
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def greedy(config, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


def forward(config, weights, ids, trace=None):
    weights = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    h = weights["embed"][torch.tensor(list(ids))]
    for index, step in run_order(config):
        if step is not None:
            h = h + weights["loop.step"][step]
        h = layer(h, config["layers"][index], weights, index, eps)
        if trace is not None:
            trace.append(h.clone())
    return zero_centred_rms_norm(h, weights["final.norm"], eps) @ weights["embed"].T * config["logit_scale"]
