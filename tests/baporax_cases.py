"""Small Baporax configurations for the tests, model folders made from them, and the comparison rule.

Five configurations that differ from one another in every size and option: numbers of heads and
groups, key sizes whose double is and is not the value size, one and several taps, windows that are
no multiple of a page, a layer without a window, a layer without a feed-forward, a looped stretch
that starts after the first layer and runs three times, one that runs once, and no loop at all.

``sharpen`` rewrites a folder's weights so that faults which random weights would hide show up:
queries and keys are scaled up until single scores stand out in the softmax (a key just inside
or just outside a window, or hundreds of positions back, then moves the output by a large part of
it), and the state-space decay is made slow, so that a state lost or mixed up hundreds of tokens
earlier still shows in the output.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, conv, diff, scale, window):
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, diff=diff, scale=scale)
    if window is not None:
        mixer["mask"] = {"size": window}
    return mixer


def mamba2(heads, vdim, state, groups, norm_groups, conv):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CASE_X = {
    "architecture": "Baporax", "vocab": 200, "width": 96, "logit_scale": 0.5, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        layer("mamba2", mamba2(4, 24, 16, 1, 4, 3), 128),
        layer("attention", attention(6, 2, 16, 40, 2, 0.3, 0.2, 24), 160),
        layer("attention", attention(2, 2, 24, 32, 4, 0.6, 0.15, None), None),
        layer("mamba2", mamba2(6, 16, 48, 3, 1, 4), 64),
    ],
}
CASE_Y = {
    "architecture": "Baporax", "vocab": 130, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", attention(4, 1, 8, 96, 1, 0.8, 0.35, 17), 96),
        layer("mamba2", mamba2(2, 40, 24, 2, 2, 5), None),
    ],
}
CASE_Z = {
    "architecture": "Baporax", "vocab": 310, "width": 128, "logit_scale": 2.0, "norm": {"eps": 1e-5},
    "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        layer("mamba2", mamba2(4, 64, 128, 1, 2, 2), 192),
        layer("attention", attention(8, 2, 64, 128, 3, 0.4, 0.125, 64), 256),
    ],
}
# widths that are no multiple of 8 (rows that are not 16-byte aligned), three query heads on one key head, odd everything
CASE_W = {
    "architecture": "Baporax", "vocab": 77, "width": 100, "logit_scale": 0.7, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 2, "times": 2},
    "layers": [
        layer("attention", attention(3, 1, 12, 20, 3, 0.25, 0.3, 10), 90),
        layer("mamba2", mamba2(3, 10, 12, 1, 3, 2), 52),
        layer("attention", attention(5, 5, 6, 7, 2, 0.5, 0.4, 33), None),
    ],
}
# a loop over three of five layers that holds both kinds of mixer; keys twice as long as values, eight query
# heads on one key head, values wider than 128, as many groups as heads, a state of 8
CASE_V = {
    "architecture": "Baporax", "vocab": 97, "width": 160, "logit_scale": 1.5, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 4, "times": 2},
    "layers": [
        layer("mamba2", mamba2(4, 32, 64, 4, 4, 2), 96),
        layer("attention", attention(2, 2, 128, 64, 2, 0.2, 0.09, 40), 224),
        layer("mamba2", mamba2(2, 80, 8, 2, 1, 4), None),
        layer("attention", attention(8, 1, 16, 32, 4, 0.7, 0.25, None), 64),
        layer("attention", attention(4, 2, 32, 160, 1, 0.45, 0.18, 70), 128),
    ],
}
CASES = {"X": (CASE_X, 21), "Y": (CASE_Y, 22), "Z": (CASE_Z, 23), "W": (CASE_W, 24), "V": (CASE_V, 25)}


def write_case(name: str, folder: Path, sharp: bool = False) -> Path:
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    raw, seed = CASES[name]
    write_random_model(config_from_dict(raw), seed, folder, torch.bfloat16)
    if sharp:
        sharpen(folder)
    return folder


def sharpen(folder: Path) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(folder) / "model.safetensors"
    tensors = load_file(str(path))
    for name in list(tensors):
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            tensors[name] = (tensors[name].float() * 5.0).to(torch.bfloat16)
        if name.endswith(".mix.A_log"):
            tensors[name] = torch.full_like(tensors[name], -4.0)  # decay per step about exp(-0.013)
        if name.endswith(".mix.lq1") or name.endswith(".mix.lk1"):
            tensors[name] = (tensors[name].float() * 8.0).to(torch.bfloat16)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata={"format": "pt"})


def read_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


FP32_REL = 2e-5
"""float32 engine against the float64 plain implementation: root mean square of the difference of a
position's logits (their mean taken off) over the root mean square of the plain logits of the
request. Every sum of the engine is float32; observed values are a few 1e-7 to a few 1e-6."""

BF16_REL = 0.03
"""The same in bfloat16: activations are rounded to 8 bits of mantissa between kernels, statistics,
scores, states and the residual stream are float32."""


def relative_error(ours: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: rms over the vocabulary of (ours - ref), mean taken off, over the rms of ref."""
    diff = ours.double() - ref.double()
    diff = diff - diff.mean(-1, keepdim=True)
    centred = ref.double() - ref.double().mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / centred.pow(2).mean().sqrt()


def check(ours: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, slack: float = 1.0) -> None:
    assert ours.shape == ref.shape, f"{what}: shape {tuple(ours.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(ours).all(), f"{what}: non-finite logits"
    error = relative_error(ours, ref)
    bound = (FP32_REL if dtype == "float32" else BF16_REL) * slack
    worst = float(error.max())
    assert worst <= bound, f"{what}: relative error {worst:.3e} at position {int(error.argmax())} (bound {bound:.1e})"
