"""Small Filezen configurations for the tests, model folders made from them, and the comparison rule.

Four configurations that differ from one another in every size and option: latent ranks of 16 to 160 (rows of
the cache that are and are not 16-byte aligned), rotated parts of 4 to 32 elements with and without frequency
scaling, windows that are no multiple of a page, a layer without a window, layers that read another layer's
rows with a larger and with a smaller window than the owner's, retention heads of 8 to 200 elements rotated in
part or in whole, one head and several, layers without a feed-forward, dense ones, and mixtures with and
without groups, with and without a shared expert, choosing one, some and all of their experts; embedding
scales and residual factors that are 1 and that are not.

``sharpen`` rewrites a folder so that faults which random weights would hide show up: queries are scaled up
until single scores stand out in the softmax (a key just inside or just outside a window, or hundreds of
positions back, then moves the output by a large part of it), and the retention decays are set close to 1, so
that a state lost or mixed up hundreds of tokens earlier still shows in the output.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, window, base, scaling=None, kv_from=None):
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=rot(base, rot_dim, scaling))
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return "latent_attention", mixer


def retention(heads, dim, vdim, decay, base, dims, scaling=None):
    return "retention", dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay), rot=rot(base, dims, scaling))


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(kind_and_mixer, mlp):
    return {"type": kind_and_mixer[0], "mixer": kind_and_mixer[1], "mlp": mlp}


CASE_A = {
    "architecture": "Filezen", "vocab": 190, "width": 96, "embedding": {"scale": 3.0}, "residual_mult": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        layer(latent(4, 24, 8, 20, 40, 0.2, 24, 5000.0, (4.0, 64, 16.0, 2.0)), moe(8, 2, 48, groups=(4, 2), shared=32)),
        layer(retention(3, 16, 24, (0.9, 0.97, 0.995), 10000.0, 8), dense(112)),
        layer(latent(2, 16, 8, 48, 40, 0.25, 40, 5000.0, (4.0, 64, 16.0, 2.0), kv_from=0), None),  # reads further back than its owner
        layer(retention(2, 40, 10, (0.95, 0.99), 500.0, 20), moe(6, 1, 40)),
    ],
}
CASE_B = {
    "architecture": "Filezen", "vocab": 140, "width": 64, "embedding": {"scale": 1.0}, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        layer(retention(1, 8, 64, (0.98,), 100.0, 8, (2.0, 32, 8.0, 1.0)), None),
        layer(latent(8, 8, 4, 8, 16, 0.3, None, 1000.0), moe(4, 4, 24, groups=(2, 2))),   # no window; every expert chosen
        layer(latent(5, 12, 4, 10, 16, 0.35, 17, 1000.0, kv_from=1), dense(72)),           # a window on rows kept for ever
        layer(latent(4, 16, 8, 24, 160, 0.2, 30, 20000.0, (16.0, 40, 4.0, 0.5)), moe(9, 3, 16, groups=(3, 1), shared=8)),
    ],
}
CASE_C = {
    "architecture": "Filezen", "vocab": 260, "width": 128, "embedding": {"scale": 7.5}, "residual_mult": 0.8, "norm": {"eps": 1e-5},
    "layers": [
        layer(latent(8, 32, 32, 16, 96, 0.12, 64, 10000.0, (6.0, 128, 24.0, 1.5)), moe(12, 3, 24, groups=(3, 2), shared=64)),
        layer(retention(4, 128, 32, (0.96, 0.98, 0.99, 0.999), 100000.0, 64), dense(96)),
        layer(latent(3, 20, 6, 28, 45, 0.22, 9, 300.0), moe(5, 2, 32, shared=16)),   # cache rows of 51 elements: not aligned
        layer(retention(2, 200, 12, (0.97, 0.9925), 10000.0, 100), None),
        layer(latent(6, 24, 32, 12, 96, 0.15, 20, 10000.0, (6.0, 128, 24.0, 1.5), kv_from=0), dense(40)),  # a shorter window than its owner
    ],
}
# everything odd: widths that are no multiple of 8, one head
CASE_D = {
    "architecture": "Filezen", "vocab": 77, "width": 100, "embedding": {"scale": 0.6}, "residual_mult": 1.3, "norm": {"eps": 1e-6},
    "layers": [
        layer(latent(1, 10, 2, 7, 18, 0.4, 5, 50.0), dense(52)),
        layer(retention(5, 6, 9, (0.9, 0.92, 0.94, 0.96, 0.98), 1000.0, 2), moe(3, 2, 20, shared=12)),
        layer(latent(3, 6, 10, 14, 18, 0.3, 33, 50.0), moe(4, 1, 12, groups=(4, 3))),
    ],
}
CASES = {"A": (CASE_A, 31), "B": (CASE_B, 32), "C": (CASE_C, 33), "D": (CASE_D, 34)}


def write_case(name: str, folder: Path, sharp: bool = False, steady: bool = False) -> Path:
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    raw, seed = CASES[name]
    if sharp:
        raw = json.loads(json.dumps(raw))
        for entry in raw["layers"]:
            if entry["type"] == "retention":
                heads = entry["mixer"]["heads"]
                entry["mixer"]["decay"] = [1.0 - 0.004 / (i + 1) for i in range(heads)]
    write_random_model(config_from_dict(raw), seed, folder, torch.bfloat16)
    if sharp:
        sharpen(folder)
    if steady:
        steady_routing(folder)
    return folder


def steady_routing(folder: Path) -> None:
    """Make every router's choice a plain function of the token, with wide margins.

    A choice among experts is a step function of the stream: where two scores nearly tie, rounding to bfloat16
    takes the other expert and the logits of that position (and, through states and cached rows, of later ones)
    move by far more than any tolerance, with nothing being wrong. Comparisons in bfloat16 therefore run on
    folders rewritten here: the first ``tags`` elements of the stream carry a code of the token (a permutation of
    0, 1, 2, ... per token), both norms' weights are zero there, so no sublayer ever adds to them, and every
    router reads expert ``e``'s logit from element ``e``. Scores then differ by a factor e between neighbours in
    rank: several experts keep a real share of the weight, groups are chosen and dropped, and no call is close.
    """
    from safetensors.torch import load_file, save_file

    config = read_config(folder)
    path = Path(folder) / "model.safetensors"
    tensors = load_file(str(path))
    tags = max([layer["mlp"]["router"]["experts"] for layer in config["layers"] if (layer.get("mlp") or {}).get("kind") == "moe"] or [0])
    if not tags:
        return
    g = torch.Generator().manual_seed(99)
    vocab = config["vocab"]
    code = torch.stack([torch.randperm(tags, generator=g) for _ in range(vocab)]).float() / float(config["embedding"]["scale"])
    embed = tensors["embed"].float()
    embed[:, :tags] = code
    tensors["embed"] = embed.to(torch.bfloat16)
    for name in list(tensors):
        if name.endswith(".norm1") or name.endswith(".norm2"):
            weight = tensors[name].float()
            weight[:tags] = 0.0
            tensors[name] = weight.to(torch.bfloat16)
        if name.endswith(".mlp.router"):
            router = torch.zeros_like(tensors[name].float())
            for e in range(router.shape[0]):
                router[e, e] = 1.0
            tensors[name] = router.to(torch.bfloat16)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata={"format": "pt"})


def sharpen(folder: Path) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(folder) / "model.safetensors"
    tensors = load_file(str(path))
    for name in list(tensors):
        if name.endswith(".mix.q") or name.endswith(".mix.uk"):
            tensors[name] = (tensors[name].float() * 4.0).to(torch.bfloat16)
        if name.endswith(".mlp.router"):
            tensors[name] = (tensors[name].float() * 3.0).to(torch.bfloat16)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata={"format": "pt"})


def read_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


FP32_REL = 3e-5
"""float32 engine against the float64 plain implementation: root mean square of the difference of a
position's logits (their mean taken off) over the root mean square of the plain logits of the
request. Every sum of the engine is float32."""

BF16_REL = 0.08
"""The same in bfloat16: activations are rounded to 8 bits of mantissa between kernels; statistics,
scores, states and the residual stream are float32. Every sublayer's output is normed to unit size before
it is added, so a rounding of 0.4 % in a small output weighs as much as in a large one; three to five layers
of that came to 0.01 to 0.06 on the first runs. A fault of the cache, a state or a window moves a position by
0.3 and more (``test_the_sharp_weights_do_make_single_rows_and_old_state_count``)."""


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
