"""Typed configuration of the Filezen decoder, read from its ``config.json``.

Filezen is a small hybrid decoder. Every layer has one mixer, either latent attention with a sliding window
(``"latent_attention"``: keys and values of all heads come from one cached latent per position plus one
shared rotated key part; a layer may read the rows another layer caches, ``kv_from``) or retention
(``"retention"``: linear attention with a fixed decay per head and a float32 state per request), and
optionally a feed-forward that is dense and gated or a mixture of experts with a shared expert. The norms
stand behind the sublayers: ``x += m * norm1(mixer(x))``, ``x += m * norm2(ff(x))``, the sublayers reading ``x``
itself. The embedding is scaled; the head is the embedding table, unscaled.

Keys of ``config.json``: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``residual_mult``, ``norm.eps``
and ``layers``: a list of ``{"type", "mixer", "mlp"}``. Latent attention: ``heads dim rot_dim vdim kv_rank scale
mask.size rot{base dims scaling{factor original fast slow}} [kv_from]``; retention: ``heads dim vdim decay[]
rot{base dims}``; ``mlp``: ``null``, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert.ff", "router{experts top
groups{count keep}}", "shared.ff"}``. Tensor names: ``embed``, ``final.norm`` and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}`` or ``l<i>.mix.{q,k,v,g,o}``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router, e<j>.gate|up|down, shared.gate|up|down}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerRun, LayerSpec, ModelSpec, PartSpec, TensorNames

ARCHITECTURE = "Filezen"

LATENT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
RETENTION_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}
MOE_NAMES = {"router": "router", "expert": "e{index}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}


class FilezenConfigError(ValueError):
    """``config.json`` asks for something the design does not have."""


def _positive(value: Any, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) < 1:
        raise FilezenConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


def _window(mixer: Mapping[str, Any]) -> int | None:
    size = (mixer.get("mask") or {}).get("size")
    return int(size) if size else None


@dataclass(frozen=True)
class FilezenConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    eps: float
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    max_position_embeddings: int = 1 << 20
    initializer_range: float = 0.05
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)
    architecture: str = ARCHITECTURE

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FilezenConfig":
        try:
            layers = data["layers"]
            vocab, width = _positive(data["vocab"], "vocab"), _positive(data["width"], "width")
            eps = float(data["norm"]["eps"])
        except (KeyError, TypeError) as exc:
            raise FilezenConfigError(f"config.json lacks {exc}") from None
        if not isinstance(layers, (list, tuple)) or not layers:
            raise FilezenConfigError("'layers' must be a non-empty list")
        checked = []
        for index, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in ("latent_attention", "retention") or not isinstance(mixer, Mapping):
                raise FilezenConfigError(f"layer {index}: unknown mixer type {kind!r}")
            required = (("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale") if kind == "latent_attention"
                        else ("heads", "dim", "vdim", "decay"))
            if kind == "latent_attention" and mixer.get("rot_dim") and "rot" not in mixer:
                raise FilezenConfigError(f"layer {index}: a rotated part of {mixer['rot_dim']} elements needs 'rot'")
            for key in required:
                if key not in mixer:
                    raise FilezenConfigError(f"layer {index}: the {kind} mixer lacks {key!r}")
            if kind == "retention" and len(mixer["decay"]) != mixer["heads"]:
                raise FilezenConfigError(f"layer {index}: {len(mixer['decay'])} decays for {mixer['heads']} heads")
            source = mixer.get("kv_from") if kind == "latent_attention" else None
            if source is not None:
                other = layers[source] if isinstance(source, int) and 0 <= source < index else None
                if other is None or other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                    raise FilezenConfigError(f"layer {index}: kv_from must name an earlier latent attention layer with a cache of its own")
                if any(other["mixer"].get(key) != mixer.get(key) for key in ("kv_rank", "rot_dim", "rot")):
                    raise FilezenConfigError(f"layer {index}: kv_rank, rot_dim and rot must equal those of layer {source}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    _positive(mlp.get("ff"), f"layer {index}: mlp.ff")
                elif mlp.get("kind") == "moe":
                    try:
                        _positive(mlp["expert"]["ff"], f"layer {index}: mlp.expert.ff")
                        _positive(mlp["router"]["experts"], f"layer {index}: mlp.router.experts")
                        _positive(mlp["router"]["top"], f"layer {index}: mlp.router.top")
                    except (KeyError, TypeError) as exc:
                        raise FilezenConfigError(f"layer {index}: the mixture of experts lacks {exc}") from None
                else:
                    raise FilezenConfigError(f"layer {index}: unknown feed-forward {mlp!r}")
            checked.append(copy.deepcopy(dict(layer)))
        known = {"architecture", "architectures", "vocab", "width", "layers", "norm", "embedding", "residual_mult",
                 "max_position_embeddings", "initializer_range", "torch_dtype"}
        return cls(vocab=vocab, width=width, layers=tuple(checked), eps=eps,
                   embedding_scale=float((data.get("embedding") or {}).get("scale", 1.0)),
                   residual_mult=float(data.get("residual_mult", 1.0)),
                   max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)),
                   initializer_range=float(data.get("initializer_range", 0.05)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        return {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
            "layers": copy.deepcopy([dict(layer) for layer in self.layers]), "norm": {"eps": self.eps},
            "max_position_embeddings": self.max_position_embeddings, "initializer_range": self.initializer_range,
        }

    # -- translation ----------------------------------------------------------------------------

    def kept_windows(self) -> dict[int, int | None]:
        """For every latent attention layer that caches rows: the window those rows are kept for, the largest of
        its own and of the layers that read them (``None``: everything)."""
        kept: dict[int, int | None] = {}
        for index, layer in enumerate(self.layers):
            if layer["type"] != "latent_attention":
                continue
            owner = layer["mixer"].get("kv_from")
            owner = index if owner is None else int(owner)
            window = _window(layer["mixer"])
            if owner not in kept:
                kept[owner] = window
            elif kept[owner] is not None:
                kept[owner] = None if window is None else max(kept[owner], window)
        return kept

    def run_order(self) -> tuple[LayerRun, ...]:
        """Every layer once; a layer with ``kv_from`` reads the cache of that layer's run."""
        runs = []
        for index, layer in enumerate(self.layers):
            source = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            runs.append(LayerRun(index, cache_from=None if source is None else int(source)))
        return tuple(runs)

    def _mixer(self, index: int, layer: Mapping[str, Any], kept: Mapping[int, int | None]) -> PartSpec:
        sizes = layer["mixer"]
        if layer["type"] == "latent_attention":
            owner = sizes.get("kv_from")
            owner = index if owner is None else int(owner)
            return PartSpec("latent_attention", dict(
                heads=sizes["heads"], dim=sizes["dim"], rot_dim=sizes["rot_dim"], vdim=sizes["vdim"], kv_rank=sizes["kv_rank"],
                scale=sizes["scale"], window=_window(sizes), cache_window=kept[owner], eps=self.eps,
                rot=copy.deepcopy(dict(sizes.get("rot") or {})), names=LATENT_NAMES))
        return PartSpec("retention", dict(
            heads=sizes["heads"], dim=sizes["dim"], vdim=sizes["vdim"], decay=tuple(float(d) for d in sizes["decay"]),
            rot=copy.deepcopy(dict(sizes.get("rot") or {})), eps=self.eps, names=RETENTION_NAMES))

    @staticmethod
    def _feed_forward(mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", dict(intermediate_size=mlp["ff"], activation="silu", names=DENSE_NAMES))
        router = mlp["router"]
        groups = router.get("groups") or {}
        shared = (mlp.get("shared") or {}).get("ff")
        return PartSpec("routed_experts", dict(
            experts=router["experts"], top=router["top"], groups=groups.get("count", 1), keep=groups.get("keep", groups.get("count", 1)),
            intermediate_size=mlp["expert"]["ff"], shared=shared, activation="silu", names=MOE_NAMES))

    def to_model_spec(self) -> ModelSpec:
        kept = self.kept_windows()
        layers, unused = [], []
        for index, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            feed_forward = ff_norm = None
            if mlp is None:
                unused.append(f"l{index}.norm2")  # a layer without a feed-forward has no use for a second norm
            else:
                feed_forward = self._feed_forward(mlp)
                ff_norm = PartSpec("rms_norm", dict(eps=self.eps, tensor="norm2"))
            layers.append(LayerSpec(
                mixer=self._mixer(index, layer, kept), feed_forward=feed_forward,
                mixer_norm=PartSpec("rms_norm", dict(eps=self.eps, tensor="norm1")), feed_forward_norm=ff_norm,
                position=None, block="output_norm", block_params=dict(residual_mult=self.residual_mult)))
        names = TensorNames(embedding="", head="head.", final_norm="final.", layer="l{index}.", mixer="mix.",
                            feed_forward="mlp.", mixer_norm="", feed_forward_norm="", prefix_rewrites=())
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            order=self.run_order(), final_norm=PartSpec("rms_norm", dict(eps=self.eps, tensor="norm")),
            embedding=PartSpec("table", dict(tensor="embed", scale=self.embedding_scale)), head=PartSpec("linear"),
            tie_word_embeddings=True, names=names, optional_tensors=tuple(unused), eos_token_ids=(),
            max_position_embeddings=self.max_position_embeddings, init_std=self.initializer_range)
