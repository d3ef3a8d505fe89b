"""Typed configuration of the Baporax decoder, read from its ``config.json``.

Baporax is a small hybrid decoder: every layer has one mixer, either differential sliding-window
attention with short convolutions on q, k and v (``"attention"``) or a Mamba-2 state-space
mixer (``"mamba2"``), and optionally a dense squared-relu feed-forward; mixer and feed-forward
read the same input (two zero-centred RMS norms) and are added to the stream together. A stretch
of layers (``loop``) is run several times with the same weights, each pass with caches and states
of its own and a learned vector added to the stream before it. The head is the embedding table
times ``logit_scale``.

Keys of ``config.json``: ``architecture``, ``vocab``, ``width``, ``logit_scale``, ``norm.eps``,
``loop`` (``start``, ``stop``, ``times``), and ``layers``: a list of ``{"type", "mixer", "mlp"}``
with the mixer's sizes (attention: ``heads kv_heads dim vdim conv diff scale mask.size``;
mamba2: ``heads vdim state groups norm_groups conv``) and ``mlp`` either ``null`` or
``{"kind": "dense", "ff"}``. Tensor names: ``embed``, ``loop.step``, ``final.norm``, and per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up``, ``l<i>.mlp.down``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerRun, LayerSpec, ModelSpec, PartSpec, TensorNames

ARCHITECTURE = "Baporax"

ATTENTION_NAMES = {
    "q": "q", "k": "k", "v": "v", "o": "o", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
    "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2",
}
MAMBA2_NAMES = {
    "in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D",
    "norm": "norm", "out": "o",
}


class BaporaxConfigError(ValueError):
    """``config.json`` asks for something the design does not have."""


def _positive(value: Any, what: str) -> int:
    number = int(value)
    if number < 1 or number != value:
        raise BaporaxConfigError(f"{what} must be a positive integer, got {value!r}")
    return number


@dataclass(frozen=True)
class BaporaxConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    eps: float
    logit_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
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

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start and self.loop_times >= 1

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BaporaxConfig":
        try:
            layers = data["layers"]
            vocab, width = _positive(data["vocab"], "vocab"), _positive(data["width"], "width")
            eps = float(data["norm"]["eps"])
        except (KeyError, TypeError) as exc:
            raise BaporaxConfigError(f"config.json lacks {exc}") from None
        if not isinstance(layers, (list, tuple)) or not layers:
            raise BaporaxConfigError("'layers' must be a non-empty list")
        checked = []
        for index, layer in enumerate(layers):
            kind = layer.get("type")
            mixer = layer.get("mixer")
            if kind not in ("attention", "mamba2") or not isinstance(mixer, Mapping):
                raise BaporaxConfigError(f"layer {index}: unknown mixer type {kind!r}")
            required = (("heads", "kv_heads", "dim", "vdim", "diff", "scale") if kind == "attention"
                        else ("heads", "vdim", "state", "groups", "norm_groups"))
            for key in required:
                if key not in mixer:
                    raise BaporaxConfigError(f"layer {index}: the {kind} mixer lacks {key!r}")
            mlp = layer.get("mlp")
            if mlp is not None and (mlp.get("kind") != "dense" or "ff" not in mlp):
                raise BaporaxConfigError(f"layer {index}: unknown feed-forward {mlp!r}")
            checked.append(copy.deepcopy(dict(layer)))
        loop = data.get("loop") or {}
        start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if loop and not (0 <= start <= stop <= len(checked) and times >= 1):
            raise BaporaxConfigError(f"loop {dict(loop)!r} does not fit {len(checked)} layers")
        known = {"architecture", "architectures", "vocab", "width", "layers", "norm", "logit_scale", "loop",
                 "max_position_embeddings", "initializer_range", "torch_dtype"}
        return cls(vocab=vocab, width=width, layers=tuple(checked), eps=eps, logit_scale=float(data.get("logit_scale", 1.0)),
                   loop_start=start, loop_stop=stop, loop_times=times,
                   max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)),
                   initializer_range=float(data.get("initializer_range", 0.05)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "layers": copy.deepcopy([dict(layer) for layer in self.layers]), "norm": {"eps": self.eps},
            "logit_scale": self.logit_scale,
            "max_position_embeddings": self.max_position_embeddings, "initializer_range": self.initializer_range,
        }
        if self.has_loop:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    # -- translation ----------------------------------------------------------------------------

    def run_order(self) -> tuple[LayerRun, ...]:
        """Every layer once, but the looped stretch ``times`` times in a row; each run owns its cache
        and the first run of a pass names the pass's row of the shift table."""
        count = len(self.layers)
        if not self.has_loop:
            return ModelSpec.sequential(count)
        runs = [LayerRun(i) for i in range(self.loop_start)]
        for pass_index in range(self.loop_times):
            for i in range(self.loop_start, self.loop_stop):
                runs.append(LayerRun(i, shift=pass_index if i == self.loop_start else None))
        runs += [LayerRun(i) for i in range(self.loop_stop, count)]
        return tuple(runs)

    def _mixer(self, kind: str, sizes: Mapping[str, Any]) -> PartSpec:
        if kind == "attention":
            window = (sizes.get("mask") or {}).get("size")
            return PartSpec("diff_attention", dict(
                heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"], vdim=sizes["vdim"],
                taps=sizes.get("conv", 1), diff=sizes["diff"], scale=sizes["scale"], window=window, eps=self.eps,
                names=ATTENTION_NAMES))
        return PartSpec("mamba2", dict(
            heads=sizes["heads"], vdim=sizes["vdim"], state=sizes["state"], groups=sizes["groups"],
            norm_groups=sizes["norm_groups"], taps=sizes.get("conv", 1), eps=self.eps, names=MAMBA2_NAMES))

    def to_model_spec(self) -> ModelSpec:
        layers = []
        unused = []  # a layer without a feed-forward has no use for a second norm, should the checkpoint hold one
        for index, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            feed_forward = ff_norm = None
            if mlp is None:
                unused.append(f"l{index}.norm2")
            if mlp is not None:
                feed_forward = PartSpec("dense_mlp", dict(intermediate_size=mlp["ff"], activation="relu2", up="up", down="down"))
                ff_norm = PartSpec("rms_norm", dict(eps=self.eps, zero_centred=True, tensor="norm2"))
            layers.append(LayerSpec(
                mixer=self._mixer(layer["type"], layer["mixer"]), feed_forward=feed_forward,
                mixer_norm=PartSpec("rms_norm", dict(eps=self.eps, zero_centred=True, tensor="norm1")),
                feed_forward_norm=ff_norm, position=None, block="parallel"))
        names = TensorNames(embedding="", head="head.", final_norm="final.", stream_shifts="loop.", layer="l{index}.",
                            mixer="mix.", feed_forward="mlp.", mixer_norm="", feed_forward_norm="", prefix_rewrites=())
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            order=self.run_order(), final_norm=PartSpec("rms_norm", dict(eps=self.eps, zero_centred=True, tensor="norm")),
            embedding=PartSpec("table", dict(tensor="embed")), head=PartSpec("linear", dict(scale=self.logit_scale)),
            tie_word_embeddings=True,
            stream_shifts=PartSpec("table", dict(rows=self.loop_times, tensor="step")) if self.has_loop else None,
            names=names, optional_tensors=tuple(unused), eos_token_ids=(), max_position_embeddings=self.max_position_embeddings,
            init_std=self.initializer_range)
