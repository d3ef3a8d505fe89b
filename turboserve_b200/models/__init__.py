"""Models: the generic decoder and the architectures registered on top of it."""

from .decoder import DecoderModel, NamedParam
from . import baporax, filezen, qwen2  # noqa: F401  (register Baporax, Filezen and Qwen2ForCausalLM)

__all__ = ["DecoderModel", "NamedParam"]
