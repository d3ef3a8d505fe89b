"""Baporax: its configuration class and its builder, registered by name.

The architecture is a translation of its ``config.json`` into parts
(:meth:`BaporaxConfig.to_model_spec`): differential window attention or a Mamba-2 mixer per
layer, a dense squared-relu feed-forward beside it, zero-centred RMS norms, a looped stretch of
layers with a shift of the stream before each pass, and a tied, scaled head.
"""

from __future__ import annotations

import torch

from ..config.baporax import ARCHITECTURE, BaporaxConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


def build_baporax(config: BaporaxConfig, dtype: torch.dtype, device: torch.device | str) -> DecoderModel:
    return DecoderModel(config.to_model_spec(), dtype, device)


register_architecture(ARCHITECTURE, BaporaxConfig, build_baporax)
