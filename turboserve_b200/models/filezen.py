"""Filezen: its configuration class and its builder, registered by name.

The architecture is a translation of its ``config.json`` into parts
(:meth:`FilezenConfig.to_model_spec`): latent attention (some layers reading the rows another layer caches) or
retention per layer, a gated feed-forward or a mixture of experts, RMS norms behind the sublayers, a scaled
embedding and a tied head.
"""

from __future__ import annotations

import torch

from ..config.filezen import ARCHITECTURE, FilezenConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


def build_filezen(config: FilezenConfig, dtype: torch.dtype, device: torch.device | str) -> DecoderModel:
    return DecoderModel(config.to_model_spec(), dtype, device)


register_architecture(ARCHITECTURE, FilezenConfig, build_filezen)
