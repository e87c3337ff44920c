from . import attention, block, feed_forward, norm, position     # registers the built-in parts
from .context import BuildContext, QueryTiles, StepFacts, Workspace
from .linear import linear, set_matmul_precision
from .model import DecoderModel, build_model, manifest_for_config
from .registry import (build_block, build_feed_forward, build_mixer, build_norm, build_position,
                       known, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

__all__ = ["BuildContext", "QueryTiles", "StepFacts", "Workspace", "linear", "set_matmul_precision", "DecoderModel",
           "build_model", "manifest_for_config", "build_block", "build_feed_forward",
           "build_mixer", "build_norm", "build_position", "known", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "LayerSpec", "ModelSpec", "PartSpec", "RunEntry"]
