from .registry import (build_block, build_part, register_block, register_part, registered_blocks,
                       registered_parts)
from .norm import RMSNorm
from .position import NoPosition, Rotary
from .attention import GQAttention
from .feed_forward import SwiGLU, interleave_gate_up
from .model import Block, DecoderModel

__all__ = ["build_part", "register_part", "registered_parts", "build_block", "register_block", "registered_blocks", "RMSNorm", "Rotary", "NoPosition",
           "GQAttention", "SwiGLU", "interleave_gate_up", "Block", "DecoderModel"]
