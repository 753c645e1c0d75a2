"""The built-in parts, registered by kind."""

from tandem_b200.parts.attention import PagedAttention
from tandem_b200.parts.block import PreNormBlock
from tandem_b200.parts.mlp import GatedMLP
from tandem_b200.parts.norm import RMSNorm
from tandem_b200.parts.rope import NoPosition, RotaryTable
from tandem_b200.registry import register_part

register_part("mixer", "attention", PagedAttention)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("norm", "rmsnorm", RMSNorm)
register_part("position", "rope", RotaryTable)
register_part("position", "none", NoPosition)
register_part("block", "prenorm", PreNormBlock)
