"""Public API: `from hexa_moe_b200 import moe as hmoe; hmoe.MoE_Cascaded(...)` (the reference's hexa_moe/moe.py:2)."""
from .impls.cascaded_moe import MoE_Buffer, MoE_Cascaded  # noqa: F401
