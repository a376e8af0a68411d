"""`hexa_moe.moe` re-exports hexa_moe_b200's MoE_Cascaded / MoE_Buffer."""
from hexa_moe_b200.impls.cascaded_moe import MoE_Buffer, MoE_Cascaded  # noqa: F401
