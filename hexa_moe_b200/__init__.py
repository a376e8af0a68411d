"""hexa_moe_b200: B200-native (sm_100a) expert-specific MoE operators behind HEXA-MoE's MoE_Cascaded API.

    from hexa_moe_b200 import moe as hmoe      # drop-in for `from hexa_moe import moe as hmoe`

The compute path is libhexa_moe_b200.so (C ABI in include/hexa_moe_b200.h); build it with
`python -m hexa_moe_b200.build`.  There is no CPU fallback.
"""
__version__ = "0.1.0"
