"""Import-name shim so code written for the reference (`from hexa_moe import moe as hmoe`) runs unchanged."""
