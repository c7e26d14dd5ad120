"""B200-native fused-MoE operator (ck_tile fused_moe surface) -- Python host mirror.

The compute lives in libfmoe_b200.so (hand-written sm_100a CUDA behind a C-ABI, see
include/fused_moe_c.h).  This package only marshals torch tensors into that ABI; there is
no Python or CPU fallback: importing the operator without the built library raises.
"""
from .api import (FusedMoeTraits, FusedMoeArgs, fused_moe, fused_moe_workspace_size,  # noqa: F401
                  moe_sorting, sort_capacity, workspace_layout, launches_per_run, describe_run, lib, LIB_PATH,
                  FmoeError, route)

__all__ = ["FusedMoeTraits", "FusedMoeArgs", "fused_moe", "fused_moe_workspace_size", "moe_sorting",
           "sort_capacity", "workspace_layout", "launches_per_run", "describe_run", "lib", "LIB_PATH", "FmoeError", "route"]
