"""sageattention_b200 -- SageAttention3 (NVFP4 attention) for NVIDIA B200, hand-written sm_100a CUDA behind a C ABI.

Public surface (mirrors the reference's): sageattn3, sageattn3_blackwell, sageattn, sageattn_varlen; sageattn3_offload for
operands in host memory.
"""
from .api import (Sage3Problem, release_workspaces, sageattn, sageattn3, sageattn3_blackwell, sageattn3_offload,
                  sageattn3_offload_release, sageattn_varlen)

__all__ = ["sageattn3", "sageattn3_blackwell", "sageattn", "sageattn_varlen", "sageattn3_offload", "sageattn3_offload_release", "Sage3Problem", "release_workspaces"]
__version__ = "0.1.0"
