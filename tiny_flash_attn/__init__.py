"""Drop-in module name of the reference's Python package (reference python/tiny_flash_attn/__init__.py:1-7).

Unlike the reference, a missing native library is an ImportError here, not a silently empty module.
"""
from tinyfa_b200.api import flash_attn_forward, flash_attn_varlen_forward

__all__ = ["flash_attn_forward", "flash_attn_varlen_forward"]
