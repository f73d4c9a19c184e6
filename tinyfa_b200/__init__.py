"""B200-native attention forward behind the TinyFA API (C ABI in include/tinyfa_b200.h)."""
from .api import (device_status, flash_attn_forward, flash_attn_varlen_forward, is_head_dim_compiled,
                  set_option)

from .host import flash_attn_forward_host

__all__ = ["flash_attn_forward", "flash_attn_forward_host", "flash_attn_varlen_forward", "is_head_dim_compiled", "device_status", "set_option"]
