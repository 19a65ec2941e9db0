"""Same module name and public function as the reference's alpha_moe_ops.py."""
from alpha_moe_b200.ops import fused_moe_w8a8_up_down

__all__ = ["fused_moe_w8a8_up_down"]
