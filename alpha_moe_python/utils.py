"""Same module path as the reference's alpha_moe_python/utils.py."""
from alpha_moe_b200.utils import get_best_config, interleave_tensor

__all__ = ["interleave_tensor", "get_best_config"]
