"""`import alpha_moe` registers torch.ops.alpha_moe.fused_moe_w8a8_up_down, as importing the
reference's extension module does (csrc/torch_interface.cpp:105-131)."""
import alpha_moe_b200 as _impl

_impl.load_torch_op()
