"""CUDA operators of the package (stand-alone launches of the kernels under csrc/)."""
from .attention import attention_decode
from .elementwise import (add, axpby, gelu, gelu_bwd, layernorm, qknorm_rope, rmsnorm, rope, scale, silu, silu_gate,
                          softmax)
from .gemm import block_weight, gemm, interleave_gate_up, linear, matmul, unblock_weight

__all__ = ["attention_decode", "gemm", "linear", "matmul", "interleave_gate_up", "block_weight", "unblock_weight", "gelu", "silu", "softmax", "scale", "add", "silu_gate",
           "gelu_bwd", "axpby", "rmsnorm", "layernorm", "rope", "qknorm_rope"]
