"""Fused operators: model kernels, tensor-parallel GEMM + collective kernels, MoE expert-parallel dispatch/combine."""
from . import fused  # noqa: F401
