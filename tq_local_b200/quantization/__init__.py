"""Codec set-up (host side)."""

from tq_local_b200.quantization.turboquant_mse import (
    ScalarCodebook,
    build_scalar_codebook,
    random_rotation_matrix,
)

__all__ = ["ScalarCodebook", "build_scalar_codebook", "random_rotation_matrix"]
