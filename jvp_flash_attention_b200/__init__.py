"""B200 (sm_100a) JVP flash attention: CUDA kernels behind the ``jvp_flash_attention`` API.

``from jvp_flash_attention_b200.jvp_attention import JVPAttn, attention`` replaces
``from jvp_flash_attention.jvp_attention import JVPAttn, attention``.
"""
from .jvp_attention import MASK_CONST, MIN_SEQUENCE_LENGTH, JVPAttn, attention, check  # noqa: F401

__all__ = ["JVPAttn", "attention", "check", "MASK_CONST", "MIN_SEQUENCE_LENGTH"]
