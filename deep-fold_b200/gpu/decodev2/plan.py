"""Import path kept from the reference (gpu/decodev2/plan.py); see ``arch``."""

from .arch import MEDIUM_LLAMA, TINY_INTERNLM, TINY_LLAMA, ArchSpec

__all__ = ["ArchSpec", "TINY_INTERNLM", "TINY_LLAMA", "MEDIUM_LLAMA"]
