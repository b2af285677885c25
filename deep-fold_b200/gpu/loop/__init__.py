"""TokenLoop: the greedy executor on the tensor-core (MMA) N=1 path."""

from .generate import Generation, TokenLoop, mma_decode

__all__ = ["Generation", "TokenLoop", "mma_decode"]
