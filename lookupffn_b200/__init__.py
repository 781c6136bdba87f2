"""lookupffn_b200: the LookupFFN layer (hash projection -> sign-bit codes -> weighted gather-add over
lookup tables) as hand-written sm_100a CUDA kernels behind a C ABI, with the reference's module and
operator interface on top.  CUDA only: importing works anywhere, calling an op needs the built
library and a GPU."""
from .lookup import BH4, Hashing, LookupFFN, SignHadamard  # noqa: F401
from . import ops  # noqa: F401

__all__ = ["LookupFFN", "Hashing", "BH4", "SignHadamard", "ops"]
