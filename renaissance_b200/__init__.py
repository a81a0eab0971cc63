"""B200 (sm_100a) kernels for the Renaissance training-backward hot path and the
host-side mirror of the reference launchers that call them."""
from ._lib import Trb200Error, load  # noqa: F401

__all__ = ["Trb200Error", "load"]
