"""uniql_b200: B200 (sm_100a) kernels behind UniQL's W4A16 linear, online Hadamard and 4-bit embedding."""
from . import ops  # noqa: F401
from ._lib import UniqlError, lib  # noqa: F401

__all__ = ["ops", "lib", "UniqlError"]
