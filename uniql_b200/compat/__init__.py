"""Stand-ins for the reference's three CUDA extension modules, backed by this package's C ABI.

`install()` registers them in sys.modules under the names UniQL imports (`quant_linear_cuda`,
`quant_embedding_cuda`, `fast_hadamard_transform_cuda`) so that the unmodified UniQL Python sources
run on these kernels.
"""
import sys

from . import fast_hadamard_transform_cuda, quant_embedding_cuda, quant_linear_cuda


def install(overwrite: bool = False) -> None:
    for mod in (quant_linear_cuda, quant_embedding_cuda, fast_hadamard_transform_cuda):
        name = mod.__name__.rsplit(".", 1)[-1]
        if overwrite or name not in sys.modules:
            sys.modules[name] = mod
