"""grape_b200: the proving hot path of Grape (Hyrax commitments, Fr field tensors, sumcheck and
lookup provers over BN254) as hand-written sm_100a CUDA behind a C ABI.

Importing the package loads ``libgrape_b200.so``; there is no CPU fallback.
"""
from . import _lib
from ._lib import GrapeError, LIB_PATH, declared_symbols

_lib.load()

from .host import (COM_SCALE, Context, DeviceBuffer, GeneratorTable, commit_fr, commit_i32,  # noqa: E402
                   commit_i32_host, decode_field, decode_jacobian, encode_field, encode_jacobian)

__all__ = ["Context", "DeviceBuffer", "GeneratorTable", "GrapeError", "commit_i32", "commit_fr",
           "commit_i32_host", "encode_field", "decode_field", "encode_jacobian", "decode_jacobian",
           "COM_SCALE", "LIB_PATH", "declared_symbols"]
