"""pet_b200 — host side of the Blackwell-native execution backend for PET operator graphs.

`lib`   : ctypes binding of libpetb200.so (the C ABI in include/petb200.h)
`ops`   : operator-level API (Context) mirroring the reference's operator arguments
`build` : nvcc build of the library for sm_100a
"""
from .lib import PetError, load  # noqa: F401
