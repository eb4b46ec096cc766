"""cupynumeric_b200: a B200 (sm_100a) implementation of cuPyNumeric's SORT task - the path
behind ``sort``, ``argsort`` and ``ndarray.sort`` - behind a C ABI (``include/b200sort.h``),
with the host-side dispatch of the reference's Python layer on top."""
from ._array import array, ndarray  # noqa: F401
from ._module.ssc_sorting import (argpartition, argsort, lexsort, partition, searchsorted, sort,  # noqa: F401
                                  sort_complex)
from ._module.sets_making import unique  # noqa: F401
from .runtime import runtime  # noqa: F401

__all__ = ["array", "ndarray", "sort", "argsort", "searchsorted", "sort_complex", "partition", "argpartition",
           "lexsort", "unique", "runtime"]
