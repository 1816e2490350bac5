"""logismos_b200 - B200-native (sm_100a) hot path of the logismos inference stack.

The product is the C-ABI library ``liblogismos_kernels.so`` declared in ``include/*.h``; this
package is the thin host-side mirror used from Python: ``ops`` mirrors the reference's op layer
(crates/praxis), ``embed`` mirrors ``StellaModel`` (crates/embed). There is no CPU fallback: every
call goes to the CUDA library and fails loudly when it is missing.
"""
from ._lib import LogismosError, lib, library_path  # noqa: F401

__all__ = ["LogismosError", "lib", "library_path"]
