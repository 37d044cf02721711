"""lockstep_b200: lockstep's MXFP4 data-parallel hot path on B200 (sm_100a).

Sub-modules mirror the reference's module names: fp4, mxfp4_gemm, dual_gemm,
fp4_linear, wire.  `install_dropins()` registers them under those top-level
names so that code written against the reference (`import fp4`) runs on this
package unchanged.
"""

import importlib
import sys

__version__ = "0.1.0"
_DROPINS = ("fp4", "mxfp4_gemm", "dual_gemm", "fp4_linear", "wire")


def install_dropins(names=_DROPINS):
    """Make `import fp4` etc. resolve to this package's modules."""
    for n in names:
        sys.modules[n] = importlib.import_module(f"{__name__}.{n}")
