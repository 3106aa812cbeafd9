"""rocmlir_b200: B200 (sm_100a) contraction kernels behind rocMLIR's boundary.

Host-side mirrors of the reference's operator interface (rock.gemm, rock.conv, rock.attention) over the
C ABI in include/rocmlir_b200.h. There is no CPU path: compute calls need the built shared library and
an sm_100 GPU and raise otherwise.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
