"""B200 (sm_100a) implementations of runtherder's row-wise decoder-layer kernels.

`kernels` mirrors the reference's kernel API; `layer_ops` issues a layer's chain; `kv_cache`,
`rope_tables`, `configs`, `synth` and `sharding` are the host pieces around it.  Everything
computes in librh_kernels.so (CUDA, built by `python -m runtherder_b200.build`); importing the
package fails if that library is absent.
"""
from . import _lib  # noqa: F401  (loads the native library or raises)
from ._lib import RhError

__all__ = ["RhError"]
__version__ = "0.1.0"
