"""B200 (sm_100a) implementations of runtherder's row-wise decoder-layer kernels.

`kernels` mirrors the reference's kernel API; `layer_ops` issues a layer's chain; `kv_cache`,
`rope_tables`, `configs`, `synth`, `host_path` and `sharding` are the host pieces around it.
Everything computes in librh_kernels.so (CUDA, built by `python -m runtherder_b200.build`);
importing any of those modules raises if that library is absent — there is no fallback path.
The package itself imports nothing native so that the build module can run before the library exists.
"""
__all__ = ["RhError"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "RhError":
        from ._lib import RhError
        return RhError
    raise AttributeError(name)
