"""B200-native drop-in for InfiniCore's paged decode path (infiniopPagedAttention and
infiniopPagedCaching behind the unchanged InfiniOp C ABI).

The operators and the ctypes binding load libinfinirt.so / libinfiniop.so (built in-tree for
sm_100a by `python -m infinicore_b200.build`) on first use and raise if the libraries are
missing - there is no CPU or pure-PyTorch fallback anywhere in this package.  The load is
deferred to first attribute access only so that the build module can be imported before the
libraries exist.
"""
_LAZY = {
    "LIBINFINIOP": "libinfiniop",
    "InfiniDeviceEnum": "libinfiniop",
    "InfiniDtype": "libinfiniop",
    "library_paths": "libinfiniop",
    "paged_attention": "ops",
    "paged_attention_multi_out": "ops",
    "paged_caching": "ops",
    "paged_attention_prefill": "ops",
    "paged_decode_step": "ops",
    "rope": "ops",
    "kv_caching": "ops",
    "RopeAlgo": "ops",
    "kernel_status": "ops",
    "DecodeStep": "decode_step",
}

__all__ = sorted(_LAZY)


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'infinicore_b200' has no attribute {name!r}")
    import importlib

    value = getattr(importlib.import_module(f"{__name__}.{mod}"), name)
    globals()[name] = value
    return value
