"""Route the reference's kernel-path callables to this library.

The reference model picks its kernels by importing, at call time,
`compression_attn_triton` and `window_attn_triton` from `nsa_fused_kernel` and
`selection_attn_triton` from `nsa_selection_backward` (nsa_model.py:316-317) when
`attn_impl="fused"`.  `install()` rebinds those names (and the launch wrappers the
reference's tests and benches import) so that an unmodified reference checkout runs on the
CUDA kernels of this package:

    import sys; sys.path.insert(0, "/path/to/openbox-llm")
    dropin = importlib.import_module("openbox-llm_b200.dropin"); dropin.install()
    from nsa_model import NSATransformer            # attn_impl="fused" now uses libnsa_b200

If the reference modules cannot be imported (no checkout on the path), modules with the same
names holding only the kernel-path callables are registered instead.
"""
import importlib
import sys
import types

from . import ops

_EXPORTS = {
    "nsa_selection_kernel": {
        "selection_forward_triton": ops.selection_forward_triton,
    },
    "nsa_selection_backward": {
        "selection_forward_triton": ops.selection_forward_triton,
        "selection_backward_triton": ops.selection_backward_triton,
        "SelectionAttnTriton": ops.SelectionAttnTriton,
        "selection_attn_triton": ops.selection_attn_triton,
    },
    "nsa_fsa": {
        "build_block_to_query_csr": ops.build_block_to_query_csr,
    },
    "nsa_fused_kernel": {
        "_RangeAttn": ops._RangeAttn,
        "window_attn_triton": ops.window_attn_triton,
        "compression_attn_triton": ops.compression_attn_triton,
        "selection_attn_triton": ops.selection_attn_triton,
        "block_mean_pool": ops.block_mean_pool,
        "nsa_fused_forward": ops.nsa_fused_forward,
        "MODE_WINDOW": ops.MODE_WINDOW,
        "MODE_COMPRESS": ops.MODE_COMPRESS,
    },
}


def install(allow_synthetic=True):
    """Rebind the kernel-path names.  Returns {module name: 'patched' | 'synthetic'}."""
    done = {}
    for mod_name, names in _EXPORTS.items():
        try:
            mod = importlib.import_module(mod_name)
            how = "synthetic" if getattr(mod, "_nsa_b200_synthetic", False) else "patched"
            if how == "synthetic" and not allow_synthetic:
                raise ImportError(f"{mod_name} is a stand-in registered by an earlier install()")
        except ImportError:
            if not allow_synthetic:
                raise
            mod = types.ModuleType(mod_name)
            mod.__doc__ = "kernel-path names served by openbox-llm_b200"
            mod._nsa_b200_synthetic = True
            sys.modules[mod_name] = mod
            how = "synthetic"
        for name, obj in names.items():
            setattr(mod, name, obj)
        done[mod_name] = how
    return done
