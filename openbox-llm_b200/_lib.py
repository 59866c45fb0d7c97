"""ctypes binding of libnsa_b200.so.  There is no fallback: if the library is missing or a
call fails, an exception is raised."""
import ctypes
import functools
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libnsa_b200.so")

DTYPE_BF16, DTYPE_F32 = 0, 1
MODE_WINDOW, MODE_COMPRESS = 0, 1
MODE_COMPRESS_STRIDED = 3   # the `window` argument is the stride of the summaries
IMPL = {"auto": 0, "simt": 1, "tc": 2}


class NsaDims(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "Hq", "Hkv", "T", "D", "dtype")]


class NsaError(RuntimeError):
    pass


_lib = None
_vp, _i, _sz, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float
_dp = ctypes.POINTER(NsaDims)

# every symbol the header declares, with its signature
SIGNATURES = {
    "nsa_last_error": (ctypes.c_char_p, []),
    "nsa_version": (_i, []),
    "nsa_tc_supported": (_i, [_dp, _i]),
    "nsa_device_status": (_i, [_vp]),
    "nsa_debug_set_device_status": (_i, [_i, _vp]),
    "nsa_launch_count": (ctypes.c_longlong, []),
    "nsa_set_option": (_i, [ctypes.c_char_p, _i]),
    "nsa_profile_enable": (None, [_i]),
    "nsa_profile_summary": (_i, [ctypes.c_char_p, _sz]),
    "nsa_range_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _dp, _i, _i, _i, _i, _i, _vp]),
    "nsa_range_attn_bwd_workspace_bytes": (_sz, [_dp, _i, _i, _i, _i]),
    "nsa_range_attn_bwd": (_i, [_vp] * 9 + [_dp, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _i, _vp]),
    "nsa_selection_fwd_workspace_bytes": (_sz, [_dp, _i, _i, _i]),
    "nsa_selection_fwd": (_i, [_vp] * 6 + [_dp, _i, _i, _vp, _sz, _i, _vp]),
    "nsa_selection_bwd_workspace_bytes": (_sz, [_dp, _i, _i, _i]),
    "nsa_selection_bwd": (_i, [_vp] * 10 + [_dp, _i, _i, _vp, _vp, _vp, _sz, _i, _vp]),
    "nsa_selection_plan_bytes": (_sz, [_dp, _i, _i]),
    "nsa_selection_plan_build": (_i, [_vp, _dp, _i, _i, _vp, _sz, _vp]),
    "nsa_selection_fwd_planned": (_i, [_vp] * 6 + [_dp, _i, _i, _vp, _sz, _vp, _vp]),
    "nsa_selection_bwd_planned": (_i, [_vp] * 10 + [_dp, _i, _i, _vp, _vp, _vp, _sz, _vp, _vp]),
    "nsa_csr_workspace_bytes": (_sz, [_i] * 5),
    "nsa_build_block_to_query_csr": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nsa_csr_builtin_scratch_bytes": (_sz, []),
    "nsa_build_block_to_query_csr_noalloc": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "nsa_block_mean_pool_fwd": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_block_mean_pool_bwd": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_block_compress_fwd": (_i, [_vp] * 5 + [_i] * 6 + [_vp]),
    "nsa_block_compress_bwd_workspace_bytes": (_sz, [_i] * 5),
    "nsa_block_compress_bwd": (_i, [_vp] * 9 + [_i] * 6 + [_vp, _sz, _vp]),
    "nsa_block_compress_strided_fwd": (_i, [_vp] * 5 + [_i] * 7 + [_vp]),
    "nsa_block_compress_strided_bwd_workspace_bytes": (_sz, [_i] * 6),
    "nsa_block_compress_strided_bwd": (_i, [_vp] * 9 + [_i] * 7 + [_vp, _sz, _vp]),
    "nsa_topn_blocks": (_i, [_vp] * 5 + [_dp, _i, _i, _i, _i, _vp]),
    "nsa_topn_blocks_forced": (_i, [_vp] * 5 + [_dp, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_topn_blocks_general": (_i, [_vp] * 5 + [_dp] + [_i] * 8 + [_vp]),
    "nsa_gate_combine_bwd_rows": (_i, [_vp] * 8 + [_dp, _vp]),
    "nsa_sum3": (_i, [_vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "nsa_sumsq_f32": (_i, [_vp, _sz, _vp, _vp]),
    "nsa_adamw_step_f32": (_i, [_vp] * 4 + [_sz] + [_f] * 5 + [_i, _vp, _f, _f, _vp]),
    "nsa_dq_reduce3": (_i, [_dp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "nsa_range_attn_bwd_acc_workspace_bytes": (_sz, [_dp, _i, _i, _i]),
    "nsa_range_attn_bwd_acc": (_i, [_vp] * 9 + [_dp, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "nsa_dq_finish": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp]),
    "nsa_fused_projection_width": (_i, [_i, _i, _i]),
    "nsa_split_heads": (_i, [_vp] * 4 + [_i] * 6 + [_vp]),
    "nsa_merge_heads": (_i, [_vp] * 4 + [_i] * 6 + [_vp]),
    "nsa_swap_heads_tokens": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "nsa_gate_combine_fwd": (_i, [_vp] * 5 + [_dp, _vp]),
    "nsa_gate_combine_bwd": (_i, [_vp] * 9 + [_dp, _vp]),
}


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NsaError(f"{LIB_PATH} is missing: build it with `python {_HERE}/build.py`; "
                           "there is no non-CUDA fallback")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
        # tuning switches from the environment: NSA_B200_OPTIONS="name=value,name=value" (nsa_set_option)
        for item in filter(None, os.environ.get("NSA_B200_OPTIONS", "").split(",")):
            name, _, value = item.partition("=")
            check(handle.nsa_set_option(name.strip().encode(), int(value)))
    return _lib


def check(rc):
    if rc != 0:
        raise NsaError(f"libnsa_b200 error {rc}: {lib().nsa_last_error().decode()}")


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"libnsa_b200 takes bfloat16 or float32 tensors, got {t.dtype}")


def ptr(t):
    if t is None:
        return None
    assert t.is_cuda, "libnsa_b200 needs CUDA tensors; there is no CPU path"
    return ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def dims(B, Hq, Hkv, T, D, dtype):
    return NsaDims(B, Hq, Hkv, T, D, dtype)


def on_device(fn):
    """Decorator of every wrapper that launches library kernels: the CUDA tensors among the
    arguments must live on ONE device, and the call runs with that device current, so that the
    stream, the TMA tensor maps and the library's per-device symbols (status word, built-in
    scratch) belong to the device that holds the data.  Without it, tensors on cuda:1 while
    cuda:0 is current would launch on GPU 0 with GPU 1's pointers."""
    @functools.wraps(fn)
    def wrapper(*args, **kw):
        dev = None
        for a in list(args) + list(kw.values()):
            if isinstance(a, torch.Tensor) and a.is_cuda:
                if dev is None:
                    dev = a.device
                elif a.device != dev:
                    raise NsaError(f"libnsa_b200: tensors on different devices ({dev} and {a.device})")
        if dev is None or dev.index == torch.cuda.current_device():
            return fn(*args, **kw)
        with torch.cuda.device(dev):
            return fn(*args, **kw)
    return wrapper


def check_device_status():
    """Read (and clear) the current device's status word, synchronising the current stream; raise
    when a kernel gave up a bounded wait.  After such a give-up every later tcgen05 kernel
    returns at entry and leaves its outputs unwritten until the word is read, so long-running
    callers poll this at their own synchronisation points."""
    check(lib().nsa_device_status(stream()))


CHECK_STATUS_EVERY_CALL = os.environ.get("NSA_B200_CHECK_STATUS", "0") not in ("", "0")


def workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


def profile_summary():
    """{kernel name: (launches, total_ms)} since nsa_profile_enable(1)."""
    buf = ctypes.create_string_buffer(1 << 16)
    lib().nsa_profile_summary(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms = line.split()
        out[name] = (int(cnt), float(ms))
    return out
