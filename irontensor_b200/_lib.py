"""ctypes binding of the C ABI in include/irontensor_b200.h (libirontensor_b200.so, built in-tree
by irontensor_b200/build.py).  There is no fallback: a missing library or a failing call raises."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libirontensor_b200.so")

IT_OK = 0
IT_ERR_INVALID_ARG = -1
IT_ERR_UNSUPPORTED_SHAPE = -2
IT_ERR_PRECISION = -3
IT_ERR_ALIGNMENT = -4
IT_ERR_CUDA = -5
IT_ERR_TIMEOUT = -6
IT_F32 = 0
IT_BF16 = 1
IT_NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024

_c = ctypes
_vp = _c.c_void_p
_i32 = _c.c_int32

# name -> argtypes; every function returns it_status (int32) except it_last_error and it_ctx_kernel_tag.
SIGNATURES = {
    "it_ctx_create": [_c.c_int, _c.POINTER(_vp)],
    "it_ctx_destroy": [_vp],
    "it_stream_create": [_vp, _c.POINTER(_vp)],
    "it_stream_wrap": [_vp, _vp, _c.POINTER(_vp)],
    "it_stream_destroy": [_vp, _vp],
    "it_stream_sync": [_vp, _vp],
    "it_event_create": [_vp, _c.POINTER(_vp)],
    "it_event_destroy": [_vp, _vp],
    "it_event_record": [_vp, _vp, _vp],
    "it_event_query": [_vp, _vp, _c.POINTER(_i32)],
    "it_event_wait": [_vp, _vp],
    "it_ctx_check_status": [_vp, _c.POINTER(_i32)],
    "it_event_elapsed_ms": [_vp, _vp, _vp, _c.POINTER(_c.c_float)],
    "it_buf_alloc": [_vp, _c.c_size_t, _c.POINTER(_vp)],
    "it_buf_free": [_vp, _vp],
    "it_host_alloc": [_vp, _c.c_size_t, _c.POINTER(_vp)],
    "it_host_free": [_vp, _vp],
    "it_buf_upload": [_vp, _vp, _vp, _vp, _c.c_size_t],
    "it_buf_download": [_vp, _vp, _vp, _vp, _c.c_size_t],
    "it_buf_memset_async": [_vp, _vp, _vp, _c.c_int, _c.c_size_t],
    "it_flash_attention_fwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "it_flash_attention_bwd_workspace_bytes": [_c.c_int, _i32, _i32, _i32, _i32, _c.POINTER(_c.c_size_t)],
    "it_flash_attention_bwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32] + [_vp] * 9 + [_vp, _c.c_size_t],
    "it_attention_fwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "it_host_step_create": [_vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _c.POINTER(_vp)],
    "it_host_step_run": [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32],
    "it_host_step_destroy": [_vp],
    "it_linear_scatter_add": [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _c.POINTER(_vp), _i32, _i32],
    "it_attention_cross_fwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "it_attention_bwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32] + [_vp] * 9 + [_vp, _c.c_size_t],
    "it_attention_gqa_fwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "it_attention_gqa_bwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32] + [_vp] * 9 + [_vp, _c.c_size_t],
    "it_attention_packed_fwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp],
    "it_attention_packed_bwd": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32, _c.c_float, _i32, _vp, _vp, _vp, _vp, _vp,
                                _vp, _c.c_size_t],
    "it_rope_qk": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _c.c_float, _i32, _i32, _vp, _vp, _vp, _vp],
    "it_attention_gqa_bwd_rope": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32, _c.c_float, _i32] + [_vp] * 9 +
                                 [_vp, _c.c_size_t],
    "it_attention_decode_workspace_bytes": [_i32, _i32, _i32, _c.POINTER(_c.c_size_t)],
    "it_attention_decode": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _c.c_size_t],
    "it_linear_fwd": [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp],
    "it_qkv_rope_workspace_bytes": [_i32, _i32, _c.POINTER(_c.c_size_t)],
    "it_qkv_rope_fwd": [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _c.c_float, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _c.c_size_t],
    "it_linear_bwd": [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "it_flash_attention_bwd_noalloc": [_vp, _vp, _c.c_int, _i32, _i32, _i32, _i32, _i32] + [_vp] * 9,
    "it_attention_status_poll": [_vp, _vp, _c.POINTER(_i32)],
    "it_ctx_launch_count": [_vp, _c.POINTER(_c.c_uint64)],
    "it_ctx_enable_kernel_timing": [_vp, _i32],
    "it_ctx_kernel_ms": [_vp, _i32, _c.POINTER(_c.c_float)],
    "it_selftest_umma": [_vp, _vp, _i32, _vp, _vp, _vp],
    "it_selftest_wait_timeout": [_vp, _vp, _i32],
}

_lib = None


class ITError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"irontensor_b200 status {status}: {message}")
        self.status = status


def load():
    """Loads the shared library (once) and declares every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m irontensor_b200.build` "
                "(there is no CPU or PyTorch fallback for the attention path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i32
        lib.it_last_error.argtypes = []
        lib.it_last_error.restype = _c.c_char_p
        lib.it_ctx_kernel_tag.argtypes = [_i32]
        lib.it_ctx_kernel_tag.restype = _c.c_char_p
        _lib = lib
    return _lib


def check(status):
    if status != IT_OK:
        raise ITError(status, load().it_last_error().decode("utf-8", "replace"))
