"""ctypes binding of libgct_b200.so (the C ABI declared in include/gct_b200.h).

There is no fallback: if the library is missing the import fails loudly, and every compute entry
point needs a CUDA device.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgct_b200.so")

GCT_OK = 0
ERR_INVALID, ERR_POOL_EXHAUSTED, ERR_UNDERFLOW, ERR_CUDA, ERR_DEVICE_STATUS, ERR_CAPACITY = 1, 2, 3, 4, 5, 6
F32, BF16 = 0, 1
ROPE_NONE, ROPE_2D, ROPE_3D = 0, 1, 2


class GctError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[gct_b200 error {code}] {msg}")
        self.code = code


class MgrConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_blocks", "tokens_per_frame", "num_heads", "head_dim", "num_special_tokens",
        "scale_frames", "sliding_window", "max_total_frames")]


class MgrGeometry(C.Structure):
    _fields_ = [("page_size", C.c_int32), ("max_patch_pages", C.c_int32), ("max_num_pages", C.c_int32),
                ("pool_bytes", C.c_int64)]


_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_pi, _pi32, _pi64, _pf = C.POINTER(C.c_int), C.POINTER(C.c_int32), C.POINTER(C.c_int64), C.c_void_p

# name -> (restype, argtypes); every symbol include/gct_b200.h declares
SIGNATURES = {
    "gct_last_error": (C.c_char_p, []),
    "gct_version": (_i, []),
    "gct_mgr_create": (_i, [C.POINTER(_vp), C.POINTER(MgrConfig), C.POINTER(MgrGeometry)]),
    "gct_mgr_destroy": (_i, [_vp]),
    "gct_mgr_bind": (_i, [_vp, C.POINTER(_vp), _vp, _sz]),
    "gct_mgr_workspace_bytes": (_i, [_vp, C.POINTER(_sz)]),
    "gct_mgr_append": (_i, [_vp, _i, _vp, _i, _vp, _i, _vp]),
    "gct_mgr_append_bookkeeping": (_i, [_vp, _i]),
    "gct_mgr_scan_keys": (_i, [_vp, _i, _vp]),
    "gct_mgr_set_bounded_mode": (_i, [_vp, _i]),
    "gct_mgr_append_fused": (_i, [_vp, _i, _vp, _i, _i64, _pf, _pf, _pf, _pf, _pf, _i, _vp, _vp]),
    "gct_mgr_evict": (_i, [_vp, _i, _i]),
    "gct_mgr_exec_deferred": (_i, [_vp, _i, _i]),
    "gct_mgr_set_defer": (_i, [_vp, _i]),
    "gct_mgr_get_defer": (_i, [_vp, _pi]),
    "gct_mgr_rollback": (_i, [_vp, _i]),
    "gct_mgr_reset": (_i, [_vp]),
    "gct_mgr_visible_table": (_i, [_vp, _i, _pi32, _i, _pi, _pi]),
    "gct_mgr_stats": (_i, [_vp, _i, _pi64]),
    "gct_mgr_free_list": (_i, [_vp, _i, _i, _pi32, _i, _pi]),
    "gct_mgr_plan": (_i, [_vp, _i, _i, _vp]),
    "gct_mgr_attention": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "gct_mgr_attention_partial": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "gct_mgr_device_status": (_i, [_vp, _vp, _pi]),
    "gct_mgr_launch_count": (_i, [_vp, _pi64]),
    "gct_mgr_kernel_timing": (_i, [_vp, _i]),
    "gct_mgr_kernel_time": (_i, [_vp, C.POINTER(C.c_double), _pi]),
    "gct_attn_launch_shape": (_i, [_i, _i, _i, _i, _i, _pi, _pi, _pi]),
    "gct_attn_dense": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _pi64, _pi64, _pi64, _vp, _sz, _vp]),
    "gct_prep_qkv": (_i, [_vp, _i, _i64, _i, _i, _i, _pf, _pf, _pf, _pf, _pf, _i, _vp, _vp, _vp, _vp]),
    "gct_rope3d_table": (_i, [_i, _i, _i, _i, _vp, _vp]),
    "gct_rope2d_table": (_i, [_i, _i, _i, C.c_float, _vp, _vp]),
    "gct_lse_merge": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "gct_lse_merge_strided": (_i, [_vp, _vp, _i, _i, _i, _i64, _i64, _vp, _vp, _vp]),
    "gct_kv_exchange_sizes": (_i, [_i, _i, _i, C.POINTER(_sz), C.POINTER(_sz), _pi]),
    "gct_mgr_attention_exchange": (_i, [_vp, _i, _vp, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                        _i, _i, _vp]),
    "gct_decode_workspace_bytes": (_i, [_i, _i, C.POINTER(_sz)]),
    "gct_decode_attention": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "gct_frustum_cull": (_i, [_vp, _i64, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_float, C.c_float, C.c_float,
                              C.c_float, _i, _i, C.c_float, C.c_float, _vp, _vp]),
    "gct_voxel_morton": (_i, [_vp, _vp, C.c_float, _i64, _vp, _vp, _vp, _vp]),
    "gct_mark_unique": (_i, [_vp, _i64, _vp, _vp]),
    "gct_attn_paged_static": (_i, [_vp, _i, _i, _i, _pi32, _i, _i, _vp, _i, _vp, _vp, _pi]),
}

_lib = None


def load():
    """Load the shared library (once) and set the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python lingbot-map_b200/build.py` "
                "(or __graft_entry__.build()); this backend has no fallback path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc):
    if rc != GCT_OK:
        msg = load().gct_last_error()
        raise GctError(rc, msg.decode() if msg else "unknown error")
