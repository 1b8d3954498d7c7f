"""Loader for libojasx_lut_b200.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libojasx_lut_b200.so")

_vp, _i, _sz, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_float



class GgmlTensor(C.Structure):
    """``struct ojasx_ggml_tensor`` of include/ojasx_ggml_b200.h (ojasx_ggml_adapter.h:35-41)."""
    _fields_ = [("type", C.c_int), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("data", C.c_void_p),
                ("extra", C.c_void_p)]

    @classmethod
    def of(cls, array=None, extra=None, type_=0):
        """Describes a C-contiguous float32 numpy array (GGML order: innermost extent first)."""
        t = cls()
        t.type = type_
        shape = list(array.shape[::-1]) if array is not None else []
        strides = list(array.strides[::-1]) if array is not None else []
        for i in range(4):
            t.ne[i] = shape[i] if i < len(shape) else 1
            t.nb[i] = strides[i] if i < len(strides) else (strides[-1] * shape[-1] if strides else 0)
        t.data = array.ctypes.data if array is not None else None
        t.extra = extra
        return t


# name -> (restype, argtypes); mirrors include/ojasx_lut_b200.h and include/ojasx_ggml_b200.h
SIGNATURES = {
    "ojasx_get_version": (C.c_char_p, []),
    "ojasx_get_backend_name": (C.c_char_p, []),
    "ojasx_create_linear": (_vp, [_i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "ojasx_set_linear_outliers": (_i, [_vp, _i, _vp, _vp, _vp]),
    "ojasx_linear_forward": (_i, [_vp, _vp, _vp, _i, _i]),
    "ojasx_get_compressed_size": (_sz, [_vp]),
    "ojasx_get_dense_size": (_sz, [_vp]),
    "ojasx_get_lut_sram_size": (_sz, [_vp]),
    "ojasx_get_compression_ratio": (_f, [_vp]),
    "ojasx_destroy_linear": (None, [_vp]),
    "ojasx_ggml_init": (_i, []),
    "ojasx_ggml_forward_linear": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "ojasx_ggml_forward_moe": (_i, [_vp, _vp, _vp, _vp, _i, _vp]),
    "ojasx_ggml_forward_kv_attention": (_i, [_vp, _vp, _i, _f, _vp]),
    "ojasx_b200_paged_kv_quantize": (_i, [_vp, _i, _sz, _i, _vp, _vp, _vp]),
    "ojasx_b200_paged_kv_scratch_floats": (_i, [_i, _i, _i, _i]),
    "ojasx_b200_paged_kv_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp, _vp]),
    "ojasx_b200_vq_assign": (_i, [_vp, _sz, _i, _vp, _i, _vp, _vp, _vp, _vp]),
    "ojasx_b200_last_error": (C.c_char_p, []),
    "ojasx_b200_launch_count": (C.c_ulonglong, []),
    "ojasx_b200_linear_forward": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "ojasx_b200_linear_forward_tensor": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "ojasx_b200_take_device_error": (_i, []),
    "ojasx_b200_linear_forward_raw": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp,
                                           _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "ojasx_b200_rvq_fused_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "ojasx_b200_create_linear_group": (_vp, [_vp, _i]),
    "ojasx_b200_linear_group_forward": (_i, [_vp, _vp, _sz, _vp, _sz, _i, _vp]),
    "ojasx_b200_destroy_linear_group": (None, [_vp]),
    "ojasx_create_kv_cache": (_vp, [_i, _i, _i, _i]),
    "ojasx_kv_cache_append": (_i, [_vp, _i, _vp, _vp]),
    "ojasx_kv_cache_attention": (_i, [_vp, _i, _vp, _vp, _f]),
    "ojasx_kv_cache_get_memory_size": (_sz, [_vp]),
    "ojasx_kv_cache_get_compression_ratio": (_f, [_vp]),
    "ojasx_destroy_kv_cache": (None, [_vp]),
    "ojasx_create_moe": (_vp, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ojasx_moe_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i]),
    "ojasx_moe_get_compressed_size": (_sz, [_vp]),
    "ojasx_moe_get_compression_ratio": (_f, [_vp]),
    "ojasx_destroy_moe": (None, [_vp]),
    "ojasx_b200_moe_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "ojasx_b200_moe_forward_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "ojasx_b200_silu_mul": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "ojasx_b200_build_lut": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _vp]),
    "ojasx_b200_moe_reserve": (_i, [_vp, _i, _i]),
    "ojasx_b200_moe_set_outliers": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "ojasx_b200_moe_set_router": (_i, [_vp, _vp, _i]),
    "ojasx_b200_moe_set_expert_offset": (_i, [_vp, _i]),
    "ojasx_b200_moe_route": (_i, [_vp, _vp, _i, _i, _vp, _vp, _i, _vp]),
    "ojasx_b200_moe_forward_routed": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "ojasx_b200_kvq_create": (_vp, [_i, _i, _i, _i, _i, _i, _vp, _vp]),
    "ojasx_b200_kvq_load": (_i, [_vp, _vp, _vp, _i]),
    "ojasx_b200_kvq_read": (_i, [_vp, _vp, _vp, _i, _i]),
    "ojasx_b200_kvq_seq_len": (_i, [_vp]),
    "ojasx_b200_kvq_reset": (_i, [_vp]),
    "ojasx_b200_kvq_append": (_i, [_vp, _vp, _vp, _i, _vp]),
    "ojasx_b200_kvq_decode": (_i, [_vp, _vp, _vp, _f, _i, _vp]),
    "ojasx_b200_kvq_decode_gather": (_i, [_vp, _vp, _vp, _f, _i, _i, _i, _vp, _vp]),
    "ojasx_b200_kvq_destroy": (None, [_vp]),
    "ojasx_b200_kvq_set_static_plan": (_i, [_vp, _i]),
    "ojasx_b200_kvq_sync_len": (_i, [_vp]),
    "ojasx_b200_kvq_crop": (_i, [_vp, _i]),
    "ojasx_b200_kvq_get_memory_size": (_sz, [_vp]),
    "ojasx_b200_moe_set_gate_limit": (_i, [_vp, _f]),
    "ojasx_b200_peer_alloc": (_vp, [_sz]),
    "ojasx_b200_peer_free": (_i, [_vp]),
    "ojasx_b200_peer_export": (_i, [_vp, _vp]),
    "ojasx_b200_peer_open": (_vp, [_vp]),
    "ojasx_b200_peer_close": (_i, [_vp]),
    "ojasx_b200_peer_link_create": (_vp, [_vp, _i, _i, _sz]),
    "ojasx_b200_peer_link_destroy": (None, [_vp]),
    "ojasx_b200_peer_signal": (_i, [_vp, _vp]),
    "ojasx_b200_peer_wait": (_i, [_vp, _vp]),
    "ojasx_b200_peer_put": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "ojasx_b200_peer_take_status": (_i, [_vp]),
    "ojasx_b200_linear_forward_gather": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "ojasx_b200_linear_group_set_rows": (_i, [_vp, _i, _i]),
    "ojasx_b200_linear_group_forward_gather": (_i, [_vp, _vp, _sz, _vp, _sz, _i, _vp, _vp]),
    "ojasx_b200_moe_forward_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "ojasx_b200_moe_forward_routed_gather": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "ojasx_b200_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "ojasx_b200_rope_qk": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "ojasx_b200_add_int": (_i, [_vp, _i, _i, _vp]),
}

_lib = None


class OjasxB200Error(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (run build.py / __graft_entry__.build())."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OjasxB200Error(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(PKG_DIR, 'build.py')}`; "
                "this package has no CPU or PyTorch fallback")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().ojasx_b200_last_error().decode(errors="replace")
        raise OjasxB200Error(f"{what} failed with status {rc}" + (f": {msg}" if msg else ""))


def launch_count() -> int:
    return int(lib().ojasx_b200_launch_count())
