"""ctypes face of the CPU checkers (TEST INFRASTRUCTURE ONLY).

Two libraries are wrapped:

* ``liboracle_port.so``  -- the plain-C restatement in ``oracle_port.c`` (always buildable).
* ``_ref/libojasx_lut.so`` -- the reference's own C++ library compiled from the reference
  sources by ``oracle/Makefile`` (``make ref``); present when it was built in a container
  that holds the reference tree.  ``_ref/libojasx_lut_native.so`` is the same with
  ``-march=native``.

Only tests, ``__graft_entry__.smoke()`` and bench.py's CPU-baseline legs import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(HERE, "liboracle_port.so")
REF_PATH = os.path.join(HERE, "_ref", "libojasx_lut.so")
REF_NATIVE_PATH = os.path.join(HERE, "_ref", "libojasx_lut_native.so")

_vp = C.c_void_p
_i = C.c_int


def build(ref: bool = True) -> None:
    """Compile the port (and, when the reference tree is present, the reference library)."""
    subprocess.run(["make", "-s", "-C", HERE, "port"], check=True)
    if ref:
        subprocess.run(["make", "-s", "-C", HERE, "ref"], check=True)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _u8(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint8)


_port = None


def port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_PATH):
            build(ref=False)
        _port = C.CDLL(PORT_PATH)
        _port.oracle_linear_forward.restype = _i
        _port.oracle_linear_forward_f64.restype = _i
        _port.oracle_moe_forward.restype = _i
        _port.oracle_router_topk.restype = _i
    return _port


# ----------------------------------------------------------------------------- port
def linear_forward(codebook, codes, scales, bias, csr, x, *, block_dim, row_start=0, row_stop=None,
                   codebook_size=256):
    """y[B, rows] of the restated ``SplitManifoldLinear::forward_cpu``.  csr = (row_ptrs, cols, vals) or None."""
    codes = _u8(codes)
    M, G = codes.shape
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    K = x2.shape[1]
    assert K // block_dim == G, (K, block_dim, G)
    row_stop = M if row_stop is None else row_stop
    y = np.empty((x2.shape[0], row_stop - row_start), dtype=np.float32)
    cb, sc, bi = _f32(codebook), _f32(scales), _f32(bias)
    rp, ci, va = (None, None, None) if csr is None else (_i32(csr[0]), _i32(csr[1]), _f32(csr[2]))
    nnz = 0 if csr is None else int(va.shape[0])
    rc = port().oracle_linear_forward(_i(K), _i(M), _i(block_dim), _i(codebook_size), _ptr(cb), _ptr(codes),
                                      _ptr(sc), _ptr(bi), _i(nnz), _ptr(rp), _ptr(ci), _ptr(va),
                                      _ptr(x2), _ptr(y), _i(x2.shape[0]), _i(row_start), _i(row_stop))
    assert rc == 0, rc
    return y.reshape(*x.shape[:-1], row_stop - row_start)


def linear_forward_f64(codebook, codes, scales, bias, csr, x, *, block_dim, codebook_size=256):
    codes = _u8(codes)
    M, G = codes.shape
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    K = x2.shape[1]
    y = np.empty((x2.shape[0], M), dtype=np.float64)
    cb, sc, bi = _f32(codebook), _f32(scales), _f32(bias)
    rp, ci, va = (None, None, None) if csr is None else (_i32(csr[0]), _i32(csr[1]), _f32(csr[2]))
    nnz = 0 if csr is None else int(va.shape[0])
    rc = port().oracle_linear_forward_f64(_i(K), _i(M), _i(block_dim), _i(codebook_size), _ptr(cb), _ptr(codes),
                                          _ptr(sc), _ptr(bi), _i(nnz), _ptr(rp), _ptr(ci), _ptr(va),
                                          _ptr(x2), _ptr(y), _i(x2.shape[0]))
    assert rc == 0, rc
    return y.reshape(*x.shape[:-1], M)


def build_lut(x, codebook, *, block_dim, codebook_size=256):
    x = _f32(x)
    G = x.shape[0] // block_dim
    lut = np.empty((G, codebook_size), dtype=np.float32)
    cb = _f32(codebook)
    port().oracle_build_lut(_ptr(x), _ptr(cb), _i(G), _i(block_dim), _i(codebook_size), _ptr(lut))
    return lut


def moe_forward(cb_in, cb_down, gu_codes, gu_scales, dn_codes, dn_scales, x, idx, w, *, block_dim,
                gu_csr=None, dn_csr=None, codebook_size=256):
    """One token through the restated ``SplitManifoldMoE::forward_cpu`` (+ optional expert CSR)."""
    gu_codes, dn_codes = _u8(gu_codes), _u8(dn_codes)
    E, I2, G = gu_codes.shape
    I = I2 // 2
    H = dn_codes.shape[1]
    x, w, idx = _f32(x), _f32(w), _i32(idx)
    cbi, cbd, gs, ds = _f32(cb_in), _f32(cb_down), _f32(gu_scales), _f32(dn_scales)
    y = np.zeros(H, dtype=np.float32)

    def csr(c):
        if c is None:
            return 0, None, None, None
        return int(len(c[2])), _i32(c[0]), _i32(c[1]), _f32(c[2])

    gn, grp, gci, gva = csr(gu_csr)
    dn, drp, dci, dva = csr(dn_csr)
    rc = port().oracle_moe_forward(_i(E), _i(H), _i(I), _i(block_dim), _i(codebook_size), _ptr(cbi), _ptr(cbd),
                                   _ptr(gu_codes), _ptr(gs), _ptr(dn_codes), _ptr(ds),
                                   _i(gn), _ptr(grp), _ptr(gci), _ptr(gva),
                                   _i(dn), _ptr(drp), _ptr(dci), _ptr(dva),
                                   _ptr(x), _ptr(idx), _ptr(w), _i(len(idx)), _ptr(y))
    assert rc == 0, rc
    return y


def router_topk(x, Wr, k, return_probs=False):
    x = _f32(x)
    x2 = x.reshape(-1, x.shape[-1])
    Wr = _f32(Wr)
    B, H = x2.shape
    E = Wr.shape[0]
    idx = np.empty((B, k), dtype=np.int32)
    w = np.empty((B, k), dtype=np.float32)
    probs = np.empty((B, E), dtype=np.float32) if return_probs else None
    rc = port().oracle_router_topk(_ptr(x2), _ptr(Wr), _i(B), _i(H), _i(E), _i(k), _ptr(idx), _ptr(w), _ptr(probs))
    assert rc == 0, rc
    return (idx, w, probs) if return_probs else (idx, w)


def kv_legacy_append(k, v, *, block_dim):
    k, v = _f32(k), _f32(v)
    hd = k.shape[0]
    G = hd // block_dim
    kc, vc = np.empty(G, np.uint8), np.empty(G, np.uint8)
    ks, vs = C.c_float(), C.c_float()
    port().oracle_kv_legacy_append(_ptr(k), _ptr(v), _i(hd), _i(block_dim), _ptr(kc), _ptr(vc),
                                   C.byref(ks), C.byref(vs))
    return kc, vc, np.float32(ks.value), np.float32(vs.value)


def kv_legacy_attention(q, k_codes, v_codes, k_scales, v_scales, *, block_dim, scale=-1.0):
    q = _f32(q)
    hd = q.shape[0]
    kc, vc, ks, vs = _u8(k_codes), _u8(v_codes), _f32(k_scales), _f32(v_scales)
    out = np.zeros(hd, np.float32)
    port().oracle_kv_legacy_attention(_ptr(q), _i(hd), _i(block_dim), _i(kc.shape[0]), _ptr(kc), _ptr(vc),
                                      _ptr(ks), _ptr(vs), C.c_float(scale), _ptr(out))
    return out


def kvq_encode(vec, codebook, *, block_dim):
    vec, cb = _f32(vec), _f32(codebook)
    hd = vec.shape[-1]
    v2 = vec.reshape(-1, hd)
    out = np.empty((v2.shape[0], hd // block_dim), np.uint8)
    for i in range(v2.shape[0]):
        port().oracle_kvq_encode(_ptr(v2[i]), _i(hd), _i(block_dim), _ptr(cb), _i(cb.shape[0]), _ptr(out[i]))
    return out.reshape(*vec.shape[:-1], hd // block_dim)


def kvq_decode(q, k_codes, v_codes, k_cb, v_cb, *, block_dim, scale=-1.0, kv_block=256):
    """q [n_q, head_dim] (heads sharing this KV head); codes [T, G]; returns float64 [n_q, head_dim]."""
    q = _f32(q)
    n_q, hd = q.shape
    kc, vc = _u8(k_codes), _u8(v_codes)
    kcb, vcb = _f32(k_cb), _f32(v_cb)
    out = np.zeros((n_q, hd), np.float64)
    port().oracle_kvq_decode(_ptr(q), _i(n_q), _i(hd), _i(block_dim), _i(kc.shape[0]), _ptr(kc), _ptr(vc),
                             _ptr(kcb), _ptr(vcb), C.c_double(scale), _i(kv_block), _ptr(out))
    return out


# ------------------------------------------------------------------------ reference
class RefLib:
    """The reference's own library (handle ABI of ojasx_lut_c_api.h), host numpy in and out."""

    def __init__(self, path=REF_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        L = self.lib = C.CDLL(path)
        L.ojasx_get_version.restype = C.c_char_p
        L.ojasx_get_backend_name.restype = C.c_char_p
        L.ojasx_create_linear.restype = _vp
        L.ojasx_create_linear.argtypes = [_i, _i, _i, _i, _vp, _vp, _vp, _vp]
        L.ojasx_set_linear_outliers.restype = _i
        L.ojasx_set_linear_outliers.argtypes = [_vp, _i, _vp, _vp, _vp]
        L.ojasx_linear_forward.restype = _i
        L.ojasx_linear_forward.argtypes = [_vp, _vp, _vp, _i, _i]
        L.ojasx_destroy_linear.argtypes = [_vp]
        L.ojasx_create_moe.restype = _vp
        L.ojasx_create_moe.argtypes = [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]
        L.ojasx_moe_forward.restype = _i
        L.ojasx_moe_forward.argtypes = [_vp, _vp, _vp, _vp, _vp, _i]
        L.ojasx_destroy_moe.argtypes = [_vp]
        L.ojasx_create_kv_cache.restype = _vp
        L.ojasx_create_kv_cache.argtypes = [_i, _i, _i, _i]
        L.ojasx_kv_cache_append.restype = _i
        L.ojasx_kv_cache_append.argtypes = [_vp, _i, _vp, _vp]
        L.ojasx_kv_cache_attention.restype = _i
        L.ojasx_kv_cache_attention.argtypes = [_vp, _i, _vp, _vp, C.c_float]
        L.ojasx_destroy_kv_cache.argtypes = [_vp]

    def backend(self):
        return self.lib.ojasx_get_backend_name().decode()

    def make_linear(self, codebook, codes, scales, bias, csr, *, block_dim, codebook_size=256):
        codes = _u8(codes)
        M, G = codes.shape
        cb, sc, bi = _f32(codebook), _f32(scales), _f32(bias)
        h = self.lib.ojasx_create_linear(G * block_dim, M, block_dim, codebook_size, _ptr(cb), _ptr(codes),
                                         _ptr(sc), _ptr(bi))
        assert h
        if csr is not None:
            rp, ci, va = _i32(csr[0]), _i32(csr[1]), _f32(csr[2])
            assert self.lib.ojasx_set_linear_outliers(h, len(va), _ptr(rp), _ptr(ci), _ptr(va)) == 0
        return h

    def linear_forward_handle(self, h, x, M, threads=1):
        x = _f32(x)
        x2 = x.reshape(-1, x.shape[-1])
        y = np.zeros((x2.shape[0], M), np.float32)
        assert self.lib.ojasx_linear_forward(h, _ptr(x2), _ptr(y), x2.shape[0], threads) == 0
        return y.reshape(*x.shape[:-1], M)

    def linear_forward(self, codebook, codes, scales, bias, csr, x, *, block_dim, threads=1, codebook_size=256):
        h = self.make_linear(codebook, codes, scales, bias, csr, block_dim=block_dim, codebook_size=codebook_size)
        try:
            return self.linear_forward_handle(h, x, codes.shape[0], threads)
        finally:
            self.lib.ojasx_destroy_linear(h)

    def make_moe(self, cb_in, cb_down, gu_codes, gu_scales, dn_codes, dn_scales, *, block_dim, top_k=10):
        gu_codes, dn_codes = _u8(gu_codes), _u8(dn_codes)
        E, I2, G = gu_codes.shape
        H = dn_codes.shape[1]
        a = [_f32(cb_in), _f32(cb_down), gu_codes, _f32(gu_scales), dn_codes, _f32(dn_scales)]
        h = self.lib.ojasx_create_moe(E, H, I2 // 2, top_k, block_dim, *[_ptr(t) for t in a])
        assert h
        return h

    def moe_forward_handle(self, h, x, idx, w, H):
        x, idx, w = _f32(x), _i32(idx), _f32(w)
        y = np.zeros(H, np.float32)
        assert self.lib.ojasx_moe_forward(h, _ptr(x), _ptr(idx), _ptr(w), _ptr(y), len(idx)) == 0
        return y

    def moe_forward(self, cb_in, cb_down, gu_codes, gu_scales, dn_codes, dn_scales, x, idx, w, *, block_dim):
        h = self.make_moe(cb_in, cb_down, gu_codes, gu_scales, dn_codes, dn_scales, block_dim=block_dim,
                          top_k=len(idx))
        try:
            return self.moe_forward_handle(h, x, idx, w, dn_codes.shape[1])
        finally:
            self.lib.ojasx_destroy_moe(h)

    def kv_run(self, ks, vs, q, *, block_dim, scale=-1.0, max_seq=16):
        """Append every (k, v) row to head 0 of a fresh cache, then attend with q."""
        ks, vs, q = _f32(ks), _f32(vs), _f32(q)
        hd = q.shape[0]
        h = self.lib.ojasx_create_kv_cache(1, hd, max_seq, block_dim)
        try:
            for t in range(ks.shape[0]):
                assert self.lib.ojasx_kv_cache_append(h, 0, _ptr(ks[t]), _ptr(vs[t])) == 0
            out = np.zeros(hd, np.float32)
            assert self.lib.ojasx_kv_cache_attention(h, 0, _ptr(q), _ptr(out), C.c_float(scale)) == 0
            return out
        finally:
            self.lib.ojasx_destroy_kv_cache(h)


def ref_available(path=REF_PATH) -> bool:
    return os.path.exists(path)
