"""The plain C++ twins of the kernels (llmengine/csrc/ref/kernels_ref.cpp) behind numpy arrays.

Each function takes and returns numpy arrays on the host; the C++ side is a scalar loop per kernel
that restates the reference's formula. The tests compare the CUDA kernels with these twins, and the
twins with the plain Python implementation."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        from llmengine.csrc.build import reference_library_path
        _LIB = ctypes.CDLL(reference_library_path())
    return _LIB


def _p(a):
    return c_void_p(0) if a is None else a.ctypes.data_as(c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def embed(table, ids):
    table, ids = _f32(table), _i32(ids)
    out = np.empty((len(ids), table.shape[1]), dtype=np.float32)
    lib().ref_embed(_p(table), _p(ids), _p(out), c_int(len(ids)), c_int(table.shape[1]))
    return out


def rmsnorm(h, w, eps, delta=None, write_back=True, round_bf16=False):
    """-> (out, h after the fused residual sum). delta: [parts, rows, dim] or None."""
    h, w = _f32(h).copy(), _f32(w)
    out = np.empty_like(h)
    d = None if delta is None else _f32(delta)
    lib().ref_rmsnorm(_p(h), _p(d), c_int(0 if d is None else d.shape[0]), c_longlong(0 if d is None else d.shape[1] * d.shape[2]),
                      _p(w), _p(out), c_int(h.shape[0]), c_int(h.shape[1]), c_float(eps), c_int(1 if write_back else 0),
                      c_int(1 if round_bf16 else 0))
    return out, h


def gemm(a, w):
    a, w = _f32(a), _f32(w)
    out = np.empty((a.shape[0], w.shape[0]), dtype=np.float32)
    lib().ref_gemm(_p(a), _p(w), _p(out), c_int(a.shape[0]), c_int(w.shape[0]), c_int(a.shape[1]))
    return out


def silu_mul(gate, up):
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().ref_silu_mul(_p(gate), _p(up), _p(out), c_longlong(gate.size))
    return out


def rope_tables(head_dim, theta, max_pos, scaling=None):
    """scaling: (factor, low_freq_factor, high_freq_factor, original_max_positions) or None."""
    cos = np.empty((max_pos, head_dim // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    f, lo, hi, orig = scaling if scaling else (1.0, 1.0, 1.0, 0)
    lib().ref_rope_tables(c_int(head_dim), c_float(theta), c_int(1 if scaling else 0), c_float(f), c_float(lo), c_float(hi),
                          c_int(orig), c_int(max_pos), _p(cos), _p(sin))
    return cos, sin


def rope_kv_write(qkv, positions, token_seq, block_table, cos, sin, kcache, vcache, nq, nkv, hd, round_bf16=False):
    """Rotates q and k of qkv [n, (nq + 2 nkv) hd] and writes k, v into the caches [pages, nkv, page, hd]
    (both may be None). -> (qkv, kcache, vcache) after the call."""
    qkv = _f32(qkv).copy()
    positions, token_seq, block_table = _i32(positions), _i32(token_seq), _i32(block_table)
    kc = None if kcache is None else _f32(kcache).copy()
    vc = None if vcache is None else _f32(vcache).copy()
    cos = None if cos is None else _f32(cos)
    sin = None if sin is None else _f32(sin)
    page = 1 if kc is None else kc.shape[2]
    lib().ref_rope_kv_write(_p(qkv), _p(positions), _p(token_seq), _p(block_table), c_int(block_table.shape[1]), _p(cos), _p(sin),
                            _p(kc), _p(vc), c_int(qkv.shape[0]), c_int(nq), c_int(nkv), c_int(hd), c_int(page),
                            c_int(1 if round_bf16 else 0))
    return qkv, kc, vc


def paged_attention(q, kcache, vcache, positions, token_seq, block_table, nq, nkv, hd, scale, window=0):
    q, kcache, vcache = _f32(q), _f32(kcache), _f32(vcache)
    positions, token_seq, block_table = _i32(positions), _i32(token_seq), _i32(block_table)
    out = np.empty((q.shape[0], nq * hd), dtype=np.float32)
    lib().ref_paged_attention(_p(q), c_longlong(q.shape[1]), _p(kcache), _p(vcache), _p(positions), _p(token_seq), _p(block_table),
                              c_int(block_table.shape[1]), _p(out), c_longlong(nq * hd), c_int(q.shape[0]), c_int(nq), c_int(nkv),
                              c_int(hd), c_int(kcache.shape[2]), c_float(scale), c_int(window))
    return out


def sample(logits, temperature=None, seeds=None, draws=None):
    logits = _f32(logits)
    out = np.empty(logits.shape[0], dtype=np.int32)
    t = None if temperature is None else _f32(temperature)
    s = None if seeds is None else _i32(seeds)
    d = None if draws is None else _i32(draws)
    lib().ref_sample(_p(logits), c_longlong(logits.shape[1]), _p(t), _p(s), _p(d), _p(out), c_int(logits.shape[0]), c_int(logits.shape[1]))
    return out
