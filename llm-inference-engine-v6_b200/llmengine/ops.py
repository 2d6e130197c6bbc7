"""Python face of the hand-written CUDA kernels.

Each method checks what the kernel cannot check for itself (device, dtype, contiguity), passes raw
pointers and the current stream to an `extern "C"` launcher, and raises `KernelError` with the
kernel's own message when it refuses a size. There is no other implementation behind these
methods: without a CUDA device or without the compiled library they raise, they never fall back
to library or CPU code.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, rows_contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (the kernels have no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if rows_contiguous and t.dim() >= 1 and t.stride(-1) != 1 and t.shape[-1] != 1:
        raise KernelError(f"{name}: last dimension must be contiguous")


class CudaOps:
    """Loads a kernel library on first use of an op that lives in it."""

    def __init__(self):
        self._libs = {}
        self.launches = 0  # kernels launched through this object (a counter for measurements)

    # ------------------------------------------------------------------ loading
    def lib(self, name: str = "core"):
        lib = self._libs.get(name)
        if lib is None:
            if not torch.cuda.is_available():
                raise KernelError("no CUDA device: this engine runs only on its CUDA kernels")
            path = _build.kernel_library_path(name)
            lib = ctypes.CDLL(path)
            lib.llm_last_error.restype = ctypes.c_char_p
            self._libs[name] = lib
        return lib

    def _check(self, rc: int, lib) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(lib.llm_last_error().decode())

    # ------------------------------------------------------------------ elementwise
    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[n,:] (float32) = table[ids[n],:]."""
        _need(table, "embed.table"); _need(ids, "embed.ids", torch.int32); _need(out, "embed.out", torch.float32)
        lib = self.lib()
        n, dim = out.shape
        assert table.shape[1] == dim and table.is_contiguous() and out.is_contiguous() and ids.numel() >= n
        self._check(lib.llm_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out), c_int(n),
                                  c_int(dim), c_int(table.shape[0]), _stream()), lib)
        return out

    def rmsnorm(self, h: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, write_back: bool = True) -> torch.Tensor:
        """x = h[r] (+ delta[r], or + sum_p delta[p][r] for a 3-d delta); out = (w*x)/rms(x).
        With `delta` and write_back, h[r] is replaced by x (the fused residual sum).
        With `rows` (int32), output row i reads source row rows[i] and h is left as it is."""
        _need(h, "rmsnorm.h", torch.float32); _need(weight, "rmsnorm.weight", torch.float32); _need(out, "rmsnorm.out")
        lib = self.lib()
        dim = h.shape[-1]
        n_out = (rows.numel() if n_rows is None else n_rows) if rows is not None else (h.shape[0] if n_rows is None else n_rows)
        assert h.is_contiguous() and out.is_contiguous() and weight.numel() == dim and out.shape[-1] == dim
        assert out.shape[0] >= n_out
        n_part, pstride = 0, 0
        if delta is not None:
            _need(delta, "rmsnorm.delta", torch.float32)
            assert delta.is_contiguous() and delta.shape[-1] == dim
            n_part, pstride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        if rows is not None:
            _need(rows, "rmsnorm.rows", torch.int32)
            write_back = False
        self._check(lib.llm_rmsnorm(_ptr(h), _ptr(delta), c_int(n_part), c_longlong(pstride), _ptr(weight),
                                    _ptr(rows), _ptr(out), c_int(dtype_code(out.dtype)), c_int(n_out), c_int(dim),
                                    c_float(eps), c_int(1 if (write_back and delta is not None) else 0),
                                    _stream()), lib)
        return out

    def residual_add(self, h: torch.Tensor, delta: torch.Tensor, n_rows: Optional[int] = None) -> torch.Tensor:
        _need(h, "residual_add.h", torch.float32); _need(delta, "residual_add.delta", torch.float32)
        lib = self.lib()
        assert h.is_contiguous() and delta.is_contiguous()
        n = (h.shape[0] if n_rows is None else n_rows) * h.shape[-1]
        n_part, pstride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        self._check(lib.llm_residual_add(_ptr(h), _ptr(delta), c_int(n_part), c_longlong(pstride), c_longlong(n),
                                         _stream()), lib)
        return h

    def silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """gate_up [n, 2*ff] (gate columns first) -> out [n, ff] = silu(gate)*up."""
        _need(gate_up, "silu_mul.in"); _need(out, "silu_mul.out", gate_up.dtype)
        lib = self.lib()
        n, ff = out.shape
        assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape == (n, 2 * ff)
        self._check(lib.llm_silu_mul(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(n), c_int(ff),
                                     _stream()), lib)
        return out

    # ------------------------------------------------------------------ matrix products
    def gemm(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[m,n] = sum_k a[m,k]*w[n,k]; float32 accumulation; a and w of one dtype; out float32
        or that dtype. Rows may be strided views."""
        _need(a, "gemm.a"); _need(w, "gemm.w", a.dtype); _need(out, "gemm.out")
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and out.shape == (M, N)
        lib = self.lib()
        self._check(lib.llm_gemm_simt(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                      c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                      c_int(dtype_code(a.dtype)), c_int(dtype_code(out.dtype)), _stream()), lib)
        return out

    # ------------------------------------------------------------------ attention
    def rope_kv_write(self, qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                      block_table: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                      kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], n_tokens: int, nq: int,
                      nkv: int, hd: int) -> None:
        """Rotates q and k of qkv [n, (nq+2nkv)*hd] in place by the tables cos/sin [max_pos, hd/2]
        and writes k, v of each token into its page: kcache/vcache [pages, nkv, page_size, hd]."""
        _need(qkv, "rope.qkv"); _need(positions, "rope.positions", torch.int32)
        _need(token_seq, "rope.token_seq", torch.int32); _need(block_table, "rope.block_table", torch.int32)
        page_size = 1
        if kcache is not None:
            _need(kcache, "rope.kcache", qkv.dtype); _need(vcache, "rope.vcache", qkv.dtype)
            assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape == vcache.shape
            assert kcache.shape[1] == nkv and kcache.shape[3] == hd
            page_size = kcache.shape[2]
        if cos is not None:
            _need(cos, "rope.cos", torch.float32); _need(sin, "rope.sin", torch.float32)
            assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == hd // 2
        assert qkv.shape[1] == (nq + 2 * nkv) * hd and block_table.is_contiguous()
        lib = self.lib()
        self._check(lib.llm_rope_kv_write(_ptr(qkv), c_longlong(qkv.stride(0)), c_int(dtype_code(qkv.dtype)),
                                          _ptr(positions), _ptr(token_seq), _ptr(block_table),
                                          c_int(block_table.shape[1]), _ptr(cos), _ptr(sin), _ptr(kcache),
                                          _ptr(vcache), c_int(n_tokens), c_int(nq), c_int(nkv), c_int(hd),
                                          c_int(page_size), _stream()), lib)

    def paged_attention(self, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                        positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                        out: torch.Tensor, n_tokens: int, nq: int, nkv: int, hd: int, scale: float,
                        window: int = 0) -> torch.Tensor:
        """q: rows of [nq*hd] (may be a view of the qkv buffer); out [n, nq*hd]."""
        _need(q, "attention.q"); _need(kcache, "attention.kcache", q.dtype); _need(vcache, "attention.vcache", q.dtype)
        _need(out, "attention.out", q.dtype)
        _need(positions, "attention.positions", torch.int32); _need(token_seq, "attention.token_seq", torch.int32)
        _need(block_table, "attention.block_table", torch.int32)
        assert kcache.is_contiguous() and vcache.is_contiguous() and block_table.is_contiguous()
        assert kcache.shape[1] == nkv and kcache.shape[3] == hd
        lib = self.lib()
        self._check(lib.llm_paged_attention_simt(_ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                                 c_int(dtype_code(q.dtype)), _ptr(positions), _ptr(token_seq),
                                                 _ptr(block_table), c_int(block_table.shape[1]), _ptr(out),
                                                 c_longlong(out.stride(0)), c_int(n_tokens), c_int(nq), c_int(nkv),
                                                 c_int(hd), c_int(kcache.shape[2]), c_float(scale), c_int(window),
                                                 _stream()), lib)
        return out

    # ------------------------------------------------------------------ sampling
    def sample(self, logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               seeds: Optional[torch.Tensor] = None, draws: Optional[torch.Tensor] = None,
               n_rows: Optional[int] = None) -> torch.Tensor:
        """out[r] (int32) = greedy or temperature choice for logits row r (float32)."""
        _need(logits, "sample.logits", torch.float32); _need(out, "sample.out", torch.int32)
        n = logits.shape[0] if n_rows is None else n_rows
        for t, nm in ((temperature, "temperature"), (seeds, "seeds"), (draws, "draws")):
            if t is not None:
                _need(t, f"sample.{nm}", torch.float32 if nm == "temperature" else torch.int32)
        lib = self.lib()
        self._check(lib.llm_sample(_ptr(logits), c_longlong(logits.stride(0)), _ptr(temperature), _ptr(seeds),
                                   _ptr(draws), _ptr(out), c_int(n), c_int(logits.shape[1]), _stream()), lib)
        return out


_OPS: Optional[CudaOps] = None


def get_ops() -> CudaOps:
    global _OPS
    if _OPS is None:
        _OPS = CudaOps()
    return _OPS
