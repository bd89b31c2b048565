"""TEST INFRASTRUCTURE — numpy/ctypes front end of the CPU oracle.

Two checkers live here and neither is part of the shipped engine:

* ``Oracle``  – ``libvoxoracle.so``, the plain-C restatement in ``attn_oracle.c``.
* ``RefGgml`` – ``_ref/libvoxref_<isa>.so``, the reference's own ggml CPU backend compiled
  unmodified (see ``Makefile``), driven through ``ref_harness.cpp``.  Present only when it
  was built where the reference checkout exists; ``RefGgml.available()`` says so.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
F32, F16, Q8_0 = 0, 1, 8
PATH_AUTO, PATH_ROW, PATH_ROW_F32, PATH_TILED, PATH_F64, PATH_SPLIT_KV = 0, 1, 2, 3, 4, 5


# checkout of the reference project, if any: VOX_REFERENCE_DIR, or a directory named "reference" beside this repository
REFERENCE_DIR = os.environ.get("VOX_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref: bool = True) -> None:
    """Compile the C restatement, and the reference library when its sources are present."""
    subprocess.run(["make", "-C", HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)
    if ref and os.path.exists(os.path.join(REFERENCE_DIR, "third_party/ggml/src/ggml.c")):
        subprocess.run(["make", "-C", HERE, "-j8", "ref", f"REF={REFERENCE_DIR}"], check=True, stdout=subprocess.DEVNULL)
        # a graph node built with the reference's ggml.h, run through include/vox_attn_ggml.h (needs the engine library)
        subprocess.run(["make", "-C", HERE, "probe", f"REF={REFERENCE_DIR}"], check=True, stdout=subprocess.DEVNULL)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class _Tensor(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("ne", ctypes.c_int64 * 4), ("nb", ctypes.c_size_t * 4),
                ("data", ctypes.c_void_p)]


def kv_row_bytes(kv_type: int, D: int) -> int:
    return {F32: 4 * D, F16: 2 * D, Q8_0: 34 * (D // 32)}[kv_type]


def _contig(kv_type, ne, arr):
    t = _Tensor()
    t.type = kv_type
    rb = kv_row_bytes(kv_type, ne[0])
    for i in range(4):
        t.ne[i] = ne[i]
    t.nb[0] = {F32: 4, F16: 2, Q8_0: 34}[kv_type]
    t.nb[1] = rb
    t.nb[2] = rb * ne[1]
    t.nb[3] = rb * ne[1] * ne[2]
    t.data = arr.ctypes.data
    return t


class Oracle:
    """The C restatement.  Arrays are numpy, laid out as the reference lays tensors out with
    dim0 fastest: q ``[B, H, n_q, D]`` f32, k/v ``[B, HK, n_kv, D]`` (f32 / f16 arrays, or
    uint8 ``[B, HK, n_kv, 34*D/32]`` for q8_0), mask ``[ne3, ne2, n_q, n_kv]`` f16 bits."""

    def __init__(self):
        so = os.path.join(HERE, "libvoxoracle.so")
        src = os.path.join(HERE, "attn_oracle.c")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            build(ref=False)
        self.lib = ctypes.CDLL(so)
        self.lib.voxo_flash_attn_ext.restype = ctypes.c_int
        self.lib.voxo_fp32_to_fp16.restype = ctypes.c_uint16
        self.lib.voxo_fp32_to_fp16.argtypes = [ctypes.c_float]
        self.lib.voxo_fp16_to_fp32.restype = ctypes.c_float
        self.lib.voxo_fp16_to_fp32.argtypes = [ctypes.c_uint16]

    def quantize_q8_0(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        assert x.shape[-1] % 32 == 0
        out = np.zeros(x.shape[:-1] + (x.shape[-1] // 32 * 34,), np.uint8)
        self.lib.voxo_quantize_row_q8_0(_ptr(x), _ptr(out), ctypes.c_int64(x.size))
        return out

    def dequantize_q8_0(self, blocks: np.ndarray) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, np.uint8)
        out = np.zeros(blocks.shape[:-1] + (blocks.shape[-1] // 34 * 32,), np.float32)
        self.lib.voxo_dequantize_row_q8_0(_ptr(blocks), _ptr(out), ctypes.c_int64(out.size))
        return out

    def kv_store(self, x: np.ndarray, kv_type: int) -> np.ndarray:
        """What appending f32 rows to an f16 / q8_0 cache stores."""
        x = np.ascontiguousarray(x, np.float32)
        D = x.shape[-1]
        if kv_type == F32:
            return x.copy()
        if kv_type == F16:
            out = np.zeros(x.shape, np.uint16)
        else:
            out = np.zeros(x.shape[:-1] + (D // 32 * 34,), np.uint8)
        self.lib.voxo_kv_store(_ptr(x), ctypes.c_int64(x.size // D), ctypes.c_int64(D), kv_type, _ptr(out))
        return out.view(np.float16) if kv_type == F16 else out

    def rope_table(self, positions, freq_base=10000.0, attn_factor=1.0, freq_factors=None, n_dims=64) -> np.ndarray:
        """(cos, sin) table [n_pos, n_dims/2, 2] of the reference's rotary embedding."""
        pos = np.ascontiguousarray(positions, np.int32)
        ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, np.float32)
        out = np.zeros((len(pos), n_dims // 2, 2), np.float32)
        self.lib.voxo_rope_table(_ptr(pos), ctypes.c_int64(len(pos)), int(n_dims), ctypes.c_float(freq_base),
                                 ctypes.c_float(attn_factor), _ptr(ff), _ptr(out))
        return out

    def rope(self, x, table, pos_index=None) -> np.ndarray:
        """NEOX rotation of rows x[..., n_dims]; row r uses table[pos_index[r]] (default: x.shape[0]
        leading index, i.e. x is [n_pos, ..., n_dims])."""
        x = np.array(x, np.float32, order="C")
        n_dims = x.shape[-1]
        rows = x.reshape(-1, n_dims)
        if pos_index is None:
            per = rows.shape[0] // x.shape[0]
            pos_index = np.repeat(np.arange(x.shape[0], dtype=np.int32), per)
        pos_index = np.ascontiguousarray(pos_index, np.int32)
        assert len(pos_index) == rows.shape[0]
        self.lib.voxo_rope_neox(_ptr(rows), ctypes.c_int64(rows.shape[0]), int(n_dims), _ptr(np.ascontiguousarray(table, np.float32)),
                                _ptr(pos_index))
        return rows.reshape(x.shape)

    def mul_mat_f16(self, x, w) -> np.ndarray:
        """ggml_mul_mat with f16 weights: x [n_tok, k] f32, w [n_out, k] f16 -> [n_tok, n_out] f32."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float16)
        n_tok, k = x.shape
        n_out = w.shape[0]
        out = np.zeros((n_tok, n_out), np.float32)
        i64 = ctypes.c_int64
        self.lib.voxo_mul_mat_f16(_ptr(x), _ptr(w.view(np.uint16)), i64(n_tok), i64(k), i64(n_out), _ptr(out))
        return out

    @staticmethod
    def mul_mat_f16_blas(x, w) -> np.ndarray:
        """The same product for sizes the scalar loop above would take minutes on: the activations rounded to f16, then an
        f32 matrix product by numpy.  Same exact products, another order of the f32 sums."""
        x16 = np.ascontiguousarray(x, np.float32).astype(np.float16).astype(np.float32)
        return x16 @ np.ascontiguousarray(w, np.float16).astype(np.float32).T

    def rms_norm_mul(self, x, w, eps) -> np.ndarray:
        """MiniCPMModel::rms_norm: x [n_tok, k] f32, w [k] f32 -> [n_tok, k] f32."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        out = np.zeros_like(x)
        i64 = ctypes.c_int64
        self.lib.voxo_rms_norm_mul(_ptr(x), _ptr(w), ctypes.c_float(eps), i64(x.shape[0]), i64(x.shape[1]), _ptr(out))
        return out

    def swiglu(self, gate, up) -> np.ndarray:
        """ggml_swiglu_split: silu(gate) * up, f32, any shape."""
        gate = np.ascontiguousarray(gate, np.float32)
        up = np.ascontiguousarray(up, np.float32)
        out = np.zeros_like(gate)
        self.lib.voxo_swiglu(_ptr(gate), _ptr(up), ctypes.c_int64(gate.size), _ptr(out))
        return out

    def causal_mask(self, positions, total_len: int) -> np.ndarray:
        pos = np.ascontiguousarray(positions, np.int32)
        out = np.zeros((len(pos), total_len), np.uint16)
        self.lib.voxo_causal_mask(_ptr(pos), len(pos), total_len, _ptr(out))
        return out.view(np.float16)

    def cfg_pair_mask(self, seq: int) -> np.ndarray:
        out = np.zeros((2 * seq, 2 * seq), np.uint16)
        self.lib.voxo_cfg_pair_mask(seq, _ptr(out))
        return out.view(np.float16)

    def attn(self, q, k, v, mask=None, scale=0.125, kv_type=F16, path=PATH_AUTO, n_chunks=1) -> np.ndarray:
        q = np.ascontiguousarray(q, np.float32)
        B, H, n_q, D = q.shape
        k = np.ascontiguousarray(k)
        v = np.ascontiguousarray(v)
        HK, n_kv = k.shape[1], k.shape[2]
        tq = _contig(F32, (D, n_q, H, B), q)
        tk = _contig(kv_type, (D, n_kv, HK, B), k)
        tv = _contig(kv_type, (D, n_kv, HK, B), v)
        tm = None
        if mask is not None:
            mask = np.ascontiguousarray(mask)
            assert mask.dtype == np.float16 and mask.ndim == 4
            ne3, ne2, mq, mkv = mask.shape
            tm = _contig(F16, (mkv, mq, ne2, ne3), mask)
        out = np.zeros((B, n_q, H, D), np.float32)
        rc = self.lib.voxo_flash_attn_ext(ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                          ctypes.byref(tm) if tm is not None else None,
                                          ctypes.c_float(scale), path, n_chunks, _ptr(out))
        if rc != 0:
            raise ValueError(f"oracle rejected the operands (code {rc})")
        return out


def _isa() -> str:
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return "v3"
    need = ("avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512cd")
    return "v4" if all(f in flags for f in need) else "v3"


class RefGgml:
    """The reference's ggml CPU backend, unmodified.  Same array conventions as ``Oracle``;
    k/v may carry a leading layer axis when ``n_layers`` > 1 (one graph of that many nodes)."""

    @staticmethod
    def path() -> str:
        return os.path.join(HERE, "_ref", f"libvoxref_{_isa()}.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.path())

    def __init__(self):
        self.lib = ctypes.CDLL(self.path())
        self.lib.voxref_attn.restype = ctypes.c_int
        self.isa = _isa()

    def quantize_q8_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape[:-1] + (x.shape[-1] // 32 * 34,), np.uint8)
        self.lib.voxref_quantize_q8_0(_ptr(x), _ptr(out), ctypes.c_int64(x.size))
        return out

    def dequantize_q8_0(self, blocks):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        out = np.zeros(blocks.shape[:-1] + (blocks.shape[-1] // 34 * 32,), np.float32)
        self.lib.voxref_dequantize_q8_0(_ptr(blocks), _ptr(out), ctypes.c_int64(out.size))
        return out

    def fp32_to_fp16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape, np.uint16)
        self.lib.voxref_fp32_to_fp16(_ptr(x), _ptr(out), ctypes.c_int64(x.size))
        return out.view(np.float16)

    def rope(self, x, positions, freq_base=10000.0, attn_factor=1.0, freq_factors=None, n_ctx_orig=32768, n_threads=1):
        """ggml_rope_ext (NEOX) on x [n_tok, n_heads, D] f32 with one position per token."""
        x = np.ascontiguousarray(x, np.float32)
        n_tok, n_heads, D = x.shape
        pos = np.ascontiguousarray(positions, np.int32)
        ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, np.float32)
        out = np.zeros_like(x)
        i64 = ctypes.c_int64
        rc = self.lib.voxref_rope(_ptr(x), i64(D), i64(n_heads), i64(n_tok), _ptr(pos), _ptr(ff), int(n_ctx_orig),
                                  ctypes.c_float(freq_base), ctypes.c_float(attn_factor), int(n_threads), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"reference harness failed (code {rc})")
        return out

    def mul_mat_f16(self, x, w, n_threads=1) -> np.ndarray:
        """The reference's ggml_mul_mat: x [n_tok, k] f32, w [n_out, k] f16 -> [n_tok, n_out] f32."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float16)
        n_tok, k = x.shape
        n_out = w.shape[0]
        out = np.zeros((n_tok, n_out), np.float32)
        i64 = ctypes.c_int64
        rc = self.lib.voxref_mul_mat_f16(_ptr(w.view(np.uint16)), _ptr(x), i64(k), i64(n_out), i64(n_tok), int(n_threads), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"reference harness failed (code {rc})")
        return out

    def rms_norm_mul(self, x, w, eps, n_threads=1) -> np.ndarray:
        """The reference's ggml_rms_norm + ggml_mul: x [n_tok, k] f32, w [k] f32 -> [n_tok, k] f32."""
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        out = np.zeros_like(x)
        i64 = ctypes.c_int64
        rc = self.lib.voxref_rms_norm_mul(_ptr(x), _ptr(w), ctypes.c_float(eps), i64(x.shape[1]), i64(x.shape[0]), int(n_threads), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"reference harness failed (code {rc})")
        return out

    def swiglu(self, gate, up, n_threads=1) -> np.ndarray:
        """The reference's ggml_swiglu_split: gate, up [n_tok, n] f32 -> [n_tok, n] f32."""
        gate = np.ascontiguousarray(gate, np.float32)
        up = np.ascontiguousarray(up, np.float32)
        out = np.zeros_like(gate)
        i64 = ctypes.c_int64
        rc = self.lib.voxref_swiglu(_ptr(gate), _ptr(up), i64(gate.shape[1]), i64(gate.shape[0]), int(n_threads), _ptr(out))
        if rc != 0:
            raise RuntimeError(f"reference harness failed (code {rc})")
        return out

    def attn(self, q, k, v, mask=None, scale=0.125, kv_type=F16, n_threads=1, iters=1, use_ref=False,
             n_layers=1, return_ms=False):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k)
        v = np.ascontiguousarray(v)
        if n_layers == 1 and q.ndim == 4:
            q, k, v = q[None], k[None], v[None]
        L, B, H, n_q, D = q.shape
        assert L == n_layers
        HK, n_kv = k.shape[2], k.shape[3]
        ne2 = ne3 = 1
        if mask is not None:
            mask = np.ascontiguousarray(mask)
            assert mask.dtype == np.float16 and mask.ndim == 4
            ne3, ne2 = mask.shape[0], mask.shape[1]
        out = np.zeros((L, B, n_q, H, D), np.float32)
        ms = np.zeros(iters, np.float64)
        i64 = ctypes.c_int64
        rc = self.lib.voxref_attn(L, _ptr(q), _ptr(k), _ptr(v), _ptr(mask), kv_type, i64(D), i64(n_q), i64(n_kv),
                                  i64(H), i64(HK), i64(B), i64(ne2), i64(ne3), ctypes.c_float(scale),
                                  int(n_threads), int(iters), int(bool(use_ref)), _ptr(out), _ptr(ms))
        if rc != 0:
            raise RuntimeError(f"reference harness failed (code {rc})")
        out = out[0] if n_layers == 1 else out
        return (out, ms) if return_ms else out
