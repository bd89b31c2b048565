"""ctypes binding of ``include/vox_attn.h``.

Every wrapper raises ``VoxError`` carrying the C status and the engine's error string; nothing
here computes attention.  Tensors are described the way the reference describes them
(type, ``ne`` with dim 0 fastest, byte strides ``nb``), see ``Tensor.from_torch``.
"""
from __future__ import annotations

import ctypes as C
import weakref
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
F32, F16, Q8_0 = 0, 1, 8

STATUS = {0: "OK", 1: "INVALID_ARGUMENT", 2: "UNSUPPORTED", 3: "WORKSPACE_TOO_SMALL", 4: "CUDA_ERROR", 5: "TIMEOUT",
          6: "OUT_OF_MEMORY", 7: "DEVICE_STATE"}


class VoxError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS.get(status, status)}: {message}")
        self.status = status
        self.status_name = STATUS.get(status, str(status))


class Tensor(C.Structure):
    _fields_ = [("type", C.c_int32), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("data", C.c_void_p)]

    @classmethod
    def make(cls, type_, ne, nb, data):
        t = cls()
        t.type = type_
        for i in range(4):
            t.ne[i] = ne[i]
            t.nb[i] = nb[i]
        t.data = data
        return t

    @classmethod
    def from_torch(cls, x, type_=None):
        """A torch tensor of shape [d3, d2, d1, d0] (any strides, dim0 contiguous) as a ggml-style
        tensor with ne = [d0, d1, d2, d3].  uint8 tensors with last dim 34*k are q8_0 rows."""
        import torch
        assert x.dim() == 4
        if type_ is None:
            type_ = {torch.float32: F32, torch.float16: F16, torch.uint8: Q8_0}[x.dtype]
        es = x.element_size()
        ne = [x.shape[3], x.shape[2], x.shape[1], x.shape[0]]
        nb = [x.stride(3) * es, x.stride(2) * es, x.stride(1) * es, x.stride(0) * es]
        if type_ == Q8_0:
            ne[0] = x.shape[3] // 34 * 32
            nb[0] = 34
        return cls.make(type_, ne, nb, x.data_ptr())

    @classmethod
    def none(cls):
        return cls.make(F16, [0, 0, 0, 0], [0, 0, 0, 0], None)


class AttnArgs(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("mask", Tensor), ("dst", Tensor), ("scale", C.c_float),
                ("max_bias", C.c_float), ("logit_softcap", C.c_float), ("has_sinks", C.c_int32)]


class KVConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_streams", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("max_len", C.c_int32), ("type", C.c_int32)]


class DecodeArgs(C.Structure):
    _fields_ = [("cache", C.c_void_p), ("layer", C.c_int32), ("n_streams", C.c_int32), ("n_heads", C.c_int32),
                ("kv_len", C.c_void_p), ("kv_bound", C.c_int32), ("q", C.c_void_p), ("q_nb_head", C.c_size_t),
                ("q_nb_stream", C.c_size_t), ("dst", C.c_void_p), ("scale", C.c_float), ("k_new", C.c_void_p),
                ("v_new", C.c_void_p), ("new_nb_head", C.c_size_t), ("new_nb_stream", C.c_size_t), ("flags", C.c_uint32),
                ("rope_table", C.c_void_p), ("stream_order", C.c_void_p)]


class QkvArgs(C.Structure):
    _fields_ = [("n_streams", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("x", C.c_void_p), ("x_nb_stream", C.c_size_t), ("w_qkv", C.c_void_p),
                ("w_nb_row", C.c_size_t), ("w_type", C.c_int32), ("rope_table", C.c_void_p), ("q", C.c_void_p),
                ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("cache", C.c_void_p), ("layer", C.c_int32), ("positions", C.c_void_p),
                ("pos_offset", C.c_int32)]


class LinearArgs(C.Structure):
    _fields_ = [("n_tokens", C.c_int32), ("k_dim", C.c_int32), ("n_out", C.c_int32), ("mode", C.c_int32), ("x", C.c_void_p),
                ("x_nb_token", C.c_size_t), ("w", C.c_void_p), ("w_nb_row", C.c_size_t), ("w_type", C.c_int32), ("out", C.c_void_p),
                ("out_nb_token", C.c_size_t), ("residual", C.c_void_p), ("res_nb_token", C.c_size_t), ("scale", C.c_float),
                ("norm_weight", C.c_void_p), ("norm_eps", C.c_float), ("x_type", C.c_int32), ("out_type", C.c_int32)]


LINEAR_PLAIN, LINEAR_RESIDUAL, LINEAR_SWIGLU = 0, 1, 2


class RopeConfig(C.Structure):
    _fields_ = [("freq_base", C.c_float), ("attn_factor", C.c_float), ("freq_factors", C.c_void_p)]


class LocditArgs(C.Structure):
    _fields_ = [("n_streams", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("seq", C.c_int32), ("head_dim", C.c_int32), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
                ("dst", C.c_void_p), ("scale", C.c_float)]


class GroupConfig(C.Structure):
    _fields_ = [("n_streams", C.c_int32), ("base_layers", C.c_int32), ("res_layers", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("max_len", C.c_int32), ("kv_type", C.c_int32),
                ("locdit_layers", C.c_int32), ("locdit_seq", C.c_int32), ("cfm_steps", C.c_int32),
                ("cfm_zero_init_steps", C.c_int32)]


class StepBuffers(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("lm_q", "lm_k_new", "lm_v_new", "lm_out", "dit_q", "dit_k", "dit_v", "dit_out", "lm_hidden")]


def library_path() -> str:
    """The in-tree build, or another build of the same sources named by VOX_ATTN_LIBRARY (developer aid)."""
    return os.environ.get("VOX_ATTN_LIBRARY") or os.path.join(HERE, "libvoxattn.so")


def declared_symbols() -> list[str]:
    """Every function ``include/vox_attn.h`` declares."""
    text = open(os.path.join(ROOT, "include", "vox_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vox_[a-z0-9_]+)\s*\(", text)))


_LIB = None


def lib() -> C.CDLL:
    """Load the engine.  Raises if it has not been built: there is no other implementation."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python voxcpm.cpp_b200/build.py` (nvcc, sm_100a); "
                           "the engine has no CPU or PyTorch fallback")
    L = C.CDLL(path)
    vp, i32, sz = C.c_void_p, C.c_int, C.c_size_t
    sig = {
        "vox_engine_create": (i32, [i32, C.POINTER(vp)]),
        "vox_engine_destroy": (None, [vp]),
        "vox_attn_last_error_string": (C.c_char_p, []),
        "vox_attn_status_string": (C.c_char_p, [i32]),
        "vox_engine_launch_count": (C.c_uint64, [vp]),
        "vox_engine_sync_status": (i32, [vp, vp]),
        "vox_engine_selftest_wait": (i32, [vp, C.c_longlong, vp]),
        "vox_rope_table": (i32, [vp, C.POINTER(RopeConfig), vp, i32, i32, vp, vp]),
        "vox_group_set_rope": (i32, [vp, C.POINTER(RopeConfig), vp]),
        "vox_group_set_qkv_weights": (i32, [vp, vp, i32, sz, sz]),
        "vox_group_set_bound": (i32, [vp, i32]),
        "vox_group_advance": (i32, [vp, i32]),
        "vox_attn_supported": (i32, [C.POINTER(AttnArgs)]),
        "vox_attn_workspace_bytes": (sz, [C.POINTER(AttnArgs)]),
        "vox_attn_forward": (i32, [vp, C.POINTER(AttnArgs), vp, sz, vp]),
        "vox_attn_forward_host": (i32, [vp, C.POINTER(AttnArgs), vp]),
        "vox_attn_prefill": (i32, [vp, C.POINTER(AttnArgs), vp, sz, vp]),
        "vox_attn_prefill_workspace_bytes": (sz, [C.POINTER(AttnArgs)]),
        "vox_kv_create": (i32, [vp, C.POINTER(KVConfig), C.POINTER(vp)]),
        "vox_kv_destroy": (None, [vp]),
        "vox_kv_clear": (i32, [vp, i32, vp]),
        "vox_kv_bytes": (sz, [vp]),
        "vox_kv_append": (i32, [vp, i32, i32, i32, vp, i32, vp, vp, sz, sz, sz, vp]),
        "vox_kv_view": (i32, [vp, i32, i32, i32, C.POINTER(Tensor), C.POINTER(Tensor)]),
        "vox_kv_export": (i32, [vp, i32, i32, i32, vp, vp]),
        "vox_kv_import": (i32, [vp, i32, i32, i32, vp, vp]),
        "vox_kv_copy_from": (i32, [vp, vp, vp]),
        "vox_qkv_workspace_bytes": (sz, [i32, i32]),
        "vox_qkv_project": (i32, [vp, C.POINTER(QkvArgs), vp, sz, vp]),
        "vox_linear_workspace_bytes": (sz, [i32, i32]),
        "vox_linear": (i32, [vp, C.POINTER(LinearArgs), vp, sz, vp]),
        "vox_attn_decode_workspace_bytes": (sz, [i32, i32, i32, i32]),
        "vox_attn_decode": (i32, [vp, C.POINTER(DecodeArgs), vp, sz, vp]),
        "vox_attn_decode_static": (i32, [vp, C.POINTER(DecodeArgs), vp]),
        "vox_attn_locdit_step": (i32, [vp, C.POINTER(LocditArgs), vp]),
        "vox_group_create": (i32, [vp, C.POINTER(GroupConfig), C.POINTER(vp)]),
        "vox_group_destroy": (None, [vp]),
        "vox_group_cache": (vp, [vp, i32]),
        "vox_group_set_kv_len": (i32, [vp, vp]),
        "vox_group_get_kv_len": (i32, [vp, vp]),
        "vox_group_fill_synthetic": (i32, [vp, C.c_uint64, vp]),
        "vox_group_step_bytes": (sz, [vp, i32]),
        "vox_group_step": (i32, [vp, C.POINTER(StepBuffers), i32, vp]),
        "vox_group_step_host": (i32, [vp, C.POINTER(StepBuffers), i32]),
        "vox_partition_streams": (i32, [vp, i32, i32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = L
    return L


def _check(rc: int):
    if rc != 0:
        raise VoxError(rc, lib().vox_attn_last_error_string().decode())


def _stream_ptr(stream):
    if stream is None:
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return C.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)


def attn_args(q, k, v, dst, mask=None, scale=0.125, k_type=None, v_type=None) -> AttnArgs:
    a = AttnArgs()
    a.q = Tensor.from_torch(q)
    a.k = Tensor.from_torch(k, k_type)
    a.v = Tensor.from_torch(v, v_type)
    a.mask = Tensor.from_torch(mask) if mask is not None else Tensor.none()
    a.dst = Tensor.from_torch(dst)
    a.scale = scale
    return a


class Engine:
    """One per GPU (``vox_engine``)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        _check(lib().vox_engine_create(device, C.byref(h)))
        self.h = h
        self.device = device
        self._ws = None
        self._children = weakref.WeakSet()  # caches and groups created from this engine: they go before it does

    def close(self):
        if self.h:
            for child in list(self._children):
                child.close()
            lib().vox_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def launches(self) -> int:
        return int(lib().vox_engine_launch_count(self.h))

    def sync_status(self, stream=None):
        _check(lib().vox_engine_sync_status(self.h, _stream_ptr(stream)))

    def rope_table(self, positions, freq_base=10000.0, attn_factor=1.0, freq_factors=None, pos_offset=0, stream=None):
        """``vox_rope_table``: positions int32 device [n] -> (cos, sin) table [n, 32, 2] f32 on the device."""
        import torch
        n = positions.numel()
        table = torch.empty((n, 32, 2), dtype=torch.float32, device=positions.device)
        cfg = RopeConfig(freq_base, attn_factor, freq_factors.data_ptr() if freq_factors is not None else None)
        _check(lib().vox_rope_table(self.h, C.byref(cfg), positions.data_ptr(), pos_offset, n, table.data_ptr(), _stream_ptr(stream)))
        return table

    def selftest_wait(self, limit_cycles=2_000_000, stream=None):
        """Launches the wait that nothing satisfies; the next ``sync_status`` raises TIMEOUT."""
        _check(lib().vox_engine_selftest_wait(self.h, limit_cycles, _stream_ptr(stream)))

    def workspace(self, nbytes: int):
        import torch
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=f"cuda:{self.device}")
        return self._ws

    def forward(self, q, k, v, mask=None, scale=0.125, stream=None, dst=None):
        """``ggml_flash_attn_ext`` on device tensors: q [B,H,n_q,64] f32, k/v [B,HK,n_kv,*],
        mask [ne3,ne2,n_q,n_kv] f16 or None.  Returns [B,n_q,H,64] f32."""
        import torch
        B, H, n_q, D = q.shape
        if dst is None:
            dst = torch.empty((B, n_q, H, D), dtype=torch.float32, device=q.device)
        a = attn_args(q, k, v, dst, mask, scale)
        ws_bytes = lib().vox_attn_workspace_bytes(C.byref(a))
        ws = self.workspace(ws_bytes)
        _check(lib().vox_attn_forward(self.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(stream)))
        return dst

    def forward_host(self, q, k, v, mask=None, scale=0.125, stream=None):
        """Same operator on HOST tensors (copies in the timed path)."""
        import torch
        B, H, n_q, D = q.shape
        dst = torch.empty((B, n_q, H, D), dtype=torch.float32)
        a = attn_args(q, k, v, dst, mask, scale)
        _check(lib().vox_attn_forward_host(self.h, C.byref(a), _stream_ptr(stream)))
        return dst

    def prefill(self, q, k, v, scale=0.125, stream=None, dst=None):
        import torch
        B, H, n_q, D = q.shape
        if dst is None:
            dst = torch.empty((B, n_q, H, D), dtype=torch.float32, device=q.device)
        a = attn_args(q, k, v, dst, None, scale)
        ws_bytes = lib().vox_attn_prefill_workspace_bytes(C.byref(a))
        ws = self.workspace(ws_bytes)
        _check(lib().vox_attn_prefill(self.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(stream)))
        return dst

    def qkv_project(self, x, w, n_heads, n_kv_heads, rope_table=None, cache=None, layer=0, positions=None, stream=None):
        """``vox_qkv_project``: x [n_streams, hidden] f32, w [(H + 2 HK) * 64, hidden] f16 (ggml's layout).  Returns
        q [n_streams, H, 64] and, without a cache, k_new / v_new [n_streams, HK, 64]; with one, the rows are stored
        at ``positions`` and (q, None, None) comes back."""
        import torch
        S, hidden = x.shape
        q = torch.empty((S, n_heads, 64), dtype=torch.float32, device=x.device)
        k_new = v_new = None
        a = QkvArgs(S, hidden, n_heads, n_kv_heads, 64, x.data_ptr(), x.stride(0) * 4, w.data_ptr(), w.stride(0) * 2, F16)
        a.rope_table = rope_table.data_ptr() if rope_table is not None else None
        a.q = q.data_ptr()
        if cache is None:
            k_new = torch.empty((S, n_kv_heads, 64), dtype=torch.float32, device=x.device)
            v_new = torch.empty((S, n_kv_heads, 64), dtype=torch.float32, device=x.device)
            a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
        else:
            a.cache, a.layer, a.positions = cache.h, layer, positions.data_ptr()
        ws = self.workspace(lib().vox_qkv_workspace_bytes(S, hidden))
        _check(lib().vox_qkv_project(self.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(stream)))
        return q, k_new, v_new

    def linear(self, x, w, mode=LINEAR_PLAIN, residual=None, scale=1.0, norm_weight=None, norm_eps=0.0, out=None, out_f16=False,
               stream=None):
        """``vox_linear``: x [n_tokens, k] f32 or f16, w [rows, k] f16 (ggml's layout) -> [n_tokens, n_out] f32 (f16 with
        ``out_f16``); n_out = rows, or rows / 2 in the SwiGLU mode (gate rows first).  ``residual`` [n_tokens, n_out] for
        LINEAR_RESIDUAL."""
        import torch
        n_tok, k = x.shape
        x16 = x.dtype == torch.float16
        n_out = w.shape[0] // 2 if mode == LINEAR_SWIGLU else w.shape[0]
        if out is None:
            out = torch.empty((n_tok, n_out), dtype=torch.float16 if out_f16 else torch.float32, device=x.device)
        out16 = out.dtype == torch.float16
        a = LinearArgs(n_tok, k, n_out, mode, x.data_ptr(), x.stride(0) * (2 if x16 else 4), w.data_ptr(), w.stride(0) * 2, F16,
                       out.data_ptr(), out.stride(0) * (2 if out16 else 4))
        if residual is not None:
            a.residual, a.res_nb_token = residual.data_ptr(), residual.stride(0) * 4
        a.scale = scale
        if norm_weight is not None:
            a.norm_weight, a.norm_eps = norm_weight.data_ptr(), norm_eps
        a.x_type, a.out_type = (F16 if x16 else F32), (F16 if out16 else F32)
        ws = self.workspace(max(256, lib().vox_linear_workspace_bytes(n_tok, k)))
        _check(lib().vox_linear(self.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(stream)))
        return out

    def supported(self, a: AttnArgs) -> bool:
        return bool(lib().vox_attn_supported(C.byref(a)))

    def locdit_step(self, q, k, v, scale=0.125, stream=None, dst=None):
        """q [S,L,2,H,seq,64], k/v [S,L,2,HK,seq,64] f32 -> [S,L,2,seq,H,64]."""
        import torch
        S, L, two, H, seq, D = q.shape
        HK = k.shape[3]
        if dst is None:
            dst = torch.empty((S, L, 2, seq, H, D), dtype=torch.float32, device=q.device)
        a = LocditArgs(S, L, H, HK, seq, D, q.data_ptr(), k.data_ptr(), v.data_ptr(), dst.data_ptr(), scale)
        _check(lib().vox_attn_locdit_step(self.h, C.byref(a), _stream_ptr(stream)))
        return dst


class KVCache:
    """``vox_kv_cache``: the f16 / q8_0 replacement of MiniCPMKVCache."""

    def __init__(self, engine: Engine, n_layers, n_streams, n_kv_heads=2, max_len=4096, type_=F16, head_dim=64, handle=None):
        self.engine = engine
        self.cfg = KVConfig(n_layers, n_streams, n_kv_heads, head_dim, max_len, type_)
        self.owned = handle is None
        if handle is None:
            h = C.c_void_p()
            _check(lib().vox_kv_create(engine.h, C.byref(self.cfg), C.byref(h)))
            self.h = h
            engine._children.add(self)
        else:
            self.h = C.c_void_p(handle)

    def close(self):
        if self.h and self.owned and self.engine.h:  # a cache never outlives its engine (Engine.close closes it first)
            lib().vox_kv_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def nbytes(self):
        return lib().vox_kv_bytes(self.h)

    def clear(self, stream_id=-1, stream=None):
        _check(lib().vox_kv_clear(self.h, stream_id, _stream_ptr(stream)))

    def append(self, layer, k, v, positions=None, pos0=0, stream=None):
        """k, v: [n_streams, n_tok, HK, 64] f32 device tensors (the projection layout)."""
        S, T, HK, D = k.shape
        es = 4
        _check(lib().vox_kv_append(self.h, layer, S, T, C.c_void_p(positions.data_ptr()) if positions is not None else None,
                                   pos0, C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()), k.stride(2) * es,
                                   k.stride(1) * es, k.stride(0) * es, _stream_ptr(stream)))

    def view(self, layer, stream_id, seq_len):
        k, v = Tensor(), Tensor()
        _check(lib().vox_kv_view(self.h, layer, stream_id, seq_len, C.byref(k), C.byref(v)))
        return k, v

    def row_bytes(self):
        return 128 if self.cfg.type == F16 else 68

    def export(self, layer, stream_id, n_pos):
        import numpy as np
        shape = (self.cfg.n_kv_heads, n_pos, self.row_bytes())
        k = np.zeros(shape, np.uint8)
        v = np.zeros(shape, np.uint8)
        _check(lib().vox_kv_export(self.h, layer, stream_id, n_pos, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))
        if self.cfg.type == F16:
            return k.view(np.float16), v.view(np.float16)
        return k, v

    def import_(self, layer, stream_id, k, v):
        import numpy as np
        k = np.ascontiguousarray(k)
        v = np.ascontiguousarray(v)
        n_pos = k.shape[1]
        _check(lib().vox_kv_import(self.h, layer, stream_id, n_pos, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))

    def copy_from(self, other: "KVCache", stream=None):
        _check(lib().vox_kv_copy_from(self.h, other.h, _stream_ptr(stream)))

    def _decode_args(self, layer, q, kv_len, kv_bound, dst, scale, k_new, v_new, cache_stable, rope_table, stream_order):
        S, H, D = q.shape
        a = DecodeArgs(self.h, layer, S, H, kv_len.data_ptr(), kv_bound, q.data_ptr(), q.stride(1) * 4, q.stride(0) * 4,
                       dst.data_ptr(), scale)
        a.flags = 1 if cache_stable else 0
        a.rope_table = rope_table.data_ptr() if rope_table is not None else None
        a.stream_order = stream_order.data_ptr() if stream_order is not None else None
        if k_new is not None or v_new is not None:
            a.k_new = k_new.data_ptr() if k_new is not None else None
            a.v_new = v_new.data_ptr() if v_new is not None else None
            ref = k_new if k_new is not None else v_new
            a.new_nb_head, a.new_nb_stream = ref.stride(1) * 4, ref.stride(0) * 4
        return a

    def decode(self, layer, q, kv_len, kv_bound, scale=0.125, stream=None, dst=None, k_new=None, v_new=None, cache_stable=False,
               rope_table=None, stream_order=None):
        """q [n_streams, H, 64] f32, kv_len int32 device [n_streams] -> [n_streams, H, 64].

        ``k_new`` / ``v_new`` [n_streams, HK, 64] f32: the token's own rows, stored at position
        ``kv_len - 1`` by the same launch (no separate append)."""
        import torch
        S, H, D = q.shape
        if dst is None:
            dst = torch.empty((S, H, D), dtype=torch.float32, device=q.device)
        ws_bytes = lib().vox_attn_decode_workspace_bytes(S, H, self.cfg.n_kv_heads, kv_bound)
        ws = self.engine.workspace(ws_bytes)
        a = self._decode_args(layer, q, kv_len, kv_bound, dst, scale, k_new, v_new, cache_stable, rope_table, stream_order)
        _check(lib().vox_attn_decode(self.engine.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr(stream)))
        return dst

    def decode_static(self, layer, q, kv_len, kv_bound, dst, scale=0.125, stream=None, k_new=None, v_new=None, rope_table=None):
        """``vox_attn_decode_static``: the caller passes inputs and the output only; the split-KV
        scratch is the array built into the library, so nothing is allocated by the call."""
        a = self._decode_args(layer, q, kv_len, kv_bound, dst, scale, k_new, v_new, False, rope_table, None)
        _check(lib().vox_attn_decode_static(self.engine.h, C.byref(a), _stream_ptr(stream)))
        return dst


class Group:
    """``vox_group``: all streams one GPU serves, and the attention of one decode step."""

    def __init__(self, engine: Engine, n_streams, max_len=4096, kv_type=F16, base_layers=24, res_layers=6, n_heads=16,
                 n_kv_heads=2, locdit_layers=8, locdit_seq=9, cfm_steps=10, cfm_zero_init_steps=0):
        self.engine = engine
        self.cfg = GroupConfig(n_streams, base_layers, res_layers, n_heads, n_kv_heads, 64, max_len, kv_type,
                               locdit_layers, locdit_seq, cfm_steps, cfm_zero_init_steps)
        h = C.c_void_p()
        _check(lib().vox_group_create(engine.h, C.byref(self.cfg), C.byref(h)))
        self.h = h
        engine._children.add(self)

    def close(self):
        if self.h and self.engine.h:  # a group never outlives its engine (Engine.close closes it first)
            lib().vox_group_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def cache(self, stack: int) -> KVCache:
        c = self.cfg
        layers = c.base_layers if stack == 0 else c.res_layers
        return KVCache(self.engine, layers, c.n_streams, c.n_kv_heads, c.max_len, c.kv_type,
                       handle=lib().vox_group_cache(self.h, stack))

    def set_bound(self, kv_bound: int):
        """Size every grid for lengths up to ``kv_bound`` (0: exact), so that a step can be captured and replayed."""
        _check(lib().vox_group_set_bound(self.h, int(kv_bound)))

    def advance(self, steps: int = 1):
        """Host bookkeeping after ``steps`` replays of a captured advancing step."""
        _check(lib().vox_group_advance(self.h, int(steps)))

    def set_rope(self, freq_base=10000.0, attn_factor=1.0, freq_factors=None):
        """Rotary embedding inside the step (``vox_group_set_rope``); ``freq_factors``: 32 floats on the host."""
        import numpy as np
        cfg = RopeConfig(freq_base, attn_factor, None)
        ff = None if freq_factors is None else np.ascontiguousarray(freq_factors, np.float32)
        assert ff is None or ff.shape == (32,)
        _check(lib().vox_group_set_rope(self.h, C.byref(cfg), None if ff is None else ff.ctypes.data_as(C.c_void_p)))

    def set_qkv_weights(self, w):
        """``vox_group_set_qkv_weights``: w [L, (H + 2 HK) * 64, hidden] f16 on the device (kept alive here), or None."""
        self._qkv_w = w
        if w is None:
            _check(lib().vox_group_set_qkv_weights(self.h, None, 0, 0, 0))
        else:
            _check(lib().vox_group_set_qkv_weights(self.h, w.data_ptr(), w.shape[2], w.stride(1) * 2, w.stride(0) * 2))

    def set_kv_len(self, kv_len):
        import numpy as np
        a = np.ascontiguousarray(kv_len, np.int32)
        assert a.shape == (self.cfg.n_streams,)
        _check(lib().vox_group_set_kv_len(self.h, a.ctypes.data_as(C.c_void_p)))

    def kv_len(self):
        import numpy as np
        a = np.zeros(self.cfg.n_streams, np.int32)
        _check(lib().vox_group_get_kv_len(self.h, a.ctypes.data_as(C.c_void_p)))
        return a

    def fill_synthetic(self, seed=0, stream=None):
        _check(lib().vox_group_fill_synthetic(self.h, seed, _stream_ptr(stream)))

    def step_bytes(self, which: int) -> int:
        return lib().vox_group_step_bytes(self.h, which)

    def buffer_shapes(self):
        c = self.cfg
        L, S, D = c.base_layers + c.res_layers, c.n_streams, 64
        return {
            "lm_q": (L, S, c.n_heads, D), "lm_k_new": (L, S, c.n_kv_heads, D), "lm_v_new": (L, S, c.n_kv_heads, D),
            "lm_out": (L, S, c.n_heads, D),
            "dit_q": (c.cfm_steps, S, c.locdit_layers, 2, c.n_heads, c.locdit_seq, D),
            "dit_k": (c.cfm_steps, S, c.locdit_layers, 2, c.n_kv_heads, c.locdit_seq, D),
            "dit_v": (c.cfm_steps, S, c.locdit_layers, 2, c.n_kv_heads, c.locdit_seq, D),
            "dit_out": (c.cfm_steps, S, c.locdit_layers, 2, c.locdit_seq, c.n_heads, D),
        }

    @staticmethod
    def _buffers(t: dict) -> StepBuffers:
        b = StepBuffers()
        for name, _ in StepBuffers._fields_:
            x = t.get(name)
            setattr(b, name, x.data_ptr() if x is not None and x.numel() > 0 else None)
        return b

    def step(self, tensors: dict, advance=True, stream=None):
        b = self._buffers(tensors)
        _check(lib().vox_group_step(self.h, C.byref(b), int(advance), _stream_ptr(stream)))

    def step_host(self, tensors: dict, advance=True):
        b = self._buffers(tensors)
        _check(lib().vox_group_step_host(self.h, C.byref(b), int(advance)))


def partition_streams(kv_len, n_gpus: int):
    import numpy as np
    a = np.ascontiguousarray(kv_len, np.int32)
    owner = np.zeros(len(a), np.int32)
    _check(lib().vox_partition_streams(a.ctypes.data_as(C.c_void_p), len(a), n_gpus, owner.ctypes.data_as(C.c_void_p)))
    return owner
