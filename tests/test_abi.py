"""CPU tests of the C-ABI library: it loads, exports what the header declares, and its pure
host functions (capability query, workspace sizing, stream partition) behave.  No GPU needed."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def L(pkg):
    return pkg.lib()


def test_library_exports_every_declared_symbol(pkg, L):
    names = pkg.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, f"declared in include/vox_attn.h but not exported: {missing}"


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    from voxcpm_cpp_b200 import binding
    monkeypatch.setattr(binding, "_LIB", None)
    monkeypatch.setattr(binding, "library_path", lambda: str(tmp_path / "libvoxattn.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        binding.lib()


def test_status_strings(L):
    assert L.vox_attn_status_string(0) == b"ok"
    assert L.vox_attn_status_string(5) == b"device-side wait timed out"
    assert L.vox_attn_status_string(99) == b"unknown status"


def _args(pkg, n_q=1, n_kv=256, H=16, HK=2, B=1, kv_type=1, D=64):
    T = pkg.Tensor
    rb = {0: 4 * D, 1: 2 * D, 8: 34 * (D // 32)}[kv_type]
    a = pkg.AttnArgs()
    a.q = T.make(0, [D, n_q, H, B], [4, 4 * D, 4 * D * n_q, 4 * D * n_q * H], None)
    a.k = T.make(kv_type, [D, n_kv, HK, B], [{0: 4, 1: 2, 8: 34}[kv_type], rb, rb * n_kv, rb * n_kv * HK], None)
    a.v = T.make(kv_type, [D, n_kv, HK, B], [{0: 4, 1: 2, 8: 34}[kv_type], rb, rb * n_kv, rb * n_kv * HK], None)
    a.mask = T.none()
    a.dst = T.make(0, [D, H, n_q, B], [4, 4 * D, 4 * D * H, 4 * D * H * n_q], None)
    a.scale = 0.125
    return a


def test_supported_is_a_pure_host_query(pkg, L):
    for kv_type in (0, 1, 8):
        assert L.vox_attn_supported(C.byref(_args(pkg, kv_type=kv_type))) == 1
    assert L.vox_attn_supported(C.byref(_args(pkg, n_q=512, n_kv=512, B=8))) == 1
    assert L.vox_attn_supported(C.byref(_args(pkg, n_q=18, n_kv=18, kv_type=0))) == 1
    assert L.vox_attn_supported(None) == 0


@pytest.mark.parametrize("mutate, fragment", [
    (lambda a: setattr(a, "max_bias", 1.0), b"max_bias"),
    (lambda a: setattr(a, "logit_softcap", 30.0), b"max_bias"),
    (lambda a: setattr(a, "has_sinks", 1), b"sinks"),
    (lambda a: a.q.ne.__setitem__(2, 15), b"not a multiple"),
    (lambda a: a.q.ne.__setitem__(0, 128), b"head_dim"),
    (lambda a: setattr(a.k, "type", 2), b"K/V type"),
    (lambda a: a.k.nb.__setitem__(1, 64), b"smaller than a row"),
    (lambda a: a.v.ne.__setitem__(1, 255), b"rows"),
    (lambda a: a.dst.ne.__setitem__(1, 8), b"dst"),
])
def test_unsupported_operands_are_refused_with_a_reason(pkg, L, mutate, fragment):
    a = _args(pkg)
    mutate(a)
    assert L.vox_attn_supported(C.byref(a)) == 0
    assert fragment in L.vox_attn_last_error_string()


def test_mask_must_be_contiguous_f16_and_broadcastable(pkg, L):
    a = _args(pkg, n_q=4, n_kv=32)
    a.mask = pkg.Tensor.make(1, [32, 4, 1, 1], [2, 64, 256, 256], 0x1000)
    assert L.vox_attn_supported(C.byref(a)) == 1
    a.mask.ne[2] = 3  # 16 heads do not divide over 3 mask planes (ggml.c:5300)
    a.mask.nb[3] = 256 * 3
    assert L.vox_attn_supported(C.byref(a)) == 0
    a = _args(pkg, n_q=4, n_kv=32)
    a.mask = pkg.Tensor.make(1, [32, 4, 1, 1], [2, 128, 512, 512], 0x1000)  # padded rows: not contiguous
    assert L.vox_attn_supported(C.byref(a)) == 0
    a.mask = pkg.Tensor.make(0, [32, 4, 1, 1], [4, 128, 512, 512], 0x1000)  # f32 mask
    assert L.vox_attn_supported(C.byref(a)) == 0


def test_workspace_sizing(pkg, L):
    # two partial slots (8 heads x 66 floats each) per CTA of the launch: one CTA for a short cache ...
    slot = 8 * 66 * 4
    assert L.vox_attn_decode_workspace_bytes(1, 16, 2, 64) == 2 * slot
    # ... a run of at least 4 tiles per CTA while the launch is small (2 pairs x 16 tiles) ...
    assert L.vox_attn_decode_workspace_bytes(1, 16, 2, 1024) == 2 * 8 * slot
    # ... and never more than one wave of CTAs (4 per SM on 148 SMs), whatever the streams and their lengths
    big = L.vox_attn_decode_workspace_bytes(32, 16, 2, 8192)
    assert big == 2 * 4 * 148 * slot
    assert L.vox_attn_decode_workspace_bytes(4096, 16, 2, 65536) == big
    assert L.vox_attn_workspace_bytes(C.byref(_args(pkg, n_kv=8192, B=32))) == big
    assert L.vox_attn_workspace_bytes(C.byref(_args(pkg, n_q=9, n_kv=9, kv_type=0))) == 0
    for bad in [(0, 16, 2, 64), (-1, 16, 2, 64), (1, 0, 2, 64), (1, 16, 0, 64), (1, 15, 2, 64)]:
        assert L.vox_attn_decode_workspace_bytes(*bad) == 0


def test_entry_points_reject_null_without_a_gpu(L):
    assert L.vox_engine_create(0, None) == 1
    assert L.vox_attn_forward(None, None, None, 0, None) == 1
    assert L.vox_attn_decode(None, None, None, 0, None) == 1
    assert L.vox_attn_decode_static(None, None, None) == 1
    assert L.vox_attn_locdit_step(None, None, None) == 1
    assert L.vox_kv_create(None, None, None) == 1
    assert L.vox_group_create(None, None, None) == 1
    assert L.vox_engine_sync_status(None, None) == 1
    assert L.vox_engine_launch_count(None) == 0


def test_partition_streams_balances_kv_bytes(pkg):
    rng = np.random.default_rng(12345)
    lens = rng.integers(128, 4097, 256).astype(np.int32)
    for n in (1, 2, 4, 8):
        owner = pkg.partition_streams(lens, n)
        assert owner.min() >= 0 and owner.max() < n
        loads = np.array([lens[owner == g].sum() for g in range(n)], np.float64)
        counts = np.array([(owner == g).sum() for g in range(n)])
        assert loads.sum() == lens.sum() and counts.sum() == 256
        assert loads.max() / loads.mean() < 1.01          # byte load within 1 % of even
        assert counts.max() - counts.min() <= 256 // n // 4
    assert list(pkg.partition_streams(np.array([], np.int32), 4)) == []


def test_header_is_plain_c_and_links_against_the_library(pkg, tmp_path):
    """The boundary is a C ABI: the header must compile as C (no C++ in it) and a C program that names every
    declared entry point must link against the shared library (what a cgo / FFI binding of the reference's host
    language would do).  The program only calls host-side queries: no GPU is needed."""
    import os
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    names = pkg.declared_symbols()
    src = tmp_path / "abi.c"
    src.write_text(
        '#include "vox_attn.h"\n#include <stdio.h>\n'
        "typedef void (*entry_point)(void);\n"
        "static const entry_point table[] = {" + ", ".join(f"(entry_point) {n}" for n in names) + "};\n"
        "int main(void) {\n"
        "    vox_attn_args a = {0};\n"
        "    int32_t len[4] = {4000, 100, 2000, 2100}, owner[4];\n"
        "    if (vox_attn_supported(&a)) return 1;                       /* zero shapes are refused */\n"
        "    if (vox_partition_streams(len, 4, 2, owner) != VOX_ATTN_OK) return 2;\n"
        "    if (owner[0] == owner[2] && owner[0] == owner[3]) return 3;  /* the long stream does not share with both */\n"
        "    if (vox_attn_decode_workspace_bytes(256, 16, 2, 4096) == 0) return 4;\n"
        '    printf("%d symbols, status 0 = %s\\n", (int) (sizeof(table) / sizeof(table[0])), vox_attn_status_string(0));\n'
        "    return 0;\n}\n")
    exe = tmp_path / "abi"
    lib_dir = os.path.dirname(pkg.library_path())
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(root, "include"), str(src), "-o", str(exe),
                    "-L", lib_dir, "-l:libvoxattn.so", f"-Wl,-rpath,{lib_dir}"], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    assert out.startswith(f"{len(names)} symbols")
