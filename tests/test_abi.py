"""The C-ABI shared library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fa_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"^FA_API\s+[\w\s\*]+?\b(fa_\w+)\s*\(", text, flags=re.M)


def test_header_and_binding_agree():
    from fa_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 13
    assert sorted(names) == sorted(_lib.SYMBOLS)


def test_library_loads_and_exports_every_symbol():
    from fa_b200 import _lib

    assert os.path.exists(_lib.LIB_PATH), "build with: python flash-attention-rdna3_b200/build.py"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert _lib.load().fa_abi_version() == 3


def test_struct_sizes_match_the_header():
    """Compile a tiny C program against the header and compare sizeof with the ctypes mirrors."""
    import subprocess
    import tempfile

    from fa_b200 import _lib

    src = ('#include "fa_b200.h"\n#include <stdio.h>\nint main(void){printf("%zu %zu %zu %zu %zu\\n",'
           "sizeof(fa_attn_params),sizeof(fa_decode_params),sizeof(fa_combine_params),sizeof(fa_paged_params),"
           "sizeof(fa_tiny_params));return 0;}\n")
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "sz.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "sz")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        sizes = [int(x) for x in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    mirrors = [_lib.AttnParams, _lib.DecodeParams, _lib.CombineParams, _lib.PagedParams, _lib.TinyParams]
    assert sizes == [ctypes.sizeof(m) for m in mirrors]


def test_argument_errors_are_reported_without_a_gpu():
    from fa_b200 import _lib

    lib = _lib.load()
    p = _lib.AttnParams()
    assert lib.fa_fwd(ctypes.byref(p), None) == -1          # FA_ERR_INVALID_ARGUMENT, nothing launched
    assert b"positive" in lib.fa_last_error_string() or b"dtype" in lib.fa_last_error_string()
    assert lib.fa_fwd(None, None) == -1
    d = _lib.DecodeParams()
    assert lib.fa_decode_splitk(ctypes.byref(d), None) == -1
    t = _lib.TinyParams()
    assert lib.fa_tiny_fwd(ctypes.byref(t), None) == -1


def test_workspace_bytes_match_what_the_python_layer_allocates():
    from fa_b200 import _lib

    lib = _lib.load()
    d = _lib.DecodeParams()
    d.batch, d.heads_q, d.heads_kv, d.seqlen_q, d.seqlen_k, d.head_dim, d.num_splits = 2, 8, 2, 3, 4096, 128, 6
    assert lib.fa_workspace_bytes(_lib.FA_WS_DECODE_O_PARTIAL, ctypes.byref(d)) == 6 * 2 * 8 * 3 * 128 * 4
    assert lib.fa_workspace_bytes(_lib.FA_WS_DECODE_LSE_PARTIAL, ctypes.byref(d)) == 6 * 2 * 8 * 3 * 4
    d.num_splits = 1
    assert lib.fa_workspace_bytes(_lib.FA_WS_DECODE_O_PARTIAL, ctypes.byref(d)) == 0
    p = _lib.PagedParams()
    p.batch, p.heads_q, p.heads_kv, p.head_dim, p.num_splits = 4, 32, 8, 128, 10
    assert lib.fa_workspace_bytes(_lib.FA_WS_PAGED_O_PARTIAL, ctypes.byref(p)) == 4 * 32 * 10 * 128 * 4
    assert lib.fa_workspace_bytes(_lib.FA_WS_PAGED_LSE_PARTIAL, ctypes.byref(p)) == 4 * 32 * 10 * 4
    a = _lib.AttnParams()
    a.batch, a.heads_q, a.seqlen_q = 2, 16, 2048
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DELTA, ctypes.byref(a)) == 2 * 16 * 2048 * 4
    assert lib.fa_workspace_bytes(99, ctypes.byref(a)) == -1
    # dS scratch of the dense backward: one 32 KB tile per (batch, query head, key tile, query tile); none for packed
    # sequences or for dtypes / head dims the tensor-core backward does not take
    a.dtype, a.heads_kv, a.seqlen_k, a.head_dim = _lib.FA_F16, 4, 1000, 128
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == 2 * 16 * 16 * 8 * 32768
    # head dims above 128 up to 512 keep the P tile beside the dS tile; above 512 there is no scratch form
    for wide in (160, 512):
        a.head_dim = wide
        assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == 2 * 2 * 16 * 16 * 8 * 32768
    a.head_dim = 520
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == 0
    # forward scratch, head dims above 256 only: one P tile per tile pair and 8 bytes per row of the padded query tiles
    a.head_dim = 512
    assert lib.fa_workspace_bytes(_lib.FA_WS_FWD_P, ctypes.byref(a)) == 2 * 16 * (16 * 8 * 32768 + 16 * 128 * 8)
    a.head_dim = 256
    assert lib.fa_workspace_bytes(_lib.FA_WS_FWD_P, ctypes.byref(a)) == 0
    # fp32 inputs (head dims to 256) that opt into tensor-core products: the same plus V rounded to fp16
    a.dtype, a.head_dim = _lib.FA_F32, 128
    assert lib.fa_workspace_bytes(_lib.FA_WS_FWD_P, ctypes.byref(a)) == (2 * 16 * (16 * 8 * 32768 + 16 * 128 * 8)
                                                                          + 2 * 4 * 1000 * 128 * 2)
    a.dtype = _lib.FA_F16
    a.head_dim = 128
    a.varlen, a.total_q = 1, 4096
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == 0
    # fp32 inputs that opt into tensor-core products: the two tiles plus Q, dO and K rounded to fp16
    a.varlen, a.dtype = 0, _lib.FA_F32
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == (2 * 2 * 16 * 16 * 8 * 32768
                                                                           + 2 * 2 * 128 * (2 * 16 * 2048 + 4 * 1000))
    a.head_dim = 512
    assert lib.fa_workspace_bytes(_lib.FA_WS_BWD_DS, ctypes.byref(a)) == 0


def test_library_sources_call_no_allocator():
    """The header promises that the library allocates and frees nothing: no source file may name an allocating or
    freeing CUDA runtime call (the two fixed arrays it uses are file-scope __device__ arrays)."""
    csrc = os.path.join(ROOT, "flash-attention-rdna3_b200", "csrc")
    banned = re.compile(r"\bcuda(Malloc\w*|Free\w*|Memset\w*|HostAlloc|MallocAsync)\s*\(|\bcuMemAlloc\w*\s*\(")
    for f in sorted(os.listdir(csrc)):
        text = open(os.path.join(csrc, f)).read()
        assert not banned.search(text), f


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from fa_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "flash-attention-rdna3_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("forced-split oracle", ""), os.path.join(dirpath, f)


def test_build_entry_point_runs():
    """The repository's build entry compiles what is out of date (nothing, after a build), loads the library and checks
    its ABI version and exports against the package; it broke once on an ABI bump that only changed the header."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("graft_entry_under_test", os.path.join(ROOT, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
