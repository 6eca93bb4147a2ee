"""CPU-only checks of the boundary: the library builds, loads, exports every symbol the public header
declares, and its host logic (status side channel, column sharding) behaves.  No kernel runs here."""
import os
import re
import subprocess

import numpy as np
import pytest

import skl_b200 as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "skl-b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"SKL_FUNC\s+[\w\s\*]+?\b(skl_\w+)\s*\(", text)))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    assert len(names) >= 45
    for must in ("skl_gemm_i8rc_i8rc_i32rc_sm100a", "skl_gemm_f8e5m2c_f8e5m2_f32_sm100a", "skl_gemm_ex_sm100a",
                 "skl_cvt_sat_bf16_f8e5m2_sm100a", "skl_pack_e32rc_e32rcprc_sm100a", "skl_unpack_e8rcprc_e8rc_sm100a",
                 "skl_transpose_e16_sm100a", "skl_b200_last_status"):
        assert must in names


def test_library_exports_every_declared_symbol(skl):
    for name in declared_symbols():
        assert hasattr(skl, name), f"{name} declared in skl-b200.h but not exported"
        assert name in S.SIGNATURES, f"{name} has no ctypes signature in skl_b200/__init__.py"


def test_header_compiles_as_c99_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "skl-b200.h"\n#include "skl-b200-compat.h"\nint main(void){return (int)SKL_B200_OK;}\n')
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", inc, "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)
    cpp = tmp_path / "t.cpp"
    cpp.write_text('#include "skl-b200.h"\nint main(){return (int)SKL_B200_OK;}\n')
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", inc, "-c", str(cpp), "-o",
                    str(tmp_path / "t2.o")], check=True)


def test_shard_columns_partitions_exactly():
    for n in (14336, 1792, 1000, 7, 0):
        for parts in (1, 2, 4, 8):
            for align in (1, 16, 256):
                covered = 0
                for idx in range(parts):
                    s, c = S.shard_columns(n, parts, idx, align)
                    assert s == covered
                    assert c == 0 or s % align == 0
                    covered += c
                assert covered == n
    assert S.shard_columns(14336, 8, 3, 256) == (3 * 1792, 1792)
    assert S.shard_columns(10, 4, 9, 1) == (0, 0)


def test_status_strings(skl):
    assert skl.skl_b200_status_string(0) == b"ok"
    assert b"unsupported" in skl.skl_b200_status_string(5)


def test_stream_and_async_setters_round_trip(skl):
    skl.skl_b200_set_stream(0x1234)
    assert skl.skl_b200_get_stream() == 0x1234
    skl.skl_b200_set_stream(None)
    assert not skl.skl_b200_get_stream()
    skl.skl_b200_set_async(1)
    skl.skl_b200_set_async(0)


def test_unsupported_pair_is_reported_without_touching_memory(skl):
    c = np.zeros(4, np.float32)
    a = np.zeros(4, np.float32)
    skl.skl_gemm_ex_sm100a(2, 2, 2, S.F32, S.ptr(a), 2, 1, S.F32, S.ptr(a), 2, 1, 1.0, None, None, 0.0, S.F32, S.ptr(c), 2, 1)
    assert skl.skl_b200_last_status() == 5
    with pytest.raises(S.SklB200Error):
        S.check()


def test_no_device_means_error_not_fallback(skl):
    """Without a usable GPU a compute call must fail loudly and leave C alone."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = np.ones((4, 4), np.int8)
    c = np.full((4, 4), 7, np.int32)
    skl.skl_gemm_i8_i8_i32_sm100a(4, 4, 4, 1, S.ptr(a), 4, S.ptr(a), 4, 0, S.ptr(c), 4)
    assert skl.skl_b200_last_status() == 2
    assert np.all(c == 7)
    with pytest.raises(S.SklB200Error):
        S.check()


def test_fused_struct_layout_matches_the_header(tmp_path):
    """The ctypes mirror of skl_b200_fused_t must have the C compiler's size and field offsets."""
    import ctypes
    import subprocess

    fields = [name for name, _ in S.Fused._fields_]
    src = tmp_path / "layout.c"
    prints = "\n".join(f'  printf("%zu\\n", offsetof(skl_b200_fused_t, {f}));' for f in fields)
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "skl-b200.h"\nint main(void) {\n'
                   '  printf("%zu\\n", sizeof(skl_b200_fused_t));\n' + prints + "\n  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert out[0] == ctypes.sizeof(S.Fused)
    assert out[1:] == [getattr(S.Fused, f).offset for f in fields]
