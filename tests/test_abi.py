"""The C-ABI library loads without a GPU, exports every symbol include/fso_b200.h declares, and refuses malformed
arguments before touching the device (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "fso_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fso_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(fso):
    from fish_scales_ops_b200 import _lib

    names = _declared()
    assert "fso_gemm_mxfp8" in names and "fso_moe_combine" in names and len(names) >= 14
    handle = ctypes.CDLL(_lib.lib_path())
    for n in names:
        assert hasattr(handle, n), n
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_plan(fso):
    from fish_scales_ops_b200 import _lib, _ops

    assert _lib.lib().fso_b200_version() == 1
    p = _ops.moe_plan(8192, 2, 8)        # Mixtral bucket: 16384 pairs -> 135 blocks -> 17408 rows
    assert (p.pairs, p.num_blocks, p.rows) == (16384, 135, 17408)
    p = _ops.moe_plan(4096, 8, 256)      # DeepSeek-V3 bucket: 510 blocks -> 65408 rows
    assert (p.num_blocks, p.rows) == (510, 65408)
    p = _ops.moe_plan(1, 2, 8)
    assert (p.num_blocks, p.rows, p.route_scratch_bytes) == (2, 384, 0)   # (2 + 127*2) // 128
    with pytest.raises(ValueError):
        _ops.moe_plan(4, 2, 2000)


def test_refusals_launch_nothing(fso):
    from fish_scales_ops_b200 import _lib

    L = _lib.lib()
    one = ctypes.c_void_p(256)   # never dereferenced: every call below is refused on its shape
    assert L.fso_quantize_1x32(one, one, one, 4, 100, 0, None) == -1
    assert "multiple of 128" in _lib.last_error()
    assert L.fso_gemm_mxfp8(one, one, one, one, one, 4, 100, 128, None, 0, None) == -1
    assert L.fso_gemm_mxfp8(ctypes.c_void_p(8), one, one, one, one, 4, 128, 128, None, 0, None) == -1
    assert "16-byte" in _lib.last_error()
    v = ctypes.c_int64(-1)
    assert L.fso_gemm_mxfp8_ws_bytes(0, 128, 128, ctypes.byref(v)) == 0 and v.value == 0
    assert L.fso_moe_combine(one, one, one, None, one, one, 4, 2, 128, None) == -1   # bias_scale without bias
    assert L.fso_requant_bs128_to_mx(one, one, one, one, 100, 128, 0, None) == -1
    # an empty problem is a successful no-op
    assert L.fso_quantize_1x32(None, None, None, 0, 128, 0, None) == 0
    assert L.fso_gemm_mxfp8(None, None, None, None, None, 0, 128, 128, None, 0, None) == 0


def test_missing_library_fails_loudly(fso, monkeypatch):
    from fish_scales_ops_b200 import _build, _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_build, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "fish_scales_ops_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.replace("no oracle", ""), os.path.join(base, f)


_NOT_PROBED = {"fso_b200_version", "fso_b200_last_error", "fso_stream_fence"}     # no arguments to refuse


def test_every_entry_point_refuses_an_all_zero_call(fso):
    """Zero sizes and NULL pointers everywhere: each entry point answers FSO_ERR_INVALID (-1) with a message of its
    own before it reaches the device (a positive code would be a CUDA error, i.e. a call that got that far)."""
    from fish_scales_ops_b200 import _lib

    L = _lib.lib()
    probed = 0
    for name, sig in sorted(_lib.SIGNATURES.items()):
        if name in _NOT_PROBED:
            continue
        args = [0 if t in (ctypes.c_int64, ctypes.c_int, ctypes.c_int32) else None for t in sig]
        assert getattr(L, name)(*args) == -1, name
        assert _lib.last_error().startswith("fso_"), (name, _lib.last_error())
        probed += 1
    assert probed >= 28


def test_null_pointers_are_refused_after_the_shape_checks(fso):
    """Well-formed sizes with NULL operands: refused by the pointer check, still before any launch."""
    from fish_scales_ops_b200 import _lib

    L = _lib.lib()
    n = None
    calls = {
        "fso_quantize_1x32": (n, n, n, 128, 128, 0, n),
        "fso_quantize_activation_1x32": (n, n, n, 128, 128, n),
        "fso_silu_mul_quantize_1x32": (n, n, n, 128, 128, n),
        "fso_requant_bs128_to_mx": (n, n, n, n, 128, 128, 0, n),
        "fso_gemm_mxfp8": (n, n, n, n, n, 128, 128, 128, n, 0, n),
        "fso_gemm_mxfp8_epilogue": (n, n, n, n, n, 128, 128, 128, n, n, 0, n, 0, n),
        "fso_gemm_mxfp8_quantized": (n, n, n, n, n, n, 128, 128, 128, n, 0, n),
        "fso_gemm_mxfp8_swiglu": (n, n, n, n, n, n, 128, 256, 128, n),
        "fso_moe_gather_quant": (n, n, 4, 2, 128, 256, n, n, n),
        "fso_moe_fc1_swiglu": (n, n, n, n, n, n, 8, 128, 128, 1, 256, n, n, n),
        "fso_moe_fc2": (n, n, n, n, n, n, 8, 128, 128, 1, 256, n, n),
        "fso_moe_combine": (n, n, n, n, n, n, 4, 2, 128, n),
    }
    for name, args in calls.items():
        assert len(args) == len(_lib.SIGNATURES[name]), name
        assert getattr(L, name)(*args) == -1, name
        assert "NULL" in _lib.last_error(), (name, _lib.last_error())


_C_CALLER = r"""
#include <stdio.h>
#include <string.h>
#include "fso_b200.h"

int main(void)
{
    fso_moe_plan plan;
    int32_t route[6];
    if (fso_b200_version() != 1) return 1;
    if (fso_moe_plan_make(8192, 2, 8, &plan) != 0 || plan.num_blocks != 135 || plan.rows != 17408) return 2;
    if (fso_gemm_mxfp8_describe(8192, 28672, 4096, 148, route) != 0) return 3;
    printf("route %d %d %d %d %d %d\n", route[0], route[1], route[2], route[3], route[4], route[5]);
    if (fso_gemm_mxfp8(0, 0, 0, 0, 0, 4, 100, 128, 0, 0, 0) != FSO_ERR_INVALID) return 4;
    if (strstr(fso_b200_last_error(), "multiples of 128") == 0) return 5;
    printf("ok\n");
    return 0;
}
"""


def test_a_c_program_links_the_library_and_calls_it(fso, tmp_path):
    """The boundary is a C ABI: a C99 translation unit that includes the header links against the library with gcc and
    calls it (host-only entry points, so this runs without a GPU)."""
    import shutil
    import subprocess

    from fish_scales_ops_b200 import _lib

    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    src = tmp_path / "caller.c"
    src.write_text(_C_CALLER)
    libdir = os.path.dirname(_lib.lib_path())
    exe = tmp_path / "caller"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-lfso_b200", f"-Wl,-rpath,{libdir}"], check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True, timeout=120).stdout.split("\n")
    assert out[0] == "route 0 256 1 32 1 3584" and out[1] == "ok"
