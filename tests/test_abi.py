"""CPU-side checks of the boundary: the C-ABI library loads, exports every symbol the
header declares, and the ops refuse to run without CUDA tensors (no CPU fallback)."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge

    ge.build()
    from flaggems_sglang_b200 import _C

    return _C.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fmoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmoe_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from flaggems_sglang_b200 import _C

    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fmoe_b200.h but not exported"
        assert n in _C.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_C.SIGNATURES) == names


def test_struct_layout_matches_header():
    import ctypes

    from flaggems_sglang_b200 import _C

    # struct_size + w_layout, 8 int32, 6 int64, 10 pointers, bias pointer + 2 floats, out_rows, split_ws + its size, scale_mode + a_scale_gather
    assert ctypes.sizeof(_C.GemmArgs) == 8 + 8 * 4 + 6 * 8 + 10 * 8 + (8 + 4 + 4) + 8 + 16 + 8
    assert _C.GemmArgs.struct_size.offset == 0 and _C.GemmArgs.numel.offset == 40 and _C.GemmArgs.a.offset == 88
    # struct_size + w_layout, 8 int32, 3 int64, 2 float, 9 pointers, 1 int64, 2 pointers + 2 floats, out_rows
    assert ctypes.sizeof(_C.FusedArgs) == 8 + 144 + (8 + 8 + 4 + 4) + 8 and _C.FusedArgs.hidden.offset == 72
    assert _C.GemmArgs().struct_size == ctypes.sizeof(_C.GemmArgs)
    assert _C.FusedArgs(T=3).struct_size == ctypes.sizeof(_C.FusedArgs)


def test_unknown_struct_size_is_refused(lib):
    """A binding compiled against another version of the header is caught before any field is trusted."""
    import ctypes

    from flaggems_sglang_b200 import _C

    g = _C.GemmArgs(dtype=_C.BF16, num_experts=4, top_k=2, block_size=16, numel=8, n=128, k=128)
    g.struct_size -= 8  # the size of a struct that ends before scale_mode / a_scale_gather (ABI version 3)
    assert lib.fmoe_gemm2(ctypes.byref(g), None) == _C.ERR_INVALID_ARG and b"struct_size" in lib.fmoe_last_error()
    assert lib.fmoe_gemm1_silu(ctypes.byref(g), None) == _C.ERR_INVALID_ARG
    f = _C.FusedArgs(dtype=_C.BF16, num_experts=4, top_k=2, T=4, H=128, I=128)
    f.struct_size = 0
    assert lib.fmoe_fused_experts_workspace_bytes(ctypes.byref(f)) < 0 and b"struct_size" in lib.fmoe_last_error()
    assert lib.fmoe_fused_experts(ctypes.byref(f), None) == _C.ERR_INVALID_ARG
    assert lib.fmoe_fused_experts_static(ctypes.byref(f), None) == _C.ERR_INVALID_ARG


def _integration_snippet():
    """The ctypes stub INTEGRATION.md shows to a maintainer of the reference, as source text."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    stub = [b for b in blocks if "class GemmArgs" in b]
    assert len(stub) == 1, "INTEGRATION.md must hold exactly one ctypes stub with a GemmArgs mirror"
    return stub[0]


def test_integration_stub_struct_matches_binding(lib):
    """The struct mirror printed in INTEGRATION.md has the layout of the real one (a stale copy there would make
    the library read past the caller's struct)."""
    import ctypes

    from flaggems_sglang_b200 import _C

    ns = {"LIBFMOE_PATH": _C.LIB_PATH}
    exec(compile(_integration_snippet(), "INTEGRATION.md", "exec"), ns)
    G = ns["GemmArgs"]
    assert ctypes.sizeof(G) == ctypes.sizeof(_C.GemmArgs)
    assert [(n, getattr(G, n).offset) for n, _ in G._fields_] == \
        [(n, getattr(_C.GemmArgs, n).offset) for n, _ in _C.GemmArgs._fields_]
    assert G(n=1).struct_size == ctypes.sizeof(_C.GemmArgs)


def test_version_and_error_buffer(lib):
    assert lib.fmoe_version() == 4
    # an invalid call reports through the status code and the message buffer, without touching a device
    rc = lib.fmoe_topk_softmax(None, 4, 0, 1, 1, None, None, None)
    assert rc == 1
    assert b"E" in lib.fmoe_last_error()
    rc = lib.fmoe_moe_align_block_size(None, 8, 4, 0, None, 0, None, 0, None, None)
    assert rc == 1 and b"block" in lib.fmoe_last_error()


def test_ops_refuse_cpu_tensors():
    import flaggems_sglang_b200 as fg

    x = torch.randn(4, 256)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.fused_topk(x, torch.randn(4, 8), 2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.moe_align_block_size(torch.zeros(4, 2, dtype=torch.int32), 16, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.fused_experts(x, torch.randn(8, 64, 256), torch.randn(8, 256, 32), torch.rand(4, 2),
                         torch.zeros(4, 2, dtype=torch.int32))


def test_namespace_mirrors_reference_exports():
    import flaggems_sglang_b200 as fg

    for name in ("triton_kernel_fused_experts", "fused_moe_flagos", "fused_moe", "fused_experts",
                 "moe_align_block_size", "topk", "grouped_topk", "fused_topk", "moe_sum"):
        assert callable(getattr(fg, name))
        assert name in fg.all_registered_ops()


def test_reference_entry_point_keeps_its_assertions():
    """Argument checks of the reference op fire before any device work (ref fused_moe.py:170-195)."""
    import flaggems_sglang_b200 as fg

    x = torch.randn(4, 128, dtype=torch.bfloat16)
    w1 = torch.randn(8, 128, 512, dtype=torch.bfloat16)
    w2 = torch.randn(8, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="use_fp8_w8a8 is not supported"):
        fg.triton_kernel_fused_experts(x, w1, w2, None, None, None, use_fp8_w8a8=True)
    with pytest.raises(AssertionError, match="Inplace is not supported"):
        fg.triton_kernel_fused_experts(x, w1, w2, None, None, None, inplace=True)
    with pytest.raises(AssertionError, match="hidden_states must be bfloat16"):
        fg.triton_kernel_fused_experts(x.float(), w1, w2, None, None, None)
    with pytest.raises(AssertionError, match="hidden size mismatch"):
        fg.triton_kernel_fused_experts(x[:, :64], w1, w2, None, None, None)
    with pytest.raises(ValueError, match="Unsupported FusedMoe activation"):
        fg.triton_kernel_fused_experts(x, w1, w2, None, None, None, activation="relu")


def test_variant_selection_is_shape_only():
    from flaggems_sglang_b200.ops.fused_moe import _pick_variant

    bf = torch.bfloat16
    assert _pick_variant(torch.float32, 32, 8, 512, 256, None) == ("simt", 16)
    assert _pick_variant(bf, 2, 8, 14336, 4096, None) == ("stream", 8)        # Mixtral T=1
    assert _pick_variant(bf, 32, 8, 14336, 4096, None)[0] == "stream"         # Mixtral T=16
    assert _pick_variant(bf, 128, 8, 14336, 4096, None)[0] == "tcgen05"       # Mixtral T=64 (HBM-bound, 128-row tiles)
    assert _pick_variant(bf, 8192, 8, 14336, 4096, None) == ("tcgen05", 128)  # Mixtral T=4096
    assert _pick_variant(bf, 65536, 128, 768, 2048, None) == ("tcgen05", 128)
    assert _pick_variant(torch.float8_e4m3fn, 512, 256, 2048, 7168, None) == ("stream", 8)   # DSV3 T=64
    assert _pick_variant(torch.float8_e4m3fn, 2048, 256, 2048, 7168, None)[0] == "tcgen05"   # DSV3 T=256
    assert _pick_variant(torch.float8_e4m3fn, 131072, 256, 2048, 7168, None) == ("tcgen05", 128)


def test_header_compiles_as_plain_c_and_cpp(tmp_path):
    """The boundary is a C ABI: the public header must be self-contained C99 (and valid C++), and a C translation unit
    that fills both argument structs must agree with the ctypes mirrors on their sizes."""
    import ctypes
    import shutil
    import subprocess

    from flaggems_sglang_b200 import _C

    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no gcc")
    header = os.path.join(ROOT, "include", "fmoe_b200.h")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", header], check=True)
    gxx = shutil.which("g++")
    if gxx:
        subprocess.run([gxx, "-std=c++11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", header], check=True)
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include "fmoe_b200.h"\nint main(void) {\n'
                   '  fmoe_gemm_args g = {0}; fmoe_fused_args f = {0};\n'
                   '  g.struct_size = (uint32_t)sizeof g; f.struct_size = (uint32_t)sizeof f;\n'
                   '  printf("%u %u %d %d\\n", g.struct_size, f.struct_size, FMOE_W_N_MAJOR, FMOE_SCALE_CHANNEL);\n'
                   '  return 0;\n}\n')
    exe = tmp_path / "sizes"
    subprocess.run([gcc, "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in out] == [ctypes.sizeof(_C.GemmArgs), ctypes.sizeof(_C.FusedArgs), _C.W_N_MAJOR, _C.SCALE_CHANNEL]
