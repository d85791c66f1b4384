"""The shared library loads and exports every symbol the public header declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from glq_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "glq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glqb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/glq_b200.h but not exported"


def test_binding_lists_every_declared_symbol():
    from glq_b200 import _lib
    assert sorted(_lib.EXPORTS) == _declared()


def test_struct_layout_matches_header(tmp_path):
    from glq_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "glq_b200.h"\nint main(){printf("%zu %zu %zu %zu\\n",'
                   'sizeof(GlqbLinearDesc), __builtin_offsetof(GlqbLinearDesc, su),'
                   '__builtin_offsetof(GlqbLinearDesc, batch), __builtin_offsetof(GlqbLinearDesc, x_is_rotated));}')
    exe = tmp_path / "sz"
    import subprocess
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    D = _lib.LinearDesc
    assert [int(v) for v in out] == [ctypes.sizeof(D), D.su.offset, D.batch.offset, D.x_is_rotated.offset]


def test_moe_struct_layout_matches_header(tmp_path):
    from glq_b200 import _lib
    src = tmp_path / "szm.c"
    src.write_text('#include <stdio.h>\n#include "glq_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu\\n",'
                   'sizeof(GlqbMoeDesc), __builtin_offsetof(GlqbMoeDesc, w2_packed),'
                   '__builtin_offsetof(GlqbMoeDesc, ids_are_int64), __builtin_offsetof(GlqbMoeDesc, format),'
                   '__builtin_offsetof(GlqbMoeDesc, w2_inv_rs));}')
    exe = tmp_path / "szm"
    import subprocess
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    D = _lib.MoeDesc
    assert [int(v) for v in out] == [ctypes.sizeof(D), D.w2_packed.offset, D.ids_are_int64.offset, D.format.offset,
                                     D.w2_inv_rs.offset]


def test_host_side_calls_without_gpu(lib):
    assert lib.glqb_trellis_kernel_supported(64, 64) == 1
    assert lib.glqb_trellis_kernel_supported(48, 64) == 0
    assert b"sm_100a" in lib.glqb_version()
    # argument validation happens before any CUDA call
    rc = lib.glqb_decompress_trellis_3inst(None, 4, None, 0, 0.0, 32, 32, None, 0, None)
    assert rc == -1 and b"decompress" in lib.glqb_last_error()
