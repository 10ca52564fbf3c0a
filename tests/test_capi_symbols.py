"""The shared library loads without a GPU and exports exactly what include/roller_b200.h
declares; calls that need no device behave."""
import ctypes
import re
from pathlib import Path

from mlir_roller_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "roller_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return set(re.findall(r"\b(roller_b200_\w+)\s*\(", text))


def test_header_library_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 14
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(lib, name), f"{name} declared but not exported"
    assert names == set(_lib.SIGNATURES), names ^ set(_lib.SIGNATURES)


def test_every_declaration_cites_the_reference():
    text = HEADER.read_text()
    # each entry point's comment names the reference interface it replaces, or says it has none
    for m in re.finditer(r"/\*((?:(?!\*/).)*)\*/\s*(?:int|const char\*)\s+(roller_b200_\w+)\s*\(", text, flags=re.S):
        comment, name = m.group(1), m.group(2)
        assert ("src/" in comment) or ("no counterpart" in comment), name


def test_host_only_calls():
    lib = _lib.load()
    n = lib.roller_b200_kernel_count()
    assert n == 9
    kt = _lib.KTile()
    assert lib.roller_b200_kernel_desc(0, ctypes.byref(kt)) == _lib.OK
    assert lib.roller_b200_kernel_desc(n, ctypes.byref(kt)) == _lib.ERR_INVALID
    assert lib.roller_b200_kernel_desc(-1, ctypes.byref(kt)) == _lib.ERR_INVALID
    for code in range(0, -9, -1):
        assert lib.roller_b200_strerror(code)
    assert lib.roller_b200_strerror(_lib.ERR_TIMEOUT).decode().startswith("a bounded")
    # argument validation happens before any device call
    h = ctypes.c_void_p()
    assert lib.roller_b200_gemm_create(None, 1, 1, 1, 1, 1, 1, 3, 0, ctypes.byref(h)) == _lib.ERR_INVALID
    tile = _lib.kernel_tiles()[0]
    assert lib.roller_b200_gemm_create(ctypes.byref(tile), 0, 8, 8, 8, 8, 8, 3, 0, ctypes.byref(h)) == _lib.ERR_INVALID
    assert lib.roller_b200_gemm_create(ctypes.byref(tile), 8, 8, 8, 4, 8, 8, 3, 0, ctypes.byref(h)) == _lib.ERR_INVALID
    assert lib.roller_b200_gemm_create(ctypes.byref(tile), 8, 8, 8, 8, 8, 8, 2, 0, ctypes.byref(h)) == _lib.ERR_INVALID
    bad = _lib.KTile(block_m=96, block_n=96, rstep=32, cta_group=1)
    assert lib.roller_b200_gemm_create(ctypes.byref(bad), 8, 8, 8, 8, 8, 8, 3, 0, ctypes.byref(h)) == _lib.ERR_UNSUPPORTED
    assert lib.roller_b200_gemm_run(None, None, None, None, None) == _lib.ERR_INVALID
    assert lib.roller_b200_gemm_destroy(None) == _lib.OK


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    try:
        _lib.load()
    except RuntimeError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("load() must raise when the library is missing")


def test_product_does_not_import_the_oracle():
    pkg = Path(__file__).resolve().parent.parent / "mlir_roller_b200"
    for src in list(pkg.glob("*.py")) + list((pkg / "csrc").glob("*")):
        text = src.read_text()
        assert "oracle" not in text, f"{src} mentions the oracle"


C_CALLER = r"""
#include <stdio.h>
#include "roller_b200.h"
int main(void) {
  int n = roller_b200_kernel_count();
  int i;
  printf("%d\n", n);
  for (i = 0; i < n; ++i) {
    roller_ktile t;
    if (roller_b200_kernel_desc(i, &t) != ROLLER_OK) return 2;
    printf("%d %d %d %d\n", t.block_m, t.block_n, t.cta_group, t.layout);
  }
  {
    roller_plan* plan = 0;
    if (roller_b200_gemm_create(0, 1, 1, 1, 1, 1, 1, ROLLER_MODE_3XTF32, 0, &plan) != ROLLER_ERR_INVALID)
      return 3;
  }
  printf("%s\n", roller_b200_strerror(ROLLER_ERR_TIMEOUT));
  return 0;
}
"""


def test_header_is_plain_c_and_links_from_a_c_program(tmp_path):
    """The boundary is a C ABI: the header compiles as strict C99 and a C program that links
    the library enumerates the same rTiles as the Python binding."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        import pytest
        pytest.skip("no C compiler")
    src = tmp_path / "caller.c"
    src.write_text(C_CALLER)
    exe = tmp_path / "caller"
    libdir = str(_lib.LIB_PATH.parent)
    subprocess.run([gcc, "-std=c99", "-pedantic", "-Wall", "-Werror", f"-I{HEADER.parent}", str(src),
                    "-o", str(exe), f"-L{libdir}", "-lroller_b200", f"-Wl,-rpath,{libdir}"],
                   check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    tiles = _lib.kernel_tiles()
    assert int(out[0]) == len(tiles)
    for line, kt in zip(out[1:], tiles):
        assert [int(x) for x in line.split()] == [kt.block_m, kt.block_n, kt.cta_group, kt.layout]
    assert out[1 + len(tiles)].startswith("a bounded")
