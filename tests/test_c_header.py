"""The generated public header of the native library: current, plain C, and matching the symbols the
library exports (the kernel-level C ABI that ``ctypes`` here and ``purego`` from Go both call)."""
import ctypes
import re
import shutil
import subprocess

import pytest

from mimir_b200 import _native
from mimir_b200._native import header


def test_header_is_current():
    assert header.OUT.read_text() == header.render(), "run: python -m mimir_b200._native.header"


def test_every_declared_function_is_exported_and_nothing_is_missing():
    lib = _native.lib()
    text = header.OUT.read_text()
    decls = [line for line in text.splitlines() if line.endswith(");") and not line.startswith(("/*", " *"))]
    names = [re.search(r"\b(mimir_[a-z0-9_]+)\(", line).group(1) for line in decls]
    assert len(names) >= 100 and len(set(names)) == len(names)
    for n in names:
        assert hasattr(lib, n), n


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_header_is_plain_c_and_links(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "mimir_b200.h"\n#include <stdio.h>\n'
                   'int main(void) { printf("%d\\n", mimir_version()); return mimir_cpu_qgemv_has_int8() < 0; }\n')
    exe = tmp_path / "t"
    from mimir_b200._native import build as nb
    libdir = str(nb.LIB.parent)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", str(header.OUT.parent), str(src), "-o", str(exe),
                    "-L", libdir, "-l:libmimir_b200.so", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    assert int(out) >= 100
