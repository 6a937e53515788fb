"""The C ABI: the built library loads, exports every function include/leat_sampler.h declares, and
the ctypes mirror of leat_sample_args has the layout a C compiler gives the header's struct.  No
compute is called here (no GPU needed)."""

import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "leat_sampler.h"


def declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(leat_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_function():
    from leat_b200 import _lib

    names = declared()
    assert "leat_sample" in names and "leat_verify_draft" in names and len(names) >= 13
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_struct_layout_matches_the_header(tmp_path):
    from leat_b200 import _lib

    fields = [name for name, _ in _lib.SampleArgs._fields_]
    source = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {",
             '  printf("%zu\\n", sizeof(leat_sample_args));']
    lines += [f'  printf("%zu\\n", offsetof(leat_sample_args, {f}));' for f in fields]
    lines += ["  return 0;", "}"]
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-o", str(binary), str(source)], check=True)
    out = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.SampleArgs)
    for name, offset in zip(fields, out[1:]):
        assert int(offset) == getattr(_lib.SampleArgs, name).offset, name


def test_host_side_argument_errors_need_no_gpu():
    from leat_b200 import _lib

    assert _lib.lib.leat_sampler_workspace_bytes(0, 1000, 64) == 0
    assert _lib.lib.leat_sampler_workspace_bytes(8, 1000, 4096) == 0  # k_max beyond 1024
    assert _lib.lib.leat_sampler_workspace_bytes(8, 262144, 256) > 0
    handle = C.c_void_p()
    assert _lib.lib.leat_sampler_create(None, 0, 0, 8, 1000, 64, C.byref(handle)) == _lib.E_ARGUMENT
    assert _lib.lib.leat_sample(None, None, None) == _lib.E_ARGUMENT
    assert _lib.lib.leat_verify_draft(None, None, None, 1, 1, None, None, None) == _lib.E_ARGUMENT
    assert _lib.lib.leat_sampler_tune(None, 0, 0) == _lib.E_ARGUMENT


def test_package_fails_loudly_without_the_library(tmp_path):
    code = ("import os, sys; os.environ['LEAT_SAMPLER_LIBRARY'] = r'%s'; sys.path.insert(0, r'%s')\n"
            "try:\n    import leat_b200; leat_b200.sample\nexcept ImportError as e:\n    print('ImportError', e)\n"
            % (tmp_path / "missing.so", ROOT))  # fmt: skip
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True).stdout
    assert out.startswith("ImportError") and "no CPU or eager fallback" in out
