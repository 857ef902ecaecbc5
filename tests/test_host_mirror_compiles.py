"""The public header is valid C, and the C++ host mirror compiles and links against the library."""
import shutil
import subprocess
from pathlib import Path

import pytest

from gptoss_b200 import capi

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_header_is_plain_c(tmp_path):
    src = tmp_path / "h.c"
    src.write_text('#include "gptoss_b200.h"\nint main(void) { gptoss_moe_dims d; d.hidden = 0; return d.hidden + (int)sizeof(gptoss_ctx *) * 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-c", str(src), "-I", str(ROOT / "include"),
                    "-o", str(tmp_path / "h.o")], check=True)


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_cpp_host_mirror_links_and_rejects_bad_dims(tmp_path):
    if capi.needs_build():
        if shutil.which("nvcc") is None:
            pytest.skip("library not built and nvcc absent")
        capi.build()
    src = tmp_path / "m.cpp"
    src.write_text('''
#include <cstdio>
#include "moe_ops.hpp"
int main() {
  gptoss_moe_dims bad{30, 64, 32, 4, 1, 7.0f};  // hidden not a multiple of 8
  try { gptoss::MoeLayerOps ops(bad, 0, 0, 1, 16); } catch (const gptoss::Error &e) {
    std::printf("rejected %d\\n", e.code); return e.code == GPTOSS_ERR_BAD_ARG ? 0 : 2; }
  return 1;
}
''')
    exe = tmp_path / "m"
    subprocess.run(["g++", "-std=c++17", str(src), "-I", str(ROOT / "include"),
                    "-I", str(capi.PKG_DIR / "host"), "-L", str(capi.CSRC), "-lgptoss_b200",
                    f"-Wl,-rpath,{capi.CSRC}", "-o", str(exe)], check=True)
    r = subprocess.run([str(exe)], stdout=subprocess.PIPE, text=True)
    assert r.returncode == 0 and "rejected 1" in r.stdout
