"""CPU: the C++ shim with the reference's operator signatures (include/basalt_shim.hpp) compiles against the C ABI and
keeps the reference's error behaviour."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_shim_compiles_and_runs(lib, tmp_path):
    exe = tmp_path / "shim_smoke"
    libdir = ROOT / "basalt_b200" / "lib"
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(ROOT / "tests" / "cpp" / "shim_smoke.cpp"),
                           "-L", str(libdir), "-lbasalt_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "shim ok" in out.stdout
