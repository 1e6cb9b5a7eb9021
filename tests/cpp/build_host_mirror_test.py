"""Builds the C++ test programs under tests/cpp against the in-tree library and the C oracle."""
from __future__ import annotations

import pathlib
import shutil
import subprocess

ROOT = pathlib.Path(__file__).resolve().parents[2]
OUT = ROOT / "tests" / "cpp" / "_build" / "host_mirror_test"


def build(name: str = "host_mirror_test") -> pathlib.Path:
    import sys

    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    import oracle
    from augur_v100_b200 import abi

    library = pathlib.Path(abi.library_path())
    oracle_library = pathlib.Path(oracle.build())
    cuda = pathlib.Path(shutil.which("nvcc")).resolve().parents[1] if shutil.which("nvcc") else pathlib.Path("/usr/local/cuda")
    OUT.parent.mkdir(parents=True, exist_ok=True)
    out = OUT.parent / name
    compiler = "/usr/bin/g++" if pathlib.Path("/usr/bin/g++").exists() else "g++"
    command = [compiler, "-std=c++17", "-O1", "-Wall", "-Wextra", "-o", str(out), str(ROOT / "tests" / "cpp" / f"{name}.cpp"),
               f"-I{ROOT / 'include'}", f"-I{ROOT / 'oracle'}", f"-I{cuda / 'include'}",
               str(library), str(oracle_library), f"-L{cuda / 'lib64'}", "-lcudart", "-lpthread", "-lm",
               f"-Wl,-rpath,{library.parent}", f"-Wl,-rpath,{oracle_library.parent}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"{name} does not compile:\n" + done.stderr)
    return out


if __name__ == "__main__":
    print(build())
