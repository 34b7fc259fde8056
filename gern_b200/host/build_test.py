"""Compiles tests/cpp/test_host.cpp against the host headers and libgern_b200.so.
Used by the pytest wrappers; prints the path of the executable."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def build() -> str:
    out_dir = os.path.join(ROOT, "build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "test_host")
    src = os.path.join(ROOT, "tests", "cpp", "test_host.cpp")
    lib_dir = os.path.join(ROOT, "gern_b200")
    deps = [src] + [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".hpp")]
    deps.append(os.path.join(lib_dir, "libgern_b200.so"))
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-I", HERE, "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(cuda, "include"), src, "-o", exe,
           "-L", lib_dir, "-lgern_b200", f"-Wl,-rpath,{lib_dir}",
           "-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + " ".join(cmd) + "\n" + res.stderr)
    return exe


if __name__ == "__main__":
    print(build())
