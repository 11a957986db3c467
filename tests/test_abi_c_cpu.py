"""The host library's C ABI exercised by a plain C program (gcc), with no Python, Rust or C++ in the caller: native MLP
training, a three-rank rendezvous in threads, the reference transport, the digest.  This is the stand-in for the Rust
facade's own tests, which cannot run where no Rust toolchain exists."""
import shutil
import socket
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_plain_c_program_drives_the_host_library(tmp_path):
    from incin_b200 import _build, _native
    _build.build_host()
    lib = _native.host_library_path()
    exe = tmp_path / "abi_host"
    subprocess.run(["gcc", "-O1", "-std=c11", "-Wall", "-o", str(exe), str(ROOT / "tests" / "abi_c" / "abi_host.c"),
                    "-I", str(ROOT / "csrc" / "include"), "-L", str(lib.parent), "-lincin_host", "-lpthread", "-lm",
                    f"-Wl,-rpath,{lib.parent}"], check=True, capture_output=True, text=True)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    p = subprocess.run([str(exe), f"127.0.0.1:{port}"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "ABI_OK" in p.stdout, p.stdout + p.stderr
