"""A plain C99 program written against include/eoq_b200.h the way a caller of the reference's headers is
(tests/c/abi_check.c): it must compile with gcc -std=c99, link against libeoq_b200.so and -- on a GPU -- run the
eoq_parallel_decode sequence with the reference's results and error codes."""
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from eoq_quantization_b200 import _lib as L
from oracle import oracle as O

SRC = os.path.join(ROOT, "tests", "c", "abi_check.c")


def _build(tmp_path) -> str:
    L.lib()                                              # makes sure the library exists
    exe = str(tmp_path / "abi_check")
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-O1", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L", libdir, "-leoq_b200", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return exe


def _env():
    env = dict(os.environ)
    try:                                                 # the CUDA runtime the library was linked against
        import torch
        cand = [os.path.join(os.path.dirname(torch.__file__), "lib"), "/usr/local/cuda/lib64"]
        env["LD_LIBRARY_PATH"] = os.pathsep.join(cand + [env.get("LD_LIBRARY_PATH", "")])
    except Exception:
        pass
    return env


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_caller_compiles_links_and_validates_arguments(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, env=_env())
    assert r.returncode == 0 and "ok (0 failures)" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_caller_runs_the_parallel_decode_sequence(tmp_path):
    exe = _build(tmp_path)
    rng = np.random.default_rng(42)
    blob = bytearray()
    specs = [(256, 16, 256, 5000), (256, 16, 256, 257), (15, 12, 4096, 20000), (256, 16, 256, 1), (31, 14, 256, 3333), (3, 8, 128, 900)]
    blob += struct.pack("<I", len(specs))
    for alphabet, p, block, n in specs:
        sym = np.clip(rng.normal(alphabet / 2, alphabet / 6, n), 0, alphabet - 1).astype(np.int64)
        hdr, payload = O.make_c_payload(O.encode_blocked(sym, alphabet, block, p))
        blob += struct.pack("<7I", *[int(v) for v in hdr]) + struct.pack("<I", len(payload)) + bytes(payload) + sym.astype(np.uint8).tobytes()
    path = tmp_path / "tensors.bin"
    path.write_bytes(bytes(blob))
    r = subprocess.run([exe, str(path)], capture_output=True, text=True, env=_env())
    assert r.returncode == 0 and "ok (0 failures)" in r.stdout, r.stdout + r.stderr
