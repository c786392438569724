"""The C-ABI boundary: the library loads without a GPU, exports exactly what include/splosh_cuda.h
declares, and refuses to compute where there is no sm_100 device (there is no CPU fallback)."""
import ctypes
import os
import re
import subprocess

import pytest

import splosh_b200 as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "splosh_cuda.h")).read()
    return sorted(set(re.findall(r"\b(spl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(S.library_path())
    names = declared()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), name


def test_every_exported_entry_point_is_declared():
    out = subprocess.run(["nm", "-D", "--defined-only", S.library_path()], capture_output=True, text=True, check=True).stdout
    exported = sorted(line.split()[-1] for line in out.splitlines() if " T spl_" in line)
    assert exported == declared()


def test_header_cites_the_reference_interface_it_replaces():
    text = open(os.path.join(ROOT, "include", "splosh_cuda.h")).read()
    assert len(re.findall(r"Engine\.swift:\d+", text)) >= 20


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "splosh_cuda.h"\nint main(void) { spl_row r; r.slot = 0; return (int)sizeof(spl_tables) * 0 + r.slot; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_no_gpu_means_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(S.EngineError) as caught:
        S.Engine(S.tiny_geometry())
    assert caught.value.case == "unsupportedDevice"
    import numpy as np
    with pytest.raises(S.EngineError):
        S.gemm_q4(np.zeros((16, 32), np.uint32), np.zeros((16, 4), np.uint16), np.zeros((16, 4), np.uint16), np.zeros((1, 256), np.float32))


def test_product_sources_never_reach_for_the_oracle():
    """Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may touch oracle/."""
    for folder, _, files in os.walk(os.path.join(ROOT, "splosh_b200")):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(folder, name)).read()
                for needle in ("import oracle", "from oracle", "liboracle", "oracle/", "orc_"):
                    assert needle not in text, (os.path.join(folder, name), needle)
