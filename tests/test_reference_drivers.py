"""The reference's own drivers against this repository's C++ veneer.

Where the reference checkout is present (the build machine), every driver under its test/ directory is
compiled UNMODIFIED, from where it lies, with include paths that map the reference's header names onto
include/grape_veneer.hpp (oracle/veneer_shim/), and linked with libgrape_b200.so: the veneer offers the
whole host API those drivers use.  On a GPU the one driver that needs no model dumps (test/HyraxTest.cu:
commit, commit of an Fr tensor, open, and the verifier identities it asserts) is run as built.
"""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = Path(os.environ.get("GRAPE_REFERENCE_DIR", str(ROOT.parent / "reference")))
DRIVERS = ["HyraxTest", "matmul", "tlookupTest", "tlookupMapTest", "eleWiseMul", "combine_value", "commit", "ppgen", "llm"]


def test_every_reference_driver_compiles_and_links_against_the_veneer():
    if not (REF / "test" / "HyraxTest.cu").exists():
        pytest.skip("the reference checkout is not on this machine")
    if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
        pytest.skip("needs nvcc")
    res = subprocess.run(["make", "-C", str(ROOT / "oracle"), "-j4", "drivers", f"REF={REF}"], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    for name in DRIVERS:
        assert (ROOT / "oracle" / "_ref" / "veneer" / name).exists(), name


@pytest.mark.gpu
def test_reference_hyrax_driver_runs_unmodified(tmp_path):
    exe = ROOT / "oracle" / "_ref" / "veneer" / "HyraxTest"
    if not exe.exists():
        pytest.skip("oracle/_ref/veneer/HyraxTest was not built (no reference checkout at build time)")
    if shutil.disk_usage(tmp_path).free < 6 << 30:
        pytest.skip("needs 6 GB of scratch disk for the reference's points.bin")
    (tmp_path / "data").mkdir()
    (tmp_path / "build").mkdir()
    gen = tmp_path / "make_points"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(ROOT / "tests/cpp/make_points.cpp"),
                    "-L", str(ROOT / "grape_b200"), "-lgrape_b200", f"-Wl,-rpath,{ROOT / 'grape_b200'}", "-o", str(gen)],
                   check=True)
    # the driver reads a table of npoints * com_scale = 262 144 generators (test/HyraxTest.cu:13-29)
    res = subprocess.run([str(gen), str(16384 * 16)], cwd=tmp_path / "build", capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr
    assert (tmp_path / "data" / "points.bin").stat().st_size == 16384 * 16 * 256 * 64
    env = dict(os.environ, OMP_NUM_THREADS=str(min(os.cpu_count() or 1, 16)))
    res = subprocess.run([str(exe), "1"], cwd=tmp_path / "build", capture_output=True, text=True, timeout=1800, env=env)
    assert res.returncode == 0, (res.stdout[-1500:], res.stderr[-1500:])   # its asserts are live: a failed identity aborts
    assert "verify done" in res.stdout and "free_data done" in res.stdout
