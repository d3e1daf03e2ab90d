"""The line parser that the device kernels run (comet_b200/csrc/mtxparse.cuh) is plain C++ that also
compiles for the host: here it is built with g++ and held against strtoll / strtod on a few hundred
thousand decimal strings (benchmark-style %.17g values, short decimals, long digit strings, exponents
in and beyond the exact range, halfway cases).  Every string it accepts must give the bits strtod
gives; what it does not accept it must hand to the host, never mis-parse."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_device_line_parser_agrees_with_strtod(tmp_path):
    exe = str(tmp_path / "mtxparse_check")
    src = os.path.join(ROOT, "tests", "cpu_checks", "mtxparse_check.cpp")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-o", exe, src])
    out = subprocess.run([exe, "400000"], stdout=subprocess.PIPE, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:]
    word, accepted, to_host = out.stdout.split()
    assert word == "ok" and int(accepted) > 250000
