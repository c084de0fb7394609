"""Runs the Triton-backend cases in a process of their own.

The interpreter oracle of the other tests needs TRITON_INTERPRET=1 from before Triton is imported (it turns
every @triton.jit function, Triton's own library included, into an interpreted one); the backend needs the
compiler front end of those same functions. One process cannot hold both, so the cases live in
triton_backend_cases.py / triton_backend_gpu_cases.py and run here through a fresh interpreter.
"""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(case_file: str, *extra: str) -> None:
    env = {k: v for k, v in os.environ.items() if k != "TRITON_INTERPRET"}
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider",
                           os.path.join(HERE, case_file), *extra],
                          env=env, cwd=os.path.dirname(HERE), capture_output=True, text=True, timeout=1500)
    tail = "\n".join((proc.stdout + proc.stderr).splitlines()[-60:])
    assert proc.returncode == 0, f"{case_file} failed:\n{tail}"
    assert " passed" in proc.stdout, tail  # cases that need the reference checkout skip themselves where it is absent


def test_triton_backend_cases_cpu(built_libs):
    _run("triton_backend_cases.py")


@pytest.mark.gpu
def test_triton_backend_cases_gpu(built_libs, cuda_device):
    _run("triton_backend_gpu_cases.py", "-m", "gpu")
