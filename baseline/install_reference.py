#!/usr/bin/env python3
"""Installs the unmodified reference (brave30/mini-inference-engine, package ``inference_engine``)
into ``baseline/_ref`` for ``bench.py --impl reference``.

    python baseline/install_reference.py /path/to/mini-inference-engine

The reference is a bare source tree (no setup.py, no pyproject.toml), which pip refuses.  So the tree
is copied to a temporary folder, a minimal ``pyproject.toml`` that names the package is put beside the
copy (no file of the reference is changed), and pip installs from there, offline and without
dependencies (torch, triton and safetensors are in the image):

    python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy>
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))

PYPROJECT = """[build-system]
requires = ["setuptools"]
build-backend = "setuptools.build_meta"

[project]
name = "inference_engine"
version = "0.0.0"

[tool.setuptools.packages.find]
include = ["inference_engine*"]
"""


def install(source: str, target: str = os.path.join(HERE, "_ref")) -> str:
    if not os.path.isdir(os.path.join(source, "inference_engine")):
        raise FileNotFoundError(f"{source!r} holds no inference_engine package")
    with tempfile.TemporaryDirectory(prefix="mie_ref_src_") as tmp:
        copy = os.path.join(tmp, "src")
        shutil.copytree(source, copy)
        with open(os.path.join(copy, "pyproject.toml"), "w") as f:
            f.write(PYPROJECT)
        if os.path.isdir(target):
            shutil.rmtree(target)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", target, copy]
        subprocess.run(cmd, check=True)
    return target


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print("installed into", install(sys.argv[1]))
