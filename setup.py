"""Packaging of the Python side and the native libraries.

``python -m pip install --no-build-isolation --no-index .`` builds ``libhcomm.so`` and the PyTorch extension in the
tree (``hcomm_b200/build.py``: nvcc for sm_100a, g++ for the host runtime) and installs the packages ``hcomm_b200`` and
``hccl`` with the libraries and the public headers as package data.  (The reference ships its Python package the same
way, python/setup.py in its tree, next to the installer its build.sh produces.)
"""
import os
import sys
from pathlib import Path

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


class BuildNative(build_py):
    """Builds the shared objects before the Python files are collected, and carries the headers along."""

    def run(self):
        sys.path.insert(0, str(ROOT))
        from hcomm_b200 import build as native
        if os.environ.get("HCOMM_SKIP_NATIVE_BUILD") != "1":
            native.build_all()
        super().run()
        dst = Path(self.build_lib) / "hcomm_b200" / "include"
        for header in sorted((ROOT / "include").rglob("*")):
            if header.is_file():
                out = dst / header.relative_to(ROOT / "include")
                out.parent.mkdir(parents=True, exist_ok=True)
                self.copy_file(str(header), str(out))


setup(
    name="hcomm-b200",
    version="0.2.0",
    description="Collective communication library for NVIDIA B200 (sm_100a) with the API of HCCL / HCOMM",
    packages=find_packages(include=["hcomm_b200", "hcomm_b200.*", "hccl", "hccl.*"]),
    package_data={"hcomm_b200": ["lib/libhcomm.so", "lib/_hcomm_torch.so", "utils/tune_tables/*.json"]},
    python_requires=">=3.10",
    install_requires=["numpy"],
    extras_require={"torch": ["torch"]},
    cmdclass={"build_py": BuildNative},
    zip_safe=False,
)
