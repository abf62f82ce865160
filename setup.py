"""Packaging of fairscale_b200.  The CUDA library is built in-tree by ``python -m fairscale_b200._native`` (nvcc, sm_100a);
``pip install -e .`` only registers the Python package and the ``wgit`` console script."""
import re

from setuptools import find_packages, setup


def _version() -> str:
    src = open("fairscale_b200/version.py").read()
    return ".".join(re.search(r"\((\d+), (\d+), (\d+)\)", src).groups())


setup(
    name="fairscale_b200",
    version=_version(),
    description="Blackwell-native sharded / pipelined / expert / tensor-parallel training library with the fairscale API",
    packages=find_packages(include=["fairscale_b200", "fairscale_b200.*"]),
    package_data={"fairscale_b200": ["csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "lib/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy"],
    entry_points={"console_scripts": ["wgit = fairscale_b200.experimental.wgit.cli:main"]},
)
