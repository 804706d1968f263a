"""Packaging for metaseq_b200.  ``pip install -e .`` builds the native libraries in-tree (``metaseq_b200/_C``)
with nvcc for sm_100a and installs the console entry points."""
from setuptools import find_packages, setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop


def _build_native():
    from metaseq_b200 import build_ext

    build_ext.build(verbose=True)


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


class Develop(develop):
    def run(self):
        _build_native()
        super().run()


setup(
    name="metaseq_b200",
    version=open("metaseq_b200/version.txt").read().strip(),
    description="OPT-style language model training and serving for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["metaseq_b200", "metaseq_b200.*"]),
    package_data={"metaseq_b200": ["_C/*.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/host/*.cpp", "version.txt"]},
    python_requires=">=3.9",
    install_requires=["torch>=2.4", "numpy", "tokenizers"],
    extras_require={"service": ["flask"], "dev": ["pytest"]},
    entry_points={
        "console_scripts": [
            "metaseq-train = metaseq_b200.cli.train:cli_main",
            "metaseq-validate = metaseq_b200.cli.validate:cli_main",
            "opt-baselines = metaseq_b200.launcher.opt_baselines:cli_main",
            "metaseq-api-local = metaseq_b200.cli.interactive_hosted:cli_main",
            "metaseq-interactive = metaseq_b200.cli.interactive_cli:cli_main",
        ],
    },
    cmdclass={"build_py": BuildPy, "develop": Develop},
)
