"""Packaging for an in-place (editable) install: ``pip install --no-build-isolation -e .``

The CUDA/C++ extension is not a setuptools extension: it is compiled in-tree by
``budgetformer_b200.ops._ext.build()`` (nvcc, ``-gencode arch=compute_100a,code=sm_100a``) into
``budgetformer_b200/csrc/build/`` and loaded from there, so a source checkout and an editable install behave the
same.  ``BF_SKIP_KERNEL_BUILD=1`` skips the compile step (it then happens on first use)."""
import os

from setuptools import find_packages, setup
from setuptools.command.develop import develop


class DevelopWithKernels(develop):
    def run(self):
        super().run()
        if os.environ.get("BF_SKIP_KERNEL_BUILD") != "1":
            from budgetformer_b200.ops import _ext
            _ext.build()


setup(
    name="budgetformer-b200",
    version="0.1.0",
    description="Blackwell-native (sm_100a) distributed full-graph Graph-Transformer training",
    packages=find_packages(include=["budgetformer_b200", "budgetformer_b200.*"]),
    package_data={"budgetformer_b200": ["csrc/*.cu", "csrc/*.cpp", "csrc/*.h", "csrc/cpu/*.cpp"]},
    py_modules=["main_node_fullgraph_sp", "main_node_sp"],
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "scipy"],
    extras_require={"datasets": ["torch_geometric", "ogb"], "metrics": ["scikit-learn"], "test": ["pytest"]},
    cmdclass={"develop": DevelopWithKernels},
    entry_points={"console_scripts": [
        "bf-train-fullgraph=main_node_fullgraph_sp:cli",
        "bf-train-minibatch=main_node_sp:cli",
        "bf-preprocess=budgetformer_b200.utils.preprocess_data:main",
    ]},
)
