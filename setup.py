"""Build and install: compiles the C++ host runtime and every sm_100a CUDA kernel in-tree, then packages them.

    python setup.py build_ext --inplace     # or: python -m xllm_wxh_b200.build_ext
    pip install -e . --no-build-isolation
"""
from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py


class BuildNative(Command):
    description = "compile the host runtime (_core) and the CUDA kernel library (libxllm_kernels.so) in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        from xllm_wxh_b200 import build_ext
        build_ext.build_all()


class BuildPy(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


setup(
    name="xllm_wxh_b200",
    version="0.1.0",
    description="B200-native LLM serving framework",
    packages=find_packages(include=["xllm_wxh_b200*", "xllm*"]),
    package_data={"xllm_wxh_b200": ["*.so", "csrc/**/*"]},
    python_requires=">=3.10",
    cmdclass={"build_ext": BuildNative, "build_py": BuildPy},
    entry_points={"console_scripts": ["xllm=xllm_wxh_b200.cli:main", "xllm-service=xllm_wxh_b200.service.router:main",
            "xllm-kv-store=xllm_wxh_b200.service.kv_store:main"]},
)
