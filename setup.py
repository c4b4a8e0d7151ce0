"""``python setup.py build_ext --inplace`` builds the sm_100a extension in-tree; ``pip install -e .`` installs the package."""
from setuptools import find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext


class build_ext(_build_ext):
    def run(self):
        import importlib.util
        import os
        spec = importlib.util.spec_from_file_location(
            "picotron_b200_build", os.path.join(os.path.dirname(os.path.abspath(__file__)), "picotron_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()


setup(name="picotron_b200", version="0.1.0", packages=find_packages(include=["picotron_b200", "picotron_b200.*"]),
      cmdclass={"build_ext": build_ext}, python_requires=">=3.10",
      install_requires=["torch>=2.6", "numpy>=1.26", "safetensors"],
      extras_require={"hf": ["datasets", "transformers", "huggingface_hub"], "tracking": ["wandb"], "slurm": ["jinja2"],
                      "test": ["pytest", "psutil"]})
