from setuptools import find_packages, setup

setup(
    name="lite_lang_b200",
    version="0.1.0",
    description="A small, whole single-GPU inference engine for B200 (sm_100a)",
    packages=find_packages(include=["lite_lang_b200", "lite_lang_b200.*"]),
    package_data={"lite_lang_b200.csrc": ["*.cu", "*.cuh", "*.h"]},
    install_requires=["torch", "safetensors", "numpy", "click"],
    entry_points={"console_scripts": ["litelang = lite_lang_b200.cli:main"]},
    scripts=["bin/trace_run"],
)
