"""CUDA sources (sm_100a), their build and their Python launchers."""
from .build import KernelBuildError, build_all, load_library

__all__ = ["KernelBuildError", "build_all", "load_library"]
