from . import kernels
from ._build import BuildError, build_all
from .kernels import GemmOut, KernelError

__all__ = ["BuildError", "GemmOut", "KernelError", "build_all", "kernels"]
