from .build import BuildError, build_all, ensure_built
from .ops import KernelError, KernelOps, get_ops

__all__ = ["BuildError", "build_all", "ensure_built", "KernelError", "KernelOps", "get_ops"]
