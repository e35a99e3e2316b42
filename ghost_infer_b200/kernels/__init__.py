from .library import KernelError
