"""Physical compressed-cache decode kernels (mirrors the reference's ``dynakv.kernels``)."""
from .router import KernelPolicy, compressed_decode_attention  # noqa: F401
