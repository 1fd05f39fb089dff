"""dynakv_b200 -- B200 (sm_100a) implementation of DynaKV's physical compressed-cache decode path.

The package keeps the reference's ``dynakv.kernels`` surface (``KernelPolicy``,
``compressed_decode_attention``, ``fused_attention_dispatch``, ``abx_sparse``, ``avx``,
``CustomDynamicCache``) and runs hand-written CUDA kernels through a C-ABI shared library.
There is no CPU path: calling an operator without the built library or without a CUDA device
raises.
"""
__version__ = "0.1.0"
