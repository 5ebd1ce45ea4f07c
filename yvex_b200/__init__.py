"""yvex_b200: B200-native (sm_100a) quantized MoE execution path behind yvex's backend operator
surface. The product is the shared library yvex_b200/libyvex_b200.so (hand-written CUDA kernels +
C11 host boundary, built in-tree by `python -m yvex_b200.build`); this package is the thin Python
loader used by the tests and the benchmark. There is no CPU fallback: importing `yvex_b200.lib`
without the built library, or calling a compute entry point without a CUDA device, raises.
"""
__all__ = ["synth"]
