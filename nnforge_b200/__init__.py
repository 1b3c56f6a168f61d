"""nnforge_b200: B200 (sm_100a) kernels for nnForge's batch-norm / activation / add / softmax /
max-subsampling layers behind a C ABI (include/nnf_b200.h).

``nnforge_b200.capi`` is the ctypes binding of that ABI. There is no CPU fallback: importing
``capi`` fails when the compiled library is missing.
"""
__all__ = ["capi"]
