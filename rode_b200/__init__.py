"""rode_b200: the RoDe hot path (row-decomposition preprocessing, SpMM, SDDMM) for B200.

``rode_b200.capi``        ctypes binding of the C ABI (``include/rode_b200.h``)
``rode_b200.rode_sddmm``  drop-in for the reference's Python wrapper (needs the torch binding)
``rode_b200.workloads``   seeded synthetic matrices and the nnz-balanced row partition
``rode_b200.build``       in-tree build of ``librode_b200.so`` and the torch binding
"""
__version__ = "0.1.0"
