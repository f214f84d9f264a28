"""B200-native build of KuTACC's gated-attention path.

``kutacc_b200.api``       ctypes binding of libkutacc.so (the reference's operator interface)
``kutacc_b200.build``     nvcc build of the library (sm_100a only)
``kutacc_b200.workloads`` seeded synthetic inputs of the benchmark shapes
``kutacc_b200.runner``    glue that runs a workload through the library on device or host buffers
"""
__all__ = ["api", "build", "workloads", "runner"]
