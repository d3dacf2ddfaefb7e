"""sofie_b200: B200-native back end of SOFIE's dense-contraction inference path.

csrc/        hand-written sm_100a kernels and the C ABI (include/sofie_cuda.h)
capi, ops    ctypes binding of the C ABI, operator calls on torch CUDA tensors
runner       Python mirror of the emitted Session (plan, upload, graph, infer)
configs      the five seeded benchmark configurations
onnx_wire    protobuf-free ONNX reader / writer
"""
__all__ = ["capi", "ops", "runner", "configs", "onnx_wire"]
