"""sofie_b200: B200-native back end of SOFIE's dense-contraction inference path.

csrc/        hand-written sm_100a kernels and the C ABI (include/sofie_cuda.h)
capi, ops    ctypes binding of the C ABI, operator calls on torch CUDA tensors
generated    emits, compiles and loads the C++ Session the generator writes for a model
host/        the C++ generator (RModelParser_ONNX, RModel, ROperator_*): the planner of this package
configs      the five seeded benchmark configurations
onnx_wire    protobuf-free ONNX reader / writer
"""
__all__ = ["capi", "ops", "generated", "configs", "onnx_wire"]
