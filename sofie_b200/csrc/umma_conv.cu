// Tensor-core implicit-GEMM convolution (placeholder until the kernel lands): reports "shape not
// covered" so the dispatcher takes the CUDA-core direct convolution.
#include "contract.cuh"

namespace sofie {

int launch_conv2d_f32_umma(cudaStream_t, const ConvGeom &, const float *, const float *, const float *, float *)
{
   return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "no tensor-core convolution for this shape");
}
int launch_qconv2d_umma(cudaStream_t, const ConvGeom &, const uint8_t *, const int8_t *, const float *, const int32_t *,
                        int, int, uint8_t *)
{
   return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "no tensor-core convolution for this shape");
}

} // namespace sofie
