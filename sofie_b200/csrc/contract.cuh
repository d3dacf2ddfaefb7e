// Internal launcher interface between api.cu (validation, dispatch) and the kernel files.
#pragma once
#include "common.cuh"

namespace sofie {

struct ConvGeom {
   int N, C, H, W, Cout, kH, kW, pad_h, pad_w, sh, sw, dh, dw, group;
   int oH, oW;    // convolution output extent
   int pH, pW;    // stored output extent (halved when pool == 2)
   int x_nhwc, y_nhwc, w_packed, relu, pool;
};

int launch_gemm_f32_simt(cudaStream_t, const sofie_gemm_f32_desc &, const float *, const float *, const float *, float *);
int launch_gemm_f32_umma(cudaStream_t, const sofie_gemm_f32_desc &, const float *, const float *, const float *, float *);
int launch_qgemm_simt(cudaStream_t, const sofie_qgemm_desc &, const uint8_t *, const int8_t *, const float *,
                      const int32_t *, uint8_t *, float *Yf32, float dq_scale);
int launch_qgemm_umma(cudaStream_t, const sofie_qgemm_desc &, const uint8_t *, const int8_t *, const float *,
                      const int32_t *, uint8_t *, float *Yf32, float dq_scale);
int launch_gemm_e4m3_simt(cudaStream_t, const sofie_fp8_gemm_desc &, const uint8_t *, const uint8_t *, const float *,
                          uint16_t *, uint8_t *, float *Yf32, const float *a_scale_dev = nullptr);
int launch_gemm_e4m3_umma(cudaStream_t, const sofie_fp8_gemm_desc &, const uint8_t *, const uint8_t *, const float *,
                          uint16_t *, uint8_t *, float *Yf32, const float *a_scale_dev = nullptr);
int launch_conv2d_f32_simt(cudaStream_t, const ConvGeom &, const float *, const float *, const float *, float *);
int launch_conv2d_f32_umma(cudaStream_t, const ConvGeom &, const float *, const float *, const float *, float *);
int launch_qconv2d_simt(cudaStream_t, const ConvGeom &, const uint8_t *, const int8_t *, const float *, const int32_t *,
                        int x_zp, int y_zp, uint8_t *);
int launch_qconv2d_umma(cudaStream_t, const ConvGeom &, const uint8_t *, const int8_t *, const float *, const int32_t *,
                        int x_zp, int y_zp, uint8_t *);
// pooled-window kernel (umma_conv_pool.cu): -1 when the shape is not its own
int launch_qconv2d_umma_pooled(cudaStream_t, const ConvGeom &, const uint8_t *, const int8_t *, const float *, const int32_t *,
                               int x_zp, int y_zp, uint8_t *);
// fused chain of small Gemm layers on the tensor cores (umma_mlp.cu): -1 when the widths are not its own
int launch_mlp_f32_umma(cudaStream_t, const sofie_mlp_desc *, const float *, const float *const *, const float *const *, float *);
// first-layer kernels (conv_first.cu): -1 when the shape is not theirs
int launch_conv2d_f32_first(cudaStream_t, const ConvGeom &, const float *, const float *, const float *, float *);
int launch_qconv2d_first(cudaStream_t, const ConvGeom &, const uint8_t *, const int8_t *, const float *, const int32_t *,
                         int x_zp, int y_zp, uint8_t *);
// split-K skinny GEMM (splitk_gemm.cu)
bool splitk_shape_ok(const sofie_gemm_f32_desc &);
bool rowblock_shape_ok(const sofie_gemm_f32_desc &, const float *A, const float *B);
int launch_gemm_f32_rowblock(cudaStream_t, const sofie_gemm_f32_desc &, const float *, const float *, const float *, float *);
int launch_gemm_f32_splitk(cudaStream_t, const sofie_gemm_f32_desc &, const float *, const float *, const float *, float *,
                           float *scratch, size_t scratch_floats);
int launch_gemm_f32_splitk_auto(cudaStream_t, const sofie_gemm_f32_desc &, const float *, const float *, const float *,
                                float *);
// gives the split-K scratch buffer of a stream back to the per-device pool (context teardown)
void splitk_scratch_release(int device, cudaStream_t stream);
template <typename T>
int launch_pack_ohwi(cudaStream_t, const T *, T *, int Cout, int C, int kH, int kW);

} // namespace sofie
