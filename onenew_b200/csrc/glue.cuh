// glue.cuh -- HBM-bound helper kernels around the contraction: layout transforms, operand
// packing, quantisation and the explicit im2col fallback.  All are coalesced / vectorised
// streaming kernels; none of them is on the timed path of a prepared NHWC network except the
// stem's im2col.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace one {

enum DType { DT_F32 = 0, DT_BF16 = 1, DT_S8 = 2, DT_F16 = 3 };
inline int dtype_size(int dt) { return dt == DT_F32 ? 4 : ((dt == DT_BF16 || dt == DT_F16) ? 2 : 1); }

// x[N][C][HW] f32  ->  y[N][HW][C] in `dt`.  DT_F32 with round_tf32: values rounded to tf32.
// DT_S8: quantised with x*(inv_scale), clamp, roundf (device/x86/Conv/conv.c:961-973).
cudaError_t nchw_to_nhwc(const float *x, void *y, int N, int C, int HW, int dt, int round_tf32,
                         float inv_scale, cudaStream_t s);
// x[N][HW][C] in `dt` (f32 / bf16) -> y[N][C][HW] f32.
cudaError_t nhwc_to_nchw(const void *x, float *y, int N, int C, int HW, int dt, cudaStream_t s);

// Weights OIHW -> [OC][Kp], k = (kh*KW + kw)*C + c, zero padded to Kp.  src_is_s8: the source is
// the int8 image the quantiser leaves at the start of the weight buffer
// (tools/optimize/model_quant.hpp:6-29).  Float sources are rounded to the target type.
cudaError_t pack_conv_weight(const void *w, void *out, int OC, int C, int KH, int KW, int Kp, int dt,
                             int src_is_s8, cudaStream_t s);
// rows: a[R][K] f32 -> out[R][Kp] in `dt`, zero padded.
cudaError_t pack_rows(const float *a, void *out, long long R, int K, int Kp, int dt, cudaStream_t s);
// b[batch][K][N] f32 -> out[batch][N][Kp] in `dt` (transposed, zero padded).
cudaError_t pack_transposed(const float *b, void *out, int batch, int K, int N, int Kp, int dt,
                            cudaStream_t s);
// Explicit im2col: out[M][Kp], M = N*OH*OW, k = (kh*KW + kw)*C + c; zero for padding and k >= K.
// src_nhwc = 0: source is NCHW f32; 1: source is NHWC in `src_dt`.  Output type `dt`; DT_S8 from
// an f32 source quantises with inv_scale.
cudaError_t im2col_pack(const void *x, void *out, int N, int C, int H, int W, int KH, int KW, int OH,
                        int OW, int stride_w, int stride_h, int pad_t, int pad_l, int Kp, int src_nhwc,
                        int src_dt, int dt, float inv_scale, cudaStream_t s);
// Space-to-depth of an NCHW fp32 image for stride-2 convolutions: out[n][hs][ws][(bh*BW+bw)*C + c] =
// x[n][c][2hs+bh][2(ws-OFF)+bw], bh < 2, bw < BW, OFF = BW/2 - 1 (zero outside the image and for channel
// slots >= 2*BW*C), in `dt`; Ws counts the positions of the output (image width / 2 rounded up, + OFF).  BW = 2 is the plain re-layout; BW = 4 lets every position also carry the two columns of its
// right neighbour, so that one filter position covers four taps along w (rows twice as wide, half as many
// of them: the tensor-map load rate is per row).
cudaError_t s2d_pack(const float *x, void *out, int N, int C, int H, int W, int Hs, int Ws, int Cp, int bw, int dt,
                     float inv_scale, cudaStream_t s);
// Weights for the space-to-depth rewrite: out[oc][a_h][a_w][(bh*BW+bw)*C + c] = w[oc][c][2a_h+bh-eh][BW*a_w+bw-ew],
// zero where that tap does not exist; row length KH2*KW2*Cp.
cudaError_t pack_conv_weight_s2d(const void *w, void *out, int OC, int C, int KH, int KW, int KH2, int KW2, int eh,
                                 int ew, int Cp, int bw, int dt, int src_is_s8, cudaStream_t s);
// Depthwise convolution on NCHW fp32 (group == C == OC, weight [C][1][KH][KW]), CUDA cores, HBM bound:
// one pass over x and y.  bias may be null.
cudaError_t dwconv_nchw(const float *x, const float *w, const float *bias, float *y, int N, int C, int H, int W, int OH, int OW,
                        int KH, int KW, int sx, int sy, int pt, int pl, int act, float p0, float p1, const float *lut,
                        cudaStream_t s);
// The int8 flavour: fp32 input quantised on the fly with 1 / in_scale, int8 weights, int32 bias (may be
// null), aux = weight_aux[C]; every side padded by `pad`.  Bit-exact with the reference.
cudaError_t dwconv_s8_nchw(const float *x, const int8_t *w, const int *bias, const float *aux, float *y, int N, int C, int H,
                           int W, int OH, int OW, int KH, int KW, int sx, int sy, int pad, float in_scale, int act, float p0,
                           float p1, const float *lut, cudaStream_t s);
// im2col matrix of non-overlapping patches (stride == kernel, no padding) of an NCHW fp32 image:
// out[(n, oh, ow)][(c, kh, kw)] in `dt`, row length Kp (zero beyond C*KH*KW).  KW and W multiples of 4.
cudaError_t patch_pack(const float *x, void *out, int N, int C, int H, int W, int KH, int KW, int Kp, int dt, cudaStream_t s);
// int32 -> float (exact C cast), used for the int8 path's bias.
cudaError_t cast_s32_f32(const int *x, float *y, long long n, cudaStream_t s);
// Elementwise f32 -> s8 quantisation (any layout).
cudaError_t quantize_s8(const float *x, int8_t *q, long long n, float inv_scale, cudaStream_t s);

}  // namespace one
