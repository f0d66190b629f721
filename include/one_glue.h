/*
 * one_glue.h -- C ABI of the device-side glue operators around the Conv / Gemm / MatMul path:
 * the operators that sit between the convolutions of ResNet-50 (MaxPool, Add, Relu,
 * GlobalAveragePool) and the layout / type conversions at the edges of a device-resident
 * network.  Activations are NHWC (batch, rows, columns, channels) in fp32 or bf16; `dtype` is
 * 0 = fp32, 1 = bf16.  `stream` is a cudaStream_t; every call only enqueues.  Return codes are
 * the ONE_ERR_* of one_cuda.h.
 */
#ifndef ONE_GLUE_H
#define ONE_GLUE_H

#include "one_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* MaxPool, replaces device/x86/MaxPool/maxpool.c:7-93: every side padded by `pad` (the
 * reference uses pads[0] for all sides), window maximum starting from -3276800. */
ONE_API int one_glue_maxpool_nhwc(const void *x, void *y, int dtype, int N, int H, int W, int C, int kh, int kw,
                                  int sh, int sw, int pad, void *stream);
/* y = a + b (b may be NULL: y = a), optionally followed by max(., 0).  Replaces the equal-shape
 * branch of device/x86/Add/add.c:17-86 and device/x86/Relu/relu.c.  Layout-agnostic. */
ONE_API int one_glue_add_relu(const void *a, const void *b, void *y, int dtype, long long n, int relu, void *stream);
/* GlobalAveragePool, replaces device/x86/GlobalAveragePool/global_avgpool.c:27-43:
 * x [N][HW][C] -> y [N][C], sequential sum * (1/HW). */
ONE_API int one_glue_gap_nhwc(const void *x, void *y, int dtype, int N, int HW, int C, void *stream);
/* Reference layout (NCHW fp32) -> NHWC in `dtype`, and back. */
ONE_API int one_glue_to_nhwc(const float *x_nchw, void *y, int dtype, int N, int C, int HW, void *stream);
ONE_API int one_glue_to_nchw_f32(const void *x_nhwc, float *y, int dtype, int N, int C, int HW, void *stream);
/* Elementwise fp32 <-> bf16. */
ONE_API int one_glue_cast(const void *x, void *y, int src_dtype, int dst_dtype, long long n, void *stream);


/* ---- operators between the MatMul / Gemm calls of a transformer encoder; fp32, row-major ---- */
/* LayerNormalization over the last axis, replaces device/x86/LayerNormalization/
 * layer_normalization.c:59-98: x [rows][D], w [D], b [D]. */
ONE_API int one_glue_layernorm(const float *x, const float *w, const float *b, float *y, long long rows, int D, void *stream);
/* Gelu by table, replaces device/x86/Gelu/gelu.c:22-38; `lut` is the 8192-entry device copy of the
 * table host/ops/gelu.h:80-96 builds. */
ONE_API int one_glue_gelu_lut(const float *x, const float *lut, float *y, long long n, void *stream);
/* Softmax over the last axis, replaces device/x86/Softmax/softmax.c:31-76: x [rows][D]. */
ONE_API int one_glue_softmax_rows(const float *x, float *y, long long rows, int D, void *stream);
/* Transpose of up to 6 dims, replaces device/x86/Transpose/transpose.c:27-140:
 * out.shape[i] = in_shape[perm[i]]. */
ONE_API int one_glue_transpose(const float *x, float *y, int ndim, const int *in_shape, const int *perm, void *stream);
/* y[r * y_stride + i] = x[(r % x_reps) * x_stride + i] for r < reps, i < chunk: one input of a
 * Concat (device/x86/Concat/concat.c:10-66; x_reps = 1 repeats an initialiser over the batch) or a
 * Gather with a fixed index (device/x86/Gather/gather.c:10-33). */
ONE_API int one_glue_copy_chunks(const float *x, float *y, long long reps, long long chunk, long long x_reps,
                                 long long x_stride, long long y_stride, void *stream);
/* Broadcasting y = a (op) b, op 0 add, 1 sub, 2 mul, 3 div; both shapes given with `ndim`
 * entries (pad the shorter one with leading 1s).  Replaces device/x86/Add/add.c:17-86 and its
 * Sub / Mul / Div twins. */
ONE_API int one_glue_binary(int op, const float *a, const float *b, float *y, int ndim, const int *a_shape,
                            const int *b_shape, void *stream);


/* ---- post-training quantiser (tools/optimize/model_quant.hpp), statistics taken on the device ---- */
/* *dev_max = max(*dev_max, max |x|) over a device tensor (fp32 or bf16, any layout); clear *dev_max to
 * 0 before the first tensor.  First calibration pass, model_quant.hpp:482-507. */
ONE_API int one_quant_abs_max(const void *x, int dtype, long long n, float *dev_max, void *stream);
/* dev_hist[2048] += histogram of |x| * 2048 / max_abs (zeros skipped, last bin saturating).  Second
 * calibration pass, model_quant.hpp:541-570. */
ONE_API int one_quant_abs_histogram(const void *x, int dtype, long long n, float max_abs, unsigned int *dev_hist, void *stream);
/* Host: the threshold whose 128-level quantisation has the least squared error over the histogram
 * (model_quant.hpp:575-610); input_scale = threshold / 127.  `hist` is a host copy of dev_hist. */
ONE_API int one_quant_mse_threshold(const unsigned int *hist, long long elem_count, float max_abs, float *threshold);
/* KL-divergence threshold from the same histogram (tools/optimize/model_quant.hpp:338-430): host arithmetic. */
ONE_API int one_quant_kl_threshold(const unsigned int *hist, long long elem_count, float max_abs, float *threshold);
/* Append every element with |x| >= thr to dev_out (at most cap; *dev_count keeps counting so an overflow
 * shows).  The percent method (model_quant.hpp:147-163) needs each image's largest |x| values; with thr
 * taken from the histogram this finds them without sorting the tensor. */
ONE_API int one_quant_collect_abs_ge(const void *x, int dtype, long long n, float thr, float *dev_out, unsigned int cap,
                                     unsigned int *dev_count, void *stream);
/* Host: per-output-channel weight / bias quantisation (model_quant.hpp:6-29): w [OC][inner] ->
 * int8 (truncating), bias -> int32, weight_aux[oc] = max |w[oc]|.  bias / bias_s32 may be NULL. */
ONE_API int one_quant_weights(const float *w, const float *bias, int OC, int inner, signed char *w_s8, int *bias_s32,
                              float *weight_aux);

#ifdef __cplusplus
}
#endif
#endif /* ONE_GLUE_H */
