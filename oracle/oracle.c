/*
 * oracle.c -- plain-C restatement of the reference's Conv / Gemm / MatMul arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with; it is
 * loaded by the tests, by the smoke test and by the benchmark's CPU-baseline leg, never by the
 * product path.  Parity status: PINNED -- every function below is checked against the
 * reference's own object code (the unmodified sources compiled into oracle/_ref/ by the
 * Makefile in this directory) in tests/test_oracle_vs_reference.py, and against the golden
 * vectors in tests/golden/ that were produced by that same reference build.
 *
 * Each function cites the reference lines it follows.  Build with -ffp-contract=off: the
 * reference is compiled as -std=c11, where GCC does not fuse a*b+c, and the int8 epilogue's
 * rounding depends on that.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* activation codes: ACT_TYPE_E, common/nn_common.h:129-137 */
enum { A_NONE = 0, A_RELU = 1, A_RELU6 = 2, A_SILU = 3, A_CLIP = 4, A_HARDSILU = 5, A_LEAKY = 6 };

#define SILU_LUT_LEN 8192

/* host/ops/conv.h:178-194 -- 8192-entry table of x/(1+expf(-x)) on [-8, 8) with step 1/512. */
void oracle_silu_lut(float *lut)
{
    float single_limit = 8.0f;
    float step = 1.0 / 512;
    for (int i = 0; i < SILU_LUT_LEN; ++i) {
        float x = i * step - single_limit;
        lut[i] = x / (1 + expf(-x));
    }
}

/* device/x86/Conv/conv.c:1216-1304 (do_act).  RELU6 has no branch there: it leaves y as is. */
void oracle_act(float *y, int64_t n, int act, float clip_min, float clip_max, float leaky,
                float hs_alpha, float hs_beta, const float *lut)
{
    if (act == A_RELU) {
        for (int64_t i = 0; i < n; ++i) y[i] = (y[i] > 0.0f) ? y[i] : 0.0f;
    } else if (act == A_SILU) {
        for (int64_t i = 0; i < n; ++i) {
            float v = y[i];
            if (v < -8.0f) y[i] = 0;
            else if (v >= 8.0f) { }
            else y[i] = lut[(int)((v + 8.0f) * 512.0f)];
        }
    } else if (act == A_CLIP) {
        for (int64_t i = 0; i < n; ++i) {
            float v = (y[i] > clip_min) ? y[i] : clip_min;
            y[i] = (v < clip_max) ? v : clip_max;
        }
    } else if (act == A_LEAKY) {
        for (int64_t i = 0; i < n; ++i) y[i] = (y[i] > 0.f) ? y[i] : leaky * y[i];
    } else if (act == A_HARDSILU) {
        for (int64_t i = 0; i < n; ++i) {
            float t = hs_alpha * y[i] + hs_beta;
            t = (t > 0) ? t : 0;
            y[i] = y[i] * ((t < 1) ? t : 1);
        }
    }
}

/*
 * fp32 convolution, NCHW, group 1: what eval_mxn_img2col (conv.c:300-415) and eval_1x1j1
 * (conv.c:68-166) compute -- zero pad (conv_pad.h:61-96), K ordered c,kh,kw (im2col,
 * conv.c:168-258), C = W*col, then + bias (conv.c:404-412).  The x86 SGEMM's summation order
 * (opt_gemm.h:59-172: groups of four k) is not reproduced; float parity is by tolerance.
 * Images are independent (the reference handles one per call, host/ops/conv.h:43).
 * bias may be NULL (eval_mxn_img2col_no_bias, conv.c:417-525).
 */
void oracle_conv_f32(const float *x, const float *w, const float *bias, float *y, int N, int C,
                     int H, int W, int OC, int KH, int KW, int stride_x, int stride_y, int pt,
                     int pl, int pb, int pr)
{
    int OH = (H + pt + pb - KH) / stride_y + 1;
    int OW = (W + pl + pr - KW) / stride_x + 1;
#pragma omp parallel for collapse(2)
    for (int n = 0; n < N; ++n)
        for (int oc = 0; oc < OC; ++oc) {
            const float *xi = x + (int64_t)n * C * H * W;
            float *yo = y + ((int64_t)n * OC + oc) * OH * OW;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    float acc = 0.f;
                    for (int c = 0; c < C; ++c)
                        for (int kh = 0; kh < KH; ++kh) {
                            int ih = oh * stride_y + kh - pt;
                            if (ih < 0 || ih >= H) continue;
                            for (int kw = 0; kw < KW; ++kw) {
                                int iw = ow * stride_x + kw - pl;
                                if (iw < 0 || iw >= W) continue;
                                float p = w[(((int64_t)oc * C + c) * KH + kh) * KW + kw] *
                                          xi[((int64_t)c * H + ih) * W + iw];
                                acc = acc + p;
                            }
                        }
                    if (bias) acc += bias[oc];
                    yo[oh * OW + ow] = acc;
                }
        }
}

/* conv.c:961-973 -- x*(1/scale), clamp to [-128,127], roundf (half away from zero). */
void oracle_quantize_s8(const float *x, int8_t *q, int64_t n, float input_scale)
{
    float inv = 1.0f / input_scale;
    for (int64_t i = 0; i < n; ++i) {
        float t = x[i] * inv;
        t = (t < -128) ? -128 : (t > 127) ? 127 : t;
        q[i] = (int8_t)roundf(t);
    }
}

/*
 * int8 convolution, eval_mxn_img2col_W8A32_with_input_scale (conv.c:901-1059; the bias-less
 * twin at :1061-1214 skips the bias add).  Steps: quantise x (above); pad all four sides by
 * `pad` (the reference uses pads[0] for every side, conv.c:979-999); s8*s8 -> s32 sum
 * (:1024-1039); y = (float)acc * input_scale; y += (float)bias_s32 (:1043-1044);
 * y *= weight_aux[oc] * 1 / 127.0f (:1050-1056).  acc_out / q_out (either may be NULL) receive
 * the s32 accumulators (NCHW) and the quantised input.
 */
void oracle_conv_s8(const float *x, const int8_t *w_s8, const int32_t *bias_s32, float *y,
                    int32_t *acc_out, int8_t *q_out, int N, int C, int H, int W, int OC, int KH,
                    int KW, int stride_x, int stride_y, int pad, float input_scale,
                    const float *weight_aux)
{
    int OH = (H + 2 * pad - KH) / stride_y + 1;
    int OW = (W + 2 * pad - KW) / stride_x + 1;
    int64_t in_elems = (int64_t)N * C * H * W;
    int8_t *q = q_out ? q_out : (int8_t *)malloc(in_elems);
    oracle_quantize_s8(x, q, in_elems, input_scale);
#pragma omp parallel for collapse(2)
    for (int n = 0; n < N; ++n)
        for (int oc = 0; oc < OC; ++oc) {
            const int8_t *qi = q + (int64_t)n * C * H * W;
            int64_t obase = ((int64_t)n * OC + oc) * OH * OW;
            float dequant_coeff = weight_aux[oc] * 1 / 127.0f;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    int32_t acc = 0;
                    for (int c = 0; c < C; ++c)
                        for (int kh = 0; kh < KH; ++kh) {
                            int ih = oh * stride_y + kh - pad;
                            if (ih < 0 || ih >= H) continue;
                            for (int kw = 0; kw < KW; ++kw) {
                                int iw = ow * stride_x + kw - pad;
                                if (iw < 0 || iw >= W) continue;
                                acc += (int32_t)w_s8[(((int64_t)oc * C + c) * KH + kh) * KW + kw] *
                                       (int32_t)qi[((int64_t)c * H + ih) * W + iw];
                            }
                        }
                    if (acc_out) acc_out[obase + oh * OW + ow] = acc;
                    float v = acc * input_scale;
                    if (bias_s32) v += bias_s32[oc];
                    v = v * dequant_coeff;
                    y[obase + oh * OW + ow] = v;
                }
        }
    if (!q_out) free(q);
}

/* tools/optimize/model_quant.hpp:6-29 -- per-output-channel weight/bias quantisation; the C
 * casts truncate toward zero.  w_s8 has OC*inner entries, bias may be NULL. */
void oracle_quant_weight_bias(const float *w, const float *bias, int OC, int inner, int8_t *w_s8,
                              int32_t *bias_s32, float *weight_aux)
{
    for (int oc = 0; oc < OC; ++oc) {
        const float *cw = w + (int64_t)oc * inner;
        float m = 0;
        for (int i = 0; i < inner; ++i) m = fabs(cw[i]) > m ? fabs(cw[i]) : m;
        for (int i = 0; i < inner; ++i) w_s8[(int64_t)oc * inner + i] = (int8_t)(cw[i] * 127 / m);
        if (bias) bias_s32[oc] = (int32_t)(bias[oc] * 127 / m);
        weight_aux[oc] = m;
    }
}

/* device/x86/Gemm/gemm.c:9-79 -- Y[M,N] = A[M,K] * W[N,K]^T + bias[N], sequential-k sums. */
void oracle_gemm(const float *a, const float *w, const float *bias, float *y, int M, int N, int K)
{
#pragma omp parallel for
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float s = 0;
            for (int k = 0; k < K; ++k) s += a[(int64_t)m * K + k] * w[(int64_t)n * K + k];
            y[(int64_t)m * N + n] = s + bias[n];
        }
}

/* device/x86/MatMul/mat_mul.c:10-101 -- out[b,M,N] = A[b,M,K] * B[(b,)K,N]; B is shared by all
 * batches iff it holds exactly K*N elements (:42-46, :75-79). b_elems = element count of B. */
void oracle_matmul(const float *a, const float *b, float *y, int batch, int M, int N, int K,
                   int64_t b_elems)
{
    int shared = (b_elems == (int64_t)K * N);
#pragma omp parallel for collapse(2)
    for (int bi = 0; bi < batch; ++bi)
        for (int m = 0; m < M; ++m) {
            const float *ap = a + ((int64_t)bi * M + m) * K;
            const float *bp = shared ? b : b + (int64_t)bi * K * N;
            float *yp = y + ((int64_t)bi * M + m) * N;
            for (int n = 0; n < N; ++n) yp[n] = 0.f;
            for (int k = 0; k < K; ++k) {
                float av = ap[k];
                for (int n = 0; n < N; ++n) yp[n] = yp[n] + av * bp[(int64_t)k * N + n];
            }
        }
}

/*
 * MSE calibration of one Conv input, tools/optimize/model_quant.hpp:437-623.
 * Pass 1 (:519-533): max |x| over the calibration images.  Pass 2 (:559-575): 2048-bin histogram of
 * |x| * 2048 / max, zeros skipped, the top bin clamped.  Search (:598-616): for bins in [128, 2047],
 * step = bins / 127, loss = sum hist[i] * ((i + 0.5) - min(round((i + 0.5) / step), 127) * step)^2
 * / elem_size; threshold = (best + 0.5) * max / 2048 (:618).  input_scale = threshold / 127 (:668).
 * Parity status of THIS function: unpinned (the optimiser tool cannot be built here); it only
 * produces scales, which are inputs of the int8 parity tests, not results.
 */
float oracle_abs_max(const float *x, int64_t n, float cur)
{
    for (int64_t i = 0; i < n; ++i) cur = cur > fabsf(x[i]) ? cur : fabsf(x[i]);
    return cur;
}

void oracle_hist_accumulate(const float *x, int64_t n, float max_abs, float *hist /* 2048 */)
{
    const int num_his_bins = 2048;
    for (int64_t i = 0; i < n; ++i) {
        if (x[i] == 0.0f) continue;
        /* float arithmetic throughout: in the reference's C++ translation unit "math.h" is visible
           (host/ops/gelu.h:5 through ops_head.h, optimize.hpp:28), so fabs(float) is the float overload */
        int idx = (int)(fabsf(x[i]) * num_his_bins * 1.0f / max_abs);
        if (idx > num_his_bins - 1) idx = num_his_bins - 1;
        hist[idx] += 1;
    }
}

float oracle_mse_threshold(const float *hist /* 2048 */, int32_t elem_size, float max_abs)
{
    const int num_his_bins = 2048, target_bin = 128, min_num_bins = 128;
    int best_bins = 0;
    float loss_min = 32768.0f;
    for (int bins_i = min_num_bins; bins_i < num_his_bins; bins_i++) {
        float loss = 0.0f;
        float err;
        const float step = (float)bins_i / (target_bin - 1);
        for (int idx = 0; idx < num_his_bins; ++idx) {
            float idx_quanted = roundf(((float)idx + 0.5f) / step);
            idx_quanted = idx_quanted > 127.0f ? 127.0f : idx_quanted;
            idx_quanted *= step;
            err = (float)idx + 0.5 - idx_quanted;
            loss += (hist[idx] * err * err) / elem_size;
        }
        if (loss < loss_min) {
            loss_min = loss;
            best_bins = bins_i;
        }
    }
    return (best_bins + 0.5f) * max_abs / num_his_bins;
}

/* KL calibration threshold, tools/optimize/model_quant.hpp:338-430, in the reference's float order.
 * hist: the 2048-bin |x| histogram (float counts); elem_size: elements seen; max_abs: the histogram's
 * range.  For every width in [128, 2048): P keeps the first `bins` bins (+1e-7) with the tail added to
 * the last, both P and the tail-less copy divided by elem_size in double; Q squeezes the tail-less copy
 * into 128 levels (fractional bin overlaps weighted) and spreads it back (+1e-7); KL = sum P log(P/Q).
 * The reference reads p_histogram[bins] (one past the end) when a level's right edge equals `bins`,
 * multiplied by an exactly-zero weight; that term is left out. */
float oracle_kl_threshold(const float *hist /* 2048 */, int32_t elem_size, float max_abs)
{
    enum { NB = 2048, TB = 128 };
    float *p = (float *)malloc(sizeof(float) * NB), *ap = (float *)malloc(sizeof(float) * NB);
    float *eq = (float *)malloc(sizeof(float) * NB), q[TB];
    const float eps = 1e-7;
    float best_kl = 32768.6f;
    int best_bins = 0;
    for (int bins = TB; bins < NB; ++bins) {
        for (int i = 0; i < bins; ++i) {
            ap[i] = eps; p[i] = eps;
            ap[i] += hist[i];
            p[i] += hist[i];
        }
        for (int i = bins; i < NB; ++i) ap[bins - 1] += hist[i];
        for (int i = 0; i < bins; ++i) ap[i] = ap[i] / (double)elem_size;
        for (int i = 0; i < bins; ++i) p[i] = p[i] / (double)elem_size;
        const float ratio = (float)bins * 1.0f / TB;
        for (int i = 0; i < TB; ++i) {
            const float st = i * ratio;
            const float ed = (i + 1) * ratio;
            q[i] = 0.0f;
            if (floorf(st) == floorf(ed)) {
                q[i] += (ed - st) * p[(int)floorf(st)];
            } else {
                q[i] += (ceilf(st) - st) * p[(int)floorf(st)];
                for (int j = (int)ceilf(st); j < (int)floorf(ed); ++j) q[i] += p[j];
                if ((int)floorf(ed) < bins) q[i] += (ed - floorf(ed)) * p[(int)floorf(ed)];
            }
            q[i] /= (ed - st);
        }
        for (int i = 0; i < bins; ++i) eq[i] = eps;
        for (int i = 0; i < TB; ++i) {
            const float st = i * ratio;
            const float ed = (i + 1) * ratio;
            if (floorf(st) == floorf(ed)) {
                eq[(int)floorf(st)] += (ed - st) * q[i];
            } else {
                eq[(int)floorf(st)] += (ceilf(st) - st) * q[i];
                for (int j = (int)ceilf(st); j < (int)floorf(ed); ++j) eq[j] += 1.0f * q[i];
                int tail = (int)floorf(ed) >= bins ? bins - 1 : (int)floorf(ed);
                eq[tail] += (ed - floorf(ed)) / 1.0f * q[i];
            }
        }
        float kl = 0;
        for (int i = 0; i < bins; ++i) kl += ap[i] * logf(ap[i] / eq[i]);
        if (kl < best_kl) {
            best_kl = kl;
            best_bins = bins;
        }
    }
    free(p); free(ap); free(eq);
    return (best_bins + 0.5f) * max_abs / NB;
}

/* Depthwise fp32 convolution: eval_depthwise_conv_mxn_img2col (conv.c:527-615) and its 3x3/pad-1
 * twin (:617-755).  One input channel per output channel, taps summed kh-outer / kw-inner, then
 * + bias.  Taps that fall in the padding contribute nothing (the reference multiplies by a padded
 * zero or skips them; the sums are equal). */
void oracle_dwconv_f32(const float *x, const float *w, const float *bias, float *y, int N, int C, int H, int W, int KH,
                       int KW, int stride_x, int stride_y, int pt, int pl, int pb, int pr)
{
    int OH = (H + pt + pb - KH) / stride_y + 1;
    int OW = (W + pl + pr - KW) / stride_x + 1;
#pragma omp parallel for collapse(2)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const float *xi = x + ((int64_t)n * C + c) * H * W;
            const float *wc = w + (int64_t)c * KH * KW;
            float *yo = y + ((int64_t)n * C + c) * OH * OW;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    float psum = 0;
                    for (int kh = 0; kh < KH; ++kh) {
                        int ih = oh * stride_y + kh - pt;
                        if (ih < 0 || ih >= H) continue;
                        for (int kw = 0; kw < KW; ++kw) {
                            int iw = ow * stride_x + kw - pl;
                            if (iw < 0 || iw >= W) continue;
                            psum += wc[kh * KW + kw] * xi[(int64_t)ih * W + iw];
                        }
                    }
                    yo[oh * OW + ow] = bias ? psum + bias[c] : psum;
                }
        }
}

/* Depthwise int8 convolution, eval_depthwise_conv_mxn_img2col_W8A32 (conv.c:617-760): the input is
 * quantised like the dense int8 conv's, every side is padded by `pad` (= pads[0]), the int8 taps of
 * the one channel are summed in int32, then (float)psum * input_scale + (float)bias_s32[c]
 * (:738), then * weight_aux[c] * 1 / 127.0f (:745-751).  The reference handles one image per call;
 * the batch loop applies it image by image. */
void oracle_dwconv_s8(const float *x, const int8_t *w_s8, const int32_t *bias_s32, float *y, int N, int C, int H, int W,
                      int KH, int KW, int stride_x, int stride_y, int pad, float input_scale, const float *weight_aux)
{
    int OH = (H + 2 * pad - KH) / stride_y + 1;
    int OW = (W + 2 * pad - KW) / stride_x + 1;
    int64_t in_elems = (int64_t)N * C * H * W;
    int8_t *q = (int8_t *)malloc(in_elems);
    oracle_quantize_s8(x, q, in_elems, input_scale);
#pragma omp parallel for collapse(2)
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const int8_t *qi = q + ((int64_t)n * C + c) * H * W;
            const int8_t *wc = w_s8 + (int64_t)c * KH * KW;
            float *yo = y + ((int64_t)n * C + c) * OH * OW;
            float dequant_coeff = weight_aux[c] * 1 / 127.0f;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    int32_t psum = 0;
                    for (int kh = 0; kh < KH; ++kh) {
                        int ih = oh * stride_y + kh - pad;
                        if (ih < 0 || ih >= H) continue;
                        for (int kw = 0; kw < KW; ++kw) {
                            int iw = ow * stride_x + kw - pad;
                            if (iw < 0 || iw >= W) continue;
                            psum += (int32_t)wc[kh * KW + kw] * (int32_t)qi[(int64_t)ih * W + iw];
                        }
                    }
                    float v = (float)psum * input_scale;
                    if (bias_s32) v += (float)bias_s32[c];
                    yo[oh * OW + ow] = v * dequant_coeff;
                }
        }
    free(q);
}

/* Gelu table, host/ops/gelu.h:80-96: 8192 entries over [-8, 8) in steps of 1/512,
 * x * 0.5 * (1 + erf(x / 1.4142)) with the product formed in double and erf taken in float
 * (the C++ overload the reference's call resolves to). */
void oracle_gelu_lut(float *lut)
{
    const float single_limit = 8.0f;
    const float step = 1.0 / 512;
    const int lut_len = (int)(2.0f * single_limit / step);
    const float inv_sqrt2 = 1.0f / 1.4142f;
    for (int i = 0; i < lut_len; ++i) {
        float x = i * step - single_limit;
        /* host/ops/gelu.h:89 with "math.h" visible in C++: erf(float) is the float function and 1 + erf(...)
           a float sum; only the product with x * 0.5 is formed in double */
        const float one_plus_erf = 1 + erff(x * inv_sqrt2);
        lut[i] = (float)((double)x * 0.5 * (double)one_plus_erf);
    }
}
