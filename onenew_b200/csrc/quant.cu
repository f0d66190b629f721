// quant.cu -- the statistics and the arithmetic of the reference's post-training quantiser
// (tools/optimize/model_quant.hpp), with the per-tensor passes on the device so that calibration runs on
// the activations where they are produced:
//   one_quant_abs_max        running max |x| of a device tensor            model_quant.hpp:482-507 (first pass)
//   one_quant_abs_histogram  2048-bin histogram of |x| / max                model_quant.hpp:541-570 (second pass)
//   one_quant_mse_threshold  threshold minimising the quantisation MSE      model_quant.hpp:575-610
//   one_quant_kl_threshold   threshold minimising the KL divergence          model_quant.hpp:338-430
//   one_quant_collect_abs_ge every element with |x| >= a bound (the percent method's "largest
//                            values of this image", model_quant.hpp:147-163, without sorting the tensor)
//   one_quant_weights        per-output-channel int8 weights / int32 bias   model_quant.hpp:6-29
// The two device passes are HBM-bound reads of the tensor (fp32 or bf16, any layout); the histogram
// is privatised in shared memory per block and merged with integer atomics.  The reference counts in a
// float histogram (`+= 1`), which stops growing at 2^24 per bin; the counts here are integers and are
// converted to float for the search, so the two agree while no bin exceeds 2^24.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <vector>

#include "../../include/one_glue.h"
#include "ctx.h"
#include "glue.cuh"

using namespace one;

namespace {

constexpr int BINS = 2048;

template <typename T> __device__ __forceinline__ float ldf(const T *p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float *p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p, long long i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ldf<__half>(const __half *p, long long i) { return __half2float(p[i]); }

template <typename T>
__global__ void k_abs_max(const T *__restrict__ x, long long n, float *__restrict__ out)
{
    float m = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        m = fmaxf(m, fabsf(ldf<T>(x, i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // non-negative floats order like their bit patterns
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int *>(out), __float_as_int(m));
}

template <typename T>
__global__ void k_abs_hist(const T *__restrict__ x, long long n, float max_abs, unsigned int *__restrict__ hist)
{
    __shared__ unsigned int sh[BINS];
    for (int i = threadIdx.x; i < BINS; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    // The bin index is formed in single precision, as the reference's expression is: in its C++
    // translation unit "math.h" is visible (host/ops/gelu.h:5 through ops_head.h, optimize.hpp:28), so
    // fabs(float) * int * 1.0f / float is float arithmetic.  Multiply and divide stay separate roundings.
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = ldf<T>(x, i);
        if (v == 0.0f) continue;
        int idx = (int)__fdiv_rn(__fmul_rn(__fmul_rn(fabsf(v), (float)BINS), 1.0f), max_abs);
        idx = idx > BINS - 1 ? BINS - 1 : idx;
        atomicAdd(&sh[idx], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < BINS; i += blockDim.x)
        if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

// Appends every element with |x| >= thr to `out` (order unspecified); `count` keeps counting past `cap`
// so that the caller can tell an overflow.
template <typename T>
__global__ void k_collect_abs_ge(const T *__restrict__ x, long long n, float thr, float *__restrict__ out, unsigned int cap,
                                 unsigned int *__restrict__ count)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = ldf<T>(x, i);
        if (fabsf(v) >= thr) {
            const unsigned int k = atomicAdd(count, 1u);
            if (k < cap) out[k] = v;
        }
    }
}

inline int grid_for(long long n)
{
    long long g = (n + 255) / 256;
    return (int)(g > 148 * 8 ? 148 * 8 : (g < 1 ? 1 : g));
}

}  // namespace

extern "C" int one_quant_abs_max(const void *x, int dtype, long long n, float *dev_max, void *stream)
{
    if (!x || !dev_max || n < 0) return fail(ONE_ERR_BAD_ARG, "abs_max: bad argument");
    if (n == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == DT_F32) k_abs_max<float><<<grid_for(n), 256, 0, st>>>((const float *)x, n, dev_max);
    else if (dtype == DT_BF16) k_abs_max<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16 *)x, n, dev_max);
    else if (dtype == DT_F16) k_abs_max<__half><<<grid_for(n), 256, 0, st>>>((const __half *)x, n, dev_max);
    else return fail(ONE_ERR_UNSUPPORTED, "abs_max: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "abs_max launch");
}

extern "C" int one_quant_abs_histogram(const void *x, int dtype, long long n, float max_abs, unsigned int *dev_hist, void *stream)
{
    if (!x || !dev_hist || n < 0 || !(max_abs > 0.f)) return fail(ONE_ERR_BAD_ARG, "abs_histogram: bad argument");
    if (n == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == DT_F32) k_abs_hist<float><<<grid_for(n), 256, 0, st>>>((const float *)x, n, max_abs, dev_hist);
    else if (dtype == DT_BF16) k_abs_hist<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16 *)x, n, max_abs, dev_hist);
    else if (dtype == DT_F16) k_abs_hist<__half><<<grid_for(n), 256, 0, st>>>((const __half *)x, n, max_abs, dev_hist);
    else return fail(ONE_ERR_UNSUPPORTED, "abs_histogram: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "abs_histogram launch");
}

// Host arithmetic, in the reference's float order.
extern "C" int one_quant_mse_threshold(const unsigned int *hist, long long elem_count, float max_abs, float *threshold)
{
    if (!hist || !threshold || elem_count <= 0 || elem_count > 0x7fffffffLL || !(max_abs > 0.f))
        return fail(ONE_ERR_BAD_ARG, "mse_threshold: bad argument");
    const int num_his_bins = BINS, target_bin = 128, min_num_bins = 128;
    const int elem_size = (int)elem_count;
    int best_bins = 0;
    float loss_min = 32768.0f;
    for (int bins_i = min_num_bins; bins_i < num_his_bins; bins_i++) {
        float loss = 0.0f;
        const float step = (float)bins_i / (target_bin - 1);
        for (int idx = 0; idx < num_his_bins; ++idx) {
            float idx_quanted = roundf(((float)idx + 0.5f) / step);
            idx_quanted = idx_quanted > 127.0f ? 127.0f : idx_quanted;
            idx_quanted *= step;
            const float err = (float)((float)idx + 0.5 - idx_quanted);
            loss += ((float)hist[idx] * err * err) / elem_size;
        }
        if (loss < loss_min) {
            loss_min = loss;
            best_bins = bins_i;
        }
    }
    *threshold = (best_bins + 0.5f) * max_abs / num_his_bins;
    return ONE_OK;
}

extern "C" int one_quant_collect_abs_ge(const void *x, int dtype, long long n, float thr, float *dev_out, unsigned int cap,
                                        unsigned int *dev_count, void *stream)
{
    if (!x || !dev_out || !dev_count || n < 0 || !(thr >= 0.f)) return fail(ONE_ERR_BAD_ARG, "collect_abs_ge: bad argument");
    if (n == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == DT_F32) k_collect_abs_ge<float><<<grid_for(n), 256, 0, st>>>((const float *)x, n, thr, dev_out, cap, dev_count);
    else if (dtype == DT_BF16) k_collect_abs_ge<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16 *)x, n, thr, dev_out, cap, dev_count);
    else if (dtype == DT_F16) k_collect_abs_ge<__half><<<grid_for(n), 256, 0, st>>>((const __half *)x, n, thr, dev_out, cap, dev_count);
    else return fail(ONE_ERR_UNSUPPORTED, "collect_abs_ge: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "collect_abs_ge launch");
}

// KL search (model_quant.hpp:338-430), float arithmetic in the reference's order.  For each candidate width
// `bins` in [128, 2048): P = the first `bins` bins with the tail folded into the last one, Q = the same
// bins (tail dropped) squeezed into 128 levels and spread back over `bins`, both seeded with 1e-7;
// the width with the smallest sum P * log(P / Q) wins and the threshold is the centre of its last bin.
// (Where the reference reads one element past its P vector -- the 128th level's right edge is exactly
// `bins` -- the factor multiplying that read is exactly zero; the read is skipped here.)
extern "C" int one_quant_kl_threshold(const unsigned int *hist, long long elem_count, float max_abs, float *threshold)
{
    if (!hist || !threshold || elem_count <= 0 || elem_count > 0x7fffffffLL || !(max_abs > 0.f))
        return fail(ONE_ERR_BAD_ARG, "kl_threshold: bad argument");
    const int num_his_bins = BINS, target_bin = 128, min_num_bins = 128;
    const int elem_size = (int)elem_count;
    const float kl_eps = 1e-7;
    float best_kl = 32768.6f;
    int best_bins = 0;
    std::vector<float> p, accp, q(target_bin), eq;
    for (int bins = min_num_bins; bins < num_his_bins; ++bins) {
        p.assign(bins, kl_eps);
        accp.assign(bins, kl_eps);
        for (int i = 0; i < bins; ++i) {
            accp[i] += (float)hist[i];
            p[i] += (float)hist[i];
        }
        for (int i = bins; i < num_his_bins; ++i) accp[bins - 1] += (float)hist[i];
        for (auto &v : accp) v = (float)(v / (double)elem_size);
        for (auto &v : p) v = (float)(v / (double)elem_size);
        const float ratio = (float)bins * 1.0f / target_bin;
        for (int i = 0; i < target_bin; ++i) {
            const float st = i * ratio, ed = (i + 1) * ratio;
            const float fs = floorf(st), fe = floorf(ed), cs = ceilf(st);
            float acc = 0.0f;
            if (fs == fe) acc += (ed - st) * p[(int)fs];
            else {
                acc += (cs - st) * p[(int)fs];
                for (int j = (int)cs; j < (int)fe; ++j) acc += p[j];
                if ((int)fe < bins) acc += (ed - fe) * p[(int)fe];
            }
            q[i] = acc / (ed - st);
        }
        eq.assign(bins, kl_eps);
        for (int i = 0; i < target_bin; ++i) {
            const float st = i * ratio, ed = (i + 1) * ratio;
            const float fs = floorf(st), fe = floorf(ed), cs = ceilf(st);
            if (fs == fe) eq[(int)fs] += (ed - st) * q[i];
            else {
                eq[(int)fs] += (cs - st) * q[i];
                for (int j = (int)cs; j < (int)fe; ++j) eq[j] += 1.0f * q[i];
                const int tail = (int)fe >= bins ? bins - 1 : (int)fe;
                eq[tail] += (ed - fe) / 1.0f * q[i];
            }
        }
        float kl = 0;
        for (int i = 0; i < bins; ++i) kl += accp[i] * logf(accp[i] / eq[i]);
        if (kl < best_kl) {
            best_kl = kl;
            best_bins = bins;
        }
    }
    *threshold = (best_bins + 0.5f) * max_abs / num_his_bins;
    return ONE_OK;
}

extern "C" int one_quant_weights(const float *w, const float *bias, int OC, int inner, signed char *w_s8, int *bias_s32,
                                 float *weight_aux)
{
    if (!w || !w_s8 || !weight_aux || OC <= 0 || inner <= 0) return fail(ONE_ERR_BAD_ARG, "quant_weights: bad argument");
    for (int oc = 0; oc < OC; ++oc) {
        const float *cw = w + (long long)oc * inner;
        float m = 0;
        for (int i = 0; i < inner; ++i) m = fabs(cw[i]) > m ? fabs(cw[i]) : m;
        for (int i = 0; i < inner; ++i) w_s8[(long long)oc * inner + i] = (signed char)(cw[i] * 127 / m);   // C cast: truncation
        if (bias && bias_s32) bias_s32[oc] = (int)(bias[oc] * 127 / m);
        weight_aux[oc] = m;
    }
    return ONE_OK;
}
