// net_ops.cu -- device versions of the glue operators that sit between the convolutions of
// ResNet-50 so a network stays resident on the GPU: MaxPool, Add, Relu, GlobalAveragePool and
// layout / type conversion.  All are HBM-bound streaming kernels on NHWC activations with
// 16-byte vector accesses along the channel axis.  Public view: include/one_glue.h.
//
// Reference arithmetic followed:
//   MaxPool  device/x86/MaxPool/maxpool.c:40-93   window max starting from -3276800, every side
//                                                 padded by pads[0] (pad cells never win);
//   Add      device/x86/Add/add.c:17-86           equal-shape elementwise sum;
//   Relu     device/x86/Relu/relu.c               max(x, 0);
//   GlobalAveragePool device/x86/GlobalAveragePool/global_avgpool.c:27-43   sequential sum over
//                                                 H*W, then * (1.0f / (H*W)).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/one_glue.h"
#include "ctx.h"
#include "glue.cuh"

using namespace one;

namespace {

template <typename T> struct Vec;   // 16-byte vector of T
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float *p, float (&v)[4])
    {
        const float4 t = *reinterpret_cast<const float4 *>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4])
    {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ float ld1(const float *p) { return *p; }
    static __device__ __forceinline__ void st1(float *p, float v) { *p = v; }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8])
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162 *>(&w[i]);
            v[2 * i] = __low2float(h);
            v[2 * i + 1] = __high2float(h);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float ld1(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Vec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half *p, float (&v)[8])
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            v[2 * i] = __low2float(h);
            v[2 * i + 1] = __high2float(h);
        }
    }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float ld1(const __half *p) { return __half2float(*p); }
    static __device__ __forceinline__ void st1(__half *p, float v) { *p = __float2half_rn(v); }
};

// ------------------------------------------------------------------ MaxPool (NHWC)
template <typename T, bool VEC>
__global__ void k_maxpool_nhwc(const T *__restrict__ x, T *__restrict__ y, int N, int H, int W, int C, int OH, int OW,
                               int kh, int kw, int sh, int sw, int pad)
{
    constexpr int V = VEC ? Vec<T>::N : 1;
    const int cv = C / V;
    const long long total = (long long)N * OH * OW * cv;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cv) * V;
        long long t = i / cv;
        const int ow = (int)(t % OW); t /= OW;
        const int oh = (int)(t % OH);
        const int n = (int)(t / OH);
        float m[V];
#pragma unroll
        for (int j = 0; j < V; ++j) m[j] = -3276800.f;
        for (int a = 0; a < kh; ++a) {
            const int ih = oh * sh + a - pad;
            if (ih < 0 || ih >= H) continue;
            for (int b = 0; b < kw; ++b) {
                const int iw = ow * sw + b - pad;
                if (iw < 0 || iw >= W) continue;
                const T *p = x + (((size_t)n * H + ih) * W + iw) * C + c;
                if constexpr (VEC) {
                    float v[V];
                    Vec<T>::load(p, v);
#pragma unroll
                    for (int j = 0; j < V; ++j) m[j] = v[j] > m[j] ? v[j] : m[j];
                } else {
                    const float v = Vec<T>::ld1(p);
                    m[0] = v > m[0] ? v : m[0];
                }
            }
        }
        T *q = y + (((size_t)n * OH + oh) * OW + ow) * C + c;
        if constexpr (VEC) Vec<T>::store(q, m);
        else Vec<T>::st1(q, m[0]);
    }
}

// 3x3 window, stride 2 (the ResNet / YOLO stem pool), 16-byte vectors: one thread produces two outputs that
// are neighbours along w from one 3 x 5 patch (15 loads instead of 18), all loads issued before the first
// comparison so that their latencies overlap.
template <typename T>
__global__ void k_maxpool3x3s2_nhwc(const T *__restrict__ x, T *__restrict__ y, int N, int H, int W, int C, int OH, int OW, int pad)
{
    constexpr int V = Vec<T>::N;
    const int cv = C / V;
    const int owp = (OW + 1) / 2;
    const long long total = (long long)N * OH * owp * cv;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cv) * V;
        long long t = i / cv;
        const int ow0 = (int)(t % owp) * 2; t /= owp;
        const int oh = (int)(t % OH);
        const int n = (int)(t / OH);
        float v[3][5][V];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int ih = oh * 2 + a - pad;
#pragma unroll
            for (int b = 0; b < 5; ++b) {
                const int iw = ow0 * 2 + b - pad;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) Vec<T>::load(x + (((size_t)n * H + ih) * W + iw) * C + c, v[a][b]);
                else {
#pragma unroll
                    for (int j = 0; j < V; ++j) v[a][b][j] = -3276800.f;
                }
            }
        }
        float m0[V], m1[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            m0[j] = -3276800.f;
            m1[j] = -3276800.f;
        }
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int b = 0; b < 3; ++b)
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    m0[j] = v[a][b][j] > m0[j] ? v[a][b][j] : m0[j];
                    m1[j] = v[a][b + 2][j] > m1[j] ? v[a][b + 2][j] : m1[j];
                }
        T *q = y + (((size_t)n * OH + oh) * OW + ow0) * C + c;
        Vec<T>::store(q, m0);
        if (ow0 + 1 < OW) Vec<T>::store(q + C, m1);
    }
}

// The same for 16-bit activations (T2 = __half2 or __nv_bfloat162), 8 channels per thread: the maxima are taken
// on the packed pairs as they lie in memory, without a conversion per element (the generic kernel spends its
// time converting 15 x 8 values to float and back).  Padding is minus infinity; every window holds a real pixel.
template <typename T2>
__device__ __forceinline__ uint4 max_pairs(uint4 a, uint4 b)
{
    uint4 r;
    T2 t;
    t = __hmax2(*reinterpret_cast<const T2 *>(&a.x), *reinterpret_cast<const T2 *>(&b.x)); r.x = *reinterpret_cast<const uint32_t *>(&t);
    t = __hmax2(*reinterpret_cast<const T2 *>(&a.y), *reinterpret_cast<const T2 *>(&b.y)); r.y = *reinterpret_cast<const uint32_t *>(&t);
    t = __hmax2(*reinterpret_cast<const T2 *>(&a.z), *reinterpret_cast<const T2 *>(&b.z)); r.z = *reinterpret_cast<const uint32_t *>(&t);
    t = __hmax2(*reinterpret_cast<const T2 *>(&a.w), *reinterpret_cast<const T2 *>(&b.w)); r.w = *reinterpret_cast<const uint32_t *>(&t);
    return r;
}
template <typename T2>
__global__ void k_maxpool3x3s2_nhwc_p16(const uint4 *__restrict__ x, uint4 *__restrict__ y, int N, int H, int W, int C, int OH, int OW, int pad,
                                        uint32_t minus_inf2)
{
    const int cv = C / 8;
    const int owp = (OW + 1) / 2;
    const long long total = (long long)N * OH * owp * cv;
    const uint4 ninf = make_uint4(minus_inf2, minus_inf2, minus_inf2, minus_inf2);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cv);
        long long t = i / cv;
        const int ow0 = (int)(t % owp) * 2; t /= owp;
        const int oh = (int)(t % OH);
        const int n = (int)(t / OH);
        uint4 v[3][5];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int ih = oh * 2 + a - pad;
#pragma unroll
            for (int b = 0; b < 5; ++b) {
                const int iw = ow0 * 2 + b - pad;
                v[a][b] = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? __ldg(x + (((size_t)n * H + ih) * W + iw) * cv + c) : ninf;
            }
        }
        uint4 col[5];   // maxima down the three rows, then across three columns for each of the two outputs
#pragma unroll
        for (int b = 0; b < 5; ++b) col[b] = max_pairs<T2>(max_pairs<T2>(v[0][b], v[1][b]), v[2][b]);
        const uint4 m0 = max_pairs<T2>(max_pairs<T2>(col[0], col[1]), col[2]);
        const uint4 m1 = max_pairs<T2>(max_pairs<T2>(col[2], col[3]), col[4]);
        uint4 *q = y + (((size_t)n * OH + oh) * OW + ow0) * cv + c;
        q[0] = m0;
        if (ow0 + 1 < OW) q[cv] = m1;
    }
}

// ------------------------------------------------------------------ Add / Relu (any layout)
template <typename T, bool VEC>
__global__ void k_add_relu(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y, long long n, int has_b,
                           int relu)
{
    constexpr int V = VEC ? Vec<T>::N : 1;
    const long long nv = n / V;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        float va[V], vb[V];
        if constexpr (VEC) {
            Vec<T>::load(a + i * V, va);
            if (has_b) Vec<T>::load(b + i * V, vb);
        } else {
            va[0] = Vec<T>::ld1(a + i);
            if (has_b) vb[0] = Vec<T>::ld1(b + i);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            float v = has_b ? __fadd_rn(va[j], vb[j]) : va[j];
            va[j] = relu ? (v > 0.f ? v : 0.f) : v;
        }
        if constexpr (VEC) Vec<T>::store(y + i * V, va);
        else Vec<T>::st1(y + i, va[0]);
    }
}

// ------------------------------------------------------------------ GlobalAveragePool (NHWC)
// One thread per (image, channel); consecutive threads read consecutive channels of a pixel.
template <typename T>
__global__ void k_gap_nhwc(const T *__restrict__ x, T *__restrict__ y, int N, int HW, int C)
{
    const long long total = (long long)N * C;
    const float coeff = 1.0f / (float)HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const long long n = i / C;
        const T *p = x + (size_t)n * HW * C + c;
        float s = 0.f;
        for (int k = 0; k < HW; ++k) s = __fadd_rn(s, Vec<T>::ld1(p + (size_t)k * C));
        Vec<T>::st1(y + i, __fmul_rn(s, coeff));
    }
}

// 16-byte vectors: one thread per (image, group of channels); the pixel sum keeps the reference's order
// (global_avgpool.c:27-43), the loads of several pixels are issued together.
template <typename T>
__global__ void k_gap_nhwc_vec(const T *__restrict__ x, T *__restrict__ y, int N, int HW, int C)
{
    constexpr int V = Vec<T>::N;
    const int cv = C / V;
    const long long total = (long long)N * cv;
    const float coeff = 1.0f / (float)HW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % cv) * V;
        const long long n = i / cv;
        const T *p = x + (size_t)n * HW * C + c;
        float s[V];
#pragma unroll
        for (int j = 0; j < V; ++j) s[j] = 0.f;
        int k = 0;
        for (; k + 7 <= HW; k += 7) {
            float v[7][V];
#pragma unroll
            for (int u = 0; u < 7; ++u) Vec<T>::load(p + (size_t)(k + u) * C, v[u]);
#pragma unroll
            for (int u = 0; u < 7; ++u)
#pragma unroll
                for (int j = 0; j < V; ++j) s[j] = __fadd_rn(s[j], v[u][j]);
        }
        for (; k < HW; ++k) {
            float v[V];
            Vec<T>::load(p + (size_t)k * C, v);
#pragma unroll
            for (int j = 0; j < V; ++j) s[j] = __fadd_rn(s[j], v[j]);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) s[j] = __fmul_rn(s[j], coeff);
        Vec<T>::store(y + (size_t)n * C + c, s);
    }
}

template <typename TI, typename TO>
__global__ void k_cast(const TI *__restrict__ x, TO *__restrict__ y, long long n)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        Vec<TO>::st1(y + i, Vec<TI>::ld1(x + i));
}

inline int grid_for(long long work, int block)
{
    long long g = (work + block - 1) / block;
    const long long cap = 148LL * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int one_glue_maxpool_nhwc(const void *x, void *y, int dtype, int N, int H, int W, int C, int kh, int kw,
                                     int sh, int sw, int pad, void *stream)
{
    if (!x || !y) return fail(ONE_ERR_BAD_ARG, "MaxPool: null tensor");
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || pad < 0)
        return fail(ONE_ERR_BAD_SHAPE, "MaxPool: bad shape");
    const int OH = (H + 2 * pad - kh) / sh + 1, OW = (W + 2 * pad - kw) / sw + 1;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 256;
    if (dtype == DT_F32) {
        const bool vec = (C % 4 == 0) && aligned16(x) && aligned16(y);
        const long long work = (long long)N * OH * OW * (vec ? C / 4 : C);
        if (vec && kh == 3 && kw == 3 && sh == 2 && sw == 2)
            k_maxpool3x3s2_nhwc<float><<<grid_for((long long)N * OH * ((OW + 1) / 2) * (C / 4), block), block, 0, st>>>((const float *)x, (float *)y, N, H, W, C, OH, OW, pad);
        else if (vec) k_maxpool_nhwc<float, true><<<grid_for(work, block), block, 0, st>>>((const float *)x, (float *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
        else k_maxpool_nhwc<float, false><<<grid_for(work, block), block, 0, st>>>((const float *)x, (float *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
    } else if (dtype == DT_BF16) {
        const bool vec = (C % 8 == 0) && aligned16(x) && aligned16(y);
        const long long work = (long long)N * OH * OW * (vec ? C / 8 : C);
        if (vec && kh == 3 && kw == 3 && sh == 2 && sw == 2)
            k_maxpool3x3s2_nhwc_p16<__nv_bfloat162><<<grid_for((long long)N * OH * ((OW + 1) / 2) * (C / 8), block), block, 0, st>>>((const uint4 *)x, (uint4 *)y, N, H, W, C, OH, OW, pad, 0xFF80FF80u);
        else if (vec) k_maxpool_nhwc<__nv_bfloat16, true><<<grid_for(work, block), block, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
        else k_maxpool_nhwc<__nv_bfloat16, false><<<grid_for(work, block), block, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
    } else if (dtype == DT_F16) {
        const bool vec = (C % 8 == 0) && aligned16(x) && aligned16(y);
        const long long work = (long long)N * OH * OW * (vec ? C / 8 : C);
        if (vec && kh == 3 && kw == 3 && sh == 2 && sw == 2)
            k_maxpool3x3s2_nhwc_p16<__half2><<<grid_for((long long)N * OH * ((OW + 1) / 2) * (C / 8), block), block, 0, st>>>((const uint4 *)x, (uint4 *)y, N, H, W, C, OH, OW, pad, 0xFC00FC00u);
        else if (vec) k_maxpool_nhwc<__half, true><<<grid_for(work, block), block, 0, st>>>((const __half *)x, (__half *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
        else k_maxpool_nhwc<__half, false><<<grid_for(work, block), block, 0, st>>>((const __half *)x, (__half *)y, N, H, W, C, OH, OW, kh, kw, sh, sw, pad);
    } else return fail(ONE_ERR_UNSUPPORTED, "MaxPool: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "maxpool launch");
}

extern "C" int one_glue_add_relu(const void *a, const void *b, void *y, int dtype, long long n, int relu, void *stream)
{
    if (!a || !y) return fail(ONE_ERR_BAD_ARG, "Add/Relu: null tensor");
    if (n <= 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 256;
    const int has_b = b != nullptr;
    if (dtype == DT_F32) {
        const bool vec = (n % 4 == 0) && aligned16(a) && aligned16(y) && (!b || aligned16(b));
        if (vec) k_add_relu<float, true><<<grid_for(n / 4, block), block, 0, st>>>((const float *)a, (const float *)b, (float *)y, n, has_b, relu);
        else k_add_relu<float, false><<<grid_for(n, block), block, 0, st>>>((const float *)a, (const float *)b, (float *)y, n, has_b, relu);
    } else if (dtype == DT_BF16) {
        const bool vec = (n % 8 == 0) && aligned16(a) && aligned16(y) && (!b || aligned16(b));
        if (vec) k_add_relu<__nv_bfloat16, true><<<grid_for(n / 8, block), block, 0, st>>>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)y, n, has_b, relu);
        else k_add_relu<__nv_bfloat16, false><<<grid_for(n, block), block, 0, st>>>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)y, n, has_b, relu);
    } else if (dtype == DT_F16) {
        const bool vec = (n % 8 == 0) && aligned16(a) && aligned16(y) && (!b || aligned16(b));
        if (vec) k_add_relu<__half, true><<<grid_for(n / 8, block), block, 0, st>>>((const __half *)a, (const __half *)b, (__half *)y, n, has_b, relu);
        else k_add_relu<__half, false><<<grid_for(n, block), block, 0, st>>>((const __half *)a, (const __half *)b, (__half *)y, n, has_b, relu);
    } else return fail(ONE_ERR_UNSUPPORTED, "Add/Relu: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "add/relu launch");
}

extern "C" int one_glue_gap_nhwc(const void *x, void *y, int dtype, int N, int HW, int C, void *stream)
{
    if (!x || !y) return fail(ONE_ERR_BAD_ARG, "GlobalAveragePool: null tensor");
    if (N <= 0 || HW <= 0 || C <= 0) return fail(ONE_ERR_BAD_SHAPE, "GlobalAveragePool: bad shape");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 128;
    const long long work = (long long)N * C;
    if (dtype == DT_F32 && C % 4 == 0 && aligned16(x) && aligned16(y))
        k_gap_nhwc_vec<float><<<grid_for(work / 4, block), block, 0, st>>>((const float *)x, (float *)y, N, HW, C);
    else if (dtype == DT_BF16 && C % 8 == 0 && aligned16(x) && aligned16(y))
        k_gap_nhwc_vec<__nv_bfloat16><<<grid_for(work / 8, block), block, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, N, HW, C);
    else if (dtype == DT_F16 && C % 8 == 0 && aligned16(x) && aligned16(y))
        k_gap_nhwc_vec<__half><<<grid_for(work / 8, block), block, 0, st>>>((const __half *)x, (__half *)y, N, HW, C);
    else if (dtype == DT_F32) k_gap_nhwc<float><<<grid_for(work, block), block, 0, st>>>((const float *)x, (float *)y, N, HW, C);
    else if (dtype == DT_BF16) k_gap_nhwc<__nv_bfloat16><<<grid_for(work, block), block, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, N, HW, C);
    else if (dtype == DT_F16) k_gap_nhwc<__half><<<grid_for(work, block), block, 0, st>>>((const __half *)x, (__half *)y, N, HW, C);
    else return fail(ONE_ERR_UNSUPPORTED, "GlobalAveragePool: dtype %d", dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "gap launch");
}

extern "C" int one_glue_to_nhwc(const float *x_nchw, void *y, int dtype, int N, int C, int HW, void *stream)
{
    if (!x_nchw || !y) return fail(ONE_ERR_BAD_ARG, "to_nhwc: null tensor");
    cudaError_t e = nchw_to_nhwc(x_nchw, y, N, C, HW, dtype, dtype == DT_F32, 1.f, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "to_nhwc launch");
}

extern "C" int one_glue_to_nchw_f32(const void *x_nhwc, float *y, int dtype, int N, int C, int HW, void *stream)
{
    if (!x_nhwc || !y) return fail(ONE_ERR_BAD_ARG, "to_nchw: null tensor");
    cudaError_t e = nhwc_to_nchw(x_nhwc, y, N, C, HW, dtype, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "to_nchw launch");
}

extern "C" int one_glue_cast(const void *x, void *y, int src_dtype, int dst_dtype, long long n, void *stream)
{
    if (!x || !y) return fail(ONE_ERR_BAD_ARG, "cast: null tensor");
    if (n <= 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 256;
    if (src_dtype == DT_F32 && dst_dtype == DT_BF16) k_cast<float, __nv_bfloat16><<<grid_for(n, block), block, 0, st>>>((const float *)x, (__nv_bfloat16 *)y, n);
    else if (src_dtype == DT_F32 && dst_dtype == DT_F16) k_cast<float, __half><<<grid_for(n, block), block, 0, st>>>((const float *)x, (__half *)y, n);
    else if (src_dtype == DT_BF16 && dst_dtype == DT_F32) k_cast<__nv_bfloat16, float><<<grid_for(n, block), block, 0, st>>>((const __nv_bfloat16 *)x, (float *)y, n);
    else if (src_dtype == DT_F16 && dst_dtype == DT_F32) k_cast<__half, float><<<grid_for(n, block), block, 0, st>>>((const __half *)x, (float *)y, n);
    else return fail(ONE_ERR_UNSUPPORTED, "cast %d -> %d", src_dtype, dst_dtype);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "cast launch");
}
