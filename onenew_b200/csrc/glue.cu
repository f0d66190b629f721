// glue.cu -- see glue.cuh.  Replaces, on the device, the reference's data-movement helpers:
// do_pad_conv* (device/x86/Conv/conv_pad.h:1-96: padding is folded into the TMA zero fill or
// the im2col predicate here), im2col / im2col_s8 (device/x86/Conv/conv.c:168-298) for the
// shapes the tensor-map path cannot address, and the two scalar quantisation passes of the
// int8 path (conv.c:961-973).
#include "glue.cuh"
#include "ctx.h"
#include "act.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace one {

__device__ __forceinline__ float tf32_rna(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}
__device__ __forceinline__ int8_t q8(float v, float inv_scale)
{
    float t = __fmul_rn(v, inv_scale);
    t = (t < -128.f) ? -128.f : (t > 127.f) ? 127.f : t;
    return (int8_t)(int)roundf(t);
}

template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float from(float v, int round_tf32, float) { return round_tf32 ? tf32_rna(v) : v; }
    static __device__ __forceinline__ float to(float v) { return v; }
    static __device__ __forceinline__ float zero() { return 0.f; }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ __nv_bfloat16 from(float v, int, float) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 zero() { return __float2bfloat16_rn(0.f); }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ __half from(float v, int, float) { return __float2half_rn(v); }
    static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half zero() { return __float2half_rn(0.f); }
};
template <> struct Cvt<int8_t> {
    static __device__ __forceinline__ int8_t from(float v, int, float inv) { return q8(v, inv); }
    static __device__ __forceinline__ float to(int8_t v) { return (float)v; }
    static __device__ __forceinline__ int8_t zero() { return 0; }
};

// ------------------------------------------------------------------ NCHW <-> NHWC
// Per image a [C][HW] -> [HW][C] transpose through a padded 32x32 shared tile; both the read
// (along HW) and the write (along C) are coalesced.
template <typename T>
__global__ void k_nchw_to_nhwc(const float *__restrict__ x, T *__restrict__ y, int C, int HW, int round_tf32,
                               float inv_scale)
{
    __shared__ float tile[32][33];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
    const float *xi = x + (size_t)n * C * HW;
    T *yo = y + (size_t)n * C * HW;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, p = p0 + threadIdx.x;
        if (c < C && p < HW) tile[i][threadIdx.x] = xi[(size_t)c * HW + p];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int p = p0 + i, c = c0 + threadIdx.x;
        if (c < C && p < HW) yo[(size_t)p * C + c] = Cvt<T>::from(tile[threadIdx.x][i], round_tf32, inv_scale);
    }
}

template <typename T>
__global__ void k_nhwc_to_nchw(const T *__restrict__ x, float *__restrict__ y, int C, int HW)
{
    __shared__ float tile[32][33];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
    const T *xi = x + (size_t)n * C * HW;
    float *yo = y + (size_t)n * C * HW;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int p = p0 + i, c = c0 + threadIdx.x;
        if (c < C && p < HW) tile[i][threadIdx.x] = Cvt<T>::to(xi[(size_t)p * C + c]);
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, p = p0 + threadIdx.x;
        if (c < C && p < HW) yo[(size_t)c * HW + p] = tile[threadIdx.x][i];
    }
}

cudaError_t nchw_to_nhwc(const float *x, void *y, int N, int C, int HW, int dt, int round_tf32, float inv_scale,
                         cudaStream_t s)
{
    if (N <= 0 || C <= 0 || HW <= 0) return cudaSuccess;
    dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
    if (dt == DT_F32) k_nchw_to_nhwc<float><<<grid, block, 0, s>>>(x, (float *)y, C, HW, round_tf32, inv_scale);
    else if (dt == DT_BF16) k_nchw_to_nhwc<__nv_bfloat16><<<grid, block, 0, s>>>(x, (__nv_bfloat16 *)y, C, HW, 0, inv_scale);
    else if (dt == DT_F16) k_nchw_to_nhwc<__half><<<grid, block, 0, s>>>(x, (__half *)y, C, HW, 0, inv_scale);
    else k_nchw_to_nhwc<int8_t><<<grid, block, 0, s>>>(x, (int8_t *)y, C, HW, 0, inv_scale);
    count_launch();
    return cudaGetLastError();
}

cudaError_t nhwc_to_nchw(const void *x, float *y, int N, int C, int HW, int dt, cudaStream_t s)
{
    if (N <= 0 || C <= 0 || HW <= 0) return cudaSuccess;
    dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
    if (dt == DT_F32) k_nhwc_to_nchw<float><<<grid, block, 0, s>>>((const float *)x, y, C, HW);
    else if (dt == DT_BF16) k_nhwc_to_nchw<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16 *)x, y, C, HW);
    else if (dt == DT_F16) k_nhwc_to_nchw<__half><<<grid, block, 0, s>>>((const __half *)x, y, C, HW);
    else if (dt == DT_S8) k_nhwc_to_nchw<int8_t><<<grid, block, 0, s>>>((const int8_t *)x, y, C, HW);   // the quantised integers as floats
    else return cudaErrorInvalidValue;
    count_launch();
    return cudaGetLastError();
}

// ------------------------------------------------------------------ operand packing
template <typename T>
__global__ void k_pack_conv_weight(const void *__restrict__ w, T *__restrict__ out, int OC, int C, int KH, int KW,
                                   int Kp, int src_is_s8)
{
    const long long total = (long long)OC * Kp;
    const int K = C * KH * KW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int oc = (int)(i / Kp), k = (int)(i % Kp);
        if (k >= K) {
            out[i] = Cvt<T>::zero();
            continue;
        }
        const int c = k % C, t = k / C, kw = t % KW, kh = t / KW;
        const long long src = (((long long)oc * C + c) * KH + kh) * KW + kw;
        if (src_is_s8) {
            const int8_t v = reinterpret_cast<const int8_t *>(w)[src];
            if constexpr (sizeof(T) == 1) out[i] = v;
            else out[i] = Cvt<T>::from((float)v, 0, 1.f);
        } else {
            out[i] = Cvt<T>::from(reinterpret_cast<const float *>(w)[src], 1, 1.f);
        }
    }
}

cudaError_t pack_conv_weight(const void *w, void *out, int OC, int C, int KH, int KW, int Kp, int dt, int src_is_s8,
                             cudaStream_t s)
{
    const long long total = (long long)OC * Kp;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block > 4096 ? 4096 : (total + block - 1) / block);
    if (dt == DT_F32) k_pack_conv_weight<float><<<grid, block, 0, s>>>(w, (float *)out, OC, C, KH, KW, Kp, src_is_s8);
    else if (dt == DT_BF16) k_pack_conv_weight<__nv_bfloat16><<<grid, block, 0, s>>>(w, (__nv_bfloat16 *)out, OC, C, KH, KW, Kp, src_is_s8);
    else if (dt == DT_F16) k_pack_conv_weight<__half><<<grid, block, 0, s>>>(w, (__half *)out, OC, C, KH, KW, Kp, src_is_s8);
    else k_pack_conv_weight<int8_t><<<grid, block, 0, s>>>(w, (int8_t *)out, OC, C, KH, KW, Kp, src_is_s8);
    count_launch();
    return cudaGetLastError();
}

template <typename T>
__global__ void k_pack_rows(const float *__restrict__ a, T *__restrict__ out, long long R, int K, int Kp)
{
    const long long total = R * Kp;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / Kp;
        const int k = (int)(i % Kp);
        out[i] = (k < K) ? Cvt<T>::from(a[r * K + k], 1, 1.f) : Cvt<T>::zero();
    }
}

cudaError_t pack_rows(const float *a, void *out, long long R, int K, int Kp, int dt, cudaStream_t s)
{
    const long long total = R * Kp;
    if (total <= 0) return cudaSuccess;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block > 148 * 16 ? 148 * 16 : (total + block - 1) / block);
    if (dt == DT_F32) k_pack_rows<float><<<grid, block, 0, s>>>(a, (float *)out, R, K, Kp);
    else if (dt == DT_BF16) k_pack_rows<__nv_bfloat16><<<grid, block, 0, s>>>(a, (__nv_bfloat16 *)out, R, K, Kp);
    else if (dt == DT_F16) k_pack_rows<__half><<<grid, block, 0, s>>>(a, (__half *)out, R, K, Kp);
    else return cudaErrorInvalidValue;
    count_launch();
    return cudaGetLastError();
}

template <typename T>
__global__ void k_pack_transposed(const float *__restrict__ b, T *__restrict__ out, int K, int N, int Kp)
{
    __shared__ float tile[32][33];
    const int bi = blockIdx.z;
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    const float *src = b + (size_t)bi * K * N;
    T *dst = out + (size_t)bi * N * Kp;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int k = k0 + i, n = n0 + threadIdx.x;
        tile[i][threadIdx.x] = (k < K && n < N) ? src[(size_t)k * N + n] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int n = n0 + i, k = k0 + threadIdx.x;
        if (n < N && k < Kp) dst[(size_t)n * Kp + k] = Cvt<T>::from(tile[threadIdx.x][i], 1, 1.f);
    }
}

cudaError_t pack_transposed(const float *b, void *out, int batch, int K, int N, int Kp, int dt, cudaStream_t s)
{
    if (batch <= 0 || K <= 0 || N <= 0) return cudaSuccess;
    dim3 grid((N + 31) / 32, (Kp + 31) / 32, batch), block(32, 8);
    if (dt == DT_F32) k_pack_transposed<float><<<grid, block, 0, s>>>(b, (float *)out, K, N, Kp);
    else if (dt == DT_BF16) k_pack_transposed<__nv_bfloat16><<<grid, block, 0, s>>>(b, (__nv_bfloat16 *)out, K, N, Kp);
    else if (dt == DT_F16) k_pack_transposed<__half><<<grid, block, 0, s>>>(b, (__half *)out, K, N, Kp);
    else return cudaErrorInvalidValue;
    count_launch();
    return cudaGetLastError();
}

// ------------------------------------------------------------------ patch matrix
// Non-overlapping patches (stride == kernel, no padding; a ViT patch embedding): the im2col matrix is a
// pure re-ordering of the NCHW image.  K runs (c, kh, kw), the order of the weight tensor itself, so
// the weights need no re-ordering; a thread moves 4 consecutive kw (16 bytes in, 16 or 8 bytes out).
template <typename T>
__global__ void k_patch_pack(const float *__restrict__ x, T *__restrict__ out, long long M, int C, int H, int W, int KH, int KW,
                             int OH, int OW, int Kp)
{
    const int K = C * KH * KW, k4n = Kp >> 2;
    const long long total = M * k4n;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / k4n;
        const int k = (int)(i - m * k4n) << 2;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < K) {
            const int c = k / (KH * KW), r = k - c * KH * KW, kh = r / KW, kw = r - kh * KW;
            const int ow = (int)(m % OW);
            const long long t = m / OW;
            const int oh = (int)(t % OH);
            const long long n = t / OH;
            v = *reinterpret_cast<const float4 *>(x + ((n * C + c) * H + (oh * KH + kh)) * (long long)W + ow * KW + kw);
        }
        T *dst = out + m * Kp + k;
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4 *>(dst) = make_float4(Cvt<T>::from(v.x, 1, 1.f), Cvt<T>::from(v.y, 1, 1.f), Cvt<T>::from(v.z, 1, 1.f), Cvt<T>::from(v.w, 1, 1.f));
        } else {
            dst[0] = Cvt<T>::from(v.x, 1, 1.f); dst[1] = Cvt<T>::from(v.y, 1, 1.f);
            dst[2] = Cvt<T>::from(v.z, 1, 1.f); dst[3] = Cvt<T>::from(v.w, 1, 1.f);
        }
    }
}

cudaError_t patch_pack(const float *x, void *out, int N, int C, int H, int W, int KH, int KW, int Kp, int dt, cudaStream_t s)
{
    const int OH = H / KH, OW = W / KW;
    const long long M = (long long)N * OH * OW, total = M * (Kp / 4);
    if (total <= 0) return cudaSuccess;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block > 148 * 32 ? 148 * 32 : (total + block - 1) / block);
    if (dt == DT_F32) k_patch_pack<float><<<grid, block, 0, s>>>(x, (float *)out, M, C, H, W, KH, KW, OH, OW, Kp);
    else if (dt == DT_BF16) k_patch_pack<__nv_bfloat16><<<grid, block, 0, s>>>(x, (__nv_bfloat16 *)out, M, C, H, W, KH, KW, OH, OW, Kp);
    else if (dt == DT_F16) k_patch_pack<__half><<<grid, block, 0, s>>>(x, (__half *)out, M, C, H, W, KH, KW, OH, OW, Kp);
    else return cudaErrorInvalidValue;
    count_launch();
    return cudaGetLastError();
}

// ------------------------------------------------------------------ explicit im2col
// One thread per output element, k fastest: writes are fully coalesced; reads of an NHWC source
// are coalesced along c, reads of an NCHW source are gathers served from L2.
template <typename TS, typename TD>
__global__ void k_im2col_pack(const TS *__restrict__ x, TD *__restrict__ out, int N, int C, int H, int W, int KH, int KW,
                              int OH, int OW, int stride_w, int stride_h, int pad_t, int pad_l, int Kp, int src_nhwc,
                              float inv_scale)
{
    const long long M = (long long)N * OH * OW;
    const long long total = M * Kp;
    const int K = C * KH * KW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / Kp;
        const int k = (int)(i % Kp);
        TD v = Cvt<TD>::zero();
        if (k < K) {
            const int c = k % C, t = k / C, kw = t % KW, kh = t / KW;
            const int ow = (int)(m % OW);
            const long long t2 = m / OW;
            const int oh = (int)(t2 % OH), n = (int)(t2 / OH);
            const int ih = oh * stride_h + kh - pad_t, iw = ow * stride_w + kw - pad_l;
            if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                const size_t src = src_nhwc ? (((size_t)n * H + ih) * W + iw) * C + c
                                            : (((size_t)n * C + c) * H + ih) * W + iw;
                if constexpr (sizeof(TS) == sizeof(TD)) {
                    if constexpr (sizeof(TS) == 4) v = Cvt<TD>::from(x[src], 1, inv_scale);
                    else v = x[src];
                } else {
                    v = Cvt<TD>::from(Cvt<TS>::to(x[src]), 1, inv_scale);
                }
            }
        }
        out[i] = v;
    }
}

cudaError_t im2col_pack(const void *x, void *out, int N, int C, int H, int W, int KH, int KW, int OH, int OW,
                        int stride_w, int stride_h, int pad_t, int pad_l, int Kp, int src_nhwc, int src_dt, int dt,
                        float inv_scale, cudaStream_t s)
{
    const long long total = (long long)N * OH * OW * Kp;
    if (total <= 0) return cudaSuccess;
    const int block = 256;
    long long g = (total + block - 1) / block;
    const int grid = (int)(g > 148LL * 32 ? 148LL * 32 : g);
#define ONE_I2C(TS, TD)                                                                                      \
    k_im2col_pack<TS, TD><<<grid, block, 0, s>>>((const TS *)x, (TD *)out, N, C, H, W, KH, KW, OH, OW, stride_w, \
                                                 stride_h, pad_t, pad_l, Kp, src_nhwc, inv_scale)
    if (src_dt == DT_F32 && dt == DT_F32) ONE_I2C(float, float);
    else if (src_dt == DT_F32 && dt == DT_BF16) ONE_I2C(float, __nv_bfloat16);
    else if (src_dt == DT_F32 && dt == DT_F16) ONE_I2C(float, __half);
    else if (src_dt == DT_F32 && dt == DT_S8) ONE_I2C(float, int8_t);
    else if (src_dt == DT_BF16 && dt == DT_BF16) ONE_I2C(__nv_bfloat16, __nv_bfloat16);
    else if (src_dt == DT_F16 && dt == DT_F16) ONE_I2C(__half, __half);
    else if (src_dt == DT_S8 && dt == DT_S8) ONE_I2C(int8_t, int8_t);
    else return cudaErrorInvalidValue;
#undef ONE_I2C
    count_launch();
    return cudaGetLastError();
}

// ------------------------------------------------------------------ space-to-depth (stride-2 stems)
// One thread per output pixel (n, hs, ws): it reads, for every channel and both source rows, the two
// horizontally adjacent source values (consecutive threads read consecutive pairs: coalesced) and
// writes its CP channel slots as one contiguous, 16-byte vectorised run.  Slot order
// (bh*2 + bw)*C + c; slots >= 4C and positions outside the image are zero.  C is a template
// parameter so the slots live in registers.
template <typename T, int C, int BW>
__global__ void k_s2d_pack(const float *__restrict__ x, T *__restrict__ out, int N, int H, int W, int Hs, int Ws, float inv_scale)
{
    constexpr int CB = 2 * BW * C * (int)sizeof(T);
    constexpr int CP = (CB <= 32 ? 32 : (CB <= 64 ? 64 : 128)) / (int)sizeof(T);   // must match s2d_plan
    constexpr int NV = CP * (int)sizeof(T) / 16;
    constexpr int OFF = BW / 2 - 1;
    const long long total = (long long)N * Hs * Ws;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ws = (int)(i % Ws);
        const long long t = i / Ws;
        const int hs = (int)(t % Hs);
        const int n = (int)(t / Hs);
        __align__(16) T v[CP];
#pragma unroll
        for (int k = 0; k < CP; ++k) v[k] = Cvt<T>::zero();
#pragma unroll
        for (int c = 0; c < C; ++c) {
#pragma unroll
            for (int bh = 0; bh < 2; ++bh) {
                // position ws carries the columns 2 * (ws - OFF) + bw: with BW = 4 the first position
                // starts two columns left of the image so that every window of four is addressable
                const int ih = 2 * hs + bh, iw = 2 * (ws - OFF);
                if (ih < H) {
                    const float *src = x + (((size_t)n * C + c) * H + ih) * W + iw;
#pragma unroll
                    for (int b2 = 0; b2 < BW; b2 += 2) {   // two columns at a time (8-byte loads when aligned)
                        float a0 = 0.f, a1 = 0.f;
                        const bool in0 = iw + b2 >= 0 && iw + b2 < W, in1 = iw + b2 + 1 >= 0 && iw + b2 + 1 < W;
                        if (in0 && in1 && ((reinterpret_cast<uintptr_t>(src + b2) & 7) == 0)) {
                            const float2 q = *reinterpret_cast<const float2 *>(src + b2);
                            a0 = q.x; a1 = q.y;
                        } else {
                            if (in0) a0 = src[b2];
                            if (in1) a1 = src[b2 + 1];
                        }
                        if (in0) v[(bh * BW + b2) * C + c] = Cvt<T>::from(a0, 1, inv_scale);
                        if (in1) v[(bh * BW + b2 + 1) * C + c] = Cvt<T>::from(a1, 1, inv_scale);
                    }
                }
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)i * CP);
        const uint4 *sv = reinterpret_cast<const uint4 *>(v);
#pragma unroll
        for (int k = 0; k < NV; ++k) dst[k] = sv[k];
    }
}

cudaError_t s2d_pack(const float *x, void *out, int N, int C, int H, int W, int Hs, int Ws, int Cp, int bw, int dt, float inv_scale,
                     cudaStream_t s)
{
    const long long total = (long long)N * Hs * Ws;
    if (total <= 0) return cudaSuccess;
    const int es = dtype_size(dt);
    if (C < 1 || C > 8 || (bw != 2 && bw != 4) || (bw == 4 && C > 4) || 2 * bw * C * es > 128 ||
        Cp != (2 * bw * C * es <= 32 ? 32 : (2 * bw * C * es <= 64 ? 64 : 128)) / es)
        return cudaErrorInvalidValue;   // must match s2d_plan
    const int block = 256;
    long long g = (total + block - 1) / block;
    const int grid = (int)(g > 148LL * 32 ? 148LL * 32 : g);
#define ONE_S2D(T, CC, BB) k_s2d_pack<T, CC, BB><<<grid, block, 0, s>>>(x, (T *)out, N, H, W, Hs, Ws, inv_scale)
#define ONE_S2D_C(T)                                                                                      \
    if (bw == 4) {                                                                                        \
        switch (C) {                                                                                      \
        case 1: ONE_S2D(T, 1, 4); break; case 2: ONE_S2D(T, 2, 4); break; case 3: ONE_S2D(T, 3, 4); break; \
        default: ONE_S2D(T, 4, 4); break;                                                                 \
        }                                                                                                 \
    } else {                                                                                              \
        switch (C) {                                                                                      \
        case 1: ONE_S2D(T, 1, 2); break; case 2: ONE_S2D(T, 2, 2); break; case 3: ONE_S2D(T, 3, 2); break; \
        case 4: ONE_S2D(T, 4, 2); break; case 5: ONE_S2D(T, 5, 2); break; case 6: ONE_S2D(T, 6, 2); break; \
        case 7: ONE_S2D(T, 7, 2); break; default: ONE_S2D(T, 8, 2); break;                                \
        }                                                                                                 \
    }
    if (dt == DT_F32) { ONE_S2D_C(float) }
    else if (dt == DT_BF16) { ONE_S2D_C(__nv_bfloat16) }
    else if (dt == DT_F16) { ONE_S2D_C(__half) }
    else { ONE_S2D_C(int8_t) }
#undef ONE_S2D_C
#undef ONE_S2D
    count_launch();
    return cudaGetLastError();
}

template <typename T>
__global__ void k_pack_conv_weight_s2d(const void *__restrict__ w, T *__restrict__ out, int OC, int C, int KH, int KW, int KH2,
                                       int KW2, int eh, int ew, int Cp, int bwid, int src_is_s8)
{
    const int pitch = KH2 * KW2 * Cp;
    const long long total = (long long)OC * pitch;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int oc = (int)(i / pitch);
        int r = (int)(i % pitch);
        const int cs = r % Cp; r /= Cp;
        const int aw = r % KW2, ah = r / KW2;
        T v = Cvt<T>::zero();
        if (cs < 2 * bwid * C) {
            const int c = cs % C, b = cs / C, bh = b / bwid, bw = b % bwid;
            const int kh = 2 * ah + bh - eh, kw = bwid * aw + bw - ew;
            if (kh >= 0 && kh < KH && kw >= 0 && kw < KW) {
                const long long src = (((long long)oc * C + c) * KH + kh) * KW + kw;
                if (src_is_s8) {
                    const int8_t q = reinterpret_cast<const int8_t *>(w)[src];
                    if constexpr (sizeof(T) == 1) v = q;
                    else v = Cvt<T>::from((float)q, 0, 1.f);
                } else {
                    v = Cvt<T>::from(reinterpret_cast<const float *>(w)[src], 1, 1.f);
                }
            }
        }
        out[i] = v;
    }
}

cudaError_t pack_conv_weight_s2d(const void *w, void *out, int OC, int C, int KH, int KW, int KH2, int KW2, int eh, int ew,
                                 int Cp, int bw, int dt, int src_is_s8, cudaStream_t s)
{
    const long long total = (long long)OC * KH2 * KW2 * Cp;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block > 4096 ? 4096 : (total + block - 1) / block);
    if (dt == DT_F32) k_pack_conv_weight_s2d<float><<<grid, block, 0, s>>>(w, (float *)out, OC, C, KH, KW, KH2, KW2, eh, ew, Cp, bw, src_is_s8);
    else if (dt == DT_BF16) k_pack_conv_weight_s2d<__nv_bfloat16><<<grid, block, 0, s>>>(w, (__nv_bfloat16 *)out, OC, C, KH, KW, KH2, KW2, eh, ew, Cp, bw, src_is_s8);
    else if (dt == DT_F16) k_pack_conv_weight_s2d<__half><<<grid, block, 0, s>>>(w, (__half *)out, OC, C, KH, KW, KH2, KW2, eh, ew, Cp, bw, src_is_s8);
    else k_pack_conv_weight_s2d<int8_t><<<grid, block, 0, s>>>(w, (int8_t *)out, OC, C, KH, KW, KH2, KW2, eh, ew, Cp, bw, src_is_s8);
    count_launch();
    return cudaGetLastError();
}

// ------------------------------------------------------------------ depthwise convolution (NCHW fp32)
// One thread per output element, consecutive threads along the output row.  The taps are summed in
// the reference's order (kh outer, kw inner, separate multiply and add, taps that fall in the
// padding skipped), then + bias, then the activation: bit-identical to
// eval_depthwise_conv_mxn_img2col / eval_depthwise_conv_3x3_pad1 (device/x86/Conv/conv.c:527-755).
__global__ void k_dwconv_nchw(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
                              float *__restrict__ y, int N, int C, int H, int W, int OH, int OW, int KH, int KW, int sx, int sy,
                              int pt, int pl, int act, float p0, float p1, const float *__restrict__ lut)
{
    const long long total = (long long)N * C * OH * OW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(i % OW);
        long long t = i / OW;
        const int oh = (int)(t % OH); t /= OH;
        const int c = (int)(t % C);
        const int n = (int)(t / C);
        const float *xi = x + ((size_t)n * C + c) * H * W;
        const float *wc = w + (size_t)c * KH * KW;
        float psum = 0.f;
        for (int kh = 0; kh < KH; ++kh) {
            const int ih = oh * sy + kh - pt;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < KW; ++kw) {
                const int iw = ow * sx + kw - pl;
                if (iw < 0 || iw >= W) continue;
                psum = __fadd_rn(psum, __fmul_rn(wc[kh * KW + kw], xi[(size_t)ih * W + iw]));
            }
        }
        if (bias) psum = __fadd_rn(psum, bias[c]);
        y[i] = apply_act(psum, act, p0, p1, lut);
    }
}

// int8 flavour, eval_depthwise_conv_mxn_img2col_W8A32 (device/x86/Conv/conv.c:617-760): the fp32 input
// is quantised as it is read (x * (1 / input_scale), clamped, roundf), the int8 taps are summed in
// int32 (exact, so the order is free), then (float)psum * input_scale + (float)bias_s32[c], then
// * (weight_aux[c] * 1 / 127.0f), then the activation.  The reference pads every side by pads[0].
__global__ void k_dwconv_s8_nchw(const float *__restrict__ x, const int8_t *__restrict__ w, const int *__restrict__ bias,
                                 const float *__restrict__ aux, float *__restrict__ y, int N, int C, int H, int W, int OH, int OW,
                                 int KH, int KW, int sx, int sy, int pad, float in_scale, float inv_scale, int act, float p0,
                                 float p1, const float *__restrict__ lut)
{
    const long long total = (long long)N * C * OH * OW;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ow = (int)(i % OW);
        long long t = i / OW;
        const int oh = (int)(t % OH); t /= OH;
        const int c = (int)(t % C);
        const int n = (int)(t / C);
        const float *xi = x + ((size_t)n * C + c) * H * W;
        const int8_t *wc = w + (size_t)c * KH * KW;
        int psum = 0;
        for (int kh = 0; kh < KH; ++kh) {
            const int ih = oh * sy + kh - pad;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < KW; ++kw) {
                const int iw = ow * sx + kw - pad;
                if (iw < 0 || iw >= W) continue;
                psum += (int)wc[kh * KW + kw] * (int)q8(xi[(size_t)ih * W + iw], inv_scale);
            }
        }
        float v = __fmul_rn((float)psum, in_scale);
        if (bias) v = __fadd_rn(v, (float)bias[c]);
        v = __fmul_rn(v, __fdiv_rn(__fmul_rn(aux[c], 1.f), 127.0f));
        y[i] = apply_act(v, act, p0, p1, lut);
    }
}

static inline int dw_grid(long long total, int block)
{
    long long g = (total + block - 1) / block;
    return (int)(g > 148LL * 32 ? 148LL * 32 : g);
}

cudaError_t dwconv_nchw(const float *x, const float *w, const float *bias, float *y, int N, int C, int H, int W, int OH, int OW,
                        int KH, int KW, int sx, int sy, int pt, int pl, int act, float p0, float p1, const float *lut,
                        cudaStream_t s)
{
    const long long total = (long long)N * C * OH * OW;
    if (total <= 0) return cudaSuccess;
    k_dwconv_nchw<<<dw_grid(total, 256), 256, 0, s>>>(x, w, bias, y, N, C, H, W, OH, OW, KH, KW, sx, sy, pt, pl, act, p0, p1, lut);
    count_launch();
    return cudaGetLastError();
}

cudaError_t dwconv_s8_nchw(const float *x, const int8_t *w, const int *bias, const float *aux, float *y, int N, int C, int H,
                           int W, int OH, int OW, int KH, int KW, int sx, int sy, int pad, float in_scale, int act, float p0,
                           float p1, const float *lut, cudaStream_t s)
{
    const long long total = (long long)N * C * OH * OW;
    if (total <= 0) return cudaSuccess;
    k_dwconv_s8_nchw<<<dw_grid(total, 256), 256, 0, s>>>(x, w, bias, aux, y, N, C, H, W, OH, OW, KH, KW, sx, sy, pad, in_scale,
                                                         1.0f / in_scale, act, p0, p1, lut);
    count_launch();
    return cudaGetLastError();
}

__global__ void k_cast_s32_f32(const int *__restrict__ x, float *__restrict__ y, long long n)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) y[i] = (float)x[i];
}

cudaError_t cast_s32_f32(const int *x, float *y, long long n, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    k_cast_s32_f32<<<(int)((n + 255) / 256 > 1024 ? 1024 : (n + 255) / 256), 256, 0, s>>>(x, y, n);
    count_launch();
    return cudaGetLastError();
}

__global__ void k_quantize_s8(const float *__restrict__ x, int8_t *__restrict__ q, long long n, float inv_scale)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        q[i] = q8(x[i], inv_scale);
}

cudaError_t quantize_s8(const float *x, int8_t *q, long long n, float inv_scale, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    const int block = 256;
    long long g = (n + block - 1) / block;
    k_quantize_s8<<<(int)(g > 148LL * 16 ? 148LL * 16 : g), block, 0, s>>>(x, q, n, inv_scale);
    count_launch();
    return cudaGetLastError();
}

}  // namespace one
