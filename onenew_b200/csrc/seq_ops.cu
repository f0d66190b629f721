// seq_ops.cu -- device versions of the glue operators between the MatMul / Gemm calls of a
// transformer encoder (ViT), so the token sequence stays resident on the GPU:
// LayerNormalization, Gelu (table), Softmax, Transpose, the copy operators (Concat, Gather with a
// fixed index) and the broadcasting arithmetic operators (Add, Sub, Mul, Div).  All tensors are
// fp32 in the reference's row-major layout.  Every kernel is a streaming, HBM-bound pass: one read
// and one write of each element, 16-byte accesses where the shape allows.
//
// Reference arithmetic followed:
//   LayerNormalization  device/x86/LayerNormalization/layer_normalization.c:59-98  one pass sum and
//       sum of squares, var = E[x^2] - mean^2 (+1e-20), y = (x - mean) * (1/sqrt(var)) * w + b;
//   Gelu     device/x86/Gelu/gelu.c:22-38      x < -8 -> 0, x >= 8 -> x, else table[(int)((x+8)*512)];
//   Softmax  device/x86/Softmax/softmax.c:31-76  last axis, running maximum starts at -32768;
//   Transpose  device/x86/Transpose/transpose.c:27-140  out[o] = in[sum o_i * in_stride[perm[i]]];
//   Concat   device/x86/Concat/concat.c:10-66; Gather  device/x86/Gather/gather.c:10-33;
//   Add / Sub / Mul / Div  device/x86/Add/add.c:17-86 (numpy broadcasting; a scalar divisor is
//       applied as a multiplication by its reciprocal, device/x86/Div/div.c:104-118).
#include "../../include/one_glue.h"
#include "ctx.h"

using namespace one;

namespace {

inline int grid_for(long long work, int block)
{
    long long g = (work + block - 1) / block;
    const long long cap = 148LL * 16;
    if (g > cap) g = cap;
    return g < 1 ? 1 : (int)g;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------ LayerNormalization
// One warp per row; the row is read once into registers when it fits (D <= 32 * 4 * RV).
template <int RV>   // float4 per lane kept in registers
__global__ void k_layernorm(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                            float *__restrict__ y, long long rows, int D)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const int dv = D >> 2;
    const float inv_d = 1.0f / D;
    for (long long r = warp; r < rows; r += nwarps) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + r * D);
        float4 v[RV];
        float s = 0.f, ss = 0.f;
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int j = lane + 32 * i;
            if (j < dv) {
                v[i] = xr[j];
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
            }
        }
        s = warp_sum(s);
        ss = warp_sum(ss);
        const float mean = s * inv_d;
        float var = inv_d * ss - mean * mean;
        var = (float)((double)var + 1e-20);
        const float inv_std = 1.0f / sqrtf(var);
        float4 *yr = reinterpret_cast<float4 *>(y + r * D);
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int j = lane + 32 * i;
            if (j < dv) {
                const float4 ww = reinterpret_cast<const float4 *>(w)[j], bb = reinterpret_cast<const float4 *>(b)[j];
                float4 o;
                o.x = (v[i].x - mean) * inv_std * ww.x + bb.x;
                o.y = (v[i].y - mean) * inv_std * ww.y + bb.y;
                o.z = (v[i].z - mean) * inv_std * ww.z + bb.z;
                o.w = (v[i].w - mean) * inv_std * ww.w + bb.w;
                yr[j] = o;
            }
        }
    }
}

// Any D: two passes over the row (the second one is served from cache).
__global__ void k_layernorm_any(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                                float *__restrict__ y, long long rows, int D)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const float inv_d = 1.0f / D;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * D;
        float s = 0.f, ss = 0.f;
        for (int j = lane; j < D; j += 32) {
            const float t = xr[j];
            s += t;
            ss += t * t;
        }
        s = warp_sum(s);
        ss = warp_sum(ss);
        const float mean = s * inv_d;
        float var = inv_d * ss - mean * mean;
        var = (float)((double)var + 1e-20);
        const float inv_std = 1.0f / sqrtf(var);
        for (int j = lane; j < D; j += 32) y[r * D + j] = (xr[j] - mean) * inv_std * w[j] + b[j];
    }
}

// ------------------------------------------------------------------ Gelu (table)
__device__ __forceinline__ float gelu_lut(float v, const float *__restrict__ lut)
{
    if (v < -8.0f) return 0.f;
    if (v >= 8.0f) return v;
    return lut[(int)((v + 8.0f) * 512.0f)];
}
template <bool VEC>
__global__ void k_gelu(const float *__restrict__ x, const float *__restrict__ lut, float *__restrict__ y, long long n)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const long long nv = n >> 2;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
            float4 t = reinterpret_cast<const float4 *>(x)[i];
            t.x = gelu_lut(t.x, lut); t.y = gelu_lut(t.y, lut); t.z = gelu_lut(t.z, lut); t.w = gelu_lut(t.w, lut);
            reinterpret_cast<float4 *>(y)[i] = t;
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) y[i] = gelu_lut(x[i], lut);
    }
}

// ------------------------------------------------------------------ Softmax over the last axis
// One warp per row, the row held in registers (D <= 32 * RV), exp evaluated once per element.
template <int RV>
__global__ void k_softmax(const float *__restrict__ x, float *__restrict__ y, long long rows, int D)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * D;
        float v[RV];
        float m = -32768.0f;
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int j = lane + 32 * i;
            v[i] = j < D ? xr[j] : -32768.0f;
            m = fmaxf(m, v[i]);
        }
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int j = lane + 32 * i;
            v[i] = j < D ? expf(v[i] - m) : 0.f;
            s += v[i];
        }
        s = warp_sum(s);
        const float inv = 1.0f / s;
#pragma unroll
        for (int i = 0; i < RV; ++i) {
            const int j = lane + 32 * i;
            if (j < D) y[r * D + j] = v[i] * inv;
        }
    }
}
__global__ void k_softmax_any(const float *__restrict__ x, float *__restrict__ y, long long rows, int D)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *xr = x + r * D;
        float m = -32768.0f;
        for (int j = lane; j < D; j += 32) m = fmaxf(m, xr[j]);
        m = warp_max(m);
        float s = 0.f;
        for (int j = lane; j < D; j += 32) {
            const float e = expf(xr[j] - m);
            y[r * D + j] = e;
            s += e;
        }
        s = warp_sum(s);
        const float inv = 1.0f / s;
        for (int j = lane; j < D; j += 32) y[r * D + j] *= inv;
    }
}

// ------------------------------------------------------------------ Transpose (up to 6 dims)
struct Dims6 {
    int shape[6];          // output shape, padded with 1 in front
    long long stride[6];   // input stride of each output dim
};
// Generic gather: consecutive threads write consecutive outputs.
__global__ void k_transpose(const float *__restrict__ x, float *__restrict__ y, long long n, Dims6 d)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long t = i, off = 0;
#pragma unroll
        for (int k = 5; k >= 0; --k) {
            const int q = (int)(t % d.shape[k]);
            t /= d.shape[k];
            off += q * d.stride[k];
        }
        y[i] = x[off];
    }
}
// The two innermost output dims swap memory order (out[.., a, b] = in[.., b, a] with `a` contiguous
// in the input): 32x32 tiles through shared memory keep both sides coalesced.  `outer` output
// dims (4) are folded into blockIdx.z.
__global__ void k_transpose_tile(const float *__restrict__ x, float *__restrict__ y, Dims6 d, int A, int B,
                                 long long stride_b_in)
{
    __shared__ float tile[32][33];
    long long z = blockIdx.z, off_in = 0;
#pragma unroll
    for (int k = 3; k >= 0; --k) {
        const int q = (int)(z % d.shape[k]);
        z /= d.shape[k];
        off_in += q * d.stride[k];
    }
    const long long off_out = (long long)blockIdx.z * A * B;
    const int a0 = blockIdx.y * 32, b0 = blockIdx.x * 32;
    // out[a][b] = in[b * stride_b_in + a]
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int b = b0 + i, a = a0 + threadIdx.x;
        if (a < A && b < B) tile[i][threadIdx.x] = x[off_in + b * stride_b_in + a];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int a = a0 + i, b = b0 + threadIdx.x;
        if (a < A && b < B) y[off_out + (long long)a * B + b] = tile[threadIdx.x][i];
    }
}

// ------------------------------------------------------------------ chunk copy (Concat / Gather)
// y[r * y_stride + i] = x[(r % x_reps) * x_stride + i]   for r < reps, i < chunk
template <bool VEC>
__global__ void k_copy_chunks(const float *__restrict__ x, float *__restrict__ y, long long reps, long long chunk,
                              long long x_reps, long long x_stride, long long y_stride)
{
    const long long cw = VEC ? (chunk >> 2) : chunk;
    const long long total = reps * cw;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cw, c = i - r * cw;
        if (VEC)
            reinterpret_cast<float4 *>(y + r * y_stride)[c] = reinterpret_cast<const float4 *>(x + (r % x_reps) * x_stride)[c];
        else
            y[r * y_stride + c] = x[(r % x_reps) * x_stride + c];
    }
}

// ------------------------------------------------------------------ broadcasting arithmetic
template <int OP> __device__ __forceinline__ float binop(float a, float b)
{
    if (OP == 0) return a + b;
    if (OP == 1) return a - b;
    if (OP == 2) return a * b;
    if (OP == 4) return a * (1.0f / b);   // scalar divisor, as device/x86/Div/div.c:104-118 applies it
    return a / b;
}
// b repeats with period `period` over the flat index of a (equal shapes, a scalar, a trailing
// vector such as a bias, or a tensor broadcast over the leading batch dim).
template <int OP, bool VEC, bool SWAP>
__global__ void k_binary_period(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, long long n,
                                long long period)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const long long nv = n >> 2, pv = period >> 2;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
            const float4 p = reinterpret_cast<const float4 *>(a)[i];
            const float4 q = reinterpret_cast<const float4 *>(b)[i % pv];
            float4 o;
            o.x = SWAP ? binop<OP>(q.x, p.x) : binop<OP>(p.x, q.x);
            o.y = SWAP ? binop<OP>(q.y, p.y) : binop<OP>(p.y, q.y);
            o.z = SWAP ? binop<OP>(q.z, p.z) : binop<OP>(p.z, q.z);
            o.w = SWAP ? binop<OP>(q.w, p.w) : binop<OP>(p.w, q.w);
            reinterpret_cast<float4 *>(y)[i] = o;
        }
    } else {
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
            const float p = a[i], q = b[i % period];
            y[i] = SWAP ? binop<OP>(q, p) : binop<OP>(p, q);
        }
    }
}
// Anything else: per-dim strides (0 on a broadcast dim).
template <int OP>
__global__ void k_binary_strided(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, long long n,
                                 Dims6 da, Dims6 db)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        long long t = i, oa = 0, ob = 0;
#pragma unroll
        for (int k = 5; k >= 0; --k) {
            const int q = (int)(t % da.shape[k]);
            t /= da.shape[k];
            oa += q * da.stride[k];
            ob += q * db.stride[k];
        }
        y[i] = binop<OP>(a[oa], b[ob]);
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int OP>
cudaError_t launch_binary_period(const float *a, const float *b, float *y, long long n, long long period, bool swap,
                                 cudaStream_t st)
{
    const bool vec = (n % 4 == 0) && (period % 4 == 0) && aligned16(a) && aligned16(b) && aligned16(y);
    const int block = 256;
    const int grid = grid_for(vec ? n / 4 : n, block);
    if (vec) {
        if (swap) k_binary_period<OP, true, true><<<grid, block, 0, st>>>(a, b, y, n, period);
        else k_binary_period<OP, true, false><<<grid, block, 0, st>>>(a, b, y, n, period);
    } else {
        if (swap) k_binary_period<OP, false, true><<<grid, block, 0, st>>>(a, b, y, n, period);
        else k_binary_period<OP, false, false><<<grid, block, 0, st>>>(a, b, y, n, period);
    }
    return cudaGetLastError();
}

}  // namespace

extern "C" int one_glue_layernorm(const float *x, const float *w, const float *b, float *y, long long rows, int D, void *stream)
{
    if (!x || !w || !b || !y || rows < 0 || D <= 0) return fail(ONE_ERR_BAD_ARG, "layernorm: bad argument");
    if (rows == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 256;
    const int grid = grid_for(rows * 32, block);
    const bool vec = D % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(w) && aligned16(b);
    if (vec && D <= 256) k_layernorm<2><<<grid, block, 0, st>>>(x, w, b, y, rows, D);
    else if (vec && D <= 1024) k_layernorm<8><<<grid, block, 0, st>>>(x, w, b, y, rows, D);
    else k_layernorm_any<<<grid, block, 0, st>>>(x, w, b, y, rows, D);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "layernorm launch");
}

extern "C" int one_glue_gelu_lut(const float *x, const float *lut, float *y, long long n, void *stream)
{
    if (!x || !lut || !y || n < 0) return fail(ONE_ERR_BAD_ARG, "gelu: bad argument");
    if (n == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool vec = n % 4 == 0 && aligned16(x) && aligned16(y);
    if (vec) k_gelu<true><<<grid_for(n / 4, 256), 256, 0, st>>>(x, lut, y, n);
    else k_gelu<false><<<grid_for(n, 256), 256, 0, st>>>(x, lut, y, n);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "gelu launch");
}

extern "C" int one_glue_softmax_rows(const float *x, float *y, long long rows, int D, void *stream)
{
    if (!x || !y || rows < 0 || D <= 0) return fail(ONE_ERR_BAD_ARG, "softmax: bad argument");
    if (rows == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int block = 256;
    const int grid = grid_for(rows * 32, block);
    if (D <= 64) k_softmax<2><<<grid, block, 0, st>>>(x, y, rows, D);
    else if (D <= 256) k_softmax<8><<<grid, block, 0, st>>>(x, y, rows, D);
    else if (D <= 1024) k_softmax<32><<<grid, block, 0, st>>>(x, y, rows, D);
    else k_softmax_any<<<grid, block, 0, st>>>(x, y, rows, D);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "softmax launch");
}

extern "C" int one_glue_transpose(const float *x, float *y, int ndim, const int *in_shape, const int *perm, void *stream)
{
    if (!x || !y || !in_shape || !perm || ndim < 1 || ndim > 6) return fail(ONE_ERR_BAD_ARG, "transpose: 1..6 dims");
    long long in_stride[6], n = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        if (in_shape[i] <= 0) return fail(ONE_ERR_BAD_SHAPE, "transpose: non-positive dimension");
        in_stride[i] = n;
        n *= in_shape[i];
    }
    Dims6 d;
    const int pad = 6 - ndim;
    for (int k = 0; k < pad; ++k) { d.shape[k] = 1; d.stride[k] = 0; }
    unsigned seen = 0;
    for (int i = 0; i < ndim; ++i) {
        if (perm[i] < 0 || perm[i] >= ndim || (seen >> perm[i] & 1)) return fail(ONE_ERR_BAD_ARG, "transpose: perm is not a permutation");
        seen |= 1u << perm[i];
        d.shape[pad + i] = in_shape[perm[i]];
        d.stride[pad + i] = in_stride[perm[i]];
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    long long outer = 1;
    for (int k = 0; k < 4; ++k) outer *= d.shape[k];
    // out[.., a, b] with the input contiguous along a (stride 1) and b a strided input dim
    if (d.stride[4] == 1 && d.shape[4] >= 8 && d.shape[5] >= 8 && outer <= 0x7fffffffLL / 2 && outer <= 65535) {
        dim3 grid((d.shape[5] + 31) / 32, (d.shape[4] + 31) / 32, (unsigned)outer), block(32, 8);
        k_transpose_tile<<<grid, block, 0, st>>>(x, y, d, d.shape[4], d.shape[5], d.stride[5]);
    } else {
        k_transpose<<<grid_for(n, 256), 256, 0, st>>>(x, y, n, d);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "transpose launch");
}

extern "C" int one_glue_copy_chunks(const float *x, float *y, long long reps, long long chunk, long long x_reps,
                                    long long x_stride, long long y_stride, void *stream)
{
    if (!x || !y || reps < 0 || chunk < 0 || x_reps <= 0) return fail(ONE_ERR_BAD_ARG, "copy_chunks: bad argument");
    if (reps == 0 || chunk == 0) return ONE_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool vec = chunk % 4 == 0 && x_stride % 4 == 0 && y_stride % 4 == 0 && aligned16(x) && aligned16(y);
    if (vec) k_copy_chunks<true><<<grid_for(reps * (chunk / 4), 256), 256, 0, st>>>(x, y, reps, chunk, x_reps, x_stride, y_stride);
    else k_copy_chunks<false><<<grid_for(reps * chunk, 256), 256, 0, st>>>(x, y, reps, chunk, x_reps, x_stride, y_stride);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "copy_chunks launch");
}

extern "C" int one_glue_binary(int op, const float *a, const float *b, float *y, int ndim, const int *a_shape,
                               const int *b_shape, void *stream)
{
    if (!a || !b || !y || !a_shape || !b_shape || ndim < 1 || ndim > 6 || op < 0 || op > 3)
        return fail(ONE_ERR_BAD_ARG, "binary: bad argument");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int os[6];
    long long n = 1, na = 1, nb = 1;
    for (int i = 0; i < ndim; ++i) {
        if (a_shape[i] <= 0 || b_shape[i] <= 0) return fail(ONE_ERR_BAD_SHAPE, "binary: non-positive dimension");
        if (a_shape[i] != b_shape[i] && a_shape[i] != 1 && b_shape[i] != 1)
            return fail(ONE_ERR_BAD_SHAPE, "binary: shapes do not broadcast (dim %d: %d vs %d)", i, a_shape[i], b_shape[i]);
        os[i] = a_shape[i] > b_shape[i] ? a_shape[i] : b_shape[i];
        n *= os[i]; na *= a_shape[i]; nb *= b_shape[i];
    }
    // periodic forms: the smaller operand is the trailing part of the larger one (its leading dims are 1)
    auto trailing = [&](const int *small, long long nsmall) {
        long long p = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            if (p == nsmall) return true;
            if (small[i] != os[i]) return false;
            p *= small[i];
        }
        return p == nsmall;
    };
    cudaError_t e;
    if (na == n && trailing(b_shape, nb)) {
        switch (op == 3 && nb == 1 ? 4 : op) {
        case 0: e = launch_binary_period<0>(a, b, y, n, nb, false, st); break;
        case 4: e = launch_binary_period<4>(a, b, y, n, nb, false, st); break;
        case 1: e = launch_binary_period<1>(a, b, y, n, nb, false, st); break;
        case 2: e = launch_binary_period<2>(a, b, y, n, nb, false, st); break;
        default: e = launch_binary_period<3>(a, b, y, n, nb, false, st); break;
        }
    } else if (nb == n && trailing(a_shape, na)) {
        switch (op) {
        case 0: e = launch_binary_period<0>(b, a, y, n, na, true, st); break;
        case 1: e = launch_binary_period<1>(b, a, y, n, na, true, st); break;
        case 2: e = launch_binary_period<2>(b, a, y, n, na, true, st); break;
        default: e = launch_binary_period<3>(b, a, y, n, na, true, st); break;
        }
    } else {
        Dims6 da, db;
        const int pad = 6 - ndim;
        for (int k = 0; k < pad; ++k) { da.shape[k] = 1; da.stride[k] = 0; db.shape[k] = 1; db.stride[k] = 0; }
        long long sa = 1, sb = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            da.shape[pad + i] = db.shape[pad + i] = os[i];
            da.stride[pad + i] = a_shape[i] == 1 ? 0 : sa;
            db.stride[pad + i] = b_shape[i] == 1 ? 0 : sb;
            sa *= a_shape[i];
            sb *= b_shape[i];
        }
        const int grid = grid_for(n, 256);
        switch (op) {
        case 0: k_binary_strided<0><<<grid, 256, 0, st>>>(a, b, y, n, da, db); break;
        case 1: k_binary_strided<1><<<grid, 256, 0, st>>>(a, b, y, n, da, db); break;
        case 2: k_binary_strided<2><<<grid, 256, 0, st>>>(a, b, y, n, da, db); break;
        default: k_binary_strided<3><<<grid, 256, 0, st>>>(a, b, y, n, da, db); break;
        }
        e = cudaGetLastError();
    }
    count_launch();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "binary launch");
}
