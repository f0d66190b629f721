// ctx.cu -- context, workspace, error text and tensor-map encoding (see ctx.h).
#include "ctx.h"

#include <stdarg.h>
#include <stdio.h>

#include <atomic>
#include <map>
#include <mutex>

#include "../../include/one_cuda.h"

namespace one {

static thread_local std::string g_err;
static std::atomic<unsigned long long> g_launches{0};

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

void set_error(const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
}

int fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char *what)
{
    return fail(ONE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

void *ws_alloc(one_ctx *c, size_t bytes)
{
    const size_t off = (c->ws_off + 255) & ~size_t(255);
    if (off + bytes > c->ws_bytes) return nullptr;
    c->ws_off = off + bytes;
    return c->ws + off;
}

// ------------------------------------------------------------------ driver entry points
typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*PFN_encodeIm2col)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encodeTiled = nullptr;
static PFN_encodeIm2col g_encodeIm2col = nullptr;
static int g_driver_version = 0;
static std::once_flag g_entry_once;

static void load_entry_points()
{
    // Resolved through the runtime so the library carries no link-time dependency on libcuda.
    cudaDriverEntryPointQueryResult q;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
        g_encodeTiled = reinterpret_cast<PFN_encodeTiled>(fn);
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
        g_encodeIm2col = reinterpret_cast<PFN_encodeIm2col>(fn);
    cudaDriverGetVersion(&g_driver_version);
}

static CUtensorMapDataType tm_type(int t)
{
    return t == TM_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (t == TM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : (t == TM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8));
}
static CUtensorMapSwizzle tm_swizzle(uint32_t bytes)
{
    if (bytes == TM_SWIZZLE_128B_ATOM_32B) return CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    if (bytes == 0) return CU_TENSOR_MAP_SWIZZLE_NONE;
    return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}
static size_t tm_esize(int t) { return t == TM_F32 ? 4 : ((t == TM_BF16 || t == TM_F16) ? 2 : 1); }

int make_tmap_tiled(CUtensorMap *m, int type, const void *base, uint64_t inner, uint64_t rows, uint64_t batch,
                    uint64_t row_pitch_bytes, uint64_t batch_pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                    uint32_t swizzle_bytes)
{
    std::call_once(g_entry_once, load_entry_points);
    if (!g_encodeTiled) return fail(ONE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_pitch_bytes & 15) || (batch_pitch_bytes & 15))
        return fail(ONE_ERR_BAD_ARG, "tensor map operand is not 16-byte aligned (base %p, pitch %llu)", base,
                    (unsigned long long)row_pitch_bytes);
    const cuuint32_t rank = batch > 0 ? 3 : 2;
    cuuint64_t dims[3] = {inner, rows, batch > 0 ? batch : 1};
    cuuint64_t strides[2] = {row_pitch_bytes, batch_pitch_bytes};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encodeTiled(m, tm_type(type), rank, const_cast<void *>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, tm_swizzle(swizzle_bytes),
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ONE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d): inner %llu rows %llu pitch %llu box %u x %u",
                    (int)r, (unsigned long long)inner, (unsigned long long)rows,
                    (unsigned long long)row_pitch_bytes, box_inner, box_rows);
    return ONE_OK;
}

int make_tmap_im2col(CUtensorMap *m, int type, const void *base, int C, int W, int H, int N, int pad_l, int pad_t,
                     int pad_r, int pad_b, int KW, int KH, int stride_w, int stride_h, uint32_t channels,
                     uint32_t pixels, uint32_t swizzle_bytes)
{
    std::call_once(g_entry_once, load_entry_points);
    if (!g_encodeIm2col) return fail(ONE_ERR_CUDA, "cuTensorMapEncodeIm2col is not available from this driver");
    const size_t es = tm_esize(type);
    if ((reinterpret_cast<uintptr_t>(base) & 15) || ((C * es) & 15))
        return fail(ONE_ERR_BAD_ARG, "im2col tensor map operand is not 16-byte aligned");
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)C * es, (cuuint64_t)W * C * es, (cuuint64_t)H * W * C * es};
    // Bounding box of the base pixel (the filter's top-left tap), innermost (W) first: it starts
    // in the padding and stops where the filter's far edge meets the far padding.
    int lower[2] = {-pad_l, -pad_t};
    int upper[2] = {pad_r - (KW - 1), pad_b - (KH - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)stride_w, (cuuint32_t)stride_h, 1};
    CUresult r = g_encodeIm2col(m, tm_type(type), 4, const_cast<void *>(base), dims, strides, lower, upper, channels,
                                pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, tm_swizzle(swizzle_bytes),
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ONE_ERR_CUDA, "cuTensorMapEncodeIm2col failed (%d): C %d W %d H %d N %d", (int)r, C, W, H, N);
    // Drivers up to 13.1 encode im2col maps of tensors smaller than 128 KiB with a flag that
    // makes the loads misbehave; the CUTLASS im2col descriptor builder clears bit 21 of the
    // second 64-bit word in that case, and so do we.
    if (g_driver_version <= 13010 && (size_t)N * H * W * C * es < 131072)
        reinterpret_cast<uint64_t *>(m)[1] &= ~(1ull << 21);
    return ONE_OK;
}

// ------------------------------------------------------------------ default contexts
static std::mutex g_ctx_mu;
static std::map<int, one_ctx *> g_default_ctx;

int default_ctx(one_ctx **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice (no usable CUDA device: this backend has no CPU fallback)");
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    auto it = g_default_ctx.find(dev);
    if (it != g_default_ctx.end()) {
        *out = it->second;
        return ONE_OK;
    }
    one_ctx *c = nullptr;
    int rc = one_cuda_init(dev, 0, &c);
    if (rc != ONE_OK) return rc;
    g_default_ctx[dev] = c;
    *out = c;
    return ONE_OK;
}

}  // namespace one

using namespace one;

extern "C" int one_cuda_init(int device, size_t workspace_bytes, one_ctx **out)
{
    if (!out) return fail(ONE_ERR_BAD_ARG, "one_cuda_init: out is null");
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return fail(ONE_ERR_CUDA, "no usable CUDA device (%s): this backend has no CPU fallback",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= ndev) return fail(ONE_ERR_BAD_ARG, "device %d out of range [0,%d)", device, ndev);
    int prev = 0;
    cudaGetDevice(&prev);
    if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
    if (prop.major != 10)
        return fail(ONE_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library holds sm_100a code only", device,
                    prop.major, prop.minor);
    one_ctx *c = new one_ctx();
    c->device = device;
    c->ws_bytes = workspace_bytes ? workspace_bytes : (size_t(256) << 20);
    if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaMalloc(&c->ws, c->ws_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&c->status_dev, sizeof(unsigned int))) != cudaSuccess ||
        (e = cudaMemset(c->status_dev, 0, sizeof(unsigned int))) != cudaSuccess ||
        (e = cudaMalloc(&c->ident16[0], 2 * 64 * 64 * 2)) != cudaSuccess) {
        int rc = cuda_fail(e, "one_cuda_init allocation");
        if (c->ws) cudaFree(c->ws);
        if (c->status_dev) cudaFree(c->status_dev);
        if (c->ident16[0]) cudaFree(c->ident16[0]);
        if (c->stream) cudaStreamDestroy(c->stream);
        delete c;
        cudaSetDevice(prev);
        return rc;
    }
    {   // 1.0 on the diagonal: 0x3F80 in bf16, 0x3C00 in fp16
        static uint16_t host[2][64 * 64];
        for (int f = 0; f < 2; ++f)
            for (int i = 0; i < 64 * 64; ++i) host[f][i] = (i / 64 == i % 64) ? (f ? 0x3C00 : 0x3F80) : 0;
        c->ident16[1] = reinterpret_cast<uint8_t *>(c->ident16[0]) + 64 * 64 * 2;
        if ((e = cudaMemcpy(c->ident16[0], host, sizeof(host), cudaMemcpyHostToDevice)) != cudaSuccess) {
            int rc = cuda_fail(e, "one_cuda_init identity upload");
            one_cuda_release(c);
            cudaSetDevice(prev);
            return rc;
        }
    }
    cudaSetDevice(prev);
    *out = c;
    return ONE_OK;
}

extern "C" int one_cuda_release(one_ctx *c)
{
    if (!c) return ONE_OK;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    cudaFree(c->ws);
    cudaFree(c->status_dev);
    cudaFree(c->ident16[0]);
    cudaStreamDestroy(c->stream);
    delete c;
    return ONE_OK;
}

extern "C" void *one_cuda_stream(one_ctx *c) { return c ? (void *)c->stream : nullptr; }

extern "C" int one_cuda_status(one_ctx *c)
{
    if (!c) return fail(ONE_ERR_BAD_ARG, "one_cuda_status: null context");
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) return cuda_fail(e, "stream synchronise");
    unsigned int st = 0;
    if ((e = cudaMemcpy(&st, c->status_dev, sizeof(st), cudaMemcpyDeviceToHost)) != cudaSuccess)
        return cuda_fail(e, "status read");
    if (st) {
        cudaMemset(c->status_dev, 0, sizeof(st));
        return status_fail(st);
    }
    return ONE_OK;
}

extern "C" const char *one_cuda_last_error(void) { return g_err.c_str(); }

extern "C" unsigned long long one_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
