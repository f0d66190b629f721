// ctx.h -- per-device context of the backend: stream, scratch workspace (bump allocated,
// stream ordered), device status word, driver entry points for tensor-map encoding, and the
// error-text channel.  Internal to the library; the public view is include/one_cuda.h.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

struct one_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    uint8_t *ws = nullptr;      // scratch workspace
    size_t ws_bytes = 0;
    size_t ws_off = 0;          // bump offset of the call in progress
    unsigned int *status_dev = nullptr;
    bool allow_split = true;    // split-K contractions may take scratch for their partial sums
    void *ident16[2] = {nullptr, nullptr};   // 64 x 64 identity matrices in bf16 [0] and fp16 [1] (residual added by the tensor core)
};

namespace one {

void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);          // set_error + return code
int cuda_fail(cudaError_t e, const char *what);    // ONE_ERR_CUDA with the runtime's text
int status_fail(unsigned int status_word);         // the error a non-zero device status word stands for

// Workspace: reset at the start of every operator call, 256-byte aligned blocks.
inline void ws_reset(one_ctx *c) { c->ws_off = 0; }
void *ws_alloc(one_ctx *c, size_t bytes);          // nullptr when the workspace is too small

// Process-wide default context of the current device (created on first use), used by the
// drop-in eval entry points which carry no context argument.
int default_ctx(one_ctx **out);

// Every kernel launch of this library is counted (read with one_cuda_launch_count()).
void count_launch(int n = 1);

enum TmapType { TM_F32 = 0, TM_BF16 = 1, TM_U8 = 2, TM_F16 = 3 };
// `swizzle_bytes` value selecting the 128-byte swizzle that moves 32-byte chunks (the layout the
// tensor core wants for an MN-major operand of 32-bit elements).
constexpr uint32_t TM_SWIZZLE_128B_ATOM_32B = 129;
// Tiled map over a row-major matrix (optionally batched): dims (inner, rows[, batch]).
int make_tmap_tiled(CUtensorMap *m, int type, const void *base, uint64_t inner, uint64_t rows, uint64_t batch,
                    uint64_t row_pitch_bytes, uint64_t batch_pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                    uint32_t swizzle_bytes);
// im2col-mode map over an NHWC activation: dims (C, W, H, N); the box walks 128 output pixels.
int make_tmap_im2col(CUtensorMap *m, int type, const void *base, int C, int W, int H, int N, int pad_l, int pad_t,
                     int pad_r, int pad_b, int KW, int KH, int stride_w, int stride_h, uint32_t channels,
                     uint32_t pixels, uint32_t swizzle_bytes);

}  // namespace one
