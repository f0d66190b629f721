// igemm.cuh -- parameters of the implicit-GEMM contraction kernel shared by Conv, Gemm and
// MatMul:  D[M, N] = A[M, K] * B[N, K]^T  (+ epilogue), both operands K-major.
//   Conv:   M = batch*OH*OW output pixels, N = OC, K = KH*KW*C; A is the NHWC activation read
//           through an im2col-mode tensor map (padding = out-of-bounds zero fill, stride = the
//           map's traversal stride), B is the weight re-ordered to [OC][KH][KW][C].
//   Gemm / MatMul / 1x1 stride-1 conv: A is a plain row-major [M][K] matrix (tiled map).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace one {

enum OutMode { OUT_F32 = 0, OUT_BF16 = 1, OUT_RAW32 = 2 /* accumulator bits, no epilogue */, OUT_F16 = 3 };
__host__ __device__ inline bool out_is_16(int mode) { return mode == OUT_BF16 || mode == OUT_F16; }
// BIAS_S32_DEQUANT: the int8 three-step epilogue; `bias` then holds the int32 bias ALREADY converted
// to float (an exact int -> float cast, done once by the host or by a small kernel).
enum BiasMode { BIAS_NONE = 0, BIAS_F32 = 1, BIAS_S32_DEQUANT = 2 };

struct IgemmParams {
    int M, N, num_kb;
    int slab_bytes;   // bytes of K per pipeline stage row: 32, 64 or 128 (= the TMA swizzle span)
    int slab_elems;   // slab_bytes / element size
    // A addressing
    int a_im2col;     // 0: tiled 2-D [M][K]; 1: im2col 4-D (C, W, H, N)
    int batched, batch;          // batched MatMul: 3-D maps (K, rows, batch), grid.y = batch
    long long out_batch_stride;  // elements between consecutive batches of out
    int OW, OH, stride_w, stride_h, pad_l, pad_t, KW, KH, c_slabs;
    int dil_w;            // im2col: positions between consecutive filter taps along w (1 unless space-to-depth x4)
    // epilogue
    void *out;            // [M][ldo] f32 / bf16 / fp16 / raw 32-bit; may be null when out_q is set
    long long ldo;        // row pitch of out, residual and out_q, in elements
    int out_mode;
    int bias_mode;
    const void *bias;     // f32[N]
    const float *coeff;   // int8: weight_aux[oc] * 1 / 127.0f, per column
    float in_scale;       // int8: activation scale of this layer's input
    int act;              // ACT_TYPE_E
    float act_p0, act_p1; // clip min/max | leaky alpha | hard-sigmoid alpha, beta
    const float *lut;     // SiLU / Gelu table (8192 entries)
    int lut_smem;         // stage the table in shared memory (only without a residual; 16-byte aligned table)
    const void *residual; // optional [M][ldo], same element type as out; added before res_relu
    int res_relu;         // relu after the residual add
    int round_tf32;       // round f32 outputs to tf32 (nearest) so a tf32 consumer sees exact values
    int ab_f16;           // 16-bit kind: the operands are fp16, not bf16
    int res_mma;          // 16-bit kinds, plain tiles, 128-byte slabs: the residual is added by the tensor core -- the
                          // launcher's tmR is then an operand map over the residual tensor (box 64 columns x 128 rows)
                          // and tmI one over a 64 x 64 identity; `residual` is null and the epilogue adds nothing
    int8_t *out_q;        // optional int8 copy of the output quantised for the next int8 layer
    float q_inv_scale;    // 1.0f / next layer's input_scale
    int tma_store;        // epilogue writes through the third tensor map: 1 = out (no out_q, N % 32 == 0), 2 = out_q only (int8)
    // Split-K (launches with fewer tiles than SMs): split_k > 1 cuts the K blocks into split_k ranges of
    // kb_per_split; work unit (tile, z) accumulates range z and stores its raw fp32 partial sums into
    // plane z of `out` ([split_k][M][ldo], planes out_batch_stride apart).  Bias, activation and residual
    // are then applied by splitk_reduce, which adds the planes in a fixed order.
    int split_k, kb_per_split;
    int pdl;              // launched with programmatic stream serialisation (see launch_igemm)
    int epi_mode;         // bit 0: both epilogue groups share a CTA's only tile; bit 1: two output patches per warp; bit 2: early accumulator release
    unsigned int *status; // device status word (timeouts, fp16 range)
};

// Host-side launcher.  kind: 0 tf32, 1 bf16, 2 int8.  bn: 64, 128, 192 or 256.  pair: run as clusters of two
// CTAs sharing 256-row tiles (bn 128 / 192 / 256; not batched, not split-K); tmB's box then holds bn / 2 rows.
// tmC / tmR (may be null): maps over the output and the residual with a 32-column x 32-row box; used
// when p.tma_store (tmR when a residual is given as well).
// epi_warps: 8, or 12 (three epilogue groups; plain tiles of width 64 / 128 only, shallower operand ring).
// mh: 128-row halves per CTA tile, 1 or 2 (2: single CTAs with bn 64 / 128 only; a K block then brings 256 rows of A).
cudaError_t launch_igemm(int kind, int bn, bool pair, int mh, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap *tmC,
                         const CUtensorMap *tmR, const IgemmParams &p, cudaStream_t stream, const CUtensorMap *tmI = nullptr, int epi_warps = 8);
size_t igemm_smem_bytes(int bn, bool pair = false, int mh = 1, int epi_warps = 8);

// Second step of a split-K contraction: out[m][n] = epilogue(sum_z partial[z][m][n]) with the same
// bias / activation / residual / rounding steps, in the same order, as the kernel's own epilogue.
// The planes are added z = 0, 1, ... in that fixed order, so results do not depend on scheduling.
struct SplitKReduceParams {
    const float *partial;       // [split_k][M][partial_ld] fp32, planes plane_stride elements apart
    long long plane_stride;
    int partial_ld;             // row pitch of a plane (N rounded up to the store box)
    int split_k, M, N;
    void *out;                  // [M][ldo] f32, bf16 or fp16
    long long ldo;
    int out_mode;               // OUT_F32 / OUT_BF16 / OUT_F16
    const float *bias;          // f32[N] or null
    int act;
    float act_p0, act_p1;
    const float *lut;
    const void *residual;       // [M][ldo], type of out, or null
    int res_relu, round_tf32;
    unsigned int *status;       // device status word (fp16 range)
};
cudaError_t launch_splitk_reduce(const SplitKReduceParams &p, cudaStream_t stream);
// Programmatic dependent launch for the contraction kernels of this library (on by default): each
// launch may begin its prologue while the previous kernel on the stream drains.
void set_pdl(int on);
void set_epilogue_mode(int bits);   // tuning switch for IgemmParams::epi_mode (default 15)
int get_epilogue_mode();
int get_pdl();
// Self test of the bounded-wait machinery (see one_cuda_selftest_wait_timeout).
cudaError_t launch_wait_probe(unsigned int *status, long long limit_clocks, cudaStream_t stream);

}  // namespace one
