// attn.cu -- fused multi-head self-attention for a token sequence that fits one tile
// (T <= 256 tokens, head width 32 or 64), tf32 tensor cores, fp32 in HBM.
//
// Replaces, for one transformer block, the operator chain the reference runs one by one:
//   Gather x3 / Reshape / Transpose (head split)      device/x86/Gather/gather.c:13-33, Transpose/transpose.c:27-75
//   Mul (q * scale)                                   device/x86/Mul/mul.c:100-115
//   MatMul (q k^T)                                    device/x86/MatMul/mat_mul.c:17-98
//   Softmax (last axis)                               device/x86/Softmax/softmax.c:31-76
//   MatMul (p v), Transpose, Reshape (head merge)
// None of the intermediates ([B,H,T,T] scores and probabilities, the per-head copies of q, k, v)
// touches HBM: the kernel reads the fused qkv tensor [B][T][3*D] once and writes ctx [B][T][D].
//
// One CTA per (image, head, 128-query-row tile), two CTAs resident per SM so that one CTA's loads
// and MMAs overlap the other's softmax.  Warp 4 issues TMA and tcgen05.mma; warps 0-3 own one TMEM
// lane quarter each (32 query rows) and do the softmax and the epilogue.
//   1. TMA: Q tile [128][hd] and K [T16][hd] straight out of the qkv tensor (the head split is the
//      tensor map's column coordinate; rows past T are zero-filled), 128-byte swizzle.
//   2. S = Q K^T: M = 128, N = T16, K = hd; both operands K-major; accumulator in TMEM columns [0, T16).
//   3. Q and K are dead: V [T8][hd] is loaded over them (32-byte-chunk swizzle: it is used as it
//      lies, [token][hd], as an MN-major B operand) while the softmax warps make their first pass
//      over S in TMEM (row maximum).
//   4. Second pass, 32 columns at a time: p = exp(scale * (s - max)), accumulated into the row sum
//      and written (un-normalised, columns >= T as 0) to a ring of 128 x 32 K-major A-operand blocks;
//      the MMA warp consumes each block as soon as it is full: O += P_c V_c, M = 128, N = hd, K = 32.
//      O lives in TMEM columns [0, hd), i.e. over the first S columns, which both sides make sure
//      have been read before the first of these MMAs is issued.
//   5. epilogue: O * (1 / row sum) -> swizzled 32 x 32 patches -> TMA store into ctx (rows >= T clipped).
// Every wait is bounded; a wait that runs out sets the status word and the CTA unwinds.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/one_cuda.h"
#include "ctx.h"
#include "sm100_prims.cuh"

namespace one {

struct AttnParams {
    int T, heads, hd, batch;
    int tp16, tp8;          // T rounded up to 16 (N of S) and to 8 (K of P V)
    int m_tiles;
    int q_off, k_off, v_off;   // column (float) offsets of the q / k / v blocks inside a qkv row
    int ring;               // P blocks in the ring (2 or 3)
    float scale;
    unsigned int *status;
};

namespace {

constexpr int ATTN_THREADS = 160;
constexpr uint32_t TMEM_COLS = 256;
constexpr int MAX_RING = 3;

// MN-major operand tile of 32-bit elements: rows of 128 bytes (32 floats along MN) stored with the
// 128-byte swizzle that moves 32-byte chunks (layout type 1); 32-float column blocks `lbo` bytes
// apart, groups of K rows `sbo` bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(ATTN_THREADS, 2)
attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
            const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttnParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int hdb = p.hd >> 5;                       // 32-float column blocks per head
    const uint32_t q_bytes = (uint32_t)hdb * 128u * 128u;
    const uint32_t k_blk = (uint32_t)p.tp16 * 128u, v_blk = (uint32_t)p.tp8 * 128u;
    const uint32_t k_bytes = (uint32_t)hdb * k_blk, v_bytes = (uint32_t)hdb * v_blk;
    // region shared in time: first Q | K, then V | ring of P blocks, then the output patches
    uint8_t *sQ = smem, *sK = smem + q_bytes, *sV = smem, *sRing = smem + v_bytes;
    const uint32_t qk = q_bytes + k_bytes, vr = v_bytes + (uint32_t)p.ring * 16384u;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (qk > vr ? qk : vr));
    // barriers: qk, v, s, o, full[MAX_RING], empty[MAX_RING]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4 + 2 * MAX_RING);
    int *abort_flag = reinterpret_cast<int *>(tmem_slot + 1);
    const uint32_t bar_qk = smem_u32(bars), bar_v = smem_u32(bars + 1), bar_s = smem_u32(bars + 2), bar_o = smem_u32(bars + 3);
    const uint32_t full0 = smem_u32(bars + 4), empty0 = smem_u32(bars + 4 + MAX_RING);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x;
    const int mt = tile % p.m_tiles, bh = tile / p.m_tiles;
    const int h = bh % p.heads, img = bh / p.heads;
    const int m0 = mt * 128;
    const int chunks = (p.tp16 + 31) >> 5;           // 32-column blocks of S (== blocks of P)
    const int ksteps = p.tp8 >> 3;                   // K = 8 steps of P V
    const int NR = p.ring;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_qk, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        for (int s = 0; s < MAX_RING; ++s) {
            mbar_init(full0 + 8 * s, 4);    // one arrival per softmax warp
            mbar_init(empty0 + 8 * s, 1);   // tcgen05.commit
        }
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    bool v_issued = false;
    if (warp == 4) {
        // ------------------------------------------------------------ TMA + MMA issue
        if (lane == 0) {
            mbar_arrive_expect_tx(bar_qk, q_bytes + k_bytes);
            for (int kb = 0; kb < hdb; ++kb)
                tma_load_3d(smem_u32(sQ + kb * 16384), &tmQ, bar_qk, p.q_off + h * p.hd + kb * 32, m0, img);
            for (int kb = 0; kb < hdb; ++kb)
                tma_load_3d(smem_u32(sK + kb * k_blk), &tmK, bar_qk, p.k_off + h * p.hd + kb * 32, 0, img);
        }
        __syncwarp();
        bool ok = mbar_wait(bar_qk, 0, abort_flag);
        if (ok) {
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t idesc = make_idesc<KIND_TF32>(128, p.tp16);
                // descriptor start addresses count 16-byte units: a 32-byte K step is 2
                const uint64_t dq = make_smem_desc(smem_u32(sQ), 128), dk = make_smem_desc(smem_u32(sK), 128);
                for (int kb = 0; kb < hdb; ++kb) {
                    const uint64_t a = dq + (uint64_t)(kb * (16384 >> 4)), b = dk + (uint64_t)(kb * (k_blk >> 4));
                    tc_mma<KIND_TF32>(tmem_base, a, b, idesc, (uint32_t)(kb != 0));
                    tc_mma<KIND_TF32>(tmem_base, a + 2, b + 2, idesc, 1u);
                    tc_mma<KIND_TF32>(tmem_base, a + 4, b + 4, idesc, 1u);
                    tc_mma<KIND_TF32>(tmem_base, a + 6, b + 6, idesc, 1u);
                }
                tc_commit(bar_s);
            }
            __syncwarp();
            // the S MMAs have finished reading Q and K: V may land on top of them
            ok = mbar_wait(bar_s, 0, abort_flag);
        }
        if (ok) {
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_v, v_bytes);
                for (int kb = 0; kb < hdb; ++kb)
                    tma_load_3d(smem_u32(sV + kb * v_blk), &tmV, bar_v, p.v_off + h * p.hd + kb * 32, 0, img);
            }
            v_issued = true;
            __syncwarp();
            ok = mbar_wait(bar_v, 0, abort_flag);
        }
        if (ok) {
            const uint32_t idesc = make_idesc<KIND_TF32>(128, p.hd) | (1u << 16);   // B is MN-major
            const uint64_t desc_p0 = make_smem_desc(smem_u32(sRing), 128), desc_v0 = make_smem_desc_mn(smem_u32(sV), v_blk, 512u);
            // O overwrites the first hd columns of S: wait until the block holding the last of them is full
            const int guard = (hdb - 1 < chunks - 1) ? hdb - 1 : chunks - 1;
            for (int c = 0; c < chunks && ok; ++c) {
                const int s = c % NR;
                ok = mbar_wait(full0 + 8 * s, (uint32_t)((c / NR) & 1), abort_flag);
                if (ok && c == 0 && guard > 0) ok = mbar_wait(full0 + 8 * (guard % NR), 0, abort_flag);
                if (!ok) break;
                // tcgen05 ordering is needed once: the first O MMA overwrites S columns the softmax warps
                // have read with tcgen05.ld.  Later blocks only wait for P in shared memory (ordered by the
                // barrier), and a fence per block would stall the issue until the previous MMAs drain.
                if (c == 0) tc_fence_after_sync();
                if (lane == 0) {
                    const int nk = ksteps - 4 * c < 4 ? ksteps - 4 * c : 4;
                    const uint64_t dp = desc_p0 + (uint64_t)(s * (16384 >> 4)), dv = desc_v0 + (uint64_t)((1024u >> 4) * (4 * c));
                    for (int k = 0; k < nk; ++k)
                        tc_mma<KIND_TF32>(tmem_base, dp + 2 * k, dv + (uint64_t)((1024u >> 4) * k), idesc, (uint32_t)((c | k) != 0));
                    tc_commit(empty0 + 8 * s);
                    if (c == chunks - 1) tc_commit(bar_o);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) atomicOr(p.status, ST_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------ softmax + epilogue (warps 0-3)
        const int row = 32 * warp + lane;              // accumulator row (TMEM lane) of this thread
        const uint32_t t_row = tmem_base + ((uint32_t)(32 * warp) << 16);
        bool ok = mbar_wait(bar_s, 0, abort_flag);
        float sum = 0.f;
        if (ok) {
            tc_fence_after_sync();
            // Two passes over the accumulator row in TMEM, 32 columns at a time.  The load of the next
            // block is in flight while the current one is processed (two register buffers), and the
            // running maximum / sum are kept in four independent chains.
            uint32_t va[32], vb[32];
            float mx4[4] = {-32768.0f, -32768.0f, -32768.0f, -32768.0f};   // softmax.c:53
            auto pass1 = [&](const uint32_t (&v)[32], int c) {
                const int lim = p.T - 32 * c;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < lim) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(v[j]));
            };
            tmem_ld_32x32(t_row, va);
            for (int c = 0; c < chunks; c += 2) {
                tmem_ld_wait();
                if (c + 1 < chunks) tmem_ld_32x32(t_row + 32 * (c + 1), vb);
                pass1(va, c);
                if (c + 1 < chunks) {
                    tmem_ld_wait();
                    if (c + 2 < chunks) tmem_ld_32x32(t_row + 32 * (c + 2), va);
                    pass1(vb, c + 1);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // exp(scale * (s - max)) as 2^(s * a - b)
            const float a2 = p.scale * 1.4426950408889634f, b2 = mx * a2;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            auto pass2 = [&](const uint32_t (&v)[32], int c) -> bool {
                const int lim = p.T - 32 * c;
                float e[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float t = ex2_approx(fmaf(__uint_as_float(v[j]), a2, -b2));
                    e[j] = (j < lim) ? t : 0.f;
                    sum4[j & 3] += e[j];
                }
                const int s = c % NR;
                // the ring slot is free once the MMAs that read its previous block have completed
                if (c >= NR && !mbar_wait(empty0 + 8 * s, (uint32_t)((c / NR - 1) & 1), abort_flag)) return false;
                uint8_t *prow = sRing + s * 16384 + row * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float4 *>(prow + ((j ^ (row & 7)) << 4)) = make_float4(e[4 * j], e[4 * j + 1], e[4 * j + 2], e[4 * j + 3]);
                tc_fence_before_sync();     // this block of S has been read (the first blocks are overwritten by O)
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
                return true;
            };
            tmem_ld_32x32(t_row, va);
            for (int c = 0; c < chunks && ok; c += 2) {
                tmem_ld_wait();
                if (c + 1 < chunks) tmem_ld_32x32(t_row + 32 * (c + 1), vb);
                ok = pass2(va, c);
                if (ok && c + 1 < chunks) {
                    tmem_ld_wait();
                    if (c + 2 < chunks) tmem_ld_32x32(t_row + 32 * (c + 2), va);
                    ok = pass2(vb, c + 1);
                }
            }
            tmem_ld_wait();
            sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (ok) ok = mbar_wait(bar_o, 0, abort_flag);
        }
        if (ok) {
            tc_fence_after_sync();
            const float inv = 1.0f / sum;
            uint8_t *patch = smem + warp * (hdb * 4096);   // V and the ring are dead once O is complete
            uint32_t v[32];
            for (int cb = 0; cb < hdb; ++cb) {
                tmem_ld_32x32(t_row + 32 * cb, v);
                tmem_ld_wait();
                uint8_t *prow = patch + cb * 4096 + lane * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float4 *>(prow + ((j ^ (lane & 7)) << 4)) =
                        make_float4(__uint_as_float(v[4 * j]) * inv, __uint_as_float(v[4 * j + 1]) * inv,
                                    __uint_as_float(v[4 * j + 2]) * inv, __uint_as_float(v[4 * j + 3]) * inv);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && m0 + 32 * warp < p.T) {
                for (int cb = 0; cb < hdb; ++cb)
                    tma_store_3d(&tmO, smem_u32(patch + cb * 4096), h * p.hd + cb * 32, m0 + 32 * warp, img);
                bulk_commit();
                bulk_wait_read0();
            }
        } else if (lane == 0) {
            atomicOr(p.status, ST_TIMEOUT_EPILOGUE);
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        if (*abort_flag) {   // let a load in flight land before the shared memory is given back
            int dummy = 0;
            if (!(mbar_wait(bar_qk, 0, &dummy) && (!v_issued || mbar_wait(bar_v, 0, &dummy))) && lane == 0)
                atomicOr(p.status, ST_TIMEOUT_DRAIN);
        }
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace
}  // namespace one

using namespace one;

extern "C" int one_cuda_attention(one_ctx *ctx, const float *qkv, float *out, int batch, int T, int heads, int hd,
                                  int row_floats, int q_off, int k_off, int v_off, int out_row_floats, float scale,
                                  void *stream)
{
    if (!ctx || !qkv || !out) return fail(ONE_ERR_BAD_ARG, "attention: null argument");
    if (batch <= 0 || T <= 0 || heads <= 0) return fail(ONE_ERR_BAD_SHAPE, "attention: non-positive dimension");
    if (T > 256) return fail(ONE_ERR_UNSUPPORTED, "attention: at most 256 tokens fit the fused kernel (got %d)", T);
    if (hd != 32 && hd != 64) return fail(ONE_ERR_UNSUPPORTED, "attention: head width must be 32 or 64 (got %d)", hd);
    if ((q_off | k_off | v_off) % 32 || q_off < 0 || k_off < 0 || v_off < 0 || row_floats % 4 || out_row_floats % 4 ||
        q_off + heads * hd > row_floats || k_off + heads * hd > row_floats || v_off + heads * hd > row_floats ||
        heads * hd > out_row_floats)
        return fail(ONE_ERR_BAD_SHAPE, "attention: q / k / v blocks must start on a multiple of 32 floats inside a row");
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(stream) : ctx->stream;
    AttnParams p;
    p.T = T; p.heads = heads; p.hd = hd; p.batch = batch;
    p.tp16 = (T + 15) & ~15; p.tp8 = (T + 7) & ~7;
    p.m_tiles = (T + 127) / 128;
    p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
    p.scale = scale;
    p.status = ctx->status_dev;
    const int hdb = hd / 32;
    const size_t qk = (size_t)hdb * (128 + p.tp16) * 128, vb = (size_t)hdb * p.tp8 * 128;
    // three ring slots when two CTAs still fit an SM with them, else two
    p.ring = (1024 + (vb + 3 * 16384 > qk ? vb + 3 * 16384 : qk) + 128) * 2 <= 227 * 1024 ? 3 : 2;
    const size_t vr = vb + (size_t)p.ring * 16384;
    const size_t smem = 1024 + (qk > vr ? qk : vr) + 128;
    if (smem > 227 * 1024) return fail(ONE_ERR_UNSUPPORTED, "attention: %zu bytes of shared memory needed", smem);
    CUtensorMap tmQ, tmK, tmV, tmO;
    const uint64_t pitch = (uint64_t)row_floats * 4, bpitch = pitch * T;
    int rc = make_tmap_tiled(&tmQ, TM_F32, qkv, row_floats, T, batch, pitch, bpitch, 32, 128, 128);
    if (rc == ONE_OK) rc = make_tmap_tiled(&tmK, TM_F32, qkv, row_floats, T, batch, pitch, bpitch, 32, p.tp16, 128);
    if (rc == ONE_OK) rc = make_tmap_tiled(&tmV, TM_F32, qkv, row_floats, T, batch, pitch, bpitch, 32, p.tp8, TM_SWIZZLE_128B_ATOM_32B);
    if (rc == ONE_OK)
        rc = make_tmap_tiled(&tmO, TM_F32, out, out_row_floats, T, batch, (uint64_t)out_row_floats * 4,
                             (uint64_t)out_row_floats * 4 * T, 32, 32, 128);
    if (rc != ONE_OK) return rc;
    static bool attr_set[64] = {};
    int dev = ctx->device;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return cuda_fail(e, "attention: shared memory attribute");
        attr_set[dev] = true;
    }
    const long long tiles = (long long)batch * heads * p.m_tiles;
    if (tiles > 0x7fffffffLL) return fail(ONE_ERR_BAD_SHAPE, "attention: too many tiles");
    attn_kernel<<<(unsigned)tiles, ATTN_THREADS, smem, st>>>(tmQ, tmK, tmV, tmO, p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ONE_OK : cuda_fail(e, "attention launch");
}
