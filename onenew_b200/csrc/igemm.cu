// igemm.cu -- the sm_100a implicit-GEMM kernel behind Conv, Gemm and MatMul.
//
// Persistent kernel: one CTA per SM walks the 128 x BN output tiles of D = A * B^T with a static
// stride.  Roles (320 threads):
//   warp 0, one lane : TMA producer.  Per K block it issues one load of the A tile
//                      (128 rows x slab_bytes; im2col mode for convolutions) and one of the B tile
//                      (BN rows x slab_bytes) into a STAGES-deep shared-memory ring that runs
//                      across tile boundaries, so the next tile's operands stream in while the
//                      current tile is still being multiplied and written out.
//   warp 1, one lane : issues tcgen05.mma (one per 32 bytes of K) into one of TWO accumulator
//                      buffers in TMEM; tcgen05.commit frees the stage and publishes the tile.
//   warps 2..9       : epilogue.  tcgen05.ld the finished accumulator (each warp its lane
//                      quarter), apply bias / int8 de-quantisation / activation, transpose
//                      through a swizzled shared-memory patch so that every global access
//                      (residual read, output write) covers whole 128-byte rows, then hand the
//                      TMEM buffer back.  The epilogue of tile i overlaps the main loop of i+1.
// Replaces, in the reference, the pad + im2col + SGEMM + bias pass + activation pass chain of
// device/x86/Conv/conv.c:300-415 (and :68-166, :901-1059, :1216-1304), the SGEMM of
// device/x86_utils/opt_gemm.h:17-174, device/x86/Gemm/gemm.c:9-79 and
// device/x86/MatMul/mat_mul.c:10-101.
//
// Algorithmic bytes per tile: A 128*K*es + B BN*K*es read, 128*BN*out_es written; the
// im2col matrix is never materialised.
#include "igemm.cuh"
#include "sm100_prims.cuh"
#include "act.cuh"
#include "ctx.h"

#include <cuda_bf16.h>
#include "h16.cuh"
#include <string.h>

#include <atomic>
#include <utility>

namespace one {

static constexpr int TILE_M = 128;
static constexpr int A_STAGE_BYTES = TILE_M * 128;   // room for the widest (128 B) slab
// Epilogue warps per CTA: 8 (two groups of four, one warp per TMEM lane quarter) or, for the narrow tiles of
// store-bound layers, 12 (three groups): with 14 warps every scheduler holds at most four, which still leaves a
// thread 128 registers.  Twelve warps need 96 KB of patches, so those instantiations run shallower operand rings.
static constexpr int NUM_EPI_WARPS = 8;
__host__ __device__ constexpr int num_threads_for(int nw) { return 64 + nw * 32; }   // producer warp + MMA warp + epilogue warps

static constexpr int EPI_PATCH_BYTES = 32 * 128;     // per epilogue warp: 32 rows x 32 fp32

// accumulator buffers in the 512 TMEM columns (a buffer holds mh * bn columns)
__host__ __device__ constexpr int acc_stages_for(int bn, int mh = 1) { return bn * mh >= 192 ? 2 : 4; }
// Ring depth at 128-byte slabs.  A CTA of a pair loads only half of B's rows per K block, so its stages
// are smaller and more of them fit.
// `mh` = 2: a CTA's tile is two 128-row halves that share each B stage (twice the A bytes per stage).
__host__ __device__ constexpr int stages_for(int bn, bool pair = false, int mh = 1, int nw = NUM_EPI_WARPS)
{
    if (nw == 12) return bn == 64 ? 4 : 3;   // plain tiles of width 64 / 128 only
    return mh == 2 ? (bn == 128 ? 3 : 4) : (pair ? (bn == 256 ? 5 : (bn == 192 ? 5 : 6)) : (bn == 256 ? 3 : (bn >= 128 ? 4 : 6)));
}
__host__ __device__ constexpr int b_rows_for(int bn, bool pair) { return pair ? bn / 2 : bn; }
// A 64 x 64 16-bit identity tile (residual added by the tensor core), where the ring leaves room for it
// (plain tiles other than the 192-wide one, whose ring already fills the shared memory)
__host__ __device__ constexpr int ident_bytes_for(int bn, bool pair, int mh) { return (!pair && mh == 1 && bn != 192) ? 64 * 128 : 0; }
// TMEM is allocated in powers of two columns
__host__ __device__ constexpr uint32_t tmem_cols_for(int bn, int mh = 1)
{
    return acc_stages_for(bn, mh) * bn * mh > 256 ? 512u : (acc_stages_for(bn, mh) * bn * mh > 128 ? 256u : 128u);
}

__host__ __device__ constexpr size_t smem_layout_bytes(int bn, bool pair = false, int mh = 1, int nw = NUM_EPI_WARPS)
{
    return (size_t)stages_for(bn, pair, mh, nw) * (mh * A_STAGE_BYTES + b_rows_for(bn, pair) * 128) + 2 * nw * EPI_PATCH_BYTES /* output + residual patches */ +
           ident_bytes_for(bn, pair, mh) + 1024 /* barriers etc. */;
}

size_t igemm_smem_bytes(int bn, bool pair, int mh, int nw) { return smem_layout_bytes(bn, pair, mh, nw) + 1024; }

// Round to the nearest tf32 (10 mantissa bits), ties away from zero, like cvt.rna.tf32.f32 -- but with
// two integer instructions: the conversion instruction runs on the 16-lane special-function pipe and,
// at one per output element, was a measurable share of the epilogue (that pipe 42 % busy on a 3x3
// 64-channel layer).  Adding half an ulp to the magnitude bits and clearing the low 13 carries into the
// exponent correctly.  Infinities and NaNs (exponent all ones) pass through untouched: the add would
// carry a NaN's mantissa into the sign bit and turn it into -0.0, and cvt.rna keeps NaNs too.
__device__ __forceinline__ float round_to_tf32(float v)
{
    const uint32_t u = __float_as_uint(v);
    return ((u & 0x7f800000u) == 0x7f800000u) ? v : __uint_as_float((u + 0x1000u) & 0xffffe000u);
}

// Quantise for an int8 consumer: x * (1/scale), clamp to [-128, 127], roundf
// (device/x86/Conv/conv.c:961-973).
__device__ __forceinline__ int quant_s8(float v, float inv_scale)
{
    float t = __fmul_rn(v, inv_scale);
    t = (t < -128.f) ? -128.f : (t > 127.f) ? 127.f : t;
    return (int)roundf(t);
}

// A 32-row x 64-column patch of 16-bit values in shared memory, as the TMA store / load with a 128-byte
// swizzle lays it out: 128-byte rows, 16-byte piece j of row r at j ^ (r & 7); lane = row; half h of the
// columns is pieces 4h .. 4h + 3.
template <bool F16>
__device__ __forceinline__ void add_patch16(float (&v)[32], const uint4 *patch, int lane, int h)
{
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 q = patch[lane * 8 + ((4 * h + j) ^ (lane & 7))];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 h = h16_unpack2(w[e], F16);
            v[8 * j + 2 * e] = __fadd_rn(v[8 * j + 2 * e], h.x);
            v[8 * j + 2 * e + 1] = __fadd_rn(v[8 * j + 2 * e + 1], h.y);
        }
    }
}
template <bool F16>
__device__ __forceinline__ void store_patch16(const float (&v)[32], uint4 *patch, int lane, int h)
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
        patch[lane * 8 + ((4 * h + j) ^ (lane & 7))] =
            make_uint4(h16_pack2(v[8 * j], v[8 * j + 1], F16), h16_pack2(v[8 * j + 2], v[8 * j + 3], F16),
                       h16_pack2(v[8 * j + 4], v[8 * j + 5], F16), h16_pack2(v[8 * j + 6], v[8 * j + 7], F16));
}

// The 32 x 32 form (a 16-bit output of the tf32 instantiation): 64-byte rows, 64-byte swizzle, piece j of row r
// at j ^ ((r >> 1) & 3).
template <bool F16>
__device__ __forceinline__ void add_patch16_narrow(float (&v)[32], const uint4 *patch, int lane)
{
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 q = patch[lane * 4 + (j ^ ((lane >> 1) & 3))];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 h = h16_unpack2(w[e], F16);
            v[8 * j + 2 * e] = __fadd_rn(v[8 * j + 2 * e], h.x);
            v[8 * j + 2 * e + 1] = __fadd_rn(v[8 * j + 2 * e + 1], h.y);
        }
    }
}
template <bool F16>
__device__ __forceinline__ void store_patch16_narrow(const float (&v)[32], uint4 *patch, int lane)
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
        patch[lane * 4 + (j ^ ((lane >> 1) & 3))] =
            make_uint4(h16_pack2(v[8 * j], v[8 * j + 1], F16), h16_pack2(v[8 * j + 2], v[8 * j + 3], F16),
                       h16_pack2(v[8 * j + 4], v[8 * j + 5], F16), h16_pack2(v[8 * j + 6], v[8 * j + 7], F16));
}

// PAIR: the kernel runs as clusters of two CTAs that share 256-row tiles (tcgen05 cta_group::2): CTA r of a
// pair loads rows [128 r, 128 r + 128) of the tile's A and rows [BN / 2 * r, ...) of its B, the even CTA
// issues every MMA and signals both CTAs' barriers, each CTA's epilogue drains its own 128 accumulator rows.
// MH = 2 (single CTAs, BN 64 / 128): a tile is two 128-row halves.  Each K block brings both halves of A
// and ONE tile of B, and the issuer multiplies both halves by it: per 128 rows of output a third (BN 128) or
// a sixth (BN 64) less operand traffic through the SM's L2 port, and half as many barrier hand-overs -- the
// two things that bound the narrow tiles.
template <int KIND, int BN, bool PAIR, int MH, int NEW>
__global__ void __launch_bounds__(num_threads_for(NEW), 1)
igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
             const __grid_constant__ CUtensorMap tmI, const IgemmParams p)
{
    static_assert(MH == 1 || (MH == 2 && !PAIR && BN <= 128), "two halves per CTA: single CTAs, BN 64 or 128");
    static_assert(NEW == 8 || (NEW == 12 && !PAIR && MH == 1 && BN <= 128), "twelve epilogue warps: plain tiles of width 64 / 128");
    constexpr int STAGES = stages_for(BN, PAIR, MH, NEW);   // ring depth at 128-byte slabs
    constexpr int NG = NEW / 4;                        // epilogue groups
    constexpr int NUM_THREADS = num_threads_for(NEW);
    constexpr int BROWS = b_rows_for(BN, PAIR);        // rows of B this CTA loads per K block
    constexpr int TILE_ROWS = PAIR ? 2 * TILE_M : MH * TILE_M;   // rows of D per tile (of the pair / of both halves)
    constexpr int ACC_COLS = MH * BN;                  // TMEM columns of one accumulator buffer
    constexpr int MAX_STAGES = 4 * STAGES;
    // Narrower slabs (few-channel layers) get proportionally more, smaller stages out of the same
    // space: the operand stream is bound by the bytes in flight per SM, not by the stage count.
    // Slabs are handed over two at a time where the ring depth is even: mbarrier instructions
    // are expensive for the thread that issues them (measured: a wait on a completed phase ~165 cycles, an
    // arrive ~93, and the MMA / TMA issue does not overlap them), so a stage carries 256 bytes of K per
    // wait / arrive / commit instead of 128.  Same bytes in flight, half the barrier operations.
    // Only the narrowest tile does this (plain or two-half, any slab width): there the barrier operations are
    // the largest share of a K block (measured -13 % time on 3x3 64->64, -10 % on the 7x7 stem's 64-byte slabs),
    // while wider tiles are bound by the operand stream and lost a few percent to the shallower ring.
    constexpr int KPS_MAX = (!PAIR && BN == 64 && (STAGES & 1) == 0) ? 2 : 1;
    const int kps = (KPS_MAX == 2 && p.num_kb > 1) ? 2 : 1;   // K blocks per stage
    const int stages = STAGES * (128 / p.slab_bytes) / kps;
    const uint32_t a_half = (uint32_t)TILE_M * (uint32_t)p.slab_bytes;   // one 128-row half of A
    const uint32_t a_slab = a_half * (uint32_t)MH, b_slab = (uint32_t)BROWS * (uint32_t)p.slab_bytes;
    const uint32_t a_stage = a_slab * (uint32_t)kps, b_stage = b_slab * (uint32_t)kps;
    constexpr int ACC = acc_stages_for(BN, MH);
    constexpr int B_STAGE_BYTES = BROWS * 128;
    constexpr int A_STAGE = MH * A_STAGE_BYTES;

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles, done as an offset into the __shared__ array so the
    // compiler keeps emitting shared-space (not generic) loads and stores for everything below
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *sA = smem;
    uint8_t *sB = sA + STAGES * A_STAGE;
    uint8_t *sPatch = sB + STAGES * B_STAGE_BYTES;
    uint8_t *sRes = sPatch + NEW * EPI_PATCH_BYTES;
    uint8_t *sIdent = sRes + NEW * EPI_PATCH_BYTES;   // 64 x 64 identity tile (RES_MMA launches)
    uint64_t *bars = reinterpret_cast<uint64_t *>(sIdent + ident_bytes_for(BN, PAIR, MH));
    // barriers: full[MAX_STAGES], empty[MAX_STAGES], acc_full[ACC], acc_empty[ACC], res[NUM_EPI_WARPS][RES_SLOTS], ident
    constexpr int RES_SLOTS = 3;   // residual patches in flight per epilogue warp, at most
    static_assert((2 * MAX_STAGES + 2 * ACC + RES_SLOTS * NEW + 1) * 8 + 8 <= 1024, "barrier space");
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * MAX_STAGES + 2 * ACC + RES_SLOTS * NEW + 1);
    // Residual added by the tensor core (16-bit kinds, plain tiles): after a tile's own K blocks the producer
    // brings the matching 128 x BN piece of the residual tensor as BN / 64 further A stages and the issuer
    // multiplies each by a 64 x 64 identity held in shared memory, accumulating into the 64 columns it belongs
    // to.  The residual then travels as four 16 KB operand loads per 128 x 256 tile instead of sixteen 4 KB
    // patches, and the epilogue has no residual to wait for, unpack and add.  Exact: x * 1.0 in fp32.
    constexpr bool RES_MMA_OK = KIND == KIND_BF16 && ident_bytes_for(BN, PAIR, MH) > 0;
    const bool res_mma = RES_MMA_OK && p.res_mma;
    constexpr uint32_t RES_PIECE = (uint32_t)TILE_M * 128u;   // 128 rows x 64 16-bit columns
    int *abort_flag = reinterpret_cast<int *>(tmem_slot + 1);

    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + MAX_STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * MAX_STAGES);
    const uint32_t acc_empty0 = smem_u32(bars + 2 * MAX_STAGES + ACC);
    const uint32_t res_bar0 = smem_u32(bars + 2 * MAX_STAGES + 2 * ACC);
    const uint32_t ident_bar = smem_u32(bars + 2 * MAX_STAGES + 2 * ACC + RES_SLOTS * NEW);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // position in the launch: a single CTA, or CTA `rank` of pair `cid`
    uint32_t rank = 0;
    if constexpr (PAIR) rank = cluster_ctarank();
    const int cid = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int ncta = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int row_off = (int)rank * TILE_M;          // this CTA's first row inside a tile
    const int n_tiles = (p.N + BN - 1) / BN;
    const int m_tiles = (p.M + TILE_ROWS - 1) / TILE_ROWS;
    const long long tiles_per_batch = (long long)n_tiles * m_tiles;
    // third tile coordinate: the batch of a batched MatMul, or the K range of a split-K launch
    const int zdim = p.batched ? p.batch : (p.split_k > 1 ? p.split_k : 1);
    const long long total_tiles = tiles_per_batch * zdim;
    const bool z_store = p.batched || p.split_k > 1;   // the store map has a third dimension

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < ACC; ++a) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, PAIR ? 8 : 4);   // one arrival per warp of the epilogue group that drained it (in both CTAs of a pair)
        }
        for (int w = 0; w < RES_SLOTS * NEW; ++w) mbar_init(res_bar0 + 8 * w, 1);
        mbar_init(ident_bar, 1);
        fence_mbar_init();
        if (res_mma) tma_prefetch_desc(&tmI);
    }
    if (warp == 1) {
        if constexpr (PAIR) {   // the same warp of both CTAs, same destination offset
            tmem_alloc_pair(smem_u32(tmem_slot), tmem_cols_for(BN, MH));
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), tmem_cols_for(BN, MH));
            tmem_relinquish();
        }
    }
    // Activation table (8192 floats) staged in the residual patches' space: the host sets lut_smem only
    // when no residual is added, so the two uses never meet.
    const float *slut = reinterpret_cast<const float *>(sRes);
    if (p.lut_smem) {
        static_assert(NEW * EPI_PATCH_BYTES >= 8192 * 4, "the table must fit the residual patches");
        const float4 *g4 = reinterpret_cast<const float4 *>(p.lut);
        for (int i = threadIdx.x; i < 2048; i += NUM_THREADS) reinterpret_cast<float4 *>(sRes)[i] = __ldg(g4 + i);
    }
    tc_fence_before_sync();
    // a pair: the peer's barriers and tensor memory must exist before anything of this CTA signals or writes them
    if constexpr (PAIR) cluster_sync();
    else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    // Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch, the
    // constant table) touched nothing an earlier kernel writes, so it may run while that kernel drains.
    // From here on activations are read and written: wait until the previous kernel on the stream has
    // completed and its writes are visible.  Every thread executes the wait, so each role's global
    // accesses are ordered after it.  The next kernel may start its own prologue right away; it cannot
    // touch data before its own wait, which in turn covers this whole grid.
    if (p.pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }

    long long issued = 0;   // producer: ring stages whose loads were issued (ring position)

    // The producer and MMA warps run their loops with all 32 lanes converged (every lane waits on the
    // barriers, lane 0 alone issues): a lone lane spinning while its 31 siblings sit in the final
    // __syncthreads would leave the warp permanently diverged.
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // bytes one K block brings in: this CTA's, or (counted on the even CTA's barrier) both CTAs' of a pair
        const uint32_t tx_bytes = (uint32_t)(MH * TILE_M + BROWS) * (uint32_t)p.slab_bytes * (PAIR ? 2u : 1u);
        const int hw = p.OH * p.OW;
        bool ok = true;
        int ps = 0;            // ring slot and phase of the next K block (running, no division in the loop)
        uint32_t pph = 0;
        if (res_mma && lane == 0) {   // the identity tile, once
            mbar_arrive_expect_tx(ident_bar, 64 * 128);
            tma_load_2d(smem_u32(sIdent), &tmI, ident_bar, 0, 0);
        }
        for (long long tile = cid; tile < total_tiles && ok; tile += ncta) {
            const int bz = (int)(tile / tiles_per_batch);
            const int tin = (int)(tile - bz * tiles_per_batch);
            const int m0 = (tin / n_tiles) * TILE_ROWS + row_off;
            const int n0 = (tin % n_tiles) * BN + (int)rank * BROWS;   // a CTA of a pair loads its half of B's rows
            // base pixel of each 128-row half (im2col mode)
            int cw[MH], ch[MH], cn[MH];
#pragma unroll
            for (int h = 0; h < MH; ++h) {
                cw[h] = ch[h] = cn[h] = 0;
                if (p.a_im2col) {
                    const int mh0 = m0 + h * TILE_M;
                    cn[h] = mh0 / hw;
                    const int rem = mh0 - cn[h] * hw;
                    const int oh = rem / p.OW;
                    const int ow = rem - oh * p.OW;
                    cw[h] = ow * p.stride_w - p.pad_l;
                    ch[h] = oh * p.stride_h - p.pad_t;
                }
            }
            int kb_begin = 0, kb_end = p.num_kb;
            if (p.split_k > 1) {
                kb_begin = bz * p.kb_per_split;
                kb_end = kb_begin + p.kb_per_split < p.num_kb ? kb_begin + p.kb_per_split : p.num_kb;
            }
            // filter tap and channel slab of the first K block of this range
            int cs = 0, kw = 0, kh = 0;
            if (p.a_im2col && kb_begin) {
                cs = kb_begin % p.c_slabs;
                kw = (kb_begin / p.c_slabs) % p.KW;
                kh = (kb_begin / p.c_slabs) / p.KW;
            }
            for (int kb = kb_begin; kb < kb_end; kb += kps, ++issued) {
                const int s = ps;
                const uint32_t ph = pph;
                if (++ps == stages) { ps = 0; pph ^= 1; }
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) {
                    if (lane == 0) atomicOr(p.status, ST_TIMEOUT_PRODUCER);
                    ok = false;
                    break;
                }
                const int nk = kb_end - kb < kps ? kb_end - kb : kps;   // K blocks in this stage (the last may hold one)
                if (lane == 0 && rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, tx_bytes * (uint32_t)nk);
#pragma unroll
                for (int j = 0; j < KPS_MAX; ++j) {
                    if (j >= nk) break;
                    if (lane == 0) {
                        const uint32_t dstA = smem_u32(sA) + s * a_stage + j * a_slab;
                        const uint32_t dstB = smem_u32(sB) + s * b_stage + j * b_slab;
                        const int k0 = (kb + j) * p.slab_elems;
                        if constexpr (PAIR) {
                            if (p.a_im2col)
                                tma_load_im2col_4d_pair(dstA, &tmA, full0 + 8 * s, cs * p.slab_elems, cw[0], ch[0], cn[0], (uint16_t)(kw * p.dil_w), (uint16_t)kh);
                            else
                                tma_load_2d_pair(dstA, &tmA, full0 + 8 * s, k0, m0);
                            tma_load_2d_pair(dstB, &tmB, full0 + 8 * s, k0, n0);
                        } else {
#pragma unroll
                            for (int h = 0; h < MH; ++h) {   // one load per 128-row half
                                if (p.a_im2col)
                                    tma_load_im2col_4d(dstA + h * a_half, &tmA, full0 + 8 * s, cs * p.slab_elems, cw[h], ch[h], cn[h], (uint16_t)(kw * p.dil_w), (uint16_t)kh);
                                else if (p.batched)
                                    tma_load_3d(dstA + h * a_half, &tmA, full0 + 8 * s, k0, m0 + h * TILE_M, bz);
                                else
                                    tma_load_2d(dstA + h * a_half, &tmA, full0 + 8 * s, k0, m0 + h * TILE_M);
                            }
                        }
                        if constexpr (!PAIR) {
                            if (p.batched)
                                tma_load_3d(dstB, &tmB, full0 + 8 * s, k0, n0, bz);
                            else
                                tma_load_2d(dstB, &tmB, full0 + 8 * s, k0, n0);
                        }
                    }
                    if (p.a_im2col && ++cs == p.c_slabs) {
                        cs = 0;
                        if (++kw == p.KW) {
                            kw = 0;
                            ++kh;
                        }
                    }
                }
                __syncwarp();
            }
            // the residual's 128 x BN piece, 64 columns (16 KB) at a time (see res_mma above): a ring stage takes
            // one piece in its A slot and as many as fit in its B slot, so a 128 x 256 tile needs two stages
            if (res_mma) {
                const int nres = (p.N - n0 < BN ? p.N - n0 : BN) / 64;
                const int cap = 1 + (int)(b_stage / RES_PIECE);
                for (int j = 0; j < nres && ok; ++issued) {
                    const int s = ps;
                    const uint32_t ph = pph;
                    if (++ps == stages) { ps = 0; pph ^= 1; }
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) {
                        if (lane == 0) atomicOr(p.status, ST_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const int take = nres - j < cap ? nres - j : cap;
                    if (lane == 0) {
                        mbar_arrive_expect_tx(full0 + 8 * s, (uint32_t)take * RES_PIECE);
                        for (int t = 0; t < take; ++t)
                            tma_load_2d(t == 0 ? smem_u32(sA) + s * a_stage : smem_u32(sB) + s * b_stage + (uint32_t)(t - 1) * RES_PIECE, &tmR,
                                        full0 + 8 * s, n0 + (j + t) * 64, m0);
                    }
                    j += take;
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // the 16-bit kind multiplies bf16 (format 1) or fp16 (format 0) operands
        const uint32_t idesc = make_idesc<KIND>(PAIR ? 2 * TILE_M : TILE_M, BN) & ((KIND == KIND_BF16 && p.ab_f16) ? ~((7u << 7) | (7u << 10)) : ~0u);
        const int mma_per_kb = p.slab_bytes >> 5;
        // One MMA / one barrier signal, for a single CTA or for a pair.  The pair's barriers exist in both
        // CTAs (each CTA's producer and epilogue wait on their own copy), so the even CTA signals twice:
        // its own copy and, through the cluster window, the peer's.
        auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t acc) {
            if constexpr (PAIR) tc_mma_pair<KIND>(d, da, db, idesc, acc);
            else tc_mma<KIND>(d, da, db, idesc, acc);
        };
        auto commit = [&](uint32_t bar) {
            if constexpr (PAIR) {
                tc_commit_pair(mapa_shared(bar, 0));
                tc_commit_pair(mapa_shared(bar, 1));
            } else {
                tc_commit(bar);
            }
        };
        const uint64_t desc_a0 = make_smem_desc(smem_u32(sA), p.slab_bytes), desc_b0 = make_smem_desc(smem_u32(sB), p.slab_bytes);
        int ms = 0;            // ring slot and phase of the next K block
        uint32_t mph = 0;
        bool ok = true;
        bool ident_ready = false;   // the identity tile has landed (RES_MMA launches)
        int lt = 0;   // tiles this CTA has started
        // (the odd CTA of a pair issues nothing: its tensor core is driven by the even CTA's instructions)
        for (long long tile = cid; tile < total_tiles && ok && rank == 0; tile += ncta, ++lt) {
            const int a = lt % ACC;
            // wait until the epilogue has drained this accumulator buffer (ACC tiles ago)
            if (!mbar_wait(acc_empty0 + 8 * a, (uint32_t)(((lt / ACC) & 1) ^ 1), abort_flag)) {
                if (lane == 0) atomicOr(p.status, ST_TIMEOUT_MMA);
                break;
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * ACC_COLS);
            int kb_begin = 0, kb_end = p.num_kb;
            if (p.split_k > 1) {
                const int bz = (int)(tile / tiles_per_batch);
                kb_begin = bz * p.kb_per_split;
                kb_end = kb_begin + p.kb_per_split < p.num_kb ? kb_begin + p.kb_per_split : p.num_kb;
            }
            for (int kb = kb_begin; kb < kb_end; kb += kps) {
                const int s = ms;
                const uint32_t ph = mph;
                if (++ms == stages) { ms = 0; mph ^= 1; }
                if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) {
                    if (lane == 0) atomicOr(p.status, ST_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                // No tcgen05 fence here: the full barrier orders the TMA writes before the MMAs that read
                // them, and a fence in this loop would hold the issue back until the previous K block's MMAs
                // had drained (the accumulator hand-over above is the only tcgen05-to-tcgen05 ordering).
                if (lane == 0) {
                    // Descriptors are not rebuilt per instruction: the start-address field counts 16-byte
                    // units, so a stage is `s * stage_bytes / 16` and a K step of 32 bytes is 2 further on.
                    // (Built from scratch each time, the issue loop -- not the tensor pipe -- set the pace:
                    // 155 cycles per MMA against 128 for a full-rate 128 x 256 x 8 tf32 instruction.)
                    const int nk = kb_end - kb < kps ? kb_end - kb : kps;
                    const int kfirst = kb - kb_begin;   // 0 on the first K block of the tile: overwrite the accumulator
#pragma unroll
                    for (int j = 0; j < KPS_MAX; ++j) {
                        if (j >= nk) break;
                        const uint64_t da = desc_a0 + (uint64_t)((s * a_stage + j * a_slab) >> 4);
                        const uint64_t db = desc_b0 + (uint64_t)((s * b_stage + j * b_slab) >> 4);
                        if constexpr (MH == 2) {
                            // both halves of A against the same B step; half h accumulates into its own BN columns
                            const uint64_t dh = (uint64_t)(a_half >> 4);
                            for (int k = 0; k < mma_per_kb; ++k) {
                                const uint32_t acc = (uint32_t)((kfirst | j | k) != 0);
                                mma(d_tmem, da + 2 * k, db + 2 * k, acc);
                                mma(d_tmem + BN, da + dh + 2 * k, db + 2 * k, acc);
                            }
                        } else if (mma_per_kb == 4) {
                            mma(d_tmem, da, db, (uint32_t)((kfirst | j) != 0));
                            mma(d_tmem, da + 2, db + 2, 1u);
                            mma(d_tmem, da + 4, db + 4, 1u);
                            mma(d_tmem, da + 6, db + 6, 1u);
                        } else {
                            for (int k = 0; k < mma_per_kb; ++k)
                                mma(d_tmem, da + 2 * k, db + 2 * k, (uint32_t)((kfirst | j | k) != 0));
                        }
                    }
                    commit(empty0 + 8 * s);   // stage reusable once these MMAs have read it
                }
                __syncwarp();
            }
            // the residual: each 128 x 64 stage times the identity, into the 64 accumulator columns it belongs to
            if (res_mma && ok) {
                const int n0 = (int)((tile % tiles_per_batch) % n_tiles) * BN;
                const uint32_t idesc_r = make_idesc<KIND>(TILE_M, 64) & (p.ab_f16 ? ~((7u << 7) | (7u << 10)) : ~0u);
                const uint64_t desc_i = make_smem_desc(smem_u32(sIdent), 128);
                const int nres = (p.N - n0 < BN ? p.N - n0 : BN) / 64;
                const int cap = 1 + (int)(b_stage / RES_PIECE);
                for (int j = 0; j < nres;) {
                    const int s = ms;
                    const uint32_t ph = mph;
                    if (++ms == stages) { ms = 0; mph ^= 1; }
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag) || (!ident_ready && !mbar_wait(ident_bar, 0, abort_flag))) {
                        if (lane == 0) atomicOr(p.status, ST_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    ident_ready = true;
                    const int take = nres - j < cap ? nres - j : cap;
                    if (lane == 0) {
                        for (int t = 0; t < take; ++t) {
                            const uint64_t da = make_smem_desc(t == 0 ? smem_u32(sA) + s * a_stage : smem_u32(sB) + s * b_stage + (uint32_t)(t - 1) * RES_PIECE, 128);
#pragma unroll
                            for (int k = 0; k < 4; ++k) tc_mma<KIND>(d_tmem + (uint32_t)((j + t) * 64), da + 2 * k, desc_i + 2 * k, idesc_r, 1u);
                        }
                        commit(empty0 + 8 * s);
                    }
                    j += take;
                    __syncwarp();
                }
            }
            if (ok && lane == 0) commit(acc_full0 + 8 * a);   // accumulator of this tile complete
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (2 groups x 4 warps)
        // The two groups take alternate tiles, so one group's epilogue overlaps the other's and the
        // main loop.  Within a group each warp owns one TMEM lane quarter.  Per 32-column chunk:
        //   A. tcgen05.ld: thread = accumulator row, 32 raw 32-bit columns; written to the warp's
        //      patch as 8 x 16 bytes, chunk j of row r at position j ^ (r & 7) (conflict free);
        //   B. read back transposed: 8 lanes cover one 128-byte row, so a lane owns 4 fixed columns
        //      for 8 rows.  Bias / de-quantisation / activation / residual / rounding happen here,
        //      and every global access is a whole 128-byte row segment.
        const int ew = warp - 2;                    // 0..7
        const int quarter = warp & 3;               // TMEM lane quarter this warp may read
        const int group = ew >> 2;                  // which alternate tiles this warp takes
        // When no CTA has more than one tile (a launch of at most one wave: small batches, split-K units)
        // alternating tiles would leave one group idle while the other walks the whole tile; instead both
        // groups drain the same accumulator, group g taking the 32-column chunks g, g + 2, ...
        const bool share_tile = (p.epi_mode & 1) && total_tiles <= (long long)ncta;
        const bool out16 = out_is_16(p.out_mode), f16 = p.out_mode == OUT_F16;
        // Chunk v of a tile: CW columns starting at (v % (BN / CW)) * CW of half v / (BN / CW).  A chunk is what
        // one TMA store writes (and one TMA load of the residual brings): 32 rows x 128 bytes, i.e. 32 fp32 or
        // 64 16-bit columns -- the TMA unit takes about as long for a 2 KB box as for a 4 KB one (measured: ~90 /
        // ~150 cycles per store / load box per SM whatever its size), so boxes are as large as the patch allows.
        // A 64-column chunk is computed as two 32-column halves.  The plain-store path works on 32 columns.
        // Only the 16-bit instantiation has the two-half form (the others keep a single straight-line half).
        constexpr int CW_MAX = (KIND == KIND_BF16) ? 64 : 32;
        const int CW = (CW_MAX == 64 && p.tma_store == 1 && out16) ? 64 : 32;
        const int CHUNKS = BN / CW, VCHUNKS = MH * CHUNKS;
        const int v_start = share_tile ? group : 0, v_step = share_tile ? NG : 1;
        float vmax = 0.f;   // largest magnitude this thread wrote as fp16
        uint4 *patch = reinterpret_cast<uint4 *>(sPatch + ew * EPI_PATCH_BYTES);
        // Second output patch (the residual patches' space, when neither a residual nor the activation
        // table lives there): a chunk is written into one patch while the TMA store of the previous chunk
        // is still reading the other, instead of waiting for that store before every chunk.
        const bool two_patches = (p.epi_mode & 2) && p.tma_store && p.residual == nullptr && !p.lut_smem;
        uint4 *patch_alt = reinterpret_cast<uint4 *>(sRes + ew * EPI_PATCH_BYTES);
        const bool vec_ok = (p.ldo % 4 == 0) && (p.out_batch_stride % 4 == 0) &&
                            (((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.residual) |
                               reinterpret_cast<uintptr_t>(p.out_q)) & 15) == 0);
        const int chunk = lane & 7;                 // 16-byte column group owned in phase B
        const int rsub = lane >> 3;                 // row within each group of 4 rows
        const int act = p.act;
        // Residual through TMA (fast path only).  The patches of the residual tensor that line up with this
        // warp's next output patches are fetched ahead into a ring of 4 KB slots, each with its own barrier.
        // The warp's sequence of (tile, chunk) positions is walked by a second cursor that runs ahead of the
        // one the chunk loop follows; a tile's coordinates are computed once per tile, not per chunk.
        const uint32_t res_bytes = (out16 && CW == 32) ? 32 * 64 : 32 * 128;
        const bool res_tma = p.tma_store && p.residual != nullptr;
        const int res_slots = 1;
        auto res_slot = [&](int sl) -> const uint4 * { return reinterpret_cast<const uint4 *>(sRes + (ew + sl * NEW) * EPI_PATCH_BYTES); };
        const long long first_tile = share_tile ? (long long)cid : (long long)cid + (long long)group * ncta;
        const long long tile_step = (share_tile ? 1 : NG) * (long long)ncta;   // this warp's next tile
        // first chunk of a tile starting at column n_, from v on in this warp's stride, that lies inside the matrix
        auto next_chunk = [&](int n_, int v) {
            while (v < VCHUNKS && n_ + (v - (v >= CHUNKS ? CHUNKS : 0)) * CW >= p.N) v += v_step;   // MH <= 2: no division
            return v;
        };
        long long pf_tile = first_tile;   // prefetch cursor: tile, chunk and the tile's coordinates
        int pf_v = 0, pf_bz = 0, pf_r0 = 0, pf_n0 = 0;
        auto pf_enter = [&]() {           // coordinates of pf_tile, its first chunk
            if (pf_tile >= total_tiles) return;
            pf_bz = (int)(pf_tile / tiles_per_batch);
            const int tin_ = (int)(pf_tile - pf_bz * tiles_per_batch);
            pf_r0 = (tin_ / n_tiles) * TILE_ROWS + row_off + quarter * 32;
            pf_n0 = (tin_ % n_tiles) * BN;
            pf_v = next_chunk(pf_n0, v_start);
        };
        int res_issued = 0, res_taken = 0;   // patches requested / consumed by this warp so far
        auto issue_res = [&]() {             // request the patch at the prefetch cursor (if any is left), advance it
            while (res_tma && pf_tile < total_tiles) {
                const int pf_half = pf_v >= CHUNKS ? 1 : 0;
                const int r0 = pf_r0 + pf_half * TILE_M, n_ = pf_n0 + (pf_v - pf_half * CHUNKS) * CW, bz_ = pf_bz;
                pf_v = next_chunk(pf_n0, pf_v + v_step);
                if (pf_v >= VCHUNKS) {
                    pf_tile += tile_step;
                    pf_enter();
                }
                if (r0 >= p.M) continue;     // rows outside the matrix: no patch (the chunk loop skips it the same way)
                const int sl = res_issued % res_slots;
                if (lane == 0) {
                    const uint32_t bar = res_bar0 + 8 * (ew * RES_SLOTS + sl);
                    mbar_arrive_expect_tx(bar, res_bytes);
                    if (p.batched) tma_load_3d(smem_u32(res_slot(sl)), &tmR, bar, n_, r0, bz_);
                    else tma_load_2d(smem_u32(res_slot(sl)), &tmR, bar, n_, r0);
                }
                ++res_issued;
                return;
            }
        };
        pf_enter();
        for (int i = 0; i < res_slots; ++i) issue_res();
        int lt = 0;
        for (long long tile = cid; tile < total_tiles; tile += ncta, ++lt) {
            if (!share_tile && (lt % NG) != group) continue;
            const int a = lt % ACC;
            const int bz = (int)(tile / tiles_per_batch);
            const int tin = (int)(tile - bz * tiles_per_batch);
            const int m0 = (tin / n_tiles) * TILE_ROWS + row_off;
            const int n0 = (tin % n_tiles) * BN;
            if (!mbar_wait(acc_full0 + 8 * a, (uint32_t)((lt / ACC) & 1), abort_flag)) {
                if (lane == 0) atomicOr(p.status, ST_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * ACC_COLS);
            // The accumulator buffer goes back to the MMA issuer as soon as this warp's last TMEM load of the tile
            // has landed in registers (fast path), not after the math and the store that follow it: the issuer's
            // next tile into this buffer then overlaps the rest of this one's epilogue.
            bool released = false;
            auto release_acc = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && rank != 0) mbar_arrive_cluster(mapa_shared(acc_empty0 + 8 * a, 0));   // the even CTA's issuer waits for both CTAs
                    else mbar_arrive(acc_empty0 + 8 * a);
                }
                released = true;
            };
            int last_vc = -1;
            for (int v = v_start; v < VCHUNKS; v += v_step)
                if (n0 + (v - (v >= CHUNKS ? CHUNKS : 0)) * CW < p.N) last_vc = v;
            for (int vc = v_start; vc < VCHUNKS; vc += v_step) {
                const int half = vc >= CHUNKS ? 1 : 0, c0 = (vc - half * CHUNKS) * CW;
                if (n0 + c0 >= p.N) continue;
                const uint32_t taddr = taddr0 + (uint32_t)(half * BN);
                const int row0 = m0 + half * TILE_M + quarter * 32;
                if (p.tma_store) {
                    // Fast path (N % 32 == 0): all math in the accumulator's own layout (thread = row), the
                    // finished patch goes out with one TMA store, which also clips the M tail (and, for a
                    // 64-column chunk, a second half that lies beyond N).
                    const bool res_here = res_tma && row0 < p.M;
                    const uint4 *rpatch = nullptr;
                    bool gave_up = false;
#pragma unroll
                    for (int h = 0; h < CW_MAX / 32; ++h) {
                    if (h * 32 >= CW) break;
                    const int cc = c0 + 32 * h;      // this half's first column within the tile
                    if (n0 + cc >= p.N) break;
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + cc, r);
                    float v[32];
                    const float4 *bp4 = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.bias) + n0 + cc);
                    if constexpr (KIND == KIND_I8) {
                        const float4 *kp4 = reinterpret_cast<const float4 *>(p.coeff + n0 + cc);
                        const float in_scale = p.in_scale;
                        const bool has_b = p.bias != nullptr;
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 b = has_b ? __ldg(bp4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                            const float4 k = __ldg(kp4 + j);
                            v[4 * j] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)r[4 * j]), in_scale), b.x), k.x);
                            v[4 * j + 1] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 1]), in_scale), b.y), k.y);
                            v[4 * j + 2] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 2]), in_scale), b.z), k.z);
                            v[4 * j + 3] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 3]), in_scale), b.w), k.w);
                        }
                    } else {
                        if (p.bias_mode == BIAS_F32) {
                            float4 b[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) b[j] = __ldg(bp4 + j);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                v[4 * j] = __fadd_rn(__uint_as_float(r[4 * j]), b[j].x);
                                v[4 * j + 1] = __fadd_rn(__uint_as_float(r[4 * j + 1]), b[j].y);
                                v[4 * j + 2] = __fadd_rn(__uint_as_float(r[4 * j + 2]), b[j].z);
                                v[4 * j + 3] = __fadd_rn(__uint_as_float(r[4 * j + 3]), b[j].w);
                            }
                        } else {
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        }
                    }
                    if ((p.epi_mode & 4) && vc == last_vc && (h * 32 + 32 >= CW || n0 + cc + 32 >= p.N)) release_acc();   // the tile's last load is in registers
                    // uniform branches outside the unrolled loops: the 32 elements' chains interleave
                    if (act == 1) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
                    } else if (act == 3) {
                        if (p.lut_smem) {
                            // the table sits in shared memory: a gather from global memory runs at about one
                            // lookup per clock per SM and would bound the whole kernel
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = silu_table(v[j], slut);
                        } else {
                            const float *lut = p.lut;
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = silu_table(v[j], lut);
                        }
                    } else if (act != 0) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], act, p.act_p0, p.act_p1, p.lut);
                    }
                    if (res_here) {
                        // add the prefetched residual patch (same swizzle as the output patch), then relu
                        if (h == 0) {
                            const int sl = res_taken % res_slots;
                            if (!mbar_wait(res_bar0 + 8 * (ew * RES_SLOTS + sl), (uint32_t)((res_taken / res_slots) & 1), abort_flag)) {
                                if (lane == 0) atomicOr(p.status, ST_TIMEOUT_EPILOGUE);
                                gave_up = true;
                                break;
                            }
                            ++res_taken;
                            rpatch = res_slot(sl);
                        }
                        if (out16) {
                            // the format is chosen outside the unrolled loops, so that each holds one conversion
                            if (CW == 64) {
                                if (f16) add_patch16<true>(v, rpatch, lane, h);
                                else add_patch16<false>(v, rpatch, lane, h);
                            } else {
                                if (f16) add_patch16_narrow<true>(v, rpatch, lane);
                                else add_patch16_narrow<false>(v, rpatch, lane);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint4 q = rpatch[lane * 8 + (j ^ (lane & 7))];
                                v[4 * j] = __fadd_rn(v[4 * j], __uint_as_float(q.x));
                                v[4 * j + 1] = __fadd_rn(v[4 * j + 1], __uint_as_float(q.y));
                                v[4 * j + 2] = __fadd_rn(v[4 * j + 2], __uint_as_float(q.z));
                                v[4 * j + 3] = __fadd_rn(v[4 * j + 3], __uint_as_float(q.w));
                            }
                        }
                        if (p.res_relu) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
                        }
                    }
                    // the store that last read this patch has finished with it (with two patches that is the
                    // store before the previous one)
                    if (h == 0) {
                        if (lane == 0) {
                            if (two_patches) bulk_wait_read1();
                            else bulk_wait_read0();
                        }
                        __syncwarp();
                    }
                    if (p.tma_store == 2) {
                        // int8-only output: quantise for the next layer (conv.c:961-973 at the producer); rows of
                        // 32 bytes, lane = row: the patch is written linearly (no swizzle, no bank conflicts)
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            w[j] = ((uint32_t)quant_s8(v[4 * j], p.q_inv_scale) & 0xff) | (((uint32_t)quant_s8(v[4 * j + 1], p.q_inv_scale) & 0xff) << 8) |
                                   (((uint32_t)quant_s8(v[4 * j + 2], p.q_inv_scale) & 0xff) << 16) |
                                   (((uint32_t)quant_s8(v[4 * j + 3], p.q_inv_scale) & 0xff) << 24);
                        patch[lane * 2] = make_uint4(w[0], w[1], w[2], w[3]);
                        patch[lane * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
                    } else if (out16) {
                        if (f16) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) vmax = fmaxf(vmax, fabsf(v[j]));
                        }
                        if (CW == 64) {
                            if (f16) store_patch16<true>(v, patch, lane, h);
                            else store_patch16<false>(v, patch, lane, h);
                        } else {
                            if (f16) store_patch16_narrow<true>(v, patch, lane);
                            else store_patch16_narrow<false>(v, patch, lane);
                        }
                    } else {
                        if (p.round_tf32) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = round_to_tf32(v[j]);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            patch[lane * 8 + (j ^ (lane & 7))] =
                                make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                                           __float_as_uint(v[4 * j + 3]));
                    }
                    }   // halves of the chunk
                    if (gave_up) break;
                    if (res_here) {
                        __syncwarp();   // every lane has read the slot: it takes the next patch of the sequence
                        issue_res();
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (row0 < p.M) {
                            if (z_store) tma_store_3d(&tmC, smem_u32(patch), n0 + c0, row0, bz);
                            else tma_store_2d(&tmC, smem_u32(patch), n0 + c0, row0);
                        }
                        bulk_commit();   // committed even when empty: the wait above counts groups, one per chunk
                    }
                    if (two_patches) {
                        uint4 *t = patch;
                        patch = patch_alt;
                        patch_alt = t;
                    }
                    continue;
                }
                // this lane's 4 columns and their per-column constants (issued before the TMEM load so
                // the global latency hides behind it); a missing bias is 0.0f: x + 0.0f == x
                const int col = n0 + c0 + chunk * 4;         // first of this lane's 4 columns
                const int nvalid = p.N - col;                 // > 3: all four columns exist
                const bool full = vec_ok && nvalid >= 4 && (col % 4 == 0);
                float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), k4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (nvalid > 0) {
                    if (p.bias_mode == BIAS_F32) {
                        const float *bp = reinterpret_cast<const float *>(p.bias) + col;
                        if (nvalid >= 4 && (reinterpret_cast<uintptr_t>(bp) & 15) == 0) b4 = __ldg(reinterpret_cast<const float4 *>(bp));
                        else {
                            b4.x = __ldg(bp);
                            if (nvalid > 1) b4.y = __ldg(bp + 1);
                            if (nvalid > 2) b4.z = __ldg(bp + 2);
                            if (nvalid > 3) b4.w = __ldg(bp + 3);
                        }
                    } else if (p.bias_mode == BIAS_S32_DEQUANT) {
                        if (p.bias) {
                            const float *bp = reinterpret_cast<const float *>(p.bias) + col;
                            b4.x = __ldg(bp);
                            if (nvalid > 1) b4.y = __ldg(bp + 1);
                            if (nvalid > 2) b4.z = __ldg(bp + 2);
                            if (nvalid > 3) b4.w = __ldg(bp + 3);
                        }
                        const float *kp = p.coeff + col;
                        k4.x = __ldg(kp);
                        if (nvalid > 1) k4.y = __ldg(kp + 1);
                        if (nvalid > 2) k4.z = __ldg(kp + 2);
                        if (nvalid > 3) k4.w = __ldg(kp + 3);
                    }
                }
                {   // phase A
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        patch[lane * 8 + (j ^ (lane & 7))] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                }
                __syncwarp();
                // phase B
                const long long col_off = (long long)bz * p.out_batch_stride + col;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = i * 4 + rsub;
                    const int grow = row0 + rr;
                    const uint4 raw = patch[rr * 8 + (chunk ^ (rr & 7))];
                    if (grow >= p.M || nvalid <= 0) continue;
                    const long long off = col_off + (long long)grow * p.ldo;
                    if (p.out_mode == OUT_RAW32) {
                        uint32_t *o = reinterpret_cast<uint32_t *>(p.out) + off;
                        if (full) *reinterpret_cast<uint4 *>(o) = raw;
                        else {
                            o[0] = raw.x;
                            if (nvalid > 1) o[1] = raw.y;
                            if (nvalid > 2) o[2] = raw.z;
                            if (nvalid > 3) o[3] = raw.w;
                        }
                        continue;
                    }
                    float t[4];
                    if constexpr (KIND == KIND_I8) {
                        // (float)acc * input_scale; += (float)bias_s32; *= weight_aux / 127
                        t[0] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)raw.x), p.in_scale), b4.x), k4.x);
                        t[1] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)raw.y), p.in_scale), b4.y), k4.y);
                        t[2] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)raw.z), p.in_scale), b4.z), k4.z);
                        t[3] = __fmul_rn(__fadd_rn(__fmul_rn(__int2float_rn((int)raw.w), p.in_scale), b4.w), k4.w);
                    } else {
                        t[0] = __fadd_rn(__uint_as_float(raw.x), b4.x);
                        t[1] = __fadd_rn(__uint_as_float(raw.y), b4.y);
                        t[2] = __fadd_rn(__uint_as_float(raw.z), b4.z);
                        t[3] = __fadd_rn(__uint_as_float(raw.w), b4.w);
                    }
                    if (act == 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) t[e] = t[e] > 0.f ? t[e] : 0.f;
                    } else if (act == 3) {
                        if (p.lut_smem) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) t[e] = silu_table(t[e], slut);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) t[e] = silu_table(t[e], p.lut);
                        }
                    } else if (act != 0) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) t[e] = apply_act(t[e], act, p.act_p0, p.act_p1, p.lut);
                    }
                    if (p.residual) {
                        if (out16) {
                            const uint16_t *rp = reinterpret_cast<const uint16_t *>(p.residual) + off;
                            if (full) {
                                const uint2 q = *reinterpret_cast<const uint2 *>(rp);
                                const float2 lo = h16_unpack2(q.x, f16), hi = h16_unpack2(q.y, f16);
                                t[0] = __fadd_rn(t[0], lo.x); t[1] = __fadd_rn(t[1], lo.y);
                                t[2] = __fadd_rn(t[2], hi.x); t[3] = __fadd_rn(t[3], hi.y);
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e) if (e < nvalid) t[e] = __fadd_rn(t[e], h16_unpack1(rp[e], f16));
                            }
                        } else {
                            const float *rp = reinterpret_cast<const float *>(p.residual) + off;
                            if (full) {
                                const float4 q = *reinterpret_cast<const float4 *>(rp);
                                t[0] = __fadd_rn(t[0], q.x); t[1] = __fadd_rn(t[1], q.y);
                                t[2] = __fadd_rn(t[2], q.z); t[3] = __fadd_rn(t[3], q.w);
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e) if (e < nvalid) t[e] = __fadd_rn(t[e], rp[e]);
                            }
                        }
                        if (p.res_relu) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) t[e] = t[e] > 0.f ? t[e] : 0.f;
                        }
                    }
                    if (p.out_q) {
                        int8_t *q = p.out_q + off;
                        if (full) {
                            const uint32_t b0 = (uint32_t)quant_s8(t[0], p.q_inv_scale) & 0xff;
                            const uint32_t b1 = (uint32_t)quant_s8(t[1], p.q_inv_scale) & 0xff;
                            const uint32_t b2 = (uint32_t)quant_s8(t[2], p.q_inv_scale) & 0xff;
                            const uint32_t b3 = (uint32_t)quant_s8(t[3], p.q_inv_scale) & 0xff;
                            *reinterpret_cast<uint32_t *>(q) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (e < nvalid) q[e] = (int8_t)quant_s8(t[e], p.q_inv_scale);
                        }
                    }
                    if (p.out == nullptr) continue;
                    if (out16) {
                        uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + off;
                        if (f16) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (e < nvalid) vmax = fmaxf(vmax, fabsf(t[e]));
                        }
                        if (full) {
                            uint2 q;
                            q.x = h16_pack2(t[0], t[1], f16);
                            q.y = h16_pack2(t[2], t[3], f16);
                            *reinterpret_cast<uint2 *>(o) = q;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (e < nvalid) o[e] = h16_pack1(t[e], f16);
                        }
                    } else {
                        if (p.round_tf32) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) t[e] = round_to_tf32(t[e]);
                        }
                        float *o = reinterpret_cast<float *>(p.out) + off;
                        if (full) *reinterpret_cast<float4 *>(o) = make_float4(t[0], t[1], t[2], t[3]);
                        else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (e < nvalid) o[e] = t[e];
                        }
                    }
                }
                __syncwarp();
            }
            // hand the accumulator buffer back to the MMA issuer (if the fast path has not done so already)
            if (!released) release_acc();
        }
        if (p.tma_store && lane == 0) bulk_wait_read0();   // patches must outlive the stores' reads
        // after a give-up: residual patches that were requested but never consumed must still land (bounded
        // wait) before the block may go
        {
            int local_abort = 0;
            while (res_tma && res_taken < res_issued) {
                const int sl = res_taken % res_slots;
                if (!mbar_wait(res_bar0 + 8 * (ew * RES_SLOTS + sl), (uint32_t)((res_taken / res_slots) & 1), &local_abort)) break;
                ++res_taken;
            }
        }
        if (f16 && __any_sync(0xffffffffu, vmax > F16_MAX) && lane == 0) atomicOr(p.status, ST_RANGE_F16);
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && warp == 0 && rank == 0) {
        // A role gave up.  Before the CTA exits, wait (bounded) for the loads that were issued so
        // that no copy lands in shared memory after the block has gone.  (In a pair every load's bytes
        // are counted on the even CTA's barriers, and the odd CTA leaves only after the cluster barrier
        // below, i.e. after the even CTA has seen them land.)
        int dummy = 0;
        const long long first = issued > stages ? issued - stages : 0;
        for (long long kb = first; kb < issued; ++kb) {
            if (!mbar_wait(full0 + 8 * (int)(kb % stages), (uint32_t)((kb / stages) & 1), &dummy)) {
                if (lane == 0) atomicOr(p.status, ST_TIMEOUT_DRAIN);
                break;
            }
        }
        if (res_mma && !mbar_wait(ident_bar, 0, &dummy) && lane == 0) atomicOr(p.status, ST_TIMEOUT_DRAIN);   // the identity tile
    }
    // A pair leaves together: until here the peer may still signal this CTA's barriers, and the even
    // CTA's MMAs read the odd CTA's shared memory and write its tensor memory.
    if constexpr (PAIR) cluster_sync();
    if (warp == 1) {
        tc_fence_after_sync();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, tmem_cols_for(BN, MH));
        else tmem_dealloc(tmem_base, tmem_cols_for(BN, MH));
    }
}

// Second step of a split-K contraction (see SplitKReduceParams).  One thread per 4 consecutive columns;
// the planes are L2 resident (a split launch is small by construction), so this is a short streaming pass.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const SplitKReduceParams p, int pdl)
{
    if (pdl) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const bool out16 = out_is_16(p.out_mode), f16 = p.out_mode == OUT_F16;
    float vmax = 0.f;
    const long long quads_per_row = p.N >> 2;
    const long long total = (long long)p.M * quads_per_row;
    for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (long long)gridDim.x * blockDim.x) {
        const long long m = q / quads_per_row;
        const int n = (int)(q - m * quads_per_row) << 2;
        const float *src = p.partial + m * p.partial_ld + n;
        float4 acc = __ldcg(reinterpret_cast<const float4 *>(src));
        for (int z = 1; z < p.split_k; ++z) {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + (long long)z * p.plane_stride));
            acc.x = __fadd_rn(acc.x, t.x); acc.y = __fadd_rn(acc.y, t.y);
            acc.z = __fadd_rn(acc.z, t.z); acc.w = __fadd_rn(acc.w, t.w);
        }
        float v[4] = {acc.x, acc.y, acc.z, acc.w};
        if (p.bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = __fadd_rn(v[e], __ldg(p.bias + n + e));
        }
        if (p.act == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = v[e] > 0.f ? v[e] : 0.f;
        } else if (p.act != 0) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = apply_act(v[e], p.act, p.act_p0, p.act_p1, p.lut);
        }
        const long long off = m * p.ldo + n;
        if (p.residual) {
            if (out16) {
                const uint2 r = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(p.residual) + off);
                const float2 lo = h16_unpack2(r.x, f16), hi = h16_unpack2(r.y, f16);
                v[0] = __fadd_rn(v[0], lo.x); v[1] = __fadd_rn(v[1], lo.y);
                v[2] = __fadd_rn(v[2], hi.x); v[3] = __fadd_rn(v[3], hi.y);
            } else {
                const float4 r = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) + off);
                v[0] = __fadd_rn(v[0], r.x); v[1] = __fadd_rn(v[1], r.y); v[2] = __fadd_rn(v[2], r.z); v[3] = __fadd_rn(v[3], r.w);
            }
            if (p.res_relu) {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = v[e] > 0.f ? v[e] : 0.f;
            }
        }
        if (out16) {
            if (f16) vmax = fmaxf(fmaxf(vmax, fmaxf(fabsf(v[0]), fabsf(v[1]))), fmaxf(fabsf(v[2]), fabsf(v[3])));
            uint2 o;
            o.x = h16_pack2(v[0], v[1], f16);
            o.y = h16_pack2(v[2], v[3], f16);
            *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(p.out) + off) = o;
        } else {
            if (p.round_tf32) {
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = round_to_tf32(v[e]);
            }
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + off) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
    if (f16 && vmax > F16_MAX && p.status) atomicOr(p.status, ST_RANGE_F16);
}

// Failure-detection self test: one warp waits on an mbarrier that nothing will ever complete, with a
// short clock limit, then reports through the status word exactly as a stalled pipeline role would.
// The kernel returns normally; the context stays usable.
__global__ void wait_probe_kernel(unsigned int *status, long long limit_clocks)
{
    __shared__ uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncthreads();
    // the same bounded wait the pipeline roles use, with a short limit
    __shared__ int abort_flag;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    const bool done = !mbar_wait(b, 0, &abort_flag, limit_clocks);   // never completes: nobody arrives
    if (done && threadIdx.x == 0) atomicOr(status, ST_TIMEOUT_EPILOGUE);
}

cudaError_t launch_wait_probe(unsigned int *status, long long limit_clocks, cudaStream_t stream)
{
    wait_probe_kernel<<<1, 32, 0, stream>>>(status, limit_clocks);
    count_launch();
    return cudaGetLastError();
}

static std::atomic<int> g_pdl{1};
static std::atomic<int> g_epi_mode{15};
int get_epilogue_mode() { return g_epi_mode.load(std::memory_order_relaxed); }
void set_epilogue_mode(int bits) { g_epi_mode.store(bits & 15, std::memory_order_relaxed); }
void set_pdl(int on) { g_pdl.store(on ? 1 : 0, std::memory_order_relaxed); }
int get_pdl() { return g_pdl.load(std::memory_order_relaxed); }

// Launch with the programmatic-stream-serialisation attribute when `pdl` (the kernel may be scheduled
// before the previous kernel on the stream has finished and orders itself with griddepcontrol.wait) and as
// clusters of `cluster` CTAs when that is above 1.
template <typename... KArgs, typename... Args>
static cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, int cluster, Args &&...args)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static int sm_count_of(int dev)
{
    // written once per device; concurrent first calls from different threads store the same value
    static std::atomic<int> sm_count[64];
    if (dev < 0 || dev >= 64) return 148;
    int n = sm_count[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sm_count[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

template <int KIND, int BN, bool PAIR, int MH = 1, int NEW = NUM_EPI_WARPS>
static cudaError_t launch_one(const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC, const CUtensorMap &tmR, const CUtensorMap &tmI,
                              IgemmParams p, cudaStream_t stream)
{
    // per kernel instance and device; setting the attribute twice from two threads is harmless
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    const size_t smem = igemm_smem_bytes(BN, PAIR, MH, NEW);
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(igemm_kernel<KIND, BN, PAIR, MH, NEW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    constexpr int rows = PAIR ? 2 * TILE_M : MH * TILE_M;
    const long long m_tiles = (p.M + rows - 1) / rows;
    const long long n_tiles = (p.N + BN - 1) / BN;
    const long long tiles = m_tiles * n_tiles * (p.batched ? p.batch : (p.split_k > 1 ? p.split_k : 1));
    if (tiles <= 0) return cudaErrorInvalidConfiguration;
    if (PAIR && (p.batched || p.split_k > 1)) return cudaErrorInvalidValue;
    if (p.res_mma && (KIND != KIND_BF16 || ident_bytes_for(BN, PAIR, MH) == 0 || p.batched || p.split_k > 1 || p.slab_bytes != 128 || p.residual)) return cudaErrorInvalidValue;
    // persistent: one CTA per SM (the shared-memory ring and the accumulators fill an SM); a pair takes
    // the two SMs of a TPC
    const long long sms = sm_count_of(dev);
    const long long slots = PAIR ? sms / 2 : sms;
    const unsigned grid = (unsigned)(tiles < slots ? tiles : slots) * (PAIR ? 2u : 1u);
    p.pdl = get_pdl();
    p.epi_mode = g_epi_mode.load(std::memory_order_relaxed);
    cudaError_t e = launch_ex(igemm_kernel<KIND, BN, PAIR, MH, NEW>, dim3(grid), dim3(num_threads_for(NEW)), smem, stream, p.pdl != 0, PAIR ? 2 : 1, tmA, tmB, tmC, tmR, tmI, p);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_igemm(int kind, int bn, bool pair, int mh, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap *tmC_opt,
                         const CUtensorMap *tmR_opt, const IgemmParams &p, cudaStream_t stream, const CUtensorMap *tmI_opt, int epi_warps)
{
    if (epi_warps != 8 && (epi_warps != 12 || pair || mh != 1 || bn > 128)) return cudaErrorInvalidValue;
    CUtensorMap tmC, tmR, tmI;
    if (tmI_opt) tmI = *tmI_opt;
    else memset(&tmI, 0, sizeof(tmI));
    if (p.res_mma && (!tmI_opt || !tmR_opt)) return cudaErrorInvalidValue;
    if (tmC_opt) tmC = *tmC_opt;
    else memset(&tmC, 0, sizeof(tmC));
    if (tmR_opt) tmR = *tmR_opt;
    else memset(&tmR, 0, sizeof(tmR));
    if (p.tma_store && (!tmC_opt || (p.residual && !tmR_opt))) return cudaErrorInvalidValue;
    if (mh != 1 && (mh != 2 || pair || bn > 128)) return cudaErrorInvalidValue;
    IgemmParams q = p;
    if (kind == KIND_F16) {   // the 16-bit instantiation with fp16 operands
        kind = KIND_BF16;
        q.ab_f16 = 1;
    }
#define ONE_DISPATCH(K)                                                                       \
    if (epi_warps == 12) {                                                                    \
        if (bn == 64) return launch_one<K, 64, false, 1, 12>(tmA, tmB, tmC, tmR, tmI, q, stream);  \
        return launch_one<K, 128, false, 1, 12>(tmA, tmB, tmC, tmR, tmI, q, stream);          \
    }                                                                                         \
    if (mh == 2) {                                                                            \
        if (bn == 64) return launch_one<K, 64, false, 2>(tmA, tmB, tmC, tmR, tmI, q, stream);      \
        return launch_one<K, 128, false, 2>(tmA, tmB, tmC, tmR, tmI, q, stream);                   \
    }                                                                                         \
    if (pair) {                                                                               \
        switch (bn) {                                                                         \
        case 128: return launch_one<K, 128, true>(tmA, tmB, tmC, tmR, tmI, q, stream);             \
        case 192: return launch_one<K, 192, true>(tmA, tmB, tmC, tmR, tmI, q, stream);             \
        case 256: return launch_one<K, 256, true>(tmA, tmB, tmC, tmR, tmI, q, stream);             \
        default: return cudaErrorInvalidValue;                                                \
        }                                                                                     \
    }                                                                                         \
    switch (bn) {                                                                             \
    case 64: return launch_one<K, 64, false>(tmA, tmB, tmC, tmR, tmI, q, stream);                  \
    case 128: return launch_one<K, 128, false>(tmA, tmB, tmC, tmR, tmI, q, stream);                \
    case 192: return launch_one<K, 192, false>(tmA, tmB, tmC, tmR, tmI, q, stream);                \
    case 256: return launch_one<K, 256, false>(tmA, tmB, tmC, tmR, tmI, q, stream);                \
    default: return cudaErrorInvalidValue;                                                    \
    }
    if (kind == KIND_TF32) { ONE_DISPATCH(KIND_TF32) }
    if (kind == KIND_BF16) { ONE_DISPATCH(KIND_BF16) }
    if (kind == KIND_I8) { ONE_DISPATCH(KIND_I8) }
#undef ONE_DISPATCH
    return cudaErrorInvalidValue;
}

cudaError_t launch_splitk_reduce(const SplitKReduceParams &p, cudaStream_t stream)
{
    if (p.split_k < 1 || p.M <= 0 || p.N <= 0 || (p.N & 3) || (p.ldo & 3) || (p.plane_stride & 3) || (p.partial_ld & 3)) return cudaErrorInvalidValue;
    int dev = 0;
    cudaGetDevice(&dev);
    const long long total = (long long)p.M * (p.N >> 2);
    const long long want = (total + 255) / 256, cap = (long long)sm_count_of(dev) * 8;
    const int pdl = get_pdl();
    cudaError_t e = launch_ex(splitk_reduce_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, pdl != 0, 1, p, pdl);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace one
