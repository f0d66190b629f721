// igemm.cu -- the sm_100a implicit-GEMM kernel behind Conv, Gemm and MatMul.
//
// One CTA computes one 128 x BN tile of D = A * B^T.  Roles (192 threads):
//   warp 0, one lane : TMA producer.  Per K block it issues one load of the A tile
//                      (128 rows x slab_bytes; im2col mode for convolutions) and one of the B tile
//                      (BN rows x slab_bytes) into a STAGES-deep shared-memory ring.
//   warp 1, one lane : issues tcgen05.mma (one per 32 bytes of K) with the accumulator in TMEM;
//                      tcgen05.commit frees the stage and, at the end, publishes the tile.
//   warps 2..5       : epilogue.  tcgen05.ld the accumulator (each warp its lane quarter), apply
//                      bias / int8 de-quantisation / activation / residual, store NHWC rows.
// Replaces, in the reference, the pad + im2col + SGEMM + bias pass + activation pass chain of
// device/x86/Conv/conv.c:300-415 (and :68-166, :901-1059, :1216-1304), the SGEMM of
// device/x86_utils/opt_gemm.h:17-174, device/x86/Gemm/gemm.c:9-79 and
// device/x86/MatMul/mat_mul.c:10-101.
//
// Algorithmic bytes per tile: A 128*K*es + B BN*K*es read, 128*BN*out_es written; the
// im2col matrix is never materialised.
#include "igemm.cuh"
#include "sm100_prims.cuh"
#include "ctx.h"

#include <cuda_bf16.h>

namespace one {

static constexpr int TILE_M = 128;
static constexpr int A_STAGE_BYTES = TILE_M * 128;   // room for the widest (128 B) slab
static constexpr int NUM_THREADS = 192;

__host__ __device__ constexpr int stages_for(int bn) { return bn == 256 ? 4 : (bn == 128 ? 3 : 4); }

__host__ __device__ constexpr size_t smem_layout_bytes(int bn)
{
    return (size_t)stages_for(bn) * (A_STAGE_BYTES + bn * 128) + 256 /* barriers etc. */ +
           2 * (size_t)bn * 4 /* bias + coeff */;
}

size_t igemm_smem_bytes(int bn) { return smem_layout_bytes(bn) + 1024; }

// ACT_TYPE_E of the reference ABI: 0 none, 1 relu, 2 relu6 (never handled by the reference:
// identity), 3 silu (table), 4 clip, 5 hard-silu, 6 leaky relu.  Mirrors do_act,
// device/x86/Conv/conv.c:1216-1304, with the multiplies and adds kept separate as the
// reference's -std=c11 build does (no FMA contraction).
__device__ __forceinline__ float apply_act(float v, int act, float p0, float p1, const float *__restrict__ lut)
{
    switch (act) {
    case 1: return v > 0.f ? v : 0.f;
    case 3:
        if (v < -8.0f) return 0.f;
        if (v >= 8.0f) return v;
        if (v >= -8.0f && v < 8.0f) return __ldg(lut + (int)__fmul_rn(__fadd_rn(v, 8.0f), 512.0f));
        return v;
    case 4: {
        float t = v > p0 ? v : p0;
        return t < p1 ? t : p1;
    }
    case 5: {
        float t = __fadd_rn(__fmul_rn(p0, v), p1);
        t = t > 0.f ? t : 0.f;
        return __fmul_rn(v, t < 1.f ? t : 1.f);
    }
    case 6: return v > 0.f ? v : __fmul_rn(p0, v);
    default: return v;
    }
}

__device__ __forceinline__ float round_to_tf32(float v)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return __uint_as_float(r);
}

// Quantise for an int8 consumer: x * (1/scale), clamp to [-128, 127], roundf
// (device/x86/Conv/conv.c:961-973).
__device__ __forceinline__ int quant_s8(float v, float inv_scale)
{
    float t = __fmul_rn(v, inv_scale);
    t = (t < -128.f) ? -128.f : (t > 127.f) ? 127.f : t;
    return (int)roundf(t);
}

template <int KIND, int BN>
__global__ void __launch_bounds__(NUM_THREADS)
igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const IgemmParams p)
{
    constexpr int STAGES = stages_for(BN);
    constexpr int B_STAGE_BYTES = BN * 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sA = smem;
    uint8_t *sB = sA + STAGES * A_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sB + STAGES * B_STAGE_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);
    int *abort_flag = reinterpret_cast<int *>(tmem_slot + 1);
    float *s_bias = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(bars) + 256);
    float *s_coeff = s_bias + BN;

    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + STAGES);
    const uint32_t accum_bar = smem_u32(bars + 2 * STAGES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int n_tiles = (p.N + BN - 1) / BN;
    const int tn = blockIdx.x % n_tiles;
    const int tm = blockIdx.x / n_tiles;
    const int m0 = tm * TILE_M;
    const int n0 = tn * BN;
    const int bz = blockIdx.y;   // batch index of a batched MatMul (3-D operand maps)

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    int issued = 0;   // producer: K blocks whose loads were issued

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ TMA producer
        int cw = 0, ch = 0, cn = 0;
        if (p.a_im2col) {
            const int hw = p.OH * p.OW;
            cn = m0 / hw;
            const int rem = m0 - cn * hw;
            const int oh = rem / p.OW;
            const int ow = rem - oh * p.OW;
            cw = ow * p.stride_w - p.pad_l;
            ch = oh * p.stride_h - p.pad_t;
        }
        const uint32_t tx_bytes = (uint32_t)(TILE_M + BN) * (uint32_t)p.slab_bytes;
        int kh = 0, kw = 0, cs = 0;
        for (int kb = 0; kb < p.num_kb; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) {
                atomicOr(p.status, ST_TIMEOUT_PRODUCER);
                break;
            }
            mbar_arrive_expect_tx(full0 + 8 * s, tx_bytes);
            const uint32_t dstA = smem_u32(sA + s * A_STAGE_BYTES);
            if (p.a_im2col) {
                tma_load_im2col_4d(dstA, &tmA, full0 + 8 * s, cs * p.slab_elems, cw, ch, cn, (uint16_t)kw,
                                   (uint16_t)kh);
                if (++cs == p.c_slabs) {
                    cs = 0;
                    if (++kw == p.KW) {
                        kw = 0;
                        ++kh;
                    }
                }
            } else if (p.batched) {
                tma_load_3d(dstA, &tmA, full0 + 8 * s, kb * p.slab_elems, m0, bz);
            } else {
                tma_load_2d(dstA, &tmA, full0 + 8 * s, kb * p.slab_elems, m0);
            }
            if (p.batched)
                tma_load_3d(smem_u32(sB + s * B_STAGE_BYTES), &tmB, full0 + 8 * s, kb * p.slab_elems, n0, bz);
            else
                tma_load_2d(smem_u32(sB + s * B_STAGE_BYTES), &tmB, full0 + 8 * s, kb * p.slab_elems, n0);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = make_idesc<KIND>(TILE_M, BN);
        const int mma_per_kb = p.slab_bytes >> 5;
        bool ok = true;
        for (int kb = 0; kb < p.num_kb; ++kb) {
            const int s = kb % STAGES;
            const uint32_t ph = (kb / STAGES) & 1;
            if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) {
                atomicOr(p.status, ST_TIMEOUT_MMA);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
            const uint32_t b_addr = smem_u32(sB + s * B_STAGE_BYTES);
            for (int k = 0; k < mma_per_kb; ++k) {
                tc_mma<KIND>(tmem_base, make_smem_desc(a_addr + 32 * k, p.slab_bytes),
                             make_smem_desc(b_addr + 32 * k, p.slab_bytes), idesc, (uint32_t)((kb | k) != 0));
            }
            tc_commit(empty0 + 8 * s);   // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(accum_bar);    // accumulator complete
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int te = threadIdx.x - 64;   // 0..127
        for (int i = te; i < BN; i += 128) {
            const int n = n0 + i;
            float b = 0.f, c = 0.f;
            if (n < p.N) {
                if (p.bias_mode == BIAS_F32) b = reinterpret_cast<const float *>(p.bias)[n];
                else if (p.bias_mode == BIAS_S32_DEQUANT && p.bias)
                    b = __int2float_rn(reinterpret_cast<const int *>(p.bias)[n]);
                if (p.coeff) c = p.coeff[n];
            }
            s_bias[i] = b;
            s_coeff[i] = c;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");

        const int quarter = warp & 3;               // TMEM lane quarter this warp may read
        const int row = m0 + quarter * 32 + lane;   // output row (pixel) of this thread
        const bool row_ok = row < p.M;
        const bool got = mbar_wait(accum_bar, 0, abort_flag);
        if (!got) {
            if (lane == 0) atomicOr(p.status, ST_TIMEOUT_EPILOGUE);
        } else {
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const bool vec_ok = (p.ldo % 4 == 0) && (n0 % 4 == 0);
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= p.N) break;
                uint32_t r[32];
                tmem_ld_32x32(taddr + c0, r);
                tmem_ld_wait();
                if (!row_ok) continue;
                const long long obase = (long long)bz * p.out_batch_stride + (long long)row * p.ldo + n0 + c0;
                const int ncols = min(32, p.N - (n0 + c0));

                if (p.out_mode == OUT_RAW32) {
                    uint32_t *o = reinterpret_cast<uint32_t *>(p.out) + obase;
                    _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) o[j] = r[j];
                    continue;
                }
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float x;
                    if constexpr (KIND == KIND_I8) {
                        // (float)acc * input_scale; += (float)bias_s32; *= weight_aux/127
                        x = __fmul_rn(__int2float_rn((int)r[j]), p.in_scale);
                        if (p.bias_mode == BIAS_S32_DEQUANT && p.bias) x = __fadd_rn(x, s_bias[c0 + j]);
                        x = __fmul_rn(x, s_coeff[c0 + j]);
                    } else {
                        x = __uint_as_float(r[j]);
                        if (p.bias_mode == BIAS_F32) x = __fadd_rn(x, s_bias[c0 + j]);
                    }
                    v[j] = x;
                }
                if (p.act != 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act, p.act_p0, p.act_p1, p.lut);
                }
                if (p.residual) {
                    if (p.out_mode == OUT_BF16) {
                        const __nv_bfloat16 *rp = reinterpret_cast<const __nv_bfloat16 *>(p.residual) + obase;
                        _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) v[j] = __fadd_rn(v[j], __bfloat162float(rp[j]));
                    } else {
                        const float *rp = reinterpret_cast<const float *>(p.residual) + obase;
                        if (vec_ok && ncols == 32) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 t = *reinterpret_cast<const float4 *>(rp + j);
                                v[j] = __fadd_rn(v[j], t.x);
                                v[j + 1] = __fadd_rn(v[j + 1], t.y);
                                v[j + 2] = __fadd_rn(v[j + 2], t.z);
                                v[j + 3] = __fadd_rn(v[j + 3], t.w);
                            }
                        } else {
                            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) v[j] = __fadd_rn(v[j], rp[j]);
                        }
                    }
                    if (p.res_relu) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
                    }
                }
                if (p.out_q) {
                    int8_t *q = p.out_q + obase;
                    if ((p.ldo % 16 == 0) && (n0 % 16 == 0) && ncols == 32) {
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint32_t b0 = (uint32_t)quant_s8(v[4 * j], p.q_inv_scale) & 0xff;
                            uint32_t b1 = (uint32_t)quant_s8(v[4 * j + 1], p.q_inv_scale) & 0xff;
                            uint32_t b2 = (uint32_t)quant_s8(v[4 * j + 2], p.q_inv_scale) & 0xff;
                            uint32_t b3 = (uint32_t)quant_s8(v[4 * j + 3], p.q_inv_scale) & 0xff;
                            w[j] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
                        }
                        reinterpret_cast<uint4 *>(q)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        reinterpret_cast<uint4 *>(q)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
                        _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) q[j] = (int8_t)quant_s8(v[j], p.q_inv_scale);
                    }
                }
                if (p.out == nullptr) continue;
                if (p.out_mode == OUT_BF16) {
                    __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + obase;
                    if ((p.ldo % 8 == 0) && (n0 % 8 == 0) && ncols == 32) {
                        uint32_t w[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            w[j] = *reinterpret_cast<uint32_t *>(&t);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            reinterpret_cast<uint4 *>(o)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                    } else {
                        _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) o[j] = __float2bfloat16_rn(v[j]);
                    }
                } else {
                    if (p.round_tf32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = round_to_tf32(v[j]);
                    }
                    float *o = reinterpret_cast<float *>(p.out) + obase;
                    if (vec_ok && ncols == 32) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4 *>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
                        _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) o[j] = v[j];
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        // A role gave up.  Before the CTA exits, wait (bounded) for the loads that were issued so
        // that no copy lands in shared memory after the block has gone.
        int dummy = 0;
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int kb = first; kb < issued; ++kb) {
            if (!mbar_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1, &dummy)) {
                atomicOr(p.status, ST_TIMEOUT_DRAIN);
                break;
            }
        }
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, BN);
    }
}

template <int KIND, int BN>
static cudaError_t launch_one(const CUtensorMap &tmA, const CUtensorMap &tmB, const IgemmParams &p,
                              cudaStream_t stream)
{
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    const size_t smem = igemm_smem_bytes(BN);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(igemm_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const long long m_tiles = (p.M + TILE_M - 1) / TILE_M;
    const long long n_tiles = (p.N + BN - 1) / BN;
    const long long grid = m_tiles * n_tiles;
    if (grid <= 0 || grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    igemm_kernel<KIND, BN><<<dim3((unsigned)grid, p.batched ? (unsigned)p.batch : 1u), NUM_THREADS, smem, stream>>>(tmA, tmB, p);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_igemm(int kind, int bn, const CUtensorMap &tmA, const CUtensorMap &tmB,
                         const IgemmParams &p, cudaStream_t stream)
{
#define ONE_DISPATCH(K)                                                       \
    switch (bn) {                                                             \
    case 64: return launch_one<K, 64>(tmA, tmB, p, stream);                   \
    case 128: return launch_one<K, 128>(tmA, tmB, p, stream);                 \
    case 256: return launch_one<K, 256>(tmA, tmB, p, stream);                 \
    default: return cudaErrorInvalidValue;                                    \
    }
    if (kind == KIND_TF32) { ONE_DISPATCH(KIND_TF32) }
    if (kind == KIND_BF16) { ONE_DISPATCH(KIND_BF16) }
    if (kind == KIND_I8) { ONE_DISPATCH(KIND_I8) }
#undef ONE_DISPATCH
    return cudaErrorInvalidValue;
}

}  // namespace one
