/*
 * one_cuda.h -- C ABI of the B200 (sm_100a) backend for the Conv / Gemm / MatMul operators of
 * the oneNew runtime.
 *
 * Two ways in:
 *
 * 1. Drop-in operator libraries.  libConv_cu.so, libGemm_cu.so and libMatMul_cu.so each export
 *        int eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs);
 *    the symbol the reference host resolves with dlsym (host/op.h:13, :41-80) and the shape the
 *    reference's own CUDA operators have (device/cuda/MaxPool/maxpool.cu:83-86).  They forward
 *    to one_cuda_conv_eval / one_cuda_gemm_eval / one_cuda_matmul_eval below.  `params` holds
 *    HOST pointers to the descriptors of include/one_abi.h, `inputs` / `outputs` hold DEVICE
 *    pointers to fp32 tensors in the reference's layouts (NCHW activations, OIHW weights).
 *    The call runs on the calling thread's current device and returns after the result is
 *    complete, like the reference's CUDA operators (maxpool.cu:76).
 *
 * 2. Prepared operators for a device-resident graph runtime: one_cuda_init ->
 *    one_cuda_prepare (upload + re-order the weights once) -> one_cuda_eval_async (enqueue only,
 *    same three-array calling convention) -> one_cuda_status.
 *
 * Unlike the reference, whose operators always return 0 and abort through LOG_ERR
 * (common/log.h:25-32), every entry point returns 0 or a negative ONE_ERR_* code and never
 * aborts; one_cuda_last_error() gives the text.  There is no CPU fallback: without a usable
 * CUDA device every call fails with ONE_ERR_CUDA.
 */
#ifndef ONE_CUDA_H
#define ONE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#include "one_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#define ONE_API __attribute__((visibility("default")))

#define ONE_OK 0
#define ONE_ERR_BAD_ARG (-1)      /* null pointer, bad handle                         */
#define ONE_ERR_BAD_SHAPE (-2)    /* descriptor shapes inconsistent with the config   */
#define ONE_ERR_UNSUPPORTED (-3)  /* e.g. grouped convolution                          */
#define ONE_ERR_CUDA (-4)         /* a CUDA runtime / driver call failed              */
#define ONE_ERR_NOMEM (-5)        /* workspace too small for this call                */
#define ONE_ERR_TIMEOUT (-6)      /* a bounded device-side wait ran out               */
#define ONE_ERR_RANGE (-7)        /* ONE_PREC_F16: a value exceeded the fp16 range     */

/* precision / layout flags of one_cuda_prepare */
#define ONE_PREC_TF32 0x0     /* fp32 storage, tf32 tensor-core products, fp32 accumulate   */
#define ONE_PREC_BF16 0x1     /* bf16 operands and activations, fp32 accumulate             */
#define ONE_PREC_F16 0x2      /* fp16 operands and activations, fp32 accumulate: the 10-bit mantissa of
                                 tf32 in half the bytes.  Magnitudes above 65504 become infinity and are
                                 reported: one_cuda_status() then returns ONE_ERR_RANGE (run that model
                                 with ONE_PREC_TF32); magnitudes below 2^-14 lose mantissa bits            */
#define ONE_PREC_MASK 0xF
#define ONE_LAYOUT_NHWC 0x10  /* x, y and residual are NHWC in the activation type of the
                                 precision (fp32, bf16 or fp16); without it: NCHW fp32       */
#define ONE_OUT_F32 0x20      /* with ONE_PREC_BF16 / ONE_PREC_F16: write y as fp32 (network outputs) */
#define ONE_IN_S8 0x40        /* int8 conv: x already holds the quantised NHWC int8 input   */
#define ONE_FUSE_ADD_RELU 0x80 /* conv: y = relu(act(conv) + residual); residual pointer in
                                  inputs[ONE_SLOT_RESIDUAL]                                  */
#define ONE_FUSE_ADD 0x100    /* conv: y = act(conv) + residual                             */
#define ONE_FUSE_GELU 0x400   /* Gemm / MatMul: table Gelu (inputs[11] at prepare) after the bias;
                                 ONE_FUSE_ADD then adds inputs[ONE_SLOT_RESIDUAL] after it; a MatMul
                                 takes an optional bias (the folded Add of a constant vector) in inputs[2] */
#define ONE_OUT_BF16 0x800    /* with ONE_PREC_TF32 and ONE_LAYOUT_NHWC: write y as bf16 (fp32 input, bf16 consumer) */
#define ONE_IN_NCHW_F32 0x200  /* with ONE_LAYOUT_NHWC: x alone is still NCHW fp32 (network input) */
#define ONE_SLOT_RESIDUAL 10
#define ONE_SLOT_OUT_Q 1      /* outputs[1]: optional int8 NHWC copy of y for an int8 consumer */

typedef struct one_ctx one_ctx;       /* per-device context: stream, workspace, status word */
typedef struct one_packed one_packed; /* a prepared operator: re-ordered weights + launch plan */

/* Create the context of `device` with a scratch workspace of `workspace_bytes` (0 = 256 MiB).
 * The only allocating calls are this one and one_cuda_prepare. */
ONE_API int one_cuda_init(int device, size_t workspace_bytes, one_ctx **out);
ONE_API int one_cuda_release(one_ctx *ctx);
/* Stream the context's own work is enqueued on (a cudaStream_t). */
ONE_API void *one_cuda_stream(one_ctx *ctx);
/* Synchronise the context's stream and return the device status word translated to 0 or
 * ONE_ERR_TIMEOUT / ONE_ERR_CUDA; the word is cleared. */
ONE_API int one_cuda_status(one_ctx *ctx);
ONE_API const char *one_cuda_last_error(void);
/* Number of kernels this library has launched in this process so far. */
ONE_API unsigned long long one_cuda_launch_count(void);

/* Drop-in operators (replace device/x86/Conv/conv.c:13-66, device/x86/Gemm/gemm.c:9-79,
 * device/x86/MatMul/mat_mul.c:10-101).  Slot layout of the arrays: host/op.h:109-168,
 * host/ops/conv.h:65-68, :133-157, host/ops/gemm.h:108-126, host/ops/mat_mul.h:109-121. */
ONE_API int one_cuda_conv_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs);
ONE_API int one_cuda_gemm_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs);
ONE_API int one_cuda_matmul_eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs);
/* Conv for callers that must not allocate device memory.  It has no counterpart in the reference.
 * Same arrays and result as one_cuda_conv_eval, but all of its scratch comes out of one fixed array
 * of ONE_STATIC_SCRATCH_BYTES built into the library image (each GPU that loads the library holds
 * it until the process exits); the call performs no cudaMalloc / cudaFree and no other allocation.
 * Meant for hosts that gave their device memory to an arena of their own at start-up, that run
 * under a latency budget a device allocation would break, or that embed the library where the
 * allocator is not theirs to call.  Shapes whose scratch exceeds the array are refused with
 * ONE_ERR_NOMEM before anything is launched.  The work is enqueued on `stream` (a cudaStream_t, NULL =
 * default stream); the call synchronises `stream` before it returns, so the result is complete then.
 * The first call on a device also looks up the array's device address (cudaGetSymbolAddress): make that
 * first call before any stream capture is begun.  The array is shared by every call and keeps its old
 * contents (the status word is cleared per call, the rest is overwritten before use).  Two calls on
 * one device must therefore not overlap in either sense: on the GPU (different streams) they would
 * overwrite each other's scratch, and on the host (two threads) they would race on the bump offset
 * that hands the array out.  Serialise them, e.g. one calling thread per device. */
#define ONE_STATIC_SCRATCH_BYTES (32u << 20)
ONE_API int one_cuda_conv_eval_static(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs, void *stream);
/* Precision of the float path of the three calls above on this thread: ONE_PREC_TF32
 * (default) or ONE_PREC_BF16. */
ONE_API int one_cuda_set_eval_precision(int prec);

/* Prepared path.  op_type is "Conv", "Gemm" or "MatMul".  At prepare time inputs[1] / inputs[2]
 * are HOST pointers to the weight / bias exactly as the reference's fill_operands leaves them
 * (host/ops/conv.h:60-157: fp32 OIHW, or for a quantised Conv the int8 weights and int32 bias
 * at the start of those buffers); inputs[11] is the host SiLU table for a SILU conv
 * (host/ops/conv.h:178-194).  They are uploaded and re-ordered once. */
ONE_API int one_cuda_prepare(one_ctx *ctx, const char *op_type, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs,
                     int flags, one_packed **out);
/* Enqueue one evaluation on `stream` (cudaStream_t, NULL = the context's stream).  Activation
 * pointers in inputs[0] / outputs[0] are device pointers; the batch is read from
 * params[1]'s shapes[0], so one prepared operator serves any batch. */
ONE_API int one_cuda_eval_async(one_ctx *ctx, one_packed *op, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs,
                        BUFFER_INFO_S *outputs, void *stream);
ONE_API int one_cuda_packed_release(one_packed *op);
/* MatMul of two device-resident tensors (neither is a constant, so there is nothing to prepare):
 * the stream-ordered form of one_cuda_matmul_eval, same arrays (device/x86/MatMul/mat_mul.c:17-98).
 * `flags` = ONE_PREC_*.  `flops` / `bytes` (optional) receive the work of the call. */
/* Fused multi-head self-attention over a token sequence of at most 256 tokens (head width 32 or
 * 64; anything else returns ONE_ERR_UNSUPPORTED), fp32 in memory, tf32 tensor cores.  No single counterpart in the reference: it stands
 * for the chain Gather/Reshape/Transpose (head split) -> Mul(scale) -> MatMul -> Softmax -> MatMul
 * -> Transpose/Reshape (head merge) the reference evaluates operator by operator
 * (device/x86/MatMul/mat_mul.c:17-98, Softmax/softmax.c:31-76, Transpose/transpose.c:27-75).
 *   qkv  [batch][T][row_floats]: q, k, v of head h start at column q_off / k_off / v_off + h*hd
 *        (each a multiple of 32);  out [batch][T][out_row_floats]: head h at column h*hd;
 *   out[b,t,h,:] = softmax_j(scale * q[b,t,h,:] . k[b,j,h,:]) applied to v[b,j,h,:]. */
ONE_API int one_cuda_attention(one_ctx *ctx, const float *qkv, float *out, int batch, int T, int heads, int hd,
                               int row_floats, int q_off, int k_off, int v_off, int out_row_floats, float scale,
                               void *stream);
ONE_API int one_cuda_matmul_async(one_ctx *ctx, BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs,
                                  int flags, void *stream, double *flops, double *bytes);
/* A prepared Conv can also write an int8 NHWC copy of its output, quantised for the next
 * quantised Conv exactly as that Conv would quantise it itself (x * (1/scale), clamp, roundf:
 * device/x86/Conv/conv.c:943-973).  Set the consumer's input_scale here and pass the int8
 * buffer in outputs[ONE_SLOT_OUT_Q]. */
ONE_API int one_cuda_packed_set_requant(one_packed *op, float next_input_scale);
/* FLOPs (2*MACs) and compulsory bytes of the last evaluation of a prepared operator, as the
 * reference counts them (host/ops/conv.h:159-176, gemm.h:128-145, mat_mul.h:125-142). */
ONE_API int one_cuda_packed_work(one_packed *op, double *flops, double *bytes);
/* Text describing the last evaluation of a prepared operator (GEMM view M, N, K, operand type, output
 * tile, split-K ranges) for per-operator performance tables. */
ONE_API int one_cuda_packed_detail(one_packed *op, char *buf, size_t cap);
/* Failure-detection self test.  Enqueues, on the context's stream, a one-warp kernel that waits on a
 * barrier nothing ever completes, gives up after `limit_clocks` GPU clocks (at most 2^31) and records
 * that in the status word the way a stalled pipeline role of the contraction kernel would.  The next
 * one_cuda_status(ctx) then returns ONE_ERR_TIMEOUT and clears the word; the context stays usable.
 * Nothing faults, traps or hangs. */
ONE_API int one_cuda_selftest_wait_timeout(one_ctx *ctx, unsigned long long limit_clocks);
/* Tile override for tuning: 0 = heuristic, else the output-tile width 64 / 128 / 192 / 256, or 1128 / 1192 /
 * 1256 = that width run as pairs of CTAs (a cluster of two SMs shares a 256-row tile, each CTA loading half
 * of the weight tile; not for batched products), or 2064 / 2128 = that width with two 128-row halves per CTA
 * tile (each weight tile brought into shared memory serves 256 output rows; no split-K), or 4064 / 4128 = that
 * width with twelve epilogue warps instead of eight (no split-K).  Every code gives
 * the same bits as the plain tile of its width.  Applies to the calling thread's drop-in calls and to the
 * operators it prepares. */
ONE_API int one_cuda_set_tile_n(int bn);
/* Split-K override for tuning, per calling thread: 0 = the library's choice (a contraction whose output
 * tiles would occupy at most half the SMs cuts its K range into several pieces, each piece accumulated
 * by its own CTA into a scratch plane, the planes added in a fixed order by a second short kernel that
 * also applies bias / activation / residual), 1 = never split, 2..64 = that many pieces when the shape
 * allows it.  Only the float paths split; results do not depend on scheduling. */
ONE_API int one_cuda_set_split_k(int splits);
/* The same choice for one prepared operator (0: follow the calling thread's setting); used by the tile search. */
ONE_API int one_cuda_packed_set_split(one_packed *op, int splits);
/* Process-wide switch (default on) for launching the contraction kernels with programmatic stream
 * serialisation: a kernel may be scheduled while the previous kernel on its stream drains, runs its
 * set-up (barriers, tensor memory, descriptor prefetch) and then waits on the device until that
 * previous kernel has completed before it touches any tensor. */
ONE_API int one_cuda_set_launch_overlap(int on);
/* Per calling thread (default on), read when an operator is prepared: a stride-1 multi-tap convolution with
 * at most 64 output channels on device-resident NHWC tensors is evaluated on pairs of horizontally adjacent
 * output pixels (a KH x (KW + 1) filter, stride 2 along w, twice the output channels, zero taps where a
 * pixel does not reach), which gives the tensor core a full-width tile.  Every output sums the same
 * products plus exact zeros; only their grouping inside the tensor core changes, so results agree with the
 * unpaired evaluation to rounding (an infinite input next to a zero tap gives NaN instead). */
ONE_API int one_cuda_set_width_pairing(int on);
/* Process-wide switch (default on) for the tile codes 1128 / 1192 / 1256: when off, one_cuda_set_tile_n refuses
 * them (ONE_ERR_UNSUPPORTED) and the tile search therefore never picks a pair-of-CTAs launch. */
ONE_API int one_cuda_set_cta_pairs(int on);
/* The same switch (default on) for the tile codes 2064 / 2128 (two 128-row halves per CTA). */
ONE_API int one_cuda_set_half_tiles(int on);
/* The same switch (default on) for the tile codes 4064 / 4128 (twelve epilogue warps in three groups behind a
 * shallower operand ring: for layers whose time is their epilogue). */
ONE_API int one_cuda_set_wide_epilogue(int on);
/* Process-wide tuning switch for the contraction kernel's epilogue (default 15): bit 0 lets both epilogue
 * warp groups drain the same accumulator when a CTA has a single tile, bit 1 gives every epilogue warp a
 * second output patch so that a chunk is formed while the previous chunk's store is still in flight, bit 2
 * hands an accumulator back to the MMA issuer as soon as a warp's last load of the tile is in registers, bit 3
 * lets a 16-bit residual be added by the tensor core (the residual tensor as further operand stages times an
 * identity tile) instead of by the epilogue.  Bits 0-2 change no result; bit 3 adds the residual before the
 * bias instead of after it (the same fp32 terms in another order: the last bit may differ). */
ONE_API int one_cuda_set_epilogue_mode(int bits);

#ifdef __cplusplus
}
#endif
#endif /* ONE_CUDA_H */
