/*
 * one_net.h -- C ABI of the device-resident graph runtime for .one models.
 *
 * It plays the role of the reference's net / extractor pair (host/net.h:223-235, :378-397,
 * :613-641) for a GPU: load a .one image, order the operators, infer shapes, place every operand
 * in device memory, and run the whole graph stream-ordered with the Conv / Gemm / MatMul
 * operators resolved to the sm_100a backend of one_cuda.h.  One one_net serves one device and one
 * batch size; a one_net_group (end of this file) shards a batch over several GPUs of the box by
 * giving each device its own one_net and a contiguous slice of the images (no data is exchanged).
 */
#ifndef ONE_NET_H
#define ONE_NET_H

#include "one_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct one_net one_net;

#define ONE_NET_NO_FUSE 0x1000   /* keep Conv -> Add -> Relu as three operators          */
#define ONE_NET_NO_GRAPH 0x2000  /* enqueue operator by operator instead of a CUDA graph */

/* Build the runtime for the .one image at `path` (or in memory) on `device` for `batch` images
 * per run.  `flags`: ONE_PREC_TF32 or ONE_PREC_BF16, optionally ONE_NET_NO_FUSE /
 * ONE_NET_NO_GRAPH.  `workspace_bytes` sizes the scratch of the contractions (0 = default). */
ONE_API int one_net_create(const char *path, int device, int batch, int flags, size_t workspace_bytes, one_net **out);
ONE_API int one_net_create_from_memory(const void *image, size_t size, int device, int batch, int flags,
                                       size_t workspace_bytes, one_net **out);
ONE_API void one_net_destroy(one_net *net);
/* Planning only, no GPU needed: the steps the runtime would execute for this image (operators in
 * execution order after the Conv->Add->Relu folding, the physical layout / type of every output,
 * inserted conversions), one text line per step, into buf. */
ONE_API int one_net_describe(const void *image, size_t size, int batch, int flags, char *buf, size_t cap);
ONE_API const char *one_net_last_error(void);

/* Network inputs / outputs, in the order of the image's io records.  Shapes are the logical
 * (reference) shapes with the batch in dim 0; device buffers are fp32 in the reference layout. */
ONE_API int one_net_io_count(one_net *net, int is_output);
ONE_API int one_net_io_info(one_net *net, int is_output, int index, char *name256, int *shape8, int *ndim);
ONE_API void *one_net_io_ptr(one_net *net, int is_output, int index);
ONE_API void *one_net_stream(one_net *net);

/* One inference over device-resident inputs: enqueue only.  one_net_sync waits and returns the
 * device status (0, ONE_ERR_TIMEOUT, ONE_ERR_CUDA). */
ONE_API int one_net_run(one_net *net);
ONE_API int one_net_sync(one_net *net);
/* End to end from host memory: copy `host_in` (input 0) to the device, run, copy output 0 to
 * `host_out`, wait.  Pinned host buffers make the copies asynchronous. */
ONE_API int one_net_run_host(one_net *net, const float *host_in, float *host_out);
/* Pipelined form of one_net_run_host: enqueue and return.  The host->device copy of this batch goes
 * through a staging buffer on a second stream, so it overlaps the previous batch's inference; the
 * output copy follows the inference on the net's stream.  host_in must stay untouched and host_out
 * unread until one_net_sync().  Pinned host memory is required for the overlap. */
ONE_API int one_net_submit_host(one_net *net, const float *host_in, float *host_out);
/* Copy any operand, converted to the reference layout in fp32, to the host (per-layer parity). */
ONE_API int one_net_fetch(one_net *net, const char *operand, float *host, size_t capacity_elems);
/* Device view of any operand the runtime materialises (valid after a run): pointer, element count,
 * element type (0 fp32, 1 bf16, 2 int8) and layout (0 reference, 1 NHWC).  Used by calibration. */
ONE_API int one_net_operand_ptr(one_net *net, const char *operand, void **dev, long long *elems, int *dtype, int *layout);
/* Names of every operand the runtime materialises, '\n' separated, into buf. */
ONE_API int one_net_operands(one_net *net, char *buf, size_t cap);
/* Per-operator timing (CUDA events) written as the reference's tracing CSV (host/net.h:539-611): the
 * twelve columns op_name,op_type,op_st,op_ed,op_computation,,cpu,cpu_hw_info,gpu,gpu_hw_info,
 * hw_computing_power (GOPS),model name -- microseconds and MFLOP, the hardware / model fields on the
 * first data row, where tools/perf_profiling/gen_timeline_json.py:41-42 reads them -- followed by two
 * columns that tool ignores: op_bytes (compulsory bytes) and op_detail (GEMM view, tile, split).
 * one_net_trace_ex names the model and the peak the tool's efficiency figures divide by (GOPS; <= 0:
 * the nominal dense tensor peak of the network's precision). */
ONE_API int one_net_trace(one_net *net, const char *csv_path, int runs);
ONE_API int one_net_trace_ex(one_net *net, const char *csv_path, int runs, const char *model_name, double hw_gops);
/* The CSV writer on its own (host only, no GPU): n rows of name, type, start / end in microseconds,
 * MFLOP, bytes (may be NULL) and detail (may be NULL). */
ONE_API int one_net_write_timeline_csv(const char *csv_path, int n, const char *const *op_name, const char *const *op_type,
                                       const double *st_us, const double *ed_us, const double *mflop, const double *bytes,
                                       const char *const *detail, const char *gpu, const char *gpu_hw_info, double hw_gops,
                                       const char *model_name);
/* Tile search on the model's own operators (the device counterpart of tools/optimize/auto_tuning.hpp:9-75):
 * every Conv / Gemm / MatMul with a constant weight is timed at each output-tile width of the contraction
 * kernel on the operands of the last inference (one run must have happened) and left prepared with the
 * fastest; a candidate replaces the best so far only when it is 2 % faster, the library's own choice going
 * first.  For short launches a few split-K choices are timed per width as well.  `report` (may be NULL)
 * receives CSV: op_name,op_type,out_width,heuristic_us,best_tile_n,best_us,best_split_k. */
ONE_API int one_net_autotune(one_net *net, int runs, char *report, size_t cap);
/* Force one operator's tile (0 = heuristic, 64, 128, 192, 256, 1128 / 1192 / 1256 for pairs of CTAs, 2064 / 2128 for
 * two 128-row halves per CTA, 4064 / 4128 for twelve epilogue warps), e.g. to replay a saved tuning.  A model
 * whose header carries one of those widths in cuda_gemm_tile_n (common/nn_common.h:36-38) starts with it. */
ONE_API int one_net_set_tile(one_net *net, const char *op_name, int tile_n);
/* Work of one run: FLOPs of Conv/Gemm/MatMul as the reference counts them, compulsory bytes of
 * every operator, and kernels launched per run. */
ONE_API int one_net_work(one_net *net, double *flops, double *bytes, unsigned long long *launches);

/* The 8192-entry activation tables the runtime builds for its operators, as the reference host builds them
 * (kind 0: SiLU, host/ops/conv.h:178-194; kind 1: Gelu, host/ops/gelu.h:80-96).  Host arithmetic. */
ONE_API int one_net_activation_table(int kind, float *out8192);

/* ---- one process, several GPUs --------------------------------------------------------------------------
 * A group runs one model on several devices of the box from a single calling thread, the shape of the
 * reference's caller (host/net.h:613-628: load a model, call inference).  The batch of a call is cut into
 * n_devices contiguous shards of batch / n_devices images (shard i goes to devices[i]); every device has
 * its own replica of the network (weights, arena, stream, captured graph) driven by its own host thread.
 * Images are independent, so the shards exchange nothing: no collective, no peer access.
 * Errors: a device index outside [0, visible devices) or listed twice, or a batch that does not divide by
 * n_devices, returns ONE_ERR_BAD_ARG before anything is created or launched. */
typedef struct one_net_group one_net_group;
ONE_API int one_net_group_create(const char *path, const int *devices, int n_devices, int batch, int flags,
                                 size_t workspace_bytes, one_net_group **out);
ONE_API int one_net_group_create_from_memory(const void *image, size_t size, const int *devices, int n_devices, int batch,
                                             int flags, size_t workspace_bytes, one_net_group **out);
ONE_API void one_net_group_destroy(one_net_group *group);
ONE_API int one_net_group_size(one_net_group *group);
/* The partition rule on its own (host arithmetic): shard `index` of n_devices takes images
 * [first, first + count) = [index * batch / n, (index + 1) * batch / n). */
ONE_API int one_net_group_partition(int batch, int n_devices, int index, int *first, int *count);
/* Shard `index`: its device and the images [first, first + count) of the batch it runs. */
ONE_API int one_net_group_shard(one_net_group *group, int index, int *device, int *first, int *count);
/* The replica that runs shard `index` (for one_net_autotune / one_net_trace / one_net_work on it). */
ONE_API one_net *one_net_group_member(one_net_group *group, int index);
/* One inference over a whole batch in host memory (input 0, [batch][...] fp32; output 0 to host_out):
 * every shard is handed to its device's thread, which runs one_net_submit_host on its slice.  Returns at
 * once; host_in must stay untouched and host_out unread until one_net_group_sync(), which waits for every
 * device and returns the first error any shard met since the last sync (with its device in the text). */
ONE_API int one_net_group_submit_host(one_net_group *group, const float *host_in, float *host_out);
ONE_API int one_net_group_sync(one_net_group *group);
/* Failure-path testing without touching a GPU: `hook` (NULL removes it) is called on the device's host
 * thread before each shard is submitted; a non-zero return is taken as that shard's error and nothing is
 * launched for it. */
ONE_API int one_net_group_set_fault_hook(one_net_group *group, int (*hook)(int device));

#ifdef __cplusplus
}
#endif
#endif /* ONE_NET_H */
