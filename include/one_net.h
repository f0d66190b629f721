/*
 * one_net.h -- C ABI of the device-resident graph runtime for .one models.
 *
 * It plays the role of the reference's net / extractor pair (host/net.h:223-235, :378-397,
 * :613-641) for a GPU: load a .one image, order the operators, infer shapes, place every operand
 * in device memory, and run the whole graph stream-ordered with the Conv / Gemm / MatMul
 * operators resolved to the sm_100a backend of one_cuda.h.  One object serves one device and one
 * batch size; a batch is sharded over several GPUs by creating one object per device and giving
 * each a contiguous slice of the images (no data is exchanged between them).
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
 * first.  `report` (may be NULL) receives CSV: op_name,op_type,out_width,heuristic_us,best_tile_n,best_us. */
ONE_API int one_net_autotune(one_net *net, int runs, char *report, size_t cap);
/* Force one operator's tile width (0 = heuristic, 64, 128, 192, 256), e.g. to replay a saved tuning.  A model
 * whose header carries one of those widths in cuda_gemm_tile_n (common/nn_common.h:36-38) starts with it. */
ONE_API int one_net_set_tile(one_net *net, const char *op_name, int tile_n);
/* Work of one run: FLOPs of Conv/Gemm/MatMul as the reference counts them, compulsory bytes of
 * every operator, and kernels launched per run. */
ONE_API int one_net_work(one_net *net, double *flops, double *bytes, unsigned long long *launches);

#ifdef __cplusplus
}
#endif
#endif /* ONE_NET_H */
