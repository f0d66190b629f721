/* shim.c -- body of lib<Op>_cu.so: exports the `eval` symbol the reference host resolves with
 * dlsym (host/op.h:13, :58-76; same shape as device/cuda/MaxPool/maxpool.cu:83-86) and forwards
 * to the operator's entry point in libone_b200.so.  ONE_SHIM_TARGET is set per library by the
 * Makefile (one_cuda_conv_eval, one_cuda_gemm_eval, one_cuda_matmul_eval). */
#include "one_cuda.h"

__attribute__((visibility("default"))) int eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs,
                                                BUFFER_INFO_S *outputs)
{
    return ONE_SHIM_TARGET(params, inputs, outputs);
}
