/*
 * one_abi.h -- binary layout of the structures that cross the operator plug-in
 * boundary of the oneNew runtime.
 *
 * An operator library exports
 *     int eval(BUFFER_INFO_S *params, BUFFER_INFO_S *inputs, BUFFER_INFO_S *outputs);
 * and receives, through `params`, pointers to the structures declared here.  The
 * field order, widths and padding must therefore be bit-identical to the
 * reference declarations (common/nn_common.h:28-82 for the model header and
 * buffer records, :90-137 for the enums, :145-182 for OPERAND_S / BASE_CONFIG_S,
 * :222-243 for CONV_CONFIG_S, :312-320 GEMM_CONFIG_S, :366-369 MATMUL_CONFIG_S,
 * :371-379 MAX_POOL_CONFIG_S).  Only the records used by the Conv / MatMul / Gemm
 * path and the glue operators of ResNet-50 / ViT-Tiny are declared.  The
 * static assertions at the end pin every offset an operator reads.
 */
#ifndef ONE_ABI_H
#define ONE_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#define ONE_STATIC_ASSERT(c, m) static_assert(c, m)
#else
#define ONE_STATIC_ASSERT(c, m) _Static_assert(c, m)
#endif

/* file magic of a .one image: the bytes 'o','n','e' (common/nn_common.h:17) */
#define ONE_MAGIC_NUM 0x6F6E65
#define EPSILON (1e-20)

#define BUF_MAXNUM 12        /* slots in every params/inputs/outputs array   */
#define OPERAND_MAXNUM 8     /* operands an op record can name               */
#define SHAPE_LEN 8
#define OP_TYPE_LEN 256
#define OP_NAME_LEN 256
#define OPERAND_NAME_LEN 256
#define ONE_WEIGHT_AUX_LEN 4096   /* per-output-channel |w|max table of a Conv */

/* GEMM tile hints carried in the model header (x86 and cuda triples). */
typedef struct {
    int32_t x86_gemm_single_threads_tile_m, x86_gemm_single_threads_tile_n, x86_gemm_single_threads_tile_k;
    int32_t x86_gemm_multi_threads_tile_m, x86_gemm_multi_threads_tile_n, x86_gemm_multi_threads_tile_k;
    int32_t cuda_gemm_tile_m, cuda_gemm_tile_n, cuda_gemm_tile_k;
} BLOCK_INFO_S;

/* The shared scratch ("public") buffer every op may bump-allocate from. */
typedef struct {
    int64_t public_buf_size;
    int64_t public_buf_ptr;
} PUBLIC_BUF_INFO_S;

typedef struct {
    int64_t kv_cache_buf_size, kv_cache_buf_ptr, prompts_amount, max_token_supported, cur_token_index;
} KV_CACHE_INFO_S;

typedef struct {
    int32_t useful_info_magic_num;
    BLOCK_INFO_S block_info;
    PUBLIC_BUF_INFO_S public_buf_info;
    KV_CACHE_INFO_S kv_cache_info;
} USEFUL_INFO_S;

/* First record of a .one image. Offsets are from the start of the file. */
typedef struct {
    int32_t one_model_magic_num;
    int32_t version;
    int32_t node_cnt, node_cfg_offset;
    int32_t init_cnt, init_info_offset;
    int32_t io_cfg_cnt, io_cfg_offset;
    USEFUL_INFO_S useful_info;
} ONE_MODEL_DESC_S;

/* One slot of the params / inputs / outputs arrays; only `addr` is filled. */
typedef struct {
    int64_t addr;
    int32_t elem_size;
    int32_t buf_size;
} BUFFER_INFO_S;

typedef struct {
    BUFFER_INFO_S buf_info[BUF_MAXNUM];
} BUFFER_GROUP_S;

/* Element types use the ONNX numbering. */
typedef enum {
    TYPE_UNKNOWN = 0, TYPE_FP32 = 1, TYPE_UINT8 = 2, TYPE_INT8 = 3, TYPE_UINT16 = 4, TYPE_INT16 = 5,
    TYPE_INT32 = 6, TYPE_INT64 = 7, TYPE_STRING = 8, TYPE_BOOLEAN = 9, TYPE_FP16 = 10, TYPE_FP64 = 11,
    TYPE_UINT32 = 12, TYPE_UINT64 = 14, TYPE_COMPLEX128 = 15, TYPE_BF16 = 16,
} ELEM_TYPE_E;

typedef enum { FALSE = 0, TRUE = 1 } BOOL;

/* Activation fused behind a Conv. RELU6 is declared but no producer emits it. */
typedef enum {
    NOT_ACT = 0, RELU = 1, RELU6 = 2, SILU = 3, CLIP = 4, HARDSILU = 5, LEAKYRELU = 6,
} ACT_TYPE_E;

typedef struct {
    char op_type[OP_TYPE_LEN];
    char op_name[OP_NAME_LEN];
} NODE_INFO_S;

/* Tensor descriptor. shapes[] is padded with 1s; conv kernels read [0..3] = N,C,H,W. */
typedef struct {
    char operand_name[OPERAND_NAME_LEN];
    BOOL is_fixed_val;   /* initialiser (weight, bias, constant) */
    BOOL not_need_buf;   /* output aliases its input (Flatten, Reshape ...) */
    int64_t p_data;
    int32_t dim_num_of_shapes;
    int32_t shapes[SHAPE_LEN];
    ELEM_TYPE_E data_type;
} OPERAND_S;

typedef struct {
    char op_type[OP_TYPE_LEN];   /* "io" */
    char op_name[OP_NAME_LEN];   /* "input" or "output" */
    OPERAND_S operand;
} IO_CONFIG_S;

/* Common head of every operator record. */
typedef struct {
    char op_type[OP_TYPE_LEN];
    char op_name[OP_NAME_LEN];
    char in_operand_name[OPERAND_MAXNUM][OPERAND_NAME_LEN];
    char out_operand_name[OPERAND_MAXNUM][OPERAND_NAME_LEN];
    int32_t in_operand_num;
    int32_t out_operand_num;
    NODE_INFO_S producer[OPERAND_MAXNUM];
    NODE_INFO_S consumer[OPERAND_MAXNUM];
    int32_t producer_num;
    int32_t consumer_num;
    int32_t fusion_op_type;
    int64_t fusion_op_cnt_in_entire_net;
    int64_t cur_op_cnt_in_fusion_op;
} BASE_CONFIG_S;

typedef struct {
    BASE_CONFIG_S op_base_cfg;
    BOOL has_bias;
    int64_t dilations[2];        /* carried, ignored by every kernel            */
    int64_t group;
    int64_t kernel_shape[2];     /* KH, KW                                      */
    int64_t pads[4];             /* top, left, bottom, right                    */
    int64_t strides[4];          /* [0] = x (width) stride, [1] = y stride      */
    ACT_TYPE_E act_type;
    float clip_min, clip_max;
    float leaky_relu_alpha;
    float hard_sigmoid_alpha, hard_sigmoid_beta;
    ELEM_TYPE_E ifmap_quant2;    /* TYPE_INT8 selects the quantised path        */
    float input_scale;           /* activation threshold / 127                  */
    float output_scale;          /* never written, never read                   */
    float weight_aux[ONE_WEIGHT_AUX_LEN]; /* per-OC max|w| used to de-quantise  */
} CONV_CONFIG_S;

typedef struct {
    BASE_CONFIG_S op_base_cfg;
    BOOL has_bias;
    float alpha, beta;           /* carried, ignored */
    int64_t transB;              /* carried, ignored: W is always [N][K] */
} GEMM_CONFIG_S;

typedef struct { BASE_CONFIG_S op_base_cfg; } MATMUL_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } ADD_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } RELU_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } GLOBAL_AVGPOOL_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; int64_t axis; } FLATTEN_CONFIG_S;

typedef struct {
    BASE_CONFIG_S op_base_cfg;
    int64_t ceil_mode;
    int64_t kernel_shape[2];
    int64_t pads[4];
    int64_t strides[2];
} MAX_POOL_CONFIG_S;

/* ---- operators between the MatMul / Gemm calls of a transformer encoder (common/nn_common.h) ---- */
typedef struct { BASE_CONFIG_S op_base_cfg; } GELU_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } MUL_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } DIV_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; } SUB_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; int64_t axis; } CONCAT_CONFIG_S;
typedef struct {
    BASE_CONFIG_S op_base_cfg;
    int64_t axis;
    int64_t indices;             /* the fixed index when indices_from_ifmap is FALSE */
    BOOL indices_from_ifmap;
} GATHER_CONFIG_S;
typedef struct {
    BASE_CONFIG_S op_base_cfg;
    int32_t axes[8];             /* axes[0] == 1 selects the strided variant; otherwise the last axis */
    int32_t axes_num;
    int32_t keepdims;
} LAYERNORMALIZATION_CONFIG_S;
typedef struct {
    BASE_CONFIG_S op_base_cfg;
    int64_t allowzero;
    int64_t dst_shape[8];
    int64_t dst_shape_num;
} RESHAPE_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; int64_t dims; int64_t axis; } SOFTMAX_CONFIG_S;
typedef struct { BASE_CONFIG_S op_base_cfg; int64_t perm[8]; int64_t perm_num; } TRANSPOSE_CONFIG_S;

/* ---- layout pins (gcc 13, x86-64 values of the reference build) ---- */
ONE_STATIC_ASSERT(sizeof(BUFFER_INFO_S) == 16, "BUFFER_INFO_S");
ONE_STATIC_ASSERT(sizeof(OPERAND_S) == 312, "OPERAND_S size");
ONE_STATIC_ASSERT(offsetof(OPERAND_S, p_data) == 264, "OPERAND_S.p_data");
ONE_STATIC_ASSERT(offsetof(OPERAND_S, dim_num_of_shapes) == 272, "OPERAND_S.dim_num");
ONE_STATIC_ASSERT(offsetof(OPERAND_S, shapes) == 276, "OPERAND_S.shapes");
ONE_STATIC_ASSERT(offsetof(OPERAND_S, data_type) == 308, "OPERAND_S.data_type");
ONE_STATIC_ASSERT(sizeof(BASE_CONFIG_S) == 12840, "BASE_CONFIG_S size");
ONE_STATIC_ASSERT(offsetof(BASE_CONFIG_S, in_operand_num) == 4608, "BASE_CONFIG_S.in_operand_num");
ONE_STATIC_ASSERT(offsetof(BASE_CONFIG_S, producer) == 4616, "BASE_CONFIG_S.producer");
ONE_STATIC_ASSERT(offsetof(BASE_CONFIG_S, fusion_op_type) == 12816, "BASE_CONFIG_S.fusion_op_type");
ONE_STATIC_ASSERT(sizeof(CONV_CONFIG_S) == 29376, "CONV_CONFIG_S size");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, has_bias) == 12840, "CONV_CONFIG_S.has_bias");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, group) == 12864, "CONV_CONFIG_S.group");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, kernel_shape) == 12872, "CONV_CONFIG_S.kernel_shape");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, pads) == 12888, "CONV_CONFIG_S.pads");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, strides) == 12920, "CONV_CONFIG_S.strides");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, act_type) == 12952, "CONV_CONFIG_S.act_type");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, ifmap_quant2) == 12976, "CONV_CONFIG_S.ifmap_quant2");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, input_scale) == 12980, "CONV_CONFIG_S.input_scale");
ONE_STATIC_ASSERT(offsetof(CONV_CONFIG_S, weight_aux) == 12988, "CONV_CONFIG_S.weight_aux");
ONE_STATIC_ASSERT(sizeof(GEMM_CONFIG_S) == 12864, "GEMM_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(MATMUL_CONFIG_S) == 12840, "MATMUL_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(ONE_MODEL_DESC_S) == 128, "ONE_MODEL_DESC_S size");
ONE_STATIC_ASSERT(offsetof(ONE_MODEL_DESC_S, useful_info) == 32, "ONE_MODEL_DESC_S.useful_info");
ONE_STATIC_ASSERT(sizeof(USEFUL_INFO_S) == 96, "USEFUL_INFO_S size");
ONE_STATIC_ASSERT(offsetof(USEFUL_INFO_S, public_buf_info) == 40, "USEFUL_INFO_S.public_buf_info");
ONE_STATIC_ASSERT(sizeof(IO_CONFIG_S) == 824, "IO_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(CONCAT_CONFIG_S) == 12848, "CONCAT_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(GATHER_CONFIG_S) == 12864, "GATHER_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(LAYERNORMALIZATION_CONFIG_S) == 12880, "LAYERNORMALIZATION_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(RESHAPE_CONFIG_S) == 12920, "RESHAPE_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(SOFTMAX_CONFIG_S) == 12856, "SOFTMAX_CONFIG_S size");
ONE_STATIC_ASSERT(sizeof(TRANSPOSE_CONFIG_S) == 12912, "TRANSPOSE_CONFIG_S size");

#endif /* ONE_ABI_H */
