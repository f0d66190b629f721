// ops.h -- operator classes of the device-resident runtime: the three hot-path operators
// (Conv, Gemm, MatMul: mirrors of host/ops/conv.h, gemm.h, mat_mul.h) and the glue operators
// ResNet-50 needs between them (io, MaxPool, Add, Relu, GlobalAveragePool, Flatten).
#pragma once
#include <cmath>

#include "op.h"

namespace onenew {

inline const OneImage::Init *find_init(const OneImage &img, const std::string &name)
{
    auto it = img.inits.find(name);
    return it == img.inits.end() ? nullptr : &it->second;
}

// The Gelu table of host/ops/gelu.h:80-96: 8192 entries over [-8, 8), 1/sqrt(2) taken as 1/1.4142.
inline std::vector<float> build_gelu_lut()
{
    const float single_limit = 8.0f;
    const float step = 1.0 / 512;
    const int lut_len = (int)(2.0f * single_limit / step);
    std::vector<float> lut(lut_len);
    const float inv_sqrt2 = 1.0f / 1.4142f;
    for (int i = 0; i < lut_len; ++i) {
        const float x = i * step - single_limit;
        // the reference's header includes "math.h" (host/ops/gelu.h:5), so its erf(float) is the float
        // function and 1 + erf(...) a float sum; the product with x * 0.5 is formed in double
        const float one_plus_erf = 1 + erff(x * inv_sqrt2);
        lut[i] = (float)((double)x * 0.5 * (double)one_plus_erf);
    }
    return lut;
}

// The SiLU table of host/ops/conv.h:178-194.
inline std::vector<float> build_silu_lut()
{
    const float single_limit = 8.0f;
    const float step = 1.0 / 512;
    const int lut_len = (int)(2.0f * single_limit / step);
    std::vector<float> lut(lut_len);
    for (int i = 0; i < lut_len; ++i) {
        const float x = i * step - single_limit;
        lut[i] = x / (1 + expf(-x));
    }
    return lut;
}

// ---------------------------------------------------------------------------------- io
class io : public op {
public:
    IO_CONFIG_S io_cfg;
    static int create_instance(std::shared_ptr<op> &p, const char *cfg)
    {
        auto o = std::make_shared<io>();
        memcpy(&o->io_cfg, cfg, sizeof(IO_CONFIG_S));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &) override   // host/ops/io.h:49-72
    {
        op_type = io_cfg.op_type;
        op_name = io_cfg.op_name;
        if (op_name == "input") out_operands.push_back(io_cfg.operand.operand_name);
        else if (op_name == "output") in_operands.push_back(io_cfg.operand.operand_name);
        else return ONE_ERR_BAD_ARG;
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &) override { return ONE_OK; }
    int forward(one_ctx *, cudaStream_t) override { return ONE_OK; }
};
OP_REGISTER_GLOBAL(io, io::create_instance, sizeof(IO_CONFIG_S));

// ---------------------------------------------------------------------------------- Conv
class Conv : public op {
public:
    CONV_CONFIG_S conv_cfg;
    const OneImage::Init *weight = nullptr, *bias = nullptr;
    std::vector<float> lut;          // SiLU table, built as host/ops/conv.h:178-194 does
    USEFUL_INFO_S useful;
    one_packed *packed = nullptr;
    int flags = 0;
    bool fuse_relu = false;          // Relu after the folded Add (op::residual)
    bool tokens_out = false;         // the output operand is the [N][OH*OW][OC] token view (folded Reshape + Transpose)
    // int8 chain: the only reader of the output is an int8 Conv, so the epilogue writes the activation
    // already quantised with that reader's input_scale (conv.c:961-973 done at the producer) and no
    // fp32 copy exists; in_int8: this Conv's input is such an operand
    bool out_int8 = false, in_int8 = false;
    float out_q_scale = 0.f;
    OPERAND_S y_desc;                // the conv's own [N][OC][OH][OW] output descriptor
    double mflop = 0, bytes = 0;

    ~Conv() override { one_cuda_packed_release(packed); }
    bool tunable() const override { return conv_cfg.group == 1; }
    int out_width() const override { return weight ? weight->desc->shapes[0] : 0; }
    void drop_prepared() override { one_cuda_packed_release(packed); packed = nullptr; }
    int set_split() override { return packed ? one_cuda_packed_set_split(packed, split_k) : ONE_OK; }
    static int create_instance(std::shared_ptr<op> &p, const char *cfg)
    {
        auto o = std::make_shared<Conv>();
        memcpy(&o->conv_cfg, cfg, sizeof(CONV_CONFIG_S));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &img) override   // host/ops/conv.h:60-131
    {
        fill_names(&conv_cfg.op_base_cfg);
        useful = img.desc()->useful_info;
        if (in_operands.size() < 2) return ONE_ERR_BAD_ARG;
        weight = find_init(img, in_operands[1]);
        if (conv_cfg.has_bias && in_operands.size() >= 3) bias = find_init(img, in_operands[2]);
        if (!weight || (conv_cfg.has_bias && !bias)) return ONE_ERR_BAD_ARG;
        if (conv_cfg.act_type == SILU) lut = build_silu_lut();
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/conv.h:31-58
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        out.dim_num_of_shapes = 4;
        out.shapes[0] = in.shapes[0];   // the reference writes 1 here; the batch is honoured
        out.shapes[1] = weight->desc->shapes[0];
        out.shapes[2] = (in.shapes[2] + (int)conv_cfg.pads[0] + (int)conv_cfg.pads[2] - (int)conv_cfg.kernel_shape[0]) / (int)conv_cfg.strides[1] + 1;
        out.shapes[3] = (in.shapes[3] + (int)conv_cfg.pads[1] + (int)conv_cfg.pads[3] - (int)conv_cfg.kernel_shape[1]) / (int)conv_cfg.strides[0] + 1;
        out.data_type = TYPE_FP32;
        y_desc = out;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &opt, TensorInfo *out,
              std::vector<bool> *need_plain) override
    {
        if (conv_cfg.group != 1) {   // depthwise: CUDA-core kernel on the reference layout
            for (size_t i = 0; i < ins.size(); ++i) (*need_plain)[i] = ins[i]->layout != LAYOUT_PLAIN || ins[i]->dtype != DT_F32;
            out->layout = LAYOUT_PLAIN;
            out->dtype = DT_F32;
            return;
        }
        const int adt = conv_cfg.ifmap_quant2 == TYPE_INT8 ? DT_F32 : opt.act_dtype();
        // x: NHWC in the activation type (or already quantised), or the reference layout in fp32 (network input)
        // (bf16 mode: an fp32 NHWC input is the residual trunk; it is read as it is, with tf32 products)
        const bool ok_nhwc = ins[0]->layout == LAYOUT_NHWC && (ins[0]->dtype == adt || ins[0]->dtype == DT_F32 || (in_int8 && ins[0]->dtype == DT_S8));
        const bool ok_plain = ins[0]->layout == LAYOUT_PLAIN && ins[0]->dtype == DT_F32;
        (*need_plain)[0] = !(ok_nhwc || ok_plain);
        for (size_t i = 1; i < ins.size(); ++i)   // residual: same physical form as the output
            (*need_plain)[i] = false;
        // NHWC [N][OH][OW][OC] is the row-major [N][OH*OW][OC] token sequence
        out->layout = tokens_out ? LAYOUT_PLAIN : LAYOUT_NHWC;
        out->dtype = out_int8 ? DT_S8 : (keep_f32 ? DT_F32 : adt);
    }
    int prepare(one_ctx *ctx, const NetOptions &opt, const std::vector<const TensorInfo *> &ins,
                const TensorInfo &out) override
    {
        const bool int8 = conv_cfg.ifmap_quant2 == TYPE_INT8;
        // bf16 mode keeps the residual trunk in fp32: a conv that reads the trunk multiplies in tf32 (its
        // input is fp32 as it lies), a conv that writes the trunk stores fp32; everything inside a block
        // is bf16
        const bool trunk_in = opt.precision == ONE_PREC_BF16 && !int8 && ins[0]->layout == LAYOUT_NHWC && ins[0]->dtype == DT_F32;
        flags = ((int8 || trunk_in) ? ONE_PREC_TF32 : opt.precision) | ONE_LAYOUT_NHWC;
        if (!int8 && (opt.precision == ONE_PREC_BF16 || opt.precision == ONE_PREC_F16) && conv_cfg.group == 1) {
            if (trunk_in && out.dtype == DT_BF16) flags |= ONE_OUT_BF16;
            if (!trunk_in && out.dtype == DT_F32) flags |= ONE_OUT_F32;
        }
        if (conv_cfg.group != 1) flags = ONE_PREC_TF32;
        else if (ins[0]->layout == LAYOUT_PLAIN) flags |= ONE_IN_NCHW_F32;
        if (!residual.empty()) flags |= fuse_relu ? ONE_FUSE_ADD_RELU : ONE_FUSE_ADD;
        if (in_int8 && ins[0]->dtype == DT_S8) flags |= ONE_IN_S8;
        // descriptors and HOST weight pointers, in the reference's slots (host/ops/conv.h:133-157)
        BUFFER_INFO_S p[BUF_MAXNUM], in[BUF_MAXNUM];
        memset(p, 0, sizeof(p));
        memset(in, 0, sizeof(in));
        p[0].addr = (int64_t)&conv_cfg;
        p[1].addr = (int64_t)&ins[0]->desc;
        p[2].addr = (int64_t)weight->desc;
        if (conv_cfg.has_bias) p[3].addr = (int64_t)bias->desc;
        p[conv_cfg.has_bias ? 4 : 3].addr = (int64_t)&y_desc;
        p[BUF_MAXNUM - 1].addr = (int64_t)&useful;
        in[1].addr = (int64_t)weight->data;
        if (conv_cfg.has_bias) in[2].addr = (int64_t)bias->data;
        if (!lut.empty()) in[BUF_MAXNUM - 1].addr = (int64_t)lut.data();
        int rc = one_cuda_set_tile_n(tile_n);
        if (rc != ONE_OK) return rc;   // a tile this build / setting does not offer: the tuner moves on
        rc = one_cuda_prepare(ctx, "Conv", p, in, flags, &packed);
        one_cuda_set_tile_n(0);
        if (rc == ONE_OK && out_int8) rc = one_cuda_packed_set_requant(packed, out_q_scale);
        if (rc == ONE_OK) rc = one_cuda_packed_set_split(packed, split_k);
        return rc;
    }
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &) override
    {
        params_vec[0].addr = (int64_t)&conv_cfg;
        params_vec[1].addr = (int64_t)&t[in_operands[0]].desc;
        params_vec[2].addr = (int64_t)weight->desc;
        if (conv_cfg.has_bias) params_vec[3].addr = (int64_t)bias->desc;
        params_vec[conv_cfg.has_bias ? 4 : 3].addr = (int64_t)&y_desc;
        params_vec[BUF_MAXNUM - 1].addr = (int64_t)&useful;
        inputs_vec[0].addr = (int64_t)t[in_operands[0]].dev;
        if (!residual.empty()) inputs_vec[ONE_SLOT_RESIDUAL].addr = (int64_t)t[residual].dev;
        if (out_int8) {
            outputs_vec[0].addr = 0;
            outputs_vec[ONE_SLOT_OUT_Q].addr = (int64_t)t[out_operands[0]].dev;
        } else {
            outputs_vec[0].addr = (int64_t)t[out_operands[0]].dev;
        }
        return ONE_OK;
    }
    int forward(one_ctx *ctx, cudaStream_t s) override
    {
        int rc = one_cuda_eval_async(ctx, packed, params_vec.data(), inputs_vec.data(), outputs_vec.data(), s);
        if (rc == ONE_OK) {
            double f, b;
            one_cuda_packed_work(packed, &f, &b);
            mflop = f * 1e-6;
            bytes = b;
        }
        return rc;
    }
    double get_computation() override { return mflop; }   // host/ops/conv.h:159-176
    double get_bytes() override { return bytes; }
    std::string describe() override
    {
        char buf[192] = {0};
        if (packed) one_cuda_packed_detail(packed, buf, sizeof(buf));
        return buf;
    }
};
OP_REGISTER_GLOBAL(Conv, Conv::create_instance, sizeof(CONV_CONFIG_S));

// ---------------------------------------------------------------------------------- Gemm / MatMul
class GemmLike : public op {
public:
    bool is_gemm = true;
    GEMM_CONFIG_S gemm_cfg;        // MatMul uses the BASE_CONFIG_S head only
    const OneImage::Init *weight = nullptr, *bias = nullptr;
    // folded by the runtime's fusion pass: MatMul -> Add(constant vector) [-> Gelu] [-> Add(activation)]
    const OneImage::Init *fused_bias = nullptr;
    bool fuse_gelu = false;
    std::vector<float> gelu_lut;
    one_packed *packed = nullptr;
    int flags = 0, prec = ONE_PREC_TF32;
    double mflop = 0, bytes = 0;
    ~GemmLike() override { one_cuda_packed_release(packed); }
    bool tunable() const override { return weight != nullptr; }   // activation x activation products keep the heuristic
    int out_width() const override { return weight ? (is_gemm ? weight->desc->shapes[0] : weight->desc->shapes[weight->desc->dim_num_of_shapes - 1]) : 0; }
    void drop_prepared() override { one_cuda_packed_release(packed); packed = nullptr; }
    int set_split() override { return packed ? one_cuda_packed_set_split(packed, split_k) : ONE_OK; }

    int fill_operands(const OneImage &img) override   // host/ops/gemm.h:50-126, mat_mul.h:59-123
    {
        fill_names(&gemm_cfg.op_base_cfg);
        if (in_operands.size() < 2) return ONE_ERR_BAD_ARG;
        weight = find_init(img, in_operands[1]);
        if (is_gemm) {
            if (in_operands.size() < 3) return ONE_ERR_BAD_ARG;
            bias = find_init(img, in_operands[2]);
            if (!weight || !bias) return ONE_ERR_BAD_ARG;
        }
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        memcpy(out.shapes, in.shapes, sizeof(out.shapes));
        out.dim_num_of_shapes = in.dim_num_of_shapes;
        int n;
        if (is_gemm) n = bias->desc->shapes[0];               // N from the bias length (host/ops/gemm.h:39)
        else if (weight) n = weight->desc->shapes[weight->desc->dim_num_of_shapes - 1];
        else n = m[in_operands[1]].shapes[m[in_operands[1]].dim_num_of_shapes - 1];
        out.shapes[out.dim_num_of_shapes - 1] = n;
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &opt, TensorInfo *out,
              std::vector<bool> *need_plain) override
    {
        // A: row-major, either fp32 or the activation type of the precision
        (*need_plain)[0] = ins[0]->layout != LAYOUT_PLAIN || !(ins[0]->dtype == DT_F32 || ins[0]->dtype == opt.act_dtype());
        for (size_t i = 1; i < ins.size(); ++i) (*need_plain)[i] = ins[i]->layout != LAYOUT_PLAIN || ins[i]->dtype != DT_F32;
        out->layout = LAYOUT_PLAIN;
        out->dtype = DT_F32;
    }
    int prepare(one_ctx *ctx, const NetOptions &opt, const std::vector<const TensorInfo *> &ins,
                const TensorInfo &out) override
    {
        prec = opt.precision;
        if (!weight) return ONE_OK;   // activation x activation MatMul: nothing to prepare (one_cuda_matmul_async)
        flags = opt.precision | ONE_OUT_F32;
        if (ins[0]->dtype == opt.act_dtype()) flags |= ONE_LAYOUT_NHWC;   // A already in the operand type
        BUFFER_INFO_S p[BUF_MAXNUM], in[BUF_MAXNUM];
        memset(p, 0, sizeof(p));
        memset(in, 0, sizeof(in));
        if (fused_bias) in[2].addr = (int64_t)fused_bias->data;
        if (fuse_gelu) {
            gelu_lut = build_gelu_lut();
            in[BUF_MAXNUM - 1].addr = (int64_t)gelu_lut.data();
            flags |= ONE_FUSE_GELU;
        }
        if (!residual.empty()) flags |= ONE_FUSE_ADD;
        p[0].addr = (int64_t)&gemm_cfg;
        p[1].addr = (int64_t)&ins[0]->desc;
        p[2].addr = (int64_t)weight->desc;
        if (is_gemm) {
            p[3].addr = (int64_t)bias->desc;
            p[4].addr = (int64_t)&out.desc;
            in[2].addr = (int64_t)bias->data;
        } else {
            p[3].addr = (int64_t)&out.desc;
        }
        in[1].addr = (int64_t)weight->data;
        int rc = one_cuda_set_tile_n(tile_n);
        if (rc != ONE_OK) return rc;
        rc = one_cuda_prepare(ctx, is_gemm ? "Gemm" : "MatMul", p, in, flags, &packed);
        one_cuda_set_tile_n(0);
        if (rc == ONE_OK) rc = one_cuda_packed_set_split(packed, split_k);
        return rc;
    }
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &inits) override
    {
        op::rt_prepare(t, inits);
        params_vec[0].addr = (int64_t)&gemm_cfg;
        if (weight) params_vec[2].addr = (int64_t)weight->desc;
        if (is_gemm) {
            params_vec[3].addr = (int64_t)bias->desc;
            params_vec[4].addr = (int64_t)&t[out_operands[0]].desc;
        } else {
            if (!weight) {   // second activation operand
                params_vec[2].addr = (int64_t)&t[in_operands[1]].desc;
                inputs_vec[1].addr = (int64_t)t[in_operands[1]].dev;
            }
            params_vec[3].addr = (int64_t)&t[out_operands[0]].desc;
        }
        if (!residual.empty()) inputs_vec[ONE_SLOT_RESIDUAL].addr = (int64_t)t[residual].dev;
        return ONE_OK;
    }
    int forward(one_ctx *ctx, cudaStream_t s) override
    {
        if (!packed) {   // activation x activation
            double f = 0, b = 0;
            int rc = one_cuda_matmul_async(ctx, params_vec.data(), inputs_vec.data(), outputs_vec.data(), prec, s, &f, &b);
            mflop = f * 1e-6;
            bytes = b;
            return rc;
        }
        int rc = one_cuda_eval_async(ctx, packed, params_vec.data(), inputs_vec.data(), outputs_vec.data(), s);
        if (rc == ONE_OK) {
            double f, b;
            one_cuda_packed_work(packed, &f, &b);
            mflop = f * 1e-6;
            bytes = b;
        }
        return rc;
    }
    double get_computation() override { return mflop; }   // host/ops/gemm.h:128-145
    double get_bytes() override { return bytes; }
    std::string describe() override
    {
        char buf[192] = {0};
        if (packed) one_cuda_packed_detail(packed, buf, sizeof(buf));
        return buf;
    }
};

class Gemm : public GemmLike {
public:
    static int create_instance(std::shared_ptr<op> &p, const char *cfg)
    {
        auto o = std::make_shared<Gemm>();
        o->is_gemm = true;
        memcpy(&o->gemm_cfg, cfg, sizeof(GEMM_CONFIG_S));
        p = o;
        return 0;
    }
};
OP_REGISTER_GLOBAL(Gemm, Gemm::create_instance, sizeof(GEMM_CONFIG_S));

class MatMul : public GemmLike {
public:
    static int create_instance(std::shared_ptr<op> &p, const char *cfg)
    {
        auto o = std::make_shared<MatMul>();
        o->is_gemm = false;
        memset(&o->gemm_cfg, 0, sizeof(GEMM_CONFIG_S));
        memcpy(&o->gemm_cfg, cfg, sizeof(MATMUL_CONFIG_S));
        p = o;
        return 0;
    }
};
OP_REGISTER_GLOBAL(MatMul, MatMul::create_instance, sizeof(MATMUL_CONFIG_S));

// ---------------------------------------------------------------------------------- glue operators
// Shared by the elementwise / pooling operators: remembers the physical form of its input.
class GlueOp : public op {
public:
    int dtype = DT_F32;
    long long in_elems = 0, out_elems = 0;
    int n = 0, c = 0, h = 0, w = 0;
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &inits) override
    {
        op::rt_prepare(t, inits);
        const TensorInfo &x = t[in_operands[0]];
        dtype = x.dtype;
        n = x.desc.shapes[0]; c = x.desc.shapes[1]; h = x.desc.shapes[2]; w = x.desc.shapes[3];
        in_elems = operand_elem_size(&x.desc);
        out_elems = operand_elem_size(&t[out_operands[0]].desc);
        return ONE_OK;
    }
    double get_bytes() override { return (double)(in_elems * (long long)in_operands.size() + out_elems) * dtype_size(dtype); }
};

class MaxPool : public GlueOp {
public:
    MAX_POOL_CONFIG_S cfg;
    static int create_instance(std::shared_ptr<op> &p, const char *c)
    {
        auto o = std::make_shared<MaxPool>();
        memcpy(&o->cfg, c, sizeof(MAX_POOL_CONFIG_S));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &) override
    {
        fill_names(&cfg.op_base_cfg);
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/maxpool.h:29-53
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        memcpy(out.shapes, in.shapes, sizeof(out.shapes));
        out.dim_num_of_shapes = in.dim_num_of_shapes;
        out.shapes[2] = (in.shapes[2] + (int)cfg.pads[0] + (int)cfg.pads[2] - (int)cfg.kernel_shape[0]) / (int)cfg.strides[0] + 1;
        out.shapes[3] = (in.shapes[3] + (int)cfg.pads[1] + (int)cfg.pads[3] - (int)cfg.kernel_shape[1]) / (int)cfg.strides[1] + 1;
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        (*need_plain)[0] = false;   // consumes NHWC as produced by a Conv
        out->layout = LAYOUT_NHWC;
        out->dtype = ins[0]->dtype;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        // the kernel reads NHWC; a pool straight on the network input would need a re-layout first
        return ins[0]->layout == LAYOUT_NHWC ? ONE_OK : ONE_ERR_UNSUPPORTED;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        // the reference kernel reads strides[0] as the x stride and strides[1] as the y stride
        // (device/x86/MaxPool/maxpool.c:20-21) and pads every side by pads[0] (:41-57)
        return one_glue_maxpool_nhwc((const void *)inputs_vec[0].addr, (void *)outputs_vec[0].addr, dtype, n, h, w, c,
                                     (int)cfg.kernel_shape[0], (int)cfg.kernel_shape[1], (int)cfg.strides[1], (int)cfg.strides[0],
                                     (int)cfg.pads[0], s);
    }
};
OP_REGISTER_GLOBAL(MaxPool, MaxPool::create_instance, sizeof(MAX_POOL_CONFIG_S));

// Relu on whatever physical form its input has.  (Add lives in seq_ops.h with the other
// broadcasting operators.)
class Relu : public GlueOp {
public:
    RELU_CONFIG_S cfg;
    static int create_instance(std::shared_ptr<op> &p, const char *c)
    {
        auto o = std::make_shared<Relu>();
        memcpy(&o->cfg, c, sizeof(RELU_CONFIG_S));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &) override
    {
        fill_names(&cfg.op_base_cfg);
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        memcpy(out.shapes, in.shapes, sizeof(out.shapes));
        out.dim_num_of_shapes = in.dim_num_of_shapes;
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        (*need_plain)[0] = false;
        out->layout = ins[0]->layout;
        out->dtype = ins[0]->dtype;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_add_relu((const void *)inputs_vec[0].addr, nullptr, (void *)outputs_vec[0].addr, dtype, out_elems, 1, s);
    }
};
OP_REGISTER_GLOBAL(Relu, Relu::create_instance, sizeof(RELU_CONFIG_S));

class GlobalAveragePool : public GlueOp {
public:
    GLOBAL_AVGPOOL_CONFIG_S cfg;
    static int create_instance(std::shared_ptr<op> &p, const char *c)
    {
        auto o = std::make_shared<GlobalAveragePool>();
        memcpy(&o->cfg, c, sizeof(cfg));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &) override
    {
        fill_names(&cfg.op_base_cfg);
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        out.dim_num_of_shapes = 4;
        out.shapes[0] = in.shapes[0];
        out.shapes[1] = in.shapes[1];
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        (*need_plain)[0] = false;
        out->layout = LAYOUT_PLAIN;   // [N][C][1][1]: NHWC and NCHW coincide
        out->dtype = ins[0]->dtype;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        return ins[0]->layout == LAYOUT_NHWC ? ONE_OK : ONE_ERR_UNSUPPORTED;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_gap_nhwc((const void *)inputs_vec[0].addr, (void *)outputs_vec[0].addr, dtype, n, h * w, c, s);
    }
};
OP_REGISTER_GLOBAL(GlobalAveragePool, GlobalAveragePool::create_instance, sizeof(GLOBAL_AVGPOOL_CONFIG_S));

// Flatten never computes: its output is a view of its input (host/ops/flatten.h:29-60,
// host/op.h:149-155).
class Flatten : public op {
public:
    FLATTEN_CONFIG_S cfg;
    static int create_instance(std::shared_ptr<op> &p, const char *c)
    {
        auto o = std::make_shared<Flatten>();
        memcpy(&o->cfg, c, sizeof(cfg));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &) override
    {
        fill_names(&cfg.op_base_cfg);
        return ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        const int ax = (int)cfg.axis;
        if (ax < 1 || ax >= SHAPE_LEN) return ONE_ERR_BAD_SHAPE;
        out.not_need_buf = TRUE;
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        out.dim_num_of_shapes = ax + 1;
        for (int i = 0; i < ax; ++i) out.shapes[i] = in.shapes[i];
        for (int i = ax; i < SHAPE_LEN; ++i) out.shapes[ax] *= in.shapes[i];
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        (*need_plain)[0] = ins[0]->layout != LAYOUT_PLAIN;
        out->layout = LAYOUT_PLAIN;
        out->dtype = (*need_plain)[0] ? DT_F32 : ins[0]->dtype;
        out->alias_of = in_operands[0];
    }
    int forward(one_ctx *, cudaStream_t) override { return ONE_OK; }
};
OP_REGISTER_GLOBAL(Flatten, Flatten::create_instance, sizeof(FLATTEN_CONFIG_S));

}  // namespace onenew
