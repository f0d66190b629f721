// seq_ops.h -- operator classes for the glue between the MatMul / Gemm calls of a transformer
// encoder (ViT): LayerNormalization, Gelu, Softmax, Transpose, Reshape, Concat, Gather, and the
// broadcasting Add / Sub / Mul / Div.  Each mirrors its reference counterpart under host/ops/
// (shape_infer, the handling of initialiser operands) and calls the device kernels of
// include/one_glue.h.  All of them work on fp32 tensors in the reference's row-major layout.
//
// The batch rule of the runtime applies: an initialiser whose leading dimension is 1 is repeated
// over the batch (class token in Concat, position embedding in Add), and a Reshape whose target
// has a leading 1 keeps the batch of its input.
#pragma once
#include <cmath>

#include "ops.h"

namespace onenew {

// Device copy of an initialiser, owned by the operator.
struct DevConst {
    void *dev = nullptr;
    ~DevConst() { if (dev) cudaFree(dev); }
    int upload(const void *host, size_t bytes)
    {
        if (dev) { cudaFree(dev); dev = nullptr; }
        if (cudaMalloc(&dev, bytes ? bytes : 16) != cudaSuccess) return ONE_ERR_NOMEM;
        if (bytes && cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return ONE_ERR_CUDA;
        return ONE_OK;
    }
};

inline void copy_shape(OPERAND_S &dst, const OPERAND_S &src)
{
    memcpy(dst.shapes, src.shapes, sizeof(dst.shapes));
    dst.dim_num_of_shapes = src.dim_num_of_shapes;
    dst.data_type = TYPE_FP32;
}

template <typename CFG>
class SeqOp : public op {
public:
    CFG cfg;
    long long in_elems = 0, out_elems = 0;
    int fill_operands(const OneImage &) override
    {
        fill_names(&cfg.op_base_cfg);
        return ONE_OK;
    }
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &inits) override
    {
        op::rt_prepare(t, inits);
        in_elems = 0;
        for (auto &n : act_inputs(inits)) in_elems += operand_elem_size(&t[n].desc);
        out_elems = operand_elem_size(&t[out_operands[0]].desc);
        return ONE_OK;
    }
    double get_bytes() override { return (double)(in_elems + out_elems) * 4.0; }
};

#define ONE_SEQ_CREATE(cls, CFG)                                   \
    static int create_instance(std::shared_ptr<op> &p, const char *c) \
    {                                                              \
        auto o = std::make_shared<cls>();                          \
        memcpy(&o->cfg, c, sizeof(CFG));                           \
        p = o;                                                     \
        return 0;                                                  \
    }

// ---------------------------------------------------------------------------------- LayerNormalization
class LayerNormalization : public SeqOp<LAYERNORMALIZATION_CONFIG_S> {
public:
    const OneImage::Init *weight = nullptr, *bias = nullptr;
    DevConst w_dev, b_dev;
    long long rows = 0;
    int D = 0;
    ONE_SEQ_CREATE(LayerNormalization, LAYERNORMALIZATION_CONFIG_S)
    int fill_operands(const OneImage &img) override   // host/ops/layer_normalization.h
    {
        fill_names(&cfg.op_base_cfg);
        if (in_operands.size() < 3) return ONE_ERR_BAD_ARG;
        weight = find_init(img, in_operands[1]);
        bias = find_init(img, in_operands[2]);
        return (weight && bias) ? ONE_OK : ONE_ERR_BAD_ARG;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        copy_shape(m[out_operands[0]], m[in_operands[0]]);
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        if (cfg.axes[0] == 1 && ins[0]->desc.dim_num_of_shapes > 2)   // strided variant (layer_normalization.c:27-58)
            return ONE_ERR_UNSUPPORTED;
        const OPERAND_S &x = ins[0]->desc;
        D = 1;
        for (int i = SHAPE_LEN - 1; i >= 0; --i)   // the last dimension that is not 1 (layer_normalization.c:60-66)
            if (x.shapes[i] != 1) { D = x.shapes[i]; break; }
        rows = operand_elem_size(&x) / D;
        if (operand_elem_size(weight->desc) < D || operand_elem_size(bias->desc) < D) return ONE_ERR_BAD_SHAPE;
        int rc = w_dev.upload(weight->data, (size_t)D * 4);
        return rc != ONE_OK ? rc : b_dev.upload(bias->data, (size_t)D * 4);
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_layernorm((const float *)inputs_vec[0].addr, (const float *)w_dev.dev, (const float *)b_dev.dev,
                                  (float *)outputs_vec[0].addr, rows, D, s);
    }
    double get_computation() override { return (double)out_elems * 8e-6; }
};
OP_REGISTER_GLOBAL(LayerNormalization, LayerNormalization::create_instance, sizeof(LAYERNORMALIZATION_CONFIG_S));

// ---------------------------------------------------------------------------------- Gelu
class Gelu : public SeqOp<GELU_CONFIG_S> {
public:
    DevConst lut_dev;
    ONE_SEQ_CREATE(Gelu, GELU_CONFIG_S)
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        copy_shape(m[out_operands[0]], m[in_operands[0]]);
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &, const TensorInfo &) override
    {
        const std::vector<float> lut = build_gelu_lut();
        return lut_dev.upload(lut.data(), lut.size() * 4);
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_gelu_lut((const float *)inputs_vec[0].addr, (const float *)lut_dev.dev, (float *)outputs_vec[0].addr,
                                 out_elems, s);
    }
    double get_computation() override { return (double)out_elems * 5e-6; }   // host/ops/gelu.h:69-77
};
OP_REGISTER_GLOBAL(Gelu, Gelu::create_instance, sizeof(GELU_CONFIG_S));

// ---------------------------------------------------------------------------------- Softmax
class Softmax : public SeqOp<SOFTMAX_CONFIG_S> {
public:
    long long rows = 0;
    int D = 0;
    ONE_SEQ_CREATE(Softmax, SOFTMAX_CONFIG_S)
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        copy_shape(m[out_operands[0]], m[in_operands[0]]);
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        const OPERAND_S &x = ins[0]->desc;
        if (!(cfg.axis == -1 || cfg.axis == x.dim_num_of_shapes - 1)) return ONE_ERR_UNSUPPORTED;   // softmax.c:19-26
        D = x.shapes[x.dim_num_of_shapes - 1];
        rows = operand_elem_size(&x) / D;
        return ONE_OK;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_softmax_rows((const float *)inputs_vec[0].addr, (float *)outputs_vec[0].addr, rows, D, s);
    }
    double get_computation() override { return (double)out_elems * 4e-6; }
};
OP_REGISTER_GLOBAL(Softmax, Softmax::create_instance, sizeof(SOFTMAX_CONFIG_S));

// ---------------------------------------------------------------------------------- Transpose
class Transpose : public SeqOp<TRANSPOSE_CONFIG_S> {
public:
    int ndim = 0, in_shape[8], perm[8];
    ONE_SEQ_CREATE(Transpose, TRANSPOSE_CONFIG_S)
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/transpose.h:32-48
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        copy_shape(out, in);
        if (cfg.perm_num < 1 || cfg.perm_num > 6) return ONE_ERR_UNSUPPORTED;
        for (int i = 0; i < cfg.perm_num; ++i) {
            if (cfg.perm[i] < 0 || cfg.perm[i] >= cfg.perm_num) return ONE_ERR_BAD_ARG;
            out.shapes[i] = in.shapes[cfg.perm[i]];
        }
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        ndim = (int)cfg.perm_num;
        for (int i = 0; i < ndim; ++i) {
            in_shape[i] = ins[0]->desc.shapes[i];
            perm[i] = (int)cfg.perm[i];
        }
        return ONE_OK;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        return one_glue_transpose((const float *)inputs_vec[0].addr, (float *)outputs_vec[0].addr, ndim, in_shape, perm, s);
    }
};
OP_REGISTER_GLOBAL(Transpose, Transpose::create_instance, sizeof(TRANSPOSE_CONFIG_S));

// ---------------------------------------------------------------------------------- Reshape (a view)
class Reshape : public SeqOp<RESHAPE_CONFIG_S> {
public:
    ONE_SEQ_CREATE(Reshape, RESHAPE_CONFIG_S)
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/reshape.h:30-68
    {
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        out.not_need_buf = TRUE;
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        const int n = (int)cfg.dst_shape_num;
        if (n < 1 || n > SHAPE_LEN) return ONE_ERR_BAD_SHAPE;
        const long long elems = operand_elem_size(&in);
        long long known = 1;
        int unknown = -1;
        for (int i = 0; i < n; ++i) {
            long long d = cfg.dst_shape[i];
            if (i == 0 && d == 1 && in.shapes[0] > 1) d = in.shapes[0];   // the batch rule
            out.shapes[i] = (int)d;
            if (d == -1) unknown = i;
            else known *= d;
        }
        if (known <= 0) return ONE_ERR_BAD_SHAPE;
        if (unknown >= 0) out.shapes[unknown] = (int)(elems / known);
        out.dim_num_of_shapes = n;
        out.data_type = TYPE_FP32;
        return operand_elem_size(&out) == elems ? ONE_OK : ONE_ERR_BAD_SHAPE;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        (*need_plain)[0] = ins[0]->layout != LAYOUT_PLAIN || ins[0]->dtype != DT_F32;
        out->layout = LAYOUT_PLAIN;
        out->dtype = DT_F32;
        out->alias_of = in_operands[0];
    }
    int forward(one_ctx *, cudaStream_t) override { return ONE_OK; }
    double get_bytes() override { return 0.0; }
};
OP_REGISTER_GLOBAL(Reshape, Reshape::create_instance, sizeof(RESHAPE_CONFIG_S));

// ---------------------------------------------------------------------------------- Concat
class Concat : public SeqOp<CONCAT_CONFIG_S> {
public:
    struct Part {
        const OneImage::Init *init = nullptr;
        DevConst dev;
        long long chunk = 0, x_reps = 1;
        const void *src = nullptr;
    };
    std::vector<std::unique_ptr<Part>> parts;
    long long reps = 0, y_stride = 0;
    int axis = 0;
    ONE_SEQ_CREATE(Concat, CONCAT_CONFIG_S)
    int fill_operands(const OneImage &img) override   // host/ops/concat.h:72-140: an input may be an initialiser
    {
        fill_names(&cfg.op_base_cfg);
        for (auto &n : in_operands) {
            parts.emplace_back(new Part());
            parts.back()->init = find_init(img, n);
        }
        return in_operands.empty() ? ONE_ERR_BAD_ARG : ONE_OK;
    }
    const OPERAND_S &in_desc(std::unordered_map<std::string, OPERAND_S> &m, size_t i) { return parts[i]->init ? *parts[i]->init->desc : m[in_operands[i]]; }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/concat.h:31-70
    {
        OPERAND_S &out = m[out_operands[0]];
        size_t first_act = 0;
        while (first_act < parts.size() && parts[first_act]->init) ++first_act;
        if (first_act == parts.size()) return ONE_ERR_UNSUPPORTED;
        copy_shape(out, m[in_operands[first_act]]);
        axis = (int)cfg.axis;
        if (axis < 0) axis += out.dim_num_of_shapes;
        if (axis < 0 || axis >= out.dim_num_of_shapes) return ONE_ERR_BAD_ARG;
        int sum = 0;
        for (size_t i = 0; i < parts.size(); ++i) sum += in_desc(m, i).shapes[axis];
        out.shapes[axis] = sum;
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &out) override
    {
        reps = 1;
        for (int i = 0; i < axis; ++i) reps *= out.desc.shapes[i];
        long long inner = 1;
        for (int i = axis + 1; i < SHAPE_LEN; ++i) inner *= out.desc.shapes[i];
        y_stride = out.desc.shapes[axis] * inner;
        size_t ai = 0;
        for (auto &p : parts) {
            const OPERAND_S &d = p->init ? *p->init->desc : ins[ai++]->desc;
            p->chunk = d.shapes[axis] * inner;
            long long outer = 1;
            for (int i = 0; i < axis; ++i) outer *= d.shapes[i];
            if (outer != reps && !(p->init && outer == 1)) return ONE_ERR_BAD_SHAPE;
            p->x_reps = outer;   // 1: an initialiser repeated over the batch
            if (p->init) {
                int rc = p->dev.upload(p->init->data, (size_t)operand_elem_size(&d) * 4);
                if (rc != ONE_OK) return rc;
            }
        }
        return ONE_OK;
    }
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &inits) override
    {
        SeqOp::rt_prepare(t, inits);
        for (size_t i = 0; i < parts.size(); ++i) parts[i]->src = parts[i]->init ? parts[i]->dev.dev : t[in_operands[i]].dev;
        return ONE_OK;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        float *y = (float *)outputs_vec[0].addr;
        long long off = 0;
        for (auto &p : parts) {
            int rc = one_glue_copy_chunks((const float *)p->src, y + off, reps, p->chunk, p->x_reps, p->chunk, y_stride, s);
            if (rc != ONE_OK) return rc;
            off += p->chunk;
        }
        return ONE_OK;
    }
};
OP_REGISTER_GLOBAL(Concat, Concat::create_instance, sizeof(CONCAT_CONFIG_S));

// ---------------------------------------------------------------------------------- Gather (fixed index)
class Gather : public SeqOp<GATHER_CONFIG_S> {
public:
    long long reps = 0, inner = 0, x_stride = 0, x_off = 0;
    ONE_SEQ_CREATE(Gather, GATHER_CONFIG_S)
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override   // host/ops/gather.h:63-77
    {
        if (cfg.indices_from_ifmap) return ONE_ERR_UNSUPPORTED;   // index tensors (embedding lookups) are not on this path
        const OPERAND_S &in = m[in_operands[0]];
        OPERAND_S &out = m[out_operands[0]];
        const int ax = (int)cfg.axis;
        if (ax < 0 || ax >= in.dim_num_of_shapes || cfg.indices < 0 || cfg.indices >= in.shapes[ax]) return ONE_ERR_BAD_ARG;
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        out.dim_num_of_shapes = in.dim_num_of_shapes - 1;
        for (int i = 0; i < ax; ++i) out.shapes[i] = in.shapes[i];
        for (int i = ax; i < in.dim_num_of_shapes - 1; ++i) out.shapes[i] = in.shapes[i + 1];
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        const OPERAND_S &in = ins[0]->desc;
        const int ax = (int)cfg.axis;
        reps = 1;
        for (int i = 0; i < ax; ++i) reps *= in.shapes[i];
        inner = 1;
        for (int i = ax + 1; i < SHAPE_LEN; ++i) inner *= in.shapes[i];
        x_stride = in.shapes[ax] * inner;
        x_off = cfg.indices * inner;
        return ONE_OK;
    }
    int forward(one_ctx *, cudaStream_t s) override   // device/x86/Gather/gather.c:13-33
    {
        return one_glue_copy_chunks((const float *)inputs_vec[0].addr + x_off, (float *)outputs_vec[0].addr, reps, inner, reps,
                                    x_stride, inner, s);
    }
    double get_bytes() override { return (double)out_elems * 8.0; }
};
OP_REGISTER_GLOBAL(Gather, Gather::create_instance, sizeof(GATHER_CONFIG_S));

// ---------------------------------------------------------------------------------- Add / Sub / Mul / Div
// numpy broadcasting between two operands, either of which may be an initialiser
// (host/ops/add.h, mul.h, div.h; device/x86/Add/add.c:17-86).  The equal-shape sum of two
// activations keeps the NHWC / bf16 form of its inputs (residual connections of a CNN).
template <int OP>   // 0 add, 1 sub, 2 mul, 3 div
class Binary : public SeqOp<ADD_CONFIG_S> {
public:
    const OneImage::Init *init[2] = {nullptr, nullptr};
    DevConst init_dev[2];
    const void *src[2] = {nullptr, nullptr};
    int ndim = 0, shp[2][8];
    bool same_form = false;   // equal-shape activations in whatever physical form they share
    int dtype = DT_F32;
    static int create_instance(std::shared_ptr<op> &p, const char *c)
    {
        auto o = std::make_shared<Binary<OP>>();
        memcpy(&o->cfg, c, sizeof(ADD_CONFIG_S));
        p = o;
        return 0;
    }
    int fill_operands(const OneImage &img) override
    {
        fill_names(&cfg.op_base_cfg);
        if (in_operands.size() != 2) return ONE_ERR_BAD_ARG;
        for (int i = 0; i < 2; ++i) init[i] = find_init(img, in_operands[i]);
        return (init[0] && init[1]) ? ONE_ERR_UNSUPPORTED : ONE_OK;
    }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &m) override
    {
        const OPERAND_S &a = init[0] ? *init[0]->desc : m[in_operands[0]];
        const OPERAND_S &b = init[1] ? *init[1]->desc : m[in_operands[1]];
        OPERAND_S &out = m[out_operands[0]];
        const int na = a.dim_num_of_shapes, nb = b.dim_num_of_shapes;
        ndim = na > nb ? na : nb;
        if (ndim < 1 || ndim > 6) return ONE_ERR_UNSUPPORTED;
        for (int i = 0; i < SHAPE_LEN; ++i) out.shapes[i] = 1;
        for (int i = 0; i < ndim; ++i) {   // right-aligned (add.c:52-67)
            shp[0][i] = i < ndim - na ? 1 : a.shapes[i - (ndim - na)];
            shp[1][i] = i < ndim - nb ? 1 : b.shapes[i - (ndim - nb)];
            if (shp[0][i] != shp[1][i] && shp[0][i] != 1 && shp[1][i] != 1) return ONE_ERR_BAD_SHAPE;
            out.shapes[i] = shp[0][i] > shp[1][i] ? shp[0][i] : shp[1][i];
        }
        out.dim_num_of_shapes = ndim;
        out.data_type = TYPE_FP32;
        return ONE_OK;
    }
    void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &, TensorInfo *out, std::vector<bool> *need_plain) override
    {
        bool equal = !init[0] && !init[1] && ins.size() == 2;
        for (int i = 0; equal && i < ndim; ++i) equal = shp[0][i] == shp[1][i];
        same_form = equal && OP == 0 && ins[0]->layout == ins[1]->layout && ins[0]->dtype == ins[1]->dtype;
        for (size_t i = 0; i < ins.size(); ++i)
            (*need_plain)[i] = same_form ? false : (ins[i]->layout != LAYOUT_PLAIN || ins[i]->dtype != DT_F32);
        out->layout = same_form ? ins[0]->layout : LAYOUT_PLAIN;
        out->dtype = same_form ? ins[0]->dtype : DT_F32;
        dtype = out->dtype;
    }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &, const TensorInfo &) override
    {
        for (int i = 0; i < 2; ++i)
            if (init[i]) {
                int rc = init_dev[i].upload(init[i]->data, (size_t)operand_elem_size(init[i]->desc) * 4);
                if (rc != ONE_OK) return rc;
            }
        return ONE_OK;
    }
    int rt_prepare(std::unordered_map<std::string, TensorInfo> &t, const std::set<std::string> &inits) override
    {
        SeqOp::rt_prepare(t, inits);
        for (int i = 0; i < 2; ++i) src[i] = init[i] ? init_dev[i].dev : t[in_operands[i]].dev;
        return ONE_OK;
    }
    int forward(one_ctx *, cudaStream_t s) override
    {
        if (same_form) return one_glue_add_relu(src[0], src[1], (void *)outputs_vec[0].addr, dtype, out_elems, 0, s);
        return one_glue_binary(OP, (const float *)src[0], (const float *)src[1], (float *)outputs_vec[0].addr, ndim, shp[0], shp[1], s);
    }
    double get_computation() override { return (double)out_elems * 1e-6; }
    double get_bytes() override { return (double)(in_elems + out_elems) * dtype_size(dtype); }
};
typedef Binary<0> Add;
typedef Binary<1> Sub;
typedef Binary<2> Mul;
typedef Binary<3> Div;
OP_REGISTER_GLOBAL(Add, Add::create_instance, sizeof(ADD_CONFIG_S));
OP_REGISTER_GLOBAL(Sub, Sub::create_instance, sizeof(SUB_CONFIG_S));
OP_REGISTER_GLOBAL(Mul, Mul::create_instance, sizeof(MUL_CONFIG_S));
OP_REGISTER_GLOBAL(Div, Div::create_instance, sizeof(DIV_CONFIG_S));

// ---------------------------------------------------------------------------------- Attention
// Not an operator of the file format: the runtime's fusion pass puts it in place of the chain
// Gather x3 / Reshape / Transpose -> Mul(scale) -> MatMul -> Softmax -> MatMul -> Transpose -> Reshape
// of one transformer block.  Input: the fused qkv tensor viewed as [B][T][3][D]; output [B][T][D].
class Attention : public op {
public:
    int heads = 0, hd = 0, q_idx = 0, k_idx = 1, v_idx = 2;
    float scale = 1.f;
    int B = 0, T = 0, D = 0, parts = 3;
    int fill_operands(const OneImage &) override { return ONE_OK; }
    int shape_infer(std::unordered_map<std::string, OPERAND_S> &) override { return ONE_OK; }
    int prepare(one_ctx *, const NetOptions &, const std::vector<const TensorInfo *> &ins, const TensorInfo &) override
    {
        const OPERAND_S &x = ins[0]->desc;
        B = x.shapes[0]; T = x.shapes[1]; parts = x.shapes[2]; D = x.shapes[3];
        return (D == heads * hd && T <= 256) ? ONE_OK : ONE_ERR_BAD_SHAPE;
    }
    int forward(one_ctx *ctx, cudaStream_t s) override
    {
        return one_cuda_attention(ctx, (const float *)inputs_vec[0].addr, (float *)outputs_vec[0].addr, B, T, heads, hd, parts * D,
                                  q_idx * D, k_idx * D, v_idx * D, D, scale, s);
    }
    double get_computation() override { return 4.0 * B * heads * (double)T * T * hd * 1e-6; }
    double get_bytes() override { return (double)B * T * (parts + 1) * D * 4.0; }
};

}  // namespace onenew
