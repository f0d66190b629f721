// op.h -- operator base class and registry of the device-resident graph runtime.
//
// Mirrors the reference's host-side interface so an operator reads like its reference
// counterpart: class `op` with in_operands / out_operands / params_vec / inputs_vec /
// outputs_vec and the virtuals shape_infer / fill_operands / prepare / rt_prepare / forward /
// get_computation (host/op.h:15-193), and the `Manager` singleton filled by
// OP_REGISTER_GLOBAL static initialisers (host/manager/manager.h:10-43).
//
// Differences, all forced by running on the GPU:
//   * operators are not dlopen'ed per type; Conv / Gemm / MatMul call the C ABI of
//     include/one_cuda.h (prepared path), the glue operators call include/one_glue.h;
//   * prepare() uploads and re-orders initialisers once (the reference keeps them in host
//     vectors, host/ops/conv.h:133-157);
//   * forward() only enqueues on a stream and returns a status code the caller checks (the
//     reference ignores the operator's return value, host/op.h:183);
//   * every operand carries a physical layout / element type next to its logical NCHW shape,
//     because activations between convolutions stay NHWC (and bf16 in the bf16 mode).
#pragma once
#include <cuda_runtime.h>

#include <cstring>
#include <functional>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/one_cuda.h"
#include "../../include/one_glue.h"

namespace onenew {

enum Layout { LAYOUT_PLAIN = 0 /* the reference's: NCHW / row-major */, LAYOUT_NHWC = 1 };
enum DType { DT_F32 = 0, DT_BF16 = 1, DT_S8 = 2, DT_F16 = 3 };
inline size_t dtype_size(int dt) { return dt == DT_F32 ? 4 : ((dt == DT_BF16 || dt == DT_F16) ? 2 : 1); }

// Physical description of one operand on the device.
struct TensorInfo {
    OPERAND_S desc;          // logical shape (shapes[0] = batch), as shape_infer produced it
    int layout = LAYOUT_PLAIN;
    int dtype = DT_F32;
    void *dev = nullptr;
    size_t bytes = 0;
    std::string alias_of;    // zero-copy view of another operand (Flatten, fused Add/Relu)
};

struct NetOptions {
    int precision = ONE_PREC_TF32;   // float path: ONE_PREC_TF32, ONE_PREC_BF16 or ONE_PREC_F16
    int batch = 1;                   // leading dimension given to every activation
    bool fuse_residual = true;       // fold Conv -> Add -> Relu into the conv epilogue
    int act_dtype() const { return precision == ONE_PREC_BF16 ? DT_BF16 : (precision == ONE_PREC_F16 ? DT_F16 : DT_F32); }
};

inline long long operand_elem_size(const OPERAND_S *o)   // common/utils_c.h:9-16
{
    long long n = 1;
    for (int i = 0; i < SHAPE_LEN; ++i) n *= o->shapes[i];
    return n;
}

// View of a loaded .one image (host/net.h:101-221).
struct OneImage {
    const char *base = nullptr;
    size_t size = 0;
    struct Init {
        const OPERAND_S *desc;
        const char *data;
    };
    std::unordered_map<std::string, Init> inits;
    const ONE_MODEL_DESC_S *desc() const { return reinterpret_cast<const ONE_MODEL_DESC_S *>(base); }
};

class op {
public:
    std::string op_type, op_name;
    std::vector<std::string> in_operands, out_operands;
    std::vector<BUFFER_INFO_S> params_vec, inputs_vec, outputs_vec;   // BUF_MAXNUM slots each
    bool skipped = false;    // folded into another operator by the runtime's fusion pass
    int tile_n = 0;          // forced output-tile width of the contraction kernel (0: the library's heuristic)
    int split_k = 0;         // forced split-K choice of the contraction (0: the library's heuristic, 1: never, n: n ranges)
    std::string residual;    // operand added in this operator's epilogue (a folded Add); empty: none
    bool keep_f32 = false;   // bf16 mode: this operator's output stays fp32 (it lies on the residual trunk)

    op() : params_vec(BUF_MAXNUM), inputs_vec(BUF_MAXNUM), outputs_vec(BUF_MAXNUM)
    {
        memset(params_vec.data(), 0, sizeof(BUFFER_INFO_S) * BUF_MAXNUM);
        memset(inputs_vec.data(), 0, sizeof(BUFFER_INFO_S) * BUF_MAXNUM);
        memset(outputs_vec.data(), 0, sizeof(BUFFER_INFO_S) * BUF_MAXNUM);
    }
    virtual ~op() {}

    // Copy names out of the record's BASE_CONFIG_S (every fill_operands starts like this).
    void fill_names(const BASE_CONFIG_S *b)
    {
        op_type = b->op_type;
        op_name = b->op_name;
        for (int i = 0; i < b->in_operand_num && i < OPERAND_MAXNUM; ++i) in_operands.push_back(b->in_operand_name[i]);
        for (int i = 0; i < b->out_operand_num && i < OPERAND_MAXNUM; ++i) out_operands.push_back(b->out_operand_name[i]);
    }
    // Activation inputs: the in_operands that are not initialisers, in order.
    std::vector<std::string> act_inputs(const std::set<std::string> &inits) const
    {
        std::vector<std::string> v;
        for (auto &n : in_operands)
            if (!n.empty() && !inits.count(n)) v.push_back(n);
        return v;
    }

    virtual int fill_operands(const OneImage &img) = 0;
    // Logical output shapes from the input shapes; the batch (shapes[0]) is propagated.
    virtual int shape_infer(std::unordered_map<std::string, OPERAND_S> &operand_stu_map) = 0;
    // Physical layout / type of the outputs given those of the inputs; `need_plain[i]` is set
    // when activation input i has to be converted to the reference layout first.
    virtual void plan(const std::vector<const TensorInfo *> &ins, const NetOptions &opt, TensorInfo *out,
                      std::vector<bool> *need_plain)
    {
        for (size_t i = 0; i < ins.size(); ++i) (*need_plain)[i] = ins[i]->layout != LAYOUT_PLAIN || ins[i]->dtype != DT_F32;
        out->layout = LAYOUT_PLAIN;
        out->dtype = DT_F32;
    }
    // Upload constants, build the prepared operator.
    virtual int prepare(one_ctx *ctx, const NetOptions &opt, const std::vector<const TensorInfo *> &ins,
                        const TensorInfo &out)
    {
        return ONE_OK;
    }
    // Tile tuning: operators whose kernel has a selectable output-tile width say so, report the width of
    // their output (columns of the contraction) and can drop what prepare() built so that it can run again.
    virtual bool tunable() const { return false; }
    virtual int out_width() const { return 0; }
    virtual void drop_prepared() {}
    virtual int set_split() { return ONE_OK; }   // hand split_k to the prepared operator (no re-preparation needed)
    // Wire descriptor and buffer arrays (host/op.h:109-168).
    virtual int rt_prepare(std::unordered_map<std::string, TensorInfo> &tensors, const std::set<std::string> &inits)
    {
        int pi = 1, bi = 0;
        for (auto &n : act_inputs(inits)) {
            params_vec[pi++].addr = (int64_t)&tensors[n].desc;
            inputs_vec[bi++].addr = (int64_t)tensors[n].dev;
        }
        int oi = 1 + (int)in_operands.size();
        for (size_t i = 0; i < out_operands.size(); ++i) {
            params_vec[oi++].addr = (int64_t)&tensors[out_operands[i]].desc;
            outputs_vec[i].addr = (int64_t)tensors[out_operands[i]].dev;
        }
        return ONE_OK;
    }
    virtual int forward(one_ctx *ctx, cudaStream_t stream) = 0;
    virtual double get_computation() { return 0.0; }   // MFLOP, as the reference counts
    virtual double get_bytes() { return 0.0; }         // compulsory bytes of one evaluation
    virtual std::string describe() { return std::string(); }   // shape / tile of the last evaluation, for the tracing table
};

typedef std::function<int(std::shared_ptr<op> &, const char *)> creator_;

class Manager {
public:
    std::unordered_map<std::string, creator_> Opmap;
    std::unordered_map<std::string, int> op_cfg_size_map;
    static Manager &getInstance()
    {
        static Manager m;
        return m;
    }

private:
    Manager() {}
};

class OpRegistry {
public:
    OpRegistry(const char *op_type, creator_ c, int cfg_size)
    {
        Manager &m = Manager::getInstance();
        m.Opmap[op_type] = c;
        m.op_cfg_size_map[op_type] = cfg_size;
    }
};

#define OP_REGISTER_GLOBAL(name, creator, cfg_size) static ::onenew::OpRegistry g_creator_##name(#name, creator, cfg_size)

inline int align_buf_size(int n) { return (n + 63) & ~63; }   // common/utils_c.h:4-7

}  // namespace onenew
