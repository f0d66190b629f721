// net.h -- graph runtime for a .one model with device-resident tensors and stream-ordered
// execution.  Mirrors the reference's `net` / `extractor` pair (host/net.h): load_one_model ->
// instantiate_op -> build_graph (ordering + shape inference) -> create_exe -> new_output_buf ->
// prepare_for_op -> impl / impl_tracing.  What is new relative to the reference:
//   * one device arena instead of one host allocation per operand (host/net.h:419-452);
//   * the batch dimension is honoured: every non-initialiser operand whose leading dimension is 1
//     in the file gets the requested batch (the reference forces N = 1, host/ops/conv.h:43);
//   * activations between convolutions stay NHWC (and bf16 in the bf16 mode); conversions to the
//     reference layout are inserted only where an operator or a network output needs them;
//   * Conv -> Add -> Relu chains are folded into the conv epilogue;
//   * execution only enqueues on a stream; the whole step can be replayed as a CUDA graph.
#pragma once
#include <algorithm>
#include <cstdio>
#include <fstream>
#include <map>

#include "seq_ops.h"

namespace onenew {

extern "C" unsigned long long one_cuda_launch_count(void);

class net;

struct Step {
    enum Kind {
        RUN_OP = 0,
        TO_PLAIN = 1 /* NHWC any type -> reference layout fp32 */,
        CAST_F32 = 2,
        TO_NHWC = 3 /* reference layout fp32 -> NHWC in the destination's type */,
        CAST = 4 /* same layout, another element type */
    } kind;
    op *o = nullptr;
    std::string src, dst;
};

class extractor {
public:
    net *net_ptr;
    one_ctx *ctx = nullptr;
    cudaStream_t stream = nullptr;
    std::unordered_map<std::string, TensorInfo> tensors;
    std::vector<Step> steps;
    char *arena = nullptr;
    size_t arena_bytes = 0;
    cudaGraphExec_t graph_exec = nullptr;
    bool ran_eager = false;
    unsigned long long launches_per_run = 0;
    std::string error;

    explicit extractor(net *n) : net_ptr(n) {}
    ~extractor();
    int plan();
    int new_output_buf();
    int prepare_for_op();
    int run_step(const Step &s);
    int enqueue();                 // every step on `stream`, no synchronisation
    int impl(bool use_graph);      // one inference, enqueued (graph replay after the first run)
    int impl_tracing(const char *csv_path, int runs, const char *model_name = nullptr, double hw_gops = 0);
    template <typename F> int time_in_graph(F fn, int runs, cudaEvent_t e0, cudaEvent_t e1, double *us);
    int prepare_one(op *o);        // (re)build one operator's prepared form with its current tile_n
    int autotune(int runs, std::string *report);
    int set_tile(const std::string &op_name, int bn);
    int fetch_plain_f32(const std::string &name, float *host, size_t cap_elems);
};

class net {
public:
    std::vector<char> one_buf;
    OneImage img;
    NetOptions opt;
    std::vector<std::shared_ptr<op>> io_ops, node_ops;
    std::vector<std::shared_ptr<op>> op_exec_order;
    std::set<std::string> init_operands_list;
    std::unordered_map<std::string, OPERAND_S> operand_stu_map;
    std::vector<std::string> input_names, output_names;
    std::unique_ptr<extractor> exc_cls;
    std::string error;

    int load_one_buf(const char *data, size_t size)   // host/net.h:101-136
    {
        if (size < sizeof(ONE_MODEL_DESC_S)) return fail_("image smaller than its header");
        one_buf.assign(data, data + size);
        img.base = one_buf.data();
        img.size = size;
        if (img.desc()->one_model_magic_num != ONE_MAGIC_NUM) return fail_("one_model_magic_num mismatch: not a .one image");
        return ONE_OK;
    }
    int load_one_model(const char *path)
    {
        std::ifstream f(path, std::ios::binary | std::ios::ate);
        if (!f) return fail_(std::string("cannot open ") + path);
        const std::streamsize n = f.tellg();
        f.seekg(0);
        std::vector<char> buf((size_t)n);
        if (!f.read(buf.data(), n)) return fail_("short read");
        return load_one_buf(buf.data(), buf.size());
    }

    int instantiate_op()   // host/net.h:138-221
    {
        Manager &m = Manager::getInstance();
        const ONE_MODEL_DESC_S *d = img.desc();
        // initialiser records first: operators look their weights up by name
        size_t off = (size_t)d->init_info_offset;
        for (int i = 0; i < d->init_cnt; ++i) {
            if (off + sizeof(OPERAND_S) > img.size) return fail_("initialiser record past the end of the image");
            const OPERAND_S *o = reinterpret_cast<const OPERAND_S *>(img.base + off);
            long long bytes = operand_elem_size(o) * elem_size_of(o->data_type);
            if (bytes < 0 || off + sizeof(OPERAND_S) + (size_t)bytes > img.size) return fail_("initialiser data past the end of the image");
            img.inits[o->operand_name] = {o, img.base + off + sizeof(OPERAND_S)};
            init_operands_list.insert(o->operand_name);
            off += (size_t)align_buf_size((int)(sizeof(OPERAND_S) + bytes));
        }
        auto make = [&](const char *rec, std::vector<std::shared_ptr<op>> &dst) -> int {
            std::string type(rec, strnlen(rec, OP_TYPE_LEN));
            auto it = m.Opmap.find(type);
            if (it == m.Opmap.end()) return fail_("operator type '" + type + "' is not registered in this runtime");
            std::shared_ptr<op> p;
            it->second(p, rec);
            int rc = p->fill_operands(img);
            if (rc != ONE_OK) return fail_("fill_operands failed for a " + type + " record");
            // A tuned tile width in the header's cuda_gemm_tile_n (common/nn_common.h:36-38) is the model-wide
            // default; the converter's placeholder (16) is not a width this kernel has and is ignored.
            const int hdr_bn = d->useful_info.block_info.cuda_gemm_tile_n;
            if (hdr_bn == 64 || hdr_bn == 128 || hdr_bn == 192 || hdr_bn == 256) p->tile_n = hdr_bn;
            dst.push_back(p);
            return m.op_cfg_size_map[type];
        };
        off = (size_t)d->io_cfg_offset;
        for (int i = 0; i < d->io_cfg_cnt; ++i) {
            if (off + sizeof(IO_CONFIG_S) > img.size) return fail_("io record past the end of the image");
            int sz = make(img.base + off, io_ops);
            if (sz < 0) return sz;
            off += (size_t)align_buf_size(sz);
        }
        off = (size_t)d->node_cfg_offset;
        for (int i = 0; i < d->node_cnt; ++i) {
            if (off + sizeof(BASE_CONFIG_S) > img.size) return fail_("operator record past the end of the image");
            int sz = make(img.base + off, node_ops);
            if (sz < 0) return sz;
            off += (size_t)align_buf_size(sz);
        }
        return ONE_OK;
    }

    // Ordering (host/net.h:275-319, here a ready-list pass) + shape inference with the batch rule
    // + the residual fusion.
    int build_graph()
    {
        std::set<std::string> ready(init_operands_list.begin(), init_operands_list.end());
        for (auto &o : io_ops) {
            io *p = static_cast<io *>(o.get());
            if (p->op_name == "input") {
                OPERAND_S d = p->io_cfg.operand;
                if (d.shapes[0] == 1) d.shapes[0] = opt.batch;   // the batch rule
                operand_stu_map[d.operand_name] = d;
                ready.insert(d.operand_name);
                input_names.push_back(d.operand_name);
            } else {
                output_names.push_back(p->io_cfg.operand.operand_name);
            }
        }
        std::vector<std::shared_ptr<op>> pending = node_ops;
        while (!pending.empty()) {
            bool progressed = false;
            for (size_t i = 0; i < pending.size(); ++i) {
                bool ok = true;
                for (auto &n : pending[i]->in_operands) ok = ok && (n.empty() || ready.count(n));
                if (!ok) continue;
                for (auto &n : pending[i]->out_operands) ready.insert(n);
                op_exec_order.push_back(pending[i]);
                pending.erase(pending.begin() + i);
                progressed = true;
                break;
            }
            if (!progressed) return fail_("graph has a cycle or an operator reads an operand nothing produces");
        }
        for (auto &o : op_exec_order) {
            for (auto &n : o->out_operands) {
                OPERAND_S d;
                memset(&d, 0, sizeof(d));
                strncpy(d.operand_name, n.c_str(), OPERAND_NAME_LEN - 1);
                operand_stu_map[n] = d;
            }
            int rc = o->shape_infer(operand_stu_map);
            if (rc != ONE_OK) return fail_("shape inference failed at " + o->op_type + " '" + o->op_name + "'");
        }
        for (auto &n : output_names)
            if (!operand_stu_map.count(n)) return fail_("network output '" + n + "' is produced by no operator");
        if (opt.fuse_residual) {
            fuse_residual_adds();
            fuse_int8_requant();
            fuse_conv_tokens();
            fuse_attention();
            fuse_linear_chains();
            if (opt.precision == ONE_PREC_BF16) mark_residual_trunk();
        }
        return ONE_OK;
    }

    extractor *create_exe(one_ctx *ctx)
    {
        exc_cls.reset(new extractor(this));
        exc_cls->ctx = ctx;
        exc_cls->stream = (cudaStream_t)one_cuda_stream(ctx);
        return exc_cls.get();
    }

    static int elem_size_of(int dt)   // common/nn_common.h:619-637
    {
        switch (dt) {
        case TYPE_INT8: case TYPE_UINT8: case TYPE_BOOLEAN: return 1;
        case TYPE_INT16: case TYPE_UINT16: case TYPE_FP16: case TYPE_BF16: return 2;
        case TYPE_INT64: case TYPE_UINT64: case TYPE_FP64: return 8;
        default: return 4;
        }
    }

private:
    int fail_(const std::string &m)
    {
        error = m;
        return ONE_ERR_BAD_ARG;
    }

    struct UseMaps {
        std::unordered_map<std::string, std::vector<op *>> consumers;
        std::unordered_map<std::string, op *> producer;
    };
    UseMaps use_maps()
    {
        UseMaps u;
        for (auto &o : op_exec_order) {
            if (o->skipped) continue;
            for (auto &n : o->in_operands)
                if (!n.empty()) u.consumers[n].push_back(o.get());
            if (!o->residual.empty()) u.consumers[o->residual].push_back(o.get());
            for (auto &n : o->out_operands) u.producer[n] = o.get();
        }
        for (auto &n : output_names) u.consumers[n].push_back(nullptr);   // network outputs stay materialised
        return u;
    }
    size_t position_of(const op *p) const
    {
        size_t i = 0;
        while (op_exec_order[i].get() != p) ++i;
        return i;
    }

    // bf16 mode.  Rounding every activation to bf16 costs 2^-9 per layer, and along the identity path of a
    // residual network those roundings add up block after block until deep layers leave the float
    // tolerance.  The trunk -- the output of every conv that folded an Add, and the other operand of that
    // Add when a conv produces it (the projection shortcut) -- therefore stays fp32, and so does the input
    // of the conv that writes it; the remaining activations inside a block are bf16.
    void mark_residual_trunk()
    {
        UseMaps u = use_maps();
        for (auto &o : op_exec_order) {
            if (o->skipped || o->op_type != "Conv" || o->residual.empty()) continue;
            o->keep_f32 = true;
            auto it = u.producer.find(o->residual);
            if (it != u.producer.end() && it->second->op_type == "Conv") it->second->keep_f32 = true;
            // ... and so does the input of the conv that writes the trunk: that conv then multiplies in tf32
            // with fp32 weights, so what reaches the trunk has passed through one bf16 rounding, not two
            it = u.producer.find(o->in_operands[0]);
            if (it != u.producer.end() && it->second->op_type == "Conv" && static_cast<Conv *>(it->second)->conv_cfg.group == 1) it->second->keep_f32 = true;
        }
    }

    // Conv -> int8 Conv with nothing else reading the operand between them: the producer's epilogue
    // quantises with the consumer's input_scale (the arithmetic of conv.c:961-973, applied to the
    // same fp32 value) and writes int8 NHWC; the fp32 activation is never stored.
    void fuse_int8_requant()
    {
        UseMaps u = use_maps();
        for (auto &o : op_exec_order) {
            if (o->op_type != "Conv" || o->skipped) continue;
            Conv *d = static_cast<Conv *>(o.get());
            if (d->conv_cfg.ifmap_quant2 != TYPE_INT8 || d->conv_cfg.group != 1) continue;
            const std::string &x = d->in_operands[0];
            auto pit = u.producer.find(x);
            auto cit = u.consumers.find(x);
            if (pit == u.producer.end() || pit->second->op_type != "Conv" || cit == u.consumers.end() || cit->second.size() != 1) continue;
            Conv *p = static_cast<Conv *>(pit->second);
            if (p->conv_cfg.group != 1 || p->out_int8) continue;
            const int oc = p->y_desc.shapes[1];
            if (oc % 32 != 0 || !(d->conv_cfg.input_scale > 0.f)) continue;   // int8 NHWC rows must be tensor-map addressable
            p->out_int8 = true;
            p->out_q_scale = d->conv_cfg.input_scale;
            d->in_int8 = true;
        }
    }

    // Conv -> Reshape[N, OC, OH*OW] -> Transpose(0, 2, 1) (a patch embedding turned into a token
    // sequence): the conv's NHWC output already is that [N][OH*OW][OC] tensor, so the two re-layouts
    // vanish and the conv takes over the Transpose's operand.
    void fuse_conv_tokens()
    {
        UseMaps u = use_maps();
        auto only_consumer = [&](const std::string &n, const char *type) -> op * {
            auto it = u.consumers.find(n);
            if (it == u.consumers.end() || it->second.size() != 1 || !it->second[0] || it->second[0]->op_type != type) return nullptr;
            return it->second[0];
        };
        for (auto &o : op_exec_order) {
            if (o->op_type != "Conv" || o->skipped) continue;
            Conv *c = static_cast<Conv *>(o.get());
            if (c->conv_cfg.group != 1 || !c->residual.empty() || c->conv_cfg.ifmap_quant2 == TYPE_INT8) continue;
            op *r = only_consumer(c->out_operands[0], "Reshape");
            if (!r) continue;
            op *t = only_consumer(r->out_operands[0], "Transpose");
            if (!t) continue;
            const OPERAND_S &y = c->y_desc, &rd = operand_stu_map[r->out_operands[0]];
            const Transpose *tr = static_cast<const Transpose *>(t);
            if (rd.dim_num_of_shapes != 3 || rd.shapes[0] != y.shapes[0] || rd.shapes[1] != y.shapes[1] ||
                rd.shapes[2] != y.shapes[2] * y.shapes[3])
                continue;
            if (tr->cfg.perm_num != 3 || tr->cfg.perm[0] != 0 || tr->cfg.perm[1] != 2 || tr->cfg.perm[2] != 1) continue;
            c->tokens_out = true;
            c->out_operands[0] = t->out_operands[0];
            r->skipped = true;
            t->skipped = true;
        }
    }

    // Self-attention of one transformer block, as the converter leaves it:
    //   X4 = [B][T][3][D] view of the fused qkv tensor
    //   q = Transpose(0,2,1,3)(Reshape[B,T,H,hd](Gather(X4, axis 2, iq)))  [* scalar]
    //   k = Transpose(0,2,3,1)(Reshape(Gather(X4, axis 2, ik)));  v like q
    //   out = Reshape[B,T,D](Transpose(0,2,1,3)(MatMul(Softmax(MatMul(q, k)), v)))
    // with every intermediate read once.  The whole chain becomes one Attention operator that reads X4
    // and writes `out`; scores and probabilities never reach memory.
    void fuse_attention()
    {
        std::vector<op *> softmaxes;
        for (auto &o : op_exec_order)
            if (o->op_type == "Softmax" && !o->skipped) softmaxes.push_back(o.get());
        for (op *sm : softmaxes) {
            UseMaps u = use_maps();
            auto producer_of = [&](const std::string &n, const char *type) -> op * {
                auto it = u.producer.find(n);
                if (it == u.producer.end() || it->second->op_type != type || it->second->skipped) return nullptr;
                auto c = u.consumers.find(n);
                return (c != u.consumers.end() && c->second.size() == 1) ? it->second : nullptr;   // read once
            };
            auto only_consumer = [&](const std::string &n, const char *type) -> op * {
                auto it = u.consumers.find(n);
                if (it == u.consumers.end() || it->second.size() != 1 || !it->second[0] || it->second[0]->op_type != type) return nullptr;
                return it->second[0];
            };
            auto perm_is = [](const op *t, std::initializer_list<int> want) {
                const Transpose *tr = static_cast<const Transpose *>(t);
                if (tr->cfg.perm_num != (int64_t)want.size()) return false;
                int i = 0;
                for (int w : want)
                    if (tr->cfg.perm[i++] != w) return false;
                return true;
            };
            std::vector<op *> chain;
            // head split of one of q / k / v: returns the Gather, sets the index and X4
            std::string x4;
            int H = 0, hd = 0;
            auto head_split = [&](const std::string &operand, bool k_side, int *idx) -> bool {
                op *t = producer_of(operand, "Transpose");
                if (!t || !(k_side ? perm_is(t, {0, 2, 3, 1}) : perm_is(t, {0, 2, 1, 3}))) return false;
                op *r = producer_of(t->in_operands[0], "Reshape");
                if (!r) return false;
                const OPERAND_S &rd = operand_stu_map[r->out_operands[0]];
                if (rd.dim_num_of_shapes != 4) return false;
                op *g = producer_of(r->in_operands[0], "Gather");
                if (!g) return false;
                const Gather *gg = static_cast<const Gather *>(g);
                if (gg->cfg.indices_from_ifmap || gg->cfg.axis != 2) return false;
                const OPERAND_S &xd = operand_stu_map[g->in_operands[0]];
                if (xd.dim_num_of_shapes != 4 || xd.shapes[1] != rd.shapes[1] || rd.shapes[2] * rd.shapes[3] != xd.shapes[3]) return false;
                if (!x4.empty() && (x4 != g->in_operands[0] || H != rd.shapes[2] || hd != rd.shapes[3])) return false;
                x4 = g->in_operands[0];
                H = rd.shapes[2];
                hd = rd.shapes[3];
                *idx = (int)gg->cfg.indices;
                chain.push_back(t); chain.push_back(r); chain.push_back(g);
                return true;
            };
            op *qk = producer_of(sm->in_operands[0], "MatMul");
            if (!qk || static_cast<GemmLike *>(qk)->weight || qk->in_operands.size() != 2) continue;
            op *pv = only_consumer(sm->out_operands[0], "MatMul");
            if (!pv || static_cast<GemmLike *>(pv)->weight || pv->in_operands[0] != sm->out_operands[0]) continue;
            const Softmax *smx = static_cast<const Softmax *>(sm);
            if (!(smx->cfg.axis == -1 || smx->cfg.axis == 3)) continue;
            float scale = 1.f;
            std::string q_operand = qk->in_operands[0];
            if (op *mul = producer_of(q_operand, "Mul")) {   // q * scalar constant
                const Mul *m = static_cast<const Mul *>(mul);
                const int ci = m->init[0] ? 0 : 1;
                if (!m->init[ci] || m->init[1 - ci] || operand_elem_size(m->init[ci]->desc) != 1) continue;
                scale = *reinterpret_cast<const float *>(m->init[ci]->data);
                q_operand = mul->in_operands[1 - ci];
                chain.push_back(mul);
            }
            int iq = 0, ik = 0, iv = 0;
            if (!head_split(q_operand, false, &iq) || !head_split(qk->in_operands[1], true, &ik) ||
                !head_split(pv->in_operands[1], false, &iv))
                continue;
            op *tc = only_consumer(pv->out_operands[0], "Transpose");
            if (!tc || !perm_is(tc, {0, 2, 1, 3})) continue;
            op *rc = only_consumer(tc->out_operands[0], "Reshape");
            if (!rc) continue;
            const OPERAND_S &xd = operand_stu_map[x4];
            const OPERAND_S &od = operand_stu_map[rc->out_operands[0]];
            const int T = xd.shapes[1], D = xd.shapes[3];
            if (od.dim_num_of_shapes != 3 || od.shapes[1] != T || od.shapes[2] != D || T > 256 || D % 32 != 0 ||
                !(hd == 32 || hd == 64) || !(scale > 0.f))
                continue;
            chain.push_back(qk); chain.push_back(sm); chain.push_back(pv); chain.push_back(tc);
            auto at = std::make_shared<Attention>();
            at->op_type = "Attention";
            at->op_name = sm->op_name + "/fused";
            at->in_operands.push_back(x4);
            at->out_operands.push_back(rc->out_operands[0]);
            at->heads = H; at->hd = hd; at->q_idx = iq; at->k_idx = ik; at->v_idx = iv; at->scale = scale;
            for (op *c : chain) c->skipped = true;
            const size_t pos = position_of(rc);
            rc->skipped = true;
            op_exec_order.insert(op_exec_order.begin() + pos, at);
        }
    }

    // MatMul(constant B) -> Add(constant vector of length N) [-> Gelu] [-> Add(activation of equal shape)],
    // each intermediate with a single consumer: the GEMM applies the bias, the table activation and
    // the residual in its epilogue and takes over the chain's last operand.  When a residual is
    // folded the GEMM moves to that Add's slot, where the other operand is known to be ready.
    void fuse_linear_chains()
    {
        UseMaps u = use_maps();
        auto only_consumer = [&](const std::string &n) -> op * {
            auto it = u.consumers.find(n);
            return (it != u.consumers.end() && it->second.size() == 1) ? it->second[0] : nullptr;
        };
        std::vector<op *> mats;
        for (auto &o : op_exec_order)
            if (o->op_type == "MatMul" && !o->skipped && static_cast<GemmLike *>(o.get())->weight) mats.push_back(o.get());
        for (op *mo : mats) {
            GemmLike *m = static_cast<GemmLike *>(mo);
            const int N = m->weight->desc->shapes[m->weight->desc->dim_num_of_shapes - 1];
            std::string cur = m->out_operands[0];
            op *c = only_consumer(cur);
            if (c && c->op_type == "Add") {
                Add *a = static_cast<Add *>(c);
                for (int i = 0; i < 2; ++i) {
                    const OneImage::Init *v = a->init[i];
                    if (!v || a->in_operands[1 - i] != cur) continue;
                    const OPERAND_S *d = v->desc;
                    if (operand_elem_size(d) == N && d->shapes[d->dim_num_of_shapes - 1] == N) {
                        m->fused_bias = v;
                        a->skipped = true;
                        cur = a->out_operands[0];
                    }
                }
            }
            if (!m->fused_bias) continue;   // the epilogue order is bias, activation, residual
            c = only_consumer(cur);
            if (c && c->op_type == "Gelu") {
                m->fuse_gelu = true;
                c->skipped = true;
                cur = c->out_operands[0];
            }
            c = only_consumer(cur);
            if (c && c->op_type == "Add") {
                Add *a = static_cast<Add *>(c);
                const bool acts = !a->init[0] && !a->init[1] && a->in_operands[0] != a->in_operands[1];
                bool equal = acts;
                for (int i = 0; equal && i < SHAPE_LEN; ++i)
                    equal = operand_stu_map[a->in_operands[0]].shapes[i] == operand_stu_map[a->in_operands[1]].shapes[i];
                if (equal) {
                    m->residual = a->in_operands[a->in_operands[0] == cur ? 1 : 0];
                    a->skipped = true;
                    cur = a->out_operands[0];
                    const size_t from = position_of(m), to = position_of(a);
                    std::shared_ptr<op> keep = op_exec_order[from];
                    op_exec_order.erase(op_exec_order.begin() + from);
                    op_exec_order.insert(op_exec_order.begin() + (to - 1), keep);
                }
            }
            m->out_operands[0] = cur;
        }
    }

    // Conv -> Add [-> Relu] with single consumers: the conv adds the other Add input in its
    // epilogue and takes over the chain's final operand.  The conv is moved to the Add's slot in
    // the execution order, where both of its operands are known to be ready.
    void fuse_residual_adds()
    {
        std::unordered_map<std::string, std::vector<op *>> consumers;
        std::unordered_map<std::string, op *> producer;
        for (auto &o : op_exec_order) {
            for (auto &n : o->in_operands)
                if (!n.empty()) consumers[n].push_back(o.get());
            for (auto &n : o->out_operands) producer[n] = o.get();
        }
        for (auto &n : output_names) consumers[n].push_back(nullptr);   // network outputs stay materialised
        for (size_t ai = 0; ai < op_exec_order.size(); ++ai) {
            op *a = op_exec_order[ai].get();
            if (a->op_type != "Add" || a->skipped || a->in_operands.size() != 2) continue;
            {   // only the equal-shape sum of two activations folds into a conv epilogue
                const Add *ad = static_cast<const Add *>(a);
                bool equal = !ad->init[0] && !ad->init[1];
                for (int i = 0; equal && i < SHAPE_LEN; ++i)
                    equal = operand_stu_map[a->in_operands[0]].shapes[i] == operand_stu_map[a->in_operands[1]].shapes[i];
                if (!equal) continue;
            }
            int pick = -1;
            size_t pick_pos = 0;
            for (int i = 0; i < 2; ++i) {
                auto it = producer.find(a->in_operands[i]);
                if (it == producer.end() || it->second->op_type != "Conv") continue;
                Conv *c = static_cast<Conv *>(it->second);
                if (!c->residual.empty() || c->skipped || c->conv_cfg.group != 1 || consumers[a->in_operands[i]].size() != 1) continue;
                if (a->in_operands[0] == a->in_operands[1]) continue;
                size_t pos = 0;
                while (op_exec_order[pos].get() != c) ++pos;
                if (pick < 0 || pos > pick_pos) { pick = i; pick_pos = pos; }
            }
            if (pick < 0) continue;
            Conv *c = static_cast<Conv *>(producer[a->in_operands[pick]]);
            c->residual = a->in_operands[1 - pick];
            std::string final_out = a->out_operands[0];
            a->skipped = true;
            auto &cons = consumers[final_out];
            if (cons.size() == 1 && cons[0] && cons[0]->op_type == "Relu") {
                c->fuse_relu = true;
                cons[0]->skipped = true;
                final_out = cons[0]->out_operands[0];
            }
            c->out_operands[0] = final_out;
            producer[final_out] = c;
            // move the conv to the Add's slot
            std::shared_ptr<op> keep = op_exec_order[pick_pos];
            op_exec_order.erase(op_exec_order.begin() + pick_pos);
            op_exec_order.insert(op_exec_order.begin() + (ai - 1), keep);   // the Add moved one slot left; the conv goes right before it
        }
    }
};

// ------------------------------------------------------------------------------------------ extractor
inline extractor::~extractor()
{
    if (graph_exec) cudaGraphExecDestroy(graph_exec);
    if (arena) cudaFree(arena);
}

inline int extractor::plan()
{
    net &n = *net_ptr;
    tensors.clear();
    steps.clear();
    for (auto &name : n.input_names) {
        TensorInfo t;
        t.desc = n.operand_stu_map[name];
        t.layout = LAYOUT_PLAIN;
        t.dtype = DT_F32;
        tensors[name] = t;
    }
    auto plain_name = [](const std::string &s) { return s + "#plain"; };
    auto ensure_plain = [&](const std::string &src) -> std::string {
        const TensorInfo &t = tensors[src];
        if (t.layout == LAYOUT_PLAIN && t.dtype == DT_F32) return src;
        const std::string dst = plain_name(src);
        if (!tensors.count(dst)) {
            TensorInfo p;
            p.desc = t.desc;
            p.layout = LAYOUT_PLAIN;
            p.dtype = DT_F32;
            tensors[dst] = p;
            Step s;
            s.kind = (t.layout == LAYOUT_NHWC) ? Step::TO_PLAIN : Step::CAST_F32;
            s.src = src;
            s.dst = dst;
            steps.push_back(s);
        }
        return dst;
    };
    for (auto &sp : n.op_exec_order) {
        op *o = sp.get();
        if (o->skipped) continue;
        std::vector<std::string> acts = o->act_inputs(n.init_operands_list);
        if (!o->residual.empty()) acts.push_back(o->residual);
        std::vector<const TensorInfo *> ins;
        for (auto &a : acts) {
            if (!tensors.count(a)) { error = "operand '" + a + "' used before it is produced"; return ONE_ERR_BAD_ARG; }
            ins.push_back(&tensors[a]);
        }
        TensorInfo out;
        out.desc = n.operand_stu_map[o->out_operands[0]];
        std::vector<bool> need_plain(ins.size(), false);
        o->plan(ins, n.opt, &out, &need_plain);
        bool changed = false;
        for (size_t i = 0; i < acts.size(); ++i) {
            if (!need_plain[i]) continue;
            const std::string p = ensure_plain(acts[i]);
            if (p != acts[i]) {
                for (auto &nm : o->in_operands)
                    if (nm == acts[i]) nm = p;
                acts[i] = p;
                changed = true;
            }
        }
        if (changed) {   // re-plan against the converted inputs
            ins.clear();
            for (auto &a : acts) ins.push_back(&tensors[a]);
            std::vector<bool> np(ins.size(), false);
            o->plan(ins, n.opt, &out, &np);
        }
        if (!o->residual.empty()) {
            // The folded Add's other operand must have the physical form the epilogue writes.  A skip
            // connection from the network input or from a plain-layout operator (Reshape, Transpose) does
            // not: it gets a converted copy first, so such graphs run as they do in the reference.
            const TensorInfo r = tensors[o->residual];
            const int want_dt = out.dtype == DT_S8 ? DT_F32 : out.dtype;   // an int8-chain producer adds in fp32 before it quantises
            if (r.layout != out.layout || r.dtype != want_dt) {
                Step cv;
                if (r.layout == LAYOUT_PLAIN && r.dtype == DT_F32 && out.layout == LAYOUT_NHWC && r.desc.dim_num_of_shapes == 4) cv.kind = Step::TO_NHWC;
                else if (r.layout == out.layout && ((r.dtype == DT_F32 && (want_dt == DT_BF16 || want_dt == DT_F16)) || ((r.dtype == DT_BF16 || r.dtype == DT_F16) && want_dt == DT_F32))) cv.kind = Step::CAST;
                else { error = "fused residual of '" + o->op_name + "' cannot be brought into the operator's output form"; return ONE_ERR_UNSUPPORTED; }
                cv.src = o->residual;
                cv.dst = o->residual + (out.layout == LAYOUT_NHWC ? "#nhwc" : "#cast") + std::to_string(want_dt);
                if (!tensors.count(cv.dst)) {
                    TensorInfo c;
                    c.desc = r.desc;
                    c.layout = out.layout;
                    c.dtype = want_dt;
                    tensors[cv.dst] = c;
                    steps.push_back(cv);
                }
                o->residual = cv.dst;
            }
        }
        if (!out.alias_of.empty()) out.alias_of = o->in_operands[0];
        tensors[o->out_operands[0]] = out;
        Step s;
        s.kind = Step::RUN_OP;
        s.o = o;
        steps.push_back(s);
    }
    // network outputs are handed back in the reference layout, fp32
    for (auto &name : n.output_names) ensure_plain(name);
    return ONE_OK;
}

inline int extractor::new_output_buf()
{
    size_t total = 0;
    std::vector<std::pair<std::string, size_t>> offs;
    for (auto &kv : tensors) {
        TensorInfo &t = kv.second;
        if (!t.alias_of.empty()) continue;
        t.bytes = (size_t)operand_elem_size(&t.desc) * dtype_size(t.dtype);
        offs.push_back({kv.first, total});
        total += (t.bytes + 1023) & ~size_t(1023);
    }
    arena_bytes = total ? total : 1024;
    cudaError_t e = cudaMalloc(&arena, arena_bytes);
    if (e != cudaSuccess) { error = std::string("arena cudaMalloc: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
    for (auto &p : offs) tensors[p.first].dev = arena + p.second;
    // views
    for (int pass = 0; pass < 4; ++pass)
        for (auto &kv : tensors)
            if (!kv.second.alias_of.empty() && !kv.second.dev) {
                kv.second.dev = tensors[kv.second.alias_of].dev;
                kv.second.bytes = tensors[kv.second.alias_of].bytes;
            }
    return ONE_OK;
}

inline int extractor::prepare_for_op()
{
    net &n = *net_ptr;
    for (auto &s : steps) {
        if (s.kind != Step::RUN_OP) continue;
        op *o = s.o;
        std::vector<std::string> acts = o->act_inputs(n.init_operands_list);
        std::vector<const TensorInfo *> ins;
        for (auto &a : acts) ins.push_back(&tensors[a]);
        int rc = o->prepare(ctx, n.opt, ins, tensors[o->out_operands[0]]);
        if (rc != ONE_OK) { error = "prepare failed at " + o->op_type + " '" + o->op_name + "': " + one_cuda_last_error(); return rc; }
        if ((rc = o->rt_prepare(tensors, n.init_operands_list)) != ONE_OK) { error = "rt_prepare failed at " + o->op_name; return rc; }
    }
    return ONE_OK;
}

inline int extractor::run_step(const Step &s)
{
    int rc;
    if (s.kind == Step::RUN_OP) rc = s.o->forward(ctx, stream);
    else {
        const TensorInfo &src = tensors[s.src];
        TensorInfo &dst = tensors[s.dst];
        if (s.kind == Step::TO_PLAIN) {
            const int hw = src.desc.shapes[2] * src.desc.shapes[3];
            rc = one_glue_to_nchw_f32(src.dev, (float *)dst.dev, src.dtype, src.desc.shapes[0], src.desc.shapes[1], hw, stream);
        } else if (s.kind == Step::TO_NHWC) {
            const int hw = src.desc.shapes[2] * src.desc.shapes[3];
            rc = one_glue_to_nhwc((const float *)src.dev, dst.dev, dst.dtype, src.desc.shapes[0], src.desc.shapes[1], hw, stream);
        } else {
            rc = one_glue_cast(src.dev, dst.dev, src.dtype, dst.dtype, operand_elem_size(&src.desc), stream);
        }
    }
    if (rc != ONE_OK)
        error = std::string("step failed (") + (s.o ? s.o->op_type + " '" + s.o->op_name + "'" : s.src) + "): " + one_cuda_last_error();
    return rc;
}

inline int extractor::enqueue()
{
    for (auto &s : steps) {
        int rc = run_step(s);
        if (rc != ONE_OK) return rc;
    }
    return ONE_OK;
}

inline int extractor::impl(bool use_graph)
{
    if (!ran_eager || !use_graph) {
        const unsigned long long before = one_cuda_launch_count();
        int rc = enqueue();
        if (rc != ONE_OK) return rc;
        launches_per_run = one_cuda_launch_count() - before;
        ran_eager = true;
        return ONE_OK;
    }
    if (!graph_exec) {
        cudaGraph_t g = nullptr;
        cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) { error = std::string("begin capture: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
        int rc = enqueue();
        e = cudaStreamEndCapture(stream, &g);
        if (rc != ONE_OK) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) { error = std::string("end capture: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
        e = cudaGraphInstantiate(&graph_exec, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) { error = std::string("graph instantiate: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
    }
    cudaError_t e = cudaGraphLaunch(graph_exec, stream);
    if (e != cudaSuccess) { error = std::string("graph launch: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
    return ONE_OK;
}

inline int extractor::prepare_one(op *o)
{
    net &n = *net_ptr;
    std::vector<std::string> acts = o->act_inputs(n.init_operands_list);
    std::vector<const TensorInfo *> ins;
    for (auto &a : acts) ins.push_back(&tensors[a]);
    o->drop_prepared();
    int rc = o->prepare(ctx, n.opt, ins, tensors[o->out_operands[0]]);
    if (rc != ONE_OK) { error = "prepare failed at " + o->op_type + " '" + o->op_name + "': " + one_cuda_last_error(); return rc; }
    if ((rc = o->rt_prepare(tensors, n.init_operands_list)) != ONE_OK) { error = "rt_prepare failed at " + o->op_name; return rc; }
    if (graph_exec) { cudaGraphExecDestroy(graph_exec); graph_exec = nullptr; }   // the captured step holds the old operator
    return ONE_OK;
}

inline int extractor::set_tile(const std::string &op_name, int bn)
{
    if (bn != 0 && bn != 64 && bn != 128 && bn != 192 && bn != 256 && bn != 1128 && bn != 1192 && bn != 1256 && bn != 2064 && bn != 2128 && bn != 4064 && bn != 4128) {
        error = "tile must be 0, 64, 128, 192, 256, 1128 / 1192 / 1256 (the width plus 1000: pairs of CTAs sharing 256-row tiles) , 2064 / 2128 (plus 2000: two 128-row halves per CTA) or 4064 / 4128 (plus 4000: twelve epilogue warps)";
        return ONE_ERR_BAD_ARG;
    }
    for (auto &s : steps)
        if (s.kind == Step::RUN_OP && s.o->op_name == op_name) {
            if (!s.o->tunable()) { error = "operator '" + op_name + "' has no selectable tile"; return ONE_ERR_UNSUPPORTED; }
            cudaStreamSynchronize(stream);
            s.o->tile_n = bn;
            return prepare_one(s.o);
        }
    error = "no operator named '" + op_name + "'";
    return ONE_ERR_BAD_ARG;
}

// Tile search on the model's own operators, the device counterpart of the reference's grid search over
// GEMM tiles (tools/optimize/auto_tuning.hpp:9-75: time every candidate, keep a new one only when it beats
// the best so far by 2 %).  Each Conv / Gemm / MatMul with a packed weight is timed with CUDA events at
// every output-tile width the kernel has (the heuristic's choice first, so that it wins ties) on the
// operands of the last inference, and is left prepared with the winner.  `report` gets one CSV line per
// operator: name, type, output width, heuristic us, best tile, best us, best split-K choice (0: the
// library's own, 1: never, n: n ranges).
inline int extractor::autotune(int runs, std::string *report)
{
    if (!ran_eager) { error = "autotune needs one inference first (the operands it times on)"; return ONE_ERR_BAD_ARG; }
    if (runs < 1) runs = 1;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaStreamSynchronize(stream);
    if (report) *report = "op_name,op_type,out_width,heuristic_us,best_tile_n,best_us,best_split_k\n";
    int rc = ONE_OK;
    auto time_op = [&](op *o, double *us) -> int {
        // two measurements, the faster one counts: a candidate must not win or lose on a clock wobble
        double a = 0, b = 0;
        int r = time_in_graph([&]() { return o->forward(ctx, stream); }, runs, e0, e1, &a);
        if (r == ONE_OK) r = time_in_graph([&]() { return o->forward(ctx, stream); }, runs, e0, e1, &b);
        if (r != ONE_OK) return r;
        *us = a < b ? a : b;
        return one_cuda_status(ctx);
    };
    for (auto &s : steps) {
        if (s.kind != Step::RUN_OP || !s.o->tunable()) continue;
        op *o = s.o;
        const int width = o->out_width();
        // tile codes: the four widths, three of them run as pairs of CTAs (code = width + 1000), and the two
        // narrow ones with two 128-row halves per CTA (code = width + 2000) or with twelve epilogue warps (+ 4000)
        const int cand[12] = {0, 64, 128, 192, 256, 1128, 1192, 1256, 2064, 2128, 4064, 4128};
        // split-K choices tried per width: the library's own (0), never (1), and a few forced counts, which
        // only matter for launches short enough that idle SMs and pipeline fill dominate
        const int splits[6] = {0, 1, 2, 3, 4, 8};
        double best_us = 1e30, heur_us = 0;
        int best = 0, best_split = 0;
        for (int c = 0; c < 12 && rc == ONE_OK; ++c) {
            const int bn = cand[c];
            if (bn % 1000 > 64 && bn % 1000 >= width + 64) continue;   // wider than the output by a whole narrower tile: never better
            o->tile_n = bn;
            o->split_k = 0;
            if (prepare_one(o) != ONE_OK) continue;      // a width this operator cannot take
            for (int si = 0; si < 6; ++si) {
                if (si > 1 && heur_us > 150.0) break;    // a long launch fills the GPU without splitting
                if (si > 0 && bn >= 1000) break;         // pairs of CTAs and two-half tiles do not split K
                o->split_k = splits[si];
                if (o->set_split() != ONE_OK) continue;
                double us = 0;
                if ((rc = time_op(o, &us)) != ONE_OK) { error = "autotune: '" + o->op_name + "' failed: " + one_cuda_last_error(); break; }
                if (bn == 0 && si == 0) heur_us = us;
                if (us < 0.98 * best_us) { best_us = us; best = bn; best_split = splits[si]; }
            }
        }
        if (rc != ONE_OK) break;
        o->tile_n = best;
        o->split_k = best_split;
        if ((rc = prepare_one(o)) != ONE_OK) break;
        if (report) {
            char line[512];
            snprintf(line, sizeof(line), "%s,%s,%d,%.2f,%d,%.2f,%d\n", o->op_name.c_str(), o->op_type.c_str(), width, heur_us, best, best_us, best_split);
            *report += line;
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

// Device time of `fn` (something that enqueues work on `stream`): `runs` repetitions are captured into one
// CUDA graph, the graph is launched once to warm up and once between two events.  No host enqueue cost
// is in the figure, and consecutive repetitions overlap the way consecutive operators of a replayed
// step do.
template <typename F>
inline int extractor::time_in_graph(F fn, int runs, cudaEvent_t e0, cudaEvent_t e1, double *us)
{
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    int rc = ONE_OK;
    cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) { error = std::string("begin capture: ") + cudaGetErrorString(e); return ONE_ERR_CUDA; }
    for (int r = 0; r < runs && rc == ONE_OK; ++r) rc = fn();
    e = cudaStreamEndCapture(stream, &g);
    if (rc == ONE_OK && e != cudaSuccess) { error = std::string("end capture: ") + cudaGetErrorString(e); rc = ONE_ERR_CUDA; }
    if (rc == ONE_OK && (e = cudaGraphInstantiate(&ge, g, 0)) != cudaSuccess) { error = std::string("graph instantiate: ") + cudaGetErrorString(e); rc = ONE_ERR_CUDA; }
    if (rc == ONE_OK) {
        cudaGraphLaunch(ge, stream);   // warm-up
        cudaEventRecord(e0, stream);
        cudaGraphLaunch(ge, stream);
        cudaEventRecord(e1, stream);
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) { error = cudaGetErrorString(e); rc = ONE_ERR_CUDA; }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        *us = ms * 1000.0 / runs;
    }
    if (ge) cudaGraphExecDestroy(ge);
    if (g) cudaGraphDestroy(g);
    return rc;
}

// One row of the tracing table.
struct TraceRow {
    std::string name, type, detail;
    double st_us = 0, ed_us = 0, mflop = 0, bytes = 0;
};

// The tracing CSV in the reference's schema (host/net.h:539-611): header
//   op_name,op_type,op_st,op_ed,op_computation,,cpu,cpu_hw_info,gpu,gpu_hw_info,hw_computing_power (GOPS),model name
// with times in microseconds and work in MFLOP; the hardware and model fields sit in columns 6..11 of
// the FIRST data row only, where the reference's timeline tool looks for them
// (tools/perf_profiling/gen_timeline_json.py:41-42 takes hw_computing_power from column 10 of that row).
// Two columns are appended after the reference's twelve: the operator's compulsory bytes and a free-form
// detail string (shape, tile); the reference tool ignores them.
inline int write_trace_csv(const char *path, const std::vector<TraceRow> &rows, const std::string &gpu, const std::string &gpu_hw_info,
                           double hw_gops, const std::string &model_name)
{
    FILE *f = fopen(path, "w");
    if (!f) return ONE_ERR_BAD_ARG;
    auto clean = [](std::string v) {   // the reference tool splits on commas and has no quoting
        for (auto &c : v)
            if (c == ',' || c == '\n' || c == '\r') c = ';';
        return v;
    };
    fprintf(f, "op_name,op_type,op_st,op_ed,op_computation,,cpu,cpu_hw_info,gpu,gpu_hw_info,hw_computing_power (GOPS),model name,op_bytes,op_detail\n");
    for (size_t i = 0; i < rows.size(); ++i) {
        const TraceRow &r = rows[i];
        fprintf(f, "%s,%s,%.3f,%.3f,%.6f,", clean(r.name).c_str(), clean(r.type).c_str(), r.st_us, r.ed_us, r.mflop);
        if (i == 0) fprintf(f, ",,,%s,%s,%.3f,%s", clean(gpu).c_str(), clean(gpu_hw_info).c_str(), hw_gops, clean(model_name).c_str());
        else fprintf(f, ",,,,,,");
        fprintf(f, ",%.0f,%s\n", r.bytes, clean(r.detail).c_str());
    }
    fclose(f);
    return ONE_OK;
}

// Per-operator timing with CUDA events (the device counterpart of extractor::impl_tracing,
// host/net.h:539-611).  `hw_gops` <= 0 takes the nominal dense tensor peak of the network's precision.
inline int extractor::impl_tracing(const char *csv_path, int runs, const char *model_name, double hw_gops)
{
    // Each step is captured `runs` times back to back into a CUDA graph of its own and that graph is timed
    // with a pair of events: what is measured is device time, free of the host's enqueue cost, which for a
    // small batch is longer than the kernels themselves.  (The reference times operators one by one with a
    // host clock around each synchronous call, host/net.h:578-590.)
    std::vector<double> us(steps.size(), 0.0);
    int rc = ONE_OK;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    if ((rc = enqueue()) == ONE_OK && cudaStreamSynchronize(stream) != cudaSuccess) rc = ONE_ERR_CUDA;   // operands of every step hold real data
    for (size_t i = 0; i < steps.size() && rc == ONE_OK; ++i)
        rc = time_in_graph([&]() { return run_step(steps[i]); }, runs, e0, e1, &us[i]);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != ONE_OK) return rc;
    std::vector<TraceRow> rows(steps.size());
    double t = 0;
    bool int8 = false;
    for (size_t i = 0; i < steps.size(); ++i) {
        const Step &s = steps[i];
        rows[i].name = s.o ? s.o->op_name : s.dst;
        rows[i].type = s.o ? s.o->op_type : (s.kind == Step::TO_PLAIN ? "ToPlain" : (s.kind == Step::TO_NHWC ? "ToNhwc" : "Cast"));
        rows[i].st_us = t;
        rows[i].ed_us = t + us[i];
        rows[i].mflop = s.o ? s.o->get_computation() : 0.0;
        rows[i].bytes = s.o ? s.o->get_bytes() : 0.0;
        if (s.o) rows[i].detail = s.o->describe();
        if (s.o && s.o->op_type == "Conv" && static_cast<Conv *>(s.o)->conv_cfg.ifmap_quant2 == TYPE_INT8) int8 = true;
        t += us[i];
    }
    cudaDeviceProp prop;
    std::string gpu = "gpu", info;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
        gpu = prop.name;
        info = std::to_string(prop.multiProcessorCount) + " SMs sm_" + std::to_string(prop.major) + std::to_string(prop.minor);
    }
    if (hw_gops <= 0)   // nominal dense tensor-core peaks of a B200 in GOPS: tf32, bf16, int8
        hw_gops = int8 ? 4.5e6 : (net_ptr->opt.precision != ONE_PREC_TF32 ? 2.25e6 : 1.1e6);
    if (write_trace_csv(csv_path, rows, gpu, info, hw_gops, model_name ? model_name : "model") != ONE_OK) {
        error = std::string("cannot write ") + csv_path;
        return ONE_ERR_BAD_ARG;
    }
    return ONE_OK;
}

inline int extractor::fetch_plain_f32(const std::string &name, float *host, size_t cap_elems)
{
    auto it = tensors.find(name);
    if (it == tensors.end()) { error = "no operand named '" + name + "'"; return ONE_ERR_BAD_ARG; }
    const TensorInfo &t = it->second;
    const size_t n = (size_t)operand_elem_size(&t.desc);
    if (n > cap_elems) { error = "host buffer too small"; return ONE_ERR_NOMEM; }
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { error = cudaGetErrorString(e); return ONE_ERR_CUDA; }
    if (t.layout == LAYOUT_PLAIN && t.dtype == DT_F32) {
        e = cudaMemcpy(host, t.dev, n * 4, cudaMemcpyDeviceToHost);
    } else {
        float *tmp = nullptr;
        if ((e = cudaMalloc(&tmp, n * 4)) != cudaSuccess) { error = cudaGetErrorString(e); return ONE_ERR_CUDA; }
        int rc = (t.layout == LAYOUT_NHWC)
                     ? one_glue_to_nchw_f32(t.dev, tmp, t.dtype, t.desc.shapes[0], t.desc.shapes[1], t.desc.shapes[2] * t.desc.shapes[3], stream)
                     : one_glue_cast(t.dev, tmp, t.dtype, DT_F32, (long long)n, stream);
        if (rc == ONE_OK) {
            cudaStreamSynchronize(stream);
            e = cudaMemcpy(host, tmp, n * 4, cudaMemcpyDeviceToHost);
        }
        cudaFree(tmp);
        if (rc != ONE_OK) return rc;
    }
    if (e != cudaSuccess) { error = cudaGetErrorString(e); return ONE_ERR_CUDA; }
    return ONE_OK;
}

}  // namespace onenew
