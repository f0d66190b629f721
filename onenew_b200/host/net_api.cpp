// net_api.cpp -- C ABI of the graph runtime (include/one_net.h) over host/net.h.
#include "../../include/one_net.h"

#include <string>

#include "net.h"

using namespace onenew;

struct one_net {
    net n;
    one_ctx *ctx = nullptr;
    extractor *exe = nullptr;
    bool use_graph = true;
    int device = 0;
    std::vector<std::string> plain_outputs;   // device tensors handed back for each network output
    // pipelined host path: the next batch's H2D copy runs on its own stream into a staging buffer
    cudaStream_t copy_stream = nullptr;
    void *staging = nullptr;
    cudaEvent_t ev_h2d = nullptr, ev_free = nullptr;
    bool staged_once = false;
};

static thread_local std::string g_net_err;
static int nfail(int rc, const std::string &m)
{
    g_net_err = m;
    return rc;
}

extern "C" const char *one_net_last_error(void) { return g_net_err.c_str(); }

static int build(one_net *h, int device, int batch, int flags, size_t ws, one_net **out)
{
    int rc;
    if (batch <= 0) { delete h; return nfail(ONE_ERR_BAD_ARG, "batch must be positive"); }
    h->n.opt.batch = batch;
    h->device = device;
    h->n.opt.precision = flags & ONE_PREC_MASK;
    h->n.opt.fuse_residual = !(flags & ONE_NET_NO_FUSE);
    h->use_graph = !(flags & ONE_NET_NO_GRAPH);
    if ((rc = one_cuda_init(device, ws, &h->ctx)) != ONE_OK) { std::string m = one_cuda_last_error(); delete h; return nfail(rc, m); }
    cudaSetDevice(device);
    auto bail = [&](int code, const std::string &m) { one_net_destroy(h); return nfail(code, m); };
    if ((rc = h->n.instantiate_op()) != ONE_OK) return bail(rc, h->n.error);
    if ((rc = h->n.build_graph()) != ONE_OK) return bail(rc, h->n.error);
    h->exe = h->n.create_exe(h->ctx);
    if ((rc = h->exe->plan()) != ONE_OK) return bail(rc, h->exe->error);
    if ((rc = h->exe->new_output_buf()) != ONE_OK) return bail(rc, h->exe->error);
    if ((rc = h->exe->prepare_for_op()) != ONE_OK) return bail(rc, h->exe->error);
    for (auto &name : h->n.output_names) {
        const TensorInfo &t = h->exe->tensors[name];
        h->plain_outputs.push_back((t.layout == LAYOUT_PLAIN && t.dtype == DT_F32) ? name : name + "#plain");
    }
    *out = h;
    return ONE_OK;
}

// Planning only (no device needed): operators in execution order after fusion, with the physical
// form chosen for every output.  One line per step.
extern "C" int one_net_describe(const void *image, size_t size, int batch, int flags, char *buf, size_t cap)
{
    if (!image || !buf || !cap || batch <= 0) return nfail(ONE_ERR_BAD_ARG, "one_net_describe: bad argument");
    net n;
    n.opt.batch = batch;
    n.opt.precision = flags & ONE_PREC_MASK;
    n.opt.fuse_residual = !(flags & ONE_NET_NO_FUSE);
    int rc = n.load_one_buf(static_cast<const char *>(image), size);
    if (rc == ONE_OK) rc = n.instantiate_op();
    if (rc == ONE_OK) rc = n.build_graph();
    if (rc != ONE_OK) return nfail(rc, n.error);
    extractor ex(&n);
    if ((rc = ex.plan()) != ONE_OK) return nfail(rc, ex.error);
    std::string out;
    for (auto &s : ex.steps) {
        char line[1024];
        if (s.kind == Step::RUN_OP) {
            const TensorInfo &t = ex.tensors[s.o->out_operands[0]];
            std::string ins;
            for (auto &i : s.o->in_operands) ins += (ins.empty() ? "" : ",") + i;
            std::string extra;
            if (s.o->op_type == "Conv") {
                Conv *c = static_cast<Conv *>(s.o);
                if (!c->residual.empty()) extra = " residual=" + c->residual + (c->fuse_relu ? " relu=1" : " relu=0");
            }
            snprintf(line, sizeof(line), "RUN %s %s in=%s out=%s shape=%d,%d,%d,%d layout=%s dtype=%s%s\n", s.o->op_type.c_str(),
                     s.o->op_name.c_str(), ins.c_str(), s.o->out_operands[0].c_str(), t.desc.shapes[0], t.desc.shapes[1],
                     t.desc.shapes[2], t.desc.shapes[3], t.layout == LAYOUT_NHWC ? "NHWC" : "PLAIN",
                     t.dtype == DT_F32 ? "f32" : (t.dtype == DT_BF16 ? "bf16" : "s8"), extra.c_str());
        } else {
            snprintf(line, sizeof(line), "%s %s -> %s\n", s.kind == Step::TO_PLAIN ? "TO_PLAIN" : (s.kind == Step::TO_NHWC ? "TO_NHWC" : (s.kind == Step::CAST ? "CAST" : "CAST_F32")), s.src.c_str(), s.dst.c_str());
        }
        out += line;
    }
    if (out.size() + 1 > cap) return nfail(ONE_ERR_NOMEM, "buffer too small");
    memcpy(buf, out.c_str(), out.size() + 1);
    return ONE_OK;
}

extern "C" int one_net_create(const char *path, int device, int batch, int flags, size_t ws, one_net **out)
{
    if (!path || !out) return nfail(ONE_ERR_BAD_ARG, "one_net_create: null argument");
    one_net *h = new one_net();
    int rc = h->n.load_one_model(path);
    if (rc != ONE_OK) { std::string m = h->n.error; delete h; return nfail(rc, m); }
    return build(h, device, batch, flags, ws, out);
}

extern "C" int one_net_create_from_memory(const void *image, size_t size, int device, int batch, int flags, size_t ws,
                                          one_net **out)
{
    if (!image || !out) return nfail(ONE_ERR_BAD_ARG, "one_net_create_from_memory: null argument");
    one_net *h = new one_net();
    int rc = h->n.load_one_buf(static_cast<const char *>(image), size);
    if (rc != ONE_OK) { std::string m = h->n.error; delete h; return nfail(rc, m); }
    return build(h, device, batch, flags, ws, out);
}

extern "C" void one_net_destroy(one_net *h)
{
    if (!h) return;
    if (h->ctx) cudaStreamSynchronize((cudaStream_t)one_cuda_stream(h->ctx));
    if (h->copy_stream) {
        cudaStreamSynchronize(h->copy_stream);
        cudaStreamDestroy(h->copy_stream);
        cudaFree(h->staging);
        cudaEventDestroy(h->ev_h2d);
        cudaEventDestroy(h->ev_free);
    }
    h->n.exc_cls.reset();
    h->n.op_exec_order.clear();
    h->n.node_ops.clear();   // releases the prepared operators before the context
    h->n.io_ops.clear();
    if (h->ctx) one_cuda_release(h->ctx);
    delete h;
}

static const std::vector<std::string> &io_names(one_net *h, int is_output) { return is_output ? h->n.output_names : h->n.input_names; }

extern "C" int one_net_io_count(one_net *h, int is_output) { return h ? (int)io_names(h, is_output).size() : 0; }

extern "C" int one_net_io_info(one_net *h, int is_output, int index, char *name256, int *shape8, int *ndim)
{
    if (!h || index < 0 || index >= (int)io_names(h, is_output).size()) return nfail(ONE_ERR_BAD_ARG, "io index out of range");
    const std::string &nm = io_names(h, is_output)[index];
    const OPERAND_S &d = h->exe->tensors[nm].desc;
    if (name256) snprintf(name256, 256, "%s", nm.c_str());
    if (shape8) for (int i = 0; i < SHAPE_LEN; ++i) shape8[i] = d.shapes[i];
    if (ndim) *ndim = d.dim_num_of_shapes;
    return ONE_OK;
}

extern "C" void *one_net_io_ptr(one_net *h, int is_output, int index)
{
    if (!h || index < 0 || index >= (int)io_names(h, is_output).size()) return nullptr;
    const std::string &nm = is_output ? h->plain_outputs[index] : h->n.input_names[index];
    return h->exe->tensors[nm].dev;
}

extern "C" void *one_net_stream(one_net *h) { return h ? (void *)h->exe->stream : nullptr; }

extern "C" int one_net_run(one_net *h)
{
    if (!h) return nfail(ONE_ERR_BAD_ARG, "null net");
    cudaSetDevice(h->device);
    int rc = h->exe->impl(h->use_graph);
    return rc == ONE_OK ? ONE_OK : nfail(rc, h->exe->error);
}

extern "C" int one_net_sync(one_net *h)
{
    if (!h) return nfail(ONE_ERR_BAD_ARG, "null net");
    int rc = one_cuda_status(h->ctx);
    return rc == ONE_OK ? ONE_OK : nfail(rc, one_cuda_last_error());
}

extern "C" int one_net_run_host(one_net *h, const float *host_in, float *host_out)
{
    if (!h || !host_in || !host_out) return nfail(ONE_ERR_BAD_ARG, "one_net_run_host: null argument");
    cudaSetDevice(h->device);
    const TensorInfo &in = h->exe->tensors[h->n.input_names[0]];
    const TensorInfo &out = h->exe->tensors[h->plain_outputs[0]];
    cudaError_t e = cudaMemcpyAsync(in.dev, host_in, in.bytes, cudaMemcpyHostToDevice, h->exe->stream);
    if (e != cudaSuccess) return nfail(ONE_ERR_CUDA, std::string("input copy: ") + cudaGetErrorString(e));
    int rc = h->exe->impl(h->use_graph);
    if (rc != ONE_OK) return nfail(rc, h->exe->error);
    e = cudaMemcpyAsync(host_out, out.dev, out.bytes, cudaMemcpyDeviceToHost, h->exe->stream);
    if (e != cudaSuccess) return nfail(ONE_ERR_CUDA, std::string("output copy: ") + cudaGetErrorString(e));
    return one_net_sync(h);
}

// Pipelined variant of one_net_run_host: returns without waiting.  The input goes host -> staging
// buffer on a copy stream (overlapping the previous batch's compute), then staging -> network input,
// inference and the output copy on the net's stream.  one_net_sync() waits for everything submitted.
extern "C" int one_net_submit_host(one_net *h, const float *host_in, float *host_out)
{
    if (!h || !host_in || !host_out) return nfail(ONE_ERR_BAD_ARG, "one_net_submit_host: null argument");
    cudaSetDevice(h->device);
    const TensorInfo &in = h->exe->tensors[h->n.input_names[0]];
    const TensorInfo &out = h->exe->tensors[h->plain_outputs[0]];
    cudaError_t e;
    if (!h->copy_stream) {
        if ((e = cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaMalloc(&h->staging, in.bytes)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h->ev_h2d, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&h->ev_free, cudaEventDisableTiming)) != cudaSuccess)
            return nfail(ONE_ERR_CUDA, std::string("pipeline set-up: ") + cudaGetErrorString(e));
    }
    cudaStream_t st = h->exe->stream;
    if (h->staged_once && (e = cudaStreamWaitEvent(h->copy_stream, h->ev_free, 0)) != cudaSuccess)
        return nfail(ONE_ERR_CUDA, cudaGetErrorString(e));
    if ((e = cudaMemcpyAsync(h->staging, host_in, in.bytes, cudaMemcpyHostToDevice, h->copy_stream)) != cudaSuccess ||
        (e = cudaEventRecord(h->ev_h2d, h->copy_stream)) != cudaSuccess || (e = cudaStreamWaitEvent(st, h->ev_h2d, 0)) != cudaSuccess ||
        (e = cudaMemcpyAsync(in.dev, h->staging, in.bytes, cudaMemcpyDeviceToDevice, st)) != cudaSuccess ||
        (e = cudaEventRecord(h->ev_free, st)) != cudaSuccess)
        return nfail(ONE_ERR_CUDA, std::string("input copy: ") + cudaGetErrorString(e));
    h->staged_once = true;
    int rc = h->exe->impl(h->use_graph);
    if (rc != ONE_OK) return nfail(rc, h->exe->error);
    if ((e = cudaMemcpyAsync(host_out, out.dev, out.bytes, cudaMemcpyDeviceToHost, st)) != cudaSuccess)
        return nfail(ONE_ERR_CUDA, std::string("output copy: ") + cudaGetErrorString(e));
    return ONE_OK;
}

extern "C" int one_net_fetch(one_net *h, const char *operand, float *host, size_t cap)
{
    if (!h || !operand || !host) return nfail(ONE_ERR_BAD_ARG, "one_net_fetch: null argument");
    cudaSetDevice(h->device);
    int rc = h->exe->fetch_plain_f32(operand, host, cap);
    return rc == ONE_OK ? ONE_OK : nfail(rc, h->exe->error);
}

extern "C" int one_net_operand_ptr(one_net *h, const char *operand, void **dev, long long *elems, int *dtype, int *layout)
{
    if (!h || !operand || !dev) return nfail(ONE_ERR_BAD_ARG, "one_net_operand_ptr: null argument");
    auto it = h->exe->tensors.find(operand);
    if (it == h->exe->tensors.end()) return nfail(ONE_ERR_BAD_ARG, std::string("no operand named '") + operand + "'");
    *dev = it->second.dev;
    if (elems) *elems = operand_elem_size(&it->second.desc);
    if (dtype) *dtype = it->second.dtype;
    if (layout) *layout = it->second.layout;
    return ONE_OK;
}

extern "C" int one_net_operands(one_net *h, char *buf, size_t cap)
{
    if (!h || !buf || !cap) return nfail(ONE_ERR_BAD_ARG, "one_net_operands: null argument");
    std::string all;
    for (auto &kv : h->exe->tensors) all += kv.first + "\n";
    if (all.size() + 1 > cap) return nfail(ONE_ERR_NOMEM, "buffer too small");
    memcpy(buf, all.c_str(), all.size() + 1);
    return ONE_OK;
}

extern "C" int one_net_trace_ex(one_net *h, const char *csv_path, int runs, const char *model_name, double hw_gops)
{
    if (!h || !csv_path) return nfail(ONE_ERR_BAD_ARG, "one_net_trace: null argument");
    cudaSetDevice(h->device);
    int rc = h->exe->impl_tracing(csv_path, runs < 1 ? 1 : runs, model_name, hw_gops);
    return rc == ONE_OK ? ONE_OK : nfail(rc, h->exe->error);
}

extern "C" int one_net_trace(one_net *h, const char *csv_path, int runs) { return one_net_trace_ex(h, csv_path, runs, nullptr, 0.0); }

// The CSV writer alone (host code, no device): lets a timeline be written from rows measured elsewhere
// and lets the file format be checked against the reference's timeline tool without a GPU.
extern "C" int one_net_write_timeline_csv(const char *csv_path, int n, const char *const *op_name, const char *const *op_type,
                                          const double *st_us, const double *ed_us, const double *mflop, const double *bytes,
                                          const char *const *detail, const char *gpu, const char *gpu_hw_info, double hw_gops,
                                          const char *model_name)
{
    if (!csv_path || n < 0 || (n > 0 && (!op_name || !op_type || !st_us || !ed_us || !mflop)))
        return nfail(ONE_ERR_BAD_ARG, "one_net_write_timeline_csv: null argument");
    if (!(hw_gops > 0)) return nfail(ONE_ERR_BAD_ARG, "one_net_write_timeline_csv: hw_gops must be positive (the timeline tool divides by it)");
    std::vector<TraceRow> rows((size_t)n);
    for (int i = 0; i < n; ++i) {
        rows[i].name = op_name[i] ? op_name[i] : "";
        rows[i].type = op_type[i] ? op_type[i] : "";
        rows[i].st_us = st_us[i];
        rows[i].ed_us = ed_us[i];
        rows[i].mflop = mflop[i];
        rows[i].bytes = bytes ? bytes[i] : 0.0;
        if (detail && detail[i]) rows[i].detail = detail[i];
    }
    if (write_trace_csv(csv_path, rows, gpu ? gpu : "", gpu_hw_info ? gpu_hw_info : "", hw_gops, model_name ? model_name : "model") != ONE_OK)
        return nfail(ONE_ERR_BAD_ARG, std::string("cannot write ") + csv_path);
    return ONE_OK;
}

extern "C" int one_net_autotune(one_net *h, int runs, char *report, size_t cap)
{
    if (!h) return nfail(ONE_ERR_BAD_ARG, "null net");
    cudaSetDevice(h->device);
    std::string rep;
    int rc = h->exe->autotune(runs, &rep);
    if (rc != ONE_OK) return nfail(rc, h->exe->error);
    if (report && cap) {
        if (rep.size() + 1 > cap) return nfail(ONE_ERR_NOMEM, "one_net_autotune: report buffer too small");
        memcpy(report, rep.c_str(), rep.size() + 1);
    }
    return ONE_OK;
}

extern "C" int one_net_set_tile(one_net *h, const char *op_name, int tile_n)
{
    if (!h || !op_name) return nfail(ONE_ERR_BAD_ARG, "one_net_set_tile: null argument");
    cudaSetDevice(h->device);
    int rc = h->exe->set_tile(op_name, tile_n);
    return rc == ONE_OK ? ONE_OK : nfail(rc, h->exe->error);
}

extern "C" int one_net_work(one_net *h, double *flops, double *bytes, unsigned long long *launches)
{
    if (!h) return nfail(ONE_ERR_BAD_ARG, "null net");
    double f = 0, b = 0;
    for (auto &s : h->exe->steps)
        if (s.o) {
            f += s.o->get_computation() * 1e6;
            b += s.o->get_bytes();
        }
    if (flops) *flops = f;
    if (bytes) *bytes = b;
    if (launches) *launches = h->exe->launches_per_run;
    return ONE_OK;
}
