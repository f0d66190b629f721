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
                     t.dtype == DT_F32 ? "f32" : (t.dtype == DT_BF16 ? "bf16" : (t.dtype == DT_F16 ? "f16" : "s8")), extra.c_str());
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

// The activation tables the runtime hands to its operators (host arithmetic; 8192 floats): kind 0 = SiLU
// (host/ops/conv.h:178-194), 1 = Gelu (host/ops/gelu.h:80-96).
extern "C" int one_net_activation_table(int kind, float *out8192)
{
    if (!out8192 || (kind != 0 && kind != 1)) return nfail(ONE_ERR_BAD_ARG, "one_net_activation_table: kind must be 0 (SiLU) or 1 (Gelu)");
    const std::vector<float> t = kind == 0 ? build_silu_lut() : build_gelu_lut();
    memcpy(out8192, t.data(), t.size() * sizeof(float));
    return ONE_OK;
}

// ============================================================================ one process, several GPUs
// one_net_group: the batch of one inference call cut into contiguous shards, one per device, each shard
// run by its own replica of the network (own weights, arena, stream, captured graph) from its own host
// thread.  Images are independent (the reference is strictly per image, host/ops/conv.h:43), so the shards
// exchange nothing: no collective, no peer access.  The caller keeps the reference's shape -- one thread
// that loads a model and calls inference (host/net.h:613-628) -- and still uses every GPU of the box.
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>

namespace {

struct GroupJob {
    const float *in;
    float *out;
};

struct GroupWorker {
    int device = 0, first = 0, count = 0;   // shard [first, first + count) of the batch
    one_net *net = nullptr;
    size_t in_elems = 0, out_elems = 0;     // per image
    std::thread th;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<GroupJob> jobs;
    bool stop = false, syncing = false;
    int pending = 0;                        // jobs queued or running
    int rc = ONE_OK;                        // first error of this worker since the last sync
    std::string err;
};

}  // namespace

struct one_net_group {
    std::vector<std::unique_ptr<GroupWorker>> workers;
    int batch = 0;
    int (*fault_hook)(int device) = nullptr;   // test hook: a host-side failure injected before a shard is submitted
};

static void group_worker_main(one_net_group *g, GroupWorker *w)
{
    cudaSetDevice(w->device);
    for (;;) {
        GroupJob job;
        {
            std::unique_lock<std::mutex> lk(w->mu);
            w->cv.wait(lk, [&] { return w->stop || !w->jobs.empty() || w->syncing; });
            if (w->jobs.empty()) {
                if (w->syncing) {   // everything submitted: wait for the device and report
                    lk.unlock();
                    int rc = one_net_sync(w->net);
                    lk.lock();
                    if (rc != ONE_OK && w->rc == ONE_OK) { w->rc = rc; w->err = one_net_last_error(); }
                    w->syncing = false;
                    w->cv.notify_all();
                    continue;
                }
                if (w->stop) return;
                continue;
            }
            job = w->jobs.front();
            w->jobs.pop_front();
        }
        int rc = ONE_OK;
        std::string err;
        if (g->fault_hook && (rc = g->fault_hook(w->device)) != ONE_OK) err = "injected host-side failure on device " + std::to_string(w->device);
        if (rc == ONE_OK) {
            rc = one_net_submit_host(w->net, job.in + (size_t)w->first * w->in_elems, job.out + (size_t)w->first * w->out_elems);
            if (rc != ONE_OK) err = one_net_last_error();
        }
        std::lock_guard<std::mutex> lk(w->mu);
        if (rc != ONE_OK && w->rc == ONE_OK) { w->rc = rc; w->err = err; }
        --w->pending;
        w->cv.notify_all();
    }
}

// Shard `index` of `n` over a batch: contiguous, equal, in device order.  Host arithmetic only.
extern "C" int one_net_group_partition(int batch, int n_devices, int index, int *first, int *count)
{
    if (n_devices <= 0 || index < 0 || index >= n_devices) return nfail(ONE_ERR_BAD_ARG, "one_net_group_partition: shard " + std::to_string(index) + " of " + std::to_string(n_devices));
    if (batch <= 0 || batch % n_devices) return nfail(ONE_ERR_BAD_ARG, "one_net_group_partition: batch " + std::to_string(batch) + " is not divisible by " + std::to_string(n_devices) + " devices");
    const int per = batch / n_devices;
    if (first) *first = index * per;
    if (count) *count = per;
    return ONE_OK;
}

static int group_build(const char *path, const void *image, size_t size, const int *devices, int n, int batch, int flags, size_t ws,
                       one_net_group **out)
{
    if (!out || !devices || n <= 0) return nfail(ONE_ERR_BAD_ARG, "one_net_group_create: null argument or no device");
    int rc0 = one_net_group_partition(batch, n, 0, nullptr, nullptr);
    if (rc0 != ONE_OK) return rc0;
    int have = 0;
    if (cudaGetDeviceCount(&have) != cudaSuccess) return nfail(ONE_ERR_CUDA, "one_net_group_create: no usable CUDA device (this backend has no CPU fallback)");
    for (int i = 0; i < n; ++i) {
        if (devices[i] < 0 || devices[i] >= have) return nfail(ONE_ERR_BAD_ARG, "one_net_group_create: device " + std::to_string(devices[i]) + " out of range (" + std::to_string(have) + " visible)");
        for (int j = 0; j < i; ++j)
            if (devices[j] == devices[i]) return nfail(ONE_ERR_BAD_ARG, "one_net_group_create: device " + std::to_string(devices[i]) + " listed twice");
    }
    std::unique_ptr<one_net_group> g(new one_net_group());
    g->batch = batch;
    const int per = batch / n;
    std::vector<int> rcs(n, ONE_OK);
    std::vector<std::string> errs(n);
    for (int i = 0; i < n; ++i) {
        g->workers.emplace_back(new GroupWorker());
        g->workers[i]->device = devices[i];
        one_net_group_partition(batch, n, i, &g->workers[i]->first, &g->workers[i]->count);
    }
    // the replicas are built in parallel, each from its own thread with its device current
    std::vector<std::thread> builders;
    for (int i = 0; i < n; ++i)
        builders.emplace_back([&, i] {
            GroupWorker *w = g->workers[i].get();
            rcs[i] = path ? one_net_create(path, w->device, per, flags, ws, &w->net)
                          : one_net_create_from_memory(image, size, w->device, per, flags, ws, &w->net);
            if (rcs[i] != ONE_OK) errs[i] = one_net_last_error();
        });
    for (auto &t : builders) t.join();
    for (int i = 0; i < n; ++i)
        if (rcs[i] != ONE_OK) {
            for (auto &w : g->workers) one_net_destroy(w->net);
            return nfail(rcs[i], "device " + std::to_string(devices[i]) + ": " + errs[i]);
        }
    for (auto &w : g->workers) {
        int shape[SHAPE_LEN], nd = 0;
        one_net_io_info(w->net, 0, 0, nullptr, shape, &nd);
        w->in_elems = 1;
        for (int d = 1; d < SHAPE_LEN; ++d) w->in_elems *= (size_t)shape[d];
        one_net_io_info(w->net, 1, 0, nullptr, shape, &nd);
        w->out_elems = 1;
        for (int d = 1; d < SHAPE_LEN; ++d) w->out_elems *= (size_t)shape[d];
        w->th = std::thread(group_worker_main, g.get(), w.get());
    }
    *out = g.release();
    return ONE_OK;
}

extern "C" int one_net_group_create(const char *path, const int *devices, int n_devices, int batch, int flags, size_t ws, one_net_group **out)
{
    if (!path) return nfail(ONE_ERR_BAD_ARG, "one_net_group_create: null path");
    return group_build(path, nullptr, 0, devices, n_devices, batch, flags, ws, out);
}

extern "C" int one_net_group_create_from_memory(const void *image, size_t size, const int *devices, int n_devices, int batch, int flags,
                                                size_t ws, one_net_group **out)
{
    if (!image) return nfail(ONE_ERR_BAD_ARG, "one_net_group_create_from_memory: null image");
    return group_build(nullptr, image, size, devices, n_devices, batch, flags, ws, out);
}

extern "C" int one_net_group_size(one_net_group *g) { return g ? (int)g->workers.size() : 0; }

extern "C" int one_net_group_shard(one_net_group *g, int index, int *device, int *first, int *count)
{
    if (!g || index < 0 || index >= (int)g->workers.size()) return nfail(ONE_ERR_BAD_ARG, "one_net_group_shard: index out of range");
    if (device) *device = g->workers[index]->device;
    if (first) *first = g->workers[index]->first;
    if (count) *count = g->workers[index]->count;
    return ONE_OK;
}

extern "C" one_net *one_net_group_member(one_net_group *g, int index)
{
    return (g && index >= 0 && index < (int)g->workers.size()) ? g->workers[index]->net : nullptr;
}

extern "C" int one_net_group_submit_host(one_net_group *g, const float *host_in, float *host_out)
{
    if (!g || !host_in || !host_out) return nfail(ONE_ERR_BAD_ARG, "one_net_group_submit_host: null argument");
    for (auto &w : g->workers) {
        std::lock_guard<std::mutex> lk(w->mu);
        w->jobs.push_back({host_in, host_out});
        ++w->pending;
        w->cv.notify_all();
    }
    return ONE_OK;
}

extern "C" int one_net_group_sync(one_net_group *g)
{
    if (!g) return nfail(ONE_ERR_BAD_ARG, "null group");
    int rc = ONE_OK;
    std::string err;
    for (auto &w : g->workers) {   // ask every worker first, so that the devices drain in parallel
        std::unique_lock<std::mutex> lk(w->mu);
        w->cv.wait(lk, [&] { return w->pending == 0; });
        w->syncing = true;
        w->cv.notify_all();
    }
    for (auto &w : g->workers) {
        std::unique_lock<std::mutex> lk(w->mu);
        w->cv.wait(lk, [&] { return !w->syncing; });
        if (w->rc != ONE_OK && rc == ONE_OK) { rc = w->rc; err = "device " + std::to_string(w->device) + ": " + w->err; }
        w->rc = ONE_OK;
        w->err.clear();
    }
    return rc == ONE_OK ? ONE_OK : nfail(rc, err);
}

extern "C" int one_net_group_set_fault_hook(one_net_group *g, int (*hook)(int device))
{
    if (!g) return nfail(ONE_ERR_BAD_ARG, "null group");
    one_net_group_sync(g);
    g->fault_hook = hook;
    return ONE_OK;
}

extern "C" void one_net_group_destroy(one_net_group *g)
{
    if (!g) return;
    for (auto &w : g->workers) {
        {
            std::lock_guard<std::mutex> lk(w->mu);
            w->stop = true;
            w->cv.notify_all();
        }
        if (w->th.joinable()) w->th.join();
        cudaSetDevice(w->device);
        one_net_destroy(w->net);
    }
    delete g;
}
