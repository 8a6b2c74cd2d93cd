// tenferro-device for the B200 backend: context, stream, stream-ordered pool, events,
// transfers, device preference and the error channel.
// Reference semantics: tenferro-device/src/lib.rs:30-162 (memory spaces, compute
// devices, OpKind, preferred_compute_devices, Error); tenferro-tensor/src/lib.rs:301-309,
// 660-713 (CompletionEvent, to_memory_space_async, wait, is_ready).
#include "common.h"

#include <atomic>
#include <cstdlib>

namespace tfb {
unsigned long long launch_count();

static thread_local std::string g_last_error;

void set_error(const char* msg) { g_last_error = msg ? msg : ""; }

tfb_status fail(tfb_status code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    if (env_int("TFB_LOG", 0) > 0) fprintf(stderr, "[tenferro_b200] error %d: %s\n", (int)code, buf);
    return code;
}

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    return atoi(v);
}

Scalar load_scalar(int dtype, const void* p) {
    Scalar s;
    if (!p) {
        s.re = 1;
        return s;
    }
    switch (dtype) {
        case TFB_F32: s.re = *(const float*)p; break;
        case TFB_F64: s.re = *(const double*)p; break;
        case TFB_C32: s.re = ((const float*)p)[0]; s.im = ((const float*)p)[1]; break;
        case TFB_C64: s.re = ((const double*)p)[0]; s.im = ((const double*)p)[1]; break;
    }
    return s;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches += (unsigned long long)n; }
unsigned long long launch_count() { return g_launches.load(); }

LaunchScope::LaunchScope(tfb_ctx* c, const char* name) : ctx(c) {
    count_launch(1);
    if (!c->profiling) return;
    cudaEvent_t start;
    if (cudaEventCreate(&start) != cudaSuccess) return;
    if (cudaEventCreate(&stop) != cudaSuccess) {
        cudaEventDestroy(start);
        stop = nullptr;
        return;
    }
    cudaEventRecord(start, c->stream);
    c->prof.push_back({name, start, stop});
}
LaunchScope::~LaunchScope() {
    if (stop) cudaEventRecord(stop, ctx->stream);
}

PoolBlock::~PoolBlock() {
    if (ptr && ctx) {
        DeviceGuard g(ctx->device);
        cudaFreeAsync(ptr, ctx->stream);
    }
}
tfb_status PoolBlock::alloc(tfb_ctx* c, size_t bytes) {
    ctx = c;
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMallocFromPoolAsync(&ptr, bytes, c->pool, c->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        ptr = nullptr;
        return fail(TFB_ERR_DEVICE, "pool allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    return TFB_OK;
}

}  // namespace tfb

using namespace tfb;

extern "C" {

size_t tfb_last_error(char* buf, size_t cap) {
    const std::string& m = g_last_error;
    if (buf && cap) {
        size_t n = m.size() < cap - 1 ? m.size() : cap - 1;
        memcpy(buf, m.data(), n);
        buf[n] = 0;
    }
    return m.size();
}

const char* tfb_version(void) { return "tenferro_b200 0.1 (sm_100a)"; }

tfb_status tfb_ctx_create(int device_id, tfb_ctx** out) {
    if (!out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_create: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(TFB_ERR_DEVICE,
                    "no CUDA device available (%s); this backend has no CPU path",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    if (device_id < 0 || device_id >= n)
        return fail(TFB_ERR_INVALID_ARGUMENT, "device_id %d out of range (have %d devices)", device_id, n);
    DeviceGuard g(device_id);
    if (!g.ok) return fail(TFB_ERR_DEVICE, "cudaSetDevice(%d) failed", device_id);
    // Frees whatever the context already owns when a later step of the set-up fails.
    struct Cleanup {
        void operator()(tfb_ctx* c) const {
            if (c->own_stream) cudaStreamDestroy(c->own_stream);
            if (c->dev_status) cudaFree(c->dev_status);
            if (c->pool) cudaMemPoolDestroy(c->pool);
            delete c;
        }
    };
    std::unique_ptr<tfb_ctx, Cleanup> c(new tfb_ctx);
    c->device = device_id;
    cudaDeviceProp prop;
    TFB_CUDA(cudaGetDeviceProperties(&prop, device_id));
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;
    c->total_mem = prop.totalGlobalMem;
    c->smem_optin = prop.sharedMemPerBlockOptin;
    if (prop.major < 10 && !env_int("TFB_ALLOW_ANY_GPU", 0))
        return fail(TFB_ERR_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", device_id,
                    prop.major, prop.minor);
    TFB_CUDA(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
    c->stream = c->own_stream;
    // A pool of the context's own: the device's default pool belongs to the host application,
    // whose other cudaMallocAsync users would inherit any attribute set on it.  TFB_POOL_BYTES
    // caps what the pool may hold (0 or unset: no cap); an allocation past the cap fails with
    // DeviceError and leaves the context usable.
    cudaMemPoolProps props;
    memset(&props, 0, sizeof props);
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device_id;
    const char* cap = getenv("TFB_POOL_BYTES");
    if (cap && *cap) props.maxSize = (size_t)strtoull(cap, nullptr, 10);
    c->pool_cap = props.maxSize;
    TFB_CUDA(cudaMemPoolCreate(&c->pool, &props));
    // Keep freed blocks cached in the pool instead of returning them to the driver at
    // every synchronisation: intermediates of a contraction tree are re-used each call.
    uint64_t threshold = UINT64_MAX;
    TFB_CUDA(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    TFB_CUDA(cudaMalloc(&c->dev_status, sizeof(int)));
    TFB_CUDA(cudaMemset(c->dev_status, 0, sizeof(int)));
    *out = c.release();
    return TFB_OK;
}

unsigned long long tfb_kernel_launch_count(void) { return launch_count(); }

tfb_status tfb_ctx_profile_begin(tfb_ctx* ctx) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_profile_begin: ctx is NULL");
    if (ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_profile_begin: the context is capturing");
    for (auto& r : ctx->prof) {
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    ctx->prof.clear();
    // What an event pair measures with nothing between its two records: the front end's cost
    // of taking the two timestamps.  A pair around a launch contains the same cost on top of
    // the kernel's run time, so profile_read subtracts it.
    DeviceGuard g(ctx->device);
    ctx->prof_pair_ms = 0;
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) == cudaSuccess) {
        if (cudaEventCreate(&b) == cudaSuccess) {
            float best = 1e30f;
            for (int i = 0; i < 16; ++i) {
                cudaEventRecord(a, ctx->stream);
                cudaEventRecord(b, ctx->stream);
                float ms = 0;
                if (cudaEventSynchronize(b) == cudaSuccess && cudaEventElapsedTime(&ms, a, b) == cudaSuccess && ms < best)
                    best = ms;
            }
            if (best < 1e29f) ctx->prof_pair_ms = best;
            cudaEventDestroy(b);
        }
        cudaEventDestroy(a);
    }
    ctx->profiling = true;
    return TFB_OK;
}

tfb_status tfb_ctx_profile_read(tfb_ctx* ctx, const char* kernel, size_t* launches, double* total_ms) {
    if (!ctx || !kernel || !launches || !total_ms)
        return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_profile_read: NULL argument");
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaStreamSynchronize(ctx->stream));
    *launches = 0;
    *total_ms = 0;
    for (auto& r : ctx->prof) {
        if (strcmp(r.name, kernel) != 0) continue;
        float ms = 0;
        TFB_CUDA(cudaEventElapsedTime(&ms, r.start, r.stop));
        *total_ms += ms > ctx->prof_pair_ms ? ms - ctx->prof_pair_ms : 0.f;
        ++*launches;
    }
    return TFB_OK;
}

tfb_status tfb_ctx_profile_end(tfb_ctx* ctx) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_profile_end: ctx is NULL");
    ctx->profiling = false;
    for (auto& r : ctx->prof) {
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    ctx->prof.clear();
    return TFB_OK;
}

tfb_status tfb_ctx_destroy(tfb_ctx* ctx) {
    if (!ctx) return TFB_OK;
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->sk_partial) cudaFree(ctx->sk_partial);
    if (ctx->sk_flags) cudaFree(ctx->sk_flags);
    if (ctx->pool) cudaMemPoolDestroy(ctx->pool);
    delete ctx;
    return TFB_OK;
}

tfb_status tfb_ctx_device(const tfb_ctx* ctx, int* device_id) {
    if (!ctx || !device_id) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_device: NULL argument");
    *device_id = ctx->device;
    return TFB_OK;
}

tfb_status tfb_ctx_stream(const tfb_ctx* ctx, void** stream) {
    if (!ctx || !stream) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_stream: NULL argument");
    *stream = (void*)ctx->stream;
    return TFB_OK;
}

tfb_status tfb_ctx_set_stream(tfb_ctx* ctx, void* stream) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_set_stream: ctx is NULL");
    cudaStream_t next = stream ? (cudaStream_t)stream : ctx->own_stream;
    if (next == ctx->stream) return TFB_OK;
    if (ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_set_stream: the context is capturing");
    // Work enqueued on the new stream comes after everything already enqueued on the old one:
    // pool blocks, the offset tables and the stream-K scratch of this context are all ordered
    // by "the context's stream", so the switch must not let two of its launches overlap.
    DeviceGuard g(ctx->device);
    cudaEvent_t ev;
    TFB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(next, ev, 0);
    cudaEventDestroy(ev);
    if (e != cudaSuccess) return fail(TFB_ERR_DEVICE, "tfb_ctx_set_stream: %s", cudaGetErrorString(e));
    ctx->stream = next;
    return TFB_OK;
}

// ---- capture and replay.  The context's stream goes into CUDA stream capture: every launch,
// pool allocation and copy this library enqueues until capture_end becomes a node of a graph
// instead of running.  Plans, offset tables and kernel attributes are host-side state that the
// first call of a kind sets up with calls capture does not allow, so the sequence has to have
// run once before it is captured.
tfb_status tfb_ctx_capture_begin(tfb_ctx* ctx) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_capture_begin: ctx is NULL");
    if (ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_capture_begin: the context is capturing already");
    if (ctx->profiling) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_capture_begin: end the launch profile first");
    DeviceGuard g(ctx->device);
    // Relaxed mode: the library's host-side bookkeeping between launches (event queries on the offset
    // tables' upload, attribute calls) is not work on the captured stream and stays allowed.
    TFB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    return TFB_OK;
}

tfb_status tfb_ctx_capture_end(tfb_ctx* ctx, tfb_graph** out) {
    if (!ctx || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_capture_end: NULL argument");
    *out = nullptr;
    if (!ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_capture_end: the context is not capturing");
    DeviceGuard g(ctx->device);
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();  // a call that capture does not allow has ended it; the stream is usable again
        return fail(TFB_ERR_DEVICE, "the captured sequence contained a call that cannot be captured (%s): "
                                    "run the sequence once before capturing it", cudaGetErrorString(e));
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        return fail(TFB_ERR_DEVICE, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    tfb_graph* gr = new tfb_graph;
    gr->ctx = ctx;
    gr->graph = graph;
    gr->exec = exec;
    *out = gr;
    return TFB_OK;
}

tfb_status tfb_graph_launch(tfb_graph* graph) {
    if (!graph || !graph->exec) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_graph_launch: graph is NULL");
    if (graph->ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_graph_launch: the context is capturing");
    DeviceGuard g(graph->ctx->device);
    count_launch(1);
    TFB_CUDA(cudaGraphLaunch(graph->exec, graph->ctx->stream));
    return TFB_OK;
}

void tfb_graph_destroy(tfb_graph* graph) {
    if (!graph) return;
    DeviceGuard g(graph->ctx->device);
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
}

tfb_status tfb_ctx_synchronize(tfb_ctx* ctx) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_synchronize: ctx is NULL");
    if (ctx->capturing) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_synchronize: the context is capturing");
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaStreamSynchronize(ctx->stream));
    // Kernels with bounded waits report through this word instead of trapping.
    int st = 0;
    TFB_CUDA(cudaMemcpy(&st, ctx->dev_status, sizeof st, cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(ctx->dev_status, 0, sizeof(int));
        return fail(TFB_ERR_DEVICE, "a kernel gave up a bounded wait (status word 0x%x)", st);
    }
    return TFB_OK;
}

tfb_status tfb_ctx_properties(const tfb_ctx* ctx, int* sm_count, size_t* total_mem, int* cc_major, int* cc_minor) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_ctx_properties: ctx is NULL");
    if (sm_count) *sm_count = ctx->sm_count;
    if (total_mem) *total_mem = ctx->total_mem;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    return TFB_OK;
}

tfb_status tfb_alloc(tfb_ctx* ctx, size_t bytes, void** out) {
    if (!ctx || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_alloc: NULL argument");
    *out = nullptr;
    DeviceGuard g(ctx->device);
    if (bytes == 0) bytes = 16;
    cudaError_t e = cudaMallocFromPoolAsync(out, bytes, ctx->pool, ctx->stream);
    if (e != cudaSuccess) {
        *out = nullptr;
        cudaGetLastError();
        return fail(TFB_ERR_DEVICE, "pool allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    return TFB_OK;
}

tfb_status tfb_free(tfb_ctx* ctx, void* ptr) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_free: ctx is NULL");
    if (!ptr) return TFB_OK;
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaFreeAsync(ptr, ctx->stream));
    return TFB_OK;
}

tfb_status tfb_pool_stats(tfb_ctx* ctx, size_t* reserved, size_t* used) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_pool_stats: ctx is NULL");
    DeviceGuard g(ctx->device);
    uint64_t r = 0, u = 0;
    TFB_CUDA(cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrReservedMemCurrent, &r));
    TFB_CUDA(cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrUsedMemCurrent, &u));
    if (reserved) *reserved = (size_t)r;
    if (used) *used = (size_t)u;
    return TFB_OK;
}

static tfb_status do_copy(tfb_ctx* ctx, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind,
                          const char* who) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", who);
    if (bytes == 0) return TFB_OK;
    if (!dst || !src) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: NULL buffer", who);
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaMemcpyAsync(dst, src, bytes, kind, ctx->stream));
    return TFB_OK;
}

tfb_status tfb_memcpy_h2d_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return do_copy(ctx, dst, src, bytes, cudaMemcpyHostToDevice, "tfb_memcpy_h2d_async");
}
tfb_status tfb_memcpy_d2h_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return do_copy(ctx, dst, src, bytes, cudaMemcpyDeviceToHost, "tfb_memcpy_d2h_async");
}
tfb_status tfb_memcpy_d2d_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return do_copy(ctx, dst, src, bytes, cudaMemcpyDeviceToDevice, "tfb_memcpy_d2d_async");
}

static tfb_status do_copy_2d(tfb_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width,
                             size_t height, cudaMemcpyKind kind, const char* who) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", who);
    if (width == 0 || height == 0) return TFB_OK;
    if (!dst || !src) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: NULL buffer", who);
    if (dst_pitch < width || src_pitch < width)
        return fail(TFB_ERR_INVALID_ARGUMENT, "%s: a pitch is smaller than the row width", who);
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, height, kind, ctx->stream));
    return TFB_OK;
}
tfb_status tfb_memcpy_h2d_2d_async(tfb_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                   size_t width, size_t height) {
    return do_copy_2d(ctx, dst, dst_pitch, src, src_pitch, width, height, cudaMemcpyHostToDevice, "tfb_memcpy_h2d_2d_async");
}
tfb_status tfb_memcpy_d2h_2d_async(tfb_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                   size_t width, size_t height) {
    return do_copy_2d(ctx, dst, dst_pitch, src, src_pitch, width, height, cudaMemcpyDeviceToHost, "tfb_memcpy_d2h_2d_async");
}

tfb_status tfb_memcpy_p2p_async(tfb_ctx* ctx, void* dst, int dst_device, const void* src, int src_device,
                                size_t bytes) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_memcpy_p2p_async: ctx is NULL");
    if (bytes == 0) return TFB_OK;
    if (!dst || !src) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_memcpy_p2p_async: NULL buffer");
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, ctx->stream));
    return TFB_OK;
}

tfb_status tfb_memset_async(tfb_ctx* ctx, void* dst, int value, size_t bytes) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_memset_async: ctx is NULL");
    if (bytes == 0) return TFB_OK;
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return TFB_OK;
}

tfb_status tfb_host_alloc(size_t bytes, void** out) {
    if (!out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_host_alloc: out is NULL");
    TFB_CUDA(cudaMallocHost(out, bytes ? bytes : 16));
    return TFB_OK;
}
tfb_status tfb_host_free(void* ptr) {
    if (ptr) TFB_CUDA(cudaFreeHost(ptr));
    return TFB_OK;
}

tfb_status tfb_event_record(tfb_ctx* ctx, tfb_event** out) {
    if (!ctx || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_event_record: NULL argument");
    DeviceGuard g(ctx->device);
    std::unique_ptr<tfb_event> ev(new tfb_event);
    ev->device = ctx->device;
    TFB_CUDA(cudaEventCreate(&ev->ev));
    // While the context is capturing nothing is enqueued, so there is nothing to mark: the event stays
    // unrecorded, which reads as complete (an event recorded into the capture could be neither
    // queried nor waited for from outside it).
    cudaError_t e = ctx->capturing ? cudaSuccess : cudaEventRecord(ev->ev, ctx->stream);
    if (e != cudaSuccess) {
        cudaEventDestroy(ev->ev);
        return fail(TFB_ERR_DEVICE, "cudaEventRecord failed: %s", cudaGetErrorString(e));
    }
    *out = ev.release();
    return TFB_OK;
}

tfb_status tfb_event_wait(tfb_ctx* ctx, tfb_event* ev) {
    if (!ctx || !ev) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_event_wait: NULL argument");
    DeviceGuard g(ctx->device);
    TFB_CUDA(cudaStreamWaitEvent(ctx->stream, ev->ev, 0));
    return TFB_OK;
}

tfb_status tfb_event_synchronize(tfb_event* ev) {
    if (!ev) return TFB_OK;  // CPU tensors carry no event: wait() is a no-op
    TFB_CUDA(cudaEventSynchronize(ev->ev));
    return TFB_OK;
}

tfb_status tfb_event_query(tfb_event* ev, int* ready) {
    if (!ready) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_event_query: ready is NULL");
    if (!ev) {
        *ready = 1;
        return TFB_OK;
    }
    cudaError_t e = cudaEventQuery(ev->ev);
    if (e == cudaSuccess) {
        *ready = 1;
    } else if (e == cudaErrorNotReady) {
        *ready = 0;
    } else {
        return fail(TFB_ERR_DEVICE, "cudaEventQuery failed: %s", cudaGetErrorString(e));
    }
    return TFB_OK;
}

tfb_status tfb_event_elapsed_ms(tfb_event* start, tfb_event* stop, float* ms) {
    if (!start || !stop || !ms) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_event_elapsed_ms: NULL argument");
    TFB_CUDA(cudaEventElapsedTime(ms, start->ev, stop->ev));
    return TFB_OK;
}

tfb_status tfb_event_destroy(tfb_event* ev) {
    if (!ev) return TFB_OK;
    cudaEventDestroy(ev->ev);
    delete ev;
    return TFB_OK;
}

tfb_status tfb_preferred_compute_devices(int32_t space_kind, size_t space_id, int32_t op_kind,
                                         tfb_compute_device* out, size_t cap, size_t* n_out) {
    if (!n_out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_preferred_compute_devices: n_out is NULL");
    *n_out = 0;
    if (op_kind < TFB_KIND_CONTRACT || op_kind > TFB_KIND_ELEMENTWISE_MUL)
        return fail(TFB_ERR_INVALID_ARGUMENT, "unknown op kind %d", (int)op_kind);
    if (space_kind == TFB_SPACE_MAIN_MEMORY)
        return fail(TFB_ERR_NO_COMPATIBLE_DEVICE,
                    "no compatible compute device for op kind %d on MainMemory: this backend computes on GPU "
                    "memory only",
                    (int)op_kind);
    if (space_kind != TFB_SPACE_GPU_MEMORY)
        return fail(TFB_ERR_INVALID_ARGUMENT, "unknown memory space kind %d", (int)space_kind);
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    if ((int)space_id >= n)
        return fail(TFB_ERR_NO_COMPATIBLE_DEVICE,
                    "no compatible compute device for op kind %d on GpuMemory{space_id: %zu} (%d CUDA devices)",
                    (int)op_kind, space_id, n);
    // The owning GPU first, then every peer that can map its memory (NVLink / NVSwitch).
    std::vector<tfb_compute_device> devs;
    devs.push_back({TFB_DEVICE_CUDA, (int32_t)space_id});
    for (int d = 0; d < n; ++d) {
        if (d == (int)space_id) continue;
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, d, (int)space_id) == cudaSuccess && can) devs.push_back({TFB_DEVICE_CUDA, d});
    }
    *n_out = devs.size();
    for (size_t i = 0; i < devs.size() && i < cap && out; ++i) out[i] = devs[i];
    return TFB_OK;
}

size_t tfb_compute_device_format(tfb_compute_device dev, char* buf, size_t cap) {
    const char* name = dev.kind == TFB_DEVICE_CPU ? "cpu" : dev.kind == TFB_DEVICE_CUDA ? "cuda" : "hip";
    char tmp[64];
    int n = snprintf(tmp, sizeof tmp, "%s:%d", name, (int)dev.device_id);
    if (buf && cap) {
        size_t m = (size_t)n < cap - 1 ? (size_t)n : cap - 1;
        memcpy(buf, tmp, m);
        buf[m] = 0;
    }
    return (size_t)n;
}

}  // extern "C"
