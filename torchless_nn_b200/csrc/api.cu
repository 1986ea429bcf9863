// Context lifecycle, memory, error reporting and profiling entry points of libtlnn.
#include "common.cuh"

#include <cstdarg>

static thread_local char g_last_error[1024] = "";

void tl_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int tl_cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    const char* base = strrchr(file, '/');
    tl_set_error("CUDA error %d (%s) in %s at %s:%d", (int)e, cudaGetErrorString(e), what, base ? base + 1 : file, line);
    return e == cudaErrorMemoryAllocation ? TLNN_ERR_NOMEM : TLNN_ERR_CUDA;
}

extern "C" const char* tlnn_last_error(void) { return g_last_error; }
extern "C" int tlnn_version(void) { return 100; }

extern "C" int tlnn_init(int device, tlnn_ctx** out) {
    TL_NOTNULL(out);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        tl_set_error("no CUDA device is visible (%s); libtlnn has no CPU path", cudaGetErrorString(e));
        return TLNN_ERR_CUDA;
    }
    TL_REQUIRE(device >= 0 && device < n, "device %d out of range (have %d)", device, n);
    TL_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    TL_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        tl_set_error("device %d is sm_%d%d; libtlnn is built for sm_100a only", device, prop.major, prop.minor);
        return TLNN_ERR_CUDA;
    }
    tlnn_ctx* c = new tlnn_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    TL_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    TL_CUDA(cudaDeviceGetDefaultMemPool(&c->pool, device));
    uint64_t keep = UINT64_MAX;   // keep freed blocks cached in the pool instead of returning them to the driver
    TL_CUDA(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &keep));
    TL_CUDA(cudaMalloc(&c->d_err, sizeof(tlnn_dev_err)));
    TL_CUDA(cudaMemset(c->d_err, 0, sizeof(tlnn_dev_err)));
    TL_CUDA(cudaMalloc(&c->d_sched, 256));
    TL_CUDA(cudaMemset(c->d_sched, 0, 256));
    TL_CUDA(cudaMallocHost(&c->h_err, sizeof(tlnn_dev_err)));
    memset(c->h_err, 0, sizeof(tlnn_dev_err));
    TL_CUDA(cudaEventCreate(&c->prof_a));
    TL_CUDA(cudaEventCreate(&c->prof_b));
    *out = c;
    return TLNN_OK;
}

extern "C" int tlnn_shutdown(tlnn_ctx* ctx) {
    TL_NOTNULL(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& p : ctx->pending) { cudaEventDestroy(p.start); cudaEventDestroy(p.stop); }
    for (auto& e : ctx->event_pool) cudaEventDestroy(e);
    tl_prefill_cache_free(ctx);
    if (ctx->ws) cudaFree(ctx->ws);
    cudaFree(ctx->d_err);
    cudaFree(ctx->d_sched);
    cudaFreeHost(ctx->h_err);
    cudaEventDestroy(ctx->prof_a);
    cudaEventDestroy(ctx->prof_b);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return TLNN_OK;
}

static int read_dev_err(tlnn_ctx* ctx, bool with_message) {
    TL_CUDA(cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(tlnn_dev_err), cudaMemcpyDeviceToHost, ctx->stream));
    TL_CUDA(cudaStreamSynchronize(ctx->stream));
    int code = ctx->h_err->code;
    if (code != 0) {
        if (with_message) {
            if (code == TLNN_ERR_INDEX)
                tl_set_error("index %lld is out of bounds (kernel site %d)", ctx->h_err->detail, ctx->h_err->where);
            else
                tl_set_error("a device-side wait gave up (kernel site %d, detail %lld)", ctx->h_err->where,
                             ctx->h_err->detail);
        }
        TL_CUDA(cudaMemsetAsync(ctx->d_err, 0, sizeof(tlnn_dev_err), ctx->stream));
    }
    return code;
}

extern "C" int tlnn_sync(tlnn_ctx* ctx) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    return read_dev_err(ctx, true);
}

extern "C" int tlnn_check(tlnn_ctx* ctx) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    return read_dev_err(ctx, true);
}

extern "C" void* tlnn_stream(tlnn_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

extern "C" int tlnn_device_info(tlnn_ctx* ctx, int* sm_count, size_t* total_mem, size_t* free_mem) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    size_t f = 0, t = 0;
    TL_CUDA(cudaMemGetInfo(&f, &t));
    if (sm_count) *sm_count = ctx->sm_count;
    if (total_mem) *total_mem = t;
    if (free_mem) *free_mem = f;
    return TLNN_OK;
}

extern "C" long long tlnn_launch_count(tlnn_ctx* ctx, int reset) {
    if (!ctx) return 0;
    long long n = ctx->launches;
    if (reset) ctx->launches = 0;
    return n;
}

// ---- memory ---------------------------------------------------------------------------------------
extern "C" int tlnn_alloc(tlnn_ctx* ctx, size_t bytes, void** dptr) {
    TL_NOTNULL(ctx);
    TL_NOTNULL(dptr);
    TL_CUDA(cudaSetDevice(ctx->device));
    if (bytes == 0) bytes = 16;
    if (ctx->canaries) {
        const size_t user = (bytes + 15) & ~size_t(15);
        TL_CUDA(cudaMallocAsync(dptr, user + TL_CANARY_BYTES, ctx->stream));
        TL_CUDA(cudaMemsetAsync(static_cast<char*>(*dptr) + user, TL_CANARY_BYTE, TL_CANARY_BYTES, ctx->stream));
        ctx->live[*dptr] = user;
        return TLNN_OK;
    }
    TL_CUDA(cudaMallocAsync(dptr, bytes, ctx->stream));
    return TLNN_OK;
}

// 1 if the canary behind a live block is intact, 0 if not, negative status on a CUDA error (waits for the stream).
static int canary_intact(tlnn_ctx* ctx, void* dptr, size_t user) {
    unsigned char host[TL_CANARY_BYTES];
    TL_CUDA(cudaMemcpyAsync(host, static_cast<char*>(dptr) + user, TL_CANARY_BYTES, cudaMemcpyDeviceToHost, ctx->stream));
    TL_CUDA(cudaStreamSynchronize(ctx->stream));
    for (size_t i = 0; i < TL_CANARY_BYTES; i++)
        if (host[i] != (unsigned char)TL_CANARY_BYTE) return 0;
    return 1;
}

extern "C" int tlnn_free(tlnn_ctx* ctx, void* dptr) {
    TL_NOTNULL(ctx);
    if (!dptr) return TLNN_OK;
    TL_CUDA(cudaSetDevice(ctx->device));
    auto it = ctx->live.find(dptr);
    if (it != ctx->live.end()) {
        const int ok = canary_intact(ctx, dptr, it->second);
        if (ok < 0) return ok;
        if (ok == 0) ctx->canary_failures++;
        ctx->live.erase(it);
    }
    TL_CUDA(cudaFreeAsync(dptr, ctx->stream));
    return TLNN_OK;
}

extern "C" int tlnn_debug_canaries(tlnn_ctx* ctx, int enable) {
    TL_NOTNULL(ctx);
    ctx->canaries = enable != 0;       // blocks allocated before stay unguarded; guarded blocks stay tracked until freed
    return TLNN_OK;
}

extern "C" int tlnn_debug_check(tlnn_ctx* ctx, long long* corrupted, long long* guarded) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    long long bad = ctx->canary_failures;
    for (auto& kv : ctx->live) {
        const int ok = canary_intact(ctx, kv.first, kv.second);
        if (ok < 0) return ok;
        if (ok == 0) bad++;
    }
    if (corrupted) *corrupted = bad;
    if (guarded) *guarded = (long long)ctx->live.size();
    return TLNN_OK;
}

extern "C" int tlnn_host_alloc(size_t bytes, void** hptr) {
    TL_NOTNULL(hptr);
    TL_CUDA(cudaMallocHost(hptr, bytes ? bytes : 16));
    return TLNN_OK;
}

extern "C" int tlnn_host_free(void* hptr) {
    if (hptr) TL_CUDA(cudaFreeHost(hptr));
    return TLNN_OK;
}

extern "C" int tlnn_h2d(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes) {
    TL_NOTNULL(ctx);
    if (bytes == 0) return TLNN_OK;
    TL_NOTNULL(dst);
    TL_NOTNULL(src);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return TLNN_OK;
}

// ---- double-buffered host feed ------------------------------------------------------------------------------------
struct tlnn_feeder {
    tlnn_ctx* ctx = nullptr;
    size_t bytes = 0;
    cudaStream_t copy = nullptr;
    void* host[2] = {nullptr, nullptr};
    void* dev[2] = {nullptr, nullptr};
    cudaEvent_t copied[2] = {nullptr, nullptr};      // recorded on the copy stream after a slot's copy
    cudaEvent_t released[2] = {nullptr, nullptr};    // recorded on the compute stream when a slot's consumer is enqueued
    bool has_copy[2] = {false, false}, has_release[2] = {false, false};
};

extern "C" int tlnn_feed_create(tlnn_ctx* ctx, size_t bytes_per_batch, tlnn_feeder** out) {
    TL_NOTNULL(ctx); TL_NOTNULL(out);
    TL_REQUIRE(bytes_per_batch > 0, "feed: a batch needs at least one byte");
    TL_CUDA(cudaSetDevice(ctx->device));
    tlnn_feeder* f = new tlnn_feeder();
    f->ctx = ctx;
    f->bytes = bytes_per_batch;
    cudaError_t e = cudaStreamCreateWithFlags(&f->copy, cudaStreamNonBlocking);
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        e = cudaMallocHost(&f->host[i], bytes_per_batch);
        if (e == cudaSuccess) e = cudaMalloc(&f->dev[i], bytes_per_batch);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&f->copied[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&f->released[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        tlnn_feed_destroy(f);
        return tl_cuda_fail(e, "feed_create", __FILE__, __LINE__);
    }
    *out = f;
    return TLNN_OK;
}

static int feed_slot_ok(tlnn_feeder* f, int slot) {
    TL_NOTNULL(f);
    TL_REQUIRE(slot == 0 || slot == 1, "feed: slot %d (0 or 1)", slot);
    TL_CUDA(cudaSetDevice(f->ctx->device));
    return TLNN_OK;
}

extern "C" int tlnn_feed_host(tlnn_feeder* f, int slot, void** host) {
    TL_TRY(feed_slot_ok(f, slot));
    TL_NOTNULL(host);
    *host = f->host[slot];
    return TLNN_OK;
}

extern "C" int tlnn_feed_host_wait(tlnn_feeder* f, int slot) {
    TL_TRY(feed_slot_ok(f, slot));
    if (f->has_copy[slot]) TL_CUDA(cudaEventSynchronize(f->copied[slot]));
    return TLNN_OK;
}

extern "C" int tlnn_feed_submit(tlnn_feeder* f, int slot, size_t bytes) {
    TL_TRY(feed_slot_ok(f, slot));
    TL_REQUIRE(bytes <= f->bytes, "feed: %zu bytes submitted, the feeder holds %zu per batch", bytes, f->bytes);
    // the device buffer may still be read by the work that consumed the previous batch of this slot
    if (f->has_release[slot]) TL_CUDA(cudaStreamWaitEvent(f->copy, f->released[slot], 0));
    if (bytes) TL_CUDA(cudaMemcpyAsync(f->dev[slot], f->host[slot], bytes, cudaMemcpyHostToDevice, f->copy));
    TL_CUDA(cudaEventRecord(f->copied[slot], f->copy));
    f->has_copy[slot] = true;
    return TLNN_OK;
}

extern "C" int tlnn_feed_acquire(tlnn_feeder* f, int slot, void** dev) {
    TL_TRY(feed_slot_ok(f, slot));
    TL_NOTNULL(dev);
    TL_REQUIRE(f->has_copy[slot], "feed: slot %d was acquired before anything was submitted to it", slot);
    TL_CUDA(cudaStreamWaitEvent(f->ctx->stream, f->copied[slot], 0));
    *dev = f->dev[slot];
    return TLNN_OK;
}

extern "C" int tlnn_feed_release(tlnn_feeder* f, int slot) {
    TL_TRY(feed_slot_ok(f, slot));
    TL_CUDA(cudaEventRecord(f->released[slot], f->ctx->stream));
    f->has_release[slot] = true;
    return TLNN_OK;
}

extern "C" int tlnn_feed_destroy(tlnn_feeder* f) {
    if (!f) return TLNN_OK;
    cudaSetDevice(f->ctx->device);
    if (f->copy) cudaStreamSynchronize(f->copy);
    cudaStreamSynchronize(f->ctx->stream);
    for (int i = 0; i < 2; i++) {
        if (f->host[i]) cudaFreeHost(f->host[i]);
        if (f->dev[i]) cudaFree(f->dev[i]);
        if (f->copied[i]) cudaEventDestroy(f->copied[i]);
        if (f->released[i]) cudaEventDestroy(f->released[i]);
    }
    if (f->copy) cudaStreamDestroy(f->copy);
    delete f;
    return TLNN_OK;
}

extern "C" int tlnn_d2h_async(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes) {
    TL_NOTNULL(ctx);
    if (bytes == 0) return TLNN_OK;
    TL_NOTNULL(dst);
    TL_NOTNULL(src);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return TLNN_OK;
}

extern "C" int tlnn_d2h(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes) {
    TL_TRY(tlnn_d2h_async(ctx, dst, src, bytes));
    int code = read_dev_err(ctx, true);
    return code;
}

extern "C" int tlnn_d2d(tlnn_ctx* ctx, void* dst, const void* src, size_t bytes) {
    TL_NOTNULL(ctx);
    if (bytes == 0) return TLNN_OK;
    TL_NOTNULL(dst);
    TL_NOTNULL(src);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return TLNN_OK;
}

extern "C" int tlnn_memset(tlnn_ctx* ctx, void* dst, int byte, size_t bytes) {
    TL_NOTNULL(ctx);
    if (bytes == 0) return TLNN_OK;
    TL_NOTNULL(dst);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaMemsetAsync(dst, byte, bytes, ctx->stream));
    return TLNN_OK;
}

// ---- scratch arena ---------------------------------------------------------------------------------
int tl_ws_reserve(tlnn_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->ws_bytes) return TLNN_OK;
    // Work already enqueued may still read the old arena: drain the stream before replacing it.
    TL_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->ws) TL_CUDA(cudaFree(ctx->ws));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    size_t want = bytes + bytes / 8;
    cudaError_t e = cudaMalloc(&ctx->ws, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        want = bytes;
        e = cudaMalloc(&ctx->ws, want);
    }
    if (e != cudaSuccess) return tl_cuda_fail(e, "cudaMalloc(workspace)", __FILE__, __LINE__);
    ctx->ws_bytes = want;
    return TLNN_OK;
}

// ---- launch bookkeeping and profiling ----------------------------------------------------------------
static cudaEvent_t take_event(tlnn_ctx* ctx) {
    if (!ctx->event_pool.empty()) {
        cudaEvent_t e = ctx->event_pool.back();
        ctx->event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

int tl_launch_begin(tlnn_ctx* ctx, const char* name) {
    if (ctx->prof_classes) {
        tl_prof_pending p;
        p.name = name;
        p.start = take_event(ctx);
        p.stop = take_event(ctx);
        TL_CUDA(cudaEventRecord(p.start, ctx->stream));
        ctx->pending.push_back(p);
    }
    return TLNN_OK;
}

int tl_launch_end(tlnn_ctx* ctx, const char* name) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        tl_set_error("launch of %s failed: %s", name, cudaGetErrorString(e));
        return TLNN_ERR_CUDA;
    }
    ctx->launches++;
    if (ctx->prof_classes) TL_CUDA(cudaEventRecord(ctx->pending.back().stop, ctx->stream));
    return TLNN_OK;
}

static int drain_pending(tlnn_ctx* ctx) {
    if (ctx->pending.empty()) return TLNN_OK;
    TL_CUDA(cudaStreamSynchronize(ctx->stream));
    for (auto& p : ctx->pending) {
        float ms = 0.f;
        TL_CUDA(cudaEventElapsedTime(&ms, p.start, p.stop));
        auto& row = ctx->table[p.name];
        row.first += 1;
        row.second += ms;
        ctx->event_pool.push_back(p.start);
        ctx->event_pool.push_back(p.stop);
    }
    ctx->pending.clear();
    return TLNN_OK;
}

extern "C" int tlnn_prof_begin(tlnn_ctx* ctx) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaEventRecord(ctx->prof_a, ctx->stream));
    return TLNN_OK;
}

extern "C" int tlnn_prof_end(tlnn_ctx* ctx, float* ms) {
    TL_NOTNULL(ctx);
    TL_NOTNULL(ms);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_CUDA(cudaEventRecord(ctx->prof_b, ctx->stream));
    TL_CUDA(cudaEventSynchronize(ctx->prof_b));
    TL_CUDA(cudaEventElapsedTime(ms, ctx->prof_a, ctx->prof_b));
    return TLNN_OK;
}

extern "C" int tlnn_prof_classes(tlnn_ctx* ctx, int enable) {
    TL_NOTNULL(ctx);
    TL_CUDA(cudaSetDevice(ctx->device));
    TL_TRY(drain_pending(ctx));
    if (enable && !ctx->prof_classes) ctx->table.clear();
    ctx->prof_classes = enable != 0;
    return TLNN_OK;
}

extern "C" int tlnn_prof_table(tlnn_ctx* ctx, tlnn_prof_row* rows, int cap) {
    if (!ctx) return TLNN_ERR_NULL;
    cudaSetDevice(ctx->device);
    if (drain_pending(ctx) != TLNN_OK) return TLNN_ERR_CUDA;
    int n = 0;
    for (auto& kv : ctx->table) {
        if (rows && n < cap) {
            memset(&rows[n], 0, sizeof(tlnn_prof_row));
            strncpy(rows[n].name, kv.first.c_str(), sizeof(rows[n].name) - 1);
            rows[n].launches = kv.second.first;
            rows[n].ms = kv.second.second;
        }
        n++;
    }
    return n;
}
