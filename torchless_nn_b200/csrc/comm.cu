// Multi-GPU entry points of libtlnn: one communicator per context (one process per GPU), collectives enqueued on the
// context's compute stream so that they are ordered after the kernels that produce their input.
//
// The path shards by batch rows and exchanges only results (int32 arg-max tokens, or float32 logits on request), so the
// collectives are NCCL all-gathers; nothing here reads a peer's memory from a kernel of this library.
//
// NCCL is bound at run time (dlopen), not at link time: a single-GPU user needs no NCCL installation, and a process
// that already carries an NCCL (another framework's) shares that copy instead of loading a second one.  The library
// name is TLNN_NCCL_LIB if set, else "libnccl.so.2".
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>      // types and enumerators only; every function is resolved with dlsym

#include <mutex>

namespace {

struct nccl_api {
    void* handle = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    const char* (*GetLastError)(ncclComm_t) = nullptr;
    std::string error;
};

nccl_api g_nccl;
std::once_flag g_nccl_once;

template <typename F>
bool bind(void* h, const char* name, F& fn, std::string& err) {
    fn = reinterpret_cast<F>(dlsym(h, name));
    if (!fn) { err = std::string("symbol ") + name + " not found in the NCCL library"; return false; }
    return true;
}

void load_nccl() {
    const char* path = getenv("TLNN_NCCL_LIB");
    if (!path || !*path) path = "libnccl.so.2";
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { g_nccl.error = std::string("cannot load ") + path + ": " + dlerror(); return; }
    nccl_api& a = g_nccl;
    bool ok = bind(h, "ncclGetVersion", a.GetVersion, a.error) && bind(h, "ncclGetUniqueId", a.GetUniqueId, a.error) &&
              bind(h, "ncclCommInitRank", a.CommInitRank, a.error) && bind(h, "ncclCommDestroy", a.CommDestroy, a.error) &&
              bind(h, "ncclCommAbort", a.CommAbort, a.error) && bind(h, "ncclAllGather", a.AllGather, a.error) &&
              bind(h, "ncclAllReduce", a.AllReduce, a.error) && bind(h, "ncclBroadcast", a.Broadcast, a.error) &&
              bind(h, "ncclGroupStart", a.GroupStart, a.error) && bind(h, "ncclGroupEnd", a.GroupEnd, a.error) &&
              bind(h, "ncclGetErrorString", a.GetErrorString, a.error);
    if (!ok) { dlclose(h); return; }
    a.GetLastError = reinterpret_cast<const char* (*)(ncclComm_t)>(dlsym(h, "ncclGetLastError"));   // optional
    a.handle = h;
}

int need_nccl() {
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.handle) {
        tl_set_error("multi-GPU support is unavailable: %s", g_nccl.error.c_str());
        return TLNN_ERR_CUDA;
    }
    return TLNN_OK;
}

int nccl_fail(ncclResult_t r, const char* what, ncclComm_t comm) {
    const char* more = (g_nccl.GetLastError && comm) ? g_nccl.GetLastError(comm) : "";
    tl_set_error("NCCL error %d (%s) in %s %s", (int)r, g_nccl.GetErrorString(r), what, more ? more : "");
    return TLNN_ERR_CUDA;
}

#define TL_NCCL(call, comm)                                                   \
    do {                                                                      \
        ncclResult_t r_ = (call);                                             \
        if (r_ != ncclSuccess) return nccl_fail(r_, #call, comm);             \
    } while (0)

}  // namespace

struct tlnn_comm {
    tlnn_ctx* ctx = nullptr;
    ncclComm_t nccl = nullptr;
    int rank = 0, world = 1;
    int* d_flag = nullptr;        // one int on the device: the barrier's all-reduce operand
};

extern "C" int tlnn_comm_nccl_version(int* version) {
    TL_NOTNULL(version);
    TL_TRY(need_nccl());
    TL_NCCL(g_nccl.GetVersion(version), nullptr);
    return TLNN_OK;
}

extern "C" int tlnn_comm_unique_id(void* id_bytes) {
    TL_NOTNULL(id_bytes);
    static_assert(TLNN_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the identifier is NCCL's");
    TL_TRY(need_nccl());
    ncclUniqueId id;
    TL_NCCL(g_nccl.GetUniqueId(&id), nullptr);
    memcpy(id_bytes, id.internal, TLNN_COMM_ID_BYTES);
    return TLNN_OK;
}

extern "C" int tlnn_comm_init(tlnn_ctx* ctx, const void* id_bytes, int rank, int world, tlnn_comm** out) {
    TL_NOTNULL(ctx); TL_NOTNULL(id_bytes); TL_NOTNULL(out);
    TL_REQUIRE(world >= 1 && rank >= 0 && rank < world, "comm_init: rank %d of %d", rank, world);
    // Host-side failure injection for tests: refuse before any GPU or network work.
    const char* inject = getenv("TLNN_COMM_FAIL_INIT");
    if (inject && strcmp(inject, "1") == 0) {
        tl_set_error("comm_init: refused by TLNN_COMM_FAIL_INIT=1 (failure injection)");
        return TLNN_ERR_CUDA;
    }
    TL_TRY(need_nccl());
    TL_CUDA(cudaSetDevice(ctx->device));
    tlnn_comm* c = new tlnn_comm();
    c->ctx = ctx; c->rank = rank; c->world = world;
    ncclUniqueId id;
    memcpy(id.internal, id_bytes, TLNN_COMM_ID_BYTES);
    ncclResult_t r = g_nccl.CommInitRank(&c->nccl, world, id, rank);
    if (r != ncclSuccess) { delete c; return nccl_fail(r, "ncclCommInitRank", nullptr); }
    cudaError_t e = cudaMalloc(&c->d_flag, 256);
    if (e == cudaSuccess) e = cudaMemset(c->d_flag, 0, 256);
    if (e != cudaSuccess) { g_nccl.CommAbort(c->nccl); delete c; return tl_cuda_fail(e, "comm_init", __FILE__, __LINE__); }
    *out = c;
    return TLNN_OK;
}

extern "C" int tlnn_comm_destroy(tlnn_comm* c) {
    if (!c) return TLNN_OK;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    if (c->nccl && g_nccl.handle) g_nccl.CommDestroy(c->nccl);
    if (c->d_flag) cudaFree(c->d_flag);
    delete c;
    return TLNN_OK;
}

extern "C" int tlnn_comm_rank(tlnn_comm* c, int* rank, int* world) {
    TL_NOTNULL(c);
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return TLNN_OK;
}

// Rank r contributes counts[r] elements (n_local everywhere when counts is null); `all` receives them in rank order.
static int allgather(tlnn_comm* c, const void* local, void* all, long long n_local, const long long* counts,
                     ncclDataType_t type, size_t elem, const char* name) {
    TL_NOTNULL(c); TL_NOTNULL(all);
    TL_REQUIRE(n_local >= 0, "%s: negative element count", name);
    tlnn_ctx* ctx = c->ctx;
    TL_CUDA(cudaSetDevice(ctx->device));
    bool even = true;
    long long total = 0;
    if (counts) {
        for (int r = 0; r < c->world; r++) {
            TL_REQUIRE(counts[r] >= 0, "%s: negative count for rank %d", name, r);
            even = even && counts[r] == counts[0];
            total += counts[r];
        }
        TL_REQUIRE(counts[c->rank] == n_local, "%s: this rank passes %lld elements but counts[%d] is %lld", name, n_local,
                   c->rank, counts[c->rank]);
    } else {
        total = n_local * c->world;
    }
    if (total == 0) return TLNN_OK;
    if (n_local > 0) TL_NOTNULL(local);
    if (even) {
        TL_NCCL(g_nccl.AllGather(local, all, (size_t)n_local, type, c->nccl, ctx->stream), c->nccl);
    } else {
        // ragged shards: one broadcast per rank, fused into one NCCL group
        TL_NCCL(g_nccl.GroupStart(), c->nccl);
        long long off = 0;
        for (int r = 0; r < c->world; r++) {
            if (counts[r] > 0) {
                char* dst = static_cast<char*>(all) + (size_t)off * elem;
                ncclResult_t rr = g_nccl.Broadcast(r == c->rank ? local : dst, dst, (size_t)counts[r], type, r, c->nccl, ctx->stream);
                if (rr != ncclSuccess) { g_nccl.GroupEnd(); return nccl_fail(rr, "ncclBroadcast", c->nccl); }
            }
            off += counts[r];
        }
        TL_NCCL(g_nccl.GroupEnd(), c->nccl);
    }
    return TLNN_OK;
}

extern "C" int tlnn_allgather_tokens(tlnn_comm* c, const int32_t* local, int32_t* all, long long n_local,
                                     const long long* counts) {
    return allgather(c, local, all, n_local, counts, ncclInt32, 4, "allgather_tokens");
}

extern "C" int tlnn_allgather_logits(tlnn_comm* c, const float* local, float* all, long long n_local,
                                     const long long* counts) {
    return allgather(c, local, all, n_local, counts, ncclFloat32, 4, "allgather_logits");
}

extern "C" int tlnn_comm_barrier(tlnn_comm* c) {
    TL_NOTNULL(c);
    TL_CUDA(cudaSetDevice(c->ctx->device));
    TL_NCCL(g_nccl.AllReduce(c->d_flag, c->d_flag, 1, ncclInt32, ncclSum, c->nccl, c->ctx->stream), c->nccl);
    return tlnn_sync(c->ctx);
}
