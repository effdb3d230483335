// Data parallelism behind the C ABI: one NCCL communicator per process (one process per GPU).
//
// The path shards over the batch (every convolution, activation and loss is per image; only the
// weight / bias gradients reduce over it), so the single exchange of an update is a sum of that
// network's contiguous gradient arena over the ranks - ncclAllReduce over NVLink / NVSwitch - before
// the replicated Adam step divides by the world size.  The reference has no multi-GPU code; this is
// the counterpart of nothing in it and of dcgan/main.cu:378-391 run on N shards.
//
// NCCL is not linked: the library is looked up at run time (dlopen of libnccl.so.2 - in a process
// that already uses NCCL, e.g. through torch.distributed, that is the copy already loaded), so
// libdcgan_b200.so still loads on a machine without NCCL and single-GPU users never touch it.
// The collective is enqueued on the caller's stream and never synchronises; it can be captured
// into a CUDA graph with the kernels around it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*MemAlloc)(void**, size_t) = nullptr;      // optional
    ncclResult_t (*MemFree)(void*) = nullptr;                // optional
    ncclResult_t (*CommRegister)(const ncclComm_t, void*, size_t, void**) = nullptr;   // optional
    ncclResult_t (*CommDeregister)(const ncclComm_t, void*) = nullptr;                 // optional
    ncclResult_t (*GetVersion)(int*) = nullptr;
    bool ok = false;
};

NcclApi& api()
{
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy the process already uses, if any
        if (!a.handle) a.handle = dlopen("libnccl.so.2", RTLD_NOW);
        if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW);
        if (!a.handle) return;
        auto sym = [&](const char* name) { return dlsym(a.handle, name); };
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
        a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
        a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
        a.MemAlloc = reinterpret_cast<decltype(a.MemAlloc)>(sym("ncclMemAlloc"));
        a.MemFree = reinterpret_cast<decltype(a.MemFree)>(sym("ncclMemFree"));
        a.CommRegister = reinterpret_cast<decltype(a.CommRegister)>(sym("ncclCommRegister"));
        a.CommDeregister = reinterpret_cast<decltype(a.CommDeregister)>(sym("ncclCommDeregister"));
        a.GetVersion = reinterpret_cast<decltype(a.GetVersion)>(sym("ncclGetVersion"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.CommDestroy && a.GetErrorString && a.GroupStart &&
               a.GroupEnd;
    });
    return a;
}

int nccl_fail(const char* what, ncclResult_t r)
{
    return dcg::fail(DCG_ERR_CUDA, "%s failed: %s", what, api().GetErrorString ? api().GetErrorString(r) : "NCCL error");
}

}  // namespace

struct dcg_dp {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    void* reg_handle[4] = {nullptr, nullptr, nullptr, nullptr};
    int n_reg = 0;
};

namespace dcg {

// Device memory NCCL can map for its in-switch (NVLS) user-buffer path, or nullptr when the loaded
// NCCL has no ncclMemAlloc or the allocation fails (the caller then uses cudaMalloc).
void* dp_mem_alloc(size_t bytes)
{
    NcclApi& a = api();
    if (!a.ok || !a.MemAlloc || !a.MemFree) return nullptr;
    void* p = nullptr;
    if (a.MemAlloc(&p, bytes) != ncclSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

void dp_mem_free(void* p)
{
    if (p && api().MemFree) api().MemFree(p);
}

// Registers a buffer the communicator will reduce in place over and over (best effort).
void dp_register(dcg_dp* dp, void* buf, size_t bytes)
{
    NcclApi& a = api();
    if (!dp || !dp->comm || !a.CommRegister || dp->n_reg >= 4) return;
    void* h = nullptr;
    if (a.CommRegister(dp->comm, buf, bytes, &h) == ncclSuccess && h) dp->reg_handle[dp->n_reg++] = h;
    else cudaGetLastError();
}

int dp_world(const dcg_dp* dp) { return dp ? dp->world : 1; }
int dp_rank(const dcg_dp* dp) { return dp ? dp->rank : 0; }

// Maps every rank's copy of a cudaMalloc'ed buffer into this process: each rank exports an IPC handle
// of `local_base`, the handles travel through the communicator (an all-gather of 64-byte records),
// and the peers' buffers are opened with peer access enabled.  bases[r] is rank r's buffer as seen
// from this GPU (bases[rank] = local_base).  Collective.  Every rank learns whether ALL succeeded:
// returns DCG_OK only then (the caller falls back to NCCL collectives otherwise), and on failure
// whatever this rank had opened is closed again.
int dp_map_peers(dcg_dp* dp, void* local_base, void** bases /* [world] */)
{
    NcclApi& a = api();
    DCG_CHECK_ARG(dp && dp->comm && a.ok && a.AllGather, "dcg_dp: no communicator");
    const int W = dp->world;
    DCG_CHECK_ARG(W <= 8, "dcg_dp: peer mapping supports up to 8 ranks");
    struct Record { cudaIpcMemHandle_t handle; int ok; int pad[3]; };
    Record mine;
    std::memset(&mine, 0, sizeof(mine));
    mine.ok = cudaIpcGetMemHandle(&mine.handle, local_base) == cudaSuccess ? 1 : 0;
    if (!mine.ok) cudaGetLastError();
    Record *d_send = nullptr, *d_recv = nullptr;
    Record all[8];
    cudaStream_t s = nullptr;
    bool ok = cudaMalloc(&d_send, sizeof(Record)) == cudaSuccess && cudaMalloc(&d_recv, sizeof(Record) * W) == cudaSuccess &&
              cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess;
    auto gather = [&](const Record& r) {   // collective: every rank must call it the same number of times
        if (!ok) return false;
        if (cudaMemcpyAsync(d_send, &r, sizeof(Record), cudaMemcpyHostToDevice, s) != cudaSuccess) return false;
        if (a.AllGather(d_send, d_recv, sizeof(Record), ncclChar, dp->comm, s) != ncclSuccess) return false;
        if (cudaMemcpyAsync(all, d_recv, sizeof(Record) * W, cudaMemcpyDeviceToHost, s) != cudaSuccess) return false;
        return cudaStreamSynchronize(s) == cudaSuccess;
    };
    bool fine = gather(mine);
    for (int r = 0; fine && r < W; ++r) fine = all[r].ok != 0;
    int opened = 0;
    for (int r = 0; r < W; ++r) bases[r] = nullptr;
    if (fine) {
        for (int r = 0; r < W; ++r) {
            if (r == dp->rank) { bases[r] = local_base; continue; }
            if (cudaIpcOpenMemHandle(&bases[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                bases[r] = nullptr;
                fine = false;
                break;
            }
            ++opened;
        }
    }
    // second round: did every rank manage to open every peer?
    Record verdict;
    std::memset(&verdict, 0, sizeof(verdict));
    verdict.ok = fine ? 1 : 0;
    bool all_fine = gather(verdict);
    for (int r = 0; all_fine && r < W; ++r) all_fine = all[r].ok != 0;
    if (!all_fine) {
        for (int r = 0; r < W; ++r)
            if (r != dp->rank && bases[r]) { cudaIpcCloseMemHandle(bases[r]); bases[r] = nullptr; }
        (void)opened;
    }
    if (d_send) cudaFree(d_send);
    if (d_recv) cudaFree(d_recv);
    if (s) cudaStreamDestroy(s);
    cudaGetLastError();
    return all_fine ? DCG_OK : fail(DCG_ERR_UNSUPPORTED, "dcg_dp: the ranks could not map each other's memory");
}

void dp_unmap_peers(dcg_dp* dp, void** bases)
{
    if (!dp) return;
    for (int r = 0; r < dp->world && r < 8; ++r)
        if (r != dp->rank && bases[r]) { cudaIpcCloseMemHandle(bases[r]); bases[r] = nullptr; }
}

// Several in-place sums as one NCCL group (one launch).
int dp_allreduce_group(dcg_dp* dp, float* const* bufs, const size_t* counts, int n, cudaStream_t stream)
{
    NcclApi& a = api();
    DCG_CHECK_ARG(dp && dp->comm && a.ok, "dcg_dp: no communicator");
    ncclResult_t r = a.GroupStart();
    if (r != ncclSuccess) return nccl_fail("ncclGroupStart", r);
    for (int i = 0; i < n; ++i) {
        if (counts[i] == 0) continue;
        r = a.AllReduce(bufs[i], bufs[i], counts[i], ncclFloat, ncclSum, dp->comm, stream);
        if (r != ncclSuccess) { a.GroupEnd(); return nccl_fail("ncclAllReduce", r); }
    }
    r = a.GroupEnd();
    if (r != ncclSuccess) return nccl_fail("ncclGroupEnd", r);
    return DCG_OK;
}

}  // namespace dcg

extern "C" int dcg_dp_unique_id(void* id_out)
{
    DCG_CHECK_ARG(id_out, "dcg_dp_unique_id: null output");
    static_assert(sizeof(ncclUniqueId) == DCG_DP_ID_BYTES, "unique id size");
    NcclApi& a = api();
    if (!a.ok) return dcg::fail(DCG_ERR_UNSUPPORTED, "dcg_dp: libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    const ncclResult_t r = a.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail("ncclGetUniqueId", r);
    std::memcpy(id_out, &id, sizeof(id));
    return DCG_OK;
}

extern "C" int dcg_dp_init(dcg_dp** out, int rank, int world, const void* unique_id)
{
    DCG_CHECK_ARG(out && unique_id, "dcg_dp_init: null argument");
    DCG_CHECK_ARG(world >= 1 && rank >= 0 && rank < world, "dcg_dp_init: rank %d of %d", rank, world);
    NcclApi& a = api();
    if (!a.ok) return dcg::fail(DCG_ERR_UNSUPPORTED, "dcg_dp: libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    std::memcpy(&id, unique_id, sizeof(id));
    dcg_dp* dp = new dcg_dp();
    dp->rank = rank;
    dp->world = world;
    const ncclResult_t r = a.CommInitRank(&dp->comm, world, id, rank);   // on the current device
    if (r != ncclSuccess) {
        delete dp;
        return nccl_fail("ncclCommInitRank", r);
    }
    *out = dp;
    return DCG_OK;
}

extern "C" int dcg_dp_allreduce(dcg_dp* dp, float* buf, size_t count, dcg_stream_t stream)
{
    DCG_CHECK_ARG(dp && dp->comm && buf, "dcg_dp_allreduce: null argument");
    NcclApi& a = api();
    const ncclResult_t r = a.AllReduce(buf, buf, count, ncclFloat, ncclSum, dp->comm, dcg::as_stream(stream));
    if (r != ncclSuccess) return nccl_fail("ncclAllReduce", r);
    return DCG_OK;
}

extern "C" int dcg_dp_info(const dcg_dp* dp, int* rank, int* world, int* nccl_version)
{
    DCG_CHECK_ARG(dp, "dcg_dp_info: null communicator");
    if (rank) *rank = dp->rank;
    if (world) *world = dp->world;
    if (nccl_version) {
        *nccl_version = 0;
        if (api().GetVersion) api().GetVersion(nccl_version);
    }
    return DCG_OK;
}

extern "C" void dcg_dp_finalize(dcg_dp* dp)
{
    if (!dp) return;
    NcclApi& a = api();
    if (dp->comm) {
        for (int i = 0; i < dp->n_reg; ++i)
            if (a.CommDeregister) a.CommDeregister(dp->comm, dp->reg_handle[i]);
        if (a.CommDestroy) a.CommDestroy(dp->comm);
    }
    delete dp;
}
