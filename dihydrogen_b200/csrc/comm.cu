// Sum all-reduce of short device vectors: NCCL flavour (library resolved at
// run time) and a peer-memory flavour whose kernels store every rank's
// contribution into every peer's mapped slot and fold the slots in rank order.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

namespace dcb
{

struct NcclApi
{
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t,
                              ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

static NcclApi& nccl_api()
{
    static NcclApi api;
    static bool tried = false;
    if (tried)
        return api;
    tried = true;
    // Reuse a copy that is already in the process (e.g. the one a Python
    // host loaded) before falling back to the system library.
    api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!api.handle)
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!api.handle)
        api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!api.handle)
        return api;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(
        dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(
        dlsym(api.handle, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(
        dlsym(api.handle, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(
        dlsym(api.handle, "ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(
        dlsym(api.handle, "ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy
             && api.AllReduce && api.GetErrorString;
    return api;
}

#define DCB_NCCL_TRY(expr)                                                     \
    do                                                                         \
    {                                                                          \
        ncclResult_t r__ = (expr);                                             \
        if (r__ != ncclSuccess)                                                \
        {                                                                      \
            set_last_error(std::string(#expr) + ": "                           \
                           + nccl_api().GetErrorString(r__));                  \
            return DCB_NCCL_ERROR;                                             \
        }                                                                      \
    } while (0)

constexpr size_t kCommHeader = 512; // flags (<= 64 ranks) + status
constexpr int kMaxPeerRanks = 64;

struct CommBlob
{
    WindowBlob win;
    uint32_t rank;
    uint32_t max_count;
};
static_assert(sizeof(CommBlob) <= DCB_COMM_BLOB_BYTES, "blob too large");

struct PeerPtrs
{
    char* base[kMaxPeerRanks];
};

// Store my vector into slot [parity][my rank] of every rank's window, then
// publish the epoch in every rank's flag word for me.
__device__ __forceinline__ void push_body(const PeerPtrs& peers, int nranks,
                                          int rank, int max_count,
                                          const float* data, int count,
                                          uint32_t epoch)
{
    const int par = epoch & 1;
    for (int p = 0; p < nranks; ++p)
    {
        float* slot = reinterpret_cast<float*>(peers.base[p] + kCommHeader)
                      + ((size_t) par * nranks + rank) * max_count;
        for (int i = threadIdx.x; i < count; i += blockDim.x)
            slot[i] = data[i];
    }
    __threadfence_system();
    __syncthreads();
    for (int p = threadIdx.x; p < nranks; p += blockDim.x)
        st_release_sys(reinterpret_cast<uint32_t*>(peers.base[p]) + rank,
                       epoch);
}

// Wait for every rank's flag, then fold the slots in rank order.
__device__ __forceinline__ void pull_body(char* mine, int nranks, int max_count,
                                          float* data, int count,
                                          uint32_t epoch, long long budget_ns)
{
    __shared__ int bad;
    if (threadIdx.x == 0)
        bad = 0;
    __syncthreads();
    uint32_t* flags = reinterpret_cast<uint32_t*>(mine);
    for (int r = threadIdx.x; r < nranks; r += blockDim.x)
        if (!bounded_wait_epoch(flags + r, epoch, budget_ns))
            atomicExch(&bad, 1);
    __syncthreads();
    if (bad)
    {
        if (threadIdx.x == 0)
            atomicExch(reinterpret_cast<int*>(flags + kMaxPeerRanks),
                       (int) DCB_PEER_TIMEOUT);
        return;
    }
    const int par = epoch & 1;
    const float* slots = reinterpret_cast<const float*>(mine + kCommHeader)
                         + (size_t) par * nranks * max_count;
    for (int i = threadIdx.x; i < count; i += blockDim.x)
    {
        float s = slots[i];
        for (int r = 1; r < nranks; ++r)
            s += slots[(size_t) r * max_count + i];
        data[i] = s;
    }
}

__global__ void peer_push_kernel(PeerPtrs peers, int nranks, int rank,
                                 int max_count, const float* data, int count,
                                 uint32_t epoch)
{
    push_body(peers, nranks, rank, max_count, data, count, epoch);
}

__global__ void peer_pull_kernel(char* mine, int nranks, int max_count,
                                 float* data, int count, uint32_t epoch,
                                 long long budget_ns)
{
    pull_body(mine, nranks, max_count, data, count, epoch, budget_ns);
}

__global__ void peer_allreduce_kernel(PeerPtrs peers, int nranks, int rank,
                                      int max_count, float* data, int count,
                                      uint32_t epoch, long long budget_ns)
{
    push_body(peers, nranks, rank, max_count, data, count, epoch);
    __syncthreads();
    pull_body(peers.base[rank], nranks, max_count, data, count, epoch,
              budget_ns);
}

} // namespace dcb

using namespace dcb;

struct dcb_comm
{
    int kind; // 0 nccl, 1 peer
    int rank, nranks;
    ncclComm_t nccl = nullptr;
    Window win;
    int max_count = 0;
    uint32_t epoch = 0;
    PeerMapping maps[kMaxPeerRanks];
    PeerPtrs ptrs;
    bool connected = false;
};

extern "C" {

int32_t dcb_nccl_unique_id(void* id_out)
{
    DCB_REQUIRE(id_out, "null argument");
    static_assert(sizeof(ncclUniqueId) <= DCB_NCCL_ID_BYTES, "id size");
    if (!nccl_api().ok)
    {
        set_last_error("NCCL library could not be loaded");
        return DCB_NCCL_ERROR;
    }
    ncclUniqueId id;
    DCB_NCCL_TRY(nccl_api().GetUniqueId(&id));
    std::memset(id_out, 0, DCB_NCCL_ID_BYTES);
    std::memcpy(id_out, &id, sizeof(id));
    return DCB_OK;
}

int32_t dcb_comm_create_nccl(const void* id, int32_t rank, int32_t nranks,
                             dcb_comm** out)
{
    DCB_REQUIRE(id && out, "null argument");
    DCB_REQUIRE(rank >= 0 && rank < nranks, "rank out of range");
    if (!nccl_api().ok)
    {
        set_last_error("NCCL library could not be loaded");
        return DCB_NCCL_ERROR;
    }
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    auto* c = new dcb_comm();
    c->kind = 0;
    c->rank = rank;
    c->nranks = nranks;
    ncclResult_t r = nccl_api().CommInitRank(&c->nccl, nranks, uid, rank);
    if (r != ncclSuccess)
    {
        set_last_error(std::string("ncclCommInitRank: ")
                       + nccl_api().GetErrorString(r));
        delete c;
        return DCB_NCCL_ERROR;
    }
    *out = c;
    return DCB_OK;
}

int32_t dcb_comm_create_peer(int32_t rank, int32_t nranks, int32_t max_count,
                             dcb_comm** out)
{
    DCB_REQUIRE(out, "null argument");
    DCB_REQUIRE(nranks >= 1 && nranks <= kMaxPeerRanks, "nranks must be 1..64");
    DCB_REQUIRE(rank >= 0 && rank < nranks, "rank out of range");
    DCB_REQUIRE(max_count > 0 && max_count <= (1 << 20), "max_count out of range");
    auto* c = new dcb_comm();
    c->kind = 1;
    c->rank = rank;
    c->nranks = nranks;
    c->max_count = (max_count + 3) / 4 * 4;
    const size_t bytes =
        kCommHeader + 2ull * nranks * c->max_count * sizeof(float);
    int32_t st = c->win.allocate(bytes);
    if (st != DCB_OK)
    {
        delete c;
        return st;
    }
    *out = c;
    return DCB_OK;
}

int32_t dcb_comm_export(dcb_comm* c, void* blob)
{
    DCB_REQUIRE(c && blob, "null argument");
    DCB_REQUIRE(c->kind == 1, "only peer communicators export a blob");
    CommBlob b;
    std::memset(&b, 0, sizeof(b));
    c->win.fill_blob(&b.win);
    b.rank = (uint32_t) c->rank;
    b.max_count = (uint32_t) c->max_count;
    std::memset(blob, 0, DCB_COMM_BLOB_BYTES);
    std::memcpy(blob, &b, sizeof(b));
    return DCB_OK;
}

int32_t dcb_comm_connect(dcb_comm* c, const void* blobs, int32_t nranks)
{
    DCB_REQUIRE(c && blobs, "null argument");
    DCB_REQUIRE(c->kind == 1, "only peer communicators connect");
    DCB_REQUIRE(nranks == c->nranks, "nranks differs from creation");
    for (int r = 0; r < nranks; ++r)
    {
        CommBlob b;
        std::memcpy(&b,
                    static_cast<const char*>(blobs)
                        + (size_t) r * DCB_COMM_BLOB_BYTES,
                    sizeof(b));
        DCB_REQUIRE((int) b.rank == r, "blob order does not match ranks");
        DCB_REQUIRE((int) b.max_count == c->max_count, "max_count differs");
        if (r == c->rank)
        {
            c->ptrs.base[r] = static_cast<char*>(c->win.base);
            continue;
        }
        int32_t st = c->maps[r].open(b.win, c->win.device);
        if (st != DCB_OK)
            return st;
        c->ptrs.base[r] = static_cast<char*>(c->maps[r].base);
    }
    c->connected = true;
    return DCB_OK;
}

int32_t dcb_comm_destroy(dcb_comm* c)
{
    if (!c)
        return DCB_OK;
    if (c->kind == 0 && c->nccl)
        nccl_api().CommDestroy(c->nccl);
    for (auto& m : c->maps)
        m.close();
    c->win.release();
    delete c;
    return DCB_OK;
}

static int32_t peer_ready(dcb_comm* c, int64_t count)
{
    DCB_REQUIRE(c->kind == 1, "not a peer communicator");
    DCB_REQUIRE(count >= 0 && count <= c->max_count,
                "count exceeds the communicator's max_count");
    if (!c->connected)
    {
        set_last_error("peer communicator was never connected");
        return DCB_NOT_CONNECTED;
    }
    return DCB_OK;
}

int32_t dcb_allreduce_sum(dcb_comm* c, void* data, int64_t count, void* stream)
{
    DCB_REQUIRE(c && (data || count == 0), "null argument");
    if (count == 0)
        return DCB_OK;
    if (c->kind == 0)
    {
        DCB_NCCL_TRY(nccl_api().AllReduce(data, data, (size_t) count, ncclFloat,
                                          ncclSum, c->nccl, as_stream(stream)));
        return DCB_OK;
    }
    int32_t st = peer_ready(c, 0);
    if (st != DCB_OK)
        return st;
    if (c->nranks == 1)
        return DCB_OK; // the sum over one rank is the vector itself: nothing to launch
    // A vector longer than the slots (a filter gradient, K*C*taps floats) goes
    // through in max_count-sized pieces, one epoch each.  The slots are double
    // buffered by epoch parity, and a rank can only be one epoch ahead of the
    // slowest (its pull of epoch e needs everybody's push of epoch e), so
    // back-to-back epochs never overwrite a slot that is still being read.
    float* p = static_cast<float*>(data);
    for (int64_t done = 0; done < count; done += c->max_count)
    {
        const int64_t n = count - done < c->max_count ? count - done : c->max_count;
        const uint32_t epoch = ++c->epoch;
        peer_allreduce_kernel<<<1, 256, 0, as_stream(stream)>>>(
            c->ptrs, c->nranks, c->rank, c->max_count, p + done, (int) n, epoch,
            wait_budget_ns());
        DCB_LAUNCH_CHECK();
    }
    return DCB_OK;
}

int32_t dcb_allreduce_push(dcb_comm* c, const void* data, int64_t count,
                           void* stream)
{
    DCB_REQUIRE(c && data, "null argument");
    int32_t st = peer_ready(c, count);
    if (st != DCB_OK)
        return st;
    const uint32_t epoch = ++c->epoch;
    peer_push_kernel<<<1, 256, 0, as_stream(stream)>>>(
        c->ptrs, c->nranks, c->rank, c->max_count,
        static_cast<const float*>(data), (int) count, epoch);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_allreduce_pull(dcb_comm* c, void* data, int64_t count, void* stream)
{
    DCB_REQUIRE(c && data, "null argument");
    int32_t st = peer_ready(c, count);
    if (st != DCB_OK)
        return st;
    peer_pull_kernel<<<1, 256, 0, as_stream(stream)>>>(
        static_cast<char*>(c->win.base), c->nranks, c->max_count,
        static_cast<float*>(data), (int) count, c->epoch, wait_budget_ns());
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_comm_status(dcb_comm* c, void* stream)
{
    DCB_REQUIRE(c, "null argument");
    DCB_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    if (c->kind != 1)
        return DCB_OK;
    int st = 0;
    int* word = reinterpret_cast<int*>(static_cast<uint32_t*>(c->win.base)
                                       + kMaxPeerRanks);
    DCB_CUDA_TRY(cudaMemcpy(&st, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0)
    {
        DCB_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
        set_last_error("a wait on a peer's all-reduce flag ran out of budget");
        return DCB_PEER_TIMEOUT;
    }
    return DCB_OK;
}

} // extern "C"
