// Re-distribution of a tensor between two block decompositions (sample-parallel
// <-> spatially partitioned, or any other pair): stands in for
// tensor::TensorMPICUDAShuffler
// (legacy/include/distconv/tensor/shuffle_mpi_cuda.hpp:14-512), which packs per
// destination rank, runs an MPI all-to-all-v through host-visible buffers and
// unpacks.
//
// Here every rank owns a receive window (IPC-mapped by its peers) shaped like
// its destination block, dense, W fastest, twice (consecutive shuffles
// alternate).  One kernel per rank, `put`, walks the intersections of the
// rank's source block with every destination block and stores the cells
// straight into the owners' windows (NVLink peer stores; the local part is an
// ordinary copy), then release-stores its epoch into a flag per destination.
// A second kernel, `wait_unpack`, waits (bounded) for the epochs of all ranks
// that hold a part of its block and copies the window into the destination
// tensor, skipping its halo.  No host staging, no collective call; ranks may
// run at most one shuffle apart, as with the halo exchange.
//
// HBM-bound: 8 B per cell at the sender (read + peer write), 8 B at the
// receiver (window read + tensor write).
#include "common.cuh"
#include "dcb.h"

#include <cstring>
#include <vector>

namespace dcb
{
namespace
{

constexpr int SHF_THREADS = 256;
constexpr int SHF_MAX_RANKS = 64;
constexpr size_t SHF_HEADER = 1024; // 64 flags, ticket, status

// One box to move: `rows` runs of `len` contiguous cells.  Row r decodes into
// (i1, i2, i3, i4) over ext[1..4]; its first cell sits at
// a_off + sum i_k * a_stride[k] on the strided side and at
// b_off + sum i_k * b_stride[k] on the dense side.
struct ShfJob
{
    long long rows, len;
    long long ext[4];
    long long a_off, a_stride[4];
    long long b_off, b_stride[4];
    float* peer;            // put: the destination's window (parity 0)
    long long parity_pitch; // put: floats between the two halves of that window
    uint32_t* flag;         // put: flag to publish there; wait: own flag to wait on
};

struct ShfArgs
{
    const ShfJob* jobs;
    int njobs;
    long long total_rows;
    float* tensor;
    float* window; // wait_unpack: own window of this parity
    int parity;    // put: which half of the destination windows
    uint32_t epoch;
    uint32_t* ticket;
    int* status;
    long long budget_ns;
};

__device__ __forceinline__ void shf_locate(const ShfJob& j, long long r, long long* a, long long* b)
{
    long long ao = j.a_off, bo = j.b_off;
#pragma unroll
    for (int k = 0; k < 4; ++k)
    {
        const long long i = r % j.ext[k];
        r /= j.ext[k];
        ao += i * j.a_stride[k];
        bo += i * j.b_stride[k];
    }
    *a = ao;
    *b = bo;
}

// PUT: tensor (strided) -> peers' windows (dense).  !PUT: own window -> tensor.
template <bool PUT>
__global__ void __launch_bounds__(SHF_THREADS) shuffle_kernel(ShfArgs a)
{
    if (!PUT)
    {
        __shared__ int ok;
        if (threadIdx.x == 0)
        {
            ok = 1;
            for (int q = 0; q < a.njobs && ok; ++q)
                ok = bounded_wait_epoch(a.jobs[q].flag, a.epoch, a.budget_ns) ? 1 : 0;
        }
        __syncthreads();
        if (!ok)
        {
            if (threadIdx.x == 0)
                atomicExch(a.status, (int) DCB_PEER_TIMEOUT);
            return;
        }
    }
    // a warp per row: consecutive lanes move consecutive cells
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = SHF_THREADS / 32;
    for (long long u = (long long) blockIdx.x * wpb + warp; u < a.total_rows; u += (long long) gridDim.x * wpb)
    {
        long long r = u;
        int q = 0;
        while (r >= a.jobs[q].rows)
        {
            r -= a.jobs[q].rows;
            ++q;
        }
        const ShfJob& j = a.jobs[q];
        long long ao, bo;
        shf_locate(j, r, &ao, &bo);
        float* t = a.tensor + ao;
        float* w = (PUT ? j.peer + a.parity * j.parity_pitch : a.window) + bo;
        const float* from = PUT ? t : w;
        float* to = PUT ? w : t;
        if ((j.len & 3) == 0 && ((reinterpret_cast<uintptr_t>(from) | reinterpret_cast<uintptr_t>(to)) & 15) == 0)
        {
            // 16-byte accesses where the run allows them
            const float4* f4 = reinterpret_cast<const float4*>(from);
            float4* t4 = reinterpret_cast<float4*>(to);
            for (long long e = lane; e < j.len / 4; e += 32)
                t4[e] = f4[e];
        }
        else
        {
            for (long long e = lane; e < j.len; e += 32)
                to[e] = from[e];
        }
    }
    if (PUT)
    {
        // every thread makes its peer stores visible system-wide, then the last
        // block to arrive release-stores the epoch at every destination
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0)
        {
            const unsigned prev = atomicAdd(a.ticket, 1u);
            if (prev == gridDim.x - 1)
            {
                __threadfence_system();
                *a.ticket = 0;
                for (int q = 0; q < a.njobs; ++q)
                    st_release_sys(a.jobs[q].flag, a.epoch);
            }
        }
    }
}

struct ShfBlob
{
    WindowBlob win;
    uint32_t rank;
    uint32_t reserved;
    uint64_t parity_floats;
};
static_assert(sizeof(ShfBlob) <= DCB_SHUFFLE_BLOB_BYTES, "blob too large");

struct Box
{
    long long off[DCB_MAX_DIMS], ext[DCB_MAX_DIMS];
    long long volume() const
    {
        long long v = 1;
        for (int i = 0; i < DCB_MAX_DIMS; ++i)
            v *= ext[i];
        return v;
    }
};

Box to_box(const dcb_box& b, int nd)
{
    Box r;
    for (int i = 0; i < DCB_MAX_DIMS; ++i)
    {
        r.off[i] = i < nd ? b.off[i] : 0;
        r.ext[i] = i < nd ? b.ext[i] : 1;
    }
    return r;
}

bool intersect(const Box& a, const Box& b, Box* out)
{
    for (int i = 0; i < DCB_MAX_DIMS; ++i)
    {
        const long long lo = a.off[i] > b.off[i] ? a.off[i] : b.off[i];
        const long long ha = a.off[i] + a.ext[i], hb = b.off[i] + b.ext[i];
        const long long hi = ha < hb ? ha : hb;
        if (hi <= lo)
            return false;
        out->off[i] = lo;
        out->ext[i] = hi - lo;
    }
    return true;
}

} // namespace
} // namespace dcb

using namespace dcb;

struct dcb_shuffle_plan
{
    int nd, rank, nranks;
    dcb_tensor_desc src, dst;
    std::vector<Box> src_boxes, dst_boxes;
    Window win;
    long long parity_floats;
    std::vector<PeerMapping> peer_map; // by rank; only the destinations of my cells are opened
    ShfJob* d_put = nullptr;
    ShfJob* d_wait = nullptr;
    int n_put = 0, n_wait = 0;
    long long put_rows = 0, wait_rows = 0;
    uint32_t epoch = 0;
    bool connected = false;

    uint32_t* flags() { return reinterpret_cast<uint32_t*>(win.base); }
    uint32_t* ticket() { return flags() + SHF_MAX_RANKS; }
    int* status() { return reinterpret_cast<int*>(flags() + SHF_MAX_RANKS + 1); }
    float* window() { return reinterpret_cast<float*>(static_cast<char*>(win.base) + SHF_HEADER); }
};

namespace
{
int32_t check_shard(const dcb_tensor_desc* d, const Box& mine, int nd)
{
    DCB_REQUIRE(d->ndims == nd && d->dtype == DCB_F32, "descriptor rank / type");
    const long long vol = mine.volume();
    for (int i = 0; i < nd; ++i)
    {
        DCB_REQUIRE(d->real_shape[i] == d->local_shape[i] + 2ll * d->overlap[i], "real shape != local + 2 * overlap");
        // a rank that is not the root of a replicated dimension passes an empty box
        DCB_REQUIRE(vol == 0 || mine.ext[i] == d->local_shape[i], "this rank's box does not match its shard");
    }
    DCB_REQUIRE(d->pitch == 0 || d->pitch >= d->real_shape[0], "row pitch shorter than a row");
    return DCB_OK;
}

// element strides of the halo-extended shard, dimension 0 fastest
void real_strides(const dcb_tensor_desc& d, long long* s)
{
    long long acc = 1;
    for (int i = 0; i < DCB_MAX_DIMS; ++i)
    {
        s[i] = acc;
        acc *= i < d.ndims ? (i == 0 ? row_pitch(d) : d.real_shape[i]) : 1;
    }
}
} // namespace

extern "C" {

int32_t dcb_shuffle_plan_create(const dcb_tensor_desc* src, const dcb_tensor_desc* dst, const dcb_box* src_boxes,
                                const dcb_box* dst_boxes, int32_t rank, int32_t nranks, dcb_shuffle_plan** out)
{
    DCB_REQUIRE(src && dst && src_boxes && dst_boxes && out, "null argument");
    DCB_REQUIRE(nranks >= 1 && nranks <= SHF_MAX_RANKS && rank >= 0 && rank < nranks, "rank / nranks out of range");
    DCB_REQUIRE(src->ndims == dst->ndims && (src->ndims == 4 || src->ndims == 5), "ndims must be 4 or 5");
    const int nd = src->ndims;
    auto* p = new dcb_shuffle_plan();
    p->nd = nd;
    p->rank = rank;
    p->nranks = nranks;
    p->src = *src;
    p->dst = *dst;
    for (int r = 0; r < nranks; ++r)
    {
        p->src_boxes.push_back(to_box(src_boxes[r], nd));
        p->dst_boxes.push_back(to_box(dst_boxes[r], nd));
        for (int i = 0; i < nd; ++i)
            if (src_boxes[r].ext[i] < 0 || dst_boxes[r].ext[i] < 0 || src_boxes[r].off[i] < 0 || dst_boxes[r].off[i] < 0)
            {
                delete p;
                set_last_error("bad argument: negative box");
                return DCB_BAD_ARG;
            }
    }
    int32_t st = check_shard(src, p->src_boxes[rank], nd);
    if (st == DCB_OK)
        st = check_shard(dst, p->dst_boxes[rank], nd);
    if (st != DCB_OK)
    {
        delete p;
        return st;
    }
    // the window holds my destination block twice; a multiple of 4 floats so that
    // both parities start 16-byte aligned
    p->parity_floats = (p->dst_boxes[rank].volume() + 3) / 4 * 4;
    st = p->win.allocate(SHF_HEADER + (size_t) p->parity_floats * 2 * sizeof(float));
    if (st != DCB_OK)
    {
        delete p;
        return st;
    }
    p->peer_map.resize((size_t) nranks);
    *out = p;
    return DCB_OK;
}

int32_t dcb_shuffle_plan_destroy(dcb_shuffle_plan* p)
{
    if (!p)
        return DCB_OK;
    for (auto& m : p->peer_map)
        m.close();
    cudaFree(p->d_put);
    cudaFree(p->d_wait);
    p->win.release();
    delete p;
    return DCB_OK;
}

int32_t dcb_shuffle_plan_export(dcb_shuffle_plan* p, void* blob)
{
    DCB_REQUIRE(p && blob, "null argument");
    ShfBlob b;
    std::memset(&b, 0, sizeof(b));
    p->win.fill_blob(&b.win);
    b.rank = (uint32_t) p->rank;
    b.parity_floats = (uint64_t) p->parity_floats;
    std::memset(blob, 0, DCB_SHUFFLE_BLOB_BYTES);
    std::memcpy(blob, &b, sizeof(b));
    return DCB_OK;
}

int32_t dcb_shuffle_plan_connect(dcb_shuffle_plan* p, const void* blobs, int32_t nranks)
{
    DCB_REQUIRE(p && blobs, "null argument");
    DCB_REQUIRE(nranks == p->nranks, "blob count does not match the plan");
    const int nd = p->nd;
    long long ss[DCB_MAX_DIMS], ds[DCB_MAX_DIMS];
    real_strides(p->src, ss);
    real_strides(p->dst, ds);
    const Box& my_src = p->src_boxes[p->rank];
    const Box& my_dst = p->dst_boxes[p->rank];
    std::vector<ShfJob> put, wait;
    p->put_rows = p->wait_rows = 0;
    for (int r = 0; r < nranks; ++r)
    {
        Box x;
        // what I hold of rank r's destination block
        if (my_src.volume() > 0 && p->dst_boxes[r].volume() > 0 && intersect(my_src, p->dst_boxes[r], &x))
        {
            ShfBlob b;
            std::memcpy(&b, static_cast<const char*>(blobs) + (size_t) r * DCB_SHUFFLE_BLOB_BYTES, sizeof(b));
            DCB_REQUIRE((int) b.rank == r, "blob order does not match ranks");
            char* base = nullptr;
            if (r == p->rank)
                base = static_cast<char*>(p->win.base);
            else
            {
                const int32_t st = p->peer_map[r].open(b.win, p->win.device);
                if (st != DCB_OK)
                    return st;
                base = static_cast<char*>(p->peer_map[r].base);
            }
            DCB_REQUIRE((long long) b.parity_floats == (p->dst_boxes[r].volume() + 3) / 4 * 4,
                        "peer window does not match its destination block");
            ShfJob j;
            std::memset(&j, 0, sizeof(j));
            j.len = x.ext[0];
            j.rows = 1;
            j.a_off = j.b_off = 0;
            long long dense = 1; // strides of r's dense window
            for (int i = 0; i < DCB_MAX_DIMS; ++i)
            {
                const long long a_i = x.off[i] - my_src.off[i] + (i < nd ? p->src.overlap[i] : 0);
                const long long b_i = x.off[i] - p->dst_boxes[r].off[i];
                j.a_off += a_i * ss[i];
                j.b_off += b_i * dense;
                if (i >= 1)
                {
                    j.ext[i - 1] = x.ext[i];
                    j.a_stride[i - 1] = ss[i];
                    j.b_stride[i - 1] = dense;
                    j.rows *= x.ext[i];
                }
                dense *= p->dst_boxes[r].ext[i];
            }
            j.peer = reinterpret_cast<float*>(base + SHF_HEADER);
            j.parity_pitch = (long long) b.parity_floats;
            j.flag = reinterpret_cast<uint32_t*>(base) + p->rank; // my slot among r's flags
            put.push_back(j);
            p->put_rows += j.rows;
        }
        // what rank r holds of my destination block
        if (my_dst.volume() > 0 && p->src_boxes[r].volume() > 0 && intersect(p->src_boxes[r], my_dst, &x))
        {
            ShfJob j;
            std::memset(&j, 0, sizeof(j));
            j.len = x.ext[0];
            j.rows = 1;
            long long dense = 1;
            for (int i = 0; i < DCB_MAX_DIMS; ++i)
            {
                const long long a_i = x.off[i] - my_dst.off[i] + (i < nd ? p->dst.overlap[i] : 0);
                const long long b_i = x.off[i] - my_dst.off[i];
                j.a_off += a_i * ds[i];
                j.b_off += b_i * dense;
                if (i >= 1)
                {
                    j.ext[i - 1] = x.ext[i];
                    j.a_stride[i - 1] = ds[i];
                    j.b_stride[i - 1] = dense;
                    j.rows *= x.ext[i];
                }
                dense *= my_dst.ext[i];
            }
            j.peer = nullptr;
            j.flag = p->flags() + r;
            wait.push_back(j);
            p->wait_rows += j.rows;
        }
    }
    cudaFree(p->d_put);
    cudaFree(p->d_wait);
    p->d_put = p->d_wait = nullptr;
    p->n_put = (int) put.size();
    p->n_wait = (int) wait.size();
    if (p->n_put)
    {
        DCB_CUDA_TRY(cudaMalloc(&p->d_put, put.size() * sizeof(ShfJob)));
        DCB_CUDA_TRY(cudaMemcpy(p->d_put, put.data(), put.size() * sizeof(ShfJob), cudaMemcpyHostToDevice));
    }
    if (p->n_wait)
    {
        DCB_CUDA_TRY(cudaMalloc(&p->d_wait, wait.size() * sizeof(ShfJob)));
        DCB_CUDA_TRY(cudaMemcpy(p->d_wait, wait.data(), wait.size() * sizeof(ShfJob), cudaMemcpyHostToDevice));
    }
    p->connected = true;
    return DCB_OK;
}

static unsigned shf_grid(long long rows)
{
    const long long want = (rows + SHF_THREADS / 32 - 1) / (SHF_THREADS / 32);
    const long long cap = (long long) num_sms() * 8;
    return (unsigned) (want < 1 ? 1 : (want > cap ? cap : want));
}

int32_t dcb_shuffle_put(dcb_shuffle_plan* p, const void* src, void* stream)
{
    DCB_REQUIRE(p, "null plan");
    if (!p->connected)
    {
        set_last_error("shuffle plan is not connected");
        return DCB_NOT_CONNECTED;
    }
    ++p->epoch;
    if (p->n_put == 0)
        return DCB_OK;
    DCB_REQUIRE(src, "null tensor");
    ShfArgs a;
    std::memset(&a, 0, sizeof(a));
    a.jobs = p->d_put;
    a.njobs = p->n_put;
    a.total_rows = p->put_rows;
    a.tensor = const_cast<float*>(static_cast<const float*>(src));
    a.parity = (int) (p->epoch & 1u);
    a.epoch = p->epoch;
    a.ticket = p->ticket();
    a.status = p->status();
    a.budget_ns = wait_budget_ns();
    shuffle_kernel<true><<<shf_grid(p->put_rows), SHF_THREADS, 0, as_stream(stream)>>>(a);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_shuffle_wait_unpack(dcb_shuffle_plan* p, void* dst, void* stream)
{
    DCB_REQUIRE(p, "null plan");
    if (!p->connected)
    {
        set_last_error("shuffle plan is not connected");
        return DCB_NOT_CONNECTED;
    }
    if (p->n_wait == 0)
        return DCB_OK;
    DCB_REQUIRE(dst, "null tensor");
    ShfArgs a;
    std::memset(&a, 0, sizeof(a));
    a.jobs = p->d_wait;
    a.njobs = p->n_wait;
    a.total_rows = p->wait_rows;
    a.tensor = static_cast<float*>(dst);
    a.window = p->window() + (long long) (p->epoch & 1u) * p->parity_floats;
    a.epoch = p->epoch;
    a.ticket = p->ticket();
    a.status = p->status();
    a.budget_ns = wait_budget_ns();
    shuffle_kernel<false><<<shf_grid(p->wait_rows), SHF_THREADS, 0, as_stream(stream)>>>(a);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_shuffle(dcb_shuffle_plan* p, const void* src, void* dst, void* stream)
{
    const int32_t st = dcb_shuffle_put(p, src, stream);
    if (st != DCB_OK)
        return st;
    return dcb_shuffle_wait_unpack(p, dst, stream);
}

int32_t dcb_shuffle_plan_status(dcb_shuffle_plan* p, void* stream)
{
    DCB_REQUIRE(p, "null plan");
    DCB_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    int st = 0;
    DCB_CUDA_TRY(cudaMemcpy(&st, p->status(), sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0)
    {
        const int zero = 0;
        DCB_CUDA_TRY(cudaMemcpy(p->status(), &zero, sizeof(int), cudaMemcpyHostToDevice));
    }
    return st;
}

} // extern "C"
