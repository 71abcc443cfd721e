// Halo slab kernels and the peer-store transport.
//
// A face slab of a halo-extended NC[D]HW shard is, for every dimension, a set
// of R equally spaced contiguous runs: for dimension d with `below` = product
// of the real extents of the dimensions inside d,
//     run length  L  = width * below
//     run stride  S  = real_extent_d * below
//     first run   s0 = start_d * below
//     runs        R  = product of the real extents of the dimensions outside d
// so D faces are a few long runs (whole planes), H faces are rows of planes and
// W faces are `width` elements per row.  One kernel family covers all of them:
// long runs are split into chunks that a block copies with 4-, 2- or 1-wide
// vector accesses; short runs are walked with a flat index.
//
// Pack writes the packed slab straight into the neighbour's receive slab
// (peer-mapped, so the stores cross NVLink) and the last block to finish
// release-stores the exchange epoch into the neighbour's flag.  Unpack polls
// its own flag with a bounded budget, then scatters the slab into the halo
// cells, optionally accumulating (ID / SUM / MAX / MIN).
#include "common.cuh"

namespace dcb
{

enum : int
{
    MODE_PACK = 0,
    MODE_UNPACK = 1,
    MODE_CLEAR = 2
};

struct SideJob
{
    float* tensor;
    float* packed;
    long long runs;   // R
    long long len_v;  // L / V
    long long stride; // S, in scalar elements
    long long start;  // s0, in scalar elements
    uint32_t* flag;   // pack: peer flag to publish; unpack: own flag to wait on
    uint32_t* ticket; // pack: local arrival counter
    uint32_t epoch;
    uint32_t active;
};

struct HaloArgs
{
    SideJob side[4]; // [0], [1]: the two sides; [2], [3]: halo slabs a pack launch also clears
    int op;
    long long budget_ns;
    int* status;
};

template <int V>
struct VecOf;
template <>
struct VecOf<1>
{
    using type = float;
};
template <>
struct VecOf<2>
{
    using type = float2;
};
template <>
struct VecOf<4>
{
    using type = float4;
};

__device__ __forceinline__ float accum1(float dst, float src, int op)
{
    switch (op)
    {
    case 1: return dst + src;
    case 2: return fmaxf(dst, src);
    case 3: return fminf(dst, src);
    default: return src;
    }
}
__device__ __forceinline__ float accum(float d, float s, int op)
{
    return accum1(d, s, op);
}
__device__ __forceinline__ float2 accum(float2 d, float2 s, int op)
{
    return make_float2(accum1(d.x, s.x, op), accum1(d.y, s.y, op));
}
__device__ __forceinline__ float4 accum(float4 d, float4 s, int op)
{
    return make_float4(accum1(d.x, s.x, op), accum1(d.y, s.y, op),
                       accum1(d.z, s.z, op), accum1(d.w, s.w, op));
}
template <typename T>
__device__ __forceinline__ T zero_of();
template <>
__device__ __forceinline__ float zero_of<float>()
{
    return 0.f;
}
template <>
__device__ __forceinline__ float2 zero_of<float2>()
{
    return make_float2(0.f, 0.f);
}
template <>
__device__ __forceinline__ float4 zero_of<float4>()
{
    return make_float4(0.f, 0.f, 0.f, 0.f);
}

constexpr int HALO_THREADS = 256;
constexpr int HALO_UNROLL = 4;
constexpr int HALO_CHUNK = HALO_THREADS * HALO_UNROLL; // vector elements

template <int V, int MODE>
__device__ __forceinline__ void
move_one(typename VecOf<V>::type* __restrict__ t,
         typename VecOf<V>::type* __restrict__ p, int op)
{
    using T = typename VecOf<V>::type;
    if (MODE == MODE_PACK)
        *p = *t;
    else if (MODE == MODE_UNPACK)
        *t = (op == 0) ? *p : accum(*t, *p, op);
    else
        *t = zero_of<T>();
}

// LONG = runs are split into chunks of HALO_CHUNK vector elements;
// otherwise a flat index over runs*len_v is decoded by division.
template <int V, int MODE, bool LONG>
__global__ void __launch_bounds__(HALO_THREADS) halo_kernel(HaloArgs a)
{
    using T = typename VecOf<V>::type;
    const SideJob& j = a.side[blockIdx.y];
    if (!j.active)
        return;
    if (MODE == MODE_PACK && blockIdx.y >= 2)
    {
        // a halo slab without a neighbour behind it (the boundary of the global
        // tensor): zeroed by the launch that packs this dimension, which saves
        // the separate clear_halo launch (Tensor::clear_halo before every
        // exchange, convolution.hpp:405-414)
        const long long total = j.runs * j.len_v;
        for (long long i = (long long) blockIdx.x * HALO_THREADS + threadIdx.x; i < total;
             i += (long long) gridDim.x * HALO_THREADS)
        {
            const long long r = i / j.len_v;
            reinterpret_cast<T*>(j.tensor + j.start + r * j.stride)[i - r * j.len_v] = zero_of<T>();
        }
        return;
    }

    if (MODE == MODE_UNPACK && j.flag != nullptr)
    {
        __shared__ int ok;
        if (threadIdx.x == 0)
            ok = bounded_wait_epoch(j.flag, j.epoch, a.budget_ns) ? 1 : 0;
        __syncthreads();
        if (!ok)
        {
            if (threadIdx.x == 0)
                atomicExch(a.status, (int) DCB_PEER_TIMEOUT);
            return;
        }
    }

    if (LONG)
    {
        const long long cpr = (j.len_v + HALO_CHUNK - 1) / HALO_CHUNK;
        const long long units = j.runs * cpr;
        for (long long u = blockIdx.x; u < units; u += gridDim.x)
        {
            const long long r = u / cpr;
            const long long c0 = (u - r * cpr) * HALO_CHUNK;
            T* t = reinterpret_cast<T*>(j.tensor + j.start + r * j.stride) + c0;
            T* p = reinterpret_cast<T*>(j.packed) + r * j.len_v + c0;
            const long long rem = j.len_v - c0;
            if (rem >= HALO_CHUNK && MODE != MODE_CLEAR)
            {
                // Full chunk: issue all loads before the stores.
                T v[HALO_UNROLL];
                T w[HALO_UNROLL];
#pragma unroll
                for (int k = 0; k < HALO_UNROLL; ++k)
                {
                    const int e = threadIdx.x + k * HALO_THREADS;
                    if (MODE == MODE_PACK)
                        v[k] = t[e];
                    else
                    {
                        v[k] = p[e];
                        if (a.op != 0)
                            w[k] = t[e];
                    }
                }
#pragma unroll
                for (int k = 0; k < HALO_UNROLL; ++k)
                {
                    const int e = threadIdx.x + k * HALO_THREADS;
                    if (MODE == MODE_PACK)
                        p[e] = v[k];
                    else
                        t[e] = (a.op == 0) ? v[k] : accum(w[k], v[k], a.op);
                }
            }
            else
            {
                for (long long e = threadIdx.x; e < rem && e < HALO_CHUNK;
                     e += HALO_THREADS)
                    move_one<V, MODE>(t + e, p + e, a.op);
            }
        }
    }
    else
    {
        const long long total = j.runs * j.len_v;
        const long long step = (long long) gridDim.x * HALO_THREADS;
        for (long long i = (long long) blockIdx.x * HALO_THREADS + threadIdx.x;
             i < total; i += step)
        {
            const long long r = i / j.len_v;
            const long long e = i - r * j.len_v;
            T* t = reinterpret_cast<T*>(j.tensor + j.start + r * j.stride) + e;
            T* p = reinterpret_cast<T*>(j.packed) + i;
            move_one<V, MODE>(t, p, a.op);
        }
    }

    if (MODE == MODE_PACK && j.flag != nullptr)
    {
        // Publish: every thread makes its peer stores visible system-wide,
        // then the last block to arrive release-stores the epoch.
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0)
        {
            const unsigned prev = atomicAdd(j.ticket, 1u);
            if (prev == gridDim.x - 1)
            {
                __threadfence_system();
                *j.ticket = 0;
                st_release_sys(j.flag, j.epoch);
            }
        }
    }
}

struct SlabGeom
{
    long long runs, len, stride, start;
};

static bool slab_geom(const dcb_tensor_desc& d, int dim, int side, int width,
                      bool inner, SlabGeom* g)
{
    if (dim < 0 || dim >= d.ndims || width <= 0)
        return false;
    // Rows may be padded (desc.pitch): a W face is then `width` cells per row at
    // stride pitch; H and D faces are whole rows and planes, the padding cells
    // between rows included (nobody reads them) but not those after the last
    // row: the shard may start a few floats into its allocation (owned cells on
    // a 16-byte boundary), and then its last row's padding ends beyond it.
    const long long pitch = row_pitch(d);
    long long below = 1, above = 1;
    for (int e = 0; e < dim; ++e)
        below *= e == 0 ? pitch : d.real_shape[e];
    for (int e = dim + 1; e < d.ndims; ++e)
        above *= d.real_shape[e];
    const long long n = d.real_shape[dim];
    long long start;
    // Same cell selection as the reference traversal (halo_cuda.hpp:34-88).
    if (side == DCB_RHS)
        start = inner ? n - 2ll * width : n - width;
    else
        start = inner ? width : 0;
    if (start < 0 || start + width > n)
        return false;
    g->runs = above;
    g->len = (long long) width * below - (dim > 0 ? pitch - d.real_shape[0] : 0);
    g->stride = (dim == 0 ? pitch : n) * below;
    g->start = start * below;
    return true;
}

static int pick_vec(const SlabGeom& g, const void* tensor, const void* packed)
{
    auto ok = [&](int v) {
        return g.len % v == 0 && g.stride % v == 0 && g.start % v == 0
               && reinterpret_cast<uintptr_t>(tensor) % (4 * v) == 0
               && (packed == nullptr
                   || reinterpret_cast<uintptr_t>(packed) % (4 * v) == 0);
    };
    if (ok(4))
        return 4;
    if (ok(2))
        return 2;
    return 1;
}

template <int MODE>
static int32_t launch_halo(HaloArgs& a, int vec, const SlabGeom* geoms,
                           cudaStream_t stream)
{
    long long max_units = 0;
    bool is_long = true;
    for (int s = 0; s < 2; ++s)
    {
        if (!a.side[s].active)
            continue;
        a.side[s].len_v = geoms[s].len / vec;
        if (a.side[s].len_v < 64)
            is_long = false;
    }
    const bool with_clear = MODE == MODE_PACK && (a.side[2].active || a.side[3].active);
    for (int s = 2; s < 4; ++s)
        if (a.side[s].active)
            a.side[s].len_v = a.side[s].len_v / vec; // set in scalar elements by the caller
    for (int s = 0; s < 2; ++s)
    {
        if (!a.side[s].active)
            continue;
        long long units;
        if (is_long)
            units = a.side[s].runs
                    * ((a.side[s].len_v + HALO_CHUNK - 1) / HALO_CHUNK);
        else
            units = (a.side[s].runs * a.side[s].len_v + HALO_CHUNK - 1)
                    / HALO_CHUNK;
        max_units = units > max_units ? units : max_units;
    }
    if (max_units == 0)
        return DCB_OK;
    const long long cap = (long long) num_sms() * 8;
    dim3 grid((unsigned) (max_units < cap ? max_units : cap), with_clear ? 4 : 2);
#define DCB_HALO_CASE(VV)                                                      \
    if (is_long)                                                               \
        halo_kernel<VV, MODE, true><<<grid, HALO_THREADS, 0, stream>>>(a);     \
    else                                                                       \
        halo_kernel<VV, MODE, false><<<grid, HALO_THREADS, 0, stream>>>(a);
    if (vec == 4)
    {
        DCB_HALO_CASE(4)
    }
    else if (vec == 2)
    {
        DCB_HALO_CASE(2)
    }
    else
    {
        DCB_HALO_CASE(1)
    }
#undef DCB_HALO_CASE
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

static int32_t check_desc(const dcb_tensor_desc* d)
{
    DCB_REQUIRE(d != nullptr, "null tensor descriptor");
    DCB_REQUIRE(d->ndims == 4 || d->ndims == 5, "ndims must be 4 or 5");
    DCB_REQUIRE(d->dtype == DCB_F32, "only fp32 tensors");
    for (int i = 0; i < d->ndims; ++i)
    {
        DCB_REQUIRE(d->local_shape[i] >= 0, "negative extent");
        DCB_REQUIRE(d->overlap[i] >= 0, "negative overlap");
        DCB_REQUIRE(d->real_shape[i] == d->local_shape[i] + 2ll * d->overlap[i],
                    "real_shape must be local_shape + 2*overlap");
        if (i >= d->ndims - 2)
            DCB_REQUIRE(d->overlap[i] == 0, "no overlap on C and N");
    }
    DCB_REQUIRE(d->pitch == 0 || d->pitch >= d->real_shape[0], "row pitch shorter than a row");
    return DCB_OK;
}

} // namespace dcb

using namespace dcb;

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
namespace
{
constexpr int kFlagWords = 16;
constexpr size_t kHeaderBytes = 256; // flags, tickets, status

struct HaloBlob
{
    WindowBlob win;
    uint32_t rank;
    uint32_t reserved;
    uint64_t slab_off[2][DCB_MAX_SPATIAL][2];
};
static_assert(sizeof(HaloBlob) <= DCB_HALO_BLOB_BYTES, "blob too large");
} // namespace

struct dcb_halo_plan
{
    dcb_tensor_desc desc;
    int nsd;
    int rank;
    int peers[DCB_MAX_SPATIAL][2];
    Window win;
    uint64_t slab_off[2][DCB_MAX_SPATIAL][2];
    uint32_t epoch[DCB_MAX_SPATIAL];
    PeerMapping peer_map[DCB_MAX_SPATIAL][2];
    uint64_t peer_slab_off[2][DCB_MAX_SPATIAL][2]; // [parity][dim][my side]
    bool connected;

    uint32_t* flags() { return reinterpret_cast<uint32_t*>(win.base); }
    uint32_t* tickets() { return flags() + kFlagWords; }
    int* status() { return reinterpret_cast<int*>(flags() + 2 * kFlagWords); }
    bool dim_active(int dim) const
    {
        return desc.overlap[dim] > 0
               && (peers[dim][0] >= 0 || peers[dim][1] >= 0);
    }
};

extern "C" {

int32_t dcb_halo_plan_create(const dcb_tensor_desc* desc, const int32_t* peers,
                             int32_t rank, dcb_halo_plan** out)
{
    int32_t st = check_desc(desc);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(peers != nullptr && out != nullptr, "null argument");
    auto* p = new dcb_halo_plan();
    p->desc = *desc;
    p->nsd = desc->ndims - 2;
    p->rank = rank;
    p->connected = false;
    size_t off = kHeaderBytes;
    long long local_size = 1;
    for (int i = 0; i < desc->ndims; ++i)
        local_size *= desc->local_shape[i];
    for (int d = 0; d < DCB_MAX_SPATIAL; ++d)
    {
        p->epoch[d] = 0;
        for (int s = 0; s < 2; ++s)
        {
            // An empty shard exchanges nothing (halo_exchange_cuda.hpp:327-330).
            p->peers[d][s] =
                (d < p->nsd && local_size > 0 && desc->overlap[d] > 0)
                    ? peers[2 * d + s]
                    : -1;
        }
    }
    for (int par = 0; par < 2; ++par)
        for (int d = 0; d < p->nsd; ++d)
            for (int s = 0; s < 2; ++s)
            {
                // 0 marks a side without a neighbour: no slab, and a peer that
                // tries to connect to it is refused
                p->slab_off[par][d][s] = p->peers[d][s] < 0 ? 0 : off;
                if (p->peers[d][s] < 0)
                    continue;
                SlabGeom g;
                if (!slab_geom(*desc, d, s, desc->overlap[d], false, &g))
                {
                    delete p;
                    set_last_error("shard narrower than its halo");
                    return DCB_BAD_ARG;
                }
                size_t bytes = (size_t) g.runs * g.len * sizeof(float);
                off += (bytes + 255) / 256 * 256;
            }
    st = p->win.allocate(off);
    if (st != DCB_OK)
    {
        delete p;
        return st;
    }
    *out = p;
    return DCB_OK;
}

int32_t dcb_halo_plan_destroy(dcb_halo_plan* p)
{
    if (!p)
        return DCB_OK;
    for (int d = 0; d < DCB_MAX_SPATIAL; ++d)
        for (int s = 0; s < 2; ++s)
            p->peer_map[d][s].close();
    p->win.release();
    delete p;
    return DCB_OK;
}

int32_t dcb_halo_plan_export(dcb_halo_plan* p, void* blob)
{
    DCB_REQUIRE(p && blob, "null argument");
    HaloBlob b;
    std::memset(&b, 0, sizeof(b));
    p->win.fill_blob(&b.win);
    b.rank = (uint32_t) p->rank;
    std::memcpy(b.slab_off, p->slab_off, sizeof(b.slab_off));
    std::memset(blob, 0, DCB_HALO_BLOB_BYTES);
    std::memcpy(blob, &b, sizeof(b));
    return DCB_OK;
}

int32_t dcb_halo_plan_connect(dcb_halo_plan* p, const void* blobs,
                              int32_t nranks)
{
    DCB_REQUIRE(p && blobs, "null argument");
    for (int d = 0; d < p->nsd; ++d)
        for (int s = 0; s < 2; ++s)
        {
            const int peer = p->peers[d][s];
            if (peer < 0)
                continue;
            DCB_REQUIRE(peer < nranks, "peer rank out of range");
            HaloBlob b;
            std::memcpy(&b,
                        static_cast<const char*>(blobs)
                            + (size_t) peer * DCB_HALO_BLOB_BYTES,
                        sizeof(b));
            DCB_REQUIRE((int) b.rank == peer, "blob order does not match ranks");
            // What I will store must fit into the slab the peer set aside for
            // its opposite side: a peer that sees no neighbour there (an empty
            // shard, an inconsistent peers[] table) reserved nothing, and the
            // stores would leave its window.
            SlabGeom sg;
            DCB_REQUIRE(slab_geom(p->desc, d, s, p->desc.overlap[d], false, &sg), "shard narrower than its halo");
            const uint64_t need = (uint64_t) sg.runs * (uint64_t) sg.len * sizeof(float);
            for (int par = 0; par < 2; ++par)
            {
                const uint64_t off = b.slab_off[par][d][1 - s];
                uint64_t next = b.win.bytes;
                for (int par2 = 0; par2 < 2; ++par2)
                    for (int d2 = 0; d2 < DCB_MAX_SPATIAL; ++d2)
                        for (int s2 = 0; s2 < 2; ++s2)
                            if (b.slab_off[par2][d2][s2] > off && b.slab_off[par2][d2][s2] < next)
                                next = b.slab_off[par2][d2][s2];
                DCB_REQUIRE(off >= kHeaderBytes && off + need <= next,
                            "the peer's receive slab does not match this rank's face");
            }
            int32_t st = p->peer_map[d][s].open(b.win, p->win.device);
            if (st != DCB_OK)
                return st;
            // I write into the slab the peer keeps for its opposite side.
            for (int par = 0; par < 2; ++par)
                p->peer_slab_off[par][d][s] = b.slab_off[par][d][1 - s];
        }
    p->connected = true;
    return DCB_OK;
}

int32_t dcb_halo_pack_put(dcb_halo_plan* p, const void* tensor, int32_t dim,
                          uint32_t flags, void* stream)
{
    DCB_REQUIRE(p && tensor, "null argument");
    DCB_REQUIRE(dim >= 0 && dim < p->nsd, "dimension out of range");
    if (!p->dim_active(dim))
    {
        // nobody to exchange with: only the clearing is left to do
        if ((flags & DCB_HALO_CLEAR_BOUNDARY) && !(flags & DCB_HALO_REVERSE) && p->desc.overlap[dim] > 0)
            return dcb_clear_halo(&p->desc, const_cast<void*>(tensor), dim, stream);
        return DCB_OK;
    }
    if (!p->connected)
    {
        set_last_error("halo plan has peers but was never connected");
        return DCB_NOT_CONNECTED;
    }
    const bool reverse = flags & DCB_HALO_REVERSE;
    const uint32_t epoch = ++p->epoch[dim];
    const int par = epoch & 1;
    const int width = p->desc.overlap[dim];
    HaloArgs a;
    std::memset(&a, 0, sizeof(a));
    a.budget_ns = wait_budget_ns();
    a.status = p->status();
    SlabGeom geoms[2];
    int vec = 4;
    for (int s = 0; s < 2; ++s)
    {
        if (p->peers[dim][s] < 0)
            continue;
        if (!slab_geom(p->desc, dim, s, width, !reverse, &geoms[s]))
        {
            set_last_error("shard narrower than its halo");
            return DCB_BAD_ARG;
        }
        char* peer_base = static_cast<char*>(p->peer_map[dim][s].base);
        SideJob& j = a.side[s];
        j.tensor = const_cast<float*>(static_cast<const float*>(tensor));
        j.packed =
            reinterpret_cast<float*>(peer_base + p->peer_slab_off[par][dim][s]);
        j.runs = geoms[s].runs;
        j.stride = geoms[s].stride;
        j.start = geoms[s].start;
        j.flag = reinterpret_cast<uint32_t*>(peer_base) + (2 * dim + (1 - s));
        j.ticket = p->tickets() + (2 * dim + s);
        j.epoch = epoch;
        j.active = 1;
        const int v = pick_vec(geoms[s], tensor, j.packed);
        vec = v < vec ? v : vec;
    }
    if ((flags & DCB_HALO_CLEAR_BOUNDARY) && !reverse)
    {
        // the halo slabs of this dimension that no neighbour will fill
        for (int s = 0; s < 2; ++s)
        {
            if (p->peers[dim][s] >= 0)
                continue;
            SlabGeom cg;
            if (!slab_geom(p->desc, dim, s, width, false, &cg))
                continue;
            SideJob& j = a.side[2 + s];
            j.tensor = const_cast<float*>(static_cast<const float*>(tensor));
            j.runs = cg.runs;
            j.stride = cg.stride;
            j.start = cg.start;
            j.len_v = cg.len; // scalar elements; launch_halo divides by the vector width
            j.active = cg.runs * cg.len > 0;
            const int v = pick_vec(cg, tensor, nullptr);
            vec = v < vec ? v : vec;
        }
    }
    return launch_halo<MODE_PACK>(a, vec, geoms, as_stream(stream));
}

int32_t dcb_halo_wait_unpack(dcb_halo_plan* p, void* tensor, int32_t dim,
                             uint32_t flags, void* stream)
{
    DCB_REQUIRE(p && tensor, "null argument");
    DCB_REQUIRE(dim >= 0 && dim < p->nsd, "dimension out of range");
    if (!p->dim_active(dim))
        return DCB_OK;
    const bool reverse = flags & DCB_HALO_REVERSE;
    const uint32_t epoch = p->epoch[dim];
    const int par = epoch & 1;
    const int width = p->desc.overlap[dim];
    HaloArgs a;
    std::memset(&a, 0, sizeof(a));
    a.budget_ns = wait_budget_ns();
    a.status = p->status();
    a.op = (int) ((flags >> DCB_HALO_OP_SHIFT) & 3u);
    SlabGeom geoms[2];
    int vec = 4;
    for (int s = 0; s < 2; ++s)
    {
        if (p->peers[dim][s] < 0)
            continue;
        if (!slab_geom(p->desc, dim, s, width, reverse, &geoms[s]))
        {
            set_last_error("shard narrower than its halo");
            return DCB_BAD_ARG;
        }
        SideJob& j = a.side[s];
        j.tensor = static_cast<float*>(tensor);
        j.packed = reinterpret_cast<float*>(static_cast<char*>(p->win.base)
                                            + p->slab_off[par][dim][s]);
        j.runs = geoms[s].runs;
        j.stride = geoms[s].stride;
        j.start = geoms[s].start;
        j.flag = p->flags() + (2 * dim + s);
        j.epoch = epoch;
        j.active = 1;
        const int v = pick_vec(geoms[s], tensor, j.packed);
        vec = v < vec ? v : vec;
    }
    // A shard narrower than two halo widths has overlapping inner slabs: the
    // two sides then accumulate into the same cells and must not run
    // concurrently.  Unpack LHS, then RHS.
    if (reverse && p->desc.local_shape[dim] < 2ll * width && a.side[0].active
        && a.side[1].active)
    {
        HaloArgs lhs = a, rhs = a;
        lhs.side[1].active = 0;
        rhs.side[0].active = 0;
        int32_t st = launch_halo<MODE_UNPACK>(lhs, vec, geoms, as_stream(stream));
        if (st != DCB_OK)
            return st;
        return launch_halo<MODE_UNPACK>(rhs, vec, geoms, as_stream(stream));
    }
    return launch_halo<MODE_UNPACK>(a, vec, geoms, as_stream(stream));
}

int32_t dcb_halo_exchange(dcb_halo_plan* p, void* tensor, uint32_t flags,
                          void* stream)
{
    DCB_REQUIRE(p && tensor, "null argument");
    for (int d = 0; d < p->nsd; ++d)
    {
        int32_t st = dcb_halo_pack_put(p, tensor, d, flags, stream);
        if (st != DCB_OK)
            return st;
        if (!(flags & DCB_HALO_SKIP_UNPACK))
        {
            st = dcb_halo_wait_unpack(p, tensor, d, flags, stream);
            if (st != DCB_OK)
                return st;
        }
    }
    return DCB_OK;
}

int32_t dcb_halo_unpack(dcb_halo_plan* p, void* tensor, uint32_t flags,
                        void* stream)
{
    DCB_REQUIRE(p && tensor, "null argument");
    for (int d = 0; d < p->nsd; ++d)
    {
        int32_t st = dcb_halo_wait_unpack(p, tensor, d, flags, stream);
        if (st != DCB_OK)
            return st;
    }
    return DCB_OK;
}

int32_t dcb_halo_plan_status(dcb_halo_plan* p, void* stream)
{
    DCB_REQUIRE(p, "null argument");
    DCB_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    int st = 0;
    DCB_CUDA_TRY(cudaMemcpy(&st, p->status(), sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0)
    {
        DCB_CUDA_TRY(cudaMemset(p->status(), 0, sizeof(int)));
        set_last_error("a wait on a neighbour's halo flag ran out of budget");
        return DCB_PEER_TIMEOUT;
    }
    return DCB_OK;
}

int32_t dcb_clear_halo(const dcb_tensor_desc* desc, void* tensor, int32_t dim,
                       void* stream)
{
    int32_t st = check_desc(desc);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(tensor != nullptr, "null tensor");
    DCB_REQUIRE(dim < desc->ndims, "dimension out of range");
    const int lo = dim < 0 ? 0 : dim, hi = dim < 0 ? desc->ndims - 2 : dim + 1;
    for (int d = lo; d < hi; ++d)
    {
        const int width = desc->overlap[d];
        if (width == 0)
            continue;
        HaloArgs a;
        std::memset(&a, 0, sizeof(a));
        SlabGeom geoms[2];
        int vec = 4;
        for (int s = 0; s < 2; ++s)
        {
            if (!slab_geom(*desc, d, s, width, false, &geoms[s]))
            {
                set_last_error("shard narrower than its halo");
                return DCB_BAD_ARG;
            }
            SideJob& j = a.side[s];
            j.tensor = static_cast<float*>(tensor);
            j.runs = geoms[s].runs;
            j.stride = geoms[s].stride;
            j.start = geoms[s].start;
            j.active = geoms[s].runs * geoms[s].len > 0;
            const int v = pick_vec(geoms[s], tensor, nullptr);
            vec = v < vec ? v : vec;
        }
        st = launch_halo<MODE_CLEAR>(a, vec, geoms, as_stream(stream));
        if (st != DCB_OK)
            return st;
    }
    return DCB_OK;
}

static int32_t pack_or_unpack_slab(const dcb_tensor_desc* desc, void* tensor,
                                   int32_t dim, int32_t side, int32_t width,
                                   int32_t inner, void* packed, uint32_t op,
                                   bool pack, void* stream)
{
    int32_t st = check_desc(desc);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(tensor && packed, "null argument");
    DCB_REQUIRE(side == DCB_LHS || side == DCB_RHS, "side must be 0 or 1");
    DCB_REQUIRE(dim >= 0 && dim < desc->ndims, "dimension out of range");
    DCB_REQUIRE(width <= desc->overlap[dim], "width exceeds the overlap");
    if (width == 0)
        return DCB_OK;
    if (inner)
        DCB_REQUIRE(desc->local_shape[dim] >= width, "shard narrower than width");
    HaloArgs a;
    std::memset(&a, 0, sizeof(a));
    a.op = (int) ((op >> DCB_HALO_OP_SHIFT) & 3u);
    SlabGeom geoms[2];
    // The reference's cell selection is written for width == overlap
    // (halo_cuda.hpp:57-75); a narrower slab is placed next to the shard
    // boundary, which is where the convolution reads it.
    dcb_tensor_desc d = *desc;
    if (!slab_geom(d, dim, side, desc->overlap[dim], inner != 0, &geoms[0]))
        return DCB_BAD_ARG;
    if (width != desc->overlap[dim])
    {
        long long below = 1;
        for (int e = 0; e < dim; ++e)
            below *= e == 0 ? row_pitch(d) : d.real_shape[e];
        const int ov = desc->overlap[dim];
        // Outer slabs hug the owned cells; inner slabs hug the boundary.
        long long shift = 0;
        if (side == DCB_RHS)
            shift = inner ? (ov - width) : 0;
        else
            shift = inner ? 0 : (ov - width);
        geoms[0].start += shift * below;
        geoms[0].len = (long long) width * below;
    }
    geoms[1] = geoms[0];
    SideJob& j = a.side[0];
    j.tensor = static_cast<float*>(tensor);
    j.packed = static_cast<float*>(packed);
    j.runs = geoms[0].runs;
    j.stride = geoms[0].stride;
    j.start = geoms[0].start;
    j.active = 1;
    const int vec = pick_vec(geoms[0], tensor, packed);
    return pack ? launch_halo<MODE_PACK>(a, vec, geoms, as_stream(stream))
                : launch_halo<MODE_UNPACK>(a, vec, geoms, as_stream(stream));
}

int32_t dcb_halo_pack(const dcb_tensor_desc* desc, const void* tensor,
                      int32_t dim, int32_t side, int32_t width, int32_t inner,
                      void* packed, void* stream)
{
    return pack_or_unpack_slab(desc, const_cast<void*>(tensor), dim, side,
                               width, inner, packed, 0, true, stream);
}

int32_t dcb_halo_unpack_slab(const dcb_tensor_desc* desc, void* tensor,
                             int32_t dim, int32_t side, int32_t width,
                             int32_t inner, const void* packed, uint32_t op,
                             void* stream)
{
    return pack_or_unpack_slab(desc, tensor, dim, side, width, inner,
                               const_cast<void*>(packed), op, false, stream);
}

} // extern "C"
