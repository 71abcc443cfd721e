// Batch-normalisation kernels (and LeakyReLU): HBM-bound streaming kernels.
//
// Every (n, c) plane of an NC[D]HW window is a set of contiguous runs (see
// RunGeom).  A "unit" is up to 256 x (8 or 16) vector elements of one run, or,
// where runs are short (the rows of a shard with halo cells along W, whose
// pitch keeps them apart), several consecutive runs; blocks of channel c
// (blockIdx.y) stride over that channel's units with 16-byte vector accesses
// where the strides allow.
//
// Reductions are two-stage and fixed-order: each block writes its fp64 partial
// to scratch, the last block of a channel (ticket) folds the partials in index
// order, so results are reproducible run to run.  fp32 atomics, as the
// reference uses (batchnorm.cu:39-132), are not.
#include <atomic>

#include "common.cuh"

namespace dcb
{

constexpr int BN_THREADS = 256;
// Vector elements a thread has in flight per unit.  The streaming kernels (apply,
// backward apply, LeakyReLU) want many: 16 x 16 bytes per thread measured 0.341 ms
// for the 2 GiB of the bench layer's apply against 0.367 ms with 4; the reductions
// hold accumulators beside the data and are fastest with 8 (0.155 / 0.304 ms against
// 0.168 / 0.328 ms with 16).
constexpr int BN_UNROLL_MAP = 16;
constexpr int BN_UNROLL_RED = 8;

struct UnitGeom
{
    RunGeom g;
    long long upr;   // units per run (1 when runs are packed)
    long long upc;   // units per channel
    int unit;        // scalars per unit = 256 * unroll * vector width
    // Packed short runs: a unit is up to rpu consecutive runs of one outer step,
    // vpr vector elements each.  Unpacked: rpu = 1, vpr = 0, magic = 0.
    int rpu, vpr;
    unsigned magic;  // ceil(2^32 / vpr): e / vpr = umulhi(e, magic) for the e < 4096 used here
    long long gpo;   // units per outer step
};

static UnitGeom make_units(const RunGeom& g, int vec, int unroll)
{
    const int BN_UNIT_VECS = BN_THREADS * unroll; // vector elements per unit
    UnitGeom u;
    u.g = g;
    u.unit = BN_UNIT_VECS * vec;
    u.upr = (g.len + u.unit - 1) / u.unit;
    u.upc = g.n * g.rows * u.upr;
    u.rpu = 1;
    u.vpr = 0;
    u.magic = 0;
    u.gpo = 0;
    const long long vpr = g.len / vec;
    if (g.rows_inner > 1 && vpr >= 2 && vpr * 2 <= BN_UNIT_VECS)
    {
        u.vpr = (int) vpr;
        u.rpu = (int) (BN_UNIT_VECS / vpr < g.rows_inner ? BN_UNIT_VECS / vpr : g.rows_inner);
        u.magic = (unsigned) ((0x100000000ull + (unsigned long long) vpr - 1) / (unsigned long long) vpr);
        u.gpo = (g.rows_inner + u.rpu - 1) / u.rpu;
        u.upr = 1;
        u.upc = g.n * (g.rows / g.rows_inner) * u.gpo;
    }
    return u;
}

struct UnitPos
{
    long long nn, row, e0;
    int count; // scalars in this unit (packed: in each of its runs)
    int nsub;  // runs in this unit
};

__device__ __forceinline__ UnitPos decode_unit(const UnitGeom& ug, long long u)
{
    UnitPos p;
    if (ug.vpr)
    {
        const long long grp = u % ug.gpo;
        const long long t = u / ug.gpo;
        const long long outers = ug.g.rows / ug.g.rows_inner;
        const long long first = grp * ug.rpu;
        p.row = (t % outers) * ug.g.rows_inner + first;
        p.nn = t / outers;
        p.e0 = 0;
        p.count = (int) ug.g.len;
        const long long left = ug.g.rows_inner - first;
        p.nsub = left < ug.rpu ? (int) left : ug.rpu;
        return p;
    }
    const long long chunk = u % ug.upr;
    const long long t = u / ug.upr;
    p.row = t % ug.g.rows;
    p.nn = t / ug.g.rows;
    p.e0 = chunk * ug.unit;
    const long long rem = ug.g.len - p.e0;
    p.count = rem < ug.unit ? (int) rem : ug.unit;
    p.nsub = 1;
    return p;
}

// Vector element e of a unit: which of the unit's runs it falls into and where.
struct ElemPos
{
    int sub, col;
    bool on;
    template <int V>
    __device__ __forceinline__ long long off(const RunStrides& s) const
    {
        return (long long) sub * s.s_inner + (long long) col * V;
    }
};

template <bool PACKED>
__device__ __forceinline__ ElemPos elem_pos(const UnitGeom& ug, const UnitPos& p, int e, int nv)
{
    ElemPos q;
    if (PACKED)
    {
        q.sub = (int) __umulhi((unsigned) e, ug.magic);
        q.col = e - q.sub * ug.vpr;
        q.on = q.sub < p.nsub;
    }
    else
    {
        q.sub = 0;
        q.col = e;
        q.on = e < nv;
    }
    return q;
}

__device__ __forceinline__ long long unit_offset(const RunStrides& s,
                                                 const RunGeom& g,
                                                 const UnitPos& p, int c)
{
    return p.nn * s.sn + (long long) c * s.sc
           + (p.row / g.rows_inner) * s.s_outer
           + (p.row % g.rows_inner) * s.s_inner + p.e0;
}

template <int V>
struct Vec;
template <>
struct Vec<1>
{
    float v[1];
    __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
    __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <>
struct Vec<2>
{
    float v[2];
    __device__ __forceinline__ void load(const float* p)
    {
        float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x;
        v[1] = t.y;
    }
    __device__ __forceinline__ void store(float* p) const
    {
        *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    }
};
template <>
struct Vec<4>
{
    float v[4];
    __device__ __forceinline__ void load(const float* p)
    {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x;
        v[1] = t.y;
        v[2] = t.z;
        v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const
    {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};

// Sum NV doubles across the block; result valid in thread 0.
template <int NV>
__device__ __forceinline__ void block_reduce(double (&val)[NV])
{
    __shared__ double sm[NV][BN_THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < NV; ++i)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            val[i] += __shfl_down_sync(0xffffffffu, val[i], o);
        if (lane == 0)
            sm[i][warp] = val[i];
    }
    __syncthreads();
    if (warp == 0)
    {
#pragma unroll
        for (int i = 0; i < NV; ++i)
        {
            double v = lane < BN_THREADS / 32 ? sm[i][lane] : 0.0;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1)
                v += __shfl_down_sync(0xffffffffu, v, o);
            val[i] = v;
        }
    }
    __syncthreads();
}

// Second stage: the last block of channel c folds NV x nblocks partials in
// index order and hands the totals to `emit` (thread 0).
template <int NV, typename Emit>
__device__ __forceinline__ void finish_channel(double (&val)[NV],
                                               double* partial,
                                               unsigned* tickets, Emit emit)
{
    const int c = blockIdx.y;
    const int nb = gridDim.x;
    __shared__ int last;
    if (threadIdx.x == 0)
    {
#pragma unroll
        for (int i = 0; i < NV; ++i)
            partial[((size_t) c * nb + blockIdx.x) * NV + i] = val[i];
        __threadfence();
        const unsigned prev = atomicAdd(&tickets[c], 1u);
        last = (prev == (unsigned) nb - 1);
    }
    __syncthreads();
    if (!last)
        return;
    __threadfence();
    if (threadIdx.x < 32)
    {
        double acc[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            acc[i] = 0.0;
        // Lane l takes partials l, l+32, ... in order; lanes are then folded
        // by a fixed shuffle tree.
        for (int b = threadIdx.x; b < nb; b += 32)
#pragma unroll
            for (int i = 0; i < NV; ++i)
                acc[i] += partial[((size_t) c * nb + b) * NV + i];
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                acc[i] += __shfl_down_sync(0xffffffffu, acc[i], o);
        if (threadIdx.x == 0)
        {
            emit(acc);
            tickets[c] = 0;
        }
    }
}

template <int V, bool PACKED>
__global__ void __launch_bounds__(BN_THREADS)
    bn_stats_kernel(const float* __restrict__ x, RunStrides xs, UnitGeom ug,
                    double* partial, unsigned* tickets,
                    float* __restrict__ sums, float* __restrict__ sqsums)
{
    const int c = blockIdx.y;
    double acc[2] = {0.0, 0.0};
    for (long long u = blockIdx.x; u < ug.upc; u += gridDim.x)
    {
        const UnitPos p = decode_unit(ug, u);
        const float* xp = x + unit_offset(xs, ug.g, p, c);
        const int nv = p.count / V;
        Vec<V> v[BN_UNROLL_RED];
        bool on[BN_UNROLL_RED];
#pragma unroll
        for (int k = 0; k < BN_UNROLL_RED; ++k)
        {
            const ElemPos ep = elem_pos<PACKED>(ug, p, threadIdx.x + k * BN_THREADS, nv);
            on[k] = ep.on;
            if (on[k])
                v[k].load(xp + ep.template off<V>(xs));
        }
        float s = 0.f, q = 0.f;
#pragma unroll
        for (int k = 0; k < BN_UNROLL_RED; ++k)
            if (on[k])
#pragma unroll
                for (int i = 0; i < V; ++i)
                {
                    s += v[k].v[i];
                    q = fmaf(v[k].v[i], v[k].v[i], q);
                }
        acc[0] += (double) s;
        acc[1] += (double) q;
    }
    block_reduce<2>(acc);
    finish_channel<2>(acc, partial, tickets, [&](const double(&t)[2]) {
        sums[c] = (float) t[0];
        sqsums[c] = (float) t[1];
    });
}

__global__ void bn_finalize_kernel(int channels, long long num_per_sum,
                                   float decay, float* mean, float* var,
                                   float* running_mean, float* running_var)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels)
        return;
    if (num_per_sum > 0)
    {
        // Operation order of sums_to_statistics_functor (batchnorm.cu:297-312).
        const float nps = (float) num_per_sum;
        const float m = mean[c] / nps;
        const float sq = var[c] / nps;
        float v = sq - m * m;
        v = v > 0.f ? v : 0.f;
        v *= nps / (nps - 1.f);
        mean[c] = m;
        var[c] = v;
        running_mean[c] = decay * running_mean[c] + (1.f - decay) * m;
        running_var[c] = decay * running_var[c] + (1.f - decay) * v;
    }
    else
    {
        var[c] = 1.f;
    }
}

// LEAKY: the leaky ReLU that follows the batch-norm in the same pass
// (y > 0 ? y : slope * y), one trip through HBM instead of two.
template <int V, bool LEAKY, bool PACKED>
__global__ void __launch_bounds__(BN_THREADS)
    bn_apply_kernel(const float* __restrict__ x, RunStrides xs,
                    float* __restrict__ y, RunStrides ys, UnitGeom ug,
                    const float* __restrict__ mean,
                    const float* __restrict__ var,
                    const float* __restrict__ scale,
                    const float* __restrict__ bias, float eps, float slope)
{
    const int c = blockIdx.y;
    const float m = mean[c];
    const float inv_stdev = rsqrtf(var[c] + eps);
    const float sc = scale[c], bi = bias[c];
    for (long long u = blockIdx.x; u < ug.upc; u += gridDim.x)
    {
        const UnitPos p = decode_unit(ug, u);
        const float* xp = x + unit_offset(xs, ug.g, p, c);
        float* yp = y + unit_offset(ys, ug.g, p, c);
        const int nv = p.count / V;
        Vec<V> v[BN_UNROLL_MAP];
        ElemPos ep[BN_UNROLL_MAP];
#pragma unroll
        for (int k = 0; k < BN_UNROLL_MAP; ++k)
        {
            ep[k] = elem_pos<PACKED>(ug, p, threadIdx.x + k * BN_THREADS, nv);
            if (ep[k].on)
                v[k].load(xp + ep[k].template off<V>(xs));
        }
#pragma unroll
        for (int k = 0; k < BN_UNROLL_MAP; ++k)
            if (ep[k].on)
            {
#pragma unroll
                for (int i = 0; i < V; ++i)
                {
                    const float xhat = (v[k].v[i] - m) * inv_stdev;
                    const float o = sc * xhat + bi;
                    v[k].v[i] = LEAKY ? (o > 0.f ? o : o * slope) : o;
                }
                v[k].store(yp + ep[k].template off<V>(ys));
            }
    }
}

template <int V, bool PACKED>
__global__ void __launch_bounds__(BN_THREADS)
    bn_bwd_reduce_kernel(const float* __restrict__ x, RunStrides xs,
                         const float* __restrict__ dy, RunStrides ds,
                         UnitGeom ug, const float* __restrict__ mean,
                         const float* __restrict__ var,
                         const float* __restrict__ scale, float eps,
                         double* partial, unsigned* tickets,
                         float* __restrict__ dscale, float* __restrict__ dbias,
                         float* __restrict__ dmean, float* __restrict__ dvar)
{
    const int c = blockIdx.y;
    const float m = mean[c];
    const float sc = scale[c];
    const float inv_stdev = rsqrtf(var[c] + eps);
    const float dvar_factor = inv_stdev * inv_stdev * inv_stdev / 2;
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    for (long long u = blockIdx.x; u < ug.upc; u += gridDim.x)
    {
        const UnitPos p = decode_unit(ug, u);
        const float* xp = x + unit_offset(xs, ug.g, p, c);
        const float* dp = dy + unit_offset(ds, ug.g, p, c);
        const int nv = p.count / V;
        Vec<V> vx[BN_UNROLL_RED], vd[BN_UNROLL_RED];
        bool on[BN_UNROLL_RED];
#pragma unroll
        for (int k = 0; k < BN_UNROLL_RED; ++k)
        {
            const ElemPos ep = elem_pos<PACKED>(ug, p, threadIdx.x + k * BN_THREADS, nv);
            on[k] = ep.on;
            if (on[k])
            {
                vx[k].load(xp + ep.template off<V>(xs));
                vd[k].load(dp + ep.template off<V>(ds));
            }
        }
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int k = 0; k < BN_UNROLL_RED; ++k)
            if (on[k])
#pragma unroll
                for (int i = 0; i < V; ++i)
                {
                    // backprop1 (batchnorm.cu:940-952)
                    const float xv = vx[k].v[i], g = vd[k].v[i];
                    const float xhat = (xv - m) * inv_stdev;
                    a0 += g * xhat;
                    a1 += g;
                    const float dxhat = g * sc;
                    a2 += -dxhat * inv_stdev;
                    a3 += -dxhat * (xv - m) * dvar_factor;
                }
        acc[0] += (double) a0;
        acc[1] += (double) a1;
        acc[2] += (double) a2;
        acc[3] += (double) a3;
    }
    block_reduce<4>(acc);
    finish_channel<4>(acc, partial, tickets, [&](const double(&t)[4]) {
        dscale[c] = (float) t[0];
        dbias[c] = (float) t[1];
        dmean[c] = (float) t[2];
        dvar[c] = (float) t[3];
    });
}

template <int V, bool PACKED>
__global__ void __launch_bounds__(BN_THREADS)
    bn_bwd_apply_kernel(const float* x, RunStrides xs,
                        const float* __restrict__ dy, RunStrides ds, float* dx,
                        RunStrides os, UnitGeom ug,
                        const float* __restrict__ mean,
                        const float* __restrict__ var,
                        const float* __restrict__ scale,
                        const float* __restrict__ dmean,
                        const float* __restrict__ dvar, float eps,
                        long long num_per_sum)
{
    const int c = blockIdx.y;
    const float m = mean[c];
    const float sc = scale[c];
    const float inv_stdev = rsqrtf(var[c] + eps);
    // backprop2 (batchnorm.cu:1333-1335)
    const float dmean_term = dmean[c] / (float) num_per_sum;
    const float dvar_term = dvar[c] * 2 / (float) (num_per_sum - 1);
    for (long long u = blockIdx.x; u < ug.upc; u += gridDim.x)
    {
        const UnitPos p = decode_unit(ug, u);
        const float* xp = x + unit_offset(xs, ug.g, p, c);
        const float* dp = dy + unit_offset(ds, ug.g, p, c);
        float* op = dx + unit_offset(os, ug.g, p, c);
        const int nv = p.count / V;
        Vec<V> vx[BN_UNROLL_MAP], vd[BN_UNROLL_MAP];
        ElemPos ep[BN_UNROLL_MAP];
#pragma unroll
        for (int k = 0; k < BN_UNROLL_MAP; ++k)
        {
            ep[k] = elem_pos<PACKED>(ug, p, threadIdx.x + k * BN_THREADS, nv);
            if (ep[k].on)
            {
                vx[k].load(xp + ep[k].template off<V>(xs));
                vd[k].load(dp + ep[k].template off<V>(ds));
            }
        }
#pragma unroll
        for (int k = 0; k < BN_UNROLL_MAP; ++k)
            if (ep[k].on)
            {
#pragma unroll
                for (int i = 0; i < V; ++i)
                {
                    const float dxhat = vd[k].v[i] * sc;
                    float r = dxhat * inv_stdev;
                    r += dmean_term;
                    r += dvar_term * (vx[k].v[i] - m);
                    vd[k].v[i] = r;
                }
                vd[k].store(op + ep[k].template off<V>(os));
            }
    }
}

// mode 0: y = x>0 ? x : slope*x ;  mode 1: dx = x>0 ? dy : slope*dy
template <int V, int MODE, bool PACKED>
__global__ void __launch_bounds__(BN_THREADS)
    leaky_relu_kernel(const float* x, RunStrides xs,
                      const float* __restrict__ dy, RunStrides ds, float* out,
                      RunStrides os, UnitGeom ug, float slope)
{
    const int c = blockIdx.y;
    for (long long u = blockIdx.x; u < ug.upc; u += gridDim.x)
    {
        const UnitPos p = decode_unit(ug, u);
        const float* xp = x + unit_offset(xs, ug.g, p, c);
        const float* dp = MODE ? dy + unit_offset(ds, ug.g, p, c) : nullptr;
        float* op = out + unit_offset(os, ug.g, p, c);
        const int nv = p.count / V;
#pragma unroll
        for (int k = 0; k < BN_UNROLL_MAP; ++k)
        {
            const ElemPos ep = elem_pos<PACKED>(ug, p, threadIdx.x + k * BN_THREADS, nv);
            if (ep.on)
            {
                Vec<V> vx, vd;
                vx.load(xp + ep.template off<V>(xs));
                if (MODE)
                    vd.load(dp + ep.template off<V>(ds));
#pragma unroll
                for (int i = 0; i < V; ++i)
                {
                    const float src = MODE ? vd.v[i] : vx.v[i];
                    vx.v[i] = vx.v[i] > 0.f ? src : slope * src;
                }
                vx.store(op + ep.template off<V>(os));
            }
        }
    }
}

static dim3 bn_grid(const UnitGeom& ug)
{
    long long per_c = (long long) num_sms() * 8 / (ug.g.c > 0 ? ug.g.c : 1);
    if (per_c < 1)
        per_c = 1;
    long long bx = ug.upc < per_c ? ug.upc : per_c;
    if (bx < 1)
        bx = 1;
    return dim3((unsigned) bx, (unsigned) ug.g.c);
}

// Common level / vector width for a set of same-shaped tensors.
struct MultiView
{
    UnitGeom ug;
    RunStrides s[3];
    int vec;
};

static int32_t make_multi(const dcb_nd_desc* const* descs,
                          const void* const* ptrs, int count, MultiView* mv, int unroll)
{
    int level = 2;
    for (int i = 0; i < count; ++i)
    {
        int32_t st = check_nd_desc(descs[i]);
        if (st != DCB_OK)
            return st;
        DCB_REQUIRE(same_extents(*descs[0], *descs[i]),
                    "tensor extents differ");
        const int l = run_level(*descs[i]);
        if (l < 0)
        {
            set_last_error("innermost dimension must have unit stride");
            return DCB_UNSUPPORTED;
        }
        level = l < level ? l : level;
    }
    RunGeom g;
    int vec = 4;
    for (int i = 0; i < count; ++i)
    {
        make_runs(*descs[i], level, &g, &mv->s[i]);
        const int v = run_vec(g, mv->s[i], ptrs[i]);
        vec = v < vec ? v : vec;
    }
    mv->ug = make_units(g, vec, unroll);
    mv->vec = vec;
    DCB_REQUIRE(g.c <= 65535, "too many channels");
    return DCB_OK;
}

} // namespace dcb

using namespace dcb;

struct dcb_bn_plan
{
    dcb_nd_desc xd;
    double* partial = nullptr;
    unsigned* tickets = nullptr;
    int max_blocks = 0;
};

// PACKED (several short runs per unit) is a template parameter: the kernels that
// walk long runs keep their plain indexing.
#define DCB_VEC_DISPATCH(vec, packed, CALL)                                    \
    do                                                                         \
    {                                                                          \
        if (packed)                                                            \
        {                                                                      \
            if ((vec) == 4)                                                    \
            {                                                                  \
                CALL(4, true);                                                 \
            }                                                                  \
            else if ((vec) == 2)                                               \
            {                                                                  \
                CALL(2, true);                                                 \
            }                                                                  \
            else                                                               \
            {                                                                  \
                CALL(1, true);                                                 \
            }                                                                  \
        }                                                                      \
        else if ((vec) == 4)                                                   \
        {                                                                      \
            CALL(4, false);                                                    \
        }                                                                      \
        else if ((vec) == 2)                                                   \
        {                                                                      \
            CALL(2, false);                                                    \
        }                                                                      \
        else                                                                   \
        {                                                                      \
            CALL(1, false);                                                    \
        }                                                                      \
    } while (0)

extern "C" {

int32_t dcb_bn_plan_create(const dcb_nd_desc* xd, dcb_bn_plan** out)
{
    int32_t st = check_nd_desc(xd);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(out != nullptr, "null argument");
    DCB_REQUIRE(xd->c > 0 && xd->c <= 65535, "channel count out of range");
    auto* p = new dcb_bn_plan();
    p->xd = *xd;
    p->max_blocks = num_sms() * 8;
    const size_t nb = (size_t) p->max_blocks + (size_t) xd->c;
    if (cudaMalloc(&p->partial, nb * 4 * sizeof(double)) != cudaSuccess
        || cudaMalloc(&p->tickets, (size_t) xd->c * sizeof(unsigned))
               != cudaSuccess
        || cudaMemset(p->tickets, 0, (size_t) xd->c * sizeof(unsigned))
               != cudaSuccess)
    {
        set_last_error("cudaMalloc of batch-norm scratch failed");
        (void) cudaGetLastError();
        cudaFree(p->partial);
        cudaFree(p->tickets);
        delete p;
        return DCB_CUDA_ERROR;
    }
    *out = p;
    return DCB_OK;
}

int32_t dcb_bn_plan_destroy(dcb_bn_plan* p)
{
    if (!p)
        return DCB_OK;
    cudaFree(p->partial);
    cudaFree(p->tickets);
    delete p;
    return DCB_OK;
}

int32_t dcb_bn_stats(dcb_bn_plan* plan, const void* x, void* sums,
                     void* sqsums, void* stream)
{
    DCB_REQUIRE(plan && x && sums && sqsums, "null argument");
    const dcb_nd_desc* descs[1] = {&plan->xd};
    const void* ptrs[1] = {x};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 1, &mv, BN_UNROLL_RED);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
    {
        DCB_CUDA_TRY(cudaMemsetAsync(sums, 0, plan->xd.c * sizeof(float),
                                     as_stream(stream)));
        DCB_CUDA_TRY(cudaMemsetAsync(sqsums, 0, plan->xd.c * sizeof(float),
                                     as_stream(stream)));
        return DCB_OK;
    }
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    bn_stats_kernel<VV, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(           \
        static_cast<const float*>(x), mv.s[0], mv.ug, plan->partial,           \
        plan->tickets, static_cast<float*>(sums), static_cast<float*>(sqsums))
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_bn_finalize(int32_t channels, int64_t num_per_sum, float decay,
                        void* mean, void* var, void* running_mean,
                        void* running_var, void* stream)
{
    DCB_REQUIRE(channels > 0, "channels must be positive");
    DCB_REQUIRE(mean && var && running_mean && running_var, "null argument");
    bn_finalize_kernel<<<(channels + 127) / 128, 128, 0, as_stream(stream)>>>(
        channels, num_per_sum, decay, static_cast<float*>(mean),
        static_cast<float*>(var), static_cast<float*>(running_mean),
        static_cast<float*>(running_var));
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

static int32_t bn_apply_impl(const dcb_nd_desc* xd, const void* x, const void* mean, const void* var,
                             const void* scale, const void* bias, float eps, bool leaky, float slope,
                             const dcb_nd_desc* yd, void* y, void* stream)
{
    DCB_REQUIRE(x && y && mean && var && scale && bias, "null argument");
    const dcb_nd_desc* descs[2] = {xd, yd};
    const void* ptrs[2] = {x, y};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 2, &mv, BN_UNROLL_MAP);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
        return DCB_OK;
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    if (leaky)                                                                 \
        bn_apply_kernel<VV, true, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>( \
            static_cast<const float*>(x), mv.s[0], static_cast<float*>(y),     \
            mv.s[1], mv.ug, static_cast<const float*>(mean),                   \
            static_cast<const float*>(var), static_cast<const float*>(scale),  \
            static_cast<const float*>(bias), eps, slope);                      \
    else                                                                       \
        bn_apply_kernel<VV, false, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(\
            static_cast<const float*>(x), mv.s[0], static_cast<float*>(y),     \
            mv.s[1], mv.ug, static_cast<const float*>(mean),                   \
            static_cast<const float*>(var), static_cast<const float*>(scale),  \
            static_cast<const float*>(bias), eps, slope)
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_bn_apply(const dcb_nd_desc* xd, const void* x, const void* mean,
                     const void* var, const void* scale, const void* bias,
                     float eps, const dcb_nd_desc* yd, void* y, void* stream)
{
    return bn_apply_impl(xd, x, mean, var, scale, bias, eps, false, 1.f, yd, y, stream);
}

int32_t dcb_bn_apply_leaky_relu(const dcb_nd_desc* xd, const void* x,
                                const void* mean, const void* var,
                                const void* scale, const void* bias, float eps,
                                float slope, const dcb_nd_desc* yd, void* y,
                                void* stream)
{
    return bn_apply_impl(xd, x, mean, var, scale, bias, eps, true, slope, yd, y, stream);
}

int32_t dcb_bn_bwd_reduce(dcb_bn_plan* plan, const void* x,
                          const dcb_nd_desc* dyd, const void* dy,
                          const void* mean, const void* var, const void* scale,
                          float eps, void* dscale, void* dbias, void* dmean,
                          void* dvar, void* stream)
{
    DCB_REQUIRE(plan && x && dy && mean && var && scale && dscale && dbias
                    && dmean && dvar,
                "null argument");
    const dcb_nd_desc* descs[2] = {&plan->xd, dyd};
    const void* ptrs[2] = {x, dy};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 2, &mv, BN_UNROLL_RED);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
    {
        for (void* v : {dscale, dbias, dmean, dvar})
            DCB_CUDA_TRY(cudaMemsetAsync(v, 0, plan->xd.c * sizeof(float),
                                         as_stream(stream)));
        return DCB_OK;
    }
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    bn_bwd_reduce_kernel<VV, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(      \
        static_cast<const float*>(x), mv.s[0], static_cast<const float*>(dy),  \
        mv.s[1], mv.ug, static_cast<const float*>(mean),                       \
        static_cast<const float*>(var), static_cast<const float*>(scale), eps, \
        plan->partial, plan->tickets, static_cast<float*>(dscale),             \
        static_cast<float*>(dbias), static_cast<float*>(dmean),                \
        static_cast<float*>(dvar))
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_bn_bwd_apply(const dcb_nd_desc* xd, const void* x,
                         const dcb_nd_desc* dyd, const void* dy,
                         const void* mean, const void* var, const void* scale,
                         const void* dmean, const void* dvar, float eps,
                         int64_t num_per_sum, const dcb_nd_desc* dxd, void* dx,
                         void* stream)
{
    DCB_REQUIRE(x && dy && dx && mean && var && scale && dmean && dvar,
                "null argument");
    const dcb_nd_desc* descs[3] = {xd, dyd, dxd};
    const void* ptrs[3] = {x, dy, dx};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 3, &mv, BN_UNROLL_MAP);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
        return DCB_OK;
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    bn_bwd_apply_kernel<VV, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(       \
        static_cast<const float*>(x), mv.s[0], static_cast<const float*>(dy),  \
        mv.s[1], static_cast<float*>(dx), mv.s[2], mv.ug,                      \
        static_cast<const float*>(mean), static_cast<const float*>(var),       \
        static_cast<const float*>(scale), static_cast<const float*>(dmean),    \
        static_cast<const float*>(dvar), eps, (long long) num_per_sum)
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_leaky_relu_fwd(const dcb_nd_desc* xd, const void* x, float slope,
                           const dcb_nd_desc* yd, void* y, void* stream)
{
    DCB_REQUIRE(x && y, "null argument");
    const dcb_nd_desc* descs[2] = {xd, yd};
    const void* ptrs[2] = {x, y};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 2, &mv, BN_UNROLL_MAP);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
        return DCB_OK;
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    leaky_relu_kernel<VV, 0, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(      \
        static_cast<const float*>(x), mv.s[0], nullptr, mv.s[0],               \
        static_cast<float*>(y), mv.s[1], mv.ug, slope)
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_leaky_relu_bwd(const dcb_nd_desc* xd, const void* x,
                           const dcb_nd_desc* dyd, const void* dy, float slope,
                           const dcb_nd_desc* dxd, void* dx, void* stream)
{
    DCB_REQUIRE(x && dy && dx, "null argument");
    const dcb_nd_desc* descs[3] = {xd, dyd, dxd};
    const void* ptrs[3] = {x, dy, dx};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 3, &mv, BN_UNROLL_MAP);
    if (st != DCB_OK)
        return st;
    if (mv.ug.upc == 0)
        return DCB_OK;
    const dim3 grid = bn_grid(mv.ug);
#define CALL(VV, PP)                                                               \
    leaky_relu_kernel<VV, 1, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(      \
        static_cast<const float*>(x), mv.s[0], static_cast<const float*>(dy),  \
        mv.s[1], static_cast<float*>(dx), mv.s[2], mv.ug, slope)
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

} // extern "C"

// ---------------------------------------------------------------------------
// Per-channel statistics without any device allocation.
//
// Some hosts cannot let a library call cudaMalloc: a training framework whose
// caching allocator already owns the whole device, code that runs between
// cudaStreamBeginCapture and EndCapture (allocation is illegal there), or a
// latency-critical loop where cudaMalloc's implicit device synchronisation is
// not acceptable.  For them this variant of dcb_bn_stats keeps its reduction
// scratch (per-block partial sums and the per-channel arrival tickets) in a
// fixed array that is part of the library image.  Every GPU that loads the
// library carries the array until the process exits.
// ---------------------------------------------------------------------------
namespace
{
constexpr int NOALLOC_MAX_CHANNELS = 1024;
constexpr int NOALLOC_MAX_BLOCKS = 4096; // blocks of one launch, all channels together
constexpr size_t NOALLOC_TICKET_BYTES = NOALLOC_MAX_CHANNELS * sizeof(unsigned);
constexpr size_t NOALLOC_PARTIAL_BYTES = (size_t) NOALLOC_MAX_BLOCKS * 2 * sizeof(double);
constexpr int NOALLOC_MAX_DEVICES = 64;

// Layout: [tickets: 1024 x u32][partials: 4096 x 2 x f64] = 68 KiB.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_TICKET_BYTES + NOALLOC_PARTIAL_BYTES];

// Device address of the array on each device, resolved on first use.  In host
// code the symbol itself is only a handle, never a pointer a kernel may use.
// Host threads may race on an entry: they would all store the same address,
// so relaxed atomics are enough.
static std::atomic<void*> g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};
} // namespace

extern "C" int32_t dcb_bn_stats_noalloc(const dcb_nd_desc* xd, const void* x, void* sums, void* sqsums,
                                        void* stream)
{
    DCB_REQUIRE(xd && x && sums && sqsums, "null argument");
    const dcb_nd_desc* descs[1] = {xd};
    const void* ptrs[1] = {x};
    MultiView mv;
    int32_t st = make_multi(descs, ptrs, 1, &mv, BN_UNROLL_RED);
    if (st != DCB_OK)
        return st;
    if (xd->c < 1 || xd->c > NOALLOC_MAX_CHANNELS)
    {
        set_last_error("dcb_bn_stats_noalloc handles 1..1024 channels; use dcb_bn_stats with a plan beyond that");
        return DCB_UNSUPPORTED;
    }
    int dev = 0;
    DCB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES)
    {
        set_last_error("dcb_bn_stats_noalloc: device ordinal beyond 63");
        return DCB_UNSUPPORTED;
    }
    void* addr = g_noalloc_addr[dev].load(std::memory_order_relaxed);
    if (addr == nullptr)
    {
        // once per device, with that device current
        DCB_CUDA_TRY(cudaGetSymbolAddress(&addr, g_noalloc_scratch));
        g_noalloc_addr[dev].store(addr, std::memory_order_relaxed);
    }
    unsigned char* base = static_cast<unsigned char*>(addr);
    unsigned* tickets = reinterpret_cast<unsigned*>(base);
    double* partial = reinterpret_cast<double*>(base + NOALLOC_TICKET_BYTES);
    if (mv.ug.upc == 0)
    {
        DCB_CUDA_TRY(cudaMemsetAsync(sums, 0, xd->c * sizeof(float), as_stream(stream)));
        DCB_CUDA_TRY(cudaMemsetAsync(sqsums, 0, xd->c * sizeof(float), as_stream(stream)));
        return DCB_OK;
    }
    dim3 grid = bn_grid(mv.ug);
    // stay inside the fixed scratch: fewer blocks per channel if need be
    if ((long long) grid.x * grid.y > NOALLOC_MAX_BLOCKS)
        grid.x = (unsigned) (NOALLOC_MAX_BLOCKS / grid.y);
    if (grid.x < 1)
    {
        set_last_error("dcb_bn_stats_noalloc: launch does not fit the fixed scratch");
        return DCB_UNSUPPORTED;
    }
    // The array keeps whatever the previous call (or an interrupted one) left:
    // the arrival tickets must start at zero.  Partials are overwritten.
    DCB_CUDA_TRY(cudaMemsetAsync(tickets, 0, xd->c * sizeof(unsigned), as_stream(stream)));
#define CALL(VV, PP)                                                               \
    bn_stats_kernel<VV, PP><<<grid, BN_THREADS, 0, as_stream(stream)>>>(           \
        static_cast<const float*>(x), mv.s[0], mv.ug, partial, tickets,        \
        static_cast<float*>(sums), static_cast<float*>(sqsums))
    DCB_VEC_DISPATCH(mv.vec, mv.ug.vpr != 0, CALL);
#undef CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}
