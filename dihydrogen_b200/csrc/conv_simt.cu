// fp32 CUDA-core convolution kernels: the general path (any stride, dilation,
// filter extent, channel count) and the numerical reference for the
// tensor-core kernels.  Cross-correlation, NC[D]HW, W unit-stride.
#include "conv_simt.cuh"

namespace dcb
{

// ---------------------------------------------------------------------------
// forward: each thread owns WT outputs along W (interleaved by 32 so every
// load and store of a warp is one contiguous 128-byte row segment) times KT
// output channels; filter taps for a slab of input channels sit in shared
// memory and are read as broadcast float4.
// ---------------------------------------------------------------------------
constexpr int FWD_TX = 32, FWD_TY = 4;

template <int KT, int WT>
__global__ void __launch_bounds__(FWD_TX* FWD_TY)
    conv_fwd_kernel(ConvGeom g, float alpha, float beta,
                    const float* __restrict__ x, const float* __restrict__ w,
                    float* y, int ctile, int ktiles, int oh_tiles)
{
    extern __shared__ __align__(16) float ws[];
    const int taps = g.f[0] * g.f[1] * g.f[2];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int tid = ty * FWD_TX + tx;
    const int kt = blockIdx.z % ktiles;
    const int n = blockIdx.z / ktiles;
    // the (plane, row tile) product is the large one: it rides on grid.x
    const int od = blockIdx.x / oh_tiles;
    const int oh = (blockIdx.x % oh_tiles) * FWD_TY + ty;
    const int ow_base = blockIdx.y * (FWD_TX * WT) + tx;
    const bool row_ok = oh < g.out[1];

    float acc[WT][KT];
#pragma unroll
    for (int j = 0; j < WT; ++j)
#pragma unroll
        for (int kk = 0; kk < KT; ++kk)
            acc[j][kk] = 0.f;

    for (int c0 = 0; c0 < g.c; c0 += ctile)
    {
        __syncthreads();
        const int nload = ctile * taps * KT;
        for (int idx = tid; idx < nload; idx += FWD_TX * FWD_TY)
        {
            const int kk = idx % KT;
            const int tap = (idx / KT) % taps;
            const int cc = idx / (KT * taps);
            const int k = kt * KT + kk, c = c0 + cc;
            ws[idx] = (k < g.k && c < g.c)
                          ? w[((size_t) k * g.c + c) * taps + tap]
                          : 0.f;
        }
        __syncthreads();
        if (!row_ok)
            continue;
        const int cend = min(ctile, g.c - c0);
        for (int cc = 0; cc < cend; ++cc)
        {
            const float* xc = x + (size_t) n * g.xs_n + (size_t) (c0 + cc) * g.xs_c;
            for (int kd = 0; kd < g.f[0]; ++kd)
            {
                const int id = od * g.stride[0] - g.pad[0] + kd * g.dil[0];
                if (id < 0 || id >= g.in[0])
                    continue;
                for (int kh = 0; kh < g.f[1]; ++kh)
                {
                    const int ih = oh * g.stride[1] - g.pad[1] + kh * g.dil[1];
                    if (ih < 0 || ih >= g.in[1])
                        continue;
                    const float* xrow = xc + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1];
                    const float* wrow =
                        ws + ((size_t) cc * taps + (kd * g.f[1] + kh) * g.f[2]) * KT;
                    for (int kw = 0; kw < g.f[2]; ++kw)
                    {
                        float wv[KT];
#pragma unroll
                        for (int q = 0; q < KT / 4; ++q)
                        {
                            const float4 t = reinterpret_cast<const float4*>(
                                wrow + kw * KT)[q];
                            wv[4 * q + 0] = t.x;
                            wv[4 * q + 1] = t.y;
                            wv[4 * q + 2] = t.z;
                            wv[4 * q + 3] = t.w;
                        }
#pragma unroll
                        for (int j = 0; j < WT; ++j)
                        {
                            const int ow = ow_base + j * FWD_TX;
                            const int iw = ow * g.stride[2] - g.pad[2] + kw * g.dil[2];
                            const float xv =
                                (ow < g.out[2] && iw >= 0 && iw < g.in[2])
                                    ? xrow[iw]
                                    : 0.f;
#pragma unroll
                            for (int kk = 0; kk < KT; ++kk)
                                acc[j][kk] = fmaf(xv, wv[kk], acc[j][kk]);
                        }
                    }
                }
            }
        }
    }
    if (!row_ok)
        return;
#pragma unroll
    for (int j = 0; j < WT; ++j)
    {
        const int ow = ow_base + j * FWD_TX;
        if (ow >= g.out[2])
            continue;
#pragma unroll
        for (int kk = 0; kk < KT; ++kk)
        {
            const int k = kt * KT + kk;
            if (k >= g.k)
                continue;
            float* yp = y + (size_t) n * g.ys_n + (size_t) k * g.ys_c
                        + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
            const float prev = beta != 0.f ? *yp : 0.f;
            *yp = alpha * acc[j][kk] + beta * prev;
        }
    }
}

template <int KT, int WT>
static int32_t launch_fwd(const ConvGeom& g, float alpha, const float* x,
                          const float* w, float beta, float* y,
                          cudaStream_t stream)
{
    const int taps = g.f[0] * g.f[1] * g.f[2];
    int ctile = (32 * 1024) / (taps * KT * (int) sizeof(float));
    if (ctile < 1)
        ctile = 1;
    if (ctile > g.c)
        ctile = g.c;
    const size_t smem = (size_t) ctile * taps * KT * sizeof(float);
    if (smem > 48 * 1024)
    {
        set_last_error("filter too large for the fp32 forward kernel");
        return DCB_UNSUPPORTED;
    }
    const int ktiles = (g.k + KT - 1) / KT;
    const int oh_tiles = (g.out[1] + FWD_TY - 1) / FWD_TY;
    const long long gy = (long long) oh_tiles * g.out[0];
    const long long gz = (long long) g.n * ktiles;
    const long long gw = (g.out[2] + FWD_TX * WT - 1) / (FWD_TX * WT);
    if (gy > 0x7fffffffll || gw > 65535 || gz > 65535)
    {
        set_last_error("tensor too large for the fp32 forward kernel grid");
        return DCB_UNSUPPORTED;
    }
    dim3 grid((unsigned) gy, (unsigned) gw, (unsigned) gz);
    dim3 block(FWD_TX, FWD_TY);
    conv_fwd_kernel<KT, WT><<<grid, block, smem, stream>>>(
        g, alpha, beta, x, w, y, ctile, ktiles, oh_tiles);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t simt_conv_fwd(const ConvGeom& g, float alpha, const float* x,
                      const float* w, float beta, float* y,
                      cudaStream_t stream)
{
    if ((long long) g.n * g.k * g.out[0] * g.out[1] * g.out[2] == 0)
        return DCB_OK;
    if (g.k > 8)
        return launch_fwd<16, 4>(g, alpha, x, w, beta, y, stream);
    if (g.k > 4)
        return launch_fwd<8, 4>(g, alpha, x, w, beta, y, stream);
    return launch_fwd<4, 4>(g, alpha, x, w, beta, y, stream);
}

__global__ void flip_transpose_kernel(const float* __restrict__ w,
                                      float* __restrict__ w2, int k, int c,
                                      int taps)
{
    const int total = k * c * taps;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += gridDim.x * blockDim.x)
    {
        const int t = i % taps;
        const int cc = (i / taps) % c;
        const int kk = i / (taps * c);
        w2[((size_t) cc * k + kk) * taps + (taps - 1 - t)] = w[i];
    }
}

int32_t flip_transpose_filter(const float* w, float* w2, int k, int c,
                              int taps, cudaStream_t stream)
{
    const int total = k * c * taps;
    if (total == 0)
        return DCB_OK;
    flip_transpose_kernel<<<(total + 255) / 256, 256, 0, stream>>>(w, w2, k, c,
                                                                   taps);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

// ---------------------------------------------------------------------------
// backward data, gather form: one thread per input cell and CT channels.
// ---------------------------------------------------------------------------
constexpr int BWD_THREADS = 128;

// acc[0..CT) += v * w[0..CT): the weights of one (filter, tap) sit in CT
// consecutive, 16-byte aligned floats of shared memory; read them as vectors.
template <int CT>
__device__ __forceinline__ void fma_tile(float (&acc)[CT], float v, const float* __restrict__ w)
{
#pragma unroll
    for (int q = 0; q < CT / 4; ++q)
    {
        const float4 w4 = *reinterpret_cast<const float4*>(w + 4 * q);
        acc[4 * q + 0] = fmaf(v, w4.x, acc[4 * q + 0]);
        acc[4 * q + 1] = fmaf(v, w4.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(v, w4.z, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(v, w4.w, acc[4 * q + 3]);
    }
}

template <int CT>
__global__ void __launch_bounds__(BWD_THREADS)
    conv_bwd_data_kernel(ConvGeom g, float alpha, float beta,
                         const float* __restrict__ w,
                         const float* __restrict__ dy, float* dx, int ktile,
                         int ctiles, int rows, int htiles)
{
    extern __shared__ __align__(16) float ws[]; // [ktile][taps][CT]
    const int taps = g.f[0] * g.f[1] * g.f[2];
    // With stride 2 along W the taps a cell receives depend on its parity: a warp
    // takes cells of one parity (every second cell), so that its lanes walk the
    // same taps and read consecutive dy cells.
    const int iw = g.stride[2] == 2
                       ? blockIdx.y * BWD_THREADS + (threadIdx.x >> 6) * 64 + 2 * (threadIdx.x & 31)
                             + ((threadIdx.x >> 5) & 1)
                       : blockIdx.y * BWD_THREADS + threadIdx.x;
    // A block stages the filter once and walks `rows` input rows with it (staging
    // costs more than one row's arithmetic); rows > 1 only when the whole filter
    // fits (one k0 pass), so that a row's sums never have to outlive a pass.
    const int ih0 = (blockIdx.x % htiles) * rows;
    const int id = blockIdx.x / htiles;
    const int ct = blockIdx.z % ctiles;
    const int n = blockIdx.z / ctiles;
    // Only the taps whose output coordinate is whole: with dilation 1 those are
    // k = (i + pad) mod stride, then every stride-th (one modulo per dimension
    // and cell instead of one per tap); a dilated filter walks all taps.
    const bool d1 = g.dil[0] == 1 && g.dil[1] == 1 && g.dil[2] == 1;
    const int sd = d1 ? g.stride[0] : 1, sh = d1 ? g.stride[1] : 1, sw = d1 ? g.stride[2] : 1;
    const int kd0 = d1 ? (id + g.pad[0]) % g.stride[0] : 0;
    const int kw0 = d1 ? (iw + g.pad[2]) % g.stride[2] : 0;
    const size_t wstep = (size_t) taps * CT;
    float acc[CT];
    for (int k0 = 0; k0 < g.k; k0 += ktile)
    {
        __syncthreads();
        const int nload = ktile * taps * CT;
        for (int idx = threadIdx.x; idx < nload; idx += BWD_THREADS)
        {
            const int cc = idx % CT;
            const int tap = (idx / CT) % taps;
            const int kk = idx / (CT * taps);
            const int k = k0 + kk, c = ct * CT + cc;
            ws[idx] = (k < g.k && c < g.c)
                          ? w[((size_t) k * g.c + c) * taps + tap]
                          : 0.f;
        }
        __syncthreads();
        if (iw >= g.in[2])
            continue;
        const int kend = min(ktile, g.k - k0);
        const float* dyn = dy + (size_t) n * g.ys_n + (size_t) k0 * g.ys_c;
        for (int r = 0; r < rows; ++r)
        {
            const int ih = ih0 + r;
            if (ih >= g.in[1])
                break;
            if (k0 == 0)
            {
#pragma unroll
                for (int i = 0; i < CT; ++i)
                    acc[i] = 0.f;
            }
            const int kh0 = d1 ? (ih + g.pad[1]) % g.stride[1] : 0;
            for (int kd = kd0; kd < g.f[0]; kd += sd)
            {
                const int td = id + g.pad[0] - kd * g.dil[0];
                if (td < 0 || td % g.stride[0])
                    continue;
                const int od = td / g.stride[0];
                if (od >= g.out[0])
                    continue;
                for (int kh = kh0; kh < g.f[1]; kh += sh)
                {
                    const int th = ih + g.pad[1] - kh * g.dil[1];
                    if (th < 0 || th % g.stride[1])
                        continue;
                    const int oh = th / g.stride[1];
                    if (oh >= g.out[1])
                        continue;
                    const float* dyrow = dyn + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1];
                    for (int kw = kw0; kw < g.f[2]; kw += sw)
                    {
                        const int tw = iw + g.pad[2] - kw * g.dil[2];
                        if (tw < 0 || tw % g.stride[2])
                            continue;
                        const int ow = tw / g.stride[2];
                        if (ow >= g.out[2])
                            continue;
                        const float* dyp = dyrow + ow;
                        const float* wp = ws + (size_t) ((kd * g.f[1] + kh) * g.f[2] + kw) * CT;
                        // four loads in flight per thread: one at a time left the
                        // loop waiting on each dy cell
                        int kk = 0;
                        for (; kk + 4 <= kend; kk += 4)
                        {
                            float v[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                            {
                                v[u] = __ldg(dyp);
                                dyp += g.ys_c;
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                            {
                                fma_tile<CT>(acc, v[u], wp);
                                wp += wstep;
                            }
                        }
                        for (; kk < kend; ++kk)
                        {
                            fma_tile<CT>(acc, __ldg(dyp), wp);
                            dyp += g.ys_c;
                            wp += wstep;
                        }
                    }
                }
            }
            if (k0 + ktile < g.k)
                continue; // rows == 1 here: the sums go on in the next pass
#pragma unroll
            for (int cc = 0; cc < CT; ++cc)
            {
                const int c = ct * CT + cc;
                if (c >= g.c)
                    continue;
                float* xp = dx + (size_t) n * g.xs_n + (size_t) c * g.xs_c
                            + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1] + iw;
                const float prev = beta != 0.f ? *xp : 0.f;
                *xp = alpha * acc[cc] + beta * prev;
            }
        }
    }
}

template <int CT>
static int32_t launch_bwd_data(const ConvGeom& g, float alpha, const float* w,
                               const float* dy, float beta, float* dx,
                               cudaStream_t stream)
{
    const int taps = g.f[0] * g.f[1] * g.f[2];
    // the whole filter in shared memory where it fits (up to 96 KiB, two blocks
    // per SM): then a block reuses it for several rows
    const size_t per_k = (size_t) taps * CT * sizeof(float);
    int ktile = g.k;
    if (per_k * ktile > 96 * 1024)
        ktile = (int) ((32 * 1024) / per_k);
    if (ktile < 1)
    {
        set_last_error("filter too large for the fp32 backward-data kernel");
        return DCB_UNSUPPORTED;
    }
    const size_t smem = per_k * ktile;
    const int rows = ktile >= g.k ? 8 : 1;
    const int htiles = (g.in[1] + rows - 1) / rows;
    const int ctiles = (g.c + CT - 1) / CT;
    const long long gy = (long long) g.in[0] * htiles;
    const long long gz = (long long) g.n * ctiles;
    const long long gw = (g.in[2] + BWD_THREADS - 1) / BWD_THREADS;
    if (gy > 0x7fffffffll || gw > 65535 || gz > 65535)
    {
        set_last_error("tensor too large for the fp32 backward-data grid");
        return DCB_UNSUPPORTED;
    }
    if (smem > 48 * 1024)
        DCB_CUDA_TRY(cudaFuncSetAttribute(conv_bwd_data_kernel<CT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int) (96 * 1024)));
    dim3 grid((unsigned) gy, (unsigned) gw, (unsigned) gz);
    conv_bwd_data_kernel<CT><<<grid, BWD_THREADS, smem, stream>>>(
        g, alpha, beta, w, dy, dx, ktile, ctiles, rows, htiles);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t simt_conv_bwd_data(const ConvGeom& g, float alpha, const float* w,
                           const float* dy, float beta, float* dx,
                           cudaStream_t stream)
{
    if ((long long) g.n * g.c * g.in[0] * g.in[1] * g.in[2] == 0)
        return DCB_OK;
    if (g.c > 8)
        return launch_bwd_data<16>(g, alpha, w, dy, beta, dx, stream);
    if (g.c > 4)
        return launch_bwd_data<8>(g, alpha, w, dy, beta, dx, stream);
    return launch_bwd_data<4>(g, alpha, w, dy, beta, dx, stream);
}

// ---------------------------------------------------------------------------
// backward filter.  A work unit is WT outputs of one output row (n, od, oh).
// The block stages that row of dy (its K slice) and the fd*fh input rows the
// row touches (its C slice) in shared memory; each thread owns KB filters x
// one (c, kd, kh) x all fw taps and keeps those sums in registers across all
// the units the block walks.  Per-block partial filters go to the workspace
// and a second kernel folds them in block order (reproducible), applying
// alpha / beta.
// ---------------------------------------------------------------------------
constexpr int BF_KB = 4;
constexpr int BF_WT = 128;
constexpr int BF_THREADS = 256;

struct BfTiling
{
    int kg_per_block; // filter groups (of KB) per block
    int c_per_block;
    int ytiles, ztiles;
    int xrow_len; // staged input row length
    int nblocks_x;
    size_t smem;
};

static BfTiling bf_tiling(const ConvGeom& g)
{
    BfTiling t;
    const int rows = g.f[0] * g.f[1];
    const int kgroups = (g.k + BF_KB - 1) / BF_KB;
    t.c_per_block = BF_THREADS / rows;
    if (t.c_per_block < 1)
        t.c_per_block = 1;
    if (t.c_per_block > g.c)
        t.c_per_block = g.c;
    t.kg_per_block = BF_THREADS / (t.c_per_block * rows);
    if (t.kg_per_block < 1)
        t.kg_per_block = 1;
    if (t.kg_per_block > kgroups)
        t.kg_per_block = kgroups;
    t.xrow_len = (BF_WT - 1) * g.stride[2] + (g.f[2] - 1) * g.dil[2] + 1;
    t.xrow_len = (t.xrow_len + 3) / 4 * 4; // rows stay 16-byte aligned for the vector loop
    // Keep shared memory within the default 48 KiB.
    while (true)
    {
        t.smem = ((size_t) t.kg_per_block * BF_KB * BF_WT
                  + (size_t) t.c_per_block * rows * t.xrow_len)
                 * sizeof(float);
        if (t.smem <= 48 * 1024 || (t.c_per_block == 1 && t.kg_per_block == 1))
            break;
        if (t.c_per_block > 1)
            t.c_per_block = (t.c_per_block + 1) / 2;
        else
            t.kg_per_block = (t.kg_per_block + 1) / 2;
    }
    t.ytiles = (kgroups + t.kg_per_block - 1) / t.kg_per_block;
    t.ztiles = (g.c + t.c_per_block - 1) / t.c_per_block;
    int per = num_sms() * 2 / (t.ytiles * t.ztiles);
    t.nblocks_x = per < 1 ? 1 : per;
    return t;
}

size_t simt_conv_bwd_filter_workspace(const ConvGeom& g)
{
    const BfTiling t = bf_tiling(g);
    const size_t fsize = (size_t) g.k * g.c * g.f[0] * g.f[1] * g.f[2];
    return (size_t) t.nblocks_x * fsize * sizeof(float);
}

template <int FW>
__global__ void __launch_bounds__(BF_THREADS)
    conv_bwd_filter_kernel(ConvGeom g, const float* __restrict__ x,
                           const float* __restrict__ dy,
                           float* __restrict__ partial, int kg_per_block,
                           int c_per_block, int xrow_len)
{
    extern __shared__ __align__(16) float sm[];
    const int rows = g.f[0] * g.f[1];
    float* sdy = sm;                                         // [kg*KB][WT]
    float* sx = sm + (size_t) kg_per_block * BF_KB * BF_WT;  // [c][rows][xrow]
    const int k_base = blockIdx.y * kg_per_block * BF_KB;
    const int c_base = blockIdx.z * c_per_block;
    const int npairs = kg_per_block * c_per_block * rows;
    const int tid = threadIdx.x;
    // pair -> (kg, cc, row); consecutive threads share kg (dy reads broadcast)
    const int row = tid % rows;
    const int cc = (tid / rows) % c_per_block;
    const int kg = tid / (rows * c_per_block);
    const bool active = tid < npairs && (c_base + cc) < g.c;

    float acc[BF_KB][FW];
#pragma unroll
    for (int i = 0; i < BF_KB; ++i)
#pragma unroll
        for (int j = 0; j < FW; ++j)
            acc[i][j] = 0.f;

    const int wchunks = (g.out[2] + BF_WT - 1) / BF_WT;
    const long long units =
        (long long) g.n * g.out[0] * g.out[1] * wchunks;
    for (long long u = blockIdx.x; u < units; u += gridDim.x)
    {
        const int wc = (int) (u % wchunks);
        long long t = u / wchunks;
        const int oh = (int) (t % g.out[1]);
        t /= g.out[1];
        const int od = (int) (t % g.out[0]);
        const int n = (int) (t / g.out[0]);
        const int ow0 = wc * BF_WT;
        const int wcount = min(BF_WT, g.out[2] - ow0);
        __syncthreads();
        // stage dy[k_base .. , ow0 ..]
        for (int idx = tid; idx < kg_per_block * BF_KB * BF_WT;
             idx += BF_THREADS)
        {
            const int wv = idx % BF_WT;
            const int kk = idx / BF_WT;
            const int k = k_base + kk;
            sdy[idx] = (k < g.k && wv < wcount)
                           ? dy[(size_t) n * g.ys_n + (size_t) k * g.ys_c
                                + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1]
                                + ow0 + wv]
                           : 0.f;
        }
        // stage the input rows, zero outside the tensor (padding)
        const int iw0 = ow0 * g.stride[2] - g.pad[2];
        for (int idx = tid; idx < c_per_block * rows * xrow_len;
             idx += BF_THREADS)
        {
            const int e = idx % xrow_len;
            const int r = (idx / xrow_len) % rows;
            const int c = c_base + idx / (xrow_len * rows);
            const int kd = r / g.f[1], kh = r % g.f[1];
            const int id = od * g.stride[0] - g.pad[0] + kd * g.dil[0];
            const int ih = oh * g.stride[1] - g.pad[1] + kh * g.dil[1];
            const int iw = iw0 + e;
            const bool ok = c < g.c && id >= 0 && id < g.in[0] && ih >= 0
                            && ih < g.in[1] && iw >= 0 && iw < g.in[2];
            sx[idx] = ok ? x[(size_t) n * g.xs_n + (size_t) c * g.xs_c
                             + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1]
                             + iw]
                         : 0.f;
        }
        __syncthreads();
        if (!active)
            continue;
        const float* dyr = sdy + (size_t) kg * BF_KB * BF_WT;
        const float* xr = sx + ((size_t) cc * rows + row) * xrow_len;
        if (g.stride[2] == 1 && g.dil[2] == 1 && FW <= 5)
        {
            // four outputs per step: one 16-byte load per filter of dy and two of
            // the input row feed 4 * KB * FW FMAs (the scalar loop below is bound
            // by its shared-memory loads).  dy is zero beyond wcount, so the
            // whole tile can be walked.
            for (int wv = 0; wv < BF_WT; wv += 4)
            {
                float4 dv[BF_KB];
#pragma unroll
                for (int i = 0; i < BF_KB; ++i)
                    dv[i] = *reinterpret_cast<const float4*>(dyr + i * BF_WT + wv);
                const float4 xa = *reinterpret_cast<const float4*>(xr + wv);
                const float4 xb = wv + 4 < xrow_len ? *reinterpret_cast<const float4*>(xr + wv + 4)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int j = 0; j < FW; ++j)
#pragma unroll
                    for (int i = 0; i < BF_KB; ++i)
                    {
                        float a = acc[i][j];
                        a = fmaf(dv[i].x, xv[j], a);
                        a = fmaf(dv[i].y, xv[j + 1], a);
                        a = fmaf(dv[i].z, xv[j + 2], a);
                        a = fmaf(dv[i].w, xv[j + 3], a);
                        acc[i][j] = a;
                    }
            }
            continue;
        }
        for (int wv = 0; wv < wcount; ++wv)
        {
            float dv[BF_KB];
#pragma unroll
            for (int i = 0; i < BF_KB; ++i)
                dv[i] = dyr[i * BF_WT + wv];
            const float* xp = xr + wv * g.stride[2];
#pragma unroll
            for (int j = 0; j < FW; ++j)
            {
                const float xv = xp[j * g.dil[2]];
#pragma unroll
                for (int i = 0; i < BF_KB; ++i)
                    acc[i][j] = fmaf(dv[i], xv, acc[i][j]);
            }
        }
    }
    if (!active)
        return;
    const int taps = rows * FW;
    const size_t fsize = (size_t) g.k * g.c * taps;
    float* out = partial + (size_t) blockIdx.x * fsize;
#pragma unroll
    for (int i = 0; i < BF_KB; ++i)
    {
        const int k = k_base + kg * BF_KB + i;
        if (k >= g.k)
            continue;
#pragma unroll
        for (int j = 0; j < FW; ++j)
            out[((size_t) k * g.c + (c_base + cc)) * taps + row * FW + j] =
                acc[i][j];
    }
}

__global__ void bwd_filter_fold_kernel(const float* __restrict__ partial,
                                       int nparts, size_t fsize, float alpha,
                                       float beta, float* dw)
{
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= fsize)
        return;
    double s = 0.0;
    for (int p = 0; p < nparts; ++p)
        s += (double) partial[(size_t) p * fsize + i];
    const float prev = beta != 0.f ? dw[i] : 0.f;
    dw[i] = alpha * (float) s + beta * prev;
}

int32_t simt_conv_bwd_filter(const ConvGeom& g, float alpha, const float* x,
                             const float* dy, float beta, float* dw,
                             float* workspace, cudaStream_t stream)
{
    const int taps = g.f[0] * g.f[1] * g.f[2];
    const size_t fsize = (size_t) g.k * g.c * taps;
    if (fsize == 0)
        return DCB_OK;
    const BfTiling t = bf_tiling(g);
    if (t.smem > 48 * 1024)
    {
        set_last_error("filter too large for the fp32 backward-filter kernel");
        return DCB_UNSUPPORTED;
    }
    dim3 grid(t.nblocks_x, t.ytiles, t.ztiles);
#define CALL(FWV)                                                              \
    conv_bwd_filter_kernel<FWV><<<grid, BF_THREADS, t.smem, stream>>>(         \
        g, x, dy, workspace, t.kg_per_block, t.c_per_block, t.xrow_len)
    switch (g.f[2])
    {
    case 1: CALL(1); break;
    case 2: CALL(2); break;
    case 3: CALL(3); break;
    case 4: CALL(4); break;
    case 5: CALL(5); break;
    case 7: CALL(7); break;
    default:
        set_last_error("filter width not in {1,2,3,4,5,7}");
        return DCB_UNSUPPORTED;
    }
#undef CALL
    DCB_LAUNCH_CHECK();
    bwd_filter_fold_kernel<<<(unsigned) ((fsize + 255) / 256), 256, 0,
                             stream>>>(workspace, t.nblocks_x, fsize, alpha,
                                       beta, dw);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

} // namespace dcb
