// Pooling on a halo-extended shard: stands in for cudnnPoolingForward /
// cudnnPoolingBackward behind GPUDNNBackend::pooling_forward / _backward as
// Pooling<BackendDNNLib, T> calls them
// (legacy/include/distconv/dnn_backend/pooling.hpp:212-283).
//
// Both passes are gathers (one thread per result cell, W fastest so that a
// warp reads and writes consecutive cells) and so are reproducible:
//
//   forward   y[o] = alpha * pool(window of o) + beta * y[o]
//   backward  dx[i] = alpha * sum over the windows o that contain i of
//                         MAX:  dy[o] if i is the first cell of o's window (scan
//                               order D, H, W) that holds the maximum, else 0
//                         AVG:  dy[o] / count(o)
//                     + beta * dx[i]
//
// Cells outside the x window are padding: ignored by MAX and by the
// count of AVERAGE_NO_PAD, zeros that count for AVERAGE.  Where a dimension is
// partitioned the caller passes pad 0 and a window that includes the halo
// cells, and the backward pass writes the halo cells of dx too; the reverse
// halo exchange with SUM then adds them to their owners
// (pooling.hpp:281, :450-467).  The halo cells of a rank at the boundary of
// the global tensor stand for padding (pooling.hpp:189-194); the reference
// hands them to cuDNN as zero data, which changes MAX and AVERAGE_NO_PAD
// against the unpartitioned result.  Here the descriptor says how many leading
// / trailing cells of the window lie outside the global tensor and those are
// padding like any other, so P ranks give what one rank gives.
//
// HBM-bound: algorithmic bytes are 4 * (|x| + |y|) forward and
// 4 * (|x| + |y| + |dy| + |dx|) backward; the window re-reads hit L1 / L2.
#include "common.cuh"
#include "dcb.h"

#include <cfloat>

namespace dcb
{
namespace
{

struct PoolGeom
{
    int n, c;
    int in[3], out[3], win[3], pad[3], stride[3];
    int lo[3], hi[3]; // real cells of the x window along each axis: [lo, hi)
    long long xs_n, xs_c, xs[3];
    long long ys_n, ys_c, ys[3];
    int mode;
};

constexpr int POOL_THREADS = 256;

__device__ __forceinline__ float pool_count(const PoolGeom& g, int od, int oh, int ow)
{
    if (g.mode == DCB_POOL_AVERAGE)
        return (float) (g.win[0] * g.win[1] * g.win[2]);
    int cnt = 1;
    const int o[3] = {od, oh, ow};
#pragma unroll
    for (int i = 0; i < 3; ++i)
    {
        const int lo = max(g.lo[i], o[i] * g.stride[i] - g.pad[i]);
        const int hi = min(g.hi[i], o[i] * g.stride[i] - g.pad[i] + g.win[i]);
        cnt *= max(0, hi - lo);
    }
    return (float) cnt;
}

// row = plane * extent + line, with the 32-bit division when the row count allows it
// (the 64-bit one is a subroutine of a hundred instructions)
__device__ __forceinline__ void pool_split_row(long long row, long long rows, int extent, int* plane, int* line)
{
    if (rows <= 0x7fffffffll)
    {
        const unsigned r = (unsigned) row, e = (unsigned) extent;
        *plane = (int) (r / e);
        *line = (int) (r - (r / e) * e);
    }
    else
    {
        *plane = (int) (row / extent);
        *line = (int) (row % extent);
    }
}

// Forward: one thread per output cell, the window scanned in D, H, W order.
// `argmax`, if given, receives the tap index kd * fh * fw + kh * fw + kw of the
// first maximum (dense [n][c][od][oh][ow]); y may then be null.
constexpr int POOL_TW = POOL_THREADS;

template <int WD, int W, int S>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_fwd_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ x, float* y,
                    unsigned char* __restrict__ argmax, int tw_log2, long long rows)
{
    // window / stride as compile-time constants where the launch found a match
    // (unrolled loops, shifts for the divisions); 0 = read them from the geometry
    const int w0_ = WD ? WD : g.win[0], w1_ = W ? W : g.win[1], w2_ = W ? W : g.win[2];
    const int s0_ = S ? (WD == 1 ? 1 : S) : g.stride[0], s1_ = S ? S : g.stride[1], s2_ = S ? S : g.stride[2];
    // a block is 256 >> tw_log2 output rows of (1 << tw_log2) cells: short rows (128
    // outputs of a 256-cell input row) would otherwise leave half the block idle
    const int ow = (blockIdx.y << tw_log2) + (threadIdx.x & ((1 << tw_log2) - 1));
    const long long row = (long long) blockIdx.x * (POOL_THREADS >> tw_log2) + (threadIdx.x >> tw_log2);
    if (ow >= g.out[2] || row >= rows)
        return;
    const int oh = (int) (row % g.out[1]), od = (int) (row / g.out[1]);
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    const float* xp = x + (size_t) n * g.xs_n + (size_t) c * g.xs_c;
    const int d0 = od * s0_ - g.pad[0], h0 = oh * s1_ - g.pad[1], w0 = ow * s2_ - g.pad[2];
    const int kw_lo = max(0, g.lo[2] - w0), kw_hi = min(w2_, g.hi[2] - w0);
    float m = -FLT_MAX, s = 0.f;
    int best = -1;
#pragma unroll
    for (int kd = 0; kd < w0_; ++kd)
    {
        const int id = d0 + kd;
        if (id < g.lo[0] || id >= g.hi[0])
            continue;
#pragma unroll
        for (int kh = 0; kh < w1_; ++kh)
        {
            const int ih = h0 + kh;
            if (ih < g.lo[1] || ih >= g.hi[1])
                continue;
            const float* row = xp + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1] + w0;
            const int tap0 = (kd * w1_ + kh) * w2_;
#pragma unroll
            for (int kw = 0; kw < w2_; ++kw)
            {
                if (kw < kw_lo || kw >= kw_hi)
                    continue;
                const float v = __ldg(row + kw);
                s += v;
                if (best < 0 || v > m)
                {
                    m = v;
                    best = tap0 + kw;
                }
            }
        }
    }
    if (argmax)
    {
        argmax[((((size_t) n * g.c + c) * g.out[0] + od) * g.out[1] + oh) * g.out[2] + ow] = (unsigned char) best;
        if (!y)
            return;
    }
    const float r = g.mode == DCB_POOL_MAX ? m : s / fmaxf(pool_count(g, od, oh, ow), 1.f);
    float* yp = y + (size_t) n * g.ys_n + (size_t) c * g.ys_c + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
    *yp = beta != 0.f ? alpha * r + beta * *yp : alpha * r;
}

// Forward for windows of 3 with stride 2 and pad 1 along W (and H; WD = 3 with stride 2
// or 1 with stride 1 along D) on rows that start on 16-byte boundaries: a thread takes
// two neighbouring outputs, i.e. input cells 4t-1 .. 4t+3 of every window row: one
// 16-byte load and the left neighbour's last cell from a shuffle, where the one-output
// kernel issues six scalar loads at every second cell.  Same scan order (D, H, W, first
// maximum wins), same arithmetic.
template <int WD>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_fwd_w3s2_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ x, float* y,
                         unsigned char* __restrict__ argmax, int tw_log2, long long rows)
{
    const int tq = (blockIdx.y << tw_log2) + (threadIdx.x & ((1 << tw_log2) - 1)); // pair of outputs
    const long long row = (long long) blockIdx.x * (POOL_THREADS >> tw_log2) + (threadIdx.x >> tw_log2);
    const bool live = 2 * tq < g.out[2] && row < rows; // dead lanes still take part in the shuffles
    int oh, od;
    pool_split_row(row, rows, g.out[1], &od, &oh);
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    const float* xp = x + (size_t) n * g.xs_n + (size_t) c * g.xs_c;
    // offsets inside one (sample, channel) volume fit 32 bits (checked at the launch)
    const int xs0 = (int) g.xs[0], xs1 = (int) g.xs[1];
    const int sd = WD == 1 ? 1 : 2;
    const int d0 = od * sd - g.pad[0], h0 = oh * 2 - g.pad[1];
    const int w4 = 4 * tq; // cells w4 - 1 .. w4 + 3
    float m[2] = {-FLT_MAX, -FLT_MAX}, s[2] = {0.f, 0.f};
    int best[2] = {-1, -1};
    const int lane = threadIdx.x & 31;
    // A warp whose windows all lie inside the real cells (every warp but those at the
    // faces) runs without range checks: tap 0 is then every window's first cell, so the
    // "first cell always becomes the maximum" rule is an assignment there and a plain
    // comparison after it.  Same results as the checked loop below.
    const bool full = live && 2 * tq + 1 < g.out[2] && d0 >= g.lo[0] && d0 + WD <= g.hi[0] && h0 >= g.lo[1]
                      && h0 + 3 <= g.hi[1] && w4 >= g.lo[2] && w4 + 3 < g.hi[2];
    const bool fast = __all_sync(0xffffffffu, full);
    // the first thread of a row: its cell w4 - 1 is the padding, tap 1 its first window's first cell
    const bool ledge = w4 - 1 < g.lo[2];
    if (fast)
    {
        const float* rp0 = xp + (d0 * xs0 + h0 * xs1 + w4);
        const bool want_max = g.mode == DCB_POOL_MAX;
#pragma unroll
        for (int kd = 0; kd < WD; ++kd)
#pragma unroll
            for (int kh = 0; kh < 3; ++kh)
            {
                const float* rp = rp0 + (kd * xs0 + kh * xs1);
                const float4 t = __ldg(reinterpret_cast<const float4*>(rp));
                float prev = __shfl_up_sync(0xffffffffu, t.w, 1);
                if (lane == 0 && !ledge)
                    prev = __ldg(rp - 1);
                const float v[5] = {prev, t.x, t.y, t.z, t.w};
                const int tap0 = (kd * 3 + kh) * 3;
                if (want_max)
                {
#pragma unroll
                    for (int o = 0; o < 2; ++o)
#pragma unroll
                        for (int kw = 0; kw < 3; ++kw)
                        {
                            const float val = v[2 * o + kw];
                            const bool row0 = kd == 0 && kh == 0;
                            bool take;
                            if (o == 0 && kw == 0)
                                take = !ledge && (row0 || val > m[o]);
                            else if (o == 0 && kw == 1 && row0)
                                take = ledge || val > m[o];
                            else
                                take = (row0 && kw == 0) || val > m[o];
                            if (take)
                            {
                                m[o] = val;
                                best[o] = tap0 + kw;
                            }
                        }
                }
                else
                {
                    s[0] += ledge ? 0.f : v[0];
                    s[0] += v[1];
                    s[0] += v[2];
#pragma unroll
                    for (int kw = 0; kw < 3; ++kw)
                        s[1] += v[2 + kw];
                }
            }
    }
#pragma unroll
    for (int kd = 0; kd < WD && !fast; ++kd)
    {
        const int id = d0 + kd;
        const bool dok = live && id >= g.lo[0] && id < g.hi[0];
#pragma unroll
        for (int kh = 0; kh < 3; ++kh)
        {
            const int ih = h0 + kh;
            const bool rok = dok && ih >= g.lo[1] && ih < g.hi[1];
            float q[4] = {0.f, 0.f, 0.f, 0.f};
            if (rok)
            {
                const float* rp = xp + (id * xs0 + ih * xs1 + w4);
                if (w4 + 3 < g.hi[2])
                {
                    const float4 t = __ldg(reinterpret_cast<const float4*>(rp));
                    q[0] = t.x;
                    q[1] = t.y;
                    q[2] = t.z;
                    q[3] = t.w;
                }
                else
                {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (w4 + e < g.hi[2])
                            q[e] = __ldg(rp + e);
                }
            }
            // cell w4 - 1: the left neighbour's q[3] (same output row: a tile is 32 lanes or more)
            float prev = __shfl_up_sync(0xffffffffu, q[3], 1);
            if (lane == 0 && rok && w4 - 1 >= g.lo[2])
                prev = __ldg(xp + (id * xs0 + ih * xs1 + w4 - 1));
            if (!rok)
                continue;
            const float v[5] = {prev, q[0], q[1], q[2], q[3]};
            const int tap0 = (kd * 3 + kh) * 3;
#pragma unroll
            for (int o = 0; o < 2; ++o)
#pragma unroll
                for (int kw = 0; kw < 3; ++kw)
                {
                    const int cell = w4 - 1 + 2 * o + kw;
                    if (cell < g.lo[2] || cell >= g.hi[2])
                        continue;
                    const float val = v[2 * o + kw];
                    s[o] += val;
                    if (best[o] < 0 || val > m[o])
                    {
                        m[o] = val;
                        best[o] = tap0 + kw;
                    }
                }
        }
    }
    if (!live)
        return;
#pragma unroll
    for (int o = 0; o < 2; ++o)
    {
        const int ow = 2 * tq + o;
        if (ow >= g.out[2])
            continue;
        if (argmax)
            argmax[((size_t) n * g.c + c) * ((size_t) g.out[0] * g.out[1] * g.out[2]) + ((od * g.out[1] + oh) * g.out[2] + ow)] =
                (unsigned char) best[o];
        if (!y)
            continue;
        const float r = g.mode == DCB_POOL_MAX ? m[o] : s[o] / fmaxf(pool_count(g, od, oh, ow), 1.f);
        float* yp =
            y + (size_t) n * g.ys_n + (size_t) c * g.ys_c + (od * (int) g.ys[0] + oh * (int) g.ys[1] + ow);
        *yp = beta != 0.f ? alpha * r + beta * *yp : alpha * r;
    }
}

// The outputs whose window holds input coordinate i: o*stride - pad <= i < o*stride - pad + win.
__device__ __forceinline__ void pool_cover(int i, int stride, int pad, int win, int nout, int* lo, int* hi)
{
    const int t = i + pad;
    const int l = t - win + 1;
    int lq, hq; // ceil(l / stride) for l > 0, floor(t / stride); strides 1 and 2 without a division
    if (stride == 1)
    {
        lq = l;
        hq = t;
    }
    else if (stride == 2)
    {
        lq = (l + 1) >> 1;
        hq = t >> 1;
    }
    else
    {
        lq = (l + stride - 1) / stride;
        hq = t / stride;
    }
    *lo = l <= 0 ? 0 : lq;
    *hi = min(hq, nout - 1);
}

template <int WD, int W, int S>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_bwd_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ y, const float* __restrict__ dy,
                    const float* __restrict__ x, float* dx, const unsigned char* __restrict__ argmax)
{
    // window / stride as compile-time constants where the launch found a match
    // (unrolled loops, shifts for the divisions); 0 = read them from the geometry
    const int w0_ = WD ? WD : g.win[0], w1_ = W ? W : g.win[1], w2_ = W ? W : g.win[2];
    const int s0_ = S ? (WD == 1 ? 1 : S) : g.stride[0], s1_ = S ? S : g.stride[1], s2_ = S ? S : g.stride[2];
    const int iw = blockIdx.y * POOL_THREADS + threadIdx.x;
    if (iw >= g.in[2])
        return;
    const int ih = blockIdx.x % g.in[1], id = blockIdx.x / g.in[1];
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    const size_t xoff = (size_t) n * g.xs_n + (size_t) c * g.xs_c;
    const size_t yoff = (size_t) n * g.ys_n + (size_t) c * g.ys_c;
    const size_t me = xoff + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1] + iw;
    int dlo, dhi, hlo, hhi, wlo, whi;
    pool_cover(id, s0_, g.pad[0], w0_, g.out[0], &dlo, &dhi);
    pool_cover(ih, s1_, g.pad[1], w1_, g.out[1], &hlo, &hhi);
    pool_cover(iw, s2_, g.pad[2], w2_, g.out[2], &wlo, &whi);
    const float xv = g.mode == DCB_POOL_MAX && !argmax ? __ldg(x + me) : 0.f;
    float acc = 0.f;
    // a cell outside the global tensor is padding: no window gives it anything
    const bool real = id >= g.lo[0] && id < g.hi[0] && ih >= g.lo[1] && ih < g.hi[1] && iw >= g.lo[2] && iw < g.hi[2];
    if (!real)
        dhi = dlo - 1;
    if (argmax)
    {
        // the index pass recorded every window's first maximum: one byte to compare
        const size_t plane = ((size_t) n * g.c + c) * g.out[0];
        for (int od = dlo; od <= dhi; ++od)
            for (int oh = hlo; oh <= hhi; ++oh)
            {
                const size_t drow = ((plane + od) * g.out[1] + oh) * g.out[2];
                const float* dyrow = dy + yoff + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1];
                const int tap0 = ((id - (od * s0_ - g.pad[0])) * w1_ + (ih - (oh * s1_ - g.pad[1])))
                                 * w2_;
                for (int ow = wlo; ow <= whi; ++ow)
                    if ((int) __ldg(argmax + drow + ow) == tap0 + iw - (ow * s2_ - g.pad[2]))
                        acc += __ldg(dyrow + ow);
            }
        dlo = dhi + 1;
    }
    for (int od = dlo; od <= dhi; ++od)
        for (int oh = hlo; oh <= hhi; ++oh)
            for (int ow = wlo; ow <= whi; ++ow)
            {
                const size_t o = yoff + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
                if (g.mode != DCB_POOL_MAX)
                {
                    acc += __ldg(dy + o) / fmaxf(pool_count(g, od, oh, ow), 1.f);
                    continue;
                }
                if (__ldg(y + o) != xv)
                    continue;
                // the maximum goes to the first cell that holds it: is one before me?
                bool first = true;
                const int d0 = od * s0_ - g.pad[0], h0 = oh * s1_ - g.pad[1],
                          w0 = ow * s2_ - g.pad[2];
                for (int jd = max(d0, g.lo[0]); jd <= id && first; ++jd)
                    for (int jh = max(h0, g.lo[1]); jh < min(h0 + w1_, g.hi[1]) && first; ++jh)
                    {
                        if (jd == id && jh > ih)
                            break;
                        const float* row = x + xoff + (size_t) jd * g.xs[0] + (size_t) jh * g.xs[1];
                        const int wend = (jd == id && jh == ih) ? iw : min(w0 + w2_, g.hi[2]);
                        for (int jw = max(w0, g.lo[2]); jw < wend; ++jw)
                            if (__ldg(row + jw) == xv)
                            {
                                first = false;
                                break;
                            }
                    }
                if (first)
                    acc += __ldg(dy + o);
            }
    dx[me] = beta != 0.f ? alpha * acc + beta * dx[me] : alpha * acc;
}

// MAX backward with the index workspace: a thread owns four consecutive cells of
// an input row, walks the (od, oh) pairs whose windows hold the row once for all
// four, and compares one byte per (cell, window).  Every instruction here is
// paid 268 M times on the bench shard: the per-cell version spent 430 per cell.
template <int WD, int W, int S>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_bwd_index_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ dy, float* dx,
                          const unsigned char* __restrict__ argmax)
{
    const int w0_ = WD ? WD : g.win[0], w1_ = W ? W : g.win[1], w2_ = W ? W : g.win[2];
    const int s0_ = S ? (WD == 1 ? 1 : S) : g.stride[0], s1_ = S ? S : g.stride[1], s2_ = S ? S : g.stride[2];
    const int iw0 = (blockIdx.y * POOL_THREADS + threadIdx.x) * 4;
    if (iw0 >= g.in[2])
        return;
    const int ih = blockIdx.x % g.in[1], id = blockIdx.x / g.in[1];
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int dlo, dhi, hlo, hhi;
    pool_cover(id, s0_, g.pad[0], w0_, g.out[0], &dlo, &dhi);
    pool_cover(ih, s1_, g.pad[1], w1_, g.out[1], &hlo, &hhi);
    if (id < g.lo[0] || id >= g.hi[0] || ih < g.lo[1] || ih >= g.hi[1])
        dhi = dlo - 1; // a row outside the global tensor is padding
    int wlo[4], whi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
    {
        pool_cover(iw0 + e, s2_, g.pad[2], w2_, g.out[2], &wlo[e], &whi[e]);
        if (iw0 + e < g.lo[2] || iw0 + e >= g.hi[2] || iw0 + e >= g.in[2])
            whi[e] = wlo[e] - 1;
    }
    const size_t plane = ((size_t) n * g.c + c) * g.out[0];
    const float* dyp = dy + (size_t) n * g.ys_n + (size_t) c * g.ys_c;
    for (int od = dlo; od <= dhi; ++od)
        for (int oh = hlo; oh <= hhi; ++oh)
        {
            const unsigned char* arow = argmax + ((plane + od) * g.out[1] + oh) * g.out[2];
            const float* dyrow = dyp + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1];
            const int tap0 = ((id - (od * s0_ - g.pad[0])) * w1_ + (ih - (oh * s1_ - g.pad[1]))) * w2_ + g.pad[2] + iw0;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                for (int ow = wlo[e]; ow <= whi[e]; ++ow)
                    if ((int) __ldg(arow + ow) == tap0 + e - ow * s2_)
                        acc[e] += __ldg(dyrow + ow);
        }
    float* xp = dx + (size_t) n * g.xs_n + (size_t) c * g.xs_c + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1] + iw0;
    if (iw0 + 4 <= g.in[2] && (reinterpret_cast<uintptr_t>(xp) & 15) == 0)
    {
        float4 o = make_float4(alpha * acc[0], alpha * acc[1], alpha * acc[2], alpha * acc[3]);
        if (beta != 0.f)
        {
            const float4 old = *reinterpret_cast<const float4*>(xp);
            o.x += beta * old.x;
            o.y += beta * old.y;
            o.z += beta * old.z;
            o.w += beta * old.w;
        }
        *reinterpret_cast<float4*>(xp) = o;
    }
    else
    {
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (iw0 + e < g.in[2])
                xp[e] = beta != 0.f ? alpha * acc[e] + beta * xp[e] : alpha * acc[e];
    }
}

// The same for windows of 3 with stride 2 and pad 1 along W (3 / stride 2 along H; WD = 3
// with stride 2 or 1 with stride 1 along D) and an even output row: cells 4t .. 4t+3 lie
// in the windows of outputs 2t, 2t+1 and 2t+2 only, so a thread loads two index bytes
// and two gradients in one access each and takes the third pair from its right-hand
// neighbour's registers; short rows share a block as in the forward kernel.  The sums
// run in the same order (D, H, then W ascending) as in the kernel above: same bits.
template <int WD>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_bwd_index_w3s2_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ dy, float* dx,
                               const unsigned char* __restrict__ argmax, int tw_log2, long long rows)
{
    const int t = (blockIdx.y << tw_log2) + (threadIdx.x & ((1 << tw_log2) - 1));
    const long long row = (long long) blockIdx.x * (POOL_THREADS >> tw_log2) + (threadIdx.x >> tw_log2);
    if (row >= rows) // a warp never spans two rows: the whole warp leaves
        return;
    const int iw0 = 4 * t, ow0 = 2 * t;
    int ih, id;
    pool_split_row(row, rows, g.in[1], &id, &ih);
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    const int sd = WD == 1 ? 1 : 2;
    int dlo, dhi, hlo, hhi;
    pool_cover(id, sd, g.pad[0], WD, g.out[0], &dlo, &dhi);
    pool_cover(ih, 2, g.pad[1], 3, g.out[1], &hlo, &hhi);
    if (id < g.lo[0] || id >= g.hi[0] || ih < g.lo[1] || ih >= g.hi[1])
        dhi = dlo - 1; // a row outside the global tensor is padding
    const int lane = threadIdx.x & 31;
    // offsets inside one (sample, channel) volume fit 32 bits (checked at the launch)
    const int ys0 = (int) g.ys[0], ys1 = (int) g.ys[1], astep = g.out[1] * g.out[2];
    const unsigned char* abase =
        argmax + ((size_t) n * g.c + c) * ((size_t) g.out[0] * astep) + ((dlo * g.out[1] + hlo) * g.out[2] + ow0);
    const float* dbase = dy + (size_t) n * g.ys_n + (size_t) c * g.ys_c + (dlo * ys0 + hlo * ys1 + ow0);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool two = ow0 + 1 < g.out[2], third = ow0 + 2 < g.out[2];
    // at most two output planes and two output rows hold this input row: all their loads
    // are issued before the first is used (which of the four exist is the same for the
    // whole warp)
    constexpr int JD = WD == 1 ? 1 : 2;
    int a0[JD * 2], a1[JD * 2];
    float d0[JD * 2], d1[JD * 2];
#pragma unroll
    for (int jd = 0; jd < JD; ++jd)
#pragma unroll
        for (int jh = 0; jh < 2; ++jh)
        {
            const int k = jd * 2 + jh;
            // 255 is the index pass's "empty window" and never a tap
            a0[k] = a1[k] = 255;
            d0[k] = d1[k] = 0.f;
            if (dlo + jd <= dhi && hlo + jh <= hhi && two)
            {
                const uchar2 a = __ldg(reinterpret_cast<const uchar2*>(abase + (jd * astep + jh * g.out[2])));
                const float2 d = __ldg(reinterpret_cast<const float2*>(dbase + (jd * ys0 + jh * ys1)));
                a0[k] = a.x;
                a1[k] = a.y;
                d0[k] = d.x;
                d1[k] = d.y;
            }
        }
#pragma unroll
    for (int jd = 0; jd < JD; ++jd)
#pragma unroll
        for (int jh = 0; jh < 2; ++jh)
        {
            const int k = jd * 2 + jh;
            const int od = dlo + jd, oh = hlo + jh;
            if (od > dhi || oh > hhi)
                continue;
            int a2 = __shfl_down_sync(0xffffffffu, a0[k], 1);
            float d2 = __shfl_down_sync(0xffffffffu, d0[k], 1);
            if (lane == 31)
            {
                a2 = third ? (int) __ldg(abase + (jd * astep + jh * g.out[2] + 2)) : 255;
                d2 = third ? __ldg(dbase + (jd * ys0 + jh * ys1 + 2)) : 0.f;
            }
            // tap of window (od, oh, ow) at cell i: tb + i - (2 ow - 1)
            const int tb = ((id - (od * sd - g.pad[0])) * 3 + (ih - (oh * 2 - g.pad[1]))) * 3;
            if (a0[k] == tb + 1)
                acc[0] += d0[k];
            if (a0[k] == tb + 2)
                acc[1] += d0[k];
            if (a1[k] == tb)
                acc[1] += d1[k];
            if (a1[k] == tb + 1)
                acc[2] += d1[k];
            if (a1[k] == tb + 2)
                acc[3] += d1[k];
            if (a2 == tb)
                acc[3] += d2;
        }
    if (iw0 >= g.in[2])
        return;
    float* xp = dx + (size_t) n * g.xs_n + (size_t) c * g.xs_c + (id * (int) g.xs[0] + ih * (int) g.xs[1] + iw0);
    if (iw0 + 4 <= g.in[2] && (reinterpret_cast<uintptr_t>(xp) & 15) == 0)
    {
        float4 o = make_float4(alpha * acc[0], alpha * acc[1], alpha * acc[2], alpha * acc[3]);
        if (beta != 0.f)
        {
            const float4 old = *reinterpret_cast<const float4*>(xp);
            o.x += beta * old.x;
            o.y += beta * old.y;
            o.z += beta * old.z;
            o.w += beta * old.w;
        }
        *reinterpret_cast<float4*>(xp) = o;
    }
    else
    {
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (iw0 + e < g.in[2])
                xp[e] = beta != 0.f ? alpha * acc[e] + beta * xp[e] : alpha * acc[e];
    }
}

// The same gather with pad 1 along H (and D, for WD = 3) as well: a thread owns the four
// cells in each row of a 2 x 2 block of input rows (planes 2p, 2p+1 x rows 2q, 2q+1; one
// plane for WD = 1).  Those rows lie in the windows of output planes p, p+1 and output
// rows q, q+1 only, at fixed taps (row 2q is tap 1 of window q; row 2q+1 tap 2 of
// window q and tap 0 of window q+1), so the index bytes and gradients of the 2 x 2
// window rows are loaded once for sixteen cells and every comparison is against a
// constant.  Cells outside the global tensor never were a window's maximum, so they
// need no mask.  Per cell the sums run in the same order (D, H, then W ascending).
template <int WD>
__global__ void __launch_bounds__(POOL_THREADS)
    pool_bwd_index_block_kernel(PoolGeom g, float alpha, float beta, const float* __restrict__ dy, float* dx,
                                const unsigned char* __restrict__ argmax, int tw_log2, int blocks_h, long long rows)
{
    constexpr int JD = WD == 1 ? 1 : 2;
    const int t = (blockIdx.y << tw_log2) + (threadIdx.x & ((1 << tw_log2) - 1));
    const long long row = (long long) blockIdx.x * (POOL_THREADS >> tw_log2) + (threadIdx.x >> tw_log2);
    if (row >= rows) // a warp never spans two row blocks: the whole warp leaves
        return;
    const int iw0 = 4 * t, ow0 = 2 * t;
    int p, q;
    pool_split_row(row, rows, blocks_h, &p, &q);
    const int c = blockIdx.z % g.c, n = blockIdx.z / g.c;
    const int lane = threadIdx.x & 31;
    // offsets inside one (sample, channel) volume fit 32 bits (checked at the launch)
    const int ys0 = (int) g.ys[0], ys1 = (int) g.ys[1], astep = g.out[1] * g.out[2];
    const unsigned char* abase =
        argmax + ((size_t) n * g.c + c) * ((size_t) g.out[0] * astep) + ((p * g.out[1] + q) * g.out[2] + ow0);
    const float* dbase = dy + (size_t) n * g.ys_n + (size_t) c * g.ys_c + (p * ys0 + q * ys1 + ow0);
    const bool two = ow0 + 1 < g.out[2], third = ow0 + 2 < g.out[2];
    // window rows (p + jd, q + jh): which exist is the same for the whole warp
    int a0[JD * 2], a1[JD * 2], a2[JD * 2];
    float d0[JD * 2], d1[JD * 2], d2[JD * 2];
#pragma unroll
    for (int jd = 0; jd < JD; ++jd)
#pragma unroll
        for (int jh = 0; jh < 2; ++jh)
        {
            const int k = jd * 2 + jh;
            // 255 is the index pass's "empty window" and never a tap
            a0[k] = a1[k] = 255;
            d0[k] = d1[k] = 0.f;
            if (p + jd < g.out[0] && q + jh < g.out[1] && two)
            {
                const uchar2 a = __ldg(reinterpret_cast<const uchar2*>(abase + (jd * astep + jh * g.out[2])));
                const float2 d = __ldg(reinterpret_cast<const float2*>(dbase + (jd * ys0 + jh * ys1)));
                a0[k] = a.x;
                a1[k] = a.y;
                d0[k] = d.x;
                d1[k] = d.y;
            }
        }
#pragma unroll
    for (int jd = 0; jd < JD; ++jd)
#pragma unroll
        for (int jh = 0; jh < 2; ++jh)
        {
            const int k = jd * 2 + jh;
            a2[k] = __shfl_down_sync(0xffffffffu, a0[k], 1);
            d2[k] = __shfl_down_sync(0xffffffffu, d0[k], 1);
            if (lane == 31)
            {
                const bool in = third && p + jd < g.out[0] && q + jh < g.out[1];
                a2[k] = in ? (int) __ldg(abase + (jd * astep + jh * g.out[2] + 2)) : 255;
                d2[k] = in ? __ldg(dbase + (jd * ys0 + jh * ys1 + 2)) : 0.f;
            }
        }
    if (iw0 >= g.in[2])
        return;
    float* xbase = dx + (size_t) n * g.xs_n + (size_t) c * g.xs_c;
    const int xs0 = (int) g.xs[0], xs1 = (int) g.xs[1];
#pragma unroll
    for (int pa = 0; pa < JD; ++pa)
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
        {
            const int id = JD == 2 ? 2 * p + pa : p, ih = 2 * q + rb;
            if (id >= g.in[0] || ih >= g.in[1])
                continue;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int jd = 0; jd < JD; ++jd)
#pragma unroll
                for (int jh = 0; jh < 2; ++jh)
                {
                    // tap of input (plane pa, row rb) in window (jd, jh): coordinate - (2 * window - 1)
                    const int kd = JD == 2 ? pa - 2 * jd + 1 : 0, kh = rb - 2 * jh + 1;
                    if (kd < 0 || kd > 2 || kh < 0 || kh > 2)
                        continue;
                    const int k = jd * 2 + jh;
                    const int tb = (kd * 3 + kh) * 3; // tap at cell i of window ow: tb + i - (2 ow - 1)
                    if (a0[k] == tb + 1)
                        acc[0] += d0[k];
                    if (a0[k] == tb + 2)
                        acc[1] += d0[k];
                    if (a1[k] == tb)
                        acc[1] += d1[k];
                    if (a1[k] == tb + 1)
                        acc[2] += d1[k];
                    if (a1[k] == tb + 2)
                        acc[3] += d1[k];
                    if (a2[k] == tb)
                        acc[3] += d2[k];
                }
            float* xp = xbase + (id * xs0 + ih * xs1 + iw0);
            if (iw0 + 4 <= g.in[2] && (reinterpret_cast<uintptr_t>(xp) & 15) == 0)
            {
                float4 o = make_float4(alpha * acc[0], alpha * acc[1], alpha * acc[2], alpha * acc[3]);
                if (beta != 0.f)
                {
                    const float4 old = *reinterpret_cast<const float4*>(xp);
                    o.x += beta * old.x;
                    o.y += beta * old.y;
                    o.z += beta * old.z;
                    o.w += beta * old.w;
                }
                *reinterpret_cast<float4*>(xp) = o;
            }
            else
            {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (iw0 + e < g.in[2])
                        xp[e] = beta != 0.f ? alpha * acc[e] + beta * xp[e] : alpha * acc[e];
            }
        }
}

int32_t pool_geom(const dcb_pool_desc* pd, const dcb_nd_desc* xd, const dcb_nd_desc* yd, PoolGeom* g)
{
    DCB_REQUIRE(pd && xd && yd, "null descriptor");
    DCB_REQUIRE(pd->nsd == 2 || pd->nsd == 3, "nsd must be 2 or 3");
    DCB_REQUIRE(xd->nsd == pd->nsd && yd->nsd == pd->nsd, "descriptor ranks do not match");
    DCB_REQUIRE(pd->mode == DCB_POOL_MAX || pd->mode == DCB_POOL_AVERAGE || pd->mode == DCB_POOL_AVERAGE_NO_PAD,
                "unknown pooling mode");
    DCB_REQUIRE(xd->n == yd->n && xd->c == yd->c, "sample / channel counts do not match");
    DCB_REQUIRE(xd->n >= 0 && xd->c >= 0 && xd->n * xd->c < (1ll << 31), "too many (n, c) planes");
    g->n = (int) xd->n;
    g->c = (int) xd->c;
    g->mode = pd->mode;
    for (int i = 0; i < 3; ++i)
    {
        DCB_REQUIRE(pd->window[i] >= 1 && pd->strides[i] >= 1 && pd->pads[i] >= 0, "bad window / stride / pad");
        DCB_REQUIRE(pd->pads[i] < pd->window[i], "a window entirely inside the padding");
        DCB_REQUIRE(xd->dims[i] < (1ll << 30) && yd->dims[i] < (1ll << 30), "extent too large");
        const long long span = xd->dims[i] + 2ll * pd->pads[i] - pd->window[i];
        DCB_REQUIRE(yd->dims[i] == (span < 0 ? 0 : span / pd->strides[i] + 1),
                    "output extent does not match input, pad, stride, window");
        g->in[i] = (int) xd->dims[i];
        g->out[i] = (int) yd->dims[i];
        g->win[i] = pd->window[i];
        g->pad[i] = pd->pads[i];
        g->stride[i] = pd->strides[i];
        g->xs[i] = xd->strides[i];
        g->ys[i] = yd->strides[i];
        DCB_REQUIRE(pd->outside_lo[i] >= 0 && pd->outside_hi[i] >= 0
                        && pd->outside_lo[i] + pd->outside_hi[i] <= xd->dims[i],
                    "outside_lo / outside_hi exceed the window");
        DCB_REQUIRE(pd->outside_lo[i] < pd->window[i] && pd->outside_hi[i] < pd->window[i],
                    "a window entirely inside the padding");
        g->lo[i] = pd->outside_lo[i];
        g->hi[i] = (int) xd->dims[i] - pd->outside_hi[i];
    }
    if (pd->nsd == 2)
        DCB_REQUIRE(pd->window[0] == 1 && pd->pads[0] == 0 && pd->strides[0] == 1, "slot 0 must be trivial for 2-D");
    DCB_REQUIRE(xd->strides[2] == 1 || xd->dims[2] <= 1, "W must be unit-stride");
    DCB_REQUIRE(yd->strides[2] == 1 || yd->dims[2] <= 1, "W must be unit-stride");
    g->xs_n = xd->sn;
    g->xs_c = xd->sc;
    g->ys_n = yd->sn;
    g->ys_c = yd->sc;
    return DCB_OK;
}

// grid.x carries (plane, row), the large product; grid.z (sample, channel)
bool pool_grid(int w, long long rows, long long planes, dim3* grid)
{
    const long long wt = (w + POOL_THREADS - 1) / POOL_THREADS;
    if (rows > 0x7fffffffll || wt > 65535 || planes > 65535)
        return false;
    *grid = dim3((unsigned) rows, (unsigned) wt, (unsigned) planes);
    return true;
}

// Picks the kernel instance whose compile-time window and stride match: cubic
// (or, for 2-D, square with a unit D slot) windows of 3 with stride 1 or 2 and of 2
// with stride 2; anything else runs the generic instance.
#define DCB_POOL_DISPATCH(g)                                                                                          \
    do                                                                                                                \
    {                                                                                                                 \
        const int w_ = (g).win[2], s_ = (g).stride[2];                                                               \
        const bool sq_ = (g).win[1] == w_ && (g).stride[1] == s_;                                                    \
        const bool flat_ = (g).win[0] == 1 && (g).stride[0] == 1;                                                    \
        const bool cube_ = (g).win[0] == w_ && (g).stride[0] == s_;                                                  \
        if (sq_ && cube_ && w_ == 3 && s_ == 2)                                                                       \
            DCB_POOL_CALL(3, 3, 2);                                                                                   \
        else if (sq_ && cube_ && w_ == 3 && s_ == 1)                                                                  \
            DCB_POOL_CALL(3, 3, 1);                                                                                   \
        else if (sq_ && cube_ && w_ == 2 && s_ == 2)                                                                  \
            DCB_POOL_CALL(2, 2, 2);                                                                                   \
        else if (sq_ && flat_ && w_ == 3 && s_ == 2)                                                                  \
            DCB_POOL_CALL(1, 3, 2);                                                                                   \
        else if (sq_ && flat_ && w_ == 3 && s_ == 1)                                                                  \
            DCB_POOL_CALL(1, 3, 1);                                                                                   \
        else if (sq_ && flat_ && w_ == 2 && s_ == 2)                                                                  \
            DCB_POOL_CALL(1, 2, 2);                                                                                   \
        else                                                                                                          \
            DCB_POOL_CALL(0, 0, 0);                                                                                   \
    } while (0)

int32_t launch_pool_fwd(const PoolGeom& g, float alpha, float beta, const float* x, float* y, unsigned char* argmax,
                        cudaStream_t stream)
{
    // the two-outputs-per-thread kernel: window 3, stride 2, pad 1 along W and H, the same or
    // a unit slot along D, input rows on 16-byte boundaries
    const bool flat = g.win[0] == 1 && g.stride[0] == 1;
    const bool cube = g.win[0] == 3 && g.stride[0] == 2;
    const bool pair = g.win[2] == 3 && g.stride[2] == 2 && g.pad[2] == 1 && g.win[1] == 3 && g.stride[1] == 2
                      && (flat || cube) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && g.xs[0] % 4 == 0
                      && g.xs[1] % 4 == 0 && g.xs_c % 4 == 0 && g.xs_n % 4 == 0 && g.out[2] >= 2
                      && (long long) g.out[0] * g.out[1] * g.out[2] < (1ll << 31)
                      && (g.out[0] - 1) * g.ys[0] + (g.out[1] - 1) * g.ys[1] + g.out[2] < (1ll << 31)
                      && (g.in[0] - 1) * g.xs[0] + (g.in[1] - 1) * g.xs[1] + g.in[2] < (1ll << 31);
    const int wcells = pair ? (g.out[2] + 1) / 2 : g.out[2]; // threads a row needs
    int tw_log2 = 8; // threads of a row per block: 32, 64, 128 or 256
    while (tw_log2 > 5 && (1 << (tw_log2 - 1)) >= wcells)
        --tw_log2;
    const long long tiles = (wcells + (1 << tw_log2) - 1) >> tw_log2;
    const long long rows = (long long) g.out[0] * g.out[1], planes = (long long) g.n * g.c;
    const long long rpb = POOL_THREADS >> tw_log2;
    const long long gx = (rows + rpb - 1) / rpb;
    if (gx > 0x7fffffffll || tiles > 65535 || planes > 65535)
    {
        set_last_error("tensor too large for the pooling grid");
        return DCB_UNSUPPORTED;
    }
    const dim3 grid((unsigned) gx, (unsigned) tiles, (unsigned) planes);
    if (pair)
    {
        if (cube)
            pool_fwd_w3s2_kernel<3><<<grid, POOL_THREADS, 0, stream>>>(g, alpha, beta, x, y, argmax, tw_log2, rows);
        else
            pool_fwd_w3s2_kernel<1><<<grid, POOL_THREADS, 0, stream>>>(g, alpha, beta, x, y, argmax, tw_log2, rows);
        DCB_LAUNCH_CHECK();
        return DCB_OK;
    }
#define DCB_POOL_CALL(WD, W, S)                                                                                        \
    pool_fwd_kernel<WD, W, S><<<grid, POOL_THREADS, 0, stream>>>(g, alpha, beta, x, y, argmax, tw_log2, rows)
    DCB_POOL_DISPATCH(g);
#undef DCB_POOL_CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

} // namespace
} // namespace dcb

using namespace dcb;

extern "C" int32_t dcb_pool_fwd(const dcb_pool_desc* pd, const dcb_nd_desc* xd, const dcb_nd_desc* yd, double alpha,
                                const void* x, double beta, void* y, void* stream)
{
    PoolGeom g;
    const int32_t st = pool_geom(pd, xd, yd, &g);
    if (st != DCB_OK)
        return st;
    if ((long long) g.n * g.c * g.out[0] * g.out[1] * g.out[2] == 0)
        return DCB_OK;
    DCB_REQUIRE(x && y, "null argument");
    return launch_pool_fwd(g, (float) alpha, (float) beta, static_cast<const float*>(x), static_cast<float*>(y),
                           nullptr, as_stream(stream));
}

extern "C" int64_t dcb_pool_bwd_workspace_bytes(const dcb_pool_desc* pd, const dcb_nd_desc* xd, const dcb_nd_desc* yd)
{
    PoolGeom g;
    if (pool_geom(pd, xd, yd, &g) != DCB_OK)
        return -1;
    if (g.mode != DCB_POOL_MAX || g.win[0] * g.win[1] * g.win[2] > 255)
        return 0;
    return (int64_t) g.n * g.c * g.out[0] * g.out[1] * g.out[2];
}

extern "C" int32_t dcb_pool_bwd(const dcb_pool_desc* pd, const dcb_nd_desc* xd, const dcb_nd_desc* yd, double alpha,
                                const void* y, const void* dy, const void* x, double beta, void* dx, void* workspace,
                                int64_t workspace_bytes, void* stream)
{
    PoolGeom g;
    const int32_t st = pool_geom(pd, xd, yd, &g);
    if (st != DCB_OK)
        return st;
    if ((long long) g.n * g.c * g.in[0] * g.in[1] * g.in[2] == 0)
        return DCB_OK;
    DCB_REQUIRE(dy && dx && (pd->mode != DCB_POOL_MAX || (x && y)), "null argument");
    dim3 grid;
    if (!pool_grid(g.in[2], (long long) g.in[0] * g.in[1], (long long) g.n * g.c, &grid))
    {
        set_last_error("tensor too large for the pooling grid");
        return DCB_UNSUPPORTED;
    }
    // With a workspace the position of every window's first maximum is worked out
    // first, by the forward kernel's separable pass (from x alone: nothing is kept
    // between calls), and the gather compares one byte per window instead of
    // scanning the window's earlier cells.
    const unsigned char* idx = nullptr;
    const int64_t need = dcb_pool_bwd_workspace_bytes(pd, xd, yd);
    if (g.mode == DCB_POOL_MAX && workspace && need > 0 && workspace_bytes >= need
        && (long long) g.n * g.c * g.out[0] * g.out[1] * g.out[2] > 0)
    {
        const int32_t st2 =
            launch_pool_fwd(g, 1.f, 0.f, static_cast<const float*>(x), nullptr, static_cast<unsigned char*>(workspace),
                            as_stream(stream));
        if (st2 != DCB_OK)
            return st2;
        idx = static_cast<const unsigned char*>(workspace);
    }
    const bool flat = g.win[0] == 1 && g.stride[0] == 1;
    const bool cube = g.win[0] == 3 && g.stride[0] == 2;
    const bool even = g.ys[0] % 2 == 0 && g.ys[1] % 2 == 0 && g.ys_c % 2 == 0 && g.ys_n % 2 == 0 && g.out[2] % 2 == 0
                      && (reinterpret_cast<uintptr_t>(dy) & 7) == 0 && (reinterpret_cast<uintptr_t>(idx) & 1) == 0;
    // offsets inside one (sample, channel) volume as 32-bit integers
    const bool small = (long long) g.out[0] * g.out[1] * g.out[2] < (1ll << 31)
                       && (g.out[0] - 1) * g.ys[0] + (g.out[1] - 1) * g.ys[1] + g.out[2] < (1ll << 31)
                       && (g.in[0] - 1) * g.xs[0] + (g.in[1] - 1) * g.xs[1] + g.in[2] < (1ll << 31);
    if (idx && g.win[2] == 3 && g.stride[2] == 2 && g.pad[2] == 1 && g.win[1] == 3 && g.stride[1] == 2
        && (flat || cube) && even && small)
    {
        const int wcells = (g.in[2] + 3) / 4; // threads a row needs
        int tw_log2 = 8;
        while (tw_log2 > 5 && (1 << (tw_log2 - 1)) >= wcells)
            --tw_log2;
        const long long tiles = (wcells + (1 << tw_log2) - 1) >> tw_log2;
        const long long rpb = POOL_THREADS >> tw_log2;
        // pad 1 along H (and D): a thread takes a 2 x 2 block of rows
        const bool block = g.pad[1] == 1 && (cube ? g.pad[0] == 1 : g.pad[0] == 0);
        if (block && tiles <= 65535)
        {
            const int blocks_h = (g.in[1] + 1) / 2;
            const long long brows = (long long) (cube ? (g.in[0] + 1) / 2 : g.in[0]) * blocks_h;
            const long long bgx = (brows + rpb - 1) / rpb;
            const dim3 gridb((unsigned) bgx, (unsigned) tiles, grid.z);
            if (cube)
                pool_bwd_index_block_kernel<3><<<gridb, POOL_THREADS, 0, as_stream(stream)>>>(
                    g, (float) alpha, (float) beta, static_cast<const float*>(dy), static_cast<float*>(dx), idx,
                    tw_log2, blocks_h, brows);
            else
                pool_bwd_index_block_kernel<1><<<gridb, POOL_THREADS, 0, as_stream(stream)>>>(
                    g, (float) alpha, (float) beta, static_cast<const float*>(dy), static_cast<float*>(dx), idx,
                    tw_log2, blocks_h, brows);
            DCB_LAUNCH_CHECK();
            return DCB_OK;
        }
        const long long rows = (long long) g.in[0] * g.in[1];
        const long long gx = (rows + rpb - 1) / rpb;
        if (gx <= 0x7fffffffll && tiles <= 65535)
        {
            const dim3 gridp((unsigned) gx, (unsigned) tiles, grid.z);
            if (cube)
                pool_bwd_index_w3s2_kernel<3><<<gridp, POOL_THREADS, 0, as_stream(stream)>>>(
                    g, (float) alpha, (float) beta, static_cast<const float*>(dy), static_cast<float*>(dx), idx,
                    tw_log2, rows);
            else
                pool_bwd_index_w3s2_kernel<1><<<gridp, POOL_THREADS, 0, as_stream(stream)>>>(
                    g, (float) alpha, (float) beta, static_cast<const float*>(dy), static_cast<float*>(dx), idx,
                    tw_log2, rows);
            DCB_LAUNCH_CHECK();
            return DCB_OK;
        }
    }
    if (idx)
    {
        const dim3 grid4(grid.x, (unsigned) ((g.in[2] + 4 * POOL_THREADS - 1) / (4 * POOL_THREADS)), grid.z);
#define DCB_POOL_CALL(WD, W, S)                                                                                       \
    pool_bwd_index_kernel<WD, W, S><<<grid4, POOL_THREADS, 0, as_stream(stream)>>>(                                  \
        g, (float) alpha, (float) beta, static_cast<const float*>(dy), static_cast<float*>(dx), idx)
        DCB_POOL_DISPATCH(g);
#undef DCB_POOL_CALL
        DCB_LAUNCH_CHECK();
        return DCB_OK;
    }
#define DCB_POOL_CALL(WD, W, S)                                                                                       \
    pool_bwd_kernel<WD, W, S><<<grid, POOL_THREADS, 0, as_stream(stream)>>>(                                         \
        g, (float) alpha, (float) beta, static_cast<const float*>(y), static_cast<const float*>(dy),                  \
        static_cast<const float*>(x), static_cast<float*>(dx), idx)
    DCB_POOL_DISPATCH(g);
#undef DCB_POOL_CALL
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}
