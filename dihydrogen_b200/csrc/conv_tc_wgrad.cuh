// tcgen05 / TMEM backward filter (strides 1 or 2, dilation 1, c*fd*fh*fw <= 128
// filter taps per output filter, K <= 16 per launch):
//
//   dw[k][c][kd][kh][kw] = sum over (n, od, oh, ow) dy[n][k][od][oh][ow] *
//                          x[n][c][od*sd+kd-pd][oh*sh+kh-ph][ow*sw+kw-pw]
//
// (written below for unit strides; with stride 2 along W a unit's input rows
// arrive as two half windows of the same shape, outputs 0..63 read the first
// and 64..127 the second, at every second cell)
//
// GEMM view: the reduction runs over the outputs, eight consecutive ow per
// MMA (the K of a TF32 instruction).  M = the (c, kd, kh, kw) taps (up to 128
// rows = TMEM lanes), N = the filters.  For one chunk of eight outputs
//   A[m][kk] = x[c][od+kd-pd][oh+kh-ph][ow0 + kk + kw-pw]     (tensor memory)
//   B[kk][k] = dy[k][od][oh][ow0 + kk]                        (shared memory)
// and the accumulator D[m][k] stays in tensor memory: two buffers, swapped every
// WG_FLUSH_UNITS units; four dump warps add the idle one into fp64 registers and
// zero it.  When the CTA has walked all its units it writes its 128 x 16 partial
// filter, and a second kernel folds the partials in CTA order (fp64) and applies
// alpha / beta.
//
// 3xTF32: D[:, 0:32] += A_hi x [B_hi | B_lo] (one instruction, N = 32) and
// D[:, 0:16] += A_lo x B_hi (N = 16); the fold adds the two column halves.
//
// A unit is 128 outputs of one output row: 8 chunks of two k-steps.  Warp 15 copies the
// fd * fh input rows (all channels, 4 cells of margin left and right, zeros
// outside the tensor = the padding) and the dy row (all filters) of the next
// unit into a two-deep shared-memory ring with bulk tensor copies.  Warps 0..11
// are three converter groups: group g takes every third chunk, lane m of its
// four warps writes row m of A (hi and lo parts) into the group's A slot and the
// group writes the chunk's B tile; warps 12..14 issue, issuer g for group g.
// All waits are bounded.
#pragma once

#include "conv_tc_kernel.cuh"

namespace dcb
{
namespace
{

// A group's chunks go round its WG_SPG slots, and each slot has an issuer warp of its
// own: issuing a tcgen05.mma (or a commit) occupies its thread for ~160 clocks whatever
// the instruction's size, a chunk is four instructions and a commit, and with one issuer
// per group that alone was over 1 ms of the kernel's 1.39 ms on the 256^3 shard.
#ifndef DCB_WG_SPG
#define DCB_WG_SPG 2
#endif
#ifndef DCB_WG_KS
#define DCB_WG_KS 2
#endif
constexpr int WG_SPG = DCB_WG_SPG;         // slots, and issuers, per converter group
constexpr int WG_ISSUER2_WARP = 20;        // issuers of the slots after a group's first: warps 20 ..
constexpr int WG_THREADS = (20 + 3 * (WG_SPG - 1)) * 32; // 12 converters, 3 issuers, 1 copy, 4 dump warps, more issuers
constexpr int WG_COPY_WARP = 15;
constexpr int WG_DUMP_WARP = 16;
constexpr int WG_TW = 128;                 // outputs per unit
constexpr int WG_KS = DCB_WG_KS;           // k-steps (of eight outputs) per chunk: one hand-off per chunk
constexpr int WG_CHUNKS = WG_TW / (8 * WG_KS); // chunks per unit
constexpr int WG_XW = WG_TW + 12;          // staged input row: 4 cells of margin left, 8 right; the 140-float
                                           // pitch keeps the taps of a warp's 32 lanes (about 11 rows x 3
                                           // columns) on different banks, 136 would fold them three deep
constexpr int WG_A_SLOTS = 3 * WG_SPG;     // slot s belongs to group s % 3
constexpr int WG_A_COLS = 16 * WG_KS;      // an A slot: per k-step 8 hi + 8 lo columns
constexpr uint32_t WG_TMEM_COLS = 64 + WG_A_SLOTS * 16 * 2 <= 256 ? 256 : 512; // two accumulator buffers of 32 columns + the A slots
constexpr int WG_ACC_COLS = 64;            // the A ring starts here
// The tensor pipe adds into an fp32 accumulator without rounding to nearest: over
// a chain of n updates the error grows like n^1.5 * 2^-24 and does not average
// out.  Measured on a 256^3 shard with one accumulator for the whole run: 4e-4
// of the gradient's scale.  So a chain is cut after this many units (1024
// outputs, 128 updates): the dump warps add the buffer into fp64 registers and
// zero it while the issuers fill the other one (5e-6 by the same estimate).
constexpr int WG_FLUSH_UNITS = 8;
constexpr int WG_B_FLOATS = 256 * WG_KS;   // the B tiles of a chunk: per k-step 8 x 32 floats

#ifndef DCB_WG_KNOCKOUT
#define DCB_WG_KNOCKOUT 0
#endif
#if DCB_WG_KNOCKOUT
#define WG_DBG(bit) ((g.dbg >> (bit)) & 1)
#else
#define WG_DBG(bit) 0
#endif

struct WgGeom
{
    int n, c, k;
    int in[3], out[3], f[3], pad[3];
    int lx, rx;             // as in TcGeom, for the staged input rows of a unit
    int dbg;                // timing knock-outs (builds with DCB_WG_KNOCKOUT only): bit 0 no tap loads,
                            // 1 no tensor-memory stores, 2 no B tile, 3 no MMAs, 4 no input copies
    int mrows;              // c * fd * fh * fw
    int tiles_w;
    long long units;        // n * out_d * out_h * tiles_w
    int stride[3];          // 1 or 2
    int xhalf_floats;       // one bulk copy's box in a unit buffer: c * fh * WG_XW floats rounded up to
                            // 128 bytes (a bulk copy's destination must be 128-byte aligned)
    int xplane_floats;      // pitch of one filter plane of a unit: stride[2] boxes
    int xplane_bytes;       // bytes one box brings: c * fh * WG_XW * 4
    int xbuf_bytes;         // fd plane pitches
    int dybuf_bytes;        // 16 x WG_TW floats
    // One launch covers c input channels (c * taps <= 128) and at most 16
    // filters; a larger filter tensor is cgroups x kgroups launches.
    int c_total, k_total, cgroups, kgroups;
};

// dw[k_off + kk][c_off + c][tap] (of a [k_total][c_total][taps] filter tensor) from the
// per-CTA partials of one launch; m = tap * c + c_index (c = channels of the launch).
__global__ void wg_fold_kernel(const float* __restrict__ part, int nparts, int mrows, int k, int taps, int c_total,
                               int c_off, int k_off, float alpha, float beta, float* dw)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x; // (filter, tap row)
    if (i >= mrows * k)
        return;
    const int kk = i / mrows, m = i % mrows;
    double s = 0.0;
    for (int p = 0; p < nparts; ++p)
        s += (double) part[((size_t) p * 128 + m) * 16 + kk];
    const int cl = mrows / taps; // channels of this launch
    float* o = dw + ((size_t) (k_off + kk) * c_total + c_off + m % cl) * taps + m / cl;
    const float prev = beta != 0.f ? *o : 0.f;
    *o = alpha * (float) s + beta * prev;
}

template <int SW> // stride along W
__global__ void __launch_bounds__(WG_THREADS, 1)
    wg_conv_kernel(WgGeom g, float* __restrict__ part, int* status, const __grid_constant__ CUtensorMap xmap,
                   const __grid_constant__ CUtensorMap dymap)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int unit_bytes = (g.xbuf_bytes + g.dybuf_bytes + 127) / 128 * 128;
    uint8_t* ubuf = smem;                                        // [2] unit buffers: x planes, then the dy row
    float* bring = reinterpret_cast<float*>(smem + 2 * unit_bytes); // [WG_A_SLOTS] B tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(bring + WG_A_SLOTS * WG_B_FLOATS);
    uint64_t* a_full = bars;                 // [6]
    uint64_t* a_empty = a_full + WG_A_SLOTS; // [6]
    uint64_t* u_full = a_empty + WG_A_SLOTS; // [2]
    uint64_t* u_empty = u_full + 2;          // [2]
    uint64_t* d_full = u_empty + 2;          // [2] issuers -> dump warps: a batch of units is in the buffer
    uint64_t* d_empty = d_full + 2;          // [2] dump warps -> issuers: the buffer is zero again
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0)
    {
        for (int s = 0; s < WG_A_SLOTS; ++s)
        {
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b)
        {
            mbar_init(&u_full[b], 1);
            mbar_init(&u_empty[b], 12);
        }
        for (int b = 0; b < 2; ++b)
        {
            mbar_init(&d_full[b], 3 * WG_SPG);
            mbar_init(&d_empty[b], 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(WG_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t nunits = (uint32_t) g.units;
    bool ok = true;

    if (warp < 12)
    {
        // ------------------------------------------------------------------
        // converters
        // ------------------------------------------------------------------
        const int gq = warp >> 2, quad = warp & 3;
        const int m = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        // where this lane's tap sits in a unit buffer (floats)
        int src = -1;
        if (m < g.mrows)
        {
            // row m of the partial filter is (tap, channel), channel fastest: with the
            // channel slowest the lanes of a warp read three filter planes at the same
            // bank offsets (a plane's rows start on a 128-byte boundary), three deep;
            // this order is two deep at worst (4 channels x 3 x 3 x 3, 140-float rows)
            const int c = m % g.c;
            int r = m / g.c;
            const int kw = r % g.f[2];
            r /= g.f[2];
            const int kh = r % g.f[1];
            const int kd = r / g.f[1];
            src = kd * g.xplane_floats + (c * g.f[1] + kh) * WG_XW + g.rx + kw;
        }
        // this lane's element of the B tile: filter quad*4 + lane/8, output lane%8
        const int bk = quad * 4 + (lane >> 3), bkk = lane & 7;
        const int b_off = (bkk >> 2) * 128 + (bk >> 3) * 32 + (bk & 7) * 4 + (bkk & 3); // + 64 for the lo half
        int lap = 0;
        uint32_t a_phase = 1, seq = 0;
        bool a_first = true;
        uint32_t ul = 0; // units done by this CTA
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++ul)
        {
            const uint32_t b = ul & 1;
            ok = mbar_wait(&u_full[b], (ul >> 1) & 1, abort_flag);
            if (!ok)
                break;
            const float* xb = reinterpret_cast<const float*>(ubuf + (size_t) b * unit_bytes);
            const float* dyb = reinterpret_cast<const float*>(ubuf + (size_t) b * unit_bytes + g.xbuf_bytes);
            // chunks are dealt to the groups in sequence over the whole run
            int q = (gq + 3 - (int) (seq % 3u)) % 3;
            for (; q < WG_CHUNKS && ok; q += 3)
            {
                const int slot = gq + 3 * lap;
                uint32_t hi[WG_KS][8], lo[WG_KS][8], dhi[WG_KS], dlo[WG_KS];
#pragma unroll
                for (int ks = 0; ks < WG_KS; ++ks)
                {
                    if (src >= 0 && !WG_DBG(0))
                    {
                        // output (q * WG_KS + ks) * 8 of the unit; with SW == 2 the second
                        // 64 outputs read the second half window
                        const int o = (q * WG_KS + ks) * 8;
                        const uint32_t s0 = smem_u32(
                            xb + src + (SW == 2 ? (o >= 64 ? g.xhalf_floats + (o - 64) * 2 : o * 2) : o));
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                        {
                            const float xe = __uint_as_float(lds_u32(s0 + 4u * (uint32_t) (e * SW)));
                            hi[ks][e] = tf32_rna(xe);
                            // exact remainder, fed as it is: the pipe reads its upper 19 bits
                            lo[ks][e] = __float_as_uint(xe - __uint_as_float(hi[ks][e]));
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            hi[ks][e] = lo[ks][e] = 0u;
                    }
                    const float dv = WG_DBG(2) ? 0.f : dyb[bk * WG_TW + (q * WG_KS + ks) * 8 + bkk];
                    dhi[ks] = tf32_rna(dv);
                    dlo[ks] = tf32_rna(dv - __uint_as_float(dhi[ks]));
                }
                if (!a_first)
                    ok = mbar_wait(&a_empty[slot], a_phase, abort_flag);
                if (!ok)
                    break;
                tc_fence_after();
                const uint32_t a_addr = lane_addr + (uint32_t) WG_ACC_COLS + (uint32_t) (slot * WG_A_COLS);
                float* bt = bring + slot * WG_B_FLOATS;
#pragma unroll
                for (int ks = 0; ks < WG_KS; ++ks)
                {
                    if (!WG_DBG(1))
                    {
                        tmem_st8(a_addr + (uint32_t) (ks * 16), hi[ks]);
                        tmem_st8(a_addr + (uint32_t) (ks * 16 + 8), lo[ks]);
                    }
                    if (!WG_DBG(2))
                    {
                        bt[ks * 256 + b_off] = __uint_as_float(dhi[ks]);
                        bt[ks * 256 + b_off + 64] = __uint_as_float(dlo[ks]);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&a_full[slot]);
                if (++lap == WG_SPG)
                {
                    lap = 0;
                    a_phase ^= 1;
                    a_first = false;
                }
            }
            seq += WG_CHUNKS;
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&u_empty[b]);
        }
    }
    else if (warp == WG_COPY_WARP)
    {
        // ------------------------------------------------------------------
        // bulk tensor copies, one unit ahead
        // ------------------------------------------------------------------
        const uint32_t bytes = (uint32_t) ((WG_DBG(4) ? 0 : g.f[0] * SW * g.xplane_bytes) + g.dybuf_bytes);
        uint32_t ul = 0;
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++ul)
        {
            const uint32_t b = ul & 1;
            if (ul >= 2)
                ok = mbar_wait(&u_empty[b], ((ul >> 1) + 1) & 1, abort_flag);
            if (!ok)
                break;
            if (lane == 0)
            {
                const uint32_t tw = u % (uint32_t) g.tiles_w;
                uint32_t r = u / (uint32_t) g.tiles_w;
                const int oh = (int) (r % (uint32_t) g.out[1]);
                r /= (uint32_t) g.out[1];
                const int od = (int) (r % (uint32_t) g.out[0]);
                const int n = (int) (r / (uint32_t) g.out[0]);
                const int ow0 = (int) tw * WG_TW;
                uint8_t* dst = ubuf + (size_t) b * unit_bytes;
                mbar_expect_tx(&u_full[b], bytes);
                // the window starts at a multiple of 4 floats at or left of the first tap
                for (int kd = 0; kd < g.f[0] && !WG_DBG(4); ++kd)
#pragma unroll
                    for (int h = 0; h < SW; ++h)
                        tma_load_5d(dst + ((size_t) kd * g.xplane_floats + (size_t) h * g.xhalf_floats) * 4, &xmap,
                                    ow0 * SW + g.lx + h * 128, oh * g.stride[1] - g.pad[1],
                                    od * g.stride[0] - g.pad[0] + kd, 0, n, &u_full[b]);
                tma_load_5d(dst + g.xbuf_bytes, &dymap, ow0, oh, od, 0, n, &u_full[b]);
            }
            __syncwarp();
        }
    }
    else if ((warp >= TC_MMA_WARP && warp < TC_MMA_WARP + 3) || warp >= WG_ISSUER2_WARP)
    {
        // ------------------------------------------------------------------
        // MMA issue: issuer (mq, mh) serves slot mq + 3 * mh, i.e. every
        // WG_SPG-th chunk of group mq
        // ------------------------------------------------------------------
        const int mq = warp < WG_ISSUER2_WARP ? warp - TC_MMA_WARP : (warp - WG_ISSUER2_WARP) % 3;
        const int mh = warp < WG_ISSUER2_WARP ? 0 : 1 + (warp - WG_ISSUER2_WARP) / 3;
        // fp32 accumulate, tf32 x tf32, A K-major (tensor memory), B K-major, M = 128
        const uint32_t idesc32 = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 4) << 24) | ((32u >> 3) << 17);
        const uint32_t idesc16 = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 4) << 24) | ((16u >> 3) << 17);
        int lap = 0;
        uint32_t full_phase = 0, seq = 0, ul = 0;
        bool open = false; // a batch this issuer has added into and not yet handed over
        uint32_t batch = 0;
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x, ++ul)
        {
            batch = ul / WG_FLUSH_UNITS;
            const uint32_t db = batch & 1;
            if (ul % WG_FLUSH_UNITS == 0)
            {
                // the buffer must have been drained and zeroed (initially: zeroed)
                ok = mbar_wait_t<0>(&d_empty[db], (batch >> 1) & 1, abort_flag);
                if (!ok)
                    break;
                open = true;
            }
            const uint32_t d_addr = tmem_base + db * 32u;
            int q = (mq + 3 - (int) (seq % 3u)) % 3;
            for (; q < WG_CHUNKS && ok; q += 3)
            {
                const int slot = mq + 3 * lap;
                if (lap == mh)
                    ok = mbar_wait_t<0>(&a_full[slot], full_phase, abort_flag);
                if (!ok)
                    break;
                tc_fence_after();
                if (lane == 0 && lap == mh)
                {
                    const uint32_t a_addr = tmem_base + (uint32_t) WG_ACC_COLS + (uint32_t) (slot * WG_A_COLS);
                    // B tile of a k-step: [2 k-chunks][4 filter groups][8][4]: 512 bytes
                    // between the k-chunks, 128 between the filter groups, 1 KiB per tile
                    const uint64_t bd = make_desc(smem_u32(bring + slot * WG_B_FLOATS), 512u, 128u, 0u);
#pragma unroll
                    for (int ks = 0; ks < WG_KS && !WG_DBG(3); ++ks)
                    {
                        mma_tf32_ts(d_addr, a_addr + (uint32_t) (ks * 16), bd + (uint64_t) (ks * 64),
                                    idesc32); // A_hi x [B_hi | B_lo]
                        mma_tf32_ts(d_addr, a_addr + (uint32_t) (ks * 16 + 8), bd + (uint64_t) (ks * 64),
                                    idesc16); // A_lo x B_hi
                    }
                    mma_commit(&a_empty[slot]);
                    tc_fence_before();
                }
                __syncwarp();
                if (++lap == WG_SPG)
                {
                    lap = 0;
                    full_phase ^= 1;
                }
            }
            seq += WG_CHUNKS;
            if (ok && ul % WG_FLUSH_UNITS == WG_FLUSH_UNITS - 1)
            {
                // this issuer's share of the batch has completed when this arrives
                if (lane == 0)
                    mma_commit(&d_full[db]);
                __syncwarp();
                open = false;
            }
        }
        if (ok && open)
        {
            if (lane == 0)
                mma_commit(&d_full[batch & 1]);
            __syncwarp();
        }
    }
    else if (warp >= WG_DUMP_WARP)
    {
        // ------------------------------------------------------------------
        // dump warps: zero both buffers, then per batch add the buffer into
        // fp64 registers (D[:, 0:16] + D[:, 16:32]) and zero it again; at the
        // end write the CTA's partial filter
        // ------------------------------------------------------------------
        const int quad = warp & 3;
        const uint32_t la = tmem_base + ((uint32_t) (quad * 32) << 16);
        for (int col = 0; col < WG_ACC_COLS; col += 16)
            tmem_st16_zero(la + col);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
        {
            mbar_arrive(&d_empty[0]);
            mbar_arrive(&d_empty[1]);
        }
        double acc[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            acc[k] = 0.0;
        uint32_t my_units = 0;
        for (uint32_t u = blockIdx.x; u < nunits; u += gridDim.x)
            ++my_units;
        const uint32_t nbatches = (my_units + WG_FLUSH_UNITS - 1) / WG_FLUSH_UNITS;
        for (uint32_t bt = 0; bt < nbatches && ok; ++bt)
        {
            const uint32_t db = bt & 1;
            ok = mbar_wait(&d_full[db], (bt >> 1) & 1, abort_flag);
            if (!ok)
                break;
            tc_fence_after();
            uint32_t v0[16], v1[16];
            tmem_ld16(la + db * 32u, v0);
            tmem_ld16(la + db * 32u + 16u, v1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tmem_st16_zero(la + db * 32u);
            tmem_st16_zero(la + db * 32u + 16u);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&d_empty[db]);
#pragma unroll
            for (int k = 0; k < 16; ++k)
                acc[k] += (double) __uint_as_float(v0[k]) + (double) __uint_as_float(v1[k]);
        }
        if (ok)
        {
            float* o = part + ((size_t) blockIdx.x * 128 + quad * 32 + lane) * 16;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                o[k] = (float) acc[k];
        }
    }

    if (!ok && lane == 0)
        atomicExch(status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP)
    {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(WG_TMEM_COLS)
                     : "memory");
    }
}

} // namespace
} // namespace dcb
