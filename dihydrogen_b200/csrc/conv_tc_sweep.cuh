// tcgen05 / TMEM convolution for filters with depth (fd > 1): the "sweep"
// kernel.  Same GEMM view as conv_tc_kernel.cuh (M = 128 outputs along W, the
// reduction runs over (c, kw) of one staged input row), but a staged row is
// converted ONCE and serves every (kd, kh) tap:
//
//   * A CTA owns a column of the volume (th output rows x 128 outputs wide)
//     and sweeps a segment of output planes od0..od1-1 along D, one input
//     plane ("step") after the other.
//   * The accumulators of fd consecutive output planes are live at once.
//     Block (row j, plane slot s = od mod fd) sits at TMEM column
//     (j * fd + s) * 16, so the fh * fd blocks that input row i feeds (rows
//     i-fh+1..i, all slots) are one contiguous column range and ONE
//     instruction of N = fh * fd * 16 updates all of them.  Which kd lands in
//     which slot depends on d mod fd: the filter image exists in fd rotations.
//   * 3xTF32 is folded into the reduction: the A columns [hi ; lo] meet the
//     B k-rows [w_hi ; w_hi], then the k-steps start over at the hi columns
//     and meet [w_lo ; 0]: one accumulator block per output row, every tap
//     written into tensor memory twice, not three times.
//   * After step d the plane od = d + pad - (fd-1) has all its terms: the
//     epilogue warps store it (if it belongs to the segment), re-zero its
//     blocks and hand them back, row by row, while the issuers carry on with
//     the next input plane; a row's blocks are only needed again th rows
//     later.  Planes outside the segment collect terms too (the instruction
//     cannot skip a slot); they are just zeroed when their turn comes, which
//     is always before the slot's next owner receives its first term.  The
//     steps before the first and after the last input plane that exist only
//     to retire planes are "virtual": nothing is copied, converted or
//     multiplied in them.
//
// Hand-offs (all mbarriers, all waits bounded):
//   raw_full / raw_empty   copy warp <-> converters, per chunk of raw rows
//   a_full / a_empty       converter group g <-> issuer g, per A slot
//   row_done[i]            issuer -> epilogue: the MMAs of input row i of this
//                          step have completed (tcgen05.commit)
//   row_free[j]            epilogue -> issuers: the blocks of output row j
//                          have been retired and are zero again
// row_done / row_free complete once per step.  A parity wait cannot tell a
// barrier that is two completions away, in either direction.
//  * Not behind: the epilogue warps wait on the same row_done barriers every
//    step.  An issuer's rows change from step to step, but with at most fh
//    issuers its last two rows of every step lie among the last fh + 1 rows,
//    and their waits cover the last output row of either epilogue half, hence
//    (each half retires in ascending order) every row_free of the previous step.
//  * Not ahead: an issuer only waits for output rows that its own row adds
//    into, and an epilogue warp only for input rows that feed its output row,
//    so the barrier's next completion needs something the waiter does after
//    the wait.  (Waiting for a row that one's own row does not touch breaks
//    this: the barrier may complete again first and the wait never ends.)
// The protocol was checked for fh in {1,2,3,5}, up to fh issuers and 2..13 rows
// per column under random schedules in a host-side model.
#pragma once

#include "conv_tc_kernel.cuh"

namespace dcb
{
namespace
{

// Per-role clock accounting (a build with -DDCB_SW_PROFILE=1 only): every warp
// adds up the clocks it spends in each phase of its loop and leaves eight
// totals in `prof` at the end; the host prints the per-role averages.
#ifndef DCB_SW_PROFILE
#define DCB_SW_PROFILE 0
#endif
// Timing knock-outs (a build with -DDCB_SW_KNOCKOUT=1 only; results are wrong
// with any bit set): bits of DCB_SW_DBG switch single pieces of work off so
// that what the kernel's time depends on can be measured.
#ifndef DCB_SW_KNOCKOUT
#define DCB_SW_KNOCKOUT 0
#endif
#if DCB_SW_KNOCKOUT
#define SW_DBG(bit) ((g.nsets >> (bit)) & 1)
#else
#define SW_DBG(bit) 0
#endif
#if DCB_SW_PROFILE
#define SW_PROF_DECL long long pf_t = clock64(), pf_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long pf_t0 = pf_t;
#define SW_PROF_MARK(slot)                                                                                            \
    {                                                                                                                 \
        const long long pf_now = clock64();                                                                           \
        pf_acc[slot] += pf_now - pf_t;                                                                                \
        pf_t = pf_now;                                                                                                \
    }
#define SW_PROF_FLUSH(prof)                                                                                           \
    if (prof != nullptr && lane == 0)                                                                                 \
    {                                                                                                                 \
        pf_acc[7] = clock64() - pf_t0;                                                                                \
        for (int pf_i = 0; pf_i < 8; ++pf_i)                                                                          \
            prof[((size_t) blockIdx.x * 32 + warp) * 8 + pf_i] = pf_acc[pf_i];                                        \
    }
#else
#define SW_PROF_DECL
#define SW_PROF_MARK(slot)
#define SW_PROF_FLUSH(prof)
#endif

constexpr int SW_NBK = 16; // accumulator columns per (output row, plane slot)


struct SwGeom
{
    int n, c, k;    // c: input channels of one launch (a group of the filter's w_c_total)
    int w_c_total;  // input channels of the filter
    int w_c_off;    // first input channel of this launch's group
    int cgroups;    // launches per convolution = w_c_total / c
    int in[3], out[3], f[3], pad[3];
    int lx, rx;     // as in TcGeom: where a staged row starts, where its first tap sits
    long long xs_n, xs_c, xs[3];
    long long ys_n, ys_c, ys[3];
    int split;      // 1: 3xTF32, 0: single TF32 pass
    uint32_t rnd_add, rnd_mask; // as in TcGeom
    int th;         // output rows per column
    int rows;       // staged rows per step = th + fh - 1
    int crows;      // c * fw
    int kr;         // A columns per slot (multiple of 8): the taps' hi parts, then (3xTF32) their lo parts
    int ks1, ksteps; // k-steps that read the A columns in order (kr / 8); all k-steps: with 3xTF32 the
                    // hi parts are read a second time, from column 0, against the filter's lo parts
    int kb;         // k-rows of the filter image = 8 * ksteps
    int ntot;       // fh * fd * SW_NBK
    int b_rot_bytes, b_bytes; // one rotation of the filter image, all fd of them
    int groups, a_slots;
    int tiles_w, tiles_h, nseg;
    long long units;
    int raw_slots, raw_slot_bytes, chunk_rows, chunks_pp;
    int nsets;      // multi-group kernel: accumulator sets the channel groups are spread over
};

struct SwUnit
{
    int n, ow0, oh0, od0, od1;
    int d_first, d_stop; // steps d_first .. d_stop-1
    int d_real_hi;       // input planes above this one only feed foreign output planes
};

__device__ __forceinline__ SwUnit sw_unit(const SwGeom& g, uint32_t u)
{
    SwUnit t;
    const uint32_t tw = u % (uint32_t) g.tiles_w;
    uint32_t r = u / (uint32_t) g.tiles_w;
    const uint32_t thi = r % (uint32_t) g.tiles_h;
    r /= (uint32_t) g.tiles_h;
    const uint32_t seg = r % (uint32_t) g.nseg;
    t.n = (int) (r / (uint32_t) g.nseg);
    t.ow0 = (int) tw * TC_M;
    t.oh0 = (int) thi * g.th;
    t.od0 = (int) (((long long) seg * g.out[0]) / g.nseg);
    t.od1 = (int) (((long long) (seg + 1) * g.out[0]) / g.nseg);
    t.d_first = t.od0 - g.pad[0];
    t.d_real_hi = t.od1 - 1 + g.f[0] - 1 - g.pad[0];
    t.d_stop = t.d_real_hi + g.f[0]; // fd - 1 more steps retire the planes the last rows spilled into
    return t;
}

__device__ __forceinline__ bool sw_real(const SwGeom& g, const SwUnit& t, int d)
{
    return d >= 0 && d < g.in[0] && d <= t.d_real_hi;
}

__device__ __forceinline__ int sw_mod(int a, int m)
{
    const int r = a % m;
    return r < 0 ? r + m : r;
}

// Filter image: [rotation][k-step][2 k-chunks][ntot/8][8 n][4 k] floats.
// Column (j, s, ko): output row offset j (kh = fh-1-j), plane slot s, filter ko.
// In rotation r (= d mod fd) slot s belongs to the output plane d + pad - kd
// with kd = (r + pad - s) mod fd.
__global__ void sw_pack_filter_kernel(const float* __restrict__ w, float* __restrict__ b, SwGeom g)
{
    const int fd = g.f[0], fh = g.f[1], fw = g.f[2];
    const int per_rot = g.kb * g.ntot;
    const long long total = (long long) fd * per_rot;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long) gridDim.x * blockDim.x)
    {
        const int rot = (int) (i / per_rot);
        const int e = (int) (i % per_rot);
        const int ki = e % 4;
        const int ni = (e / 4) % 8;
        const int ngroup = (e / 32) % (g.ntot / 8);
        const int kchunk = (e / (32 * (g.ntot / 8))) % 2;
        const int kstep = e / (64 * (g.ntot / 8));
        const int krow = kstep * 8 + kchunk * 4 + ki;
        const int ncol = ngroup * 8 + ni;
        const int j = ncol / (fd * SW_NBK);
        const int s = (ncol / SW_NBK) % fd;
        const int ko = ncol % SW_NBK;
        const int kh = fh - 1 - j;
        const int kd = sw_mod(rot + g.pad[0] - s, fd);
        // k-rows 0 .. kr-1 meet the A columns [hi | lo] (w_hi both times); the k-steps
        // after them read the A columns from 0 again and meet w_lo (zeros below the
        // columns that are not hi parts)
        int part, rem;
        if (krow < g.kr)
        {
            part = krow / g.crows; // 0: A_hi x w_hi, 1: A_lo x w_hi
            rem = krow % g.crows;
            if (part >= (g.split ? 2 : 1))
                part = 3;
        }
        else
        {
            rem = krow - g.kr;
            part = (g.split && rem < g.crows) ? 2 : 3; // 2: A_hi x w_lo
            rem = rem < g.crows ? rem : 0;
        }
        const int c = rem / fw, kw = rem % fw;
        float val = 0.f;
        if (ko < g.k && part < 3)
        {
            const float wv = w[((((size_t) ko * g.w_c_total + g.w_c_off + c) * fd + kd) * fh + kh) * fw + kw];
            const float hi = __uint_as_float((__float_as_uint(wv) + g.rnd_add) & g.rnd_mask);
            val = part < 2 ? hi : __uint_as_float(tf32_rna(wv - hi));
        }
        b[i] = val;
    }
}

// Packed fp32 pairs (two lanes of one 64-bit register): the statistics of the
// epilogue cost half the instructions this way.
__device__ __forceinline__ uint64_t f2_pack(float a, float b)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Adds the epilogue warps' partial sums in fp64 and in a fixed order: warp w of
// the block adds partials w, w + 32, ... (a serial walk by one warp is a chain of
// ~1800 dependent L2 loads, 70 us), thread (0, k) then adds the 32 warps' sums in
// warp order and gives sums[k], thread (0, 16 + k) gives sqsums[k].
constexpr int SW_FOLD_WARPS = 32;
__global__ void __launch_bounds__(SW_FOLD_WARPS * 32)
    sw_stats_fold_kernel(const float* __restrict__ part, int nparts, int nk, float* __restrict__ sums,
                         float* __restrict__ sqsums)
{
    __shared__ double sm[SW_FOLD_WARPS][32];
    const int t = threadIdx.x & 31, w = threadIdx.x >> 5;
    double acc = 0.0;
    for (int i = w; i < nparts; i += SW_FOLD_WARPS)
        acc += (double) part[(size_t) i * 32 + t];
    sm[w][t] = acc;
    __syncthreads();
    if (w != 0)
        return;
    acc = 0.0;
#pragma unroll
    for (int i = 0; i < SW_FOLD_WARPS; ++i)
        acc += sm[i][t];
    if (t < SW_NBK)
    {
        if (t < nk)
            sums[t] = (float) acc;
    }
    else if (t - SW_NBK < nk)
        sqsums[t - SW_NBK] = (float) acc;
}

// 4 channels x 3 taps, split: A columns 0..11 hi, 12..23 lo.
// ROUND_LO: the lo part rounded to TF32 as well (two more instructions per tap).
// The multi-group kernel asks for it: its accumulators take 180 and more updates
// per output, the tensor pipe's accumulation already uses most of the 1e-5 there
// and the unrounded remainder tipped a case over the bound.
template <bool ROUND_LO = false>
__device__ __forceinline__ void sw_convert_c4f3(uint32_t raw_lane, uint32_t pitch, uint32_t (&v)[3][8])
{
    uint32_t xv[12];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int kw = 0; kw < 3; ++kw)
            xv[c * 3 + kw] = lds_u32(raw_lane + 4u * ((uint32_t) c * pitch + 3u + (uint32_t) kw));
#pragma unroll
    for (int r = 0; r < 12; ++r)
    {
        const float xe = __uint_as_float(xv[r]);
        const uint32_t hi = tf32_rna(xe);
        // x - hi is exact in fp32 and below 2^-11 |x|; the tensor pipe reads the
        // upper 19 bits of it, an error below 2^-21 |x|: no rounding of its own
        const uint32_t lo =
            ROUND_LO ? tf32_rna(xe - __uint_as_float(hi)) : __float_as_uint(xe - __uint_as_float(hi));
        v[r / 8][r % 8] = hi;
        v[(12 + r) / 8][(12 + r) % 8] = lo;
    }
}

// ---------------------------------------------------------------------------
// Warps: 0..11 converters (three groups of four), 12..14 MMA issuers (issuer q
// serves group q), 15 bulk copies, 16..23 epilogue (two per TMEM quadrant,
// even / odd output rows).  TMEM columns: [accumulators th * fd * 16][A ring].
// ---------------------------------------------------------------------------
// STATS: the epilogue also adds up, per filter, the outputs it stores and their
// squares (what a batch-norm statistics pass over y would read again): each
// lane keeps its own fp32 sums, every epilogue warp leaves 32 partials in
// `stat_part` at the end, and sw_stats_fold_kernel adds those in a fixed order
// in fp64.
// BLEND: beta != 0, the old output is fetched early and blended in (plain stores).
// EPI: epilogue warps, EPI / 4 per TMEM quadrant, each retiring every
// (EPI / 4)-th output row.  Retiring a row costs its warp a tensor-memory load
// and a zeroing store back to back, well over a thousand clocks with MMAs in
// flight, and the issuers wait for the hand-back: the more rows of a plane are
// in retirement at once, the shorter the step.
// Warps: converters 0..11, issuers 12..14, the copy warp 15, epilogue 16..16+EPI-1
// (warp & 3 is the TMEM quadrant).
// XISS: the last TC_GROUPS_MAX warps are second issuers.  With two A slots per
// converter group, issuer (q, 0) takes the group's rows that land in its first slot
// and issuer (q, 1) those in the second.  Free-running, the three issuers of the
// plain kernel need as long as its busiest epilogue warps (0.35 ms on the 256^3
// shard, ~140 clocks per tcgen05.mma or commit, seven per staged row); with six the
// kernel takes 0.378 ms instead of 0.433.  The variants whose epilogue does more
// (statistics, blend) are held by their epilogue warps and by registers (the extra
// warps lower the cap to 66 per thread, their epilogues then spill): they keep
// three issuers and one slot per group.
__host__ __device__ constexpr int sw_threads(int epi, int xiss)
{
    return (TC_TMA_WARP + 1 + epi + (xiss ? TC_GROUPS_MAX : 0)) * 32;
}

template <bool C4F3, bool STATS, bool BLEND, int EPI, int XISS>
__global__ void __launch_bounds__(sw_threads(EPI, XISS), 1)
    sw_conv_kernel(SwGeom g, float alpha, float beta, const float* __restrict__ bimg, float* y, int* status,
                   const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap ymap, int use_ymap,
                   float* __restrict__ stat_part, long long* prof)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* b_smem = reinterpret_cast<float*>(smem);
    const int b_region = (g.b_bytes + 127) / 128 * 128;
    uint8_t* raw_ring = smem + b_region;
    uint32_t* ktab = reinterpret_cast<uint32_t*>(raw_ring + (size_t) g.raw_slots * g.raw_slot_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ktab + ((g.kr + 1) & ~1));
    uint64_t* a_full = bars;                        // [a_slots]
    uint64_t* a_empty = a_full + g.a_slots;         // [a_slots]
    uint64_t* row_done = a_empty + g.a_slots;       // [32]
    uint64_t* row_free = row_done + 32;             // [32]
    uint64_t* raw_full = row_free + 32;             // [raw_slots]
    uint64_t* raw_empty = raw_full + g.raw_slots;   // [raw_slots]
    uint64_t* iss_sync = raw_empty + g.raw_slots;   // [TC_GROUPS_MAX] the issuers of a group, once per step
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(iss_sync + TC_GROUPS_MAX);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // output staging for bulk stores: two 2 KiB buffers per epilogue warp
    float* stage_base = reinterpret_cast<float*>(
        (reinterpret_cast<uintptr_t>(tmem_slot + 2) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int fd = g.f[0], fh = g.f[1], R = g.rows, G = g.groups;
#if DCB_SW_PROFILE
    __shared__ volatile long long pf_issue_end[32], pf_freed[32]; // clocks: row i issued / row j handed back
#endif

    if (tid == 0)
    {
        for (int s = 0; s < g.a_slots; ++s)
        {
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);
        }
        for (int r = 0; r < 32; ++r)
        {
            mbar_init(&row_done[r], 1);
            mbar_init(&row_free[r], 4);
        }
        for (int r = 0; r < g.raw_slots; ++r)
        {
            mbar_init(&raw_full[r], 1);
            mbar_init(&raw_empty[r], 4 * g.groups);
        }
        for (int q = 0; q < TC_GROUPS_MAX; ++q)
            mbar_init(&iss_sync[q], g.a_slots / g.groups);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // k-row table: offset of the tap inside a raw chunk row, and what the row
    // carries: 0 hi part, 1 lo part, 2 zero
    for (int r = tid; r < g.kr; r += sw_threads(EPI, XISS))
    {
        const int part = r / g.crows, rem = r % g.crows;
        const int c = rem / g.f[2], kw = rem % g.f[2];
        const uint32_t off = (uint32_t) (c * g.chunk_rows * TC_RAW_W + g.rx + kw);
        const uint32_t sel = part < (g.split ? 2 : 1) ? (uint32_t) part : 2u;
        ktab[r] = sel == 2u ? ((2u << 16) | 4u) : (off | (sel << 16));
    }
    for (int i = tid; i < g.b_bytes / 16; i += sw_threads(EPI, XISS))
        reinterpret_cast<float4*>(b_smem)[i] = reinterpret_cast<const float4*>(bimg)[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_col0 = (uint32_t) (g.th * fd * SW_NBK); // first column of the A ring
    const uint32_t nunits = (uint32_t) g.units;
    bool ok = true;

    if (warp < 4 * G)
    {
        // ------------------------------------------------------------------
        // converters
        // ------------------------------------------------------------------
        const int gq = warp >> 2, quad = warp & 3;
        const int mcol = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        const int laps_a = g.a_slots / G;
        const uint32_t ktab_s = smem_u32(ktab);
        const int Rc = g.chunk_rows;
        const uint32_t pitch = (uint32_t) (g.chunk_rows * TC_RAW_W);
        int lap_a = 0;
        uint32_t cslot = 0, cphase = 0, a_phase = 1;
        bool a_first = true;
        // this group's rows of every step: a contiguous block (see the issuers)
        const int rpg = (R + G - 1) / G;
        const int my_lo = gq * rpg, my_hi = min(R, my_lo + rpg);
        SW_PROF_DECL
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
        {
            const SwUnit t = sw_unit(g, u);
            for (int d = t.d_first; d < t.d_stop && ok; ++d)
            {
                if (!sw_real(g, t, d))
                    continue;
                for (int ch = 0; ch < g.chunks_pp && ok; ++ch)
                {
                    const int lo = ch * Rc, hi = min(min(R, (ch + 1) * Rc), my_hi);
                    bool have = false;
                    for (int i = max(lo, my_lo); i < hi && ok; ++i)
                    {
                        const int a_slot = gq + G * lap_a;
                        SW_PROF_MARK(4)
                        if (!have && !SW_DBG(6))
                            ok = mbar_wait(&raw_full[cslot], cphase, abort_flag);
                        have = true;
                        SW_PROF_MARK(0)
                        if (!ok)
                            break;
                        const float* raw = reinterpret_cast<const float*>(raw_ring + (size_t) cslot * g.raw_slot_bytes)
                                           + (i - lo) * TC_RAW_W;
                        const uint32_t a_addr = lane_addr + a_col0 + (uint32_t) (a_slot * g.kr);
                        const uint32_t raw_s = smem_u32(raw) + 4u * (uint32_t) mcol;
                        if (C4F3)
                        {
                            uint32_t v[3][8];
                            if (!SW_DBG(5))
                                // the converter is written for taps that start 3 cells into the staged row
                                sw_convert_c4f3(raw_s + 4u * (uint32_t) (g.rx - 3), pitch, v);
                            else
                            {
#pragma unroll
                                for (int ck = 0; ck < 3; ++ck)
#pragma unroll
                                    for (int e = 0; e < 8; ++e)
                                        v[ck][e] = 0u;
                            }
                            SW_PROF_MARK(1)
                            if (!a_first && !SW_DBG(10))
                                ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                            SW_PROF_MARK(2)
                            if (!ok)
                                break;
                            tc_fence_after();
                            if (!SW_DBG(0))
                            {
#pragma unroll
                                for (int ck = 0; ck < 3; ++ck)
                                    tmem_st8(a_addr + (uint32_t) (ck * 8), v[ck]);
                            }
                        }
                        else
                        {
                            if (!a_first)
                                ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                            if (!ok)
                                break;
                            tc_fence_after();
                            for (int r0 = 0; r0 < g.kr; r0 += 8)
                            {
                                uint32_t v[8];
                                convert_chunk(ktab_s + 4u * r0, raw_s, v, g.rnd_add, g.rnd_mask);
                                tmem_st8(a_addr + (uint32_t) r0, v);
                            }
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&a_full[a_slot]);
                        SW_PROF_MARK(3)
                        if (++lap_a == laps_a)
                        {
                            lap_a = 0;
                            a_phase ^= 1;
                            a_first = false;
                        }
                    }
                    // every converter warp releases every chunk, and only after it
                    // has seen it arrive (a group without rows in this chunk too:
                    // no warp runs further ahead of the copies than the ring is deep)
                    if (!have && ok && !SW_DBG(6))
                        ok = mbar_wait(&raw_full[cslot], cphase, abort_flag);
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&raw_empty[cslot]);
                    if (++cslot == (uint32_t) g.raw_slots)
                    {
                        cslot = 0;
                        cphase ^= 1;
                    }
                }
            }
        }
        SW_PROF_FLUSH(prof)
    }
    else if (warp == TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // bulk tensor copies: chunk_rows raw rows of every channel per copy.
        // Rows above or below the image arrive as zeros.
        // ------------------------------------------------------------------
        const uint32_t bytes = (uint32_t) (g.c * g.chunk_rows) * TC_RAW_W * 4u;
        uint32_t slot = 0, empty_phase = 1;
        bool first_lap = true;
        SW_PROF_DECL
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
        {
            const SwUnit t = sw_unit(g, u);
            for (int d = t.d_first; d < t.d_stop && ok; ++d)
            {
                if (!sw_real(g, t, d))
                    continue;
                for (int ch = 0; ch < g.chunks_pp; ++ch)
                {
                    SW_PROF_MARK(4)
                    if (SW_DBG(6))
                        continue;
                    if (!first_lap)
                        ok = mbar_wait(&raw_empty[slot], empty_phase, abort_flag);
                    SW_PROF_MARK(0)
                    if (!ok)
                        break;
                    if (lane == 0)
                    {
                        mbar_expect_tx(&raw_full[slot], bytes);
                        // x starts 4 cells left of the column: a multiple of 4 floats
                        tma_load_5d(raw_ring + (size_t) slot * g.raw_slot_bytes, &xmap, t.ow0 + g.lx,
                                    t.oh0 - g.pad[1] + ch * g.chunk_rows, d, 0, t.n, &raw_full[slot]);
                    }
                    __syncwarp();
                    SW_PROF_MARK(1)
                    if (++slot == (uint32_t) g.raw_slots)
                    {
                        slot = 0;
                        empty_phase ^= 1;
                        first_lap = false;
                    }
                }
            }
        }
        SW_PROF_FLUSH(prof)
    }
    else if ((warp >= TC_MMA_WARP && warp < TC_TMA_WARP) || (XISS && warp >= TC_TMA_WARP + 1 + EPI))
    {
        // ------------------------------------------------------------------
        // MMA issue: issuer (mq, mh) takes the rows converter group mq wrote into
        // its A slot mq + G * mh.  Lane i issues staged row i (its descriptors
        // depend on i only).
        // ------------------------------------------------------------------
        const int mq = warp < TC_TMA_WARP ? warp - TC_MMA_WARP : warp - (TC_TMA_WARP + 1 + EPI);
        const int mh = warp < TC_TMA_WARP ? 0 : 1;
        if (mq < G && mh < g.a_slots / G)
        {
            const int my_i = lane;
            const int j_lo = max(0, fh - 1 - my_i);
            const int j_hi = min(fh, g.th + fh - 1 - my_i);
            const int blk = fd * SW_NBK; // columns of one output row
            const uint32_t my_idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((TC_M >> 4) << 24)
                                      | ((uint32_t) ((max(1, j_hi - j_lo) * blk) >> 3) << 17);
            const uint32_t my_d = tmem_base + (uint32_t) ((my_i - fh + 1 + j_lo) * blk);
            const uint32_t b_lbo = (uint32_t) (g.ntot / 8) * 128u;
            const uint32_t b_kstep_units = ((uint32_t) g.ntot * 32u) >> 4;
            const uint64_t my_b_desc =
                make_desc(smem_u32(b_smem), b_lbo, 128u, 0u) + (uint64_t) ((uint32_t) (j_lo * blk));
            const uint32_t rot_units = (uint32_t) g.b_rot_bytes >> 4;
            const uint32_t a_ring = tmem_base + a_col0;
            const int ks_lo = 0, ks_hi = g.ksteps;
            const int laps_a = g.a_slots / G;
            int lap_a = 0;
            uint32_t full_phase = 0, step = 0;
            // Rows are dealt to the issuers in contiguous blocks, not round robin.
            // MMAs whose accumulator columns overlap are executed one after the
            // other by the tensor pipe, about 150 clocks apart whatever their size;
            // only MMAs on disjoint columns overlap in the pipe.  A staged row
            // adds into the fh output rows above it, so rows dealt round robin
            // (issuers on rows i, i+1, i+2 at any time) always collide, while
            // blocks keep the issuers at least fh rows apart whenever a block has
            // fh rows or more.
            const int rpg = (R + G - 1) / G;
            const int my_lo = mq * rpg, my_hi = min(R, my_lo + rpg);
            int rot = 0; // d mod fd, kept by counting
            SW_PROF_DECL
            for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
            {
                const SwUnit t = sw_unit(g, u);
                rot = sw_mod(t.d_first, fd);
                for (int d = t.d_first; d < t.d_stop && ok; ++d, ++step, rot = rot + 1 == fd ? 0 : rot + 1)
                {
                    // The issuers of a group stay within one step of each other: the second
                    // one skips the rows it does not own without a wait (virtual steps
                    // entirely), and a parity wait cannot tell a barrier two completions
                    // away.  The first issuer waits for every row's hand-back in every step,
                    // so once both have finished a step the barriers this group looks at are
                    // at most one completion behind what either expects next.
                    if (laps_a > 1 && step != 0)
                        ok = mbar_wait_t<0>(&iss_sync[mq], (step - 1) & 1, abort_flag);
                    const bool real = sw_real(g, t, d);
                    const uint32_t par = step & 1;
                    const uint64_t bd0 = my_b_desc + (uint64_t) ((uint32_t) rot * rot_units);
                    for (int i = my_lo; i < my_hi && ok; ++i)
                    {
                        // a real row belongs to the issuer of the slot it was written to,
                        // a virtual one (nothing to multiply) to the group's first issuer
                        if (real ? (laps_a > 1 && lap_a != mh) : mh != 0)
                        {
                            if (real && ++lap_a == laps_a)
                            {
                                lap_a = 0;
                                full_phase ^= 1;
                            }
                            continue;
                        }
                        // The blocks this row adds into (output rows r_lo..r_hi) must
                        // have been retired.  Each epilogue warp of a quadrant retires
                        // its rows in ascending order, so the top EPI / 4 rows (one per
                        // warp) stand for all of them.  Only rows
                        // this row adds into may be waited for: their next retirement
                        // needs this very row, so such a barrier cannot complete again
                        // before this wait has seen it.
                        const int r_hi = min(i, g.th - 1), r_lo = max(0, i - fh + 1);
                        SW_PROF_MARK(4)
                        for (int r = r_hi; r >= r_lo && r > r_hi - EPI / 4 && ok && !SW_DBG(8); --r)
                            ok = mbar_wait_t<0>(&row_free[r], par, abort_flag);
                        SW_PROF_MARK(0)
#if DCB_SW_PROFILE
                        // how long ago the last row this one needed was handed back
                        if (step > 2)
                            pf_acc[5] += clock64() - pf_freed[r_hi];
#endif
                        if (!ok)
                            break;
                        if (real)
                        {
                            const uint32_t slot = (uint32_t) (mq + G * lap_a);
                            if (!SW_DBG(11))
                                ok = mbar_wait_t<0>(&a_full[slot], full_phase, abort_flag);
                            SW_PROF_MARK(1)
                            if (!ok)
                                break;
                            tc_fence_after();
                            if (lane == i)
                            {
                                const uint32_t a_base = a_ring + slot * (uint32_t) g.kr;
                                uint32_t a_addr = a_base + 8u * (uint32_t) ks_lo;
                                uint64_t bd = bd0 + (uint64_t) (b_kstep_units * (uint32_t) ks_lo);
                                for (int ks = ks_lo; ks < (SW_DBG(3) ? ks_lo + 1 : ks_hi); ++ks)
                                {
                                    mma_tf32_ts(my_d, a_addr, bd, SW_DBG(4) ? ((my_idesc & ~(0x3fu << 17)) | (2u << 17)) : my_idesc);
                                    // after the k-steps over [hi | lo] the hi parts are read again
                                    a_addr = ks + 1 == g.ks1 ? a_base : a_addr + 8;
                                    bd += b_kstep_units;
                                }
                                if (SW_DBG(7))
                                {
                                    mbar_arrive(&a_empty[slot]);
                                    mbar_arrive(&row_done[i]);
                                }
                                else
                                {
                                    mma_commit(&a_empty[slot]);
                                    mma_commit(&row_done[i]);
                                }
                                tc_fence_before();
#if DCB_SW_PROFILE
                                pf_issue_end[i] = clock64();
#endif
                            }
                            __syncwarp();
                            SW_PROF_MARK(2)
                            if (++lap_a == laps_a)
                            {
                                lap_a = 0;
                                full_phase ^= 1;
                            }
                        }
                        else
                        {
                            tc_fence_after();
                            if (lane == 0)
                                mbar_arrive(&row_done[i]);
                            __syncwarp();
                        }
                    }
                    if (laps_a > 1)
                    {
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&iss_sync[mq]);
                    }
                }
            }
            SW_PROF_FLUSH(prof)
        }
    }
    else if (warp >= (TC_TMA_WARP + 1) && warp < TC_TMA_WARP + 1 + EPI)
    {
        // ------------------------------------------------------------------
        // epilogue: after step d retire output plane d + pad - (fd-1)
        // ------------------------------------------------------------------
        const int quad = warp & 3;
        const int ew = warp - (TC_TMA_WARP + 1); // index among the epilogue warps
        const int half = ew >> 2, nhalf = EPI / 4;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        const int nk = g.k;
        const size_t ysc = (size_t) g.ys_c;
        // bulk stores overwrite: the blend with the old output takes the plain path
        const bool bulk = !BLEND && use_ymap != 0;
        float* stage = stage_base + ew * (2 * SW_NBK * 32);
        uint32_t nstored = 0;
        uint64_t s1[STATS ? SW_NBK / 2 : 1], s2[STATS ? SW_NBK / 2 : 1]; // packed pairs of filters
#pragma unroll
        for (int k = 0; k < (STATS ? SW_NBK / 2 : 1); ++k)
            s1[k] = s2[k] = 0ull; // two +0.0f
        // every warp zeroes the blocks of the rows it will retire, then hands
        // them out for the first step
        for (int j = half; j < g.th; j += nhalf)
            for (int col = 0; col < fd * SW_NBK; col += 16)
                tmem_st16_zero(lane_addr + (uint32_t) (j * fd * SW_NBK + col));
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
            for (int j = half; j < g.th; j += nhalf)
                mbar_arrive(&row_free[j]);
        uint32_t step = 0;
        SW_PROF_DECL
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
        {
            const SwUnit t = sw_unit(g, u);
            const int ow = t.ow0 + quad * 32 + lane;
            for (int d = t.d_first; d < t.d_stop && ok; ++d, ++step)
            {
                const int od = d + g.pad[0] - (fd - 1);
                const bool store = od >= t.od0 && od < t.od1;
                const uint32_t par = step & 1;
                const uint32_t slot_col = (uint32_t) (sw_mod(od, fd) * SW_NBK);
                for (int j = half; j < g.th && ok; j += nhalf)
                {
                    const int oh = t.oh0 + j;
                    const bool wr = store && oh < g.out[1];
                    // a blend with the old output: fetch it while the row is still in the works
                    float old[BLEND ? SW_NBK : 1];
                    float* const yrow =
                        y + (size_t) t.n * g.ys_n + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
                    if (BLEND && wr && ow < g.out[2])
                    {
#pragma unroll
                        for (int k = 0; k < (BLEND ? SW_NBK : 1); ++k)
                            if (k < nk)
                                old[k] = yrow[(size_t) k * ysc];
                    }
                    SW_PROF_MARK(4)
                    for (int i = j; i < j + fh && ok && !SW_DBG(9); ++i)
                        ok = mbar_wait(&row_done[i], par, abort_flag);
                    SW_PROF_MARK(0)
#if DCB_SW_PROFILE
                    if (step > 2 && sw_real(g, t, d))
                    {
                        long long last = 0;
                        for (int i = j; i < j + fh; ++i)
                            last = pf_issue_end[i] > last ? pf_issue_end[i] : last;
                        pf_acc[5] += clock64() - last; // issue of the last row needed -> seen complete
                    }
#endif
                    if (!ok)
                        break;
                    tc_fence_after();
                    const uint32_t addr = lane_addr + (uint32_t) (j * fd * SW_NBK) + slot_col;
                    uint32_t v[16];
                    if (wr)
                    {
                        tmem_ld16(addr, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    }
                    SW_PROF_MARK(1)
                    // hand the blocks back first: the issuers wait for that, nobody for the store
                    tmem_st16_zero(addr);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                    {
#if DCB_SW_PROFILE
                        pf_freed[j] = clock64();
#endif
                        mbar_arrive(&row_free[j]);
                    }
                    SW_PROF_MARK(2)
                    if (!wr)
                        continue;
                    if (STATS && ow < g.out[2])
                    {
                        // beta is zero whenever statistics are asked for
#pragma unroll
                        // of the raw accumulators: alpha goes on at the end
                        for (int k = 0; k < (STATS ? SW_NBK / 2 : 1); ++k)
                        {
                            const uint64_t o = f2_pack(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
                            s1[k] = f2_add(s1[k], o);
                            s2[k] = f2_fma(o, o, s2[k]);
                        }
                    }
                    if (bulk)
                    {
                        if (t.ow0 + quad * 32 >= g.out[2])
                            continue; // this warp's 32 outputs lie beyond the row
                        // registers -> staging buffer [filter][32 outputs] -> one bulk
                        // tensor store (clipped at the tensor's edges); the buffer
                        // used two rows ago must have been read by then
                        float* st = stage + (nstored & 1) * (SW_NBK * 32);
                        if (nstored >= 2)
                        {
                            if (lane == 0)
                                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                            __syncwarp();
                        }
                        const uint32_t st_s = smem_u32(st) + 4u * (uint32_t) lane;
                        if (alpha == 1.f)
                        {
                            // the usual case: the accumulator bits as they are
#pragma unroll
                            for (int k = 0; k < SW_NBK; ++k)
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(st_s + 128u * k), "r"(v[k]) : "memory");
                        }
                        else
                        {
#pragma unroll
                            for (int k = 0; k < SW_NBK; ++k)
                                asm volatile("st.shared.f32 [%0], %1;" ::"r"(st_s + 128u * k),
                                             "f"(alpha * __uint_as_float(v[k]))
                                             : "memory");
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0)
                        {
                            asm volatile(
                                "cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(
                                    reinterpret_cast<uint64_t>(&ymap)),
                                "r"(smem_u32(st)), "r"(t.ow0 + quad * 32), "r"(oh), "r"(od), "r"(0), "r"(t.n)
                                : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        ++nstored;
                        SW_PROF_MARK(3)
                    }
                    else if (ow < g.out[2])
                    {
#pragma unroll
                        for (int k = 0; k < SW_NBK; ++k)
                            if (k < nk)
                                yrow[(size_t) k * ysc] =
                                    BLEND ? alpha * __uint_as_float(v[k]) + beta * old[BLEND ? k : 0]
                                          : alpha * __uint_as_float(v[k]);
                    }
                }
            }
        }
        SW_PROF_FLUSH(prof)
        // the staged rows must have left shared memory before the CTA does
        if (bulk && lane == 0)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (STATS)
        {
            // lane k ends up with filter k's sum, lane 16 + k with its squares
            float mine = 0.f;
#pragma unroll
            for (int k = 0; k < (STATS ? SW_NBK : 1); ++k)
            {
                float a, b, a_odd, b_odd;
                f2_unpack(s1[k / 2], a, a_odd);
                f2_unpack(s2[k / 2], b, b_odd);
                if (k & 1)
                {
                    a = a_odd;
                    b = b_odd;
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
                {
                    a += __shfl_xor_sync(0xffffffffu, a, off);
                    b += __shfl_xor_sync(0xffffffffu, b, off);
                }
                if (lane == k)
                    mine = alpha * a;
                if (lane == SW_NBK + k)
                    mine = alpha * alpha * b;
            }
            stat_part[((size_t) blockIdx.x * EPI + ew) * 32 + lane] = mine;
        }
    }

    if (!ok && lane == 0)
        atomicExch(status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP)
    {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS)
                     : "memory");
    }
}

} // namespace
} // namespace dcb
