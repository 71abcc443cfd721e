// Device side of the tcgen05 / TMEM convolution: geometry record, PTX wrappers,
// the filter-image kernel and the convolution kernel itself.
#pragma once

#include "conv_simt.cuh"

#include <cuda.h>

namespace dcb
{
namespace
{

constexpr int TC_GROUPS_MAX = 3;                  // row groups of 4 converter warps
constexpr int TC_PRODUCERS = 4 * TC_GROUPS_MAX;   // warps 0..11: warp w -> group w / 4, TMEM quadrant w % 4
constexpr int TC_MMA_WARP = TC_PRODUCERS;         // warps 12..14: one MMA issuer per converter group
constexpr int TC_TMA_WARP = TC_PRODUCERS + TC_GROUPS_MAX; // warp 15 issues the bulk tensor loads
constexpr int TC_EPI_WARPS = 8;                   // warps 16..23 drain the accumulators, two per TMEM quadrant
constexpr int TC_THREADS = (TC_PRODUCERS + TC_GROUPS_MAX + 1 + TC_EPI_WARPS) * 32;
constexpr int TC_M = 128;
constexpr int TC_RAW_W = TC_M + 8;     // staged raw row: 4 cells left, 4 right
constexpr int TC_RAW_PRIV = 32 + 8;    // per-warp raw window when rows are fetched by the converters
constexpr uint32_t TC_TMEM_COLS = 512; // two accumulator buffers + the A ring

struct TcGeom
{
    int n, c, k;
    int in[3], out[3], f[3], pad[3];
    // A staged raw row holds the input cells from ow0 + lx on (lx a multiple of 4, what a
    // bulk copy can start at); tap kw of output ow0 + j sits rx + kw + j cells into it.
    // Set per launch from the input pointer's alignment (tc_row_window).
    int lx, rx;
    long long xs_n, xs_c, xs[3];
    long long ys_n, ys_c, ys[3];
    int split;   // 1: 3xTF32, 0: single TF32 pass
    // rounding of the operands' hi part, (bits + rnd_add) & rnd_mask: to TF32
    // (0x1000, 0xffffe000) or, in the bf16 mode, to bf16 (0x8000, 0xffff0000)
    uint32_t rnd_add, rnd_mask;
    int kpad;    // K rounded up to 8, 16 or 32
    int nb;      // accumulator columns per output row = kpad * (split ? 2 : 1)
    int th;      // output rows per tile
    int crows;   // c * fw
    int kr;      // k-rows per staged input row, multiple of 8
    int ksteps;  // kr / 8
    int ntot;    // fh * nb
    int b_bytes;
    int groups;     // converter row groups in use (1..3)
    int a_slots;    // A-operand ring in TMEM: slots of kr columns, a multiple of groups
    int acc_cols;   // th * nb, columns of one accumulator buffer
    int tiles_w, tiles_h;
    long long tiles;
    int use_tma;        // raw rows arrive by bulk tensor copies
    int raw_slots;      // ring of raw chunks in shared memory
    int raw_slot_bytes; // one chunk, rounded up to 128 bytes: c * chunk_rows * TC_RAW_W floats when
                        // bulk copies feed the ring, else one private window set per converter group
    int chunk_rows;     // staged rows per bulk copy
    int chunks_pp;      // bulk copies per filter plane of a tile
    // One launch covers c input channels and k filters; a convolution with more of
    // either runs as cgroups x kgroups launches on sub-ranges of the filter tensor
    // (the later channel groups add into the output).
    int c_total, k_total, w_c_off, w_k_off;
    int cgroups, kgroups;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t) __cvta_generic_to_shared(p);
}

// fp32 -> TF32, round to nearest with ties away from zero, as cvt.rna.tf32.f32
// does, but with two integer instructions: the cvt runs on the special-function
// pipe at an eighth of the integer rate, and the converters need several
// conversions per output.  (Inf / NaN payloads are not preserved; finite
// inputs give the same bits.)
__device__ __forceinline__ uint32_t tf32_rna(float x)
{
    return (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Bounded parity wait.  Returns false when the budget ran out.  Every role but
// the MMA issuer backs off between polls (SLEEP_NS > 0): a hot polling loop in
// a dozen warps would take the issue slots the MMA thread needs.
template <int SLEEP_NS>
__device__ __forceinline__ bool mbar_wait_t(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    const uint32_t addr = smem_u32(bar);
    long long t0 = 0;
    for (uint32_t it = 0; it < (1u << 24); ++it)
    {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done)
            return true;
        if (SLEEP_NS > 0)
            __nanosleep(SLEEP_NS);
        if ((it & 15) == 15 && *abort_flag)
            return false;
        if ((it & 255) == 255)
        {
            // a quarter of a second at most, whatever a poll costs
            const long long now = clock64();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > 500000000ll)
                break;
        }
    }
    *abort_flag = 1;
    return false;
}

#ifndef DCB_TC_WAIT_SLEEP_NS
#define DCB_TC_WAIT_SLEEP_NS 20
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    return mbar_wait_t<DCB_TC_WAIT_SLEEP_NS>(bar, parity, abort_flag);
}

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type)
{
    uint64_t d = 0;
    d |= (uint64_t) ((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t) ((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t) ((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46; // descriptor version for this architecture
    d |= (uint64_t) layout_type << 61;
    return d;
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_st16_zero(uint32_t taddr)
{
    const uint32_t z = 0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr),
        "r"(z)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Filter image for the B operand, built once per call from the fp32 filter.
__global__ void tc_pack_filter_kernel(const float* __restrict__ w, float* __restrict__ b, TcGeom g)
{
    const int fd = g.f[0], fh = g.f[1], fw = g.f[2];
    const long long total = (long long) fd * g.kr * g.ntot;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long) gridDim.x * blockDim.x)
    {
        // i enumerates the image in storage order
        const int ki = (int) (i % 4);
        const int ni = (int) ((i / 4) % 8);
        const int ngroup = (int) ((i / 32) % (g.ntot / 8));
        const int kchunk = (int) ((i / (32ll * (g.ntot / 8))) % 2);
        const int kstep = (int) ((i / (64ll * (g.ntot / 8))) % g.ksteps);
        const int kd = (int) (i / (64ll * (g.ntot / 8) * g.ksteps));
        const int krow = kstep * 8 + kchunk * 4 + ki;
        const int ncol = ngroup * 8 + ni;
        const int j = ncol / g.nb;          // block index, descending kh
        const int kh = fh - 1 - j;
        const int within = ncol % g.nb;
        const int half = within / g.kpad;   // 0: hi column, 1: lo column
        const int ko = within % g.kpad;
        const int part = krow / g.crows;    // 0: A_hi rows, 1: A_lo rows
        const int rem = krow % g.crows;
        const int c = rem / fw, kw = rem % fw;
        float val = 0.f;
        if (ko < g.k && part < (g.split ? 2 : 1))
        {
            const float wv =
                w[((((size_t) (ko + g.w_k_off) * g.c_total + (c + g.w_c_off)) * fd + kd) * fh + kh) * fw + kw];
            const float hi = __uint_as_float((__float_as_uint(wv) + g.rnd_add) & g.rnd_mask);
            if (half == 0)
                val = hi;
            else if (part == 0)
                val = __uint_as_float(tf32_rna(wv - hi));
        }
        b[i] = val;
    }
}

// The staged input rows of one tile, in issue order: filter planes kd in
// [kd_lo, kd_hi) x rows i in [i_lo, i_hi); everything outside lies in the zero
// padding and contributes nothing.
struct TileRows
{
    int n, od, oh0, ow0;
    int kd_lo, kd_hi, i_lo, i_hi;
    int nrows_i, count;
};

__device__ __forceinline__ TileRows tile_rows(const TcGeom& g, uint32_t tile)
{
    TileRows t;
    const uint32_t tw = tile % (uint32_t) g.tiles_w;
    uint32_t t2 = tile / (uint32_t) g.tiles_w;
    const uint32_t thi = t2 % (uint32_t) g.tiles_h;
    t2 /= (uint32_t) g.tiles_h;
    t.od = (int) (t2 % (uint32_t) g.out[0]);
    t.n = (int) (t2 / (uint32_t) g.out[0]);
    t.ow0 = (int) tw * TC_M;
    t.oh0 = (int) thi * g.th;
    t.kd_lo = max(0, g.pad[0] - t.od);
    t.kd_hi = min(g.f[0], g.in[0] + g.pad[0] - t.od);
    t.i_lo = max(0, g.pad[1] - t.oh0);
    t.i_hi = min(g.th + g.f[1] - 1, g.in[1] + g.pad[1] - t.oh0);
    t.nrows_i = max(0, t.i_hi - t.i_lo);
    t.count = max(0, t.kd_hi - t.kd_lo) * t.nrows_i;
    return t;
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 5-D tiled bulk copy global -> shared (no multicast), completion on an mbarrier.
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            int c4, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// D[tmem] += A[tmem] * B[smem]: the A operand is read from tensor memory
// (lane = row of the tile, 8 consecutive 32-bit columns = the 8 k-rows of the
// step).  An A operand fetched through a shared-memory descriptor costs about
// 120 clocks per instruction whatever N is; from tensor memory the
// instruction time follows N.
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

// Eight k-rows of one output column: hi or lo TF32 part of the tap the table
// names, or zero for a padding row.
__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}

// ktab8 / raw are shared-window addresses; the loads are explicit ld.shared so
// that they are issued back to back (generic loads were serialised).
__device__ __forceinline__ void convert_chunk(uint32_t ktab8, uint32_t raw_lane, uint32_t (&v)[8],
                                              uint32_t rnd_add = 0x1000u, uint32_t rnd_mask = 0xffffe000u)
{
    // All loads first and unconditional (a padding row reads cell 4 and is
    // zeroed afterwards), so the eight chains run in parallel without branches.
    uint32_t tb[8], xv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
        tb[e] = lds_u32(ktab8 + 4u * e);
#pragma unroll
    for (int e = 0; e < 8; ++e)
        xv[e] = lds_u32(raw_lane + ((tb[e] & 0xffffu) << 2));
#pragma unroll
    for (int e = 0; e < 8; ++e)
    {
        const uint32_t part = tb[e] >> 16;
        const float xe = part < 2 ? __uint_as_float(xv[e]) : 0.f;
        const uint32_t hi = (__float_as_uint(xe) + rnd_add) & rnd_mask;
        const uint32_t lo = tf32_rna(xe - __uint_as_float(hi));
        v[e] = part == 0 ? hi : lo;
    }
}

// Eight taps at once for rows whose tap count is a multiple of eight: the hi
// parts go to k-rows r0.., the lo parts to k-rows crows + r0.. (the table's
// first `crows` entries are the taps' offsets), each cell loaded and split once.
__device__ __forceinline__ void convert_pair(uint32_t ktab8, uint32_t raw_lane, uint32_t (&hi)[8], uint32_t (&lo)[8])
{
    uint32_t tb[8], xv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
        tb[e] = lds_u32(ktab8 + 4u * e);
#pragma unroll
    for (int e = 0; e < 8; ++e)
        xv[e] = lds_u32(raw_lane + ((tb[e] & 0xffffu) << 2));
#pragma unroll
    for (int e = 0; e < 8; ++e)
    {
        const float xe = __uint_as_float(xv[e]);
        hi[e] = tf32_rna(xe);
        lo[e] = __float_as_uint(xe - __uint_as_float(hi[e]));
    }
}

// The common case spelled out: 4 channels, 3 taps along W, pad 1, hi / lo
// split.  k-rows 0..11 are hi(c, kw), 12..23 lo(c, kw); no table, immediate
// offsets.  `pitch` is the raw window's channel pitch in floats.
__device__ __forceinline__ void convert_c4f3(uint32_t raw_lane, uint32_t pitch, uint32_t (&v)[3][8])
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
        const uint32_t lo = __float_as_uint(xe - __uint_as_float(hi)); // exact; the pipe reads its upper 19 bits
        v[r / 8][r % 8] = hi;
        v[(12 + r) / 8][(12 + r) % 8] = lo;
    }
}

// ---------------------------------------------------------------------------
// The convolution kernel.  One CTA per SM, 24 warps:
//   warp 15      streams raw input rows (all channels, 4 cells of margin each
//                side) into a shared-memory ring with bulk tensor copies, a
//                chunk of several rows per copy
//   warps 0..11  three groups of four; group g converts rows g, g+3, ... of
//                the CTA's row sequence: each lane takes one output column,
//                splits its c*fw taps into hi / lo TF32 and writes them as the
//                A operand straight into tensor memory (warp w may touch TMEM
//                lanes 32*(w%4).., hence four warps per row)
//   warps 12..14 issue tcgen05.mma (A from TMEM, B = filter image in shared
//                memory), one accumulator block range per staged row; issuer
//                q serves converter group q
//   warps 16..23 drain the accumulators: TMEM -> registers -> global
// TMEM columns: [acc 0][acc 1][A ring].  Accumulator buffers alternate between
// tiles, so a tile's epilogue overlaps the next tile's main loop.
//
// Barrier ownership.  A parity wait only tells the current phase from the
// previous one, so a barrier must never have a waiter that is two phases
// ahead.  The A ring therefore has a slot count that is a multiple of the
// group count and slot s is only ever used by group s % groups (its converter
// warps and its issuer), whose rows are processed in order.  A raw chunk is
// released by all converter warps together, so none of them can be a whole
// lap behind the copy warp.
// ---------------------------------------------------------------------------
template <int NB, bool C4F3>
__global__ void __launch_bounds__(TC_THREADS, 1)
    tc_conv_kernel(TcGeom g, float alpha, float beta, const float* __restrict__ x, const float* __restrict__ bimg,
                   float* y, int* status, const __grid_constant__ CUtensorMap xmap)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* b_smem = reinterpret_cast<float*>(smem);
    const int b_region = (g.b_bytes + 127) / 128 * 128;
    uint8_t* raw_ring = smem + b_region;
    uint32_t* ktab = reinterpret_cast<uint32_t*>(raw_ring + (size_t) g.raw_slots * g.raw_slot_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ktab + ((g.kr + 1) & ~1));
    uint64_t* a_full = bars;                    // [a_slots] converters -> MMA
    uint64_t* a_empty = a_full + g.a_slots;     // [a_slots] MMA -> converters
    uint64_t* acc_full = a_empty + g.a_slots;   // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;         // [2] epilogue -> MMA
    uint64_t* raw_full = acc_empty + 2;         // [raw_slots] copy -> converters
    uint64_t* raw_empty = raw_full + g.raw_slots; // [raw_slots] converters -> copy
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_empty + g.raw_slots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0)
    {
        for (int s = 0; s < g.a_slots; ++s)
        {
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b)
        {
            mbar_init(&acc_full[b], g.groups);
            mbar_init(&acc_empty[b], TC_EPI_WARPS);
        }
        for (int r = 0; r < g.raw_slots; ++r)
        {
            mbar_init(&raw_full[r], 1);
            mbar_init(&raw_empty[r], 4 * g.groups);
        }
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
    // k-row table: where in a raw row the tap of k-row r sits, and whether the
    // row carries the hi part (0), the lo part (1) or padding (2)
    for (int r = tid; r < g.kr; r += TC_THREADS)
    {
        const int part = r / g.crows, rem = r % g.crows;
        const int c = rem / g.f[2], kw = rem % g.f[2];
        const uint32_t off = (uint32_t) (c * (g.use_tma ? g.chunk_rows * TC_RAW_W : TC_RAW_PRIV) + g.rx + kw);
        ktab[r] = (part < (g.split ? 2 : 1)) ? (off | ((uint32_t) part << 16)) : ((2u << 16) | 4u);
    }
    for (int i = tid; i < g.b_bytes / 16; i += TC_THREADS)
        reinterpret_cast<float4*>(b_smem)[i] = reinterpret_cast<const float4*>(bimg)[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_col0 = 2u * (uint32_t) g.acc_cols; // first column of the A ring
    const uint32_t ntiles = (uint32_t) g.tiles;
    bool ok = true;

    if (warp < 4 * g.groups)
    {
        // ------------------------------------------------------------------
        // converters
        // ------------------------------------------------------------------
        const int G = g.groups, gq = warp >> 2, quad = warp & 3;
        const int mcol = g.use_tma ? quad * 32 + lane : lane; // column inside the raw window
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        const int laps_a = g.a_slots / G;
        const uint32_t ktab_s = smem_u32(ktab);
        // bulk-copy mode: a filter plane of the tile arrives as chunks_pp chunks
        // of Rc rows; otherwise the plane is one "chunk" that nothing copies
        const int Rc = g.use_tma ? g.chunk_rows : (1 << 20), chunks_pp = g.use_tma ? g.chunks_pp : 1;
        const int pitch = g.use_tma ? g.chunk_rows * TC_RAW_W : TC_RAW_PRIV; // channel pitch of a raw window
        int lap_a = 0;
        uint32_t cslot = 0, cphase = 0; // position in the chunk ring
        uint32_t a_phase = 1;           // parity of the A-slot release to wait for
        bool a_first = true;
        uint32_t base = 0; // (sequence number of the tile's first row) % G
        for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x)
        {
            const TileRows t = tile_rows(g, tile);
            for (int kd = t.kd_lo; kd < t.kd_hi && ok; ++kd)
                for (int ch = 0; ch < chunks_pp && ok; ++ch)
                {
            const int lo = max(t.i_lo, ch * Rc), hi = min(t.i_hi, (ch + 1) * Rc);
            if (lo >= hi)
                continue; // nothing but padding: the copy warp skips it too
            // rows are dealt to the groups in the tile's issue order; this
            // group's first row of the chunk:
            const uint32_t first_q = (uint32_t) ((kd - t.kd_lo) * t.nrows_i + (lo - t.i_lo));
            int i = lo + (gq + G - (int) ((base + first_q) % (uint32_t) G)) % G;
            bool have = false;
            for (; i < hi && ok; i += G)
            {
                const int a_slot = gq + G * lap_a;
                // bulk-copy mode: row i of the chunk, indexed by m; otherwise
                // this warp's private 40-cell window, indexed by lane
                float* raw = g.use_tma ? reinterpret_cast<float*>(raw_ring + (size_t) cslot * g.raw_slot_bytes)
                                             + (i - ch * Rc) * TC_RAW_W
                                       : reinterpret_cast<float*>(raw_ring + (size_t) gq * g.raw_slot_bytes)
                                             + quad * g.c * TC_RAW_PRIV;
                if (g.use_tma)
                {
                    if (!have)
                        ok = mbar_wait(&raw_full[cslot], cphase, abort_flag);
                    have = true;
                }
                else
                {
                    // any alignment: every warp fetches the 32 + 8 cells per
                    // channel that its own lanes need into its private part
                    // of the slot (no cross-warp hand-off, so no barrier)
                    __syncwarp();
                    const float* src = x + (size_t) t.n * g.xs_n + (size_t) (t.od - g.pad[0] + kd) * g.xs[0]
                                       + (size_t) (t.oh0 - g.pad[1] + i) * g.xs[1];
                    for (int e = lane; e < g.c * TC_RAW_PRIV; e += 32)
                    {
                        const int c = e / TC_RAW_PRIV, j = e - c * TC_RAW_PRIV;
                        const int iw = t.ow0 + quad * 32 + g.lx + j;
                        raw[e] = (iw >= 0 && iw < g.in[2]) ? src[(size_t) c * g.xs_c + iw] : 0.f;
                    }
                    __syncwarp();
                }
                if (!ok)
                    break;
                const uint32_t a_addr = lane_addr + a_col0 + (uint32_t) (a_slot * g.kr);
                const uint32_t raw_s = smem_u32(raw) + 4u * (uint32_t) mcol;
                if (C4F3)
                {
                    uint32_t v[3][8];
                    // the converter is written for taps that start 3 cells into the staged row
                    convert_c4f3(raw_s + 4u * (uint32_t) (g.rx - 3), (uint32_t) pitch, v);
                    if (!a_first)
                        ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                    if (!ok)
                        break;
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < 3; ++ch)
                        tmem_st8(a_addr + (uint32_t) (ch * 8), v[ch]);
                }
                else if (g.kr <= 32)
                {
                    // convert into registers first, so the split overlaps the
                    // MMAs that still read this slot's previous row
                    uint32_t v[4][8];
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
                        if (ch * 8 < g.kr)
                            convert_chunk(ktab_s + 32u * ch, raw_s, v[ch], g.rnd_add, g.rnd_mask);
                    if (!a_first)
                        ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                    if (!ok)
                        break;
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
                        if (ch * 8 < g.kr)
                            tmem_st8(a_addr + (uint32_t) (ch * 8), v[ch]);
                }
                else
                {
                    if (!a_first)
                        ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                    if (!ok)
                        break;
                    tc_fence_after();
                    if (g.split && (g.crows & 7) == 0)
                    {
                        for (int r0 = 0; r0 < g.crows; r0 += 8)
                        {
                            uint32_t hi[8], lo[8];
                            convert_pair(ktab_s + 4u * r0, raw_s, hi, lo);
                            tmem_st8(a_addr + (uint32_t) r0, hi);
                            tmem_st8(a_addr + (uint32_t) (g.crows + r0), lo);
                        }
                    }
                    else
                    {
                        for (int r0 = 0; r0 < g.kr; r0 += 8)
                        {
                            uint32_t v[8];
                            convert_chunk(ktab_s + 4u * r0, raw_s, v, g.rnd_add, g.rnd_mask);
                            tmem_st8(a_addr + (uint32_t) r0, v);
                        }
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&a_full[a_slot]);
                if (++lap_a == laps_a)
                {
                    lap_a = 0;
                    a_phase ^= 1;
                    a_first = false;
                }
            }
            if (g.use_tma)
            {
                // every converter warp releases every chunk, with or without
                // rows of its own in it
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
            base = (base + (uint32_t) t.count) % (uint32_t) G;
        }
    }
    else if (warp == TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // bulk tensor copies of raw input rows, one chunk (chunk_rows rows of
        // every channel) per instruction, raw_slots chunks ahead.  Issuing a
        // copy costs this thread a few hundred clocks whatever its size, so
        // row-sized copies cannot feed the converters.  The whole warp walks
        // the schedule, lane 0 issues.
        // ------------------------------------------------------------------
        if (g.use_tma)
        {
            const uint32_t bytes = (uint32_t) (g.c * g.chunk_rows) * TC_RAW_W * 4u;
            const int Rc = g.chunk_rows;
            uint32_t slot = 0, empty_phase = 1;
            bool first_lap = true;
            for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x)
            {
                const TileRows t = tile_rows(g, tile);
                for (int kd = t.kd_lo; kd < t.kd_hi && ok; ++kd)
                    for (int ch = 0; ch < g.chunks_pp; ++ch)
                    {
                        if (max(t.i_lo, ch * Rc) >= min(t.i_hi, (ch + 1) * Rc))
                            continue; // the converters skip the same chunks
                        if (!first_lap)
                            ok = mbar_wait(&raw_empty[slot], empty_phase, abort_flag);
                        if (!ok)
                            break;
                        if (lane == 0)
                        {
                            mbar_expect_tx(&raw_full[slot], bytes);
                            // x starts 4 cells left of the tile: a multiple of
                            // 4 floats, as the 16-byte rule for the innermost
                            // coordinate demands; rows above or below the
                            // image arrive as zeros and are never converted
                            tma_load_5d(raw_ring + (size_t) slot * g.raw_slot_bytes, &xmap, t.ow0 + g.lx,
                                        t.oh0 - g.pad[1] + ch * Rc, t.od - g.pad[0] + kd, 0, t.n, &raw_full[slot]);
                        }
                        __syncwarp();
                        if (++slot == (uint32_t) g.raw_slots)
                        {
                            slot = 0;
                            empty_phase ^= 1;
                            first_lap = false;
                        }
                    }
            }
        }
    }
    else if (warp >= TC_MMA_WARP && warp < TC_MMA_WARP + TC_GROUPS_MAX)
    {
        // ------------------------------------------------------------------
        // MMA issue.  Issuing one tcgen05.mma costs the issuing thread about
        // 150 clocks whatever its shape, three times what the tensor pipe
        // needs for it here, and several warps can issue concurrently: so
        // every converter group has an issuer of its own (issuer mq takes the
        // rows that group mq converts), and a private A slot ring between the
        // two.  Rows of different issuers reach the pipe in no fixed order;
        // they only ever add into the accumulators, so the sum is the same up
        // to fp32 rounding order.
        // Within an issuer the whole warp walks the schedule and the
        // instructions of staged row i are issued by lane i, which worked out
        // that row's instruction descriptor, accumulator offset and filter
        // image offset once (they depend on i only).
        // ------------------------------------------------------------------
        const int G = g.groups, mq = warp - TC_MMA_WARP;
        if (mq < G)
        {
            const int fh = g.f[1];
            const int my_i = lane; // the staged row this lane issues
            const int j_lo = max(0, fh - 1 - my_i);
            const int j_hi = min(fh, g.th + fh - 1 - my_i);
            // fp32 accumulate, tf32 x tf32, A K-major (tensor memory), B K-major, M = 128
            const uint32_t my_idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((TC_M >> 4) << 24)
                                      | ((uint32_t) ((max(1, j_hi - j_lo) * NB) >> 3) << 17);
            const uint32_t my_d_off = (uint32_t) ((my_i - fh + 1 + j_lo) * NB);
            const uint32_t b_lbo = (uint32_t) (g.ntot / 8) * 128u;
            const uint32_t b_kstep_units = ((uint32_t) g.ntot * 32u) >> 4;
            const uint64_t my_b_desc =
                make_desc(smem_u32(b_smem), b_lbo, 128u, 0u) + (uint64_t) ((uint32_t) j_lo * NB);
            const uint32_t kd_units = (uint32_t) g.ksteps * b_kstep_units;
            const uint32_t a_ring = tmem_base + a_col0;
            const int ksteps = g.ksteps;
            const int laps_a = g.a_slots / G;
            int lap_a = 0;
            uint32_t full_phase = 0, tcount = 0, base = 0;
            for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount)
            {
                const TileRows t = tile_rows(g, tile);
                const uint32_t buf = tcount & 1;
                ok = mbar_wait_t<0>(&acc_empty[buf], (tcount >> 1) & 1, abort_flag);
                if (!ok)
                    break;
                const uint32_t my_d = tmem_base + buf * (uint32_t) g.acc_cols + my_d_off;
                int q = (mq + G - (int) base) % G; // this issuer's first row of the tile
                int kd = t.kd_lo, i = t.i_lo + q;
                bool any = false;
                for (; q < t.count && ok; q += G, i += G)
                {
                    while (i >= t.i_hi)
                    {
                        i -= t.nrows_i;
                        ++kd;
                    }
                    const uint32_t slot = (uint32_t) (mq + G * lap_a);
                    ok = mbar_wait_t<0>(&a_full[slot], full_phase, abort_flag);
                    if (!ok)
                        break;
                    tc_fence_after();
                    if (lane == i)
                    {
                        uint32_t a_addr = a_ring + slot * (uint32_t) g.kr;
                        uint64_t bd = my_b_desc + (uint64_t) ((uint32_t) kd * kd_units);
                        for (int ks = 0; ks < ksteps; ++ks)
                        {
                            mma_tf32_ts(my_d, a_addr, bd, my_idesc);
                            a_addr += 8;
                            bd += b_kstep_units;
                        }
                        mma_commit(&a_empty[slot]);
                        // This issuer's last row of the tile also reports to
                        // the epilogue; the accumulators are complete once
                        // every issuer has (the tensor pipe retires MMAs in
                        // issue order, so a commit covers this warp's earlier
                        // rows too).
                        if (q + G >= t.count)
                            mma_commit(&acc_full[buf]);
                        tc_fence_before();
                    }
                    __syncwarp();
                    any = true;
                    if (++lap_a == laps_a)
                    {
                        lap_a = 0;
                        full_phase ^= 1;
                    }
                }
                // an issuer without a row in this tile still has to report
                if (!any && ok && lane == 0)
                    mbar_arrive(&acc_full[buf]);
                base = (base + (uint32_t) t.count) % (uint32_t) G;
            }
        }
    }
    else if (warp > TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // epilogue: TMEM -> registers -> global, then re-zero what was read.
        // Two warps per TMEM quadrant share a tile's rows (even / odd): a
        // tensor-memory load takes long while MMAs are in flight, and eight
        // warps keep enough of them outstanding.
        // ------------------------------------------------------------------
        const int quad = warp & 3; // TMEM lanes this warp may touch
        const int half = (warp - TC_TMA_WARP - 1) >> 2, nhalf = TC_EPI_WARPS / 4;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        if (half == 0)
            for (int col = 0; col < 2 * g.acc_cols; col += 16)
                tmem_st16_zero(lane_addr + col);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
        {
            mbar_arrive(&acc_empty[0]);
            mbar_arrive(&acc_empty[1]);
        }
        uint32_t tcount = 0;
        for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount)
        {
            const TileRows t = tile_rows(g, tile);
            const int ow = t.ow0 + quad * 32 + lane;
            const uint32_t buf = tcount & 1;
            ok = mbar_wait(&acc_full[buf], (tcount >> 1) & 1, abort_flag);
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t acc_addr = lane_addr + buf * (uint32_t) g.acc_cols;
            for (int r = half; r < g.th; r += nhalf)
            {
                const int oh = t.oh0 + r;
                if (oh >= g.out[1])
                    break; // uniform
                uint32_t v[NB];
#pragma unroll
                for (int q = 0; q < NB / 16; ++q)
                    tmem_ld16(acc_addr + (uint32_t) (r * NB + q * 16), *reinterpret_cast<uint32_t(*)[16]>(&v[q * 16]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ow < g.out[2])
                {
                    float* yp = y + (size_t) t.n * g.ys_n + (size_t) t.od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
                    const int kp = g.split ? NB / 2 : NB;
                    const int nk = g.k < kp ? g.k : kp;
                    const size_t ysc = (size_t) g.ys_c;
                    // the hi and lo halves of the split land in separate columns
                    if (g.split)
                    {
#pragma unroll
                        for (int k = 0; k < NB / 2; ++k)
                            v[k] = __float_as_uint(__uint_as_float(v[k]) + __uint_as_float(v[k + NB / 2]));
                    }
                    // straight-line stores: a test of beta per filter costs
                    // more than the stores themselves
                    if (beta == 0.f)
                    {
#pragma unroll
                        for (int k = 0; k < NB; ++k)
                            if (k < nk)
                                yp[(size_t) k * ysc] = alpha * __uint_as_float(v[k]);
                    }
                    else
                    {
#pragma unroll
                        for (int k = 0; k < NB; ++k)
                            if (k < nk)
                                yp[(size_t) k * ysc] = alpha * __uint_as_float(v[k]) + beta * yp[(size_t) k * ysc];
                    }
                }
            }
            // every warp re-zeroes the rows that are its to read (also those
            // below the image, which the MMAs wrote all the same)
            for (int r = half; r < g.th; r += nhalf)
                for (int col = 0; col < NB; col += 16)
                    tmem_st16_zero(acc_addr + (uint32_t) (r * NB + col));
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[buf]);
        }
    }

    if (!ok && lane == 0)
        atomicExch(status, 1);
    // Every role leaves its loop after a bounded time (all waits are bounded
    // and watch the abort flag), so the block-wide barrier is always reached.
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
