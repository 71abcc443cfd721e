// tcgen05 / TMEM implicit-GEMM convolution (stride 1, dilation 1), NC[D]HW.
//
// GEMM view.  One MMA tile is 128 consecutive outputs of one output row
// (M = 128 along W, the contiguous dimension, so the A operand is MN-major).
// For one staged input row (id, ih) the reduction index ("k-rows") runs over
// (c, kw): row (c, kw) is that input row shifted by kw - pad_w.  With the
// 3xTF32 split the k-rows are [A_hi ; A_lo] and the B operand for filter row
// kh is the 2-block [[w_hi | w_lo] ; [w_hi | 0]], so a_hi*w_hi + a_hi*w_lo +
// a_lo*w_hi lands in two column halves that the epilogue adds.
//
// A staged input row serves fh output rows (oh = ih + pad_h - kh).  Their B
// blocks are concatenated along N in descending kh, which makes the target
// accumulators of one MMA consecutive output rows: one instruction of
// N = fh * NB columns updates fh accumulator blocks at once, and the A row is
// read from shared memory once instead of fh times.
//
// Layouts (all staged by the CTA's own threads, since hi/lo splitting and the
// kw shifts need a pass over the data anyway):
//   A stage  [k-group][m-atom(4)][4 k-rows][128 B], MN-major, 128-byte swizzle
//            with 32-byte base (the only MN-major layout TF32 operands take):
//            32-byte chunk index XOR k-row index within each 512-byte atom
//   B        [kd][k-step][2 k-chunks][N/8][8 n][4 k] floats, no swizzle, K-major
//   D        TMEM, lane = output within the tile, column = r * NB + n
//
// Every wait on an mbarrier is bounded; on expiry the kernel records an error,
// releases its TMEM and returns.
#include "conv_tc.cuh"

#include <cuda.h>

namespace dcb
{

namespace
{

constexpr int TC_PRODUCERS = 12;             // warps 0..11 convert staged rows
constexpr int TC_MMA_WARP = TC_PRODUCERS;     // warp 12 issues the MMAs
constexpr int TC_TMA_WARP = TC_PRODUCERS + 1; // warp 13 issues the bulk tensor loads
constexpr int TC_THREADS = (TC_PRODUCERS + 6) * 32; // + epilogue warps 14..17
constexpr int TC_M = 128;
constexpr int TC_RAW_W = TC_M + 8;     // staged raw row: 4 cells left, 4 right
constexpr uint32_t TC_TMEM_COLS = 512; // two accumulator buffers
constexpr int TC_ACC_COLS = 256;

struct TcGeom
{
    int n, c, k;
    int in[3], out[3], f[3], pad[3];
    long long xs_n, xs_c, xs[3];
    long long ys_n, ys_c, ys[3];
    int split;   // 1: 3xTF32, 0: single TF32 pass
    int kpad;    // K rounded up to 8, 16 or 32
    int nb;      // accumulator columns per output row = kpad * (split ? 2 : 1)
    int th;      // output rows per tile
    int crows;   // c * fw
    int kr;      // k-rows per staged input row, multiple of 8
    int ksteps;  // kr / 8
    int ntot;    // fh * nb
    int stages;
    int a_stage_bytes;
    int b_bytes;
    int tiles_w, tiles_h;
    long long tiles;
    int nprod;          // producer warps in use (= stages, see the kernel)
    int use_tma;        // raw rows arrive by bulk tensor copies
    int raw_slots;      // ring of raw rows
    int raw_slot_bytes; // c * TC_RAW_W floats, rounded up to 128 bytes
};

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t) __cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t tf32_rna(float x)
{
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return u;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Bounded parity wait.  Returns false when the budget ran out.  try_wait itself
// suspends the thread for a hardware-chosen interval, so the loop is not hot.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 22); ++it)
    {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(1000u)
            : "memory");
        if (done)
            return true;
        if ((it & 15) == 15 && *abort_flag)
            return false;
    }
    *abort_flag = 1;
    return false;
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
            const float wv = w[((((size_t) ko * g.c + c) * fd + kd) * fh + kh) * fw + kw];
            const float hi = __uint_as_float(tf32_rna(wv));
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

__device__ __forceinline__ TileRows tile_rows(const TcGeom& g, long long tile)
{
    TileRows t;
    const int tw = (int) (tile % g.tiles_w);
    long long t2 = tile / g.tiles_w;
    const int thi = (int) (t2 % g.tiles_h);
    t2 /= g.tiles_h;
    t.od = (int) (t2 % g.out[0]);
    t.n = (int) (t2 / g.out[0]);
    t.ow0 = tw * TC_M;
    t.oh0 = thi * g.th;
    t.kd_lo = max(0, g.pad[0] - t.od);
    t.kd_hi = min(g.f[0], g.in[0] + g.pad[0] - t.od);
    t.i_lo = max(0, g.pad[1] - t.oh0);
    t.i_hi = min(g.th + g.f[1] - 1, g.in[1] + g.pad[1] - t.oh0);
    t.nrows_i = max(0, t.i_hi - t.i_lo);
    t.count = max(0, t.kd_hi - t.kd_lo) * t.nrows_i;
    return t;
}

// ext = {l2, l3, v0, v1, v2, v3, r0, r1}; the chunk for a tap shifted by s
// cells is ext[2 + s .. 5 + s].
__device__ __forceinline__ uint4 pick_shift(const uint32_t (&e)[8], int s)
{
    switch (s)
    {
    case -2: return make_uint4(e[0], e[1], e[2], e[3]);
    case -1: return make_uint4(e[1], e[2], e[3], e[4]);
    case 1: return make_uint4(e[3], e[4], e[5], e[6]);
    case 2: return make_uint4(e[4], e[5], e[6], e[7]);
    default: return make_uint4(e[2], e[3], e[4], e[5]);
    }
}

// Byte offset of a lane's 16-byte chunk inside a stage for k-row kr:
// [k-group][m-atom][4 k-rows][128 B] with the 32-byte-base XOR swizzle.
// lane_part holds the lane-dependent bits (m-atom, 32-byte chunk, 16-byte
// half); the k-row phase r = kr & 3 is XORed into the 32-byte chunk index.
__device__ __forceinline__ uint32_t a_chunk_off(int kr, uint32_t lane_part)
{
    const uint32_t r = (uint32_t) (kr & 3);
    return (uint32_t) ((kr >> 2) << 11) + (r << 7) + (lane_part ^ (r << 5));
}

// One channel of one staged row: ext holds the 8 cells around the lane's
// chunk.  Writes the fw shifted copies of hi (and lo) into the stage.
template <int FW, int PW>
__device__ __forceinline__ void store_channel(const TcGeom& g, uint8_t* a_stage, int c, const float (&ext)[8],
                                              uint32_t lane_part)
{
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int t = 0; t < 8; ++t)
    {
        hi[t] = tf32_rna(ext[t]);
        lo[t] = tf32_rna(ext[t] - __uint_as_float(hi[t]));
    }
    if (FW > 0)
    {
#pragma unroll
        for (int kw = 0; kw < FW; ++kw)
        {
            const int kr = c * FW + kw;
            *reinterpret_cast<uint4*>(a_stage + a_chunk_off(kr, lane_part)) = pick_shift(hi, kw - PW);
            if (g.split)
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(g.crows + kr, lane_part)) = pick_shift(lo, kw - PW);
        }
    }
    else
    {
        const int fw = g.f[2], pw = g.pad[2];
        for (int kw = 0; kw < fw; ++kw)
        {
            const int kr = c * fw + kw;
            *reinterpret_cast<uint4*>(a_stage + a_chunk_off(kr, lane_part)) = pick_shift(hi, kw - pw);
            if (g.split)
                *reinterpret_cast<uint4*>(a_stage + a_chunk_off(g.crows + kr, lane_part)) = pick_shift(lo, kw - pw);
        }
    }
}

// Row fed from a raw copy in shared memory: raw[j] = x[ow0 - 4 + j], zero
// outside the tensor (the bulk tensor copy fills out-of-range cells).
template <int FW, int PW>
__device__ __forceinline__ void convert_row_smem(const TcGeom& g, const float* raw, uint8_t* a_stage, int lane,
                                                 uint32_t lane_part)
{
    for (int c = 0; c < g.c; ++c)
    {
        const float4* rr = reinterpret_cast<const float4*>(raw + (size_t) c * TC_RAW_W);
        const float4 a = rr[lane], b = rr[lane + 1], d = rr[lane + 2];
        const float ext[8] = {a.z, a.w, b.x, b.y, b.z, b.w, d.x, d.y};
        store_channel<FW, PW>(g, a_stage, c, ext, lane_part);
    }
}

// Row fed straight from global memory (any alignment): the lane loads its
// chunk, the neighbours' cells come by shuffle, the tile edges by extra loads.
template <int FW, int PW>
__device__ __forceinline__ void convert_row_gmem(const TcGeom& g, const float* __restrict__ x, int n, int id,
                                                 int ih, int ow0, uint8_t* a_stage, int lane,
                                                 uint32_t lane_part)
{
    const float* base = x + (size_t) n * g.xs_n + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1];
    const int iw0 = ow0 + 4 * lane;
    const int wi = g.in[2];
    for (int c = 0; c < g.c; ++c)
    {
        const float* xr = base + (size_t) c * g.xs_c;
        float4 v;
        if (iw0 + 3 < wi && (reinterpret_cast<uintptr_t>(xr + iw0) & 15) == 0)
        {
            v = *reinterpret_cast<const float4*>(xr + iw0);
        }
        else
        {
            v.x = iw0 + 0 < wi ? xr[iw0 + 0] : 0.f;
            v.y = iw0 + 1 < wi ? xr[iw0 + 1] : 0.f;
            v.z = iw0 + 2 < wi ? xr[iw0 + 2] : 0.f;
            v.w = iw0 + 3 < wi ? xr[iw0 + 3] : 0.f;
        }
        float ext[8];
        ext[2] = v.x;
        ext[3] = v.y;
        ext[4] = v.z;
        ext[5] = v.w;
        ext[1] = __shfl_up_sync(0xffffffffu, v.w, 1);
        ext[0] = __shfl_up_sync(0xffffffffu, v.z, 1);
        ext[6] = __shfl_down_sync(0xffffffffu, v.x, 1);
        ext[7] = __shfl_down_sync(0xffffffffu, v.y, 1);
        if (lane == 0)
        {
            ext[1] = (iw0 - 1 >= 0 && iw0 - 1 < wi) ? xr[iw0 - 1] : 0.f;
            ext[0] = (iw0 - 2 >= 0 && iw0 - 2 < wi) ? xr[iw0 - 2] : 0.f;
        }
        if (lane == 31)
        {
            ext[6] = iw0 + 4 < wi ? xr[iw0 + 4] : 0.f;
            ext[7] = iw0 + 5 < wi ? xr[iw0 + 5] : 0.f;
        }
        store_channel<FW, PW>(g, a_stage, c, ext, lane_part);
    }
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Warp roles.  Warps 0..TC_PRODUCERS-1 each convert whole staged rows (row
// number `it` of the CTA's sequence belongs to warp it % TC_PRODUCERS, so that
// many rows are converted concurrently and the converting warps hide each
// other's instruction latency); the MMA warp issues tcgen05.mma in sequence
// order; the copy warp streams raw rows in with bulk tensor copies; four
// epilogue warps drain the accumulators.  Two accumulator buffers of 256 TMEM
// columns alternate between tiles, so a tile's epilogue overlaps the next
// tile's main loop.
template <int NB, int FW, int PW>
__global__ void __launch_bounds__(TC_THREADS, 1)
    tc_conv_kernel(TcGeom g, float alpha, float beta, const float* __restrict__ x, const float* __restrict__ bimg,
                   float* y, int* status, const __grid_constant__ CUtensorMap xmap)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment keeps the hardware swizzle phase equal to the one
    // used when writing the tiles.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem;
    float* b_smem = reinterpret_cast<float*>(smem + (size_t) g.stages * g.a_stage_bytes);
    const int b_region = (g.b_bytes + 127) / 128 * 128;
    uint8_t* raw_ring = reinterpret_cast<uint8_t*>(b_smem) + b_region;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw_ring + (size_t) g.raw_slots * g.raw_slot_bytes);
    uint64_t* full_bar = bars;                     // [stages] producer -> MMA
    uint64_t* empty_bar = bars + g.stages;         // [stages] MMA -> producer
    uint64_t* acc_full = bars + 2 * g.stages;      // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * g.stages + 2; // [2] epilogue -> MMA
    uint64_t* raw_full = bars + 2 * g.stages + 4;                // [raw_slots] copy -> producer
    uint64_t* raw_empty = bars + 2 * g.stages + 4 + g.raw_slots; // [raw_slots] producer -> copy
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * g.stages + 4 + 2 * g.raw_slots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0)
    {
        for (int s = 0; s < g.stages; ++s)
        {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b)
        {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        for (int r = 0; r < g.raw_slots; ++r)
        {
            mbar_init(&raw_full[r], 1);
            mbar_init(&raw_empty[r], 1);
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
    // zero the A ring once: padding k-rows must hold finite values
    for (int i = tid; i < g.stages * g.a_stage_bytes / 16; i += TC_THREADS)
        reinterpret_cast<float4*>(a_ring)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = tid; i < g.b_bytes / 16; i += TC_THREADS)
        reinterpret_cast<float4*>(b_smem)[i] = reinterpret_cast<const float4*>(bimg)[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp < g.nprod)
    {
        // ------------------------------------------------------------------
        // producers: raw row -> hi / lo split -> fw shifted copies in the
        // swizzled stage.  Row `it` belongs to warp it % nprod, and with
        // stages == nprod and raw_slots a multiple of nprod every stage and
        // raw slot is only ever touched by one producer warp, in order.  That
        // matters: a parity wait is only meaningful for the current or the
        // previous phase of a barrier, so a warp must never wait on a barrier
        // whose earlier phase another, possibly slower, warp still owes.
        // ------------------------------------------------------------------
        const int nprod = g.nprod;
        const uint32_t lane_part =
            (uint32_t) ((lane >> 3) << 9) + (uint32_t) (((lane & 7) >> 1) << 5) + (uint32_t) ((lane & 1) << 4);
        uint32_t base = 0; // sequence number of the tile's first row
        for (long long tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x)
        {
            const TileRows t = tile_rows(g, tile);
            // first row of this tile that belongs to this warp
            uint32_t q = (uint32_t) ((warp + nprod - (int) (base % nprod)) % nprod);
            for (; q < (uint32_t) t.count && ok; q += nprod)
            {
                const uint32_t it = base + q;
                const int kd = t.kd_lo + (int) q / t.nrows_i;
                const int i = t.i_lo + (int) q % t.nrows_i;
                const int id = t.od - g.pad[0] + kd, ih = t.oh0 - g.pad[1] + i;
                const uint32_t s = it % g.stages;
                uint32_t slot = 0;
                if (g.use_tma)
                {
                    slot = it % g.raw_slots;
                    ok = mbar_wait(&raw_full[slot], (it / g.raw_slots) & 1, abort_flag);
                    if (!ok)
                        break;
                }
                if (it >= (uint32_t) g.stages)
                    ok = mbar_wait(&empty_bar[s], ((it / g.stages) - 1) & 1, abort_flag);
                if (!ok)
                    break;
                uint8_t* a_stage = a_ring + (size_t) s * g.a_stage_bytes;
                if (g.use_tma)
                    convert_row_smem<FW, PW>(g, reinterpret_cast<const float*>(raw_ring + (size_t) slot * g.raw_slot_bytes),
                                             a_stage, lane, lane_part);
                else
                    convert_row_gmem<FW, PW>(g, x, t.n, id, ih, t.ow0, a_stage, lane, lane_part);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0)
                {
                    mbar_arrive(&full_bar[s]);
                    if (g.use_tma)
                        mbar_arrive(&raw_empty[slot]);
                }
            }
            base += (uint32_t) t.count;
        }
    }
    else if (warp == TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // bulk tensor copies of raw input rows, raw_slots rows ahead
        // ------------------------------------------------------------------
        if (lane == 0 && g.use_tma)
        {
            uint32_t it = 0;
            const uint32_t bytes = (uint32_t) g.c * TC_RAW_W * 4u;
            for (long long tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x)
            {
                const TileRows t = tile_rows(g, tile);
                for (int kd = t.kd_lo; kd < t.kd_hi && ok; ++kd)
                    for (int i = t.i_lo; i < t.i_hi; ++i, ++it)
                    {
                        const uint32_t slot = it % g.raw_slots;
                        if (it >= (uint32_t) g.raw_slots)
                            ok = mbar_wait(&raw_empty[slot], ((it / g.raw_slots) - 1) & 1, abort_flag);
                        if (!ok)
                            break;
                        mbar_expect_tx(&raw_full[slot], bytes);
                        // x starts 4 cells left of the tile: a multiple of 4
                        // floats, as the 16-byte rule for the innermost
                        // coordinate demands
                        tma_load_5d(raw_ring + (size_t) slot * g.raw_slot_bytes, &xmap, t.ow0 - 4,
                                    t.oh0 - g.pad[1] + i, t.od - g.pad[0] + kd, 0, t.n, &raw_full[slot]);
                    }
            }
        }
    }
    else if (warp == TC_MMA_WARP)
    {
        // ------------------------------------------------------------------
        // MMA issue: one thread
        // ------------------------------------------------------------------
        if (lane == 0)
        {
            // instruction descriptor without N: fp32 accumulate, tf32 x tf32,
            // A MN-major, B K-major, M = 128
            const uint32_t idesc_base =
                (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (0u << 16) | ((TC_M >> 4) << 24);
            const uint32_t a_base = smem_u32(a_ring);
            const uint32_t b_base = smem_u32(b_smem);
            const uint32_t b_lbo = (uint32_t) (g.ntot / 8) * 128u;
            const uint32_t b_kstep_bytes = (uint32_t) g.ntot * 32u;
            const int fh = g.f[1];
            uint32_t it = 0, tcount = 0;
            for (long long tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x, ++tcount)
            {
                const TileRows t = tile_rows(g, tile);
                const uint32_t buf = tcount & 1;
                ok = mbar_wait(&acc_empty[buf], (tcount >> 1) & 1, abort_flag);
                if (!ok)
                    break;
                for (int kd = t.kd_lo; kd < t.kd_hi && ok; ++kd)
                    for (int i = t.i_lo; i < t.i_hi; ++i, ++it)
                    {
                        const uint32_t s = it % g.stages;
                        ok = mbar_wait(&full_bar[s], (it / g.stages) & 1, abort_flag);
                        if (!ok)
                            break;
                        tc_fence_after();
                        const int j_lo = max(0, fh - 1 - i);
                        const int j_hi = min(fh, g.th + fh - 1 - i);
                        const uint32_t idesc = idesc_base | ((uint32_t) (((j_hi - j_lo) * NB) >> 3) << 17);
                        const uint32_t d_addr =
                            tmem_base + buf * (uint32_t) TC_ACC_COLS + (uint32_t) ((i - fh + 1 + j_lo) * NB);
                        const uint32_t a_addr = a_base + s * (uint32_t) g.a_stage_bytes;
                        const uint32_t b_addr = b_base + (uint32_t) (kd * g.ksteps) * b_kstep_bytes
                                                + (uint32_t) (j_lo * (NB / 8)) * 128u;
                        for (int ks = 0; ks < g.ksteps; ++ks)
                        {
                            const uint64_t ad = make_desc(a_addr + ks * 4096u, 512u, 2048u, 1u);
                            const uint64_t bd = make_desc(b_addr + ks * b_kstep_bytes, b_lbo, 128u, 0u);
                            mma_tf32(d_addr, ad, bd, idesc, 1u);
                        }
                        mma_commit(&empty_bar[s]);
                    }
                if (ok)
                    mma_commit(&acc_full[buf]);
            }
        }
    }
    else if (warp > TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // epilogue: TMEM -> registers -> global, then re-zero the buffer
        // ------------------------------------------------------------------
        const int quad = warp & 3; // TMEM lanes this warp may touch
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        for (int col = 0; col < (int) TC_TMEM_COLS; col += 16)
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
        for (long long tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x, ++tcount)
        {
            const TileRows t = tile_rows(g, tile);
            const int ow = t.ow0 + quad * 32 + lane;
            const uint32_t buf = tcount & 1;
            ok = mbar_wait(&acc_full[buf], (tcount >> 1) & 1, abort_flag);
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t acc_addr = lane_addr + buf * (uint32_t) TC_ACC_COLS;
            for (int r = 0; r < g.th; ++r)
            {
                const int oh = t.oh0 + r;
                if (oh >= g.out[1])
                    break; // uniform
                uint32_t v[NB];
#pragma unroll
                for (int q = 0; q < NB / 16; ++q)
                    tmem_ld16(acc_addr + (uint32_t) (r * NB + q * 16),
                              *reinterpret_cast<uint32_t(*)[16]>(&v[q * 16]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (ow < g.out[2])
                {
                    float* yp = y + (size_t) t.n * g.ys_n + (size_t) t.od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
                    const int kp = g.split ? NB / 2 : NB;
#pragma unroll
                    for (int k = 0; k < NB; ++k)
                    {
                        if (k < kp && k < g.k)
                        {
                            float acc = __uint_as_float(v[k]);
                            if (g.split)
                                acc += __uint_as_float(v[(k + NB / 2) % NB]);
                            float* p = yp + (size_t) k * g.ys_c;
                            const float prev = beta != 0.f ? *p : 0.f;
                            *p = alpha * acc + beta * prev;
                        }
                    }
                }
            }
            for (int col = 0; col < g.th * NB; col += 16)
                tmem_st16_zero(acc_addr + col);
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

size_t tc_smem_need(const TcGeom& g)
{
    return (size_t) g.stages * g.a_stage_bytes + (size_t) (g.b_bytes + 127) / 128 * 128
           + (size_t) g.raw_slots * g.raw_slot_bytes + (size_t) (2 * g.stages + 4 + 2 * g.raw_slots) * 8 + 64 + 1024;
}

bool tc_geom(const ConvGeom& cg, int math_mode, TcGeom* out)
{
    TcGeom g;
    std::memset(&g, 0, sizeof(g));
    for (int i = 0; i < 3; ++i)
    {
        if (cg.stride[i] != 1 || cg.dil[i] != 1)
            return false;
        g.in[i] = cg.in[i];
        g.out[i] = cg.out[i];
        g.f[i] = cg.f[i];
        g.pad[i] = cg.pad[i];
        g.xs[i] = cg.xs[i];
        g.ys[i] = cg.ys[i];
    }
    g.n = cg.n;
    g.c = cg.c;
    g.k = cg.k;
    g.xs_n = cg.xs_n;
    g.xs_c = cg.xs_c;
    g.ys_n = cg.ys_n;
    g.ys_c = cg.ys_c;
    if ((long long) cg.n * cg.out[0] * cg.out[1] * cg.out[2] == 0)
        return false;
    g.split = math_mode == DCB_MATH_TF32 ? 0 : 1;
    g.kpad = cg.k <= 8 ? 8 : (cg.k <= 16 ? 16 : 32);
    if (cg.k > 32)
        return false;
    g.nb = g.kpad * (g.split ? 2 : 1);
    if (g.nb < 16)
        g.nb = 16;
    g.ntot = g.f[1] * g.nb;
    if (g.ntot > 256 || g.ntot % 16)
        return false;
    g.th = TC_ACC_COLS / g.nb;
    if (g.th > 16)
        g.th = 16;
    if (g.c > 16)
        return false;
    for (int i = 0; i < 3; ++i)
        if (g.pad[i] > g.f[i] - 1)
            return false; // a window entirely inside the padding
    // taps are taken from the two cells either side of a lane's chunk
    if (g.pad[2] > 2 || g.f[2] - 1 - g.pad[2] > 2)
        return false;
    g.crows = g.c * g.f[2];
    g.kr = ((g.crows * (g.split ? 2 : 1)) + 7) / 8 * 8;
    g.ksteps = g.kr / 8;
    g.a_stage_bytes = g.kr * 512;
    g.b_bytes = g.f[0] * g.kr * g.ntot * 4;
    g.stages = (144 * 1024) / g.a_stage_bytes;
    g.stages = g.stages > TC_PRODUCERS ? TC_PRODUCERS : g.stages;
    if (g.stages < 2)
        return false;
    g.nprod = g.stages;
    // Bulk tensor copies need 16-byte aligned strides (the base address is
    // checked per call).
    g.use_tma = (cg.xs[1] % 4 == 0 && cg.xs[0] % 4 == 0 && cg.xs_c % 4 == 0 && cg.xs_n % 4 == 0) ? 1 : 0;
    g.raw_slot_bytes = (g.c * TC_RAW_W * 4 + 127) / 128 * 128;
    // a multiple of nprod (see the kernel), about 36 KiB at most
    g.raw_slots = g.use_tma ? ((36 * 1024) / g.raw_slot_bytes) / g.nprod * g.nprod : 0;
    if (g.raw_slots > 2 * g.nprod)
        g.raw_slots = 2 * g.nprod;
    if (g.use_tma && g.raw_slots < g.nprod)
        g.use_tma = 0, g.raw_slots = 0;
    const size_t need = tc_smem_need(g);
    if (need > 220 * 1024)
        return false;
    g.tiles_w = (g.out[2] + TC_M - 1) / TC_M;
    g.tiles_h = (g.out[1] + g.th - 1) / g.th;
    g.tiles = (long long) g.n * g.out[0] * g.tiles_h * g.tiles_w;
    *out = g;
    return true;
}

size_t tc_smem_bytes(const TcGeom& g)
{
    // At least 120 KiB so that a second CTA can never share the SM: the
    // kernel owns all 512 TMEM columns.
    const size_t need = tc_smem_need(g);
    return need < 120 * 1024 ? 120 * 1024 : need;
}

} // namespace

struct TcPlan
{
    bool has[2] = {false, false};
    TcGeom g[2];
    float* bimg[2] = {nullptr, nullptr};
    int* status = nullptr;
};

int32_t tc_plan_create(const ConvGeom& fwd, const ConvGeom& bwd, bool bwd_is_fwd, int math_mode, TcPlan** out)
{
    *out = nullptr;
    auto* p = new TcPlan();
    p->has[0] = tc_geom(fwd, math_mode, &p->g[0]);
    p->has[1] = bwd_is_fwd && tc_geom(bwd, math_mode, &p->g[1]);
    if (!p->has[0] && !p->has[1])
    {
        delete p;
        return DCB_OK;
    }
    bool ok = cudaMalloc(&p->status, sizeof(int)) == cudaSuccess
              && cudaMemset(p->status, 0, sizeof(int)) == cudaSuccess;
    for (int s = 0; s < 2 && ok; ++s)
        if (p->has[s])
            ok = cudaMalloc(&p->bimg[s], p->g[s].b_bytes) == cudaSuccess;
    if (!ok)
    {
        (void) cudaGetLastError();
        set_last_error("cudaMalloc of tensor-core filter image failed");
        tc_plan_destroy(p);
        return DCB_CUDA_ERROR;
    }
    *out = p;
    return DCB_OK;
}

void tc_plan_destroy(TcPlan* p)
{
    if (!p)
        return;
    cudaFree(p->bimg[0]);
    cudaFree(p->bimg[1]);
    cudaFree(p->status);
    delete p;
}

int* tc_status_word(TcPlan* p)
{
    return p ? p->status : nullptr;
}

bool tc_supports(const TcPlan* p, int which)
{
    if (!p)
        return false;
    if (which == 0)
        return p->has[0];
    if (which == 1)
        return p->has[1];
    return false;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried)
    {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void) cudaGetLastError();
    }
    return fn;
}

// Descriptor of the input window as a 5-D tensor (W, H, D, C, N) whose box is
// one raw row of every channel.  Returns false when the window cannot be
// described (alignment), in which case the register-fed producers run.
static bool make_x_map(const TcGeom& g, const float* x, CUtensorMap* map)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return false;
    const cuuint64_t dims[5] = {(cuuint64_t) g.in[2], (cuuint64_t) g.in[1], (cuuint64_t) g.in[0], (cuuint64_t) g.c,
                                (cuuint64_t) g.n};
    // a dimension of extent 1 may carry any stride; give it a valid one
    const long long s1 = g.xs[1], s0 = g.in[0] > 1 ? g.xs[0] : g.xs[1] * g.in[1];
    const cuuint64_t strides[4] = {(cuuint64_t) s1 * 4, (cuuint64_t) s0 * 4, (cuuint64_t) g.xs_c * 4,
                                   (cuuint64_t) (g.n > 1 ? g.xs_n : g.xs_c * g.c) * 4};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] == 0)
            return false;
    const cuuint32_t box[5] = {(cuuint32_t) TC_RAW_W, 1, 1, (cuuint32_t) g.c, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(x), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

template <int NB, int FW, int PW>
static int32_t tc_launch2(const TcGeom& g, float alpha, const float* x, const float* bimg, float beta, float* y,
                          int* status, const CUtensorMap& map, cudaStream_t stream)
{
    const size_t smem = tc_smem_bytes(g);
    DCB_CUDA_TRY(cudaFuncSetAttribute(tc_conv_kernel<NB, FW, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int) (224 * 1024)));
    long long grid = (long long) num_sms();
    if (grid > g.tiles)
        grid = g.tiles;
    tc_conv_kernel<NB, FW, PW><<<(unsigned) grid, TC_THREADS, smem, stream>>>(g, alpha, beta, x, bimg, y, status,
                                                                             map);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

template <int NB>
static int32_t tc_launch(const TcGeom& g_in, float alpha, const float* x, const float* bimg, float beta, float* y,
                         int* status, cudaStream_t stream)
{
    TcGeom g = g_in;
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    if (g.use_tma && !make_x_map(g, x, &map))
        g.use_tma = 0; // the raw ring stays allocated but unused
    if (g.f[2] == 3 && g.pad[2] == 1)
        return tc_launch2<NB, 3, 1>(g, alpha, x, bimg, beta, y, status, map, stream);
    if (g.f[2] == 5 && g.pad[2] == 2)
        return tc_launch2<NB, 5, 2>(g, alpha, x, bimg, beta, y, status, map, stream);
    if (g.f[2] == 1 && g.pad[2] == 0)
        return tc_launch2<NB, 1, 0>(g, alpha, x, bimg, beta, y, status, map, stream);
    return tc_launch2<NB, 0, 0>(g, alpha, x, bimg, beta, y, status, map, stream);
}

int32_t tc_conv_fwd(TcPlan* p, int slot, float alpha, const float* x, const float* w, float beta, float* y,
                    cudaStream_t stream)
{
    if (!p || slot < 0 || slot > 1 || !p->has[slot])
        return DCB_UNSUPPORTED;
    const TcGeom& g = p->g[slot];
    const long long total = (long long) g.b_bytes / 4;
    tc_pack_filter_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, stream>>>(w, p->bimg[slot], g);
    DCB_LAUNCH_CHECK();
    switch (g.nb)
    {
    case 16: return tc_launch<16>(g, alpha, x, p->bimg[slot], beta, y, p->status, stream);
    case 32: return tc_launch<32>(g, alpha, x, p->bimg[slot], beta, y, p->status, stream);
    case 64: return tc_launch<64>(g, alpha, x, p->bimg[slot], beta, y, p->status, stream);
    default: return DCB_UNSUPPORTED;
    }
}

int32_t tc_conv_bwd_filter(TcPlan*, float, const float*, const float*, float, float*, cudaStream_t)
{
    return DCB_UNSUPPORTED;
}

} // namespace dcb
