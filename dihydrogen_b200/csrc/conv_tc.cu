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

namespace dcb
{

namespace
{

constexpr int TC_THREADS = 128;
constexpr int TC_M = 128;
constexpr uint32_t TC_TMEM_COLS = 256;

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

// Bounded parity wait.  Returns false when the budget ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    const uint32_t addr = smem_u32(bar);
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
        if (*abort_flag)
            return false;
        if (it > 1024)
            __nanosleep(128);
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

template <int NB>
__global__ void __launch_bounds__(TC_THREADS)
    tc_conv_kernel(TcGeom g, float alpha, float beta, const float* __restrict__ x, const float* __restrict__ bimg,
                   float* y, int* status)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment keeps the hardware swizzle phase equal to the one
    // used when writing the tiles.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_ring = smem;
    float* b_smem = reinterpret_cast<float*>(smem + (size_t) g.stages * g.a_stage_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(b_smem) + g.b_bytes);
    uint64_t* empty_bar = bars;              // [stages]
    uint64_t* acc_bar = bars + g.stages;     // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + g.stages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int fd = g.f[0], fh = g.f[1], fw = g.f[2];

    if (tid == 0)
    {
        for (int s = 0; s < g.stages; ++s)
            mbar_init(&empty_bar[s], 1);
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0)
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
    const uint32_t lane_addr = tmem_base + ((uint32_t) (warp * 32) << 16);

    // instruction descriptor without N: fp32 accumulate, tf32 x tf32,
    // A MN-major, B K-major, M = 128
    const uint32_t idesc_base = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (0u << 16) | ((TC_M >> 4) << 24);
    const uint32_t a_base = smem_u32(a_ring);
    const uint32_t b_base = smem_u32(b_smem);
    const uint32_t b_lbo = (uint32_t) (g.ntot / 8) * 128u;
    const uint32_t b_kstep_bytes = (uint32_t) g.ntot * 32u;

    uint32_t it = 0;        // staged rows so far (ring position and parity)
    uint32_t acc_phase = 0; // completed tiles
    bool ok = true;

    for (long long tile = blockIdx.x; tile < g.tiles && ok; tile += gridDim.x)
    {
        const int tw = (int) (tile % g.tiles_w);
        long long t2 = tile / g.tiles_w;
        const int thi = (int) (t2 % g.tiles_h);
        t2 /= g.tiles_h;
        const int od = (int) (t2 % g.out[0]);
        const int n = (int) (t2 / g.out[0]);
        const int ow0 = tw * TC_M, oh0 = thi * g.th;

        // ---- zero the accumulators ----
        for (int col = 0; col < g.th * NB; col += 16)
            tmem_st16_zero(lane_addr + col);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();

        // ---- main loop over staged input rows ----
        for (int kd = 0; kd < fd && ok; ++kd)
        {
            const int id = od - g.pad[0] + kd;
            if (id < 0 || id >= g.in[0])
                continue;
            for (int i = 0; i < g.th + fh - 1 && ok; ++i)
            {
                const int ih = oh0 - g.pad[1] + i;
                if (ih < 0 || ih >= g.in[1])
                    continue;
                int j_lo = fh - 1 - i;
                j_lo = j_lo < 0 ? 0 : j_lo;
                int j_hi = g.th + fh - 1 - i;
                j_hi = j_hi > fh ? fh : j_hi;
                if (j_hi <= j_lo)
                    continue;
                const uint32_t s = it % g.stages;
                if (it >= (uint32_t) g.stages)
                    ok = mbar_wait(&empty_bar[s], ((it / g.stages) - 1) & 1, abort_flag);
                if (!ok)
                    break;
                // ---- stage: hi / lo split and the fw shifted copies ----
                uint8_t* a_stage = a_ring + (size_t) s * g.a_stage_bytes;
                const float* xrow_base = x + (size_t) n * g.xs_n + (size_t) id * g.xs[0] + (size_t) ih * g.xs[1];
                const int ntask = g.crows * 32;
                for (int task = tid; task < ntask; task += TC_THREADS)
                {
                    const int q = task & 31;       // 16-byte chunk along M
                    const int cr = task >> 5;      // (c, kw)
                    const int c = cr / fw, kw = cr - c * fw;
                    const float* xr = xrow_base + (size_t) c * g.xs_c;
                    const int iw0 = ow0 + 4 * q - g.pad[2] + kw;
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                    {
                        const int iw = iw0 + e;
                        v[e] = (iw >= 0 && iw < g.in[2]) ? xr[iw] : 0.f;
                    }
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                    {
                        hi[e] = tf32_rna(v[e]);
                        lo[e] = tf32_rna(v[e] - __uint_as_float(hi[e]));
                    }
                    const int matom = q >> 3, qq = q & 7;
                    {
                        const int kr = cr;
                        const int r = kr & 3;
                        uint8_t* dst = a_stage + ((size_t) ((kr >> 2) * 4 + matom) << 9) + (r << 7)
                                       + (((qq >> 1) ^ r) << 5) + ((qq & 1) << 4);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    }
                    if (g.split)
                    {
                        const int kr = g.crows + cr;
                        const int r = kr & 3;
                        uint8_t* dst = a_stage + ((size_t) ((kr >> 2) * 4 + matom) << 9) + (r << 7)
                                       + (((qq >> 1) ^ r) << 5) + ((qq & 1) << 4);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncthreads();
                // ---- issue ----
                if (tid == 0)
                {
                    tc_fence_after();
                    const int nblocks = j_hi - j_lo;
                    const uint32_t idesc = idesc_base | ((uint32_t) ((nblocks * NB) >> 3) << 17);
                    const uint32_t d_addr = tmem_base + (uint32_t) ((i - fh + 1 + j_lo) * NB);
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
                ++it;
            }
        }
        if (!ok)
            break;
        if (tid == 0)
            mma_commit(acc_bar);
        ok = mbar_wait(acc_bar, acc_phase & 1, abort_flag);
        ++acc_phase;
        if (!ok)
            break;
        tc_fence_after();

        // ---- epilogue: TMEM -> registers -> global ----
        const int ow = ow0 + warp * 32 + lane;
        for (int r = 0; r < g.th; ++r)
        {
            const int oh = oh0 + r;
            if (oh >= g.out[1])
                break; // uniform
            uint32_t v[NB];
#pragma unroll
            for (int q = 0; q < NB / 16; ++q)
                tmem_ld16(lane_addr + (uint32_t) (r * NB + q * 16), *reinterpret_cast<uint32_t(*)[16]>(&v[q * 16]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (ow < g.out[2])
            {
                float* yp = y + (size_t) n * g.ys_n + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
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
        tc_fence_before();
        __syncthreads();
    }

    if (!ok && tid == 0)
        atomicExch(status, 1);
    // Teardown.  On the error path threads may leave at different points, so
    // no block-wide barrier is used there: the allocating warp waits for its
    // own lanes and frees the columns.
    if (ok)
    {
        tc_fence_before();
        __syncthreads();
    }
    if (warp == 0)
    {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS)
                     : "memory");
    }
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
    g.th = (int) TC_TMEM_COLS / g.nb;
    if (g.th > 16)
        g.th = 16;
    g.crows = g.c * g.f[2];
    g.kr = ((g.crows * (g.split ? 2 : 1)) + 7) / 8 * 8;
    g.ksteps = g.kr / 8;
    g.a_stage_bytes = g.kr * 512;
    g.b_bytes = g.f[0] * g.kr * g.ntot * 4;
    g.stages = g.a_stage_bytes <= 16 * 1024 ? 4 : (g.a_stage_bytes <= 32 * 1024 ? 3 : 2);
    const size_t need = (size_t) g.stages * g.a_stage_bytes + g.b_bytes + 256 + 1024;
    if (need > 200 * 1024)
        return false;
    g.tiles_w = (g.out[2] + TC_M - 1) / TC_M;
    g.tiles_h = (g.out[1] + g.th - 1) / g.th;
    g.tiles = (long long) g.n * g.out[0] * g.tiles_h * g.tiles_w;
    *out = g;
    return true;
}

size_t tc_smem_bytes(const TcGeom& g)
{
    return (size_t) g.stages * g.a_stage_bytes + g.b_bytes + 256 + 1024;
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

template <int NB>
static int32_t tc_launch(const TcGeom& g, float alpha, const float* x, const float* bimg, float beta, float* y,
                         int* status, cudaStream_t stream)
{
    const size_t smem = tc_smem_bytes(g);
    DCB_CUDA_TRY(cudaFuncSetAttribute(tc_conv_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int) (200 * 1024)));
    // Two CTAs per SM when shared memory allows: one stages and issues while
    // the other drains its accumulators.
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    long long grid = (long long) num_sms() * per_sm;
    if (grid > g.tiles)
        grid = g.tiles;
    tc_conv_kernel<NB><<<(unsigned) grid, TC_THREADS, smem, stream>>>(g, alpha, beta, x, bimg, y, status);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
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
