// Sweep convolution for many input channels and at most four filters (the
// backward-data shape of a layer with few input channels): conv_tc_sweep.cuh's
// scheme, with the input channels walked in groups INSIDE one launch.
//
// Differences from the sweep kernel:
//   * An accumulator block is 4 columns (filters), and a row has four plane
//     slots (od & 3; with fd = 3 one of them idles each step), so a row's
//     blocks are 16 columns and one instruction covers N = fh * 16.
//   * A staged input row is converted once per channel group ("sub-row" (i, g)):
//     the group's c * fw taps, [hi ; lo], go into an A slot and are
//     multiplied with that group's filter image.  All groups of a row add into
//     the same accumulators, so nothing is blended in memory and the output is
//     written once.  Sub-rows are dealt to the converter groups / issuers in
//     sequence; row_done[i] completes when all of row i's sub-rows have.
//   * The filter image holds [channel group][rotation d & 3][k-step]...; bulk
//     copies bring all channels of a chunk of rows.
//   * The tensor pipe adds into its fp32 accumulators by truncation, and every
//     channel group adds 45 updates (27 taps x hi / lo parts in 5 k-steps x 9
//     row / plane taps) to an output's chain: with more than three groups on one
//     chain the result reaches the 1e-5 bound.  So the groups are spread over
//     `nsets` accumulator sets of th rows each (set s at TMEM column
//     s * th * 16, at most three groups per set), and the epilogue adds the
//     sets in fp32 with rounding when it retires a row.
// Hand-offs and their safety argument are those of conv_tc_sweep.cuh (an issuer
// waits only for output rows its own row adds into).
#pragma once

#include "conv_tc_sweep.cuh"

namespace dcb
{
namespace
{

constexpr int MG_NBK = 4;   // filters per accumulator block
constexpr int MG_SLOTS = 4; // plane slots per output row
constexpr int MG_BLK = MG_NBK * MG_SLOTS;
constexpr int MG_ISSUER2_WARP = TC_TMA_WARP + 1 + TC_EPI_WARPS; // second issuers: warps 24..26
constexpr int MG_IPG_MAX = 2; // issuers (= A slots) per converter group at most
constexpr int MG_THREADS = (MG_ISSUER2_WARP + (MG_IPG_MAX - 1) * TC_GROUPS_MAX) * 32;

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&v)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr));
}

__device__ __forceinline__ void tmem_st4_zero(uint32_t taddr)
{
    const uint32_t z = 0;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %1, %1, %1};" ::"r"(taddr), "r"(z) : "memory");
}

// Filter image: [group][rotation][k-step][2 k-chunks][ntot/8][8 n][4 k] floats,
// ntot = fh * 16.  Column (j, s, ko): output row offset j (kh = fh-1-j), plane
// slot s, filter ko.  In rotation r (= d & 3) slot s belongs to the output plane
// d + pad - kd with kd = (r + pad - s) & 3; kd >= fd: the slot idles, zeros.
__global__ void mg_pack_filter_kernel(const float* __restrict__ w, float* __restrict__ b, SwGeom g)
{
    const int fd = g.f[0], fh = g.f[1], fw = g.f[2];
    const int per_rot = g.kb * g.ntot;
    const long long total = (long long) g.cgroups * MG_SLOTS * per_rot;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long) gridDim.x * blockDim.x)
    {
        const int grp = (int) (i / ((long long) MG_SLOTS * per_rot));
        const int rot = (int) ((i / per_rot) % MG_SLOTS);
        const int e = (int) (i % per_rot);
        const int ki = e % 4;
        const int ni = (e / 4) % 8;
        const int ngroup = (e / 32) % (g.ntot / 8);
        const int kchunk = (e / (32 * (g.ntot / 8))) % 2;
        const int kstep = e / (64 * (g.ntot / 8));
        const int krow = kstep * 8 + kchunk * 4 + ki;
        const int ncol = ngroup * 8 + ni;
        const int j = ncol / MG_BLK;
        const int s = (ncol / MG_NBK) % MG_SLOTS;
        const int ko = ncol % MG_NBK;
        const int kh = fh - 1 - j;
        const int kd = (rot + g.pad[0] - s) & (MG_SLOTS - 1);
        // as in sw_pack_filter_kernel: [hi | lo] against w_hi, then the hi columns again against w_lo
        int part, rem;
        if (krow < g.kr)
        {
            part = krow / g.crows;
            rem = krow % g.crows;
            if (part >= (g.split ? 2 : 1))
                part = 3;
        }
        else
        {
            rem = krow - g.kr;
            part = (g.split && rem < g.crows) ? 2 : 3;
            rem = rem < g.crows ? rem : 0;
        }
        const int c = grp * g.c + rem / fw, kw = rem % fw;
        float val = 0.f;
        if (ko < g.k && kd < fd && part < 3)
        {
            const float wv = w[((((size_t) ko * g.w_c_total + c) * fd + kd) * fh + kh) * fw + kw];
            const float hi = __uint_as_float((__float_as_uint(wv) + g.rnd_add) & g.rnd_mask);
            val = part < 2 ? hi : __uint_as_float(tf32_rna(wv - hi));
        }
        b[i] = val;
    }
}

// Warps as in the sweep kernel: 0..11 converters, 12..14 issuers, 15 copies,
// 16..23 epilogue.  TMEM columns: [nsets x accumulators th * 16][A ring].
template <bool C4F3>
__global__ void __launch_bounds__(MG_THREADS, 1)
    mg_conv_kernel(SwGeom g, float alpha, const float* __restrict__ bimg, float* y, int* status,
                   const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap ymap, int use_ymap,
                   long long* prof)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* b_smem = reinterpret_cast<float*>(smem);
    const int b_region = (g.b_bytes + 127) / 128 * 128;
    uint8_t* raw_ring = smem + b_region;
    uint32_t* ktab = reinterpret_cast<uint32_t*>(raw_ring + (size_t) g.raw_slots * g.raw_slot_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ktab + ((g.kr + 1) & ~1));
    uint64_t* a_full = bars;                      // [a_slots]
    uint64_t* a_empty = a_full + g.a_slots;       // [a_slots]
    uint64_t* row_done = a_empty + g.a_slots;     // [32]
    uint64_t* row_free = row_done + 32;           // [32]
    uint64_t* raw_full = row_free + 32;           // [raw_slots]
    uint64_t* raw_empty = raw_full + g.raw_slots; // [raw_slots]
    uint64_t* iss_sync = raw_empty + g.raw_slots; // [TC_GROUPS_MAX] the issuers of a group, once per step
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(iss_sync + TC_GROUPS_MAX);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // output staging for bulk stores: two 512-byte buffers per epilogue warp
    float* stage_base = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int fd = g.f[0], fh = g.f[1], R = g.rows, G = g.groups, CG = g.cgroups;
    const int subrows = R * CG; // sub-rows per step

    if (tid == 0)
    {
        for (int s = 0; s < g.a_slots; ++s)
        {
            mbar_init(&a_full[s], 4);
            mbar_init(&a_empty[s], 1);
        }
        for (int r = 0; r < 32; ++r)
        {
            mbar_init(&row_done[r], CG);
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
    // k-row table for one channel group (the group's first channel is added per sub-row)
    for (int r = tid; r < g.kr; r += MG_THREADS)
    {
        const int part = r / g.crows, rem = r % g.crows;
        const int c = rem / g.f[2], kw = rem % g.f[2];
        const uint32_t off = (uint32_t) (c * g.chunk_rows * TC_RAW_W + g.rx + kw);
        const uint32_t sel = part < (g.split ? 2 : 1) ? (uint32_t) part : 2u;
        ktab[r] = sel == 2u ? ((2u << 16) | 4u) : (off | (sel << 16));
    }
    for (int i = tid; i < g.b_bytes / 16; i += MG_THREADS)
        reinterpret_cast<float4*>(b_smem)[i] = reinterpret_cast<const float4*>(bimg)[i];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t set_cols = (uint32_t) (g.th * MG_BLK);     // columns of one accumulator set
    const uint32_t a_col0 = (uint32_t) g.nsets * set_cols;    // first column of the A ring
    const int grp_per_set = (CG + g.nsets - 1) / g.nsets;
    const uint32_t nunits = (uint32_t) g.units;
    bool ok = true;

    if (warp < 4 * G)
    {
        // ------------------------------------------------------------------
        // converters: sub-row q = i * CG + grp of a step
        // ------------------------------------------------------------------
        const int gq = warp >> 2, quad = warp & 3;
        const int mcol = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        const int laps_a = g.a_slots / G;
        const uint32_t ktab_s = smem_u32(ktab);
        const int Rc = g.chunk_rows;
        const uint32_t pitch = (uint32_t) (g.chunk_rows * TC_RAW_W); // channel pitch inside a chunk
        int lap_a = 0;
        uint32_t cslot = 0, cphase = 0, a_phase = 1, base = 0;
        bool a_first = true;
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
                    const int lo = ch * Rc, hi = min(R, (ch + 1) * Rc);
                    const int q_lo = lo * CG, q_hi = hi * CG;
                    int q = q_lo + (gq + G - (int) ((base + (uint32_t) q_lo) % (uint32_t) G)) % G;
                    // (row, channel group) of sub-row q, kept by counting: a division
                    // per sub-row showed in the converters' and issuers' loop time
                    int i = q / CG, grp = q - i * CG;
                    bool have = false;
                    for (; q < q_hi && ok; q += G, grp += G)
                    {
                        while (grp >= CG)
                        {
                            grp -= CG;
                            ++i;
                        }
                        const int a_slot = gq + G * lap_a;
                        SW_PROF_MARK(4)
                        if (!have)
                            ok = mbar_wait(&raw_full[cslot], cphase, abort_flag);
                        have = true;
                        SW_PROF_MARK(0)
                        if (!ok)
                            break;
                        const float* raw = reinterpret_cast<const float*>(raw_ring + (size_t) cslot * g.raw_slot_bytes)
                                           + (size_t) grp * g.c * pitch + (i - lo) * TC_RAW_W;
                        const uint32_t a_addr = lane_addr + a_col0 + (uint32_t) (a_slot * g.kr);
                        const uint32_t raw_s = smem_u32(raw) + 4u * (uint32_t) mcol;
                        if (C4F3)
                        {
                            uint32_t v[3][8];
                            // the converter is written for taps that start 3 cells into the staged row
                            sw_convert_c4f3<true>(raw_s + 4u * (uint32_t) (g.rx - 3), pitch, v);
                            SW_PROF_MARK(1)
                            if (!a_first)
                                ok = mbar_wait(&a_empty[a_slot], a_phase, abort_flag);
                            SW_PROF_MARK(2)
                            if (!ok)
                                break;
                            tc_fence_after();
#pragma unroll
                            for (int ck = 0; ck < 3; ++ck)
                                tmem_st8(a_addr + (uint32_t) (ck * 8), v[ck]);
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
                    // every converter warp releases every chunk
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&raw_empty[cslot]);
                    if (++cslot == (uint32_t) g.raw_slots)
                    {
                        cslot = 0;
                        cphase ^= 1;
                    }
                }
                base = (base + (uint32_t) subrows) % (uint32_t) G;
            }
        }
        SW_PROF_MARK(4)
        SW_PROF_FLUSH(prof)
    }
    else if (warp == TC_TMA_WARP)
    {
        // ------------------------------------------------------------------
        // bulk tensor copies: chunk_rows raw rows of ALL channels per copy
        // ------------------------------------------------------------------
        const uint32_t bytes = (uint32_t) (g.w_c_total * g.chunk_rows) * TC_RAW_W * 4u;
        uint32_t slot = 0, empty_phase = 1;
        bool first_lap = true;
        for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
        {
            const SwUnit t = sw_unit(g, u);
            for (int d = t.d_first; d < t.d_stop && ok; ++d)
            {
                if (!sw_real(g, t, d))
                    continue;
                for (int ch = 0; ch < g.chunks_pp; ++ch)
                {
                    if (!first_lap)
                        ok = mbar_wait(&raw_empty[slot], empty_phase, abort_flag);
                    if (!ok)
                        break;
                    if (lane == 0)
                    {
                        mbar_expect_tx(&raw_full[slot], bytes);
                        tma_load_5d(raw_ring + (size_t) slot * g.raw_slot_bytes, &xmap, t.ow0 + g.lx,
                                    t.oh0 - g.pad[1] + ch * g.chunk_rows, d, 0, t.n, &raw_full[slot]);
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
    else if ((warp >= TC_MMA_WARP && warp < TC_MMA_WARP + TC_GROUPS_MAX) || warp >= MG_ISSUER2_WARP)
    {
        // ------------------------------------------------------------------
        // MMA issue: issuer (mq, mh) takes the sub-rows converter group mq wrote
        // into its A slot mq + G * mh (a kernel whose staged row is four sub-rows
        // of five instructions and two commits each is bound by what one thread
        // can issue).  Lane i issues the sub-rows of staged row i.
        // ------------------------------------------------------------------
        const int mq = warp < MG_ISSUER2_WARP ? warp - TC_MMA_WARP : (warp - MG_ISSUER2_WARP) % TC_GROUPS_MAX;
        const int mh = warp < MG_ISSUER2_WARP ? 0 : 1 + (warp - MG_ISSUER2_WARP) / TC_GROUPS_MAX;
        if (mq < G && mh < g.a_slots / G)
        {
            const int my_i = lane;
            const int j_lo = max(0, fh - 1 - my_i);
            const int j_hi = min(fh, g.th + fh - 1 - my_i);
            const uint32_t my_idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((TC_M >> 4) << 24)
                                      | ((uint32_t) ((max(1, j_hi - j_lo) * MG_BLK) >> 3) << 17);
            const uint32_t my_d = tmem_base + (uint32_t) ((my_i - fh + 1 + j_lo) * MG_BLK);
            const uint32_t b_lbo = (uint32_t) (g.ntot / 8) * 128u;
            const uint32_t b_kstep_units = ((uint32_t) g.ntot * 32u) >> 4;
            const uint64_t my_b_desc =
                make_desc(smem_u32(b_smem), b_lbo, 128u, 0u) + (uint64_t) ((uint32_t) (j_lo * MG_BLK));
            const uint32_t rot_units = (uint32_t) g.b_rot_bytes >> 4;
            const uint32_t a_ring = tmem_base + a_col0;
            const int ksteps = g.ksteps;
            const int laps_a = g.a_slots / G;
            int lap_a = 0;
            uint32_t full_phase = 0, step = 0, base = 0;
            SW_PROF_DECL
            for (uint32_t u = blockIdx.x; u < nunits && ok; u += gridDim.x)
            {
                const SwUnit t = sw_unit(g, u);
                for (int d = t.d_first; d < t.d_stop && ok; ++d, ++step)
                {
                    // The issuers of a group stay within one step of each other: the second
                    // one skips the rows it does not own without a wait (virtual steps
                    // entirely), and a parity wait cannot tell a barrier two completions
                    // away.  The first issuer waits for every row's hand-back in every step,
                    // so once both have finished a step the barriers this group looks at are
                    // at most one completion behind what either expects next.
                    SW_PROF_MARK(4)
                    if (laps_a > 1 && step != 0)
                        ok = mbar_wait_t<0>(&iss_sync[mq], (step - 1) & 1, abort_flag);
                    SW_PROF_MARK(3)
                    const bool real = sw_real(g, t, d);
                    const uint32_t par = step & 1;
                    const uint32_t rot = (uint32_t) (d & (MG_SLOTS - 1));
                    int q = real ? (mq + G - (int) (base % (uint32_t) G)) % G : mq;
                    int i = q / CG, grp = q - i * CG;
                    for (; q < subrows && ok; q += G, grp += G)
                    {
                        while (grp >= CG)
                        {
                            grp -= CG;
                            ++i;
                        }
                        // a real sub-row belongs to the issuer of the slot it was written to,
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
                        // only output rows this row adds into may be waited for
                        const int r_hi = min(i, g.th - 1), r_lo = max(0, i - fh + 1);
                        SW_PROF_MARK(4)
                        ok = mbar_wait_t<0>(&row_free[r_hi], par, abort_flag);
                        if (ok && r_hi - 1 >= r_lo)
                            ok = mbar_wait_t<0>(&row_free[r_hi - 1], par, abort_flag);
                        SW_PROF_MARK(0)
                        if (!ok)
                            break;
                        if (real)
                        {
                            const uint32_t slot = (uint32_t) (mq + G * lap_a);
                            ok = mbar_wait_t<0>(&a_full[slot], full_phase, abort_flag);
                            SW_PROF_MARK(1)
                            if (!ok)
                                break;
                            tc_fence_after();
                            if (lane == i)
                            {
                                const uint32_t a_base = a_ring + slot * (uint32_t) g.kr;
                                uint32_t a_addr = a_base;
                                uint64_t bd = my_b_desc
                                              + (uint64_t) (((uint32_t) grp * MG_SLOTS + rot) * rot_units);
                                // the group's accumulator set
                                const uint32_t d_addr = my_d + (uint32_t) (grp / grp_per_set) * set_cols;
                                for (int ks = 0; ks < ksteps; ++ks)
                                {
                                    mma_tf32_ts(d_addr, a_addr, bd, my_idesc);
                                    a_addr = ks + 1 == g.ks1 ? a_base : a_addr + 8;
                                    bd += b_kstep_units;
                                }
                                mma_commit(&a_empty[slot]);
                                mma_commit(&row_done[i]);
                                tc_fence_before();
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
                    if (real)
                        base = (base + (uint32_t) subrows) % (uint32_t) G;
                    if (laps_a > 1)
                    {
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&iss_sync[mq]);
                    }
                }
            }
            SW_PROF_MARK(4)
            SW_PROF_FLUSH(prof)
        }
    }
    else if (warp > TC_TMA_WARP && warp < MG_ISSUER2_WARP)
    {
        // ------------------------------------------------------------------
        // epilogue: after step d retire output plane d + pad - (fd-1)
        // ------------------------------------------------------------------
        const int quad = warp & 3;
        const int half = (warp - TC_TMA_WARP - 1) >> 2, nhalf = TC_EPI_WARPS / 4;
        const uint32_t lane_addr = tmem_base + ((uint32_t) (quad * 32) << 16);
        const int nk = g.k;
        const size_t ysc = (size_t) g.ys_c;
        const bool bulk = use_ymap != 0;
        float* stage = stage_base + (warp - TC_TMA_WARP - 1) * (2 * MG_NBK * 32);
        uint32_t nstored = 0;
        for (int j = half; j < g.th; j += nhalf)
            for (int s = 0; s < g.nsets; ++s)
                tmem_st16_zero(lane_addr + (uint32_t) s * set_cols + (uint32_t) (j * MG_BLK));
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
                const uint32_t slot_col = (uint32_t) ((od & (MG_SLOTS - 1)) * MG_NBK);
                for (int j = half; j < g.th && ok; j += nhalf)
                {
                    const int oh = t.oh0 + j;
                    const bool wr = store && oh < g.out[1];
                    SW_PROF_MARK(4)
                    for (int i = j; i < j + fh && ok; ++i)
                        ok = mbar_wait(&row_done[i], par, abort_flag);
                    SW_PROF_MARK(0)
                    if (!ok)
                        break;
                    tc_fence_after();
                    const uint32_t addr = lane_addr + (uint32_t) (j * MG_BLK) + slot_col;
                    uint32_t v[MG_NBK];
                    if (wr)
                    {
                        tmem_ld4(addr, v);
                        if (g.nsets > 1)
                        {
                            // the second set's partial sums, added with rounding
                            uint32_t v2[MG_NBK];
                            tmem_ld4(addr + set_cols, v2);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int k = 0; k < MG_NBK; ++k)
                                v[k] = __float_as_uint(__uint_as_float(v[k]) + __uint_as_float(v2[k]));
                        }
                        else
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    }
                    SW_PROF_MARK(1)
                    tmem_st4_zero(addr);
                    if (g.nsets > 1)
                        tmem_st4_zero(addr + set_cols);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&row_free[j]);
                    SW_PROF_MARK(2)
                    if (!wr)
                        continue;
                    if (bulk)
                    {
                        if (t.ow0 + quad * 32 >= g.out[2])
                            continue;
                        float* st = stage + (nstored & 1) * (MG_NBK * 32);
                        if (nstored >= 2)
                        {
                            if (lane == 0)
                                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                            __syncwarp();
                        }
                        const uint32_t st_s = smem_u32(st) + 4u * (uint32_t) lane;
#pragma unroll
                        for (int k = 0; k < MG_NBK; ++k)
                            asm volatile("st.shared.f32 [%0], %1;" ::"r"(st_s + 128u * k),
                                         "f"(alpha * __uint_as_float(v[k]))
                                         : "memory");
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
                        float* yrow =
                            y + (size_t) t.n * g.ys_n + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1] + ow;
#pragma unroll
                        for (int k = 0; k < MG_NBK; ++k)
                            if (k < nk)
                                yrow[(size_t) k * ysc] = alpha * __uint_as_float(v[k]);
                    }
                }
            }
        }
        if (bulk && lane == 0)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        SW_PROF_MARK(4)
        SW_PROF_FLUSH(prof)
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
