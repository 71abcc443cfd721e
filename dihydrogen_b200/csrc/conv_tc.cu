// tcgen05 / TMEM implicit-GEMM convolution (stride 1, dilation 1), NC[D]HW:
// host side (geometry, shared / tensor memory budgeting, tensor map, launch).
//
// GEMM view.  One MMA tile is 128 consecutive outputs of one output row
// (M = 128 along W).  For one staged input row (id, ih) the reduction index
// ("k-rows") runs over (c, kw): k-row (c, kw) is that input row shifted by
// kw - pad_w.  With the 3xTF32 split the k-rows are [A_hi ; A_lo] and the B
// operand for filter row kh is the 2-block [[w_hi | w_lo] ; [w_hi | 0]], so
// a_hi*w_hi + a_hi*w_lo + a_lo*w_hi lands in two column halves that the
// epilogue adds.
//
// A staged input row serves fh output rows (oh = ih + pad_h - kh).  Their B
// blocks are concatenated along N in descending kh, which makes the target
// accumulators of one MMA consecutive output rows: one instruction of
// N = fh * NB columns updates fh accumulator blocks at once.
//
// Operands:
//   A   tensor memory: lane = output column of the tile, 8 columns per k-step,
//       written by the converter warps (tcgen05.st) after the hi / lo split
//   B   shared memory [kd][k-step][2 k-chunks][N/8][8 n][4 k] floats, K-major,
//       no swizzle, built once per call from the fp32 filter
//   D   tensor memory, lane = output column, column = r * NB + n
//
// Every wait on an mbarrier is bounded; on expiry the kernel records an error,
// releases its tensor memory and returns.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "conv_tc.cuh"
#include "conv_tc_kernel.cuh"
#include "conv_tc_sweep.cuh"
#include "conv_tc_sweep_mg.cuh"
#include "conv_tc_wgrad.cuh"

namespace dcb
{

namespace
{

size_t tc_smem_need(const TcGeom& g)
{
    return (size_t) (g.b_bytes + 127) / 128 * 128 + (size_t) g.raw_slots * g.raw_slot_bytes
           + (size_t) ((g.kr + 1) & ~1) * 4 + (size_t) (2 * g.a_slots + 4 + 2 * g.raw_slots) * 8 + 64 + 1024;
}

// Raw-row ring.  When bulk copies feed it, one copy brings chunk_rows rows of
// every channel (about 17 KiB) and the ring holds up to four such chunks; else
// it is one private window set per converter group.
void tc_size_raw_ring(TcGeom& g)
{
    if (g.use_tma)
    {
        const int rows = g.th + g.f[1] - 1, row_bytes = g.c * TC_RAW_W * 4;
        int rc = (17 * 1024 + 512) / row_bytes;
        rc = rc < 1 ? 1 : (rc > rows ? rows : rc);
        g.chunk_rows = rc;
        g.chunks_pp = (rows + rc - 1) / rc;
        g.raw_slot_bytes = (rc * row_bytes + 127) / 128 * 128;
        int slots = (72 * 1024) / g.raw_slot_bytes;
        slots = slots > 4 ? 4 : slots;
        if (slots >= 2)
        {
            g.raw_slots = slots;
            return;
        }
        g.use_tma = 0;
    }
    g.chunk_rows = 0;
    g.chunks_pp = 1;
    g.raw_slot_bytes = (4 * g.c * TC_RAW_PRIV * 4 + 127) / 128 * 128;
    g.raw_slots = g.groups;
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
    g.xs_n = cg.xs_n;
    g.xs_c = cg.xs_c;
    g.ys_n = cg.ys_n;
    g.ys_c = cg.ys_c;
    if ((long long) cg.n * cg.out[0] * cg.out[1] * cg.out[2] == 0 || cg.c == 0 || cg.k == 0)
        return false;
    g.split = (math_mode == DCB_MATH_TF32 || math_mode == DCB_MATH_BF16) ? 0 : 1;
    g.rnd_add = math_mode == DCB_MATH_BF16 ? 0x8000u : 0x1000u;
    g.rnd_mask = math_mode == DCB_MATH_BF16 ? 0xffff0000u : 0xffffe000u;
    const int mult = g.split ? 2 : 1;
    // Filters per launch: the fh accumulator blocks of an input row are one
    // instruction's N (<= 256 columns).
    g.k_total = cg.k;
    g.kpad = cg.k <= 8 ? 8 : (cg.k <= 16 ? 16 : 32);
    while (g.kpad > 8 && g.f[1] * g.kpad * mult > 256)
        g.kpad /= 2;
    g.k = cg.k < g.kpad ? cg.k : g.kpad;
    g.kgroups = (cg.k + g.kpad - 1) / g.kpad;
    g.nb = g.kpad * mult;
    if (g.nb < 16)
        g.nb = 16;
    g.ntot = g.f[1] * g.nb;
    if (g.ntot > 256 || g.ntot % 16)
        return false;
    // Channels per launch: a staged row is c * fw taps (hi and lo) of k-rows in
    // tensor memory; at most 96 keeps two converter groups busy.
    g.c_total = cg.c;
    g.c = 0;
    for (int d = cg.c; d >= 1; --d)
        if (cg.c % d == 0 && (d * g.f[2] * mult + 7) / 8 * 8 <= 96)
        {
            g.c = d;
            break;
        }
    if (g.c == 0)
        return false;
    g.cgroups = cg.c / g.c;
    if (g.cgroups * g.kgroups > 64)
        return false;
    for (int i = 0; i < 3; ++i)
        if (g.pad[i] > g.f[i] - 1)
            return false; // a window entirely inside the padding
    // taps come from the 4 cells of margin either side of the tile
    if (g.pad[2] > 4 || g.f[2] - 1 - g.pad[2] > 4)
        return false;
    g.crows = g.c * g.f[2];
    g.kr = ((g.crows * (g.split ? 2 : 1)) + 7) / 8 * 8;
    g.ksteps = g.kr / 8;
    g.b_bytes = g.f[0] * g.kr * g.ntot * 4;
    // TMEM: two accumulator buffers of th * nb columns and the A ring of
    // a_slots * kr columns share the 512 columns.  Three converter groups
    // when the ring can hold a slot for each; rows per tile as large as the
    // rest allows.
    g.groups = 3 * g.kr <= 192 ? 3 : (2 * g.kr <= 192 ? 2 : 1);
    if (g.kr > 192)
        return false;
    // One slot per group unless the rows are narrow: a deeper ring costs
    // accumulator rows and was measured to gain nothing.
    g.a_slots = g.groups * (2 * g.groups * g.kr <= 96 ? 2 : 1);
    g.th = ((int) TC_TMEM_COLS - g.a_slots * g.kr) / (2 * g.nb);
    g.th = g.th > 16 ? 16 : g.th;
    if (g.th < 2)
        return false;
    g.acc_cols = g.th * g.nb;
    // Bulk tensor copies need 16-byte aligned strides (the base address is
    // checked per call).
    g.use_tma = (cg.xs[1] % 4 == 0 && cg.xs[0] % 4 == 0 && cg.xs_c % 4 == 0 && cg.xs_n % 4 == 0) ? 1 : 0;
    tc_size_raw_ring(g);
    if (tc_smem_need(g) > 200 * 1024)
        return false;
    g.tiles_w = (g.out[2] + TC_M - 1) / TC_M;
    g.tiles_h = (g.out[1] + g.th - 1) / g.th;
    g.tiles = (long long) g.n * g.out[0] * g.tiles_h * g.tiles_w;
    if (g.tiles >= (1ll << 31))
        return false;
    *out = g;
    return true;
}

// Epilogue warps of the sweep kernel: 12, three per TMEM quadrant (8 were
// measured slower: 0.449 / 0.542 ms without / with statistics on the 256^3
// shard against 0.432 / 0.494).  DCB_SW_EPI=8 selects the smaller team
// (measurements).
int sw_epi_warps()
{
    static int v = 0;
    if (v == 0)
    {
        const char* e = std::getenv("DCB_SW_EPI");
        v = (e && std::atoi(e) == 8) ? 8 : 12;
    }
    return v;
}

size_t sw_smem_need(const SwGeom& g)
{
    return (size_t) (g.b_bytes + 127) / 128 * 128 + (size_t) g.raw_slots * g.raw_slot_bytes
           + (size_t) ((g.kr + 1) & ~1) * 4 + (size_t) (2 * g.a_slots + 64 + 2 * g.raw_slots + TC_GROUPS_MAX) * 8 + 64 + 128
           + (size_t) 12 * 2 * SW_NBK * 32 * 4 + 1024; // staging for up to 12 epilogue warps
}

// Geometry of the sweep kernel (filters with depth).  Needs bulk-copy
// compatible strides; the base address is checked per call.
bool sw_geom(const ConvGeom& cg, int math_mode, SwGeom* out)
{
    SwGeom g;
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
        if (g.pad[i] > g.f[i] - 1)
            return false;
    }
    g.n = cg.n;
    g.k = cg.k;
    g.xs_n = cg.xs_n;
    g.xs_c = cg.xs_c;
    g.ys_n = cg.ys_n;
    g.ys_c = cg.ys_c;
    if (g.f[0] < 2 || g.f[0] > 4 || g.k > SW_NBK)
        return false;
    // Three A slots of at most 53 k-rows each fit beside the accumulators: with
    // more input channels than that allows, the channels are taken in equal
    // groups, one launch per group, each adding into the output of the one
    // before (the sum over input channels is what a convolution is).
    g.split = (math_mode == DCB_MATH_TF32 || math_mode == DCB_MATH_BF16) ? 0 : 1;
    g.rnd_add = math_mode == DCB_MATH_BF16 ? 0x8000u : 0x1000u;
    g.rnd_mask = math_mode == DCB_MATH_BF16 ? 0xffff0000u : 0xffffe000u;
    g.w_c_total = cg.c;
    g.c = 0;
    for (int cgp = cg.c; cgp >= 1; --cgp)
        if (cg.c % cgp == 0 && 3 * ((cgp * g.f[2] * (g.split ? 3 : 1) + 7) / 8 * 8) <= 160)
        {
            g.c = cgp;
            break;
        }
    if (g.c == 0 || cg.c / g.c > 8)
        return false;
    g.cgroups = cg.c / g.c;
    g.w_c_off = 0;
    if ((long long) cg.n * cg.out[0] * cg.out[1] * cg.out[2] == 0)
        return false;
    if (g.pad[2] > 4 || g.f[2] - 1 - g.pad[2] > 4)
        return false;
    if (!(cg.xs[1] % 4 == 0 && cg.xs[0] % 4 == 0 && cg.xs_c % 4 == 0 && cg.xs_n % 4 == 0))
        return false;
    g.ntot = g.f[1] * g.f[0] * SW_NBK;
    if (g.ntot > 256 || (g.f[0] * SW_NBK) % 16)
        return false;
    g.crows = g.c * g.f[2];
    g.kr = (g.crows * (g.split ? 2 : 1) + 7) / 8 * 8;
    g.ks1 = g.kr / 8;
    g.ksteps = g.ks1 + (g.split ? (g.crows + 7) / 8 : 0);
    g.kb = g.ksteps * 8;
    g.b_rot_bytes = g.kb * g.ntot * 4;
    g.b_bytes = g.f[0] * g.b_rot_bytes;
    // an issuer must own one of any fh consecutive rows (see the hand-off
    // notes in the kernel header)
    // an issuer must own one of any fh consecutive rows (see the hand-off
    // notes in the kernel header): at most fh groups
    g.groups = g.f[1] < TC_GROUPS_MAX ? g.f[1] : TC_GROUPS_MAX;
    if (g.groups * g.kr > 160)
        return false;
    int slots_per_group = 1;
    {
        // measurement knobs: converter groups / issuers, A slots per group
        const char* eg = std::getenv("DCB_SW_GROUPS");
        const char* es = std::getenv("DCB_SW_SLOTS");
        if (eg && std::atoi(eg) >= 1 && std::atoi(eg) <= g.groups)
            g.groups = std::atoi(eg);
        if (es && std::atoi(es) >= 1 && std::atoi(es) <= 3)
            slots_per_group = std::atoi(es);
    }
    g.a_slots = g.groups * slots_per_group;
    if (g.a_slots * g.kr > 256)
        return false;
    int th_max = ((int) TC_TMEM_COLS - g.a_slots * g.kr) / (g.f[0] * SW_NBK);
    if (th_max + g.f[1] - 1 > 32)
        th_max = 32 - g.f[1] + 1;
    if (th_max > g.out[1])
        th_max = g.out[1];
    if (th_max < 2)
        return false;
    // Rows per column (th) and segments along D (nseg) together decide how
    // evenly the units fill the SMs: take the pair with the fewest staged
    // rows on the busiest SM.  Fewer rows per column cost more halo rows,
    // more segments cost more spill steps; both are in the count.
    const int sms = num_sms();
    long long best_cost = -1;
    int best_th = th_max, best_ns = 1;
    // measurement knob: a fixed column height
    const int th_forced = std::getenv("DCB_SW_TH") ? std::atoi(std::getenv("DCB_SW_TH")) : 0;
    for (int th = th_max; th >= 2 && th >= th_max - 3; --th)
    {
        if (th_forced >= 2 && th_forced <= th_max && th != th_forced)
            continue;
        const long long cols = (long long) g.n * ((g.out[2] + TC_M - 1) / TC_M) * ((g.out[1] + th - 1) / th);
        for (int ns = 1; ns <= g.out[0] && ns <= 64; ++ns)
        {
            const long long units = cols * ns;
            const long long waves = (units + sms - 1) / sms;
            const long long steps = (g.out[0] + ns - 1) / ns + 2 * (g.f[0] - 1);
            const long long cost = waves * steps * (th + g.f[1] - 1);
            if (best_cost < 0 || cost < best_cost)
            {
                best_cost = cost;
                best_th = th;
                best_ns = ns;
            }
        }
    }
    g.th = best_th;
    g.nseg = best_ns;
    g.rows = g.th + g.f[1] - 1;
    // Two A slots per group (and with them a second issuer per group in the plain
    // kernel) where the chosen column height leaves the tensor-memory columns for them.
    if (!std::getenv("DCB_SW_SLOTS") && 2 * g.groups * g.kr <= 256
        && 2 * g.groups * g.kr + g.th * g.f[0] * SW_NBK <= (int) TC_TMEM_COLS)
        g.a_slots = 2 * g.groups;
    // chunks of about 17 KiB, evenly sized
    const int row_bytes = g.c * TC_RAW_W * 4;
    int rc_max = (17 * 1024 + 512) / row_bytes;
    rc_max = rc_max < 1 ? 1 : rc_max;
    g.chunks_pp = (g.rows + rc_max - 1) / rc_max;
    g.chunk_rows = (g.rows + g.chunks_pp - 1) / g.chunks_pp;
    g.raw_slot_bytes = (g.chunk_rows * row_bytes + 127) / 128 * 128;
    int slots = (72 * 1024) / g.raw_slot_bytes;
    slots = slots > 6 ? 6 : slots;
    if (slots < 2)
        return false;
    g.raw_slots = slots;
    // more epilogue warps need more staging buffers: a shallower ring pays for them
    while (g.raw_slots > 3 && sw_smem_need(g) > 200 * 1024)
        --g.raw_slots;
    if (sw_smem_need(g) > 200 * 1024)
        return false;
    g.tiles_w = (g.out[2] + TC_M - 1) / TC_M;
    g.tiles_h = (g.out[1] + g.th - 1) / g.th;
    g.units = (long long) g.n * g.tiles_w * g.tiles_h * g.nseg;
    if (g.units >= (1ll << 31))
        return false;
    *out = g;
    return true;
}

size_t mg_smem_need(const SwGeom& g)
{
    return (size_t) (g.b_bytes + 127) / 128 * 128 + (size_t) g.raw_slots * g.raw_slot_bytes
           + (size_t) ((g.kr + 1) & ~1) * 4 + (size_t) (2 * g.a_slots + 64 + 2 * g.raw_slots + TC_GROUPS_MAX) * 8 + 64 + 128
           + (size_t) TC_EPI_WARPS * 2 * MG_NBK * 32 * 4 + 1024;
}

// Geometry of the multi-group sweep kernel: at most four filters, the input
// channels in two to eight equal groups walked inside one launch.
bool mg_geom(const ConvGeom& cg, int math_mode, SwGeom* out)
{
    SwGeom g;
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
        if (g.pad[i] > g.f[i] - 1)
            return false;
    }
    g.n = cg.n;
    g.k = cg.k;
    g.xs_n = cg.xs_n;
    g.xs_c = cg.xs_c;
    g.ys_n = cg.ys_n;
    g.ys_c = cg.ys_c;
    if (g.f[0] < 2 || g.f[0] > MG_SLOTS || g.k > MG_NBK || g.f[1] < TC_GROUPS_MAX)
        return false;
    if ((long long) cg.n * cg.out[0] * cg.out[1] * cg.out[2] == 0)
        return false;
    if (g.pad[2] > 4 || g.f[2] - 1 - g.pad[2] > 4)
        return false;
    if (!(cg.xs[1] % 4 == 0 && cg.xs[0] % 4 == 0 && cg.xs_c % 4 == 0 && cg.xs_n % 4 == 0))
        return false;
    g.split = (math_mode == DCB_MATH_TF32 || math_mode == DCB_MATH_BF16) ? 0 : 1;
    g.rnd_add = math_mode == DCB_MATH_BF16 ? 0x8000u : 0x1000u;
    g.rnd_mask = math_mode == DCB_MATH_BF16 ? 0xffff0000u : 0xffffe000u;
    g.w_c_total = cg.c;
    g.c = 0;
    for (int cgp = cg.c; cgp >= 1; --cgp)
        if (cg.c % cgp == 0 && 3 * ((cgp * g.f[2] * (g.split ? 3 : 1) + 7) / 8 * 8) <= 160)
        {
            g.c = cgp;
            break;
        }
    if (g.c == 0)
        return false;
    g.cgroups = cg.c / g.c;
    // Three to six groups.  Fewer than issuers would leave an issuer without a
    // sub-row in some rows (a single group is the sweep kernel's own case).  The
    // tensor pipe adds into its accumulators by truncation, 45 updates per group
    // and output: three groups on one chain stay inside the 1e-5 contract, four
    // sat on the bound (one run in six was 1 % over it, depending on the order
    // in which the issuers' instructions landed).  So more than three groups are
    // spread over two accumulator sets that the epilogue adds with rounding; more
    // than six take the sweep kernel's group launches.
    if (g.cgroups < TC_GROUPS_MAX || g.cgroups > 2 * TC_GROUPS_MAX)
        return false;
    g.nsets = g.cgroups > TC_GROUPS_MAX ? 2 : 1;
    g.w_c_off = 0;
    g.ntot = g.f[1] * MG_BLK;
    if (g.ntot > 256)
        return false;
    g.crows = g.c * g.f[2];
    g.kr = (g.crows * (g.split ? 2 : 1) + 7) / 8 * 8;
    g.ks1 = g.kr / 8;
    g.ksteps = g.ks1 + (g.split ? (g.crows + 7) / 8 : 0);
    g.kb = g.ksteps * 8;
    g.b_rot_bytes = g.kb * g.ntot * 4;
    g.b_bytes = g.cgroups * MG_SLOTS * g.b_rot_bytes;
    g.groups = TC_GROUPS_MAX;
    // two A slots per group, each with an issuer warp of its own, where tensor memory has
    // the columns (DCB_MG_SLOTS=1: one, for measurements)
    {
        int spg = 2 * g.groups * g.kr <= 192 ? 2 : 1;
        const char* e = std::getenv("DCB_MG_SLOTS");
        if (e && std::atoi(e) >= 1 && std::atoi(e) <= MG_IPG_MAX && std::atoi(e) * g.groups * g.kr <= 256)
            spg = std::atoi(e);
        g.a_slots = g.groups * spg;
    }
    int th_max = ((int) TC_TMEM_COLS - g.a_slots * g.kr) / (g.nsets * MG_BLK);
    if (th_max + g.f[1] - 1 > 32)
        th_max = 32 - g.f[1] + 1;
    if (th_max > g.out[1])
        th_max = g.out[1];
    if (th_max < 2)
        return false;
    const int sms = num_sms();
    long long best_cost = -1;
    int best_th = th_max, best_ns = 1;
    for (int th = th_max; th >= 2 && th >= th_max - 6; --th)
    {
        const long long cols = (long long) g.n * ((g.out[2] + TC_M - 1) / TC_M) * ((g.out[1] + th - 1) / th);
        for (int ns = 1; ns <= g.out[0] && ns <= 64; ++ns)
        {
            const long long units = cols * ns;
            const long long waves = (units + sms - 1) / sms;
            const long long steps = (g.out[0] + ns - 1) / ns + 2 * (g.f[0] - 1);
            const long long cost = waves * steps * (th + g.f[1] - 1);
            if (best_cost < 0 || cost < best_cost)
            {
                best_cost = cost;
                best_th = th;
                best_ns = ns;
            }
        }
    }
    g.th = best_th;
    g.nseg = best_ns;
    g.rows = g.th + g.f[1] - 1;
    const int row_bytes = g.w_c_total * TC_RAW_W * 4;
    int rc_max = (17 * 1024 + 512) / row_bytes;
    rc_max = rc_max < 1 ? 1 : rc_max;
    g.chunks_pp = (g.rows + rc_max - 1) / rc_max;
    g.chunk_rows = (g.rows + g.chunks_pp - 1) / g.chunks_pp;
    g.raw_slot_bytes = (g.chunk_rows * row_bytes + 127) / 128 * 128;
    int slots = (54 * 1024) / g.raw_slot_bytes;
    slots = slots > 4 ? 4 : slots;
    if (slots < 2)
        return false;
    g.raw_slots = slots;
    if (mg_smem_need(g) > 210 * 1024)
        return false;
    g.tiles_w = (g.out[2] + TC_M - 1) / TC_M;
    g.tiles_h = (g.out[1] + g.th - 1) / g.th;
    g.units = (long long) g.n * g.tiles_w * g.tiles_h * g.nseg;
    if (g.units >= (1ll << 31))
        return false;
    *out = g;
    return true;
}

size_t wg_smem_need(const WgGeom& g)
{
    const size_t unit = (size_t) (g.xbuf_bytes + g.dybuf_bytes + 127) / 128 * 128;
    return 2 * unit + (size_t) WG_A_SLOTS * WG_B_FLOATS * 4 + (2 * WG_A_SLOTS + 8) * 8 + 64 + 1024;
}

// Geometry of the tensor-core backward filter: x is the forward input window,
// dy the forward output window.
bool wg_geom(const ConvGeom& cg, int math_mode, WgGeom* out)
{
    WgGeom g;
    std::memset(&g, 0, sizeof(g));
    if (math_mode == DCB_MATH_FP32_SIMT)
        return false;
    for (int i = 0; i < 3; ++i)
    {
        if (cg.stride[i] < 1 || cg.stride[i] > 2 || cg.dil[i] != 1)
            return false;
        g.stride[i] = cg.stride[i];
        g.in[i] = cg.in[i];
        g.out[i] = cg.out[i];
        g.f[i] = cg.f[i];
        g.pad[i] = cg.pad[i];
        if (g.pad[i] > g.f[i] - 1)
            return false;
    }
    g.n = cg.n;
    g.c_total = cg.c;
    g.k_total = cg.k;
    const int taps = g.f[0] * g.f[1] * g.f[2];
    g.c = 0;
    for (int d = cg.c; d >= 1; --d)
        if (cg.c % d == 0 && d * taps <= 128)
        {
            g.c = d;
            break;
        }
    if (g.c == 0 || cg.k == 0)
        return false;
    g.cgroups = cg.c / g.c;
    g.k = cg.k < 16 ? cg.k : 16;
    g.kgroups = (cg.k + 15) / 16;
    if (g.cgroups * g.kgroups > 64)
        return false; // every launch reads dy again: the CUDA-core kernel does better
    g.mrows = g.c * taps;
    if ((long long) cg.n * cg.out[0] * cg.out[1] * cg.out[2] == 0)
        return false;
    if (g.pad[2] > 4 || g.f[2] - 1 - g.pad[2] > 4 || g.f[1] > 16)
        return false;
    // bulk-copy compatible strides on both tensors (bases are checked per call)
    if (!(cg.xs[1] % 4 == 0 && cg.xs[0] % 4 == 0 && cg.xs_c % 4 == 0 && cg.xs_n % 4 == 0))
        return false;
    if (!(cg.ys[1] % 4 == 0 && cg.ys[0] % 4 == 0 && cg.ys_c % 4 == 0 && cg.ys_n % 4 == 0))
        return false;
    g.xplane_bytes = g.c * g.f[1] * WG_XW * 4;
    g.xhalf_floats = (g.xplane_bytes + 127) / 128 * 128 / 4;
    g.xplane_floats = g.stride[2] * g.xhalf_floats;
    g.xbuf_bytes = g.f[0] * g.xplane_floats * 4;
    g.dybuf_bytes = 16 * WG_TW * 4;
    if (wg_smem_need(g) > 200 * 1024)
        return false;
    g.tiles_w = (g.out[2] + WG_TW - 1) / WG_TW;
    g.units = (long long) g.n * g.out[0] * g.out[1] * g.tiles_w;
    if (g.units >= (1ll << 31))
        return false;
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

// One channel group's output, dense, rows padded to 16 bytes.
static size_t sw_scratch_floats(const SwGeom& g)
{
    const size_t wp = (size_t) (g.out[2] + 3) / 4 * 4;
    return (size_t) g.n * g.k * g.out[0] * g.out[1] * wp;
}

// y (strided window) += the sum of `nsrc` dense group outputs; one block per
// output row.
__global__ void sw_group_sum_kernel(SwGeom g, const float* __restrict__ scratch, size_t slice, int nsrc, float* y)
{
    const int wp = (g.out[2] + 3) / 4 * 4;
    long long r = blockIdx.x; // (n, k, od, oh)
    const int oh = (int) (r % g.out[1]);
    r /= g.out[1];
    const int od = (int) (r % g.out[0]);
    r /= g.out[0];
    const int k = (int) (r % g.k);
    const int n = (int) (r / g.k);
    const float* s = scratch + (size_t) blockIdx.x * wp;
    float* yp = y + (size_t) n * g.ys_n + (size_t) k * g.ys_c + (size_t) od * g.ys[0] + (size_t) oh * g.ys[1];
    for (int w = threadIdx.x; w < g.out[2]; w += blockDim.x)
    {
        float acc = yp[w];
        for (int i = 0; i < nsrc; ++i)
            acc += s[(size_t) i * slice + w];
        yp[w] = acc;
    }
}

struct TcPlan
{
    bool has[2] = {false, false};
    TcGeom g[2];
    float* bimg[2] = {nullptr, nullptr};
    // the sweep kernel, preferred where it applies (filters with depth)
    bool has_sw[2] = {false, false};
    SwGeom sw[2];
    float* sw_bimg[2] = {nullptr, nullptr};
    // the multi-group sweep kernel (few filters, many input channels: backward data)
    bool has_mg[2] = {false, false};
    SwGeom mg[2];
    float* mg_bimg[2] = {nullptr, nullptr};
    float* grp_scratch[2] = {nullptr, nullptr}; // dense outputs of the channel groups after the first
    float* stat_part = nullptr; // per epilogue warp partial sums of the fused statistics
    // tensor-core backward filter
    bool has_wg = false;
    WgGeom wg;
    ConvGeom wg_cg;             // strides of x and dy for the tensor maps
    float* wg_part = nullptr;   // one 128 x 16 partial filter per CTA
    int* status = nullptr;
};

int32_t tc_plan_create(const ConvGeom& fwd, const ConvGeom& bwd, bool bwd_is_fwd, int math_mode, TcPlan** out)
{
    *out = nullptr;
    auto* p = new TcPlan();
    p->has[0] = tc_geom(fwd, math_mode, &p->g[0]);
    p->has[1] = bwd_is_fwd && tc_geom(bwd, math_mode, &p->g[1]);
    // the sweep kernel falls back to the row kernel when a call's base address
    // is not 16-byte aligned, so it is only planned on top of it
    p->has_sw[0] = p->has[0] && sw_geom(fwd, math_mode, &p->sw[0]);
    p->has_sw[1] = p->has[1] && sw_geom(bwd, math_mode, &p->sw[1]);
    p->has_mg[0] = p->has[0] && mg_geom(fwd, math_mode, &p->mg[0]);
    p->has_mg[1] = p->has[1] && mg_geom(bwd, math_mode, &p->mg[1]);
    p->has_wg = wg_geom(fwd, math_mode, &p->wg);
    p->wg_cg = fwd;
    if (!p->has[0] && !p->has[1] && !p->has_wg)
    {
        delete p;
        return DCB_OK;
    }
    bool ok = cudaMalloc(&p->status, sizeof(int)) == cudaSuccess
              && cudaMemset(p->status, 0, sizeof(int)) == cudaSuccess;
    for (int s = 0; s < 2 && ok; ++s)
    {
        if (p->has[s])
            ok = cudaMalloc(&p->bimg[s], p->g[s].b_bytes) == cudaSuccess;
        if (ok && p->has_sw[s])
            ok = cudaMalloc(&p->sw_bimg[s], p->sw[s].b_bytes) == cudaSuccess;
        if (ok && p->has_mg[s])
            ok = cudaMalloc(&p->mg_bimg[s], p->mg[s].b_bytes) == cudaSuccess;
        if (ok && p->has_sw[s] && p->sw[s].cgroups > 1 && !p->has_mg[s])
            ok = cudaMalloc(&p->grp_scratch[s], sw_scratch_floats(p->sw[s]) * (p->sw[s].cgroups - 1) * sizeof(float))
                 == cudaSuccess;
    }
    if (ok && p->has_wg)
        ok = cudaMalloc(&p->wg_part, (size_t) num_sms() * 128 * 16 * sizeof(float)) == cudaSuccess;
    if (ok && p->has_sw[0])
        ok = cudaMalloc(&p->stat_part, (size_t) num_sms() * 12 * 32 * sizeof(float)) == cudaSuccess;
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
    cudaFree(p->sw_bimg[0]);
    cudaFree(p->sw_bimg[1]);
    cudaFree(p->mg_bimg[0]);
    cudaFree(p->mg_bimg[1]);
    cudaFree(p->grp_scratch[0]);
    cudaFree(p->grp_scratch[1]);
    cudaFree(p->stat_part);
    cudaFree(p->wg_part);
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
    return p->has_wg;
}

int tc_variant(const TcPlan* p, int which)
{
    if (!p || which < 0 || which > 2)
        return 0;
    if (which == 2)
        return p->has_wg ? 5 : 0;
    if (!p->has[which])
        return 0;
    if (p->has_mg[which])
        return 4;
    if (p->has_sw[which])
        return 3;
    return p->g[which].use_tma ? 1 : 2;
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

// Floats between the 16-byte boundary at or below x and x.  A shard with halo cells
// along W is laid out so that its OWNED cells start on a 16-byte boundary (stores and
// the streaming kernels want that); its window, which starts with the halo cells, then
// does not.  A bulk copy can over-fetch but not start in between, so such a window is
// described from the boundary below it and the kernel skips the cells in front.  Those
// cells lie in the same allocation (allocations start 16-byte aligned) and are only read.
static inline int x_skip(const float* x)
{
    return (int) ((reinterpret_cast<uintptr_t>(x) & 15) / 4);
}

// Where a staged row starts relative to the first output of a tile (lx) and where tap 0
// sits in it (rx).  Aligned window: 4 cells of margin on the left for the padding.
// Skipped cells in front (only with pad 0): the row starts at the tile's first output.
template <class Geom>
static void tc_row_window(Geom& g, int skip)
{
    g.lx = skip ? 0 : -4;
    g.rx = skip ? skip : 4 - g.pad[2];
}

// can a window that starts `skip` floats above a 16-byte boundary be staged in rows of row_w cells?
static bool skip_ok(int skip, int pad_w, int fw, int tile_w, int row_w)
{
    if (skip == 0)
        return true;
    // cells left of the window are not zeros here, so nothing may read them as padding
    return pad_w == 0 && skip + fw - 1 + tile_w <= row_w;
}

// Descriptor of the input window as a 5-D tensor (W, H, D, C, N) whose box is
// chunk_rows raw rows of every channel.  Returns false when the window cannot be
// described (alignment), in which case the register-fed producers run.
static bool make_x_map(const TcGeom& g, const float* x, CUtensorMap* map)
{
    EncodeTiledFn fn = encode_tiled_fn();
    const int skip = x_skip(x);
    if (!fn || (reinterpret_cast<uintptr_t>(x) & 3) != 0 || !skip_ok(skip, g.pad[2], g.f[2], TC_M, TC_RAW_W))
        return false;
    x -= skip;
    const cuuint64_t dims[5] = {(cuuint64_t) (g.in[2] + skip), (cuuint64_t) g.in[1], (cuuint64_t) g.in[0],
                                (cuuint64_t) g.c, (cuuint64_t) g.n};
    // a dimension of extent 1 may carry any stride; give it a valid one
    const long long s1 = g.xs[1], s0 = g.in[0] > 1 ? g.xs[0] : g.xs[1] * g.in[1];
    const cuuint64_t strides[4] = {(cuuint64_t) s1 * 4, (cuuint64_t) s0 * 4, (cuuint64_t) g.xs_c * 4,
                                   (cuuint64_t) (g.n > 1 ? g.xs_n : g.xs_c * g.c) * 4};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] == 0)
            return false;
    const cuuint32_t box[5] = {(cuuint32_t) TC_RAW_W, (cuuint32_t) g.chunk_rows, 1, (cuuint32_t) g.c, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(x), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

template <int NB>
static int32_t tc_launch(const TcGeom& g_in, float alpha, const float* x, const float* bimg, float beta, float* y,
                         int* status, cudaStream_t stream)
{
    TcGeom g = g_in;
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    if (g.use_tma && !make_x_map(g, x, &map))
    {
        g.use_tma = 0; // the converters fetch their own rows
        tc_size_raw_ring(g);
    }
    tc_row_window(g, g.use_tma ? x_skip(x) : 0);
    const size_t smem = tc_smem_bytes(g);
    if (smem > 220 * 1024)
        return DCB_UNSUPPORTED;
    long long grid = (long long) num_sms();
    if (grid > g.tiles)
        grid = g.tiles;
    // the spelled-out converter for 4 channels x 3 taps, pad 1 or 0 (a shard with its W halo), hi / lo split
    const bool c4f3 = g.c == 4 && g.f[2] == 3 && g.pad[2] <= 1 && g.split;
    if (c4f3)
    {
        DCB_CUDA_TRY(cudaFuncSetAttribute(tc_conv_kernel<NB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int) (224 * 1024)));
        tc_conv_kernel<NB, true><<<(unsigned) grid, TC_THREADS, smem, stream>>>(g, alpha, beta, x, bimg, y, status,
                                                                             map);
    }
    else
    {
        DCB_CUDA_TRY(cudaFuncSetAttribute(tc_conv_kernel<NB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int) (224 * 1024)));
        tc_conv_kernel<NB, false><<<(unsigned) grid, TC_THREADS, smem, stream>>>(g, alpha, beta, x, bimg, y, status,
                                                                              map);
    }
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

// Descriptor of the input window for the sweep kernel: box = chunk_rows raw rows
// of every channel.
static bool sw_make_x_map(const SwGeom& g, const float* x, CUtensorMap* map)
{
    TcGeom t;
    std::memset(&t, 0, sizeof(t));
    for (int i = 0; i < 3; ++i)
    {
        t.in[i] = g.in[i];
        t.xs[i] = g.xs[i];
        t.pad[i] = g.pad[i];
        t.f[i] = g.f[i];
    }
    t.n = g.n;
    t.c = g.c;
    t.xs_n = g.xs_n;
    t.xs_c = g.xs_c;
    t.chunk_rows = g.chunk_rows;
    return make_x_map(t, x, map);
}

// Descriptor of the output as a 5-D tensor (W, H, D, K, N) whose box is 32
// outputs of every filter: what one epilogue warp stores per row.  Returns
// false when the output cannot be described (alignment); the kernel then
// stores from registers.
static bool sw_make_y_map(const SwGeom& g, float* y, CUtensorMap* map)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(y) & 15) != 0)
        return false;
    // A bulk tensor store was seen to clip a row at the next 16-byte boundary,
    // not at the tensor's extent: a row of 11 outputs inside a wider allocation
    // (a column range of a shard) had its 12th cell overwritten.  Rows whose
    // extent is not a multiple of 4 floats take the register stores.
    if (g.out[2] % 4 != 0)
        return false;
    const cuuint64_t dims[5] = {(cuuint64_t) g.out[2], (cuuint64_t) g.out[1], (cuuint64_t) g.out[0], (cuuint64_t) g.k,
                                (cuuint64_t) g.n};
    const long long s1 = g.out[1] > 1 ? g.ys[1] : g.out[2];
    const long long s0 = g.out[0] > 1 ? g.ys[0] : s1 * g.out[1];
    const long long sc = g.k > 1 ? g.ys_c : s0 * g.out[0];
    const long long sn = g.n > 1 ? g.ys_n : sc * g.k;
    const cuuint64_t strides[4] = {(cuuint64_t) s1 * 4, (cuuint64_t) s0 * 4, (cuuint64_t) sc * 4, (cuuint64_t) sn * 4};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] == 0)
            return false;
    const cuuint32_t box[5] = {32, 1, 1, (cuuint32_t) SW_NBK, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

static int32_t sw_launch(const SwGeom& g_in, float alpha, const float* w, const float* x, float* bimg, float beta,
                         float* y, int* status, const CUtensorMap& map, cudaStream_t stream,
                         float* stat_part = nullptr, float* sums = nullptr, float* sqsums = nullptr)
{
    SwGeom g = g_in;
    tc_row_window(g, x_skip(x));
#if DCB_SW_KNOCKOUT
    // knock-out bits for timing experiments (results are wrong with any of them set)
    g.nsets = std::getenv("DCB_SW_DBG") ? std::atoi(std::getenv("DCB_SW_DBG")) : 0;
#endif
    CUtensorMap ymap;
    std::memset(&ymap, 0, sizeof(ymap));
    const int use_ymap = sw_make_y_map(g, y, &ymap) ? 1 : 0;
    const long long total = (long long) g.b_bytes / 4;
    sw_pack_filter_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, stream>>>(w, bimg, g);
    DCB_LAUNCH_CHECK();
    size_t smem = sw_smem_need(g);
    smem = smem < 120 * 1024 ? 120 * 1024 : smem; // one CTA per SM: it owns all of tensor memory
    long long grid = (long long) num_sms();
    if (grid > g.units)
        grid = g.units;
    const bool c4f3 = g.c == 4 && g.f[2] == 3 && g.pad[2] <= 1 && g.split;
    const bool stats = stat_part != nullptr;
    const int epi = sw_epi_warps();
    long long* prof = nullptr;
#if DCB_SW_PROFILE
    // per-role clock accounting: one launch is measured and printed, synchronously
    static int prof_left = std::getenv("DCB_SW_PROF_LAUNCHES") ? std::atoi(std::getenv("DCB_SW_PROF_LAUNCHES")) : 0;
    const size_t prof_n = (size_t) grid * 32 * 8;
    if (prof_left > 0)
    {
        DCB_CUDA_TRY(cudaMalloc(&prof, prof_n * sizeof(long long)));
        DCB_CUDA_TRY(cudaMemsetAsync(prof, 0, prof_n * sizeof(long long), stream));
    }
#endif
    const bool blend = beta != 0.f;
    // second issuers (and the second A slot of every group) for the plain variant only
    const bool xiss = !stats && !blend && g.a_slots == 2 * g.groups;
    if (!xiss)
        g.a_slots = g.groups;
    auto launch = [&](auto kernel, int xi) -> int32_t {
        DCB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) (224 * 1024)));
        kernel<<<(unsigned) grid, sw_threads(epi, xi), smem, stream>>>(g, alpha, beta, bimg, y, status, map, ymap,
                                                                       use_ymap, stat_part, prof);
        return DCB_OK;
    };
    int32_t st;
#define DCB_SW_PICK(EPI)                                                                                              \
    if (xiss)                                                                                                         \
        st = c4f3 ? launch(sw_conv_kernel<true, false, false, EPI, 1>, 1)                                             \
                  : launch(sw_conv_kernel<false, false, false, EPI, 1>, 1);                                           \
    else if (c4f3)                                                                                                    \
        st = stats ? launch(sw_conv_kernel<true, true, false, EPI, 0>, 0)                                             \
                   : (blend ? launch(sw_conv_kernel<true, false, true, EPI, 0>, 0)                                    \
                            : launch(sw_conv_kernel<true, false, false, EPI, 0>, 0));                                 \
    else                                                                                                              \
        st = stats ? launch(sw_conv_kernel<false, true, false, EPI, 0>, 0)                                            \
                   : (blend ? launch(sw_conv_kernel<false, false, true, EPI, 0>, 0)                                   \
                            : launch(sw_conv_kernel<false, false, false, EPI, 0>, 0));
    if (epi == 12)
    {
        DCB_SW_PICK(12)
    }
    else
    {
        DCB_SW_PICK(8)
    }
#undef DCB_SW_PICK
    if (st != DCB_OK)
        return st;
    DCB_LAUNCH_CHECK();
#if DCB_SW_PROFILE
    if (prof != nullptr)
    {
        --prof_left;
        std::vector<long long> h(prof_n);
        DCB_CUDA_TRY(cudaStreamSynchronize(stream));
        DCB_CUDA_TRY(cudaMemcpy(h.data(), prof, prof_n * sizeof(long long), cudaMemcpyDeviceToHost));
        cudaFree(prof);
        const int t0 = TC_TMA_WARP, e0 = TC_TMA_WARP + 1;
        auto role = [&](const char* name, int w_lo, int w_hi, const char* const* labels) {
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long n = 0;
            for (long long b = 0; b < grid; ++b)
                for (int w = w_lo; w < w_hi; ++w)
                {
                    const long long* r = &h[((size_t) b * 32 + w) * 8];
                    if (r[7] == 0)
                        continue;
                    for (int i = 0; i < 8; ++i)
                        acc[i] += (double) r[i];
                    ++n;
                }
            if (n == 0)
                return;
            std::fprintf(stderr, "[sw prof] %-10s warps %lld total %.0f:", name, n, acc[7] / n);
            for (int i = 0; i < 5; ++i)
                std::fprintf(stderr, " %s %.1f%%", labels[i], 100.0 * acc[i] / acc[7]);
            std::fprintf(stderr, " | extra clocks per warp %.0f\n", acc[5] / n);
        };
        const char* lc[5] = {"wait_raw", "convert", "wait_a_empty", "st+arrive", "other"};
        const char* li[5] = {"wait_row_free", "wait_a_full", "issue", "-", "other"};
        const char* lt[5] = {"wait_raw_empty", "copy", "-", "-", "other"};
        const char* le[5] = {"wait_row_done", "tmem_ld", "zero+arrive", "stats+store", "other"};
        role("converter", 0, TC_PRODUCERS, lc);
        role("issuer", TC_MMA_WARP, t0, li);
        role("copy", t0, t0 + 1, lt);
        role("epilogue", e0, e0 + epi, le);
    }
#endif
    if (stats)
    {
        sw_stats_fold_kernel<<<1, SW_FOLD_WARPS * 32, 0, stream>>>(stat_part, (int) grid * epi, g.k, sums, sqsums);
        DCB_LAUNCH_CHECK();
    }
    (void) x;
    return DCB_OK;
}

// Input map for the multi-group kernel: all channels of a chunk of rows.
static bool mg_make_x_map(const SwGeom& g, const float* x, CUtensorMap* map)
{
    TcGeom t;
    std::memset(&t, 0, sizeof(t));
    for (int i = 0; i < 3; ++i)
    {
        t.in[i] = g.in[i];
        t.xs[i] = g.xs[i];
        t.pad[i] = g.pad[i];
        t.f[i] = g.f[i];
    }
    t.n = g.n;
    t.c = g.w_c_total;
    t.xs_n = g.xs_n;
    t.xs_c = g.xs_c;
    t.chunk_rows = g.chunk_rows;
    return make_x_map(t, x, map);
}

// Output map with a box of 32 outputs x MG_NBK filters.
static bool mg_make_y_map(const SwGeom& g, float* y, CUtensorMap* map)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(y) & 15) != 0)
        return false;
    // A bulk tensor store was seen to clip a row at the next 16-byte boundary,
    // not at the tensor's extent: a row of 11 outputs inside a wider allocation
    // (a column range of a shard) had its 12th cell overwritten.  Rows whose
    // extent is not a multiple of 4 floats take the register stores.
    if (g.out[2] % 4 != 0)
        return false;
    const cuuint64_t dims[5] = {(cuuint64_t) g.out[2], (cuuint64_t) g.out[1], (cuuint64_t) g.out[0], (cuuint64_t) g.k,
                                (cuuint64_t) g.n};
    const long long s1 = g.out[1] > 1 ? g.ys[1] : g.out[2];
    const long long s0 = g.out[0] > 1 ? g.ys[0] : s1 * g.out[1];
    const long long sc = g.k > 1 ? g.ys_c : s0 * g.out[0];
    const long long sn = g.n > 1 ? g.ys_n : sc * g.k;
    const cuuint64_t strides[4] = {(cuuint64_t) s1 * 4, (cuuint64_t) s0 * 4, (cuuint64_t) sc * 4, (cuuint64_t) sn * 4};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] == 0)
            return false;
    const cuuint32_t box[5] = {32, 1, 1, (cuuint32_t) MG_NBK, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

static int32_t mg_launch(const SwGeom& g_in, float alpha, const float* w, const float* x, float* bimg, float* y,
                         int* status, const CUtensorMap& xmap, cudaStream_t stream)
{
    SwGeom g = g_in;
    tc_row_window(g, x_skip(x));
    CUtensorMap ymap;
    std::memset(&ymap, 0, sizeof(ymap));
    const int use_ymap = mg_make_y_map(g, y, &ymap) ? 1 : 0;
    const long long total = (long long) g.b_bytes / 4;
    mg_pack_filter_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, stream>>>(w, bimg, g);
    DCB_LAUNCH_CHECK();
    size_t smem = mg_smem_need(g);
    smem = smem < 120 * 1024 ? 120 * 1024 : smem;
    long long grid = (long long) num_sms();
    if (grid > g.units)
        grid = g.units;
    const bool c4f3 = g.c == 4 && g.f[2] == 3 && g.pad[2] <= 1 && g.split;
    long long* prof = nullptr;
#if DCB_SW_PROFILE
    // per-role clock accounting as in the sweep kernel: DCB_MG_PROF_LAUNCHES launches are
    // measured and printed, synchronously
    static int prof_left = std::getenv("DCB_MG_PROF_LAUNCHES") ? std::atoi(std::getenv("DCB_MG_PROF_LAUNCHES")) : 0;
    const size_t prof_n = (size_t) grid * 32 * 8;
    if (prof_left > 0)
    {
        DCB_CUDA_TRY(cudaMalloc(&prof, prof_n * sizeof(long long)));
        DCB_CUDA_TRY(cudaMemsetAsync(prof, 0, prof_n * sizeof(long long), stream));
    }
#endif
    if (c4f3)
    {
        DCB_CUDA_TRY(cudaFuncSetAttribute(mg_conv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int) (224 * 1024)));
        mg_conv_kernel<true><<<(unsigned) grid, MG_THREADS, smem, stream>>>(g, alpha, bimg, y, status, xmap, ymap,
                                                                           use_ymap, prof);
    }
    else
    {
        DCB_CUDA_TRY(cudaFuncSetAttribute(mg_conv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int) (224 * 1024)));
        mg_conv_kernel<false><<<(unsigned) grid, MG_THREADS, smem, stream>>>(g, alpha, bimg, y, status, xmap, ymap,
                                                                            use_ymap, prof);
    }
    DCB_LAUNCH_CHECK();
#if DCB_SW_PROFILE
    if (prof != nullptr)
    {
        --prof_left;
        std::vector<long long> h(prof_n);
        DCB_CUDA_TRY(cudaStreamSynchronize(stream));
        DCB_CUDA_TRY(cudaMemcpy(h.data(), prof, prof_n * sizeof(long long), cudaMemcpyDeviceToHost));
        cudaFree(prof);
        auto role = [&](const char* name, int w_lo, int w_hi, const char* const* labels) {
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long n = 0;
            for (long long b = 0; b < grid; ++b)
                for (int w = w_lo; w < w_hi; ++w)
                {
                    const long long* r = &h[((size_t) b * 32 + w) * 8];
                    if (r[7] == 0)
                        continue;
                    for (int i = 0; i < 8; ++i)
                        acc[i] += (double) r[i];
                    ++n;
                }
            if (n == 0)
                return;
            std::fprintf(stderr, "[mg prof] %-10s warps %lld total %.0f:", name, n, acc[7] / n);
            for (int i = 0; i < 5; ++i)
                std::fprintf(stderr, " %s %.1f%%", labels[i], 100.0 * acc[i] / acc[7]);
            std::fprintf(stderr, "\n");
        };
        const char* lc[5] = {"wait_raw", "convert", "wait_a_empty", "st+arrive", "other"};
        const char* li[5] = {"wait_row_free", "wait_a_full", "issue", "wait_iss_sync", "other"};
        const char* le[5] = {"wait_row_done", "tmem_ld", "zero+arrive", "stage+store", "other"};
        role("converter", 0, TC_PRODUCERS, lc);
        role("issuer 1", TC_MMA_WARP, TC_TMA_WARP, li);
        role("issuer 2", MG_ISSUER2_WARP, MG_THREADS / 32, li);
        role("epilogue", TC_TMA_WARP + 1, MG_ISSUER2_WARP, le);
        std::fprintf(stderr, "[mg prof] th %d nsets %d cgroups %d a_slots %d groups %d raw_slots %d chunks_pp %d\n", g.th,
                     g.nsets, g.cgroups, g.a_slots, g.groups, g.raw_slots, g.chunks_pp);
    }
#endif
    return DCB_OK;
}

int32_t tc_conv_fwd(TcPlan* p, int slot, float alpha, const float* x, const float* w, float beta, float* y,
                    cudaStream_t stream)
{
    if (!p || slot < 0 || slot > 1 || !p->has[slot])
        return DCB_UNSUPPORTED;
    if (p->has_mg[slot] && beta == 0.f)
    {
        CUtensorMap xmap;
        std::memset(&xmap, 0, sizeof(xmap));
        if (mg_make_x_map(p->mg[slot], x, &xmap))
            return mg_launch(p->mg[slot], alpha, w, x, p->mg_bimg[slot], y, p->status, xmap, stream);
    }
    if (p->has_sw[slot])
    {
        SwGeom sg = p->sw[slot];
        CUtensorMap maps[8];
        bool ok = true;
        for (int grp = 0; grp < sg.cgroups && ok; ++grp)
        {
            std::memset(&maps[grp], 0, sizeof(CUtensorMap));
            ok = sw_make_x_map(sg, x + (size_t) grp * sg.c * sg.xs_c, &maps[grp]);
        }
        if (ok)
        {
            // The first group writes the output (blending with the old one if
            // beta asks for it); every further group writes its own dense
            // scratch slice with the plain, faster kernel, and one pass adds the
            // slices into the output.  (Plans that normally take the
            // multi-group kernel own no scratch: their rare beta != 0 calls
            // blend every further group into the output instead.)
            const size_t slice = sw_scratch_floats(sg);
            for (int grp = 0; grp < sg.cgroups; ++grp)
            {
                SwGeom lg = sg;
                lg.w_c_off = grp * sg.c;
                float* dst = y;
                const bool to_scratch = grp > 0 && p->grp_scratch[slot] != nullptr;
                if (to_scratch)
                {
                    const long long wp = (sg.out[2] + 3) / 4 * 4;
                    lg.ys[2] = 1;
                    lg.ys[1] = wp;
                    lg.ys[0] = wp * sg.out[1];
                    lg.ys_c = lg.ys[0] * sg.out[0];
                    lg.ys_n = lg.ys_c * sg.k;
                    dst = p->grp_scratch[slot] + (size_t) (grp - 1) * slice;
                }
                const int32_t st = sw_launch(lg, alpha, w, x + (size_t) grp * sg.c * sg.xs_c, p->sw_bimg[slot],
                                             grp == 0 ? beta : (to_scratch ? 0.f : 1.f), dst, p->status, maps[grp],
                                             stream);
                if (st != DCB_OK)
                    return st;
            }
            if (sg.cgroups > 1 && p->grp_scratch[slot] != nullptr)
            {
                const long long rows = (long long) sg.n * sg.k * sg.out[0] * sg.out[1];
                sw_group_sum_kernel<<<(unsigned) rows, 128, 0, stream>>>(sg, p->grp_scratch[slot], slice,
                                                                         sg.cgroups - 1, y);
                DCB_LAUNCH_CHECK();
            }
            return DCB_OK;
        }
    }
    const TcGeom& g0 = p->g[slot];
    for (int kg = 0; kg < g0.kgroups; ++kg)
        for (int cgp = 0; cgp < g0.cgroups; ++cgp)
        {
            TcGeom g = g0;
            g.w_k_off = kg * g0.kpad;
            g.w_c_off = cgp * g0.c;
            g.k = g0.k_total - g.w_k_off < g0.kpad ? g0.k_total - g.w_k_off : g0.kpad;
            const long long total = (long long) g.b_bytes / 4;
            tc_pack_filter_kernel<<<(unsigned) ((total + 255) / 256), 256, 0, stream>>>(w, p->bimg[slot], g);
            DCB_LAUNCH_CHECK();
            const float* xg = x + (size_t) g.w_c_off * g.xs_c;
            float* yg = y + (size_t) g.w_k_off * g.ys_c;
            const float b = cgp == 0 ? beta : 1.f; // later channel groups add into the output
            int32_t st;
            switch (g.nb)
            {
            case 16: st = tc_launch<16>(g, alpha, xg, p->bimg[slot], b, yg, p->status, stream); break;
            case 32: st = tc_launch<32>(g, alpha, xg, p->bimg[slot], b, yg, p->status, stream); break;
            case 64: st = tc_launch<64>(g, alpha, xg, p->bimg[slot], b, yg, p->status, stream); break;
            default: st = DCB_UNSUPPORTED;
            }
            if (st != DCB_OK)
                return st;
        }
    return DCB_OK;
}

int32_t tc_conv_fwd_stats(TcPlan* p, float alpha, const float* x, const float* w, float* y, float* sums,
                          float* sqsums, cudaStream_t stream)
{
    if (!p || !p->has_sw[0] || !p->stat_part || p->sw[0].cgroups != 1)
        return DCB_UNSUPPORTED;
    CUtensorMap map;
    std::memset(&map, 0, sizeof(map));
    if (!sw_make_x_map(p->sw[0], x, &map))
        return DCB_UNSUPPORTED;
    return sw_launch(p->sw[0], alpha, w, x, p->sw_bimg[0], 0.f, y, p->status, map, stream, p->stat_part, sums, sqsums);
}

// 5-D map (W, H, D, channels, N) of a strided window with the given box.
// `skip` floats in front of the window are mapped with it (see x_skip): base - skip must be aligned.
static bool wg_make_map(const float* base, const int ext[3], int channels, int n, const long long sp[3],
                        long long s_c, long long s_n, int box_w, int box_h, int box_c, CUtensorMap* map,
                        int skip = 0)
{
    EncodeTiledFn fn = encode_tiled_fn();
    base -= skip;
    if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return false;
    const cuuint64_t dims[5] = {(cuuint64_t) (ext[2] + skip), (cuuint64_t) ext[1], (cuuint64_t) ext[0],
                                (cuuint64_t) channels, (cuuint64_t) n};
    const long long s1 = ext[1] > 1 ? sp[1] : ext[2];
    const long long s0 = ext[0] > 1 ? sp[0] : s1 * ext[1];
    const long long sc = channels > 1 ? s_c : s0 * ext[0];
    const long long sn = n > 1 ? s_n : sc * channels;
    const cuuint64_t strides[4] = {(cuuint64_t) s1 * 4, (cuuint64_t) s0 * 4, (cuuint64_t) sc * 4, (cuuint64_t) sn * 4};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] == 0)
            return false;
    const cuuint32_t box[5] = {(cuuint32_t) box_w, (cuuint32_t) box_h, 1, (cuuint32_t) box_c, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}

int32_t tc_conv_bwd_filter(TcPlan* p, float alpha, const float* x, const float* dy, float beta, float* dw,
                           cudaStream_t stream)
{
    if (!p || !p->has_wg)
        return DCB_UNSUPPORTED;
    WgGeom g = p->wg;
    const ConvGeom& cg = p->wg_cg;
    const int skip = x_skip(x);
    // cells one bulk copy's outputs span: 128 at stride 1, 64 outputs at every second cell at stride 2
    const int span = g.stride[2] == 2 ? 2 * (WG_TW / 2 - 1) + 1 : WG_TW;
    if ((reinterpret_cast<uintptr_t>(x) & 3) != 0 || !skip_ok(skip, g.pad[2], g.f[2], span, WG_XW))
        return DCB_UNSUPPORTED; // the caller falls back to the CUDA-core kernel
    tc_row_window(g, skip);
#if DCB_WG_KNOCKOUT
    g.dbg = std::getenv("DCB_WG_DBG") ? std::atoi(std::getenv("DCB_WG_DBG")) : 0;
#else
    g.dbg = 0;
#endif
    size_t smem = wg_smem_need(g);
    smem = smem < 120 * 1024 ? 120 * 1024 : smem; // one CTA per SM
    long long grid = (long long) num_sms();
    if (grid > g.units)
        grid = g.units;
    const int taps = g.f[0] * g.f[1] * g.f[2];
    // all maps first: a pointer that cannot be mapped must refuse before anything ran
    std::vector<CUtensorMap> xmaps((size_t) g.cgroups), dymaps((size_t) g.kgroups);
    for (int cgp = 0; cgp < g.cgroups; ++cgp)
    {
        std::memset(&xmaps[cgp], 0, sizeof(CUtensorMap));
        if (!wg_make_map(x + (size_t) cgp * g.c * cg.xs_c, cg.in, g.c, cg.n, cg.xs, cg.xs_c, cg.xs_n, WG_XW, g.f[1],
                         g.c, &xmaps[cgp], skip))
            return DCB_UNSUPPORTED; // the caller falls back to the CUDA-core kernel
    }
    for (int kg = 0; kg < g.kgroups; ++kg)
    {
        std::memset(&dymaps[kg], 0, sizeof(CUtensorMap));
        const int kcur = g.k_total - kg * 16 < 16 ? g.k_total - kg * 16 : 16;
        if (!wg_make_map(dy + (size_t) kg * 16 * cg.ys_c, cg.out, kcur, cg.n, cg.ys, cg.ys_c, cg.ys_n, WG_TW, 1, 16,
                         &dymaps[kg]))
            return DCB_UNSUPPORTED;
    }
    auto kernel = g.stride[2] == 2 ? wg_conv_kernel<2> : wg_conv_kernel<1>;
    DCB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) (224 * 1024)));
    for (int kg = 0; kg < g.kgroups; ++kg)
        for (int cgp = 0; cgp < g.cgroups; ++cgp)
        {
            const int kcur = g.k_total - kg * 16 < 16 ? g.k_total - kg * 16 : 16;
            kernel<<<(unsigned) grid, WG_THREADS, smem, stream>>>(g, p->wg_part, p->status, xmaps[cgp], dymaps[kg]);
            DCB_LAUNCH_CHECK();
            const int total = g.mrows * kcur;
            wg_fold_kernel<<<(total + 255) / 256, 256, 0, stream>>>(p->wg_part, (int) grid, g.mrows, kcur, taps,
                                                                    g.c_total, cgp * g.c, kg * 16, alpha, beta, dw);
            DCB_LAUNCH_CHECK();
        }
    return DCB_OK;
}

} // namespace dcb
