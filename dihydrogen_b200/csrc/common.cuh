// Shared helpers for the libdistconv_b200 kernels: status plumbing, the
// peer-mapped memory window used by the halo transport and the short-vector
// all-reduce, and bounded device-side waits.
#pragma once

#include "dcb.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace dcb
{

void set_last_error(const std::string& msg);

#define DCB_CUDA_TRY(expr)                                                     \
    do                                                                         \
    {                                                                          \
        cudaError_t err__ = (expr);                                            \
        if (err__ != cudaSuccess)                                              \
        {                                                                      \
            ::dcb::set_last_error(std::string(#expr) + ": "                    \
                                  + cudaGetErrorString(err__));                \
            return DCB_CUDA_ERROR;                                             \
        }                                                                      \
    } while (0)

#define DCB_LAUNCH_CHECK()                                                     \
    do                                                                         \
    {                                                                          \
        cudaError_t err__ = cudaGetLastError();                                \
        if (err__ != cudaSuccess)                                              \
        {                                                                      \
            ::dcb::set_last_error(std::string("kernel launch: ")               \
                                  + cudaGetErrorString(err__));                \
            return DCB_CUDA_ERROR;                                             \
        }                                                                      \
    } while (0)

#define DCB_REQUIRE(cond, msg)                                                 \
    do                                                                         \
    {                                                                          \
        if (!(cond))                                                           \
        {                                                                      \
            ::dcb::set_last_error(std::string("bad argument: ") + (msg));      \
            return DCB_BAD_ARG;                                                \
        }                                                                      \
    } while (0)

// Row pitch of a shard in elements (0 in the descriptor means dense rows).
inline long long row_pitch(const dcb_tensor_desc& d)
{
    return d.pitch > 0 ? (long long) d.pitch : (long long) d.real_shape[0];
}

inline cudaStream_t as_stream(void* s)
{
    return reinterpret_cast<cudaStream_t>(s);
}

int num_sms();
int64_t wait_budget_ns();

// ---------------------------------------------------------------------------
// A device allocation that other ranks can map.  Ranks living in the same
// process (several emulated ranks on one device in tests, or several devices
// driven by one process) exchange the raw pointer; ranks in other processes
// open the CUDA IPC handle.
// ---------------------------------------------------------------------------
struct WindowBlob
{
    cudaIpcMemHandle_t handle; // 64 bytes
    uint64_t raw_ptr;
    uint64_t bytes;
    int32_t pid;
    int32_t device;
};

struct Window
{
    void* base = nullptr;
    size_t bytes = 0;
    int device = 0;

    int32_t allocate(size_t nbytes);
    int32_t fill_blob(WindowBlob* b) const;
    void release();
};

struct PeerMapping
{
    void* base = nullptr;
    bool opened_ipc = false;
    int32_t open(const WindowBlob& b, int my_device);
    void close();
};

// ---------------------------------------------------------------------------
// Device-side bounded wait on a 32-bit epoch flag written by a peer.
// Returns true when *flag has reached `want`; false when the budget ran out.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Epochs are compared modulo 2^32 so the counter may wrap.
__device__ __forceinline__ bool epoch_reached(uint32_t have, uint32_t want)
{
    return (int32_t) (have - want) >= 0;
}

__device__ __forceinline__ bool bounded_wait_epoch(const uint32_t* flag,
                                                   uint32_t want,
                                                   int64_t budget_ns)
{
    if (epoch_reached(ld_acquire_sys(flag), want))
        return true;
    const uint64_t t0 = globaltimer_ns();
    // Two limits: wall time on the device and a hard iteration cap, so the
    // loop ends even if the timer misbehaves.
    for (uint64_t it = 0; it < (1ull << 34); ++it)
    {
        if (epoch_reached(ld_acquire_sys(flag), want))
            return true;
        if ((it & 63) == 63
            && (int64_t) (globaltimer_ns() - t0) > budget_ns)
            return false;
        __nanosleep(64);
    }
    return false;
}

// Collapsed view of an NC[D]HW tensor window: every (n, c) plane is `rows`
// contiguous runs of `len` elements.  Level 2 = the whole plane is one run,
// level 1 = one run per D slice, level 0 = one run per (D, H) row.
struct RunGeom
{
    long long n, c;
    long long rows;       // runs per (n, c) plane
    long long rows_inner; // runs per outer step
    long long len;        // contiguous elements per run
};

struct RunStrides
{
    long long sn, sc;
    long long s_inner; // between consecutive runs inside an outer step
    long long s_outer; // between outer steps
};

// Deepest collapse level the strides of d allow; -1 if W is not unit-stride.
inline int run_level(const dcb_nd_desc& d)
{
    const long long H = d.dims[1], W = d.dims[2];
    if (d.strides[2] != 1 && W > 1)
        return -1;
    if (d.strides[1] != W && H > 1)
        return 0;
    if (d.strides[0] != H * W && d.dims[0] > 1)
        return 1;
    return 2;
}

inline void make_runs(const dcb_nd_desc& d, int level, RunGeom* g,
                      RunStrides* s)
{
    const long long D = d.dims[0], H = d.dims[1], W = d.dims[2];
    g->n = d.n;
    g->c = d.c;
    s->sn = d.sn;
    s->sc = d.sc;
    if (level == 2)
    {
        g->len = D * H * W;
        g->rows = 1;
        g->rows_inner = 1;
        s->s_inner = 0;
        s->s_outer = 0;
    }
    else if (level == 1)
    {
        g->len = H * W;
        g->rows = D;
        g->rows_inner = D;
        s->s_inner = d.strides[0];
        s->s_outer = 0;
    }
    else
    {
        g->len = W;
        g->rows = D * H;
        g->rows_inner = H;
        s->s_inner = d.strides[1];
        s->s_outer = d.strides[0];
    }
}

inline bool same_extents(const dcb_nd_desc& a, const dcb_nd_desc& b)
{
    return a.nsd == b.nsd && a.n == b.n && a.c == b.c && a.dims[0] == b.dims[0]
           && a.dims[1] == b.dims[1] && a.dims[2] == b.dims[2];
}

// Largest vector width (4, 2, 1 floats) that every run start of a tensor with
// these strides honours.
inline int run_vec(const RunGeom& g, const RunStrides& s, const void* p)
{
    auto ok = [&](long long v) {
        return g.len % v == 0 && s.sn % v == 0 && s.sc % v == 0
               && s.s_inner % v == 0 && s.s_outer % v == 0
               && reinterpret_cast<uintptr_t>(p) % (4 * v) == 0;
    };
    return ok(4) ? 4 : (ok(2) ? 2 : 1);
}

inline int32_t check_nd_desc(const dcb_nd_desc* d)
{
    DCB_REQUIRE(d != nullptr, "null descriptor");
    DCB_REQUIRE(d->nsd == 2 || d->nsd == 3, "nsd must be 2 or 3");
    DCB_REQUIRE(d->n >= 0 && d->c >= 0, "negative extent");
    for (int i = 0; i < 3; ++i)
        DCB_REQUIRE(d->dims[i] >= 0, "negative extent");
    if (d->nsd == 2)
        DCB_REQUIRE(d->dims[0] == 1, "dims[0] must be 1 for 2-D tensors");
    return DCB_OK;
}

} // namespace dcb
