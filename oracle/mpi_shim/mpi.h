/*
 * TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
 *
 * A small in-process stand-in for the subset of the MPI C interface that the
 * reference's header-only CPU path uses (tensor construction, sub-communicator
 * splits, Allgather of local extents, Allreduce of filter gradients,
 * Send/Recv).  "Ranks" are threads of one process: each thread registers its
 * world rank with shim_mpi_set_rank() before making any MPI call.  Written
 * from the MPI standard's function signatures; no MPI implementation's code
 * was consulted.  Everything lives in this header (inline / static storage via
 * function-local statics) so the reference headers can simply `#include
 * "mpi.h"`.
 */
#ifndef ORACLE_MPI_SHIM_H_
#define ORACLE_MPI_SHIM_H_

#include <algorithm>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <tuple>
#include <vector>

typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Info;
typedef int MPI_Win;
typedef long MPI_Aint;
struct MPI_Status
{
    int MPI_SOURCE, MPI_TAG, MPI_ERROR;
};

enum
{
    MPI_SUCCESS = 0
};
enum
{
    MPI_CHAR = 1,
    MPI_UNSIGNED_CHAR,
    MPI_BYTE,
    MPI_SHORT,
    MPI_UNSIGNED_SHORT,
    MPI_INT,
    MPI_UNSIGNED,
    MPI_LONG,
    MPI_UNSIGNED_LONG,
    MPI_FLOAT,
    MPI_DOUBLE
};
enum
{
    MPI_SUM = 1,
    MPI_MAX,
    MPI_MIN
};
enum
{
    MPI_PROC_NULL = -2,
    MPI_ANY_SOURCE = -1,
    MPI_ANY_TAG = -1
};
enum
{
    MPI_INFO_NULL = 0,
    MPI_COMM_TYPE_SHARED = 1
};
#define MPI_IN_PLACE ((void*) 1)
#define MPI_STATUS_IGNORE ((MPI_Status*) 0)

namespace shim_mpi
{

struct Comm
{
    std::vector<int> members; // world ranks, in comm-rank order
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0;
    long generation = 0;
    std::vector<const void*> slots;  // per comm-rank scratch pointer
    std::vector<long> ints;          // per comm-rank scratch ints (3 each)
    std::vector<Comm*> split_result; // per comm-rank result of a split
    // point-to-point mailboxes keyed (src, dst, tag)
    std::map<std::tuple<int, int, int>, std::deque<std::vector<char>>> mail;
};

inline int& tl_rank()
{
    static thread_local int r = 0;
    return r;
}
inline int& world_size()
{
    static int n = 1;
    return n;
}
inline Comm*& world()
{
    static Comm* w = nullptr;
    return w;
}

inline size_t type_size(MPI_Datatype t)
{
    switch (t)
    {
    case MPI_CHAR:
    case MPI_UNSIGNED_CHAR:
    case MPI_BYTE: return 1;
    case MPI_SHORT:
    case MPI_UNSIGNED_SHORT: return 2;
    case MPI_INT:
    case MPI_UNSIGNED:
    case MPI_FLOAT: return 4;
    default: return 8;
    }
}

inline int comm_rank_of(Comm* c, int world_rank)
{
    for (size_t i = 0; i < c->members.size(); ++i)
        if (c->members[i] == world_rank)
            return (int) i;
    std::fprintf(stderr, "shim_mpi: rank %d not in communicator\n", world_rank);
    std::abort();
}

// Central sense-reversing barrier over the members of c.
inline void barrier(Comm* c)
{
    std::unique_lock<std::mutex> lk(c->mu);
    long gen = c->generation;
    if (++c->arrived == (int) c->members.size())
    {
        c->arrived = 0;
        ++c->generation;
        c->cv.notify_all();
    }
    else
    {
        c->cv.wait(lk, [&] { return c->generation != gen; });
    }
}

template <typename T>
inline void reduce_into(T* dst, const T* src, int n, MPI_Op op)
{
    for (int i = 0; i < n; ++i)
    {
        if (op == MPI_SUM)
            dst[i] += src[i];
        else if (op == MPI_MAX)
            dst[i] = std::max(dst[i], src[i]);
        else
            dst[i] = std::min(dst[i], src[i]);
    }
}

} // namespace shim_mpi

typedef shim_mpi::Comm* MPI_Comm;
#define MPI_COMM_WORLD (shim_mpi::world())
#define MPI_COMM_NULL ((MPI_Comm) 0)

// ---- shim control (called by the driver, not by the reference headers) ----
inline void shim_mpi_init_world(int nranks)
{
    auto* w = new shim_mpi::Comm;
    for (int i = 0; i < nranks; ++i)
        w->members.push_back(i);
    w->slots.resize(nranks);
    w->ints.resize(3 * nranks);
    w->split_result.resize(nranks);
    shim_mpi::world() = w;
    shim_mpi::world_size() = nranks;
}
inline void shim_mpi_set_rank(int r)
{
    shim_mpi::tl_rank() = r;
}

// ---- the MPI subset ----
inline int MPI_Comm_rank(MPI_Comm c, int* r)
{
    *r = shim_mpi::comm_rank_of(c, shim_mpi::tl_rank());
    return MPI_SUCCESS;
}
inline int MPI_Comm_size(MPI_Comm c, int* n)
{
    *n = (int) c->members.size();
    return MPI_SUCCESS;
}
inline int MPI_Barrier(MPI_Comm c)
{
    shim_mpi::barrier(c);
    return MPI_SUCCESS;
}
inline int MPI_Abort(MPI_Comm, int code)
{
    std::fprintf(stderr, "shim_mpi: MPI_Abort(%d)\n", code);
    std::abort();
}

inline int MPI_Comm_split(MPI_Comm c, int color, int key, MPI_Comm* out)
{
    using namespace shim_mpi;
    const int me = comm_rank_of(c, tl_rank());
    const int n = (int) c->members.size();
    c->ints[3 * me + 0] = color;
    c->ints[3 * me + 1] = key;
    c->ints[3 * me + 2] = tl_rank();
    barrier(c);
    // The lowest comm-rank of each colour builds the new communicator.
    bool leader = true;
    for (int i = 0; i < me; ++i)
        if (c->ints[3 * i] == color)
            leader = false;
    if (leader)
    {
        std::vector<std::tuple<long, int, long>> m; // key, old rank, world
        for (int i = 0; i < n; ++i)
            if (c->ints[3 * i] == color)
                m.emplace_back(c->ints[3 * i + 1], i, c->ints[3 * i + 2]);
        std::sort(m.begin(), m.end());
        auto* nc = new Comm;
        for (auto& t : m)
            nc->members.push_back((int) std::get<2>(t));
        const int k = (int) nc->members.size();
        nc->slots.resize(k);
        nc->ints.resize(3 * k);
        nc->split_result.resize(k);
        for (auto& t : m)
            c->split_result[std::get<1>(t)] = nc;
    }
    barrier(c);
    *out = c->split_result[me];
    barrier(c);
    return MPI_SUCCESS;
}
inline int MPI_Comm_dup(MPI_Comm c, MPI_Comm* out)
{
    int r;
    MPI_Comm_rank(c, &r);
    return MPI_Comm_split(c, 0, r, out);
}
inline int MPI_Comm_split_type(MPI_Comm c, int, int key, MPI_Info, MPI_Comm* o)
{
    return MPI_Comm_split(c, 0, key, o);
}
inline int MPI_Comm_free(MPI_Comm* c)
{
    // Communicators are leaked on purpose: the driver is short-lived and
    // member threads may free at different times.
    *c = MPI_COMM_NULL;
    return MPI_SUCCESS;
}

inline int MPI_Allgather(const void* sbuf, int scount, MPI_Datatype st,
                         void* rbuf, int rcount, MPI_Datatype rt, MPI_Comm c)
{
    using namespace shim_mpi;
    const int me = comm_rank_of(c, tl_rank());
    const size_t sbytes = (size_t) scount * type_size(st);
    const size_t rbytes = (size_t) rcount * type_size(rt);
    std::vector<char> mine;
    if (sbuf == MPI_IN_PLACE)
    {
        mine.assign((char*) rbuf + me * rbytes,
                    (char*) rbuf + (me + 1) * rbytes);
    }
    else
    {
        mine.assign((const char*) sbuf, (const char*) sbuf + sbytes);
    }
    c->slots[me] = mine.data();
    barrier(c);
    for (size_t i = 0; i < c->members.size(); ++i)
        std::memcpy((char*) rbuf + i * rbytes, c->slots[i], rbytes);
    barrier(c);
    return MPI_SUCCESS;
}

inline int MPI_Allreduce(const void* sbuf, void* rbuf, int count,
                         MPI_Datatype t, MPI_Op op, MPI_Comm c)
{
    using namespace shim_mpi;
    const int me = comm_rank_of(c, tl_rank());
    const size_t bytes = (size_t) count * type_size(t);
    std::vector<char> mine;
    const void* src = (sbuf == MPI_IN_PLACE) ? rbuf : sbuf;
    mine.assign((const char*) src, (const char*) src + bytes);
    c->slots[me] = mine.data();
    barrier(c);
    // Every rank reduces in comm-rank order, so all ranks get identical bits.
    std::vector<char> acc((const char*) c->slots[0],
                          (const char*) c->slots[0] + bytes);
    for (size_t i = 1; i < c->members.size(); ++i)
    {
        switch (t)
        {
        case MPI_FLOAT:
            reduce_into((float*) acc.data(), (const float*) c->slots[i], count,
                        op);
            break;
        case MPI_DOUBLE:
            reduce_into((double*) acc.data(), (const double*) c->slots[i],
                        count, op);
            break;
        case MPI_INT:
            reduce_into((int*) acc.data(), (const int*) c->slots[i], count, op);
            break;
        case MPI_LONG:
            reduce_into((long*) acc.data(), (const long*) c->slots[i], count,
                        op);
            break;
        case MPI_UNSIGNED_LONG:
            reduce_into((unsigned long*) acc.data(),
                        (const unsigned long*) c->slots[i], count, op);
            break;
        default:
            std::fprintf(stderr, "shim_mpi: Allreduce type %d unsupported\n", t);
            std::abort();
        }
    }
    barrier(c);
    std::memcpy(rbuf, acc.data(), bytes);
    return MPI_SUCCESS;
}

inline int MPI_Send(const void* buf, int count, MPI_Datatype t, int dst,
                    int tag, MPI_Comm c)
{
    using namespace shim_mpi;
    if (dst == MPI_PROC_NULL)
        return MPI_SUCCESS;
    const int me = comm_rank_of(c, tl_rank());
    const size_t bytes = (size_t) count * type_size(t);
    {
        std::lock_guard<std::mutex> lk(c->mu);
        c->mail[std::make_tuple(me, dst, tag)].emplace_back(
            (const char*) buf, (const char*) buf + bytes);
    }
    c->cv.notify_all();
    return MPI_SUCCESS;
}
inline int MPI_Recv(void* buf, int count, MPI_Datatype t, int src, int tag,
                    MPI_Comm c, MPI_Status*)
{
    using namespace shim_mpi;
    if (src == MPI_PROC_NULL)
        return MPI_SUCCESS;
    const int me = comm_rank_of(c, tl_rank());
    const size_t bytes = (size_t) count * type_size(t);
    std::unique_lock<std::mutex> lk(c->mu);
    auto key = std::make_tuple(src, me, tag);
    c->cv.wait(lk, [&] {
        auto it = c->mail.find(key);
        return it != c->mail.end() && !it->second.empty();
    });
    auto& q = c->mail[key];
    std::memcpy(buf, q.front().data(), std::min(bytes, q.front().size()));
    q.pop_front();
    return MPI_SUCCESS;
}

// One-sided calls appear in tensor-copy helpers that the conv path never
// reaches; they only need to compile.
inline int MPI_Win_create(void*, MPI_Aint, int, MPI_Info, MPI_Comm, MPI_Win*)
{
    std::fprintf(stderr, "shim_mpi: one-sided MPI is not provided\n");
    std::abort();
}
inline int MPI_Win_fence(int, MPI_Win)
{
    std::abort();
}
inline int MPI_Win_free(MPI_Win*)
{
    std::abort();
}
inline int MPI_Put(const void*, int, MPI_Datatype, int, MPI_Aint, int,
                   MPI_Datatype, MPI_Win)
{
    std::abort();
}

#endif // ORACLE_MPI_SHIM_H_
