// distconv_b200.hpp -- header-only C++ host side of the B200 DistConv path.
//
// Keeps DistConv's namespaces, class names, method names and argument order
// for the spatially-parallel conv + batch-norm path and forwards every device
// operation to the C ABI of libdistconv_b200 (dcb.h).  Reference interfaces
// (paths relative to the DiHydrogen tree):
//   tensor::Shape / IntVector / IndexVector   legacy/include/distconv/tensor/tensor_base.hpp, vector.hpp
//   tensor::Distribution                      legacy/include/distconv/tensor/distribution.hpp:14-270
//   tensor::LocaleMPI                         legacy/include/distconv/tensor/tensor_mpi.hpp:18-93
//   tensor::Tensor<T, LocaleMPI, CUDAAllocator>  tensor.hpp:38-653, tensor_mpi.hpp:98-574
//   internal::get_halo_sizes, create_*_tensor legacy/include/distconv/distconv.hpp:21-99, 253-515
//   tensor::HaloExchange                      halo_exchange_cuda.hpp:18-423
//   BackendDNNLib                             dnn_backend/dnn_backend.hpp:635-980
//   Convolution<BackendDNNLib, T>             dnn_backend/convolution.hpp:19-3003
//   BatchNormalization<BackendDNNLib, T>      dnn_backend/batchnorm.hpp:100-581
//
// Dimension order is DistConv's: index 0 is W, then H, [D], C, N; negative
// indices count from the end (-2 is C, -1 is N).  Only float tensors and
// spatial parallelism (no channel/filter parallelism) are provided.
//
// The header needs cuda_runtime_api.h for device memory; it needs no mpi.h:
// LocaleMPI takes the rank, the size and an allgather callback.
#pragma once

#include "dcb.h"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <array>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#if defined(DISTCONV_B200_HAS_MPI)
#include <mpi.h>
#endif
#if defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>) && !defined(DISTCONV_B200_NO_NVTX)
#include <nvtx3/nvToolsExt.h>
#endif
#endif

namespace distconv
{

using index_t = int64_t;
using int_vector = std::vector<int>;

// ---- vocabulary of legacy/include/distconv/base.hpp:23-394 ------------------
enum Side
{
    LHS = 0,
    RHS = 1
};
const Side SIDES[2] = {LHS, RHS};

inline Side operator~(const Side& s)
{
    return static_cast<Side>((~static_cast<int>(s)) & 1);
}
inline std::ostream& operator<<(std::ostream& os, const Side& s)
{
    return os << (s == LHS ? "LHS" : "RHS");
}

template <int ND, typename F>
void apply_to_sides(F&& f)
{
    for (int i = 0; i < ND; ++i)
        for (Side side : SIDES)
            f(i, side);
}
template <typename F>
void apply_to_sides(int num_dims, F&& f)
{
    for (int i = 0; i < num_dims; ++i)
        for (Side side : SIDES)
            f(i, side);
}
template <typename F>
void apply_to_spatial_sides(int num_dims, F&& f)
{
    for (int i = 0; i < num_dims - 2; ++i)
        for (Side side : SIDES)
            f(i, side);
}
template <int ND, typename F>
void apply_to_spatial_sides(F&& f)
{
    for (int i = 0; i < ND - 2; ++i)
        for (Side side : SIDES)
            f(i, side);
}

// one attribute per side of a boundary (base.hpp:58-79)
template <typename T>
struct BoundaryAttributes
{
    std::array<T, 2> m_attrs;
    BoundaryAttributes() = default;
    BoundaryAttributes(const T& v) : BoundaryAttributes(v, v) {}
    BoundaryAttributes(const T& lhs, const T& rhs) : m_attrs({lhs, rhs}) {}
    T& operator()(Side s) { return m_attrs[s]; }
    const T& operator()(Side s) const { return m_attrs[s]; }
    T* data() { return m_attrs.data(); }
    const T* data() const { return m_attrs.data(); }
};

// per dimension and side, growing on demand (base.hpp:125-173)
template <typename T>
class BoundaryAttributesV
{
public:
    BoundaryAttributesV() = default;
    BoundaryAttributesV(const T& lhs, const T& rhs) : m_default(lhs, rhs) {}
    BoundaryAttributesV(const T& attr) : BoundaryAttributesV(attr, attr) {}
    T& operator()(int d, Side s)
    {
        expand_if_needed(d);
        return m_attrs.at(d)(s);
    }
    const T& operator()(int d, Side s) const { return m_attrs.at(d)(s); }
    T* operator()(int d)
    {
        expand_if_needed(d);
        return m_attrs.at(d).data();
    }
    const T* operator()(int d) const { return m_attrs.at(d).data(); }
    void clear() { m_attrs.clear(); }

private:
    void expand_if_needed(int d)
    {
        if (d >= (int) m_attrs.size())
            m_attrs.resize(d + 1, m_default);
    }
    BoundaryAttributes<T> m_default;
    std::vector<BoundaryAttributes<T>> m_attrs;
};

// Every method maps to the one peer-store transport (base.hpp:175-240).
enum class HaloExchangeMethod
{
    MPI,
    AL,
    P2P,
    HYBRID
};
inline std::ostream& operator<<(std::ostream& os, const HaloExchangeMethod& m)
{
    static const char* names[] = {"MPI", "AL", "P2P", "HYBRID"};
    return os << names[(int) m];
}
// Unknown names are a programmer error: the reference aborts, this throws.
inline HaloExchangeMethod GetHaloExchangeMethod(const std::string& method)
{
    if (method == "MPI")
        return HaloExchangeMethod::MPI;
    if (method == "AL")
        return HaloExchangeMethod::AL;
    if (method == "P2P")
        return HaloExchangeMethod::P2P;
    if (method == "HYBRID")
        return HaloExchangeMethod::HYBRID;
    throw std::invalid_argument("Unknown method name for halo exchange: " + method);
}

enum class ShuffleMethod
{
    MPI,
    AL,
    P2P,
    HYBRID
};
inline std::ostream& operator<<(std::ostream& os, const ShuffleMethod& m)
{
    static const char* names[] = {"MPI", "AL", "P2P", "HYBRID"};
    return os << names[(int) m];
}
inline ShuffleMethod GetShuffleMethod(const std::string& method)
{
    if (method == "MPI")
        return ShuffleMethod::MPI;
    if (method == "AL")
        return ShuffleMethod::AL;
    if (method == "P2P")
        return ShuffleMethod::P2P;
    if (method == "HYBRID")
        return ShuffleMethod::HYBRID;
    throw std::invalid_argument("Unknown shuffle method: " + method);
}

// Only NONE / AUTO (= none) are provided: spatial parallelism is the path.
enum class ChannelParallelismAlgorithm
{
    NONE,
    AUTO,
    X,
    Y,
    W
};
inline std::ostream& operator<<(std::ostream& os, const ChannelParallelismAlgorithm& a)
{
    static const char* names[] = {"NONE", "AUTO", "X", "Y", "W"};
    return os << names[(int) a];
}

// MPI and AL_NCCL are the reference's names (base.hpp:308-366); both run the
// peer-memory all-reduce kernel here, which PEER names directly.
enum class BatchnormImpl
{
    MPI,
    AL_NCCL,
    PEER
};
inline std::ostream& operator<<(std::ostream& os, const BatchnormImpl& v)
{
    static const char* names[] = {"MPI", "AL_NCCL", "PEER"};
    return os << names[(int) v];
}
inline BatchnormImpl GetBatchnormImpl(const std::string& impl)
{
    if (impl == "MPI")
        return BatchnormImpl::MPI;
    if (impl == "AL_NCCL")
        return BatchnormImpl::AL_NCCL;
    if (impl == "PEER")
        return BatchnormImpl::PEER;
    throw std::invalid_argument("Unknown implementation name for batchnorm: " + impl);
}

namespace util
{
// Rank used as the prefix of the MPI print streams.  LocaleMPI sets it; before
// that it comes from the launcher's environment.
inline int& process_rank()
{
    static int rank = [] {
        for (const char* name : {"RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID"})
            if (const char* v = std::getenv(name))
                return std::atoi(v);
        return 0;
    }();
    return rank;
}

// The reference's print streams (legacy/include/distconv/util/util.hpp:142-265,
// util_mpi.hpp): a line is assembled by operator<< and written with a newline
// when the temporary dies.  Debug streams print only when DISTCONV_DEBUG is set;
// MPI streams prefix the rank; MPIRoot streams print on rank 0 only.
class PrintStream
{
public:
    PrintStream(std::ostream& os, bool enabled, const std::string& prefix = "") : m_os(os), m_enabled(enabled)
    {
        if (m_enabled)
            m_line << prefix;
    }
    PrintStream(const PrintStream&) = delete;
    ~PrintStream()
    {
        if (m_enabled)
            m_os << m_line.str() << std::endl;
    }
    template <typename T>
    PrintStream& operator<<(const T& v)
    {
        if (m_enabled)
            m_line << v;
        return *this;
    }

private:
    std::ostream& m_os;
    bool m_enabled;
    std::ostringstream m_line;
};
inline bool debug_enabled()
{
    static const bool on = std::getenv("DISTCONV_DEBUG") != nullptr;
    return on;
}
inline std::string rank_prefix()
{
    return "[" + std::to_string(process_rank()) + "] ";
}
struct PrintStreamDebug : PrintStream
{
    PrintStreamDebug() : PrintStream(std::cerr, debug_enabled()) {}
};
struct PrintStreamInfo : PrintStream
{
    PrintStreamInfo() : PrintStream(std::cout, true) {}
};
struct PrintStreamWarning : PrintStream
{
    PrintStreamWarning() : PrintStream(std::cerr, true, "Warning: ") {}
};
struct PrintStreamError : PrintStream
{
    PrintStreamError() : PrintStream(std::cerr, true, "Error: ") {}
};
struct MPIPrintStreamDebug : PrintStream
{
    MPIPrintStreamDebug() : PrintStream(std::cerr, debug_enabled(), rank_prefix()) {}
};
struct MPIPrintStreamInfo : PrintStream
{
    MPIPrintStreamInfo() : PrintStream(std::cout, true, rank_prefix()) {}
};
struct MPIPrintStreamWarning : PrintStream
{
    MPIPrintStreamWarning() : PrintStream(std::cerr, true, rank_prefix() + "Warning: ") {}
};
struct MPIPrintStreamError : PrintStream
{
    MPIPrintStreamError() : PrintStream(std::cerr, true, rank_prefix() + "Error: ") {}
};
struct MPIRootPrintStreamDebug : PrintStream
{
    MPIRootPrintStreamDebug() : PrintStream(std::cerr, debug_enabled() && process_rank() == 0) {}
};
struct MPIRootPrintStreamInfo : PrintStream
{
    MPIRootPrintStreamInfo() : PrintStream(std::cout, process_rank() == 0) {}
};

// Profiler ranges (GPU_PROFILE_RANGE_PUSH / _POP of the reference, which are
// NVTX ranges): named like the reference's ("conv/forward",
// "conv/forward/exchange_halo", ...).  NVTX's header-only C API is used when
// the toolkit ships it; otherwise the ranges are no-ops.
#if defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>) && !defined(DISTCONV_B200_NO_NVTX)
#define DISTCONV_B200_HAS_NVTX 1
#endif
#endif
inline void profile_range_push(const char* name);
inline void profile_range_pop();

inline void check(int32_t st, const char* what)
{
    if (st != DCB_OK)
        throw std::runtime_error(std::string(what) + ": " + dcb_status_string(st) + " (" + dcb_last_error() + ")");
}
// the reference's assert_always: a programmer error
inline void require(bool cond, const char* what)
{
    if (!cond)
        throw std::invalid_argument(what);
}
inline void profile_range_push(const char* name)
{
#ifdef DISTCONV_B200_HAS_NVTX
    nvtxRangePushA(name);
#else
    (void) name;
#endif
}
inline void profile_range_pop()
{
#ifdef DISTCONV_B200_HAS_NVTX
    nvtxRangePop();
#endif
}
} // namespace util

// backend::Options (legacy/include/distconv/dnn_backend/dnn_backend.hpp:46-63)
// with the environment overrides of legacy/src/dnn_backend/options.cpp:13-71: a
// variable that is SET (to anything, "0" included, as in the reference) turns
// its option on.  The workspace factor and the JIT fields are carried for
// source compatibility; plans own their workspaces and nothing is compiled at
// run time.  math_mode has no counterpart: DCB_MATH_FP32 (3xTF32 on tensor
// cores, fp32 quality), DCB_MATH_TF32, DCB_MATH_BF16 (bf16 operands, fp32
// accumulation) or DCB_MATH_FP32_SIMT.
struct Options
{
    bool overlap_halo_exchange;
    bool m_deterministic;
    bool enable_profiling;
    float ws_capacity_factor;
    bool jit_verbose;
    std::string jit_cache_path;
    int math_mode = DCB_MATH_FP32;

    Options(bool overlap_halo_exchange_in = false, bool deterministic_in = false, bool enable_profiling_in = false,
            float ws_capacity_factor_in = 1.0f, bool jit_verbose_in = false,
            const std::string& jit_cache_path_in = ".jitcache")
        : overlap_halo_exchange(overlap_halo_exchange_in), m_deterministic(deterministic_in),
          enable_profiling(enable_profiling_in), ws_capacity_factor(ws_capacity_factor_in),
          jit_verbose(jit_verbose_in), jit_cache_path(jit_cache_path_in)
    {
        auto detected = [](const char* name) {
            if (!std::getenv(name))
                return false;
            util::MPIRootPrintStreamDebug() << "Environment variable: " << name << " detected";
            return true;
        };
        if (detected("DISTCONV_OVERLAP_HALO_EXCHANGE"))
            overlap_halo_exchange = true;
        if (detected("DISTCONV_DETERMINISTIC"))
            m_deterministic = true;
        // DISTCONV_PROFILING / DISTCONV_NVTX are the runtime's switches (legacy/src/runtime.cpp:13-21)
        if (detected("DISTCONV_ENABLE_PROFILING") || detected("DISTCONV_PROFILING") || detected("DISTCONV_NVTX"))
            enable_profiling = true;
        if (detected("DISTCONV_WS_CAPACITY_FACTOR"))
            ws_capacity_factor = (float) std::atof(std::getenv("DISTCONV_WS_CAPACITY_FACTOR"));
        if (detected("DISTCONV_JIT_VERBOSE"))
            jit_verbose = true;
        if (detected("DISTCONV_JIT_CACHEPATH"))
            jit_cache_path = std::getenv("DISTCONV_JIT_CACHEPATH");
    }
};
namespace backend
{
using Options = ::distconv::Options;
}

namespace tensor
{

// Vector with DistConv's negative indexing.
template <typename T>
class Vector : public std::vector<T>
{
public:
    using std::vector<T>::vector;
    Vector() = default;
    Vector(const std::vector<T>& v) : std::vector<T>(v) {}
    T& operator[](int i) { return std::vector<T>::operator[](i < 0 ? (int) this->size() + i : i); }
    const T& operator[](int i) const { return std::vector<T>::operator[](i < 0 ? (int) this->size() + i : i); }
    int num_dims() const { return (int) this->size(); }
    T get_size() const
    {
        T p = 1;
        for (auto v : *this)
            p *= v;
        return p;
    }
};

using Shape = Vector<index_t>;
using IndexVector = Vector<index_t>;
using IntVector = Vector<int>;

class Distribution
{
public:
    Distribution() = default;
    Distribution(const Shape& locale_shape, const Shape& split_shape, const IntVector& overlap)
        : m_locale_shape(locale_shape), m_split_shape(split_shape), m_overlap(overlap)
    {
        fixup_overlap();
    }
    static Distribution make_localized_distribution(int nd)
    {
        return Distribution(Shape(nd, 1), Shape(nd, 1), IntVector(nd, 0));
    }
    static Distribution make_distribution(const Shape& ls) { return Distribution(ls, ls, IntVector(ls.size(), 0)); }
    static Distribution make_shared_distribution(const Shape& ls)
    {
        return Distribution(ls, Shape(ls.size(), 1), IntVector(ls.size(), 0));
    }
    static Distribution make_overlapped_distribution(const Shape& ls, const IntVector& overlap)
    {
        return Distribution(ls, ls, overlap);
    }
    int num_dims() const { return m_locale_shape.num_dims(); }
    const Shape& get_locale_shape() const { return m_locale_shape; }
    const Shape& get_split_shape() const { return m_split_shape; }
    const IntVector& get_overlap() const { return m_overlap; }
    int get_overlap(int dim) const { return m_overlap[dim]; }
    index_t get_num_ranks_per_split(int dim) const { return m_locale_shape[dim] / m_split_shape[dim]; }
    bool is_distributed(int dim) const { return m_split_shape[dim] > 1; }
    void set_overlap(const IntVector& o) { m_overlap = o; }
    void clear_overlap() { m_overlap = IntVector(num_dims(), 0); }
    void fixup_overlap()
    {
        for (int i = 0; i < num_dims(); ++i)
            if (!is_distributed(i))
                m_overlap[i] = 0;
    }

private:
    Shape m_locale_shape, m_split_shape;
    IntVector m_overlap;
};

// A rank of a group.  allgather(in, out, n): every rank contributes n bytes,
// out receives size * n bytes in rank order (MPI_Allgather with MPI_BYTE).
class LocaleMPI
{
public:
    using Allgather = std::function<void(const void*, void*, size_t)>;
    LocaleMPI(int rank = 0, int size = 1, Allgather ag = nullptr) : m_rank(rank), m_size(size), m_ag(std::move(ag))
    {
        util::process_rank() = rank;
    }
#if defined(DISTCONV_B200_HAS_MPI)
    // The reference's constructor (tensor_mpi.hpp:18-36): rank and size of the
    // communicator, blobs gathered with MPI_Allgather.  Compiled when the host
    // defines DISTCONV_B200_HAS_MPI (and so provides <mpi.h>).
    LocaleMPI(MPI_Comm comm, bool /*copy_comm*/ = true) : m_comm(comm)
    {
        MPI_Comm_rank(comm, &m_rank);
        MPI_Comm_size(comm, &m_size);
        util::process_rank() = m_rank;
        m_ag = [comm](const void* in, void* out, size_t n) {
            MPI_Allgather(const_cast<void*>(in), (int) n, MPI_BYTE, out, (int) n, MPI_BYTE, comm);
        };
    }
    MPI_Comm get_comm() const { return m_comm; }
#endif
    int get_rank() const { return m_rank; }
    int get_size() const { return m_size; }
    IndexVector get_rank_idx(const Distribution& dist) const
    {
        IndexVector idx(dist.num_dims(), 0);
        int r = m_rank;
        for (int i = 0; i < dist.num_dims(); ++i)
        {
            idx[i] = r % dist.get_locale_shape()[i];
            r /= (int) dist.get_locale_shape()[i];
        }
        return idx;
    }
    void allgather(const void* in, void* out, size_t n) const
    {
        if (m_size == 1)
        {
            std::memcpy(out, in, n);
            return;
        }
        if (!m_ag)
            throw std::runtime_error("LocaleMPI: no allgather callback for a multi-rank locale");
        m_ag(in, out, n);
    }

private:
    int m_rank = 0, m_size = 1;
    Allgather m_ag;
#if defined(DISTCONV_B200_HAS_MPI)
    MPI_Comm m_comm = MPI_COMM_NULL;
#endif
};

// A single-process locale (tensor_process.hpp): rank 0 of 1.
class LocaleProcess
{
public:
    int get_rank() const { return 0; }
    int get_size() const { return 1; }
    IndexVector get_rank_idx(const Distribution& dist) const { return IndexVector(dist.num_dims(), 0); }
    void allgather(const void* in, void* out, size_t n) const { std::memcpy(out, in, n); }
};

// Allocator tags (tensor/memory_cuda.hpp:28-104).  They decide the row layout of
// a shard.  CUDAAllocator keeps rows dense unless the shard carries halo cells
// along W: such rows (local + 2 * overlap floats) are padded to 16 bytes, which
// the bulk-copy fed tensor-core kernels need, and the buffer starts `lead` floats
// above a 16-byte boundary so that the OWNED cells of every row start on one
// (bulk stores and vector accesses into a shard's interior need that; readers of
// the halo-extended window fetch from the boundary below it).  At most six
// floats per row.  CUDAPitchedAllocator pads the rows of every shard to 128
// bytes, as cudaMallocPitch-style allocation does in the reference.
struct CUDAAllocator
{
    static index_t lead(index_t overlap) { return (4 - overlap % 4) % 4; }
    static index_t pitch(index_t row, index_t overlap)
    {
        return overlap > 0 ? (lead(overlap) + row + 3) / 4 * 4 : row;
    }
};
struct CUDAPitchedAllocator
{
    static index_t lead(index_t overlap) { return (4 - overlap % 4) % 4; }
    static index_t pitch(index_t row, index_t overlap) { return (lead(overlap) + row + 31) / 32 * 32; }
};
// Host memory (tensor/memory.hpp:25-55); used by the host-side gather of dump_tensor.
struct BaseAllocator
{
    static index_t lead(index_t) { return 0; }
    static index_t pitch(index_t row, index_t) { return row; }
};

// Owned or aliased buffer with an allocator's deleter (tensor/memory.hpp:57-300):
// the shared_ptr frees device (or, for BaseAllocator, host) memory when the last
// owner goes; an alias never frees.
template <typename Allocator>
class Memory
{
public:
    using allocator_type = Allocator;
    Memory() = default;
    // lead_bytes: the buffer (get()) starts this far into the allocation, which is
    // bytes + lead_bytes long, so that get() + bytes stays inside it
    int allocate(size_t bytes, size_t pitch_bytes = 0, size_t ldim_bytes = 0, size_t lead_bytes = 0)
    {
        void* p = nullptr;
        const size_t total = bytes + lead_bytes;
        if (std::is_same<Allocator, BaseAllocator>::value)
        {
            p = std::malloc(total ? total : 16);
            if (!p)
                return -1;
            m_managed = std::shared_ptr<void>(p, [](void* q) { std::free(q); });
        }
        else
        {
            if (cudaMalloc(&p, total ? total : 16) != cudaSuccess)
                return -1;
            m_managed = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
        }
        m_alias = nullptr;
        m_bytes = bytes;
        m_pitch = pitch_bytes;
        m_ldim = ldim_bytes;
        m_lead = lead_bytes;
        return 0;
    }
    void alias(void* raw, size_t bytes, size_t pitch_bytes, size_t ldim_bytes)
    {
        m_managed.reset();
        m_alias = raw;
        m_bytes = bytes;
        m_pitch = pitch_bytes;
        m_ldim = ldim_bytes;
        m_lead = 0;
    }
    void alias(const Memory& parent)
    {
        m_managed.reset();
        m_alias = parent.get();
        m_bytes = parent.m_bytes;
        m_pitch = parent.m_pitch;
        m_ldim = parent.m_ldim;
        m_lead = 0;
    }
    void nullify()
    {
        m_managed.reset();
        m_alias = nullptr;
        m_bytes = 0;
    }
    void* get() const
    {
        if (m_alias)
            return m_alias;
        return m_managed ? static_cast<char*>(m_managed.get()) + m_lead : nullptr;
    }
    bool is_null() const { return get() == nullptr; }
    size_t get_size() const { return m_bytes; }
    size_t get_pitch() const { return m_pitch; }
    size_t get_real_size() const { return m_bytes; }
    void memset(int v, cudaStream_t stream = 0)
    {
        if (is_null())
            return;
        // an owned allocation is cleared from its start (the lead cells too)
        void* from = m_alias ? m_alias : m_managed.get();
        const size_t n = m_alias ? m_bytes : m_bytes + m_lead;
        if (std::is_same<Allocator, BaseAllocator>::value)
            std::memset(from, v, n);
        else
            cudaMemsetAsync(from, v, n, stream);
    }
    // dense host array <-> this buffer (rows of ldim bytes at pitch bytes)
    void copyin(const void* host)
    {
        if (std::is_same<Allocator, BaseAllocator>::value)
            std::memcpy(get(), host, m_bytes);
        else if (m_pitch == m_ldim || m_ldim == 0)
            cudaMemcpy(get(), host, m_bytes, cudaMemcpyHostToDevice);
        else
            cudaMemcpy2D(get(), m_pitch, host, m_ldim, m_ldim, m_bytes / m_pitch, cudaMemcpyHostToDevice);
    }
    void copyout(void* host) const
    {
        if (std::is_same<Allocator, BaseAllocator>::value)
            std::memcpy(host, get(), m_bytes);
        else if (m_pitch == m_ldim || m_ldim == 0)
            cudaMemcpy(host, get(), m_bytes, cudaMemcpyDeviceToHost);
        else
            cudaMemcpy2D(host, m_ldim, get(), m_pitch, m_ldim, m_bytes / m_pitch, cudaMemcpyDeviceToHost);
    }

private:
    std::shared_ptr<void> m_managed;
    void* m_alias = nullptr;
    size_t m_bytes = 0, m_pitch = 0, m_ldim = 0, m_lead = 0;
};

// Fixed-rank index / extent array with DistConv's negative indexing
// (tensor/tensor_base.hpp:28-250).
template <int ND, typename DataType = index_t>
class Array
{
public:
    static constexpr int num_dims = ND;
    using data_type = DataType;
    Array() { m_data.fill(DataType(0)); }
    Array(DataType v) { m_data.fill(v); }
    Array(std::initializer_list<DataType> l)
    {
        util::require((int) l.size() == ND, "Array: wrong number of initialisers");
        std::copy(l.begin(), l.end(), m_data.begin());
    }
    explicit Array(const Vector<DataType>& v)
    {
        util::require(v.num_dims() == ND, "Array: wrong rank");
        std::copy(v.begin(), v.end(), m_data.begin());
    }
    DataType& operator[](int i) { return m_data[i < 0 ? ND + i : i]; }
    const DataType& operator[](int i) const { return m_data[i < 0 ? ND + i : i]; }
    DataType get_size() const
    {
        DataType p = 1;
        for (auto v : m_data)
            p *= v;
        return p;
    }
    bool operator==(const Array& o) const { return m_data == o.m_data; }
    bool operator!=(const Array& o) const { return !(*this == o); }
    Array operator+(const Array& o) const
    {
        Array r;
        for (int i = 0; i < ND; ++i)
            r[i] = m_data[i] + o.m_data[i];
        return r;
    }
    Array operator-(const Array& o) const
    {
        Array r;
        for (int i = 0; i < ND; ++i)
            r[i] = m_data[i] - o.m_data[i];
        return r;
    }
    Vector<DataType> get_vector() const { return Vector<DataType>(std::vector<DataType>(m_data.begin(), m_data.end())); }
    auto begin() const { return m_data.begin(); }
    auto end() const { return m_data.end(); }

private:
    std::array<DataType, ND> m_data;
};

// offset of an index in a dense array of the given shape / the strides of
// that shape, dimension 0 fastest (tensor_base.hpp get_offset / get_strides)
inline index_t get_offset(const IndexVector& idx, const Shape& shape)
{
    index_t off = 0, stride = 1;
    for (int i = 0; i < shape.num_dims(); ++i)
    {
        off += idx[i] * stride;
        stride *= shape[i];
    }
    return off;
}
inline Shape get_strides(const Shape& shape)
{
    Shape st(shape.size(), 1);
    for (int i = 1; i < shape.num_dims(); ++i)
        st[i] = st[i - 1] * shape[i - 1];
    return st;
}

inline index_t split_extent(index_t total, index_t parts, index_t index)
{
    return total / parts + (index < total % parts ? 1 : 0);
}

} // namespace tensor
} // namespace distconv

namespace distconv
{
namespace tensor
{

// Block-distributed float tensor shard with halo cells on both sides of every
// partitioned dimension that has an overlap.  Owns its device memory unless it
// is a view.  `local_shape_of` (optional) maps a grid index to that rank's
// local shape -- DistConv's "requested local shape" for convolution outputs.
template <typename DataType = float, typename Locale = LocaleMPI, typename Allocator = CUDAAllocator>
class Tensor
{
public:
    using data_type = DataType;
    using LocalShapeFn = std::function<Shape(const IndexVector&)>;

    Tensor() = default;
    Tensor(const Shape& shape, const Locale& locale, const Distribution& dist, LocalShapeFn fn = nullptr)
        : m_shape(shape), m_locale(locale), m_dist(dist), m_fn(std::move(fn))
    {
        const int nd = shape.num_dims();
        m_proc_idx = locale.get_rank_idx(m_dist);
        m_split_idx = IndexVector(nd, 0);
        for (int i = 0; i < nd; ++i)
            m_split_idx[i] = m_proc_idx[i] / m_dist.get_num_ranks_per_split(i);
        m_local_shape = local_of(m_proc_idx);
        m_offset = IndexVector(nd, 0);
        for (int d = 0; d < nd; ++d)
            m_offset[d] = get_dimension_rank_offset(d, (int) m_proc_idx[d]);
        m_pitch = Allocator::pitch(m_local_shape[0] + 2 * m_dist.get_overlap(0), m_dist.get_overlap(0));
    }

    Shape local_of(const IndexVector& proc_idx) const
    {
        if (m_fn)
            return m_fn(proc_idx);
        Shape out(m_shape.size(), 0);
        for (int d = 0; d < (int) m_shape.size(); ++d)
            out[d] = m_dist.is_distributed(d)
                         ? split_extent(m_shape[d], m_dist.get_split_shape()[d],
                                        proc_idx[d] / m_dist.get_num_ranks_per_split(d))
                         : m_shape[d];
        return out;
    }

    int get_num_dims() const { return m_shape.num_dims(); }
    int get_num_spatial_dims() const { return get_num_dims() - 2; }
    const Shape& get_shape() const { return m_shape; }
    const Shape& get_local_shape() const { return m_local_shape; }
    Shape get_local_real_shape() const
    {
        Shape r = m_local_shape;
        for (int i = 0; i < get_num_dims(); ++i)
            r[i] += 2 * m_dist.get_overlap(i);
        return r;
    }
    index_t get_local_size() const { return m_local_shape.get_size(); }
    index_t get_size() const { return m_shape.get_size(); }
    const IndexVector& get_global_index() const { return m_offset; }
    const Distribution& get_distribution() const { return m_dist; }
    const Locale& get_locale() const { return m_locale; }
    const IndexVector& get_split_index() const { return m_split_idx; }
    const IndexVector& get_proc_index() const { return m_proc_idx; }
    const IntVector& get_overlap() const { return m_dist.get_overlap(); }
    int get_halo_width(int dim) const { return m_dist.get_overlap(dim); }
    const LocalShapeFn& get_local_shape_fn() const { return m_fn; }
    bool is_split_root() const
    {
        for (int i = 0; i < get_num_dims(); ++i)
            if (m_proc_idx[i] % m_dist.get_num_ranks_per_split(i))
                return false;
        return true;
    }
    index_t get_dimension_rank_offset(int dim, int rank_idx) const
    {
        index_t off = 0;
        if (!m_dist.is_distributed(dim))
            return 0;
        const index_t per = m_dist.get_num_ranks_per_split(dim);
        for (index_t j = 0; j < rank_idx / per; ++j)
        {
            IndexVector idx = m_proc_idx;
            idx[dim] = j * per;
            off += local_of(idx)[dim];
        }
        return off;
    }

    // memory
    // elements between consecutive rows (tensor.hpp:184-192)
    index_t get_pitch() const { return m_pitch; }
    Shape get_local_pitched_shape() const
    {
        Shape r = get_local_real_shape();
        r[0] = m_pitch;
        return r;
    }
    index_t get_local_pitched_size() const { return get_local_pitched_shape().get_size(); }
    int allocate()
    {
        const size_t bytes = (size_t) get_local_pitched_size() * sizeof(DataType);
        if (m_data.allocate(bytes, (size_t) m_pitch * sizeof(DataType),
                            (size_t) get_local_real_shape()[0] * sizeof(DataType),
                            (size_t) Allocator::lead(m_dist.get_overlap(0)) * sizeof(DataType))
            != 0)
            return -1;
        m_data.memset(0);
        if (!std::is_same<Allocator, BaseAllocator>::value)
            cudaDeviceSynchronize();
        m_buf = static_cast<DataType*>(m_data.get());
        m_is_view = false;
        return 0;
    }
    // Alias caller memory laid out with this shard's pitch (tensor.hpp:604-623); a
    // view never frees.
    void set_view(void* raw)
    {
        m_data.alias(raw, (size_t) get_local_pitched_size() * sizeof(DataType), (size_t) m_pitch * sizeof(DataType),
                     (size_t) get_local_real_shape()[0] * sizeof(DataType));
        m_buf = static_cast<DataType*>(raw);
        m_is_view = true;
    }
    void set_view(const Memory<Allocator>& parent_mem)
    {
        m_data.alias(parent_mem);
        m_buf = static_cast<DataType*>(m_data.get());
        m_is_view = true;
    }
    bool is_view() const { return m_is_view; }
    bool is_null() const { return m_buf == nullptr; }
    Memory<Allocator>& get_data() { return m_data; }
    const Memory<Allocator>& get_data() const { return m_data; }
    void nullify()
    {
        m_data.nullify();
        m_buf = nullptr;
    }
    DataType* get_buffer() { return m_buf; }
    const DataType* get_const_buffer() const { return m_buf; }
    Shape get_strides() const
    {
        Shape st(m_shape.size(), 1);
        index_t acc = 1;
        const Shape real = get_local_pitched_shape();
        for (int i = 0; i < get_num_dims(); ++i)
        {
            st[i] = acc;
            acc *= real[i];
        }
        return st;
    }
    index_t get_local_offset(const IndexVector& idx, bool idx_include_halo = false) const
    {
        const Shape st = get_strides();
        index_t off = 0;
        for (int i = 0; i < get_num_dims(); ++i)
            off += (idx[i] + (idx_include_halo ? 0 : m_dist.get_overlap(i))) * st[i];
        return off;
    }
    DataType* get_base_ptr() { return m_buf + get_local_offset(IndexVector(m_shape.size(), 0)); }
    void zero(cudaStream_t s = 0) { m_data.memset(0, s); }
    void clear_halo(int dim, cudaStream_t s = 0)
    {
        if (get_local_size() == 0)
            return;
        dcb_tensor_desc d = desc();
        util::check(dcb_clear_halo(&d, m_buf, dim, s), "clear_halo");
    }

    // descriptors for the C ABI
    dcb_tensor_desc desc() const
    {
        dcb_tensor_desc d{};
        d.ndims = get_num_dims();
        d.dtype = DCB_F32;
        const Shape real = get_local_real_shape();
        for (int i = 0; i < d.ndims; ++i)
        {
            d.local_shape[i] = m_local_shape[i];
            d.real_shape[i] = real[i];
            d.overlap[i] = m_dist.get_overlap(i);
        }
        d.pitch = m_pitch;
        return d;
    }
    // owned cells extended by lo / hi halo cells per spatial dimension
    // (setup_tensor_descriptor, dnn_backend_impl.hpp:31-70)
    dcb_nd_desc nd_desc(const IntVector& lo, const IntVector& hi) const
    {
        const int nsd = get_num_spatial_dims();
        const Shape st = get_strides();
        dcb_nd_desc d{};
        d.nsd = nsd;
        d.n = m_local_shape[-1];
        d.c = m_local_shape[-2];
        d.sn = st[-1];
        d.sc = st[-2];
        for (int s = 0; s < 3; ++s)
        {
            d.dims[s] = 1;
            d.strides[s] = 0;
        }
        for (int i = 0; i < nsd; ++i)
        {
            d.dims[2 - i] = m_local_shape[i] + lo[i] + hi[i];
            d.strides[2 - i] = st[i];
        }
        return d;
    }
    dcb_nd_desc nd_desc() const
    {
        const IntVector z(get_num_dims(), 0);
        return nd_desc(z, z);
    }
    dcb_nd_desc full_nd_desc() const { return nd_desc(get_overlap(), get_overlap()); }
    DataType* nd_ptr(const IntVector& lo)
    {
        IndexVector idx(m_shape.size(), 0);
        for (int i = 0; i < get_num_dims(); ++i)
            idx[i] = m_dist.get_overlap(i) - (i < get_num_spatial_dims() ? lo[i] : 0);
        return m_buf + get_local_offset(idx, true);
    }

private:
    Shape m_shape, m_local_shape;
    Locale m_locale;
    Distribution m_dist;
    LocalShapeFn m_fn;
    IndexVector m_proc_idx, m_split_idx, m_offset;
    Memory<Allocator> m_data;
    DataType* m_buf = nullptr;
    index_t m_pitch = 0;
    bool m_is_view = false;
};

// tensor::View (tensor.hpp): make `t` alias caller memory / another tensor's memory.
template <typename DataType, typename Locale, typename Allocator>
inline int View(Tensor<DataType, Locale, Allocator>& t, DataType* raw_ptr)
{
    t.set_view(static_cast<void*>(raw_ptr));
    return 0;
}
template <typename DataType, typename Locale, typename Allocator>
inline int View(Tensor<DataType, Locale, Allocator>& t, const Tensor<DataType, Locale, Allocator>& parent)
{
    t.set_view(parent.get_data());
    return 0;
}

} // namespace tensor

using TensorF = tensor::Tensor<float, tensor::LocaleMPI, tensor::CUDAAllocator>;

namespace internal
{
inline int get_dilated_filter_size(int f, int d)
{
    return f + (f - 1) * (d - 1);
}

// distconv.hpp:21-99 for the rank whose geometry is given explicitly.
inline void halo_sizes_for(const tensor::Shape& shape, const tensor::Distribution& dist,
                           const tensor::IndexVector& split_idx, const tensor::IndexVector& offset,
                           const tensor::Shape& local_shape, const tensor::IntVector& filter_dims,
                           const tensor::IntVector& strides, const tensor::IntVector& dilations, bool with_padding,
                           tensor::IntVector& fwd_send, tensor::IntVector& bwd_send, tensor::IntVector& fwd_recv,
                           tensor::IntVector& bwd_recv)
{
    const int nd = shape.num_dims();
    fwd_send = bwd_send = fwd_recv = bwd_recv = tensor::IntVector(nd, 0);
    for (int i = 0; i < nd - 2; ++i)
    {
        if (dist.get_split_shape()[i] == 1)
            continue;
        const int df = get_dilated_filter_size(filter_dims[i], dilations[i]);
        if (df % 2 == 0)
            continue;
        const int radius = (df - 1) / 2, s = strides[i];
        const int off = (int) offset[i];
        if (split_idx[i] == 0)
        {
            if (with_padding)
                bwd_recv[i] = radius;
        }
        else
        {
            const int x = off - (with_padding ? 0 : radius);
            bwd_recv[i] = radius - (s - (x % s)) % s;
            bwd_send[i] = radius - (x - 1) % s;
        }
        if (!(split_idx[i] == dist.get_split_shape()[i] - 1 && !with_padding))
        {
            const int y = off + (int) local_shape[i] - 1 - (with_padding ? 0 : radius);
            fwd_recv[i] = radius - y % s;
            fwd_send[i] = radius - (s - ((y + 1) % s)) % s;
        }
        fwd_send[i] = std::max(fwd_send[i], 0);
        fwd_recv[i] = std::max(fwd_recv[i], 0);
        bwd_send[i] = std::max(bwd_send[i], 0);
        bwd_recv[i] = std::max(bwd_recv[i], 0);
    }
}

inline void get_halo_sizes(const TensorF& input, const tensor::IntVector& filter_dims,
                           const tensor::IntVector& strides, const tensor::IntVector& dilations,
                           tensor::IntVector& fwd_send, tensor::IntVector& bwd_send, tensor::IntVector& fwd_recv,
                           tensor::IntVector& bwd_recv, bool with_padding)
{
    halo_sizes_for(input.get_shape(), input.get_distribution(), input.get_split_index(), input.get_global_index(),
                   input.get_local_shape(), filter_dims, strides, dilations, with_padding, fwd_send, bwd_send,
                   fwd_recv, bwd_recv);
}
} // namespace internal
} // namespace distconv

namespace distconv
{

// ---- tensor factories (distconv.hpp:253-481) -------------------------------
inline TensorF create_input_tensor(const int_vector& shape, const int_vector& locale_shape,
                                   const int_vector& filter_dims, const int_vector& strides,
                                   const int_vector& dilations, bool /*deconv*/, const tensor::LocaleMPI& loc)
{
    const int nd = (int) shape.size();
    tensor::IntVector overlap(nd, 0);
    for (int i = 0; i < nd - 2; ++i)
    {
        if (locale_shape[i] == 1)
            continue;
        const int df = internal::get_dilated_filter_size(filter_dims[i], dilations[i]);
        if (df % 2)
            overlap[i] = (df - 1) / 2;
    }
    tensor::Shape s(shape.begin(), shape.end()), ls(locale_shape.begin(), locale_shape.end());
    return TensorF(s, loc, tensor::Distribution::make_overlapped_distribution(ls, overlap));
}

inline TensorF create_d_input_tensor(const TensorF& input)
{
    return TensorF(input.get_shape(), input.get_locale(), input.get_distribution(), input.get_local_shape_fn());
}

// filter_shape is (fw, fh, [fd,] C, K)
inline TensorF create_convolution_output_tensor(const TensorF& input, const int_vector& filter_shape,
                                                const int_vector& strides, const int_vector& pad,
                                                const int_vector& dilations, int /*num_groups*/ = 1)
{
    const int nd = input.get_num_dims(), nsd = nd - 2;
    const bool use_padding = pad[0] != 0;
    tensor::Shape out_shape(nd, 0);
    for (int i = 0; i < nsd; ++i)
    {
        const int df = internal::get_dilated_filter_size(filter_shape[i], dilations[i]);
        if (input.get_shape()[i] + 2 * pad[i] >= df)
            out_shape[i] = (input.get_shape()[i] - df + 1 + 2 * pad[i] + strides[i] - 1) / strides[i];
    }
    out_shape[-2] = filter_shape.back();
    out_shape[-1] = input.get_shape()[-1];
    tensor::Distribution dist = input.get_distribution();
    dist.clear_overlap();
    tensor::IntVector fdims(filter_shape.begin(), filter_shape.begin() + nsd);
    tensor::IntVector st(strides.begin(), strides.end()), dl(dilations.begin(), dilations.end());
    const int K = filter_shape.back();
    // get_convolution_output_local_tensor_shape (distconv.hpp:135-200) per grid index
    TensorF in_copy = input;
    auto fn = [in_copy, fdims, st, dl, use_padding, K](const tensor::IndexVector& pidx) {
        const auto& d = in_copy.get_distribution();
        const int nd2 = in_copy.get_num_dims();
        tensor::IndexVector split(nd2, 0), offset(nd2, 0);
        for (int i = 0; i < nd2; ++i)
            split[i] = pidx[i] / d.get_num_ranks_per_split(i);
        tensor::Shape local = in_copy.local_of(pidx);
        for (int dim = 0; dim < nd2; ++dim)
        {
            if (!d.is_distributed(dim))
                continue;
            const index_t per = d.get_num_ranks_per_split(dim);
            for (index_t j = 0; j < split[dim]; ++j)
            {
                tensor::IndexVector idx = pidx;
                idx[dim] = j * per;
                offset[dim] += in_copy.local_of(idx)[dim];
            }
        }
        tensor::IntVector fs, bs, fr, br;
        internal::halo_sizes_for(in_copy.get_shape(), d, split, offset, local, fdims, st, dl, use_padding, fs, bs,
                                 fr, br);
        tensor::Shape out = local;
        for (int i = 0; i < nd2 - 2; ++i)
        {
            const int df = internal::get_dilated_filter_size(fdims[i], dl[i]);
            index_t ext = local[i] + br[i] + fr[i];
            if (use_padding && d.get_split_shape()[i] == 1)
                ext += df - 1;
            out[i] = ext < df ? 0 : (ext - df + 1 + st[i] - 1) / st[i];
        }
        out[-2] = K;
        return out;
    };
    return TensorF(out_shape, input.get_locale(), dist, fn);
}

inline TensorF create_convolution_d_output_tensor(const TensorF& output, const int_vector& filter_shape,
                                                  const int_vector& dilations)
{
    const int nd = output.get_num_dims();
    tensor::Distribution dist = output.get_distribution();
    tensor::IntVector overlap(nd, 0);
    for (int i = 0; i < nd - 2; ++i)
        if (dist.get_locale_shape()[i] > 1)
            overlap[i] = (internal::get_dilated_filter_size(filter_shape[i], dilations[i]) - 1) / 2;
    // the overlap only survives on distributed dimensions, as in the reference
    tensor::Distribution d2(dist.get_locale_shape(), dist.get_split_shape(), overlap);
    TensorF out_copy = output;
    return TensorF(output.get_shape(), output.get_locale(), d2,
                   [out_copy](const tensor::IndexVector& p) { return out_copy.local_of(p); });
}

// distconv.hpp:518-581.  Odd windows with pad 0 or (window-1)/2, even windows
// with stride == window: the output extents and the per-rank split follow the
// convolution's formulas with K = C.
inline TensorF create_pooling_output_tensor(const TensorF& input, const int_vector& window,
                                            const int_vector& strides, const int_vector& pad)
{
    const int nsd = input.get_num_dims() - 2;
    int_vector fshape(window.begin(), window.begin() + nsd);
    fshape.push_back((int) input.get_shape()[-2]);
    fshape.push_back((int) input.get_shape()[-2]);
    return create_convolution_output_tensor(input, fshape, strides, pad, int_vector(nsd, 1));
}

inline TensorF create_pooling_d_output_tensor(const TensorF& output)
{
    TensorF out_copy = output;
    return TensorF(output.get_shape(), output.get_locale(), output.get_distribution(),
                   [out_copy](const tensor::IndexVector& p) { return out_copy.local_of(p); });
}

namespace tensor
{
enum class HaloExchangeAccumOp
{
    ID = 0,
    SUM = 1,
    MAX = 2,
    MIN = 3
};

} // namespace tensor
} // namespace distconv

// The communication back end is a tag here (the reference instantiates its
// halo exchange and all-reduce classes with Al::NCCLBackend): its comm_type
// carries the stream a boundary's work is ordered on.
#ifndef DISTCONV_B200_NO_AL_TAG
namespace Al
{
struct NCCLBackend
{
    class comm_type
    {
    public:
        explicit comm_type(cudaStream_t stream = 0) : m_stream(stream) {}
        cudaStream_t get_stream() const { return m_stream; }

    private:
        cudaStream_t m_stream;
    };
};
} // namespace Al
#endif

namespace distconv
{
namespace tensor
{

// tensor::HaloExchange<DataType, Allocator, AlBackend> (halo_exchange_cuda.hpp:18-423)
// on the peer-store transport.  The constructor maps the neighbours' receive
// slabs through the tensor's locale (one allgather of 256-byte blobs).
// The reference's per-side communicators and boundary streams are accepted by
// the overloads below; the whole ordered exchange is enqueued on the main
// stream, which gives the ordering the reference builds with its stream
// fan-out / fan-in (halo_exchange_cuda.hpp:68-105).
template <typename DataType = float, typename Allocator = CUDAAllocator, typename AlBackend = Al::NCCLBackend>
class HaloExchange
{
    static_assert(std::is_same<DataType, float>::value, "only float tensors");

public:
    using TensorType = Tensor<DataType, LocaleMPI, Allocator>;
    using CommType = std::shared_ptr<typename AlBackend::comm_type>;

    explicit HaloExchange(TensorType& t) : m_tensor(t)
    {
        int32_t peers[2 * DCB_MAX_DIMS];
        for (int d = 0; d < DCB_MAX_DIMS; ++d)
            for (int s = 0; s < 2; ++s)
                peers[2 * d + s] = find_peer_rank(d, s);
        dcb_tensor_desc desc = t.desc();
        util::check(dcb_halo_plan_create(&desc, peers, t.get_locale().get_rank(), &m_plan), "halo plan");
        const int n = t.get_locale().get_size();
        std::vector<char> mine(DCB_HALO_BLOB_BYTES), all((size_t) n * DCB_HALO_BLOB_BYTES);
        util::check(dcb_halo_plan_export(m_plan, mine.data()), "halo export");
        t.get_locale().allgather(mine.data(), all.data(), DCB_HALO_BLOB_BYTES);
        util::check(dcb_halo_plan_connect(m_plan, all.data(), n), "halo connect");
    }
    HaloExchange(const HaloExchange&) = delete;
    virtual ~HaloExchange() { dcb_halo_plan_destroy(m_plan); }

    int find_peer_rank(int dim, int side) const
    {
        const TensorType& t = m_tensor;
        if (dim >= t.get_num_dims() || !t.get_distribution().is_distributed(dim) || t.get_halo_width(dim) == 0
            || t.get_local_size() == 0)
            return -1;
        const auto& ls = t.get_distribution().get_locale_shape();
        const index_t j = t.get_proc_index()[dim] + (side == RHS ? 1 : -1);
        if (j < 0 || j >= ls[dim])
            return -1;
        if (t.get_dimension_rank_offset(dim, (int) j) == t.get_shape()[dim])
            return -1;
        IndexVector idx = t.get_proc_index();
        idx[dim] = j;
        if (t.local_of(idx).get_size() == 0)
            return -1;
        int r = 0, m = 1;
        for (int i = 0; i < t.get_num_dims(); ++i)
        {
            r += (int) idx[i] * m;
            m *= (int) ls[i];
        }
        return r;
    }
    bool is_exchange_required(int dim) const { return find_peer_rank(dim, LHS) >= 0 || find_peer_rank(dim, RHS) >= 0; }

    // ---- the reference's argument lists (halo_exchange_cuda.hpp:56-146) ----
    // all dimensions, widths = the tensor's halo widths
    void exchange(BoundaryAttributesV<CommType>& /*comms*/, cudaStream_t stream_main, bool /*rendezvous*/,
                  bool /*sync_back*/, bool is_reverse, bool skip_unpack,
                  HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        exchange(stream_main, is_reverse, skip_unpack, op);
    }
    // all dimensions with explicit widths.  The slabs exchanged are always the
    // tensor's whole halo (a superset of narrower requests, e.g. the one-sided
    // widths of a strided convolution): widths wider than the halo are refused.
    void exchange(const IntVector& widths_rhs_send, const IntVector& widths_rhs_recv,
                  const IntVector& widths_lhs_send, const IntVector& widths_lhs_recv,
                  BoundaryAttributesV<CommType>& comms, cudaStream_t stream_main, bool rendezvous, bool sync_back,
                  bool is_reverse, bool skip_unpack, HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        for (int i = 0; i < m_tensor.get_num_spatial_dims(); ++i)
            for (int w : {widths_rhs_send[i], widths_rhs_recv[i], widths_lhs_send[i], widths_lhs_recv[i]})
                util::require(w <= m_tensor.get_halo_width(i), "halo exchange: width exceeds the tensor's overlap");
        exchange(comms, stream_main, rendezvous, sync_back, is_reverse, skip_unpack, op);
    }
    // one dimension
    void exchange(int dim, CommType& comm_rhs, CommType& /*comm_lhs*/, bool /*rendezvous*/, bool is_reverse,
                  bool skip_unpack, HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        const cudaStream_t stream = comm_rhs ? comm_rhs->get_stream() : 0;
        pack_put(dim, stream, is_reverse, op);
        if (!skip_unpack)
            wait_unpack(dim, stream, is_reverse, op);
    }
    void exchange(int dim, int width_rhs_send, int width_rhs_recv, int width_lhs_send, int width_lhs_recv,
                  CommType& comm_rhs, CommType& comm_lhs, bool rendezvous, bool is_reverse, bool skip_unpack,
                  HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        for (int w : {width_rhs_send, width_rhs_recv, width_lhs_send, width_lhs_recv})
            util::require(w <= m_tensor.get_halo_width(dim), "halo exchange: width exceeds the tensor's overlap");
        exchange(dim, comm_rhs, comm_lhs, rendezvous, is_reverse, skip_unpack, op);
    }
    // deferred unpack of a skip_unpack exchange (halo_exchange_cuda.hpp:148-202)
    void unpack(BoundaryAttributesV<cudaStream_t>& /*streams*/, cudaStream_t stream_main, bool /*sync_back*/,
                bool is_reverse, HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        unpack(stream_main, is_reverse, op);
    }

    // ---- the same on one stream ----
    void exchange(cudaStream_t stream, bool is_reverse = false, bool skip_unpack = false,
                  HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        util::check(dcb_halo_exchange(m_plan, m_tensor.get_buffer(), flags(is_reverse, skip_unpack, op), stream),
                    "halo exchange");
    }
    // Tensor::clear_halo of every dimension followed by the forward exchange, with
    // the clearing done by the pack launches (only slabs without a neighbour need
    // it: the others are overwritten)
    void clear_and_exchange(cudaStream_t stream)
    {
        util::check(dcb_halo_exchange(m_plan, m_tensor.get_buffer(), DCB_HALO_CLEAR_BOUNDARY, stream),
                    "halo exchange");
    }
    void unpack(cudaStream_t stream, bool is_reverse = false, HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        util::check(dcb_halo_unpack(m_plan, m_tensor.get_buffer(), flags(is_reverse, false, op), stream),
                    "halo unpack");
    }
    // The two halves of one dimension's exchange, for callers that run
    // several ranks from one process on one device and therefore must launch
    // every rank's put before any rank's wait.
    void pack_put(int dim, cudaStream_t stream, bool is_reverse = false,
                  HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        util::check(dcb_halo_pack_put(m_plan, m_tensor.get_buffer(), dim, flags(is_reverse, false, op), stream),
                    "halo pack_put");
    }
    void wait_unpack(int dim, cudaStream_t stream, bool is_reverse = false,
                     HaloExchangeAccumOp op = HaloExchangeAccumOp::ID)
    {
        util::check(dcb_halo_wait_unpack(m_plan, m_tensor.get_buffer(), dim, flags(is_reverse, false, op), stream),
                    "halo wait_unpack");
    }
    int32_t status(cudaStream_t stream) { return dcb_halo_plan_status(m_plan, stream); }

private:
    static uint32_t flags(bool rev, bool skip, HaloExchangeAccumOp op)
    {
        return (rev ? DCB_HALO_REVERSE : 0u) | (skip ? DCB_HALO_SKIP_UNPACK : 0u)
               | ((uint32_t) op << DCB_HALO_OP_SHIFT);
    }
    TensorType& m_tensor;
    dcb_halo_plan* m_plan = nullptr;
};

// The reference's transports (halo_exchange_cuda_{mpi,al,p2p,hybrid}.hpp) are one
// here: packed faces go straight into the neighbour's receive slab by peer
// stores.  The names stay so that code that spells a transport compiles.
template <typename DataType = float, typename Allocator = CUDAAllocator, typename AlBackend = Al::NCCLBackend>
using HaloExchangeMPI = HaloExchange<DataType, Allocator, AlBackend>;
template <typename DataType = float, typename Allocator = CUDAAllocator, typename AlBackend = Al::NCCLBackend>
using HaloExchangeAL = HaloExchange<DataType, Allocator, AlBackend>;
template <typename DataType = float, typename Allocator = CUDAAllocator, typename AlBackend = Al::NCCLBackend>
using HaloExchangeP2P = HaloExchange<DataType, Allocator, AlBackend>;
template <typename DataType = float, typename Allocator = CUDAAllocator, typename AlBackend = Al::NCCLBackend>
using HaloExchangeHybrid = HaloExchange<DataType, Allocator, AlBackend>;

// What `rank` owns of t, in global coordinates; empty for a rank that is not
// the root of a replicated dimension.
inline dcb_box owned_box(const TensorF& t, int rank)
{
    dcb_box b;
    std::memset(&b, 0, sizeof(b));
    const int nd = t.get_num_dims();
    const auto& d = t.get_distribution();
    IndexVector pidx(nd, 0);
    int r = rank;
    bool root = true;
    for (int i = 0; i < nd; ++i)
    {
        pidx[i] = r % d.get_locale_shape()[i];
        r /= (int) d.get_locale_shape()[i];
        root = root && pidx[i] % d.get_num_ranks_per_split(i) == 0;
    }
    const Shape ext = t.local_of(pidx);
    if (!root || ext.get_size() == 0)
        return b;
    for (int i = 0; i < nd; ++i)
    {
        b.ext[i] = ext[i];
        if (!d.is_distributed(i))
            continue;
        const index_t per = d.get_num_ranks_per_split(i);
        for (index_t j = 0; j < pidx[i] / per; ++j)
        {
            IndexVector idx = pidx;
            idx[i] = j * per;
            b.off[i] += t.local_of(idx)[i];
        }
    }
    return b;
}

// tensor::TensorMPICUDAShuffler (shuffle_mpi_cuda.hpp:14-512): re-distribution
// between the distributions of two tensors of one global shape.  The optional
// work buffers of the reference's constructor are accepted and unused: cells go
// straight into the owners' receive windows.
template <typename DataType>
class TensorMPICUDAShuffler;

template <>
class TensorMPICUDAShuffler<float>
{
public:
    TensorMPICUDAShuffler(const TensorF& src_tensor, const TensorF& dst_tensor, float* /*src_buf*/ = nullptr,
                          float* /*dst_buf*/ = nullptr)
    {
        m_fwd = make(src_tensor, dst_tensor);
        m_bwd = make(dst_tensor, src_tensor);
    }
    TensorMPICUDAShuffler(const TensorMPICUDAShuffler&) = delete;
    ~TensorMPICUDAShuffler()
    {
        dcb_shuffle_plan_destroy(m_fwd);
        dcb_shuffle_plan_destroy(m_bwd);
    }
    void shuffle_forward(const float* src, float* dst, cudaStream_t stream = 0)
    {
        util::check(dcb_shuffle(m_fwd, src, dst, stream), "shuffle forward");
    }
    void shuffle_backward(const float* src, float* dst, cudaStream_t stream = 0)
    {
        util::check(dcb_shuffle(m_bwd, src, dst, stream), "shuffle backward");
    }
    // The halves of a shuffle, for callers that run several ranks on one device.
    void put(bool forward, const float* src, cudaStream_t stream)
    {
        util::check(dcb_shuffle_put(forward ? m_fwd : m_bwd, src, stream), "shuffle put");
    }
    void wait_unpack(bool forward, float* dst, cudaStream_t stream)
    {
        util::check(dcb_shuffle_wait_unpack(forward ? m_fwd : m_bwd, dst, stream), "shuffle wait_unpack");
    }
    int32_t status(bool forward, cudaStream_t stream) { return dcb_shuffle_plan_status(forward ? m_fwd : m_bwd, stream); }
    static size_t get_buf_size(const TensorF& tensor) { return (size_t) tensor.get_local_size() * sizeof(float); }

private:
    static dcb_shuffle_plan* make(const TensorF& a, const TensorF& b)
    {
        const int n = a.get_locale().get_size();
        std::vector<dcb_box> ab((size_t) n), bb((size_t) n);
        for (int r = 0; r < n; ++r)
        {
            ab[r] = owned_box(a, r);
            bb[r] = owned_box(b, r);
        }
        const dcb_tensor_desc ad = a.desc(), bd = b.desc();
        dcb_shuffle_plan* p = nullptr;
        util::check(dcb_shuffle_plan_create(&ad, &bd, ab.data(), bb.data(), a.get_locale().get_rank(), n, &p),
                    "shuffle plan");
        std::vector<char> mine(DCB_SHUFFLE_BLOB_BYTES), all((size_t) n * DCB_SHUFFLE_BLOB_BYTES);
        util::check(dcb_shuffle_plan_export(p, mine.data()), "shuffle export");
        a.get_locale().allgather(mine.data(), all.data(), DCB_SHUFFLE_BLOB_BYTES);
        util::check(dcb_shuffle_plan_connect(p, all.data(), n), "shuffle connect");
        return p;
    }
    dcb_shuffle_plan* m_fwd = nullptr;
    dcb_shuffle_plan* m_bwd = nullptr;
};
} // namespace tensor

// make_halo_exchange (dnn_backend/halo_exchange_factory.hpp:27-100): every
// method yields the one transport.
template <typename DataT, typename AllocT>
inline std::unique_ptr<tensor::HaloExchange<DataT, AllocT>>
make_halo_exchange(tensor::Tensor<DataT, tensor::LocaleMPI, AllocT>& t, HaloExchangeMethod method)
{
    util::MPIRootPrintStreamDebug() << "Using " << method << " in halo exchange (peer-store transport)";
    return std::make_unique<tensor::HaloExchange<DataT, AllocT>>(t);
}

// StreamManager (dnn_backend.hpp:66-117, legacy/src/dnn_backend/stream_manager.cpp):
// the main stream plus num_internal_streams non-blocking and as many priority
// streams.  The main stream is the caller's and is never destroyed here.
class StreamManager
{
public:
    explicit StreamManager(size_t num_internal_streams, cudaStream_t main_stream = 0) : m_stream(main_stream)
    {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        for (size_t i = 0; i < num_internal_streams; ++i)
        {
            cudaStream_t a = nullptr, b = nullptr;
            cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking);
            cudaStreamCreateWithPriority(&b, cudaStreamNonBlocking, hi);
            m_internal_streams.push_back(a);
            m_priority_streams.push_back(b);
        }
    }
    StreamManager(const StreamManager&) = delete;
    ~StreamManager() noexcept
    {
        for (auto st : m_internal_streams)
            if (st)
                cudaStreamDestroy(st);
        for (auto st : m_priority_streams)
            if (st)
                cudaStreamDestroy(st);
    }
    size_t num_streams() const noexcept { return m_internal_streams.size(); }
    cudaStream_t stream() const noexcept { return m_stream; }
    cudaStream_t internal_stream(size_t idx) const { return m_internal_streams.at(idx); }
    cudaStream_t priority_stream(size_t idx) const { return m_priority_streams.at(idx); }

private:
    cudaStream_t m_stream;
    std::vector<cudaStream_t> m_internal_streams, m_priority_streams;
};

// DNNBackend<GPUDNNBackend> = BackendDNNLib (dnn_backend.hpp:635-980,
// legacy/src/dnn_backend/dnn_backend.cpp:65-190): options, the main stream (the
// caller's), eight internal and eight priority streams with one communicator
// per priority stream, and a working all-reduce communicator (the reference
// never constructs its own, communicator_manager.cpp:26-57).  Handle_t is
// opaque and unused: there is no vendor library behind this backend.
class BackendDNNLib
{
public:
    using Handle_t = void*;
    using Stream_t = cudaStream_t;
    using AlCommType = Al::NCCLBackend::comm_type;
    using InternalCommType = Al::NCCLBackend::comm_type;
    static constexpr size_t num_internal_streams = 8;

    BackendDNNLib(const tensor::LocaleMPI& loc, cudaStream_t stream = 0, Options opts = Options{},
                  int allreduce_max_count = 32768)
        : m_loc(loc), m_opts(opts), m_streams(num_internal_streams, stream), m_al_comm(stream)
    {
        for (size_t i = 0; i < num_internal_streams; ++i)
            m_internal_comms.push_back(std::make_shared<InternalCommType>(m_streams.priority_stream(i)));
        util::check(dcb_comm_create_peer(loc.get_rank(), loc.get_size(), allreduce_max_count, &m_comm), "comm");
        std::vector<char> mine(DCB_COMM_BLOB_BYTES), all((size_t) loc.get_size() * DCB_COMM_BLOB_BYTES);
        util::check(dcb_comm_export(m_comm, mine.data()), "comm export");
        loc.allgather(mine.data(), all.data(), DCB_COMM_BLOB_BYTES);
        util::check(dcb_comm_connect(m_comm, all.data(), loc.get_size()), "comm connect");
    }
    // the earlier three-argument form
    BackendDNNLib(const tensor::LocaleMPI& loc, cudaStream_t stream, int allreduce_max_count)
        : BackendDNNLib(loc, stream, Options{}, allreduce_max_count)
    {}
#if defined(DISTCONV_B200_HAS_MPI)
    // The reference's constructors (dnn_backend.hpp:661-665).
    BackendDNNLib(MPI_Comm comm, Handle_t /*handle*/, Options opts = Options{})
        : BackendDNNLib(tensor::LocaleMPI(comm), 0, opts)
    {}
    BackendDNNLib(MPI_Comm comm, Handle_t /*handle*/, Stream_t stream, Options opts = Options{})
        : BackendDNNLib(tensor::LocaleMPI(comm), stream, opts)
    {}
    MPI_Comm get_comm() const noexcept { return m_loc.get_comm(); }
#else
    const tensor::LocaleMPI& get_comm() const { return m_loc; }
#endif
    BackendDNNLib(const BackendDNNLib&) = delete;
    virtual ~BackendDNNLib() { dcb_comm_destroy(m_comm); }

    std::string get_name() const { return "B200"; }
    const tensor::LocaleMPI& get_locale() const { return m_loc; }
    // option queries
    bool deterministic() const noexcept { return m_opts.m_deterministic; }
    bool profiling() const noexcept { return m_opts.enable_profiling; }
    bool overlap_halo_exchange() const noexcept { return m_opts.overlap_halo_exchange; }
    float ws_capacity_factor() const noexcept { return m_opts.ws_capacity_factor; }
    int math_mode() const noexcept { return m_opts.math_mode; }
    // library management
    Handle_t get_handle() const noexcept { return nullptr; }
    Stream_t get_stream() const noexcept { return m_streams.stream(); }
    Stream_t get_internal_priority_stream(size_t idx) const { return m_streams.priority_stream(idx); }
    Stream_t get_internal_stream(size_t idx) const { return m_streams.internal_stream(idx); }
    void wait() const { cudaStreamSynchronize(m_streams.stream()); }
    // communicators
    AlCommType& get_al_comm() { return m_al_comm; }
    AlCommType& get_al_nccl_comm() { return m_al_comm; }
    size_t get_num_internal_comms() const noexcept { return m_internal_comms.size(); }
    std::shared_ptr<InternalCommType> get_internal_comm(size_t idx) const { return m_internal_comms.at(idx); }

    void allreduce(float* p, index_t count)
    {
        util::check(dcb_allreduce_sum(m_comm, p, count, get_stream()), "allreduce");
    }
    // the two halves of allreduce (store to every peer / fold what arrived)
    void allreduce_push(float* p, index_t count)
    {
        util::check(dcb_allreduce_push(m_comm, p, count, get_stream()), "allreduce push");
    }
    void allreduce_pull(float* p, index_t count)
    {
        util::check(dcb_allreduce_pull(m_comm, p, count, get_stream()), "allreduce pull");
    }

private:
    tensor::LocaleMPI m_loc;
    Options m_opts;
    StreamManager m_streams;
    AlCommType m_al_comm;
    std::vector<std::shared_ptr<InternalCommType>> m_internal_comms;
    dcb_comm* m_comm = nullptr;
};
template <typename VendorBackend = void>
using DNNBackend = BackendDNNLib;

// tensor::Allreduce<T> (tensor/allreduce.hpp:8-19) over the backend's communicator.
namespace tensor
{
template <typename DataType>
class Allreduce
{
public:
    explicit Allreduce(BackendDNNLib& be) : m_be(be) {}
    void allreduce(DataType* buf, size_t count) { m_be.allreduce(buf, (index_t) count); }
    void allreduce(const DataType* send_buf, DataType* recv_buf, size_t count)
    {
        if (send_buf != recv_buf)
            cudaMemcpyAsync(recv_buf, send_buf, count * sizeof(DataType), cudaMemcpyDeviceToDevice, m_be.get_stream());
        m_be.allreduce(recv_buf, (index_t) count);
    }

private:
    BackendDNNLib& m_be;
};
} // namespace tensor

template <typename Backend, typename DataType>
class Convolution;
template <typename Backend, typename DataType>
class BatchNormalization;

// Convolution<BackendDNNLib, float> (convolution.hpp:19-3003), spatial
// parallelism only.  Filters, biases and their gradients are dense device
// arrays: filter [K][C][fd][fh][fw], bias [K].
template <>
class Convolution<BackendDNNLib, float>
{
public:
    // convolution.hpp:29-91: the four-argument form takes overlap and profiling
    // from the backend's options, the six-argument form states them.
    Convolution(BackendDNNLib& backend, int num_dims, HaloExchangeMethod method = HaloExchangeMethod::P2P,
                ChannelParallelismAlgorithm chanfilt_algo = ChannelParallelismAlgorithm::NONE)
        : Convolution(backend, num_dims, method, backend.overlap_halo_exchange(), backend.profiling(), chanfilt_algo)
    {}
    Convolution(BackendDNNLib& backend, int num_dims, HaloExchangeMethod /*method*/, bool enable_overlap,
                bool enable_profiling, ChannelParallelismAlgorithm chanfilt_algo = ChannelParallelismAlgorithm::NONE)
        : m_be(backend), m_num_dims(num_dims), m_nsd(num_dims - 2), m_math(backend.math_mode()),
          m_enable_overlap(enable_overlap), m_enable_profiling(enable_profiling)
    {
        if (chanfilt_algo != ChannelParallelismAlgorithm::NONE && chanfilt_algo != ChannelParallelismAlgorithm::AUTO)
            throw std::runtime_error("Convolution: channel / filter parallelism is not provided");
    }
    Convolution(const Convolution&) = delete;
    ~Convolution()
    {
        dcb_conv_plan_destroy(m_plan_fwd);
        dcb_conv_plan_destroy(m_plan_bwd);
        dcb_conv_plan_destroy(m_plan_wgrad);
    }

    // convolution.hpp:119-290.  filter_shape is (fw, fh, [fd,] C, K);
    // pads/strides/dilations are W first.  d_input / d_output may be null
    // (forward only).
    void setup(TensorF& input, const int_vector& filter_shape, TensorF& output, TensorF* d_input,
               TensorF* d_output, const int_vector& pads, const int_vector& strides, const int_vector& dilations,
               int num_groups = 1, int math_mode = -1)
    {
        if (num_groups != 1)
            throw std::runtime_error("Convolution: grouped convolution is not provided");
        if (math_mode < 0)
            math_mode = m_math; // the backend's option
        const int nsd = m_nsd;
        m_filter_dims = tensor::IntVector(filter_shape.begin(), filter_shape.begin() + nsd);
        m_C = filter_shape[nsd];
        m_K = filter_shape[nsd + 1];
        m_strides = tensor::IntVector(strides.begin(), strides.end());
        m_dilations = tensor::IntVector(dilations.begin(), dilations.end());
        m_math = math_mode;
        // setup_halo_xch (convolution.hpp:2672-2686); the d_output exchanger is
        // built on d_output, which is what backward data reads.
        m_halo_xch_input.reset(new tensor::HaloExchange<>(input));
        if (d_output)
            m_halo_xch_d_output.reset(new tensor::HaloExchange<>(*d_output));
        m_empty = input.get_local_size() == 0 || output.get_local_size() == 0;
        if (m_empty)
            return;
        tensor::IntVector stencil(nsd, 0);
        for (int i = 0; i < nsd; ++i)
        {
            const int wd = internal::get_dilated_filter_size(m_filter_dims[i], dilations[i]);
            if (wd % 2)
                stencil[i] = (wd - 1) / 2;
            else if (strides[i] != wd)
                throw std::runtime_error("Convolution: even filters need stride == filter size");
        }
        for (int i = 0; i < nsd; ++i)
            if (pads[i] != pads[0] || !(pads[i] == stencil[i] || pads[i] == 0))
                throw std::runtime_error("Convolution: padding must be 0 or the stencil radius on every dim");
        const bool use_padding = pads[0] != 0;
        internal::get_halo_sizes(input, m_filter_dims, m_strides, m_dilations, m_halo_fwd_send, m_halo_bwd_send,
                                 m_halo_fwd_recv, m_halo_bwd_recv, use_padding);
        // setup_convolution_descriptor (convolution.hpp:2541-2670)
        tensor::IntVector pads_fp(nsd, 0), pads_bp(nsd, 0);
        for (int i = 0; i < nsd; ++i)
        {
            pads_bp[i] = pads[i] == 0 ? stencil[i] : stencil[i] * strides[i];
            if (input.get_overlap()[i] > 0)
                pads_fp[i] = 0;
            else
                pads_fp[i] = pads_bp[i] = pads[i];
        }
        m_x_lo = m_halo_bwd_recv;
        m_xd = input.nd_desc(m_halo_bwd_recv, m_halo_fwd_recv);
        m_yd = output.nd_desc();
        m_pads_fp = pads_fp;
        m_pads_bp = pads_bp;
        m_has_bwd = d_output != nullptr;
        if (m_has_bwd)
        {
            // Backward data: the reference hands cuDNN the halo-extended d_input,
            // whose halo cells then receive partial sums nobody reads.  Where a
            // partitioned dimension has unit stride and dilation only the OWNED
            // cells are computed here: they start on a 16-byte boundary of a padded
            // row (the halo cells do not), which the bulk stores of the tensor-core
            // kernels need.  In the descriptor's terms the padding grows by
            // d_output's halo width.
            m_dyd = d_output->full_nd_desc();
            tensor::IntVector dlo = m_halo_bwd_recv, dhi = m_halo_fwd_recv;
            for (int i = 0; i < nsd; ++i)
                if (input.get_overlap()[i] > 0 && strides[i] == 1 && dilations[i] == 1)
                {
                    dlo[i] = dhi[i] = 0;
                    m_pads_bp[i] = stencil[i] + (int) d_output->get_overlap()[i];
                }
            m_dx_lo = dlo;
            m_dxd = (d_input ? *d_input : input).nd_desc(dlo, dhi);
            // Backward filter: the forward geometry with d_output's owned cells in the
            // output's place (the reference passes the halo-extended d_output with its
            // halo cleared; the owned cells alone give the same sums and need no clearing).
            m_dyod = d_output->nd_desc();
        }
        m_num_samples = (int) m_xd.n;
        make_plans();
    }

    // convolution.hpp:1147-1180: a mini-batch smaller than the tensors were
    // set up for (the last one of an epoch) changes the sample extent of every
    // descriptor; strides stay.  Plans are rebuilt for the new extent.
    void set_num_samples(int n)
    {
        util::require(n != 0, "set_num_samples: zero samples");
        if (m_empty || n == m_num_samples)
            return;
        util::MPIPrintStreamDebug() << "Setting #sample to " << n << " from " << m_num_samples;
        m_num_samples = n;
        m_xd.n = m_yd.n = n;
        if (m_has_bwd)
            m_dxd.n = m_dyd.n = m_dyod.n = n;
        dcb_conv_plan_destroy(m_plan_wgrad);
        m_plan_wgrad = nullptr;
        dcb_conv_plan_destroy(m_plan_fwd);
        dcb_conv_plan_destroy(m_plan_bwd);
        m_plan_fwd = m_plan_bwd = nullptr;
        make_plans();
    }

    // The reference's own argument list (convolution.hpp:119-135): filters
    // and their gradients are tensors of shape (fw, fh, [fd,] C, K) that every
    // rank holds whole (Distribution::make_shared_distribution).  The
    // algorithm names and the workspace size are accepted and ignored: there
    // is one kernel family and plans own their workspace.
    void setup(TensorF& input, TensorF& filter, TensorF& output, TensorF& d_input, TensorF& /*d_filter*/,
               TensorF& d_output, const int_vector& pads, const int_vector& strides, const int_vector& dilations,
               int num_groups, const std::string& /*fwd_algo*/ = "DEFAULT",
               const std::string& /*bwd_data_algo*/ = "DEFAULT", const std::string& /*bwd_filter_algo*/ = "DEFAULT",
               size_t /*ws_size*/ = 0, bool skip_bp_data = false, bool deconv = false)
    {
        if (deconv)
            throw std::runtime_error("Convolution: deconvolution is not provided");
        const tensor::Shape& fs = filter.get_shape();
        int_vector fshape(fs.begin(), fs.end());
        setup(input, fshape, output, skip_bp_data ? nullptr : &d_input, &d_output, pads, strides, dilations,
              num_groups);
    }
    int forward(float alpha, TensorF& input, TensorF& filter, float beta, TensorF& output,
                bool skip_halo_exchange = false, bool /*skip_chanfilt_comm*/ = false, bool /*dump_profile*/ = false,
                bool /*inference*/ = false)
    {
        return forward(alpha, input, filter.get_const_buffer(), beta, output, skip_halo_exchange);
    }
    int backward_data(float alpha, TensorF& filter, TensorF& d_output, float beta, TensorF& d_input,
                      bool skip_halo_exchange = false, bool /*skip_chanfilt_comm*/ = false,
                      bool /*dump_profile*/ = false)
    {
        return backward_data(alpha, filter.get_const_buffer(), d_output, beta, d_input, skip_halo_exchange);
    }
    int backward_filter(float alpha, TensorF& input, TensorF& d_output, float beta, TensorF& d_filter,
                        bool reduce = true, bool /*skip_chanfilt_comm*/ = false, bool /*dump_profile*/ = false)
    {
        return backward_filter(alpha, input, d_output, beta, d_filter.get_buffer(), reduce);
    }
    int apply_bias(float alpha, TensorF& bias, float beta, TensorF& output)
    {
        return apply_bias(alpha, bias.get_const_buffer(), beta, output);
    }
    int backward_bias(float alpha, TensorF& d_output, float beta, TensorF& bias_gradient, bool reduce = true)
    {
        return backward_bias(alpha, d_output, beta, bias_gradient.get_buffer(), reduce);
    }

    int kernel_kind(int which) const
    {
        return dcb_conv_plan_kernel_kind(which == 0 ? m_plan_fwd : (which == 1 ? m_plan_bwd : m_plan_wgrad), which);
    }
    // 0 fp32 CUDA-core, 1 / 2 tcgen05 row kernel, 3 sweep, 4 multi-group sweep, 5 tcgen05 backward filter
    int kernel_variant(int which) const
    {
        return dcb_conv_plan_kernel_variant(which == 0 ? m_plan_fwd : (which == 1 ? m_plan_bwd : m_plan_wgrad),
                                            which);
    }
    tensor::HaloExchange<>& input_halo_exchange() { return *m_halo_xch_input; }
    tensor::HaloExchange<>& d_output_halo_exchange() { return *m_halo_xch_d_output; }
    void forward_exchange_halo(TensorF&) { m_halo_xch_input->exchange(m_be.get_stream()); }
    // d_output's halo cells at the tensor's boundary stand in for the padding: cleared by the same launches
    void backward_data_exchange_halo(TensorF&) { m_halo_xch_d_output->clear_and_exchange(m_be.get_stream()); }

    // convolution.hpp:342-639, the branch without interior/boundary overlap
    int forward(float alpha, TensorF& input, const float* filter, float beta, TensorF& output,
                bool skip_halo_exchange = false)
    {
        if (input.get_local_size() == 0 || output.get_local_size() == 0)
            return 0;
        Range whole(m_enable_profiling, "conv/forward");
        set_num_samples((int) input.get_local_shape()[-1]);
        if (!skip_halo_exchange)
        {
            Range r(m_enable_profiling, "conv/forward/exchange_halo");
            m_halo_xch_input->clear_and_exchange(m_be.get_stream());
        }
        Range r(m_enable_profiling, "conv/forward/forward");
        util::check(dcb_conv_fwd(m_plan_fwd, alpha, input.nd_ptr(m_x_lo), filter, beta, output.get_base_ptr(),
                                 m_be.get_stream()),
                    "conv forward");
        return 0;
    }
    // Forward pass (beta = 0) that also leaves, per filter, the sum and the sum
    // of squares of this rank's output in sums / sqsums (K device floats
    // each): what BatchNormalization::forward_stage1 would compute from
    // `output`.  Returns 1 when the convolution's epilogue produced them, 0
    // when the plain forward pass ran and stage 1 is still to do.  No
    // counterpart in the reference, which always runs the two passes.
    int forward_with_statistics(float alpha, TensorF& input, const float* filter, TensorF& output, float* sums,
                                float* sqsums, bool skip_halo_exchange = false)
    {
        if (input.get_local_size() == 0 || output.get_local_size() == 0)
            return 0;
        if (!skip_halo_exchange)
            m_halo_xch_input->clear_and_exchange(m_be.get_stream());
        if (input.is_split_root())
        {
            const int32_t st = dcb_conv_fwd_stats(m_plan_fwd, alpha, input.nd_ptr(m_x_lo), filter,
                                                  output.get_base_ptr(), sums, sqsums, m_be.get_stream());
            if (st == DCB_OK)
                return 1;
            if (st != DCB_UNSUPPORTED)
                util::check(st, "conv forward with statistics");
        }
        forward(alpha, input, filter, 0.f, output, /*skip_halo_exchange=*/true);
        return 0;
    }
    // convolution.hpp:682-876
    int backward_data(float alpha, const float* filter, TensorF& d_output, float beta, TensorF& d_input,
                      bool skip_halo_exchange = false)
    {
        if (d_output.get_local_size() == 0 || d_input.get_local_size() == 0)
            return 0;
        Range whole(m_enable_profiling, "conv/bw_data");
        set_num_samples((int) d_input.get_local_shape()[-1]);
        if (!skip_halo_exchange)
        {
            Range r(m_enable_profiling, "conv/bw_data/exchange_halo");
            backward_data_exchange_halo(d_output);
        }
        util::check(dcb_conv_bwd_data(m_plan_bwd, alpha, filter, d_output.get_buffer(), beta,
                                      d_input.nd_ptr(m_dx_lo), m_be.get_stream()),
                    "conv backward data");
        return 0;
    }
    // convolution.hpp:878-1107, then the all-reduce of the filter gradient over every
    // rank.  Only d_output's owned cells are read, so its halo is not cleared first.
    int backward_filter(float alpha, TensorF& input, TensorF& d_output, float beta, float* d_filter,
                        bool reduce = true)
    {
        const index_t count = (index_t) m_K * m_C * m_filter_dims.get_size();
        Range whole(m_enable_profiling, "conv/bw_filter");
        if (input.get_local_size() != 0)
            set_num_samples((int) input.get_local_shape()[-1]);
        if (input.get_local_size() == 0 || d_output.get_local_size() == 0 || !input.is_split_root())
            cudaMemsetAsync(d_filter, 0, (size_t) count * sizeof(float), m_be.get_stream());
        else
        {
            util::check(dcb_conv_bwd_filter(m_plan_wgrad, alpha, input.nd_ptr(m_x_lo), d_output.get_base_ptr(), beta,
                                            d_filter, m_be.get_stream()),
                        "conv backward filter");
        }
        if (reduce)
            m_be.allreduce(d_filter, count);
        return 0;
    }
    // convolution.hpp:641-659
    int apply_bias(float alpha, const float* bias, float beta, TensorF& output)
    {
        if (output.get_local_size() == 0)
            return 0;
        const dcb_nd_desc yd = output.nd_desc();
        util::check(dcb_bias_fwd(alpha, bias, beta, &yd, output.get_base_ptr(), m_be.get_stream()), "bias");
        return 0;
    }
    // convolution.hpp:1109-1142
    int backward_bias(float alpha, TensorF& d_output, float beta, float* bias_gradient, bool reduce = true)
    {
        if (d_output.get_local_size() == 0)
            cudaMemsetAsync(bias_gradient, 0, (size_t) m_K * sizeof(float), m_be.get_stream());
        else
        {
            const dcb_nd_desc yd = d_output.nd_desc();
            util::check(dcb_bias_bwd(alpha, &yd, d_output.get_base_ptr(), beta, bias_gradient, m_be.get_stream()),
                        "bias backward");
        }
        if (reduce)
            m_be.allreduce(bias_gradient, m_K);
        return 0;
    }
    void wait() { m_be.wait(); }
    // Interior / boundary overlap (convolution.hpp:1497-1584) is not scheduled by
    // this class whatever enable_overlap says: at these sizes the whole exchange
    // is a few tens of microseconds on NVLink and the split costs more than it
    // hides (measured); the Python host mirror carries the reference's scheme.
    bool is_overlap_fwd_halo_exchange_enabled() const { return false; }
    bool is_overlap_bwd_halo_exchange_enabled() const { return false; }
    bool is_overlap_requested() const { return m_enable_overlap; }
    // DCB_OK unless a kernel of this layer gave up on a bounded wait
    int32_t status()
    {
        int32_t st = m_halo_xch_input ? m_halo_xch_input->status(m_be.get_stream()) : DCB_OK;
        if (st == DCB_OK && m_plan_fwd)
            st = dcb_conv_plan_status(m_plan_fwd, m_be.get_stream());
        return st;
    }

private:
    // a profiler range that lives as long as the scope it is declared in
    struct Range
    {
        Range(bool on, const char* name) : m_on(on)
        {
            if (m_on)
                util::profile_range_push(name);
        }
        ~Range()
        {
            if (m_on)
                util::profile_range_pop();
        }
        Range(const Range&) = delete;
        bool m_on;
    };
    void make_plans()
    {
        m_plan_fwd = make_plan(m_xd, m_yd, m_pads_fp);
        if (m_has_bwd)
        {
            m_plan_bwd = make_plan(m_dxd, m_dyd, m_pads_bp);
            m_plan_wgrad = make_plan(m_xd, m_dyod, m_pads_fp);
        }
    }
    dcb_conv_plan* make_plan(const dcb_nd_desc& xd, const dcb_nd_desc& yd, const tensor::IntVector& pads)
    {
        dcb_conv_desc cd{};
        cd.nsd = m_nsd;
        cd.k = m_K;
        cd.c = m_C;
        cd.groups = 1;
        cd.math_mode = m_math;
        for (int s = 0; s < 3; ++s)
        {
            cd.filter[s] = 1;
            cd.pads[s] = 0;
            cd.strides[s] = 1;
            cd.dilations[s] = 1;
        }
        for (int i = 0; i < m_nsd; ++i)
        {
            cd.filter[2 - i] = m_filter_dims[i];
            cd.pads[2 - i] = pads[i];
            cd.strides[2 - i] = m_strides[i];
            cd.dilations[2 - i] = m_dilations[i];
        }
        dcb_conv_plan* plan = nullptr;
        util::check(dcb_conv_plan_create(&cd, &xd, &yd, &plan), "conv plan");
        return plan;
    }
    void clear_halos(TensorF& t)
    {
        const auto& d = t.get_distribution();
        for (int dim = 0; dim < m_nsd; ++dim)
            if (d.is_distributed(dim) && d.get_locale_shape()[dim] > 1 && d.get_overlap(dim) > 0)
                t.clear_halo(dim, m_be.get_stream());
    }

    BackendDNNLib& m_be;
    int m_num_dims, m_nsd, m_K = 0, m_C = 0, m_math = DCB_MATH_FP32;
    bool m_enable_overlap = false, m_enable_profiling = false;
    bool m_empty = true, m_has_bwd = false;
    int m_num_samples = 0;
    dcb_nd_desc m_xd{}, m_yd{}, m_dxd{}, m_dyd{}, m_dyod{};
    tensor::IntVector m_pads_fp, m_pads_bp;
    tensor::IntVector m_filter_dims, m_strides, m_dilations, m_x_lo, m_dx_lo;
    tensor::IntVector m_halo_fwd_send, m_halo_bwd_send, m_halo_fwd_recv, m_halo_bwd_recv;
    std::unique_ptr<tensor::HaloExchange<>> m_halo_xch_input, m_halo_xch_d_output;
    dcb_conv_plan* m_plan_fwd = nullptr;
    dcb_conv_plan* m_plan_bwd = nullptr;
    dcb_conv_plan* m_plan_wgrad = nullptr;
};

// BatchNormalization<BackendDNNLib, float> (batchnorm.hpp:100-581).  The
// statistics vectors are C contiguous device floats; pass mean and var (and
// the gradient pairs) as the two halves of one 2C array and their all-reduce
// is one call (batchnorm.hpp:191-211).
template <>
class BatchNormalization<BackendDNNLib, float>
{
public:
    BatchNormalization(BackendDNNLib& backend, int num_dims, float decay, float epsilon, bool global_stats,
                       BatchnormImpl = BatchnormImpl::PEER)
        : m_be(backend), m_num_dims(num_dims), m_decay(decay), m_epsilon(epsilon), m_global_stats(global_stats)
    {}
    BatchNormalization(const BatchNormalization&) = delete;
    ~BatchNormalization() { dcb_bn_plan_destroy(m_plan); }

    int forward_stage1(TensorF& input, float* mean, float* var, bool is_training = true)
    {
        if (!is_training)
            return 0;
        const index_t C = input.get_local_shape()[-2];
        if (input.get_local_size() == 0 || !input.is_split_root())
        {
            cudaMemsetAsync(mean, 0, (size_t) C * sizeof(float), m_be.get_stream());
            cudaMemsetAsync(var, 0, (size_t) C * sizeof(float), m_be.get_stream());
            return 0;
        }
        util::check(dcb_bn_stats(plan(input), input.get_base_ptr(), mean, var, m_be.get_stream()), "bn stats");
        return 0;
    }
    int forward_allreduce(TensorF& input, float* mean, float* var, bool is_training = true)
    {
        if (is_training && m_global_stats)
            allreduce_pair(mean, var, input.get_local_shape()[-2]);
        return 0;
    }
    int forward_stage2(TensorF& input, float* mean, float* var, float* running_mean, float* running_var,
                       const float* scale, const float* bias, TensorF& output, bool is_training = true)
    {
        const index_t C = input.get_local_shape()[-2];
        const float *m = running_mean, *v = running_var;
        if (is_training)
        {
            util::check(dcb_bn_finalize((int32_t) C, num_per_sum(input), m_decay, mean, var, running_mean,
                                        running_var, m_be.get_stream()),
                        "bn finalize");
            m = mean;
            v = var;
        }
        if (input.get_local_size() == 0)
            return 0;
        const dcb_nd_desc xd = input.nd_desc(), yd = output.nd_desc();
        util::check(dcb_bn_apply(&xd, input.get_base_ptr(), m, v, scale, bias, m_epsilon, &yd,
                                 output.get_base_ptr(), m_be.get_stream()),
                    "bn apply");
        return 0;
    }
    // statistics_ready: mean / var already hold this rank's sums and sums of
    // squares (Convolution::forward_with_statistics returned 1)
    int forward(TensorF& input, float* mean, float* var, float* running_mean, float* running_var,
                const float* scale, const float* bias, TensorF& output, bool is_training = true,
                bool statistics_ready = false)
    {
        if (!statistics_ready)
            forward_stage1(input, mean, var, is_training);
        forward_allreduce(input, mean, var, is_training);
        return forward_stage2(input, mean, var, running_mean, running_var, scale, bias, output, is_training);
    }

    // The reference's argument list: statistics, scale and bias are tensors
    // of shape (1, 1, [1,] C, 1) held whole by every rank.
    int forward(TensorF& input, TensorF& mean, TensorF& var, TensorF& running_mean, TensorF& running_var,
                TensorF& scale, TensorF& bias, TensorF& output, bool is_training = true)
    {
        return forward(input, mean.get_buffer(), var.get_buffer(), running_mean.get_buffer(),
                       running_var.get_buffer(), scale.get_const_buffer(), bias.get_const_buffer(), output,
                       is_training);
    }
    int backward(TensorF& input, TensorF& d_output, TensorF& mean, TensorF& var, TensorF& scale,
                 TensorF& scale_gradient, TensorF& bias_gradient, TensorF& mean_gradient, TensorF& var_gradient,
                 TensorF& d_input)
    {
        return backward(input, d_output, mean.get_const_buffer(), var.get_const_buffer(), scale.get_const_buffer(),
                        scale_gradient.get_buffer(), bias_gradient.get_buffer(), mean_gradient.get_buffer(),
                        var_gradient.get_buffer(), d_input);
    }

    int backward_stage1(TensorF& input, TensorF& d_output, const float* mean, const float* var, const float* scale,
                        float* scale_gradient, float* bias_gradient, float* mean_gradient, float* var_gradient)
    {
        const size_t bytes = (size_t) input.get_local_shape()[-2] * sizeof(float);
        if (input.get_local_size() == 0 || !input.is_split_root())
        {
            for (float* g : {scale_gradient, bias_gradient, mean_gradient, var_gradient})
                cudaMemsetAsync(g, 0, bytes, m_be.get_stream());
            return 0;
        }
        const dcb_nd_desc dyd = d_output.nd_desc();
        util::check(dcb_bn_bwd_reduce(plan(input), input.get_base_ptr(), &dyd, d_output.get_base_ptr(), mean, var,
                                      scale, m_epsilon, scale_gradient, bias_gradient, mean_gradient, var_gradient,
                                      m_be.get_stream()),
                    "bn backward reduce");
        return 0;
    }
    // batchnorm.hpp:360-400: dmean||dvar when statistics are global, then dscale||dbias
    int backward_allreduce(TensorF& input, float* scale_gradient, float* bias_gradient, float* mean_gradient,
                           float* var_gradient, bool skip_weights = false)
    {
        const index_t C = input.get_local_shape()[-2];
        if (m_global_stats)
            allreduce_pair(mean_gradient, var_gradient, C);
        if (!skip_weights)
            allreduce_pair(scale_gradient, bias_gradient, C);
        return 0;
    }
    int backward_stage2(TensorF& input, TensorF& d_output, const float* mean, const float* var, const float* scale,
                        const float* mean_gradient, const float* var_gradient, TensorF& d_input)
    {
        if (input.get_local_size() == 0)
            return 0;
        const dcb_nd_desc xd = input.nd_desc(), dyd = d_output.nd_desc(), dxd = d_input.nd_desc();
        util::check(dcb_bn_bwd_apply(&xd, input.get_base_ptr(), &dyd, d_output.get_base_ptr(), mean, var, scale,
                                     mean_gradient, var_gradient, m_epsilon, num_per_sum(input), &dxd,
                                     d_input.get_base_ptr(), m_be.get_stream()),
                    "bn backward apply");
        return 0;
    }
    int backward(TensorF& input, TensorF& d_output, const float* mean, const float* var, const float* scale,
                 float* scale_gradient, float* bias_gradient, float* mean_gradient, float* var_gradient,
                 TensorF& d_input)
    {
        backward_stage1(input, d_output, mean, var, scale, scale_gradient, bias_gradient, mean_gradient,
                        var_gradient);
        backward_allreduce(input, scale_gradient, bias_gradient, mean_gradient, var_gradient);
        return backward_stage2(input, d_output, mean, var, scale, mean_gradient, var_gradient, d_input);
    }

    // batchnorm.hpp:467-475: nothing is cached per sample count here (descriptors
    // are built from the tensors at every call); kept for source compatibility.
    void set_num_samples(int /*n*/) {}

private:
    dcb_bn_plan* plan(TensorF& t)
    {
        if (!m_plan)
        {
            const dcb_nd_desc xd = t.nd_desc();
            util::check(dcb_bn_plan_create(&xd, &m_plan), "bn plan");
        }
        return m_plan;
    }
    index_t num_per_sum(const TensorF& t) const
    {
        const tensor::Shape& s = m_global_stats ? t.get_shape() : t.get_local_shape();
        return s.get_size() / s[-2];
    }
    void allreduce_pair(float* a, float* b, index_t n)
    {
        if (a + n == b)
            m_be.allreduce(a, 2 * n);
        else if (b + n == a)
            m_be.allreduce(b, 2 * n);
        else
        {
            m_be.allreduce(a, n);
            m_be.allreduce(b, n);
        }
    }
    BackendDNNLib& m_be;
    int m_num_dims;
    float m_decay, m_epsilon;
    bool m_global_stats;
    dcb_bn_plan* m_plan = nullptr; // one tensor shape per layer object
};

// Pooling<BackendDNNLib, float> (pooling.hpp:70-482).  Modes "MAX", "AVERAGE",
// "AVERAGE_NO_PAD" (pooling.hpp:27-48).
template <typename Backend, typename DataType>
class Pooling;

template <>
class Pooling<BackendDNNLib, float>
{
public:
    Pooling(BackendDNNLib& backend, int num_dims, HaloExchangeMethod = HaloExchangeMethod::P2P)
        : m_be(backend), m_num_dims(num_dims), m_nsd(num_dims - 2)
    {
    }

    // pooling.hpp:101-209
    void setup(TensorF& input, TensorF& output, TensorF& d_input, TensorF& d_output, int_vector windows,
               int_vector pads, int_vector strides, const std::string& mode)
    {
        util::require((int) windows.size() == m_nsd && (int) pads.size() == m_nsd && (int) strides.size() == m_nsd,
                      "pooling: windows / pads / strides must have one entry per spatial dimension");
        for (int i = 0; i < m_nsd; ++i)
        {
            util::require(windows[i] == windows[0] && pads[i] == pads[0] && strides[i] == strides[0],
                          "pooling: asymmetric windows are not supported");
            if (windows[i] % 2)
                util::require((pads[i] == 0 || pads[i] == (windows[i] - 1) / 2)
                                  && (strides[i] == 1 || strides[i] == (windows[i] - 1) / 2 + 1),
                              "pooling: unsupported pad / stride for an odd window");
            else
                util::require(windows[i] == strides[i] && pads[i] == 0,
                              "pooling: an even window needs stride == window and no padding");
        }
        util::require(mode == "MAX" || mode == "AVERAGE" || mode == "AVERAGE_NO_PAD", "pooling: unknown mode");
        std::memset(&m_pd, 0, sizeof(m_pd));
        m_pd.nsd = m_nsd;
        m_pd.mode = mode == "MAX" ? DCB_POOL_MAX : (mode == "AVERAGE" ? DCB_POOL_AVERAGE : DCB_POOL_AVERAGE_NO_PAD);
        const bool use_padding = pads[0] != 0;
        tensor::IntVector w(windows.begin(), windows.end()), st(strides.begin(), strides.end()), dl(m_nsd, 1);
        internal::get_halo_sizes(input, w, st, dl, m_halo_fwd_send, m_halo_bwd_send, m_halo_fwd_recv,
                                 m_halo_bwd_recv, use_padding);
        for (int s = 0; s < 3; ++s)
        {
            m_pd.window[s] = 1;
            m_pd.strides[s] = 1;
        }
        const auto& dist = input.get_distribution();
        for (int i = 0; i < m_nsd; ++i)
        {
            const bool split = dist.get_split_shape()[i] > 1;
            m_pd.window[2 - i] = windows[i];
            m_pd.strides[2 - i] = strides[i];
            // where a dimension is split the halo stands in for the padding
            // (pooling.hpp:189-194); at the boundary of the global tensor it is
            // padding, and the kernel is told so
            m_pd.pads[2 - i] = split ? 0 : pads[i];
            const bool first = input.get_split_index()[i] == 0;
            const bool last = input.get_split_index()[i] == dist.get_split_shape()[i] - 1;
            m_pd.outside_lo[2 - i] = split && first ? m_halo_bwd_recv[i] : 0;
            m_pd.outside_hi[2 - i] = split && last ? m_halo_fwd_recv[i] : 0;
        }
        m_halo_xch_input.reset(new tensor::HaloExchange<>(input));
        m_halo_xch_d_input.reset(new tensor::HaloExchange<>(d_input));
        (void) d_output;
        // index workspace of the backward pass: one byte per output cell, MAX only
        release_workspace();
        if (output.get_local_size() > 0)
        {
            const dcb_nd_desc xd = input.nd_desc(m_halo_bwd_recv, m_halo_fwd_recv), yd = output.nd_desc();
            const int64_t need = dcb_pool_bwd_workspace_bytes(&m_pd, &xd, &yd);
            if (need > 0 && cudaMalloc(&m_ws, (size_t) need) == cudaSuccess)
                m_ws_bytes = need;
        }
    }
    Pooling(const Pooling&) = delete;
    ~Pooling() { release_workspace(); }

    // pooling.hpp:212-244
    int forward(float alpha, TensorF& input, float beta, TensorF& output, bool /*training*/ = true,
                bool skip_halo_exchange = false)
    {
        if (!skip_halo_exchange)
        {
            if (m_be.profiling())
                util::profile_range_push("pooling/exchange_halo");
            m_halo_xch_input->clear_and_exchange(m_be.get_stream());
            if (m_be.profiling())
                util::profile_range_pop();
        }
        if (output.get_local_size() == 0)
            return 0;
        const dcb_nd_desc xd = input.nd_desc(m_halo_bwd_recv, m_halo_fwd_recv), yd = output.nd_desc();
        util::check(dcb_pool_fwd(&m_pd, &xd, &yd, alpha, input.nd_ptr(m_halo_bwd_recv), beta, output.get_base_ptr(),
                                 m_be.get_stream()),
                    "pooling forward");
        return 0;
    }

    // pooling.hpp:246-283: the gradients computed for halo cells return to their
    // owners with SUM; the halo cells no local window reaches are cleared first.
    int backward(float alpha, TensorF& output, TensorF& d_output, TensorF& input, float beta, TensorF& d_input,
                 bool skip_halo_exchange = false)
    {
        if (d_input.get_local_size() == 0)
            return 0;
        clear_halos(d_input);
        if (d_output.get_local_size() > 0)
        {
            const dcb_nd_desc xd = input.nd_desc(m_halo_bwd_recv, m_halo_fwd_recv), yd = output.nd_desc();
            util::check(dcb_pool_bwd(&m_pd, &xd, &yd, alpha, output.get_base_ptr(), d_output.get_base_ptr(),
                                     input.nd_ptr(m_halo_bwd_recv), beta, d_input.nd_ptr(m_halo_bwd_recv), m_ws,
                                     m_ws_bytes, m_be.get_stream()),
                        "pooling backward");
        }
        if (!skip_halo_exchange)
        {
            if (m_be.profiling())
                util::profile_range_push("pooling/exchange_halo_rev");
            m_halo_xch_d_input->exchange(m_be.get_stream(), true, false, tensor::HaloExchangeAccumOp::SUM);
            if (m_be.profiling())
                util::profile_range_pop();
        }
        return 0;
    }

    void wait() { m_be.wait(); }
    tensor::HaloExchange<>& input_halo_exchange() { return *m_halo_xch_input; }
    tensor::HaloExchange<>& d_input_halo_exchange() { return *m_halo_xch_d_input; }

private:
    void clear_halos(TensorF& t)
    {
        const auto& d = t.get_distribution();
        for (int dim = 0; dim < m_nsd; ++dim)
            if (d.is_distributed(dim) && d.get_locale_shape()[dim] > 1 && d.get_overlap(dim) > 0)
                t.clear_halo(dim, m_be.get_stream());
    }
    BackendDNNLib& m_be;
    int m_num_dims, m_nsd;
    void release_workspace()
    {
        if (m_ws)
            cudaFree(m_ws);
        m_ws = nullptr;
        m_ws_bytes = 0;
    }
    dcb_pool_desc m_pd;
    void* m_ws = nullptr;
    int64_t m_ws_bytes = 0;
    tensor::IntVector m_halo_fwd_send, m_halo_bwd_send, m_halo_fwd_recv, m_halo_bwd_recv;
    std::unique_ptr<tensor::HaloExchange<>> m_halo_xch_input, m_halo_xch_d_input;
};

// LeakyReLU<BackendDNNLib> (leaky_relu.hpp; leaky_relu.cu:14-41)
class LeakyReLU
{
public:
    explicit LeakyReLU(BackendDNNLib& backend) : m_be(backend) {}
    int forward(TensorF& input, float negative_slope, TensorF& output)
    {
        if (input.get_local_size() == 0)
            return 0;
        const dcb_nd_desc xd = input.nd_desc(), yd = output.nd_desc();
        util::check(dcb_leaky_relu_fwd(&xd, input.get_base_ptr(), negative_slope, &yd, output.get_base_ptr(),
                                       m_be.get_stream()),
                    "leaky relu");
        return 0;
    }
    int backward(TensorF& input, TensorF& d_output, float negative_slope, TensorF& d_input)
    {
        if (input.get_local_size() == 0)
            return 0;
        const dcb_nd_desc xd = input.nd_desc(), dyd = d_output.nd_desc(), dxd = d_input.nd_desc();
        util::check(dcb_leaky_relu_bwd(&xd, input.get_base_ptr(), &dyd, d_output.get_base_ptr(), negative_slope,
                                       &dxd, d_input.get_base_ptr(), m_be.get_stream()),
                    "leaky relu backward");
        return 0;
    }

private:
    BackendDNNLib& m_be;
};

// ---- dump_tensor / dump_local_tensor (legacy/include/distconv/distconv.hpp:581-671)
// rank 0 writes the GLOBAL tensor, dimension 0 fastest, halos and row padding
// stripped: raw floats to <path>.out (binary) or one value per line to
// <path>.txt, the formats the reference's validation scripts read.  The owned
// blocks travel through the locale's allgather (a debugging aid: every rank
// holds all blocks for a moment).
namespace internal
{
// this rank's owned cells, dense, dimension 0 fastest
inline std::vector<float> owned_cells_to_host(TensorF& t)
{
    const int nd = t.get_num_dims();
    const tensor::Shape pitched = t.get_local_pitched_shape();
    const tensor::Shape& loc = t.get_local_shape();
    std::vector<float> shard((size_t) pitched.get_size()), dense((size_t) loc.get_size());
    if (dense.empty() || t.get_buffer() == nullptr)
        return dense;
    cudaMemcpy(shard.data(), t.get_buffer(), shard.size() * sizeof(float), cudaMemcpyDeviceToHost);
    const tensor::Shape st = t.get_strides();
    tensor::IndexVector idx(nd, 0);
    const index_t rows = loc.get_size() / loc[0];
    for (index_t r = 0; r < rows; ++r)
    {
        index_t off = 0, rem = r;
        for (int i = 1; i < nd; ++i)
        {
            idx[i] = rem % loc[i];
            rem /= loc[i];
            off += (idx[i] + t.get_overlap()[i]) * st[i];
        }
        std::memcpy(&dense[(size_t) r * loc[0]], &shard[(size_t) off + t.get_overlap()[0]],
                    (size_t) loc[0] * sizeof(float));
    }
    return dense;
}
inline void write_floats(const std::string& path, const float* buf, size_t n, bool binary)
{
    std::ofstream out;
    if (!binary)
    {
        out.open(path, std::ios::out | std::ios::trunc);
        for (size_t i = 0; i < n; ++i)
            out << buf[i] << std::endl;
    }
    else
    {
        out.open(path, std::ios::out | std::ios::trunc | std::ios::binary);
        out.write(reinterpret_cast<const char*>(buf), (std::streamsize) (n * sizeof(float)));
    }
}
} // namespace internal

inline int dump_tensor(TensorF& t, std::string file_path, bool binary = false)
{
    file_path += binary ? ".out" : ".txt";
    const tensor::LocaleMPI& loc = t.get_locale();
    const int n = loc.get_size(), nd = t.get_num_dims();
    // every rank contributes a block of the same size: the largest shard
    size_t cells = 0;
    std::vector<dcb_box> boxes((size_t) n);
    for (int r = 0; r < n; ++r)
    {
        boxes[r] = tensor::owned_box(t, r);
        size_t c = 1;
        for (int i = 0; i < nd; ++i)
            c *= (size_t) boxes[r].ext[i];
        cells = std::max(cells, c);
    }
    std::vector<float> mine = internal::owned_cells_to_host(t);
    if (!t.is_split_root())
        mine.clear(); // a replica: rank's box is empty
    mine.resize(cells, 0.f);
    std::vector<float> all((size_t) n * cells);
    loc.allgather(mine.data(), all.data(), cells * sizeof(float));
    if (loc.get_rank() != 0)
        return 0;
    util::MPIPrintStreamDebug() << "Dumping a tensor of shape " << t.get_shape()[0] << " x ... to " << file_path;
    std::vector<float> global((size_t) t.get_size(), 0.f);
    const tensor::Shape gst = tensor::get_strides(t.get_shape());
    for (int r = 0; r < n; ++r)
    {
        const dcb_box& b = boxes[r];
        size_t c = 1;
        for (int i = 0; i < nd; ++i)
            c *= (size_t) b.ext[i];
        if (c == 0)
            continue;
        const float* src = &all[(size_t) r * cells];
        const size_t rows = c / (size_t) b.ext[0];
        for (size_t row = 0; row < rows; ++row)
        {
            size_t rem = row;
            index_t off = b.off[0];
            for (int i = 1; i < nd; ++i)
            {
                off += (b.off[i] + (index_t) (rem % (size_t) b.ext[i])) * gst[i];
                rem /= (size_t) b.ext[i];
            }
            std::memcpy(&global[(size_t) off], src + row * (size_t) b.ext[0], (size_t) b.ext[0] * sizeof(float));
        }
    }
    internal::write_floats(file_path, global.data(), global.size(), binary);
    return 0;
}

// every rank writes its own owned cells to <path>_<rank>.out / .txt
inline int dump_local_tensor(TensorF& t, std::string file_path, bool binary = false)
{
    file_path += "_" + std::to_string(t.get_locale().get_rank()) + (binary ? ".out" : ".txt");
    const std::vector<float> mine = internal::owned_cells_to_host(t);
    internal::write_floats(file_path, mine.data(), mine.size(), binary);
    return 0;
}

// the channel / sample dimensions of a tensor in DistConv's order (distconv.hpp:103-109)
inline int get_channel_dim()
{
    return -2;
}
inline int get_sample_dim()
{
    return -1;
}
// Every rank keeps whole samples: the distribution of sample-parallel layers
// (distconv.hpp make_sample_distribution).
inline tensor::Distribution make_sample_distribution(int num_dims, int num_ranks)
{
    tensor::Shape ls(num_dims, 1);
    ls[-1] = num_ranks;
    return tensor::Distribution::make_distribution(ls);
}

} // namespace distconv
