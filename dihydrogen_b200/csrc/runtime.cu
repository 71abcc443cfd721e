// Status strings, error record, device queries and the peer-mapped window.
#include "common.cuh"

#include <unistd.h>

#include <atomic>

namespace dcb
{

static thread_local std::string g_last_error;
static std::atomic<int64_t> g_wait_budget_ns{2000000000ll};

void set_last_error(const std::string& msg)
{
    g_last_error = msg;
}

int64_t wait_budget_ns()
{
    return g_wait_budget_ns.load();
}

int num_sms()
{
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess)
        return cached;
    if (dev != cached_dev)
    {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)
                == cudaSuccess
            && n > 0)
        {
            cached = n;
            cached_dev = dev;
        }
    }
    return cached;
}

int32_t Window::allocate(size_t nbytes)
{
    DCB_CUDA_TRY(cudaGetDevice(&device));
    // Round up so the whole allocation can be zeroed and mapped as one unit.
    bytes = (nbytes + 4095) / 4096 * 4096;
    DCB_CUDA_TRY(cudaMalloc(&base, bytes));
    DCB_CUDA_TRY(cudaMemset(base, 0, bytes));
    DCB_CUDA_TRY(cudaDeviceSynchronize());
    return DCB_OK;
}

int32_t Window::fill_blob(WindowBlob* b) const
{
    std::memset(b, 0, sizeof(*b));
    b->raw_ptr = reinterpret_cast<uint64_t>(base);
    b->bytes = bytes;
    b->pid = (int32_t) getpid();
    b->device = device;
    // The handle is only needed by other processes; failure to create one
    // (e.g. memory type that cannot be shared) is reported when a remote
    // process tries to open it.
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, base) == cudaSuccess)
        b->handle = h;
    else
        (void) cudaGetLastError();
    return DCB_OK;
}

void Window::release()
{
    if (base)
        cudaFree(base);
    base = nullptr;
    bytes = 0;
}

int32_t PeerMapping::open(const WindowBlob& b, int my_device)
{
    if (b.pid == (int32_t) getpid())
    {
        base = reinterpret_cast<void*>(b.raw_ptr);
        opened_ipc = false;
        if (b.device != my_device)
        {
            int can = 0;
            DCB_CUDA_TRY(cudaDeviceCanAccessPeer(&can, my_device, b.device));
            if (!can)
            {
                set_last_error("peer access between devices is not available");
                return DCB_UNSUPPORTED;
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(b.device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
            {
                set_last_error(std::string("cudaDeviceEnablePeerAccess: ")
                               + cudaGetErrorString(e));
                return DCB_CUDA_ERROR;
            }
            (void) cudaGetLastError();
        }
        return DCB_OK;
    }
    DCB_CUDA_TRY(cudaIpcOpenMemHandle(&base, b.handle,
                                      cudaIpcMemLazyEnablePeerAccess));
    opened_ipc = true;
    return DCB_OK;
}

void PeerMapping::close()
{
    if (opened_ipc && base)
        cudaIpcCloseMemHandle(base);
    base = nullptr;
    opened_ipc = false;
}

} // namespace dcb

extern "C" {

const char* dcb_status_string(int32_t s)
{
    switch (s)
    {
    case DCB_OK: return "DCB_OK";
    case DCB_BAD_ARG: return "DCB_BAD_ARG";
    case DCB_UNSUPPORTED: return "DCB_UNSUPPORTED";
    case DCB_CUDA_ERROR: return "DCB_CUDA_ERROR";
    case DCB_PEER_TIMEOUT: return "DCB_PEER_TIMEOUT";
    case DCB_NCCL_ERROR: return "DCB_NCCL_ERROR";
    case DCB_NOT_CONNECTED: return "DCB_NOT_CONNECTED";
    default: return "DCB_UNKNOWN";
    }
}

const char* dcb_last_error(void)
{
    return dcb::g_last_error.c_str();
}

int32_t dcb_version(void)
{
    return 100;
}

int32_t dcb_set_wait_budget_ns(int64_t ns)
{
    if (ns <= 0)
        return DCB_BAD_ARG;
    dcb::g_wait_budget_ns.store(ns);
    return DCB_OK;
}

} // extern "C"
