/*
 * dcb.h -- C ABI of libdistconv_b200: hand-written sm_100a kernels for the
 * DistConv spatially-parallel layer path (halo exchange, convolution forward /
 * backward-data / backward-filter on the halo-extended shard, distributed
 * batch-normalisation).
 *
 * Conventions
 *  - Every entry point returns a dcb_status (int32); nothing aborts and nothing
 *    resets the device.
 *  - Pointers named x, y, dy, ... are DEVICE pointers unless stated otherwise.
 *  - `stream` is a cudaStream_t passed as void*; all work is stream-ordered.
 *  - Tensor dimension order follows DistConv: index 0 is the innermost (W)
 *    dimension, then H, [D], C, N
 *    (legacy/include/distconv/distconv.hpp:103-109).  Memory is NC[D]HW.
 *  - The reference-side interface each entry point stands in for is cited as
 *    <file>:<line> relative to the DiHydrogen source tree.
 */
#ifndef DCB_H_
#define DCB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCB_MAX_DIMS 5
#define DCB_MAX_SPATIAL 3

typedef enum
{
    DCB_OK = 0,
    DCB_BAD_ARG = 1,
    DCB_UNSUPPORTED = 2,
    DCB_CUDA_ERROR = 3,
    DCB_PEER_TIMEOUT = 4,
    DCB_NCCL_ERROR = 5,
    DCB_NOT_CONNECTED = 6
} dcb_status;

/* Human-readable name of a status code; never NULL. */
const char* dcb_status_string(int32_t status);
/* Message of the last failing CUDA / NCCL call on the calling thread. */
const char* dcb_last_error(void);
/* Library version: major*10000 + minor*100 + patch. */
int32_t dcb_version(void);

/* ------------------------------------------------------------------------
 * Tensor shard descriptor.  Mirrors what the reference derives from a
 * tensor::Tensor<T, LocaleMPI, CUDAAllocator>: get_local_shape(),
 * get_local_real_shape() (= local + 2*overlap in partitioned dimensions) and
 * the distribution's overlap (legacy/include/distconv/tensor/tensor.hpp:171-178,
 * tensor_mpi.hpp:489-498).  The buffer a descriptor describes starts at the
 * first cell of the halo-extended shard (Tensor::get_buffer()).
 *
 * `pitch` is the distance in elements between consecutive rows (index 1) of
 * the buffer, Tensor::get_pitch() of a shard allocated with the reference's
 * CUDAPitchedAllocator (tensor/memory_cuda.hpp:68-104, tensor.hpp:184-192,
 * 483-485): 0 or real_shape[0] for a dense shard, larger when rows are padded.
 * A W-partitioned shard with halo 1 has 258-float rows, which no bulk copy
 * (TMA) can address: the pitch must be a multiple of 4 floats for the
 * tensor-core kernels to take the shard.  The host mirrors lay such a shard out
 * with a pitch of 264 and the buffer starting 3 floats above a 16-byte boundary,
 * so that the OWNED cells of every row start on one: bulk stores into the
 * interior (backward data) and 16-byte vector accesses (batch-norm) need that,
 * while the kernels that read the halo-extended window fetch from the boundary
 * below it and skip the cells in front (they are only read, and lie in the same
 * allocation since allocations start 16-byte aligned).  Any base alignment of 4
 * bytes is accepted; other layouts run on slower paths.  The padding cells
 * between rows belong to nobody: kernels may copy them along with a face but
 * never interpret them, and nothing is accessed beyond the last row's last real
 * cell.
 * ------------------------------------------------------------------------ */
typedef struct dcb_tensor_desc
{
    int32_t ndims; /* 4 or 5 */
    int32_t dtype; /* DCB_F32 */
    int64_t local_shape[DCB_MAX_DIMS];
    int64_t real_shape[DCB_MAX_DIMS];
    int32_t overlap[DCB_MAX_DIMS];
    int64_t pitch; /* row pitch in elements; 0 = real_shape[0] */
} dcb_tensor_desc;

#define DCB_F32 0

/* ------------------------------------------------------------------------
 * Halo exchange.
 * Stands in for tensor::HaloExchange<T, CUDAAllocator, AlBackend> and its six
 * transports (legacy/include/distconv/tensor/halo_exchange_cuda.hpp:18-423,
 * halo_exchange_cuda_{al,mpi,p2p,hybrid,nvshmem}.hpp) and for TraverseHalo +
 * PackFunctor (halo_cuda.hpp:898-1008, halo_packing_cuda.hpp:60-167).
 *
 * One transport: the pack kernel reads the strided face slab and stores it
 * directly into the neighbour's receive slab (peer-mapped memory, NVLink), then
 * publishes an epoch flag; the neighbour's unpack kernel waits on that flag
 * with a bounded budget and scatters the slab into its halo cells.
 * ------------------------------------------------------------------------ */
typedef struct dcb_halo_plan dcb_halo_plan;

#define DCB_LHS 0
#define DCB_RHS 1

/* flags for exchange / pack_put / wait_unpack */
#define DCB_HALO_REVERSE 0x1u     /* pack halo cells, accumulate into owned cells */
#define DCB_HALO_SKIP_UNPACK 0x2u /* start only; call dcb_halo_unpack later */
#define DCB_HALO_CLEAR_BOUNDARY 0x4u /* forward exchange: the pack launch of a
                                        dimension also zeroes that dimension's halo
                                        slabs that have no neighbour (the boundary of
                                        the global tensor), instead of a separate
                                        dcb_clear_halo pass before the exchange */
#define DCB_HALO_OP_SHIFT 4
#define DCB_HALO_OP_ID (0u << DCB_HALO_OP_SHIFT)
#define DCB_HALO_OP_SUM (1u << DCB_HALO_OP_SHIFT)
#define DCB_HALO_OP_MAX (2u << DCB_HALO_OP_SHIFT)
#define DCB_HALO_OP_MIN (3u << DCB_HALO_OP_SHIFT)

/* Size in bytes of the opaque blob a plan exports for its peers. */
#define DCB_HALO_BLOB_BYTES 256

/* peers[2*dim + side] is the rank of the neighbour on that side of that
 * dimension or -1 (MPI_PROC_NULL in HaloExchange::find_peer_rank,
 * halo_exchange_cuda.hpp:322-357).  Allocates this rank's receive slabs
 * (double-buffered), zero-filled (halo_exchange_cuda.hpp:285-303). */
int32_t dcb_halo_plan_create(const dcb_tensor_desc* desc, const int32_t* peers,
                             int32_t rank, dcb_halo_plan** plan);
int32_t dcb_halo_plan_destroy(dcb_halo_plan* plan);
/* Write this plan's blob (memory handle + slab offsets) to host memory. */
int32_t dcb_halo_plan_export(dcb_halo_plan* plan, void* blob);
/* blobs: nranks * DCB_HALO_BLOB_BYTES host bytes, indexed by rank, gathered
 * by the caller (MPI_Allgather, torch.distributed, ...).  Maps the receive
 * slabs of every neighbour.  Replaces the P2P connection set-up of
 * legacy/src/p2p/connection_ipc.cpp. */
int32_t dcb_halo_plan_connect(dcb_halo_plan* plan, const void* blobs,
                              int32_t nranks);
/* Budget of every device-side wait on a peer flag, in nanoseconds
 * (default 2e9).  On expiry the kernel records DCB_PEER_TIMEOUT and returns. */
int32_t dcb_set_wait_budget_ns(int64_t ns);

/* One dimension, pack + put to both neighbours
 * (HaloExchange::exchange(dim, ...) first half, halo_exchange_cuda_al.hpp:29-62). */
int32_t dcb_halo_pack_put(dcb_halo_plan* plan, const void* tensor, int32_t dim,
                          uint32_t flags, void* stream);
/* One dimension, wait for both neighbours' slabs and unpack them
 * (HaloExchange::unpack(dim, ...), halo_exchange_cuda.hpp:395-422). */
int32_t dcb_halo_wait_unpack(dcb_halo_plan* plan, void* tensor, int32_t dim,
                             uint32_t flags, void* stream);
/* All dimensions in order 0,1,2 (HaloExchange::exchange(comms, stream, ...),
 * halo_exchange_cuda.hpp:56-126).  With DCB_HALO_SKIP_UNPACK only the pack+put
 * half runs for every dimension; corners then need dcb_halo_unpack before the
 * next dimension's data is consumed, exactly as in the reference. */
int32_t dcb_halo_exchange(dcb_halo_plan* plan, void* tensor, uint32_t flags,
                          void* stream);
/* Deferred unpack of a DCB_HALO_SKIP_UNPACK exchange
 * (HaloExchange::unpack(streams, ...), halo_exchange_cuda.hpp:148-202). */
int32_t dcb_halo_unpack(dcb_halo_plan* plan, void* tensor, uint32_t flags,
                        void* stream);
/* Synchronises `stream`, then returns DCB_PEER_TIMEOUT if any wait of this
 * plan ran out since the last call (and clears the record), else DCB_OK. */
int32_t dcb_halo_plan_status(dcb_halo_plan* plan, void* stream);
/* Zero both outer slabs of `dim` (Tensor::clear_halo,
 * legacy/src/tensor/tensor_mpi_cuda.cu:14-82).  dim < 0 clears every
 * dimension that has an overlap. */
int32_t dcb_clear_halo(const dcb_tensor_desc* desc, void* tensor, int32_t dim,
                       void* stream);
/* Plain pack / unpack of one slab into / from a caller-provided dense device
 * buffer (TraverseHalo with PackFunctor, halo_packing_cuda.hpp:85-167).
 * inner != 0 selects the owned cells next to the boundary, 0 the halo cells.
 * op is one of DCB_HALO_OP_* and is used by unpack only. */
int32_t dcb_halo_pack(const dcb_tensor_desc* desc, const void* tensor,
                      int32_t dim, int32_t side, int32_t width, int32_t inner,
                      void* packed, void* stream);
int32_t dcb_halo_unpack_slab(const dcb_tensor_desc* desc, void* tensor,
                             int32_t dim, int32_t side, int32_t width,
                             int32_t inner, const void* packed, uint32_t op,
                             void* stream);

/* ------------------------------------------------------------------------
 * Convolution.  Stands in for the cuDNN calls behind
 * GPUDNNBackend::convolution_forward / _bwd_data / _bwd_filter
 * (legacy/src/dnn_backend/dnn_backend_cudnn.cpp.inc:245-333) on descriptors
 * built by setup_tensor_descriptor (dnn_backend_impl.hpp:31-70) and
 * Convolution::setup_convolution_descriptor (convolution.hpp:2541-2670).
 * Cross-correlation, y = alpha*op + beta*y.
 * ------------------------------------------------------------------------ */
typedef struct dcb_nd_desc
{
    int32_t nsd;                   /* 2 or 3 spatial dims */
    int64_t n, c;                  /* samples, channels */
    int64_t dims[DCB_MAX_SPATIAL]; /* D,H,W (outermost first); D=1 if nsd==2 */
    int64_t sn, sc;                /* element strides of n and c */
    int64_t strides[DCB_MAX_SPATIAL];
} dcb_nd_desc;

#define DCB_MATH_FP32 0      /* fp32 result quality: 3xTF32 on tensor cores, or
                                fp32 FMA where no tensor-core kernel applies */
#define DCB_MATH_TF32 1      /* single TF32 pass */
#define DCB_MATH_FP32_SIMT 2 /* force the fp32 CUDA-core kernels */
#define DCB_MATH_BF16 3      /* bf16 operands, fp32 accumulation: inputs and filters are
                                rounded to bf16 (ties away from zero) on their way into the
                                tensor-core kernels and multiplied in one pass; a bf16 value
                                is a TF32 value, so the TF32 instruction computes exactly what
                                a bf16 one would.  Backward filter keeps fp32 quality.  Shapes
                                without a tensor-core kernel run the fp32 CUDA-core kernels. */

typedef struct dcb_conv_desc
{
    int32_t nsd;
    int32_t k, c;                     /* filters, input channels */
    int32_t filter[DCB_MAX_SPATIAL];  /* fd,fh,fw (fd=1 if nsd==2) */
    int32_t pads[DCB_MAX_SPATIAL];
    int32_t strides[DCB_MAX_SPATIAL];
    int32_t dilations[DCB_MAX_SPATIAL];
    int32_t groups;                   /* only 1 */
    int32_t math_mode;
} dcb_conv_desc;

typedef struct dcb_conv_plan dcb_conv_plan;

/* Validates the geometry, picks kernels and allocates the backward-filter
 * split-reduction workspace (the reference borrows workspace per call from a
 * caching pool, convolution.hpp:394-398). */
int32_t dcb_conv_plan_create(const dcb_conv_desc* cd, const dcb_nd_desc* xd,
                             const dcb_nd_desc* yd, dcb_conv_plan** plan);
int32_t dcb_conv_plan_destroy(dcb_conv_plan* plan);
/* w is dense [K][C][fd][fh][fw]. */
int32_t dcb_conv_fwd(dcb_conv_plan* plan, double alpha, const void* x,
                     const void* w, double beta, void* y, void* stream);
/* y = alpha * conv(x, w), and from the same pass sums[k] = sum of y over filter
 * k's outputs, sqsums[k] = sum of y^2: what dcb_bn_stats(y) returns, taken from
 * the epilogue's registers so that a batch-norm that follows need not read y
 * for its statistics (the reference runs cuDNN's convolution and then
 * channel_sums_and_sqsums, batchnorm.cu:192-249, as separate passes; this fuses
 * them, convolution.hpp:342-639 + batchnorm.hpp:171-183).  Each lane adds its
 * outputs in fp32, the per-warp partials are folded in a fixed order in fp64.
 * DCB_UNSUPPORTED, with nothing launched, when the plan's kernel for this
 * problem has no such epilogue: call dcb_conv_fwd and dcb_bn_stats then. */
int32_t dcb_conv_fwd_stats(dcb_conv_plan* plan, double alpha, const void* x,
                           const void* w, void* y, void* sums, void* sqsums,
                           void* stream);
int32_t dcb_conv_bwd_data(dcb_conv_plan* plan, double alpha, const void* w,
                          const void* dy, double beta, void* dx, void* stream);
int32_t dcb_conv_bwd_filter(dcb_conv_plan* plan, double alpha, const void* x,
                            const void* dy, double beta, void* dw,
                            void* stream);
/* Synchronises `stream`, then reports whether a tensor-core kernel of this
 * plan gave up on one of its bounded pipeline waits since the last call
 * (DCB_CUDA_ERROR, record cleared) or not (DCB_OK).  Such a launch leaves its
 * output incomplete. */
int32_t dcb_conv_plan_status(dcb_conv_plan* plan, void* stream);
/* Which kernel family the plan resolved to for (0 fwd, 1 bwd-data,
 * 2 bwd-filter): 0 = fp32 CUDA-core, 1 = tcgen05 tensor-core. */
int32_t dcb_conv_plan_kernel_kind(const dcb_conv_plan* plan, int32_t which);
/* The kernel the plan prefers for that pass (cuDNN reports its choice as an
 * algorithm enum, util_cudnn.hpp:37-60): 0 fp32 CUDA-core; tcgen05 kernels:
 * 1 row kernel fed by bulk tensor copies, 2 row kernel whose converter warps
 * fetch their own rows (strides not multiples of 16 bytes), 3 sweep kernel
 * (filters with depth), 4 multi-group sweep kernel, 5 backward-filter kernel.
 * A call whose base pointers are not 16-byte aligned may still step down
 * (3/4 -> 2, 5 -> 0). */
int32_t dcb_conv_plan_kernel_variant(const dcb_conv_plan* plan, int32_t which);
/* y[n,k,...] = alpha*bias[k] + beta*y (cudnnAddTensor,
 * dnn_backend_cudnn.cpp.inc:386) and its gradient dbias[k] = alpha*sum dy +
 * beta*dbias (cudnnConvolutionBackwardBias, :397). */
int32_t dcb_bias_fwd(double alpha, const void* bias, double beta,
                     const dcb_nd_desc* yd, void* y, void* stream);
int32_t dcb_bias_bwd(double alpha, const dcb_nd_desc* yd, const void* dy,
                     double beta, void* dbias, void* stream);

/* ------------------------------------------------------------------------
 * Batch normalisation.  Stands in for the kernels of
 * legacy/src/dnn_backend/batchnorm.cu reached from
 * BatchNormalization<BackendDNNLib,T>::forward_stage1/2, backward_stage1/2
 * (legacy/include/distconv/dnn_backend/batchnorm.hpp:171-250, 335-430).
 * Statistics vectors are C contiguous floats.
 * ------------------------------------------------------------------------ */
typedef struct dcb_bn_plan dcb_bn_plan;
/* Owns the fixed-order two-stage reduction scratch for tensors of this shape. */
int32_t dcb_bn_plan_create(const dcb_nd_desc* xd, dcb_bn_plan** plan);
int32_t dcb_bn_plan_destroy(dcb_bn_plan* plan);
/* sums[c] = sum x, sqsums[c] = sum x^2 over the cells xd describes
 * (channel_sums_and_sqsums, batchnorm.cu:192-249).  Overwrites. */
int32_t dcb_bn_stats(dcb_bn_plan* plan, const void* x, void* sums,
                     void* sqsums, void* stream);
/* The same statistics for callers that must not trigger a device allocation
 * (no counterpart in the reference; added for hosts whose allocator owns the
 * whole GPU, for code running inside a stream capture, and for loops that
 * cannot afford cudaMalloc's device-wide synchronisation).  Needs no plan: the
 * reduction scratch is a fixed 68 KiB array inside the library image, present
 * on every GPU that loads the library.  Limits: at most 1024 channels
 * (DCB_UNSUPPORTED beyond).  The first call on each device looks up the
 * array's device address; make that call outside any stream capture.  All
 * calls share the one array, so two calls whose kernels may overlap on the
 * same GPU (different streams) race: serialise them.  The looked-up address is
 * kept per device ordinal for the life of the process: it does not survive a
 * cudaDeviceReset.  Results equal those of dcb_bn_stats. */
int32_t dcb_bn_stats_noalloc(const dcb_nd_desc* xd, const void* x, void* sums,
                             void* sqsums, void* stream);
/* In place sums -> mean, sqsums -> unbiased variance, update running stats
 * (sums_to_statistics, batchnorm.cu:288-346).  num_per_sum <= 0 sets var=1. */
int32_t dcb_bn_finalize(int32_t channels, int64_t num_per_sum, float decay,
                        void* mean, void* var, void* running_mean,
                        void* running_var, void* stream);
/* y = scale*(x-mean)*rsqrt(var+eps)+bias (batch_normalization,
 * batchnorm.cu:369-455).  yd may differ from xd in strides only. */
int32_t dcb_bn_apply(const dcb_nd_desc* xd, const void* x, const void* mean,
                     const void* var, const void* scale, const void* bias,
                     float eps, const dcb_nd_desc* yd, void* y, void* stream);
/* dcb_bn_apply followed by the leaky ReLU y > 0 ? y : slope*y in the same pass
 * (batch_normalization, batchnorm.cu:369-455, then leaky_relu.cu:14-25): saves
 * one read and one write of the tensor where a LeakyReLU follows the batch-norm. */
int32_t dcb_bn_apply_leaky_relu(const dcb_nd_desc* xd, const void* x,
                                const void* mean, const void* var,
                                const void* scale, const void* bias, float eps,
                                float slope, const dcb_nd_desc* yd, void* y,
                                void* stream);
/* Local dscale, dbias, dmean, dvar (backprop1, batchnorm.cu:899-1054).
 * Overwrites the four C-vectors. */
int32_t dcb_bn_bwd_reduce(dcb_bn_plan* plan, const void* x,
                          const dcb_nd_desc* dyd, const void* dy,
                          const void* mean, const void* var, const void* scale,
                          float eps, void* dscale, void* dbias, void* dmean,
                          void* dvar, void* stream);
/* dx = dy*scale*inv_std + dmean/n + dvar*2/(n-1)*(x-mean) (backprop2,
 * batchnorm.cu:1303-1418). */
int32_t dcb_bn_bwd_apply(const dcb_nd_desc* xd, const void* x,
                         const dcb_nd_desc* dyd, const void* dy,
                         const void* mean, const void* var, const void* scale,
                         const void* dmean, const void* dvar, float eps,
                         int64_t num_per_sum, const dcb_nd_desc* dxd, void* dx,
                         void* stream);
/* y = x > 0 ? x : slope*x, and its gradient (legacy/src/dnn_backend/leaky_relu.cu:14-41). */
int32_t dcb_leaky_relu_fwd(const dcb_nd_desc* xd, const void* x, float slope,
                           const dcb_nd_desc* yd, void* y, void* stream);
int32_t dcb_leaky_relu_bwd(const dcb_nd_desc* xd, const void* x,
                           const dcb_nd_desc* dyd, const void* dy, float slope,
                           const dcb_nd_desc* dxd, void* dx, void* stream);

/* ------------------------------------------------------------------------
 * Pooling.  Stands in for cudnnPoolingForward / cudnnPoolingBackward behind
 * GPUDNNBackend::pooling_forward / _backward as Pooling<BackendDNNLib,T> calls
 * them (legacy/include/distconv/dnn_backend/pooling.hpp:212-283): xd describes
 * the input window including the halo cells of partitioned dimensions (whose
 * pad is then 0, pooling.hpp:189-194), yd the output.  Modes as
 * pooling::get_pooling_mode maps them (pooling.hpp:27-48).
 * ------------------------------------------------------------------------ */
#define DCB_POOL_MAX 0            /* "MAX" */
#define DCB_POOL_AVERAGE 1        /* "AVERAGE": padding cells count */
#define DCB_POOL_AVERAGE_NO_PAD 2 /* "AVERAGE_NO_PAD" */

typedef struct dcb_pool_desc
{
    int32_t nsd;
    int32_t window[DCB_MAX_SPATIAL]; /* D,H,W (window[0] = 1 if nsd == 2) */
    int32_t pads[DCB_MAX_SPATIAL];
    int32_t strides[DCB_MAX_SPATIAL];
    int32_t mode;
    /* Leading / trailing cells of the x window that lie outside the global
     * tensor: the halo of a rank at the domain boundary in a partitioned,
     * padded dimension.  They are padding (ignored by MAX and by
     * AVERAGE_NO_PAD's count), not data; 0 everywhere else. */
    int32_t outside_lo[DCB_MAX_SPATIAL];
    int32_t outside_hi[DCB_MAX_SPATIAL];
} dcb_pool_desc;

/* y = alpha * pool(x) + beta * y. */
int32_t dcb_pool_fwd(const dcb_pool_desc* pd, const dcb_nd_desc* xd,
                     const dcb_nd_desc* yd, double alpha, const void* x,
                     double beta, void* y, void* stream);
/* dx = alpha * pool'(dy) + beta * dx over the whole x window (halo cells
 * included: a reverse halo exchange with SUM returns them to their owners,
 * pooling.hpp:281).  x and dx share xd, y and dy share yd.  MAX sends a
 * window's gradient to the first cell (scan order D, H, W) equal to y, which
 * must be the unscaled forward result; x and y may be null for the averages.
 * A gather over the input cells: reproducible. */
int32_t dcb_pool_bwd(const dcb_pool_desc* pd, const dcb_nd_desc* xd,
                     const dcb_nd_desc* yd, double alpha, const void* y,
                     const void* dy, const void* x, double beta, void* dx,
                     void* workspace, int64_t workspace_bytes, void* stream);
/* Device bytes dcb_pool_bwd can use for MAX (one byte per output cell; 0 for
 * the averages, -1 for a bad descriptor).  With that workspace the backward
 * pass first records every window's first maximum from x (nothing is kept
 * between calls) and the gather compares one byte per window; without it
 * (null / too small) it scans each window's earlier cells instead, an order of
 * magnitude slower.  The reference borrows cuDNN workspaces from a caching
 * pool per call (convolution.hpp:394-398); here the caller owns it. */
int64_t dcb_pool_bwd_workspace_bytes(const dcb_pool_desc* pd,
                                     const dcb_nd_desc* xd,
                                     const dcb_nd_desc* yd);

/* ------------------------------------------------------------------------
 * Re-distribution between two block decompositions of one global tensor.
 * Stands in for tensor::TensorMPICUDAShuffler
 * (legacy/include/distconv/tensor/shuffle_mpi_cuda.hpp:14-512; forward =
 * shuffle_forward, and a second plan with the tensors swapped =
 * shuffle_backward).  Boxes are in global coordinates, dimension 0 = W; box r
 * is what rank r owns (empty for a rank that is not the root of a replicated
 * dimension, tensor_mpi.hpp is_split_root).  Set-up is two-phase like the halo
 * plan: create on every rank, gather the export blobs, connect.
 * ------------------------------------------------------------------------ */
typedef struct dcb_box
{
    int64_t off[DCB_MAX_DIMS];
    int64_t ext[DCB_MAX_DIMS];
} dcb_box;

typedef struct dcb_shuffle_plan dcb_shuffle_plan;
#define DCB_SHUFFLE_BLOB_BYTES 128

/* src / dst describe the calling rank's shards (halo included, as
 * Tensor::get_buffer() sees them); src_boxes / dst_boxes have nranks entries. */
int32_t dcb_shuffle_plan_create(const dcb_tensor_desc* src,
                                const dcb_tensor_desc* dst,
                                const dcb_box* src_boxes,
                                const dcb_box* dst_boxes, int32_t rank,
                                int32_t nranks, dcb_shuffle_plan** plan);
int32_t dcb_shuffle_plan_destroy(dcb_shuffle_plan* plan);
int32_t dcb_shuffle_plan_export(dcb_shuffle_plan* plan, void* blob);
int32_t dcb_shuffle_plan_connect(dcb_shuffle_plan* plan, const void* blobs,
                                 int32_t nranks);
/* One kernel: this rank's cells go straight into their owners' receive
 * windows (peer stores), then an epoch flag per destination. */
int32_t dcb_shuffle_put(dcb_shuffle_plan* plan, const void* src, void* stream);
/* One kernel: bounded wait for every rank that holds a part of this rank's
 * block, then window -> dst (halo cells untouched).  On expiry nothing is
 * copied and dcb_shuffle_plan_status reports DCB_PEER_TIMEOUT. */
int32_t dcb_shuffle_wait_unpack(dcb_shuffle_plan* plan, void* dst,
                                void* stream);
/* put + wait_unpack (ranks on different GPUs). */
int32_t dcb_shuffle(dcb_shuffle_plan* plan, const void* src, void* dst,
                    void* stream);
int32_t dcb_shuffle_plan_status(dcb_shuffle_plan* plan, void* stream);

/* ------------------------------------------------------------------------
 * All-reduce of small device vectors (BN statistics, filter gradients).
 * Stands in for tensor::Allreduce<T> and its Aluminum/NCCL, MPI-via-host and
 * NVSHMEM implementations (legacy/include/distconv/tensor/allreduce.hpp:8-19,
 * allreduce_al.hpp:12-38, allreduce_mpi_cuda.hpp:14-48,
 * allreduce_nvshmem.hpp:69-280) and for the communicator the reference never
 * constructs (legacy/src/dnn_backend/communicator_manager.cpp:26-57).
 * ------------------------------------------------------------------------ */
typedef struct dcb_comm dcb_comm;
#define DCB_NCCL_ID_BYTES 128
#define DCB_COMM_BLOB_BYTES 128
/* NCCL flavour: rank 0 calls dcb_nccl_unique_id, the caller broadcasts the
 * id, every rank calls dcb_comm_create_nccl. */
int32_t dcb_nccl_unique_id(void* id_out);
int32_t dcb_comm_create_nccl(const void* id, int32_t rank, int32_t nranks,
                             dcb_comm** comm);
/* Peer-memory flavour for short vectors (<= max_count floats): every rank
 * stores its contribution into every peer's mapped slot and each rank sums the
 * slots in rank order, so all ranks get identical bits.  Set-up mirrors the
 * halo plan: create, export, gather blobs, connect. */
int32_t dcb_comm_create_peer(int32_t rank, int32_t nranks, int32_t max_count,
                             dcb_comm** comm);
int32_t dcb_comm_export(dcb_comm* comm, void* blob);
int32_t dcb_comm_connect(dcb_comm* comm, const void* blobs, int32_t nranks);
int32_t dcb_comm_destroy(dcb_comm* comm);
/* In-place sum all-reduce of `count` floats.  The peer flavour takes vectors
 * longer than max_count in max_count-sized pieces, one kernel each (the
 * push / pull halves below do not: they are limited to max_count). */
int32_t dcb_allreduce_sum(dcb_comm* comm, void* data, int64_t count,
                          void* stream);
/* Peer flavour only, for single-device emulation of several ranks: the two
 * halves of the all-reduce as separate launches (push contributions; wait,
 * sum, write back). */
int32_t dcb_allreduce_push(dcb_comm* comm, const void* data, int64_t count,
                           void* stream);
int32_t dcb_allreduce_pull(dcb_comm* comm, void* data, int64_t count,
                           void* stream);
int32_t dcb_comm_status(dcb_comm* comm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DCB_H_ */
