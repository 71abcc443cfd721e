// Convolution front end: plan, geometry validation, kernel selection, bias.
#include "conv_simt.cuh"
#include "conv_tc.cuh"

using namespace dcb;

struct dcb_conv_plan
{
    dcb_conv_desc cd;
    dcb_nd_desc xd, yd;
    ConvGeom g;
    float* workspace = nullptr; // backward-filter partials
    size_t workspace_bytes = 0;
    float* wflip = nullptr; // flipped/transposed filter for backward data
    TcPlan* tc = nullptr;   // tensor-core state (packed filters), may be null
    int kind[3] = {0, 0, 0};
    bool bwd_data_as_fwd = false;
};

namespace
{

int32_t build_geom(const dcb_conv_desc& cd, const dcb_nd_desc& xd,
                   const dcb_nd_desc& yd, ConvGeom* g)
{
    DCB_REQUIRE(cd.nsd == 2 || cd.nsd == 3, "nsd must be 2 or 3");
    DCB_REQUIRE(xd.nsd == cd.nsd && yd.nsd == cd.nsd, "descriptor nsd mismatch");
    DCB_REQUIRE(cd.groups == 1, "grouped convolution is not supported");
    DCB_REQUIRE(cd.k > 0 && cd.c > 0, "channel counts must be positive");
    DCB_REQUIRE(xd.c == cd.c && yd.c == cd.k, "channel counts do not match");
    DCB_REQUIRE(xd.n == yd.n, "sample counts do not match");
    DCB_REQUIRE(xd.strides[2] == 1 || xd.dims[2] <= 1, "W must be unit-stride");
    DCB_REQUIRE(yd.strides[2] == 1 || yd.dims[2] <= 1, "W must be unit-stride");
    g->n = (int) xd.n;
    g->c = cd.c;
    g->k = cd.k;
    for (int i = 0; i < 3; ++i)
    {
        DCB_REQUIRE(cd.filter[i] >= 1 && cd.strides[i] >= 1
                        && cd.dilations[i] >= 1 && cd.pads[i] >= 0,
                    "bad filter / stride / dilation / pad");
        DCB_REQUIRE(xd.dims[i] < (1ll << 30) && yd.dims[i] < (1ll << 30),
                    "extent too large");
        g->in[i] = (int) xd.dims[i];
        g->out[i] = (int) yd.dims[i];
        g->f[i] = cd.filter[i];
        g->pad[i] = cd.pads[i];
        g->stride[i] = cd.strides[i];
        g->dil[i] = cd.dilations[i];
        g->xs[i] = xd.strides[i];
        g->ys[i] = yd.strides[i];
        const long long df = cd.filter[i] + (cd.filter[i] - 1ll) * (cd.dilations[i] - 1);
        const long long span = xd.dims[i] + 2ll * cd.pads[i] - df;
        const long long expect = span < 0 ? 0 : span / cd.strides[i] + 1;
        DCB_REQUIRE(yd.dims[i] == expect,
                    "output extent does not match input, pad, stride, filter");
    }
    if (cd.nsd == 2)
        DCB_REQUIRE(cd.filter[0] == 1 && cd.pads[0] == 0 && cd.strides[0] == 1,
                    "slot 0 must be trivial for 2-D");
    g->xs_n = xd.sn;
    g->xs_c = xd.sc;
    g->ys_n = yd.sn;
    g->ys_c = yd.sc;
    return DCB_OK;
}

// The forward-shaped problem that computes backward data when all strides
// are 1: input = dy, output = dx, filter flipped and transposed,
// pad' = dilated_extent - 1 - pad.
ConvGeom bwd_as_fwd_geom(const ConvGeom& g)
{
    ConvGeom r = g;
    r.c = g.k;
    r.k = g.c;
    for (int i = 0; i < 3; ++i)
    {
        r.in[i] = g.out[i];
        r.out[i] = g.in[i];
        r.pad[i] = (g.f[i] - 1) * g.dil[i] - g.pad[i];
        r.xs[i] = g.ys[i];
        r.ys[i] = g.xs[i];
    }
    r.xs_n = g.ys_n;
    r.xs_c = g.ys_c;
    r.ys_n = g.xs_n;
    r.ys_c = g.xs_c;
    return r;
}

} // namespace

extern "C" {

int32_t dcb_conv_plan_create(const dcb_conv_desc* cd, const dcb_nd_desc* xd,
                             const dcb_nd_desc* yd, dcb_conv_plan** out)
{
    DCB_REQUIRE(cd && xd && yd && out, "null argument");
    auto* p = new dcb_conv_plan();
    p->cd = *cd;
    p->xd = *xd;
    p->yd = *yd;
    int32_t st = build_geom(*cd, *xd, *yd, &p->g);
    if (st != DCB_OK)
    {
        delete p;
        return st;
    }
    const ConvGeom& g = p->g;
    p->bwd_data_as_fwd = true;
    for (int i = 0; i < 3; ++i)
        if (g.stride[i] != 1 || (g.f[i] - 1) * g.dil[i] - g.pad[i] < 0)
            p->bwd_data_as_fwd = false;
    const size_t fbytes =
        (size_t) g.k * g.c * g.f[0] * g.f[1] * g.f[2] * sizeof(float);
    p->workspace_bytes = simt_conv_bwd_filter_workspace(g);
    bool ok = cudaMalloc(&p->workspace, p->workspace_bytes ? p->workspace_bytes : 16)
              == cudaSuccess;
    ok = ok && cudaMalloc(&p->wflip, fbytes ? fbytes : 16) == cudaSuccess;
    if (!ok)
    {
        (void) cudaGetLastError();
        set_last_error("cudaMalloc of convolution workspace failed");
        cudaFree(p->workspace);
        cudaFree(p->wflip);
        delete p;
        return DCB_CUDA_ERROR;
    }
    if (cd->math_mode != DCB_MATH_FP32_SIMT)
    {
        // Tensor-core kernels where the geometry fits; otherwise the fp32
        // CUDA-core kernels stay selected.
        st = tc_plan_create(g, p->bwd_data_as_fwd ? bwd_as_fwd_geom(g) : g,
                            p->bwd_data_as_fwd, cd->math_mode, &p->tc);
        if (st != DCB_OK)
        {
            cudaFree(p->workspace);
            cudaFree(p->wflip);
            delete p;
            return st;
        }
        if (p->tc)
        {
            p->kind[0] = tc_supports(p->tc, 0) ? 1 : 0;
            p->kind[1] = tc_supports(p->tc, 1) ? 1 : 0;
            p->kind[2] = tc_supports(p->tc, 2) ? 1 : 0;
        }
    }
    *out = p;
    return DCB_OK;
}

int32_t dcb_conv_plan_destroy(dcb_conv_plan* p)
{
    if (!p)
        return DCB_OK;
    tc_plan_destroy(p->tc);
    cudaFree(p->workspace);
    cudaFree(p->wflip);
    delete p;
    return DCB_OK;
}

int32_t dcb_conv_plan_status(dcb_conv_plan* p, void* stream)
{
    DCB_REQUIRE(p, "null argument");
    DCB_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    int* word = tc_status_word(p->tc);
    if (!word)
        return DCB_OK;
    int st = 0;
    DCB_CUDA_TRY(cudaMemcpy(&st, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0)
    {
        DCB_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
        set_last_error("a tensor-core convolution kernel gave up on a pipeline wait");
        return DCB_CUDA_ERROR;
    }
    return DCB_OK;
}

int32_t dcb_conv_plan_kernel_kind(const dcb_conv_plan* p, int32_t which)
{
    if (!p || which < 0 || which > 2)
        return -1;
    return p->kind[which];
}

int32_t dcb_conv_plan_kernel_variant(const dcb_conv_plan* p, int32_t which)
{
    if (!p || which < 0 || which > 2)
        return -1;
    return p->kind[which] == 1 ? tc_variant(p->tc, which) : 0;
}

int32_t dcb_conv_fwd(dcb_conv_plan* p, double alpha, const void* x,
                     const void* w, double beta, void* y, void* stream)
{
    DCB_REQUIRE(p && x && w && y, "null argument");
    if (p->kind[0] == 1)
        return tc_conv_fwd(p->tc, 0, (float) alpha,
                           static_cast<const float*>(x),
                           static_cast<const float*>(w), (float) beta,
                           static_cast<float*>(y), as_stream(stream));
    return simt_conv_fwd(p->g, (float) alpha, static_cast<const float*>(x),
                         static_cast<const float*>(w), (float) beta,
                         static_cast<float*>(y), as_stream(stream));
}

int32_t dcb_conv_fwd_stats(dcb_conv_plan* p, double alpha, const void* x,
                           const void* w, void* y, void* sums, void* sqsums,
                           void* stream)
{
    DCB_REQUIRE(p && x && w && y && sums && sqsums, "null argument");
    if (p->kind[0] != 1)
        return DCB_UNSUPPORTED;
    return tc_conv_fwd_stats(p->tc, (float) alpha, static_cast<const float*>(x),
                             static_cast<const float*>(w),
                             static_cast<float*>(y), static_cast<float*>(sums),
                             static_cast<float*>(sqsums), as_stream(stream));
}

int32_t dcb_conv_bwd_data(dcb_conv_plan* p, double alpha, const void* w,
                          const void* dy, double beta, void* dx, void* stream)
{
    DCB_REQUIRE(p && w && dy && dx, "null argument");
    const ConvGeom& g = p->g;
    if (p->bwd_data_as_fwd)
    {
        const int taps = g.f[0] * g.f[1] * g.f[2];
        int32_t st = flip_transpose_filter(static_cast<const float*>(w),
                                           p->wflip, g.k, g.c, taps,
                                           as_stream(stream));
        if (st != DCB_OK)
            return st;
        if (p->kind[1] == 1)
            return tc_conv_fwd(p->tc, 1, (float) alpha,
                               static_cast<const float*>(dy), p->wflip,
                               (float) beta, static_cast<float*>(dx),
                               as_stream(stream));
        return simt_conv_fwd(bwd_as_fwd_geom(g), (float) alpha,
                             static_cast<const float*>(dy), p->wflip,
                             (float) beta, static_cast<float*>(dx),
                             as_stream(stream));
    }
    return simt_conv_bwd_data(g, (float) alpha, static_cast<const float*>(w),
                              static_cast<const float*>(dy), (float) beta,
                              static_cast<float*>(dx), as_stream(stream));
}

int32_t dcb_conv_bwd_filter(dcb_conv_plan* p, double alpha, const void* x,
                            const void* dy, double beta, void* dw,
                            void* stream)
{
    DCB_REQUIRE(p && x && dy && dw, "null argument");
    if (p->kind[2] == 1)
    {
        const int32_t st = tc_conv_bwd_filter(
            p->tc, (float) alpha, static_cast<const float*>(x),
            static_cast<const float*>(dy), (float) beta,
            static_cast<float*>(dw), as_stream(stream));
        if (st != DCB_UNSUPPORTED) // unaligned base pointers take the kernel below
            return st;
    }
    return simt_conv_bwd_filter(p->g, (float) alpha,
                                static_cast<const float*>(x),
                                static_cast<const float*>(dy), (float) beta,
                                static_cast<float*>(dw), p->workspace,
                                as_stream(stream));
}

} // extern "C"

// ---------------------------------------------------------------------------
// bias
// ---------------------------------------------------------------------------
namespace
{

__global__ void bias_fwd_kernel(float alpha, const float* __restrict__ bias,
                                float beta, float* y, long long n, long long c,
                                long long rows, long long rows_inner,
                                long long len, RunStrides s)
{
    const long long plane = blockIdx.y; // n*c
    const long long cc = plane % c, nn = plane / c;
    const float b = alpha * bias[cc];
    const long long total = rows * len;
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x;
         i < total; i += (long long) gridDim.x * blockDim.x)
    {
        const long long r = i / len, e = i - r * len;
        float* yp = y + nn * s.sn + cc * s.sc + (r / rows_inner) * s.s_outer
                    + (r % rows_inner) * s.s_inner + e;
        *yp = b + (beta != 0.f ? beta * *yp : 0.f);
    }
}

__global__ void bias_bwd_kernel(float alpha, const float* __restrict__ dy,
                                float beta, float* dbias, long long n,
                                long long rows, long long rows_inner,
                                long long len, RunStrides s)
{
    const long long cc = blockIdx.x;
    double acc = 0.0;
    const long long total = n * rows * len;
    for (long long i = threadIdx.x; i < total; i += blockDim.x)
    {
        const long long e = i % len;
        const long long r = (i / len) % rows;
        const long long nn = i / (len * rows);
        acc += (double) dy[nn * s.sn + cc * s.sc + (r / rows_inner) * s.s_outer
                           + (r % rows_inner) * s.s_inner + e];
    }
    __shared__ double sm[256];
    sm[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1)
    {
        if ((int) threadIdx.x < o)
            sm[threadIdx.x] += sm[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        dbias[cc] = alpha * (float) sm[0] + (beta != 0.f ? beta * dbias[cc] : 0.f);
}

} // namespace

extern "C" {

int32_t dcb_bias_fwd(double alpha, const void* bias, double beta,
                     const dcb_nd_desc* yd, void* y, void* stream)
{
    int32_t st = check_nd_desc(yd);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(bias && y, "null argument");
    const int level = run_level(*yd);
    DCB_REQUIRE(level >= 0, "W must be unit-stride");
    RunGeom g;
    RunStrides s;
    make_runs(*yd, level, &g, &s);
    if (g.n * g.c * g.rows * g.len == 0)
        return DCB_OK;
    DCB_REQUIRE(g.n * g.c <= 65535, "too many (n, c) planes");
    long long bx = (g.rows * g.len + 1023) / 1024;
    bx = bx > 1024 ? 1024 : bx;
    bias_fwd_kernel<<<dim3((unsigned) bx, (unsigned) (g.n * g.c)), 256, 0,
                      as_stream(stream)>>>(
        (float) alpha, static_cast<const float*>(bias), (float) beta,
        static_cast<float*>(y), g.n, g.c, g.rows, g.rows_inner, g.len, s);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

int32_t dcb_bias_bwd(double alpha, const dcb_nd_desc* yd, const void* dy,
                     double beta, void* dbias, void* stream)
{
    int32_t st = check_nd_desc(yd);
    if (st != DCB_OK)
        return st;
    DCB_REQUIRE(dy && dbias, "null argument");
    const int level = run_level(*yd);
    DCB_REQUIRE(level >= 0, "W must be unit-stride");
    RunGeom g;
    RunStrides s;
    make_runs(*yd, level, &g, &s);
    if (g.c == 0)
        return DCB_OK;
    bias_bwd_kernel<<<(unsigned) g.c, 256, 0, as_stream(stream)>>>(
        (float) alpha, static_cast<const float*>(dy), (float) beta,
        static_cast<float*>(dbias), g.n, g.rows, g.rows_inner, g.len, s);
    DCB_LAUNCH_CHECK();
    return DCB_OK;
}

} // extern "C"
