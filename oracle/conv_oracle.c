/*
 * TEST INFRASTRUCTURE ONLY -- the checker, never the product.  Only tests/,
 * __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this.
 *
 * CPU restatement of the arithmetic on DistConv's conv + batch-norm path.
 *
 * Convolution: the reference hands the halo-extended shard to cuDNN
 * (legacy/src/dnn_backend/dnn_backend_cudnn.cpp.inc:245-333) in
 * cross-correlation mode (legacy/include/distconv/dnn_backend/dnn_backend.hpp:239)
 * with y = alpha*conv + beta*y; cuDNN itself is closed and absent from the
 * reference tree, so the published definition of those three calls
 * (forward, backward-data = adjoint w.r.t. x, backward-filter = adjoint
 * w.r.t. w, on strided NC[D]HW descriptors with symmetric padding, stride
 * and dilation) is restated here with fp64 accumulation.  The only in-tree
 * arithmetic, Convolution<ref::Backend> (legacy/include/distconv/ref/backend.hpp:17-166,
 * 238-365), is the 4-D stride-1 special case; tests compare the two.
 * Parity status: pinned against ref::Backend outputs for 4-D stride-1 cases;
 * unpinned (no stored answers exist in the reference) for 5-D and strided
 * cases, where the definition above is the contract.
 *
 * Batch-norm: formulas of legacy/src/dnn_backend/batchnorm.cu:288-313 (sums to
 * mean / unbiased variance / running statistics), :385-412 (normalise),
 * :920-956 (backprop1: dscale, dbias, dmean, dvar) and :1327-1362 (backprop2:
 * dx).  Sums are accumulated in fp64; the per-element formulas are evaluated
 * in fp32 in the reference's operation order.
 *
 * All tensors are described by five extents (N, C, D, H, W) and five element
 * strides, so a halo-extended shard, or a window into one, is passed without
 * copying.  A 2-D problem uses D = 1.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct
{
    int64_t n, c, d, h, w;      /* extents */
    int64_t sn, sc, sd, sh, sw; /* element strides */
} oracle_tdesc;

typedef struct
{
    int fd, fh, fw;    /* filter extents */
    int pd, ph, pw;    /* symmetric zero padding */
    int sd, sh, sw;    /* strides */
    int dd, dh, dw;    /* dilations */
} oracle_cdesc;

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count for the loops below.  Launchers such as torch.distributed.run
 * export OMP_NUM_THREADS=1; a CPU baseline timed under them sets its count
 * explicitly. */
void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void) n;
#endif
}

static inline size_t off5(const oracle_tdesc* t, int64_t n, int64_t c,
                          int64_t d, int64_t h, int64_t w)
{
    return (size_t) (n * t->sn + c * t->sc + d * t->sd + h * t->sh + w * t->sw);
}

/* y[n,k,o] = alpha * sum_{c,f} x[n,c,o*s - p + f*dil] * w[k,c,f] + beta * y
 * Filter is dense [K][C][fd][fh][fw]. */
void oracle_conv_fwd(const float* x, const oracle_tdesc* xd, const float* w,
                     float* y, const oracle_tdesc* yd, const oracle_cdesc* cd,
                     double alpha, double beta)
{
    const int64_t K = yd->c, C = xd->c;
    const int64_t total = yd->n * K * yd->d;
#pragma omp parallel for schedule(static)
    for (int64_t job = 0; job < total; ++job)
    {
        const int64_t od = job % yd->d;
        const int64_t k = (job / yd->d) % K;
        const int64_t n = job / (yd->d * K);
        for (int64_t oh = 0; oh < yd->h; ++oh)
            for (int64_t ow = 0; ow < yd->w; ++ow)
            {
                double acc = 0.0;
                for (int64_t c = 0; c < C; ++c)
                    for (int kd = 0; kd < cd->fd; ++kd)
                    {
                        const int64_t id = od * cd->sd - cd->pd + kd * cd->dd;
                        if (id < 0 || id >= xd->d)
                            continue;
                        for (int kh = 0; kh < cd->fh; ++kh)
                        {
                            const int64_t ih =
                                oh * cd->sh - cd->ph + kh * cd->dh;
                            if (ih < 0 || ih >= xd->h)
                                continue;
                            const float* wrow =
                                w
                                + ((((size_t) k * C + c) * cd->fd + kd) * cd->fh
                                   + kh)
                                      * cd->fw;
                            for (int kw = 0; kw < cd->fw; ++kw)
                            {
                                const int64_t iw =
                                    ow * cd->sw - cd->pw + kw * cd->dw;
                                if (iw < 0 || iw >= xd->w)
                                    continue;
                                acc += (double) x[off5(xd, n, c, id, ih, iw)]
                                       * (double) wrow[kw];
                            }
                        }
                    }
                float* yp = y + off5(yd, n, k, od, oh, ow);
                const double prev = beta != 0.0 ? (double) *yp : 0.0;
                *yp = (float) (alpha * acc + beta * prev);
            }
    }
}

/* dx[n,c,i] = alpha * sum_{k,f : i = o*s - p + f*dil} dy[n,k,o] * w[k,c,f]
 *             + beta * dx */
void oracle_conv_bwd_data(const float* w, const float* dy,
                          const oracle_tdesc* yd, float* dx,
                          const oracle_tdesc* xd, const oracle_cdesc* cd,
                          double alpha, double beta)
{
    const int64_t K = yd->c, C = xd->c;
    const int64_t total = xd->n * C * xd->d;
#pragma omp parallel for schedule(static)
    for (int64_t job = 0; job < total; ++job)
    {
        const int64_t id = job % xd->d;
        const int64_t c = (job / xd->d) % C;
        const int64_t n = job / (xd->d * C);
        for (int64_t ih = 0; ih < xd->h; ++ih)
            for (int64_t iw = 0; iw < xd->w; ++iw)
            {
                double acc = 0.0;
                for (int64_t k = 0; k < K; ++k)
                    for (int kd = 0; kd < cd->fd; ++kd)
                    {
                        const int64_t td = id + cd->pd - kd * cd->dd;
                        if (td < 0 || td % cd->sd)
                            continue;
                        const int64_t od = td / cd->sd;
                        if (od >= yd->d)
                            continue;
                        for (int kh = 0; kh < cd->fh; ++kh)
                        {
                            const int64_t th = ih + cd->ph - kh * cd->dh;
                            if (th < 0 || th % cd->sh)
                                continue;
                            const int64_t oh = th / cd->sh;
                            if (oh >= yd->h)
                                continue;
                            const float* wrow =
                                w
                                + ((((size_t) k * C + c) * cd->fd + kd) * cd->fh
                                   + kh)
                                      * cd->fw;
                            for (int kw = 0; kw < cd->fw; ++kw)
                            {
                                const int64_t tw = iw + cd->pw - kw * cd->dw;
                                if (tw < 0 || tw % cd->sw)
                                    continue;
                                const int64_t ow = tw / cd->sw;
                                if (ow >= yd->w)
                                    continue;
                                acc += (double) dy[off5(yd, n, k, od, oh, ow)]
                                       * (double) wrow[kw];
                            }
                        }
                    }
                float* xp = dx + off5(xd, n, c, id, ih, iw);
                const double prev = beta != 0.0 ? (double) *xp : 0.0;
                *xp = (float) (alpha * acc + beta * prev);
            }
    }
}

/* dw[k,c,f] = alpha * sum_{n,o} dy[n,k,o] * x[n,c,o*s - p + f*dil] + beta*dw */
void oracle_conv_bwd_filter(const float* x, const oracle_tdesc* xd,
                            const float* dy, const oracle_tdesc* yd, float* dw,
                            const oracle_cdesc* cd, double alpha, double beta)
{
    const int64_t K = yd->c, C = xd->c;
    const int64_t taps = (int64_t) cd->fd * cd->fh * cd->fw;
    const int64_t total = K * C * taps;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < total; ++job)
    {
        const int kw = (int) (job % cd->fw);
        const int kh = (int) ((job / cd->fw) % cd->fh);
        const int kd = (int) ((job / (cd->fw * cd->fh)) % cd->fd);
        const int64_t c = (job / taps) % C;
        const int64_t k = job / (taps * C);
        double acc = 0.0;
        for (int64_t n = 0; n < yd->n; ++n)
            for (int64_t od = 0; od < yd->d; ++od)
            {
                const int64_t id = od * cd->sd - cd->pd + kd * cd->dd;
                if (id < 0 || id >= xd->d)
                    continue;
                for (int64_t oh = 0; oh < yd->h; ++oh)
                {
                    const int64_t ih = oh * cd->sh - cd->ph + kh * cd->dh;
                    if (ih < 0 || ih >= xd->h)
                        continue;
                    for (int64_t ow = 0; ow < yd->w; ++ow)
                    {
                        const int64_t iw = ow * cd->sw - cd->pw + kw * cd->dw;
                        if (iw < 0 || iw >= xd->w)
                            continue;
                        acc += (double) dy[off5(yd, n, k, od, oh, ow)]
                               * (double) x[off5(xd, n, c, id, ih, iw)];
                    }
                }
            }
        const double prev = beta != 0.0 ? (double) dw[job] : 0.0;
        dw[job] = (float) (alpha * acc + beta * prev);
    }
}

/* ---- batch normalisation ------------------------------------------------ */

/* Per-channel sum and sum of squares over the owned cells (batchnorm.cu:39-132
 * computes the same two sums with fp32 atomics; here fp64). */
void oracle_bn_sums(const float* x, const oracle_tdesc* xd, double* sums,
                    double* sqsums)
{
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < xd->c; ++c)
    {
        double s = 0.0, q = 0.0;
        for (int64_t n = 0; n < xd->n; ++n)
            for (int64_t d = 0; d < xd->d; ++d)
                for (int64_t h = 0; h < xd->h; ++h)
                    for (int64_t w = 0; w < xd->w; ++w)
                    {
                        const double v = x[off5(xd, n, c, d, h, w)];
                        s += v;
                        q += v * v;
                    }
        sums[c] = s;
        sqsums[c] = q;
    }
}

/* batchnorm.cu:297-312.  mean_var[0..C) holds sums on entry / mean on exit,
 * mean_var[C..2C) sums of squares on entry / unbiased variance on exit. */
void oracle_bn_sums_to_statistics(int64_t num_per_sum, float decay, int64_t C,
                                  float* mean, float* var, float* running_mean,
                                  float* running_var)
{
    for (int64_t c = 0; c < C; ++c)
    {
        if (num_per_sum > 0)
        {
            const float nps = (float) num_per_sum;
            const float m = mean[c] / nps;
            const float sq = var[c] / nps;
            float v = sq - m * m;
            v = v > 0.f ? v : 0.f;
            v *= nps / (nps - 1.f);
            mean[c] = m;
            var[c] = v;
            running_mean[c] = decay * running_mean[c] + (1.f - decay) * m;
            running_var[c] = decay * running_var[c] + (1.f - decay) * v;
        }
        else
        {
            var[c] = 1.f;
        }
    }
}

/* batchnorm.cu:385-412: y = scale * (x - mean) * rsqrt(var + eps) + bias */
void oracle_bn_normalize(const float* x, const oracle_tdesc* xd,
                         const float* mean, const float* var,
                         const float* scale, const float* bias, float eps,
                         float* y, const oracle_tdesc* yd)
{
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < xd->c; ++c)
    {
        const float inv_stdev = (float) (1.0 / sqrt((double) (var[c] + eps)));
        for (int64_t n = 0; n < xd->n; ++n)
            for (int64_t d = 0; d < xd->d; ++d)
                for (int64_t h = 0; h < xd->h; ++h)
                    for (int64_t w = 0; w < xd->w; ++w)
                    {
                        const float xv = x[off5(xd, n, c, d, h, w)];
                        const float xhat = (xv - mean[c]) * inv_stdev;
                        y[off5(yd, n, c, d, h, w)] = scale[c] * xhat + bias[c];
                    }
    }
}

/* batchnorm.cu:920-956: local contributions to dscale, dbias, dmean, dvar. */
void oracle_bn_backprop1(const float* x, const oracle_tdesc* xd,
                         const float* dy, const oracle_tdesc* yd,
                         const float* mean, const float* var,
                         const float* scale, float eps, double* dscale,
                         double* dbias, double* dmean, double* dvar)
{
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < xd->c; ++c)
    {
        const float inv_stdev = (float) (1.0 / sqrt((double) (var[c] + eps)));
        const float dvar_factor = inv_stdev * inv_stdev * inv_stdev / 2;
        double a = 0, b = 0, m = 0, v = 0;
        for (int64_t n = 0; n < xd->n; ++n)
            for (int64_t d = 0; d < xd->d; ++d)
                for (int64_t h = 0; h < xd->h; ++h)
                    for (int64_t w = 0; w < xd->w; ++w)
                    {
                        const float xv = x[off5(xd, n, c, d, h, w)];
                        const float g = dy[off5(yd, n, c, d, h, w)];
                        const float xhat = (xv - mean[c]) * inv_stdev;
                        a += (double) (g * xhat);
                        b += (double) g;
                        const float dxhat = g * scale[c];
                        m += (double) (-dxhat * inv_stdev);
                        v += (double) (-dxhat * (xv - mean[c]) * dvar_factor);
                    }
        dscale[c] = a;
        dbias[c] = b;
        dmean[c] = m;
        dvar[c] = v;
    }
}

/* batchnorm.cu:1327-1362:
 * dx = dy*scale*inv_stdev + dmean/n + dvar*2/(n-1) * (x - mean) */
void oracle_bn_backprop2(const float* x, const oracle_tdesc* xd,
                         const float* dy, const oracle_tdesc* yd,
                         const float* mean, const float* var,
                         const float* scale, const float* dmean,
                         const float* dvar, float eps, int64_t num_per_sum,
                         float* dx, const oracle_tdesc* dxd)
{
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < xd->c; ++c)
    {
        const float inv_stdev = (float) (1.0 / sqrt((double) (var[c] + eps)));
        const float dmean_term = dmean[c] / (float) num_per_sum;
        const float dvar_term = dvar[c] * 2 / (float) (num_per_sum - 1);
        for (int64_t n = 0; n < xd->n; ++n)
            for (int64_t d = 0; d < xd->d; ++d)
                for (int64_t h = 0; h < xd->h; ++h)
                    for (int64_t w = 0; w < xd->w; ++w)
                    {
                        const float xv = x[off5(xd, n, c, d, h, w)];
                        const float g = dy[off5(yd, n, c, d, h, w)];
                        const float dxhat = g * scale[c];
                        float r = dxhat * inv_stdev;
                        r += dmean_term;
                        r += dvar_term * (xv - mean[c]);
                        dx[off5(dxd, n, c, d, h, w)] = r;
                    }
    }
}
