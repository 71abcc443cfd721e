// Interface of the tcgen05 / TMEM convolution kernels.
#pragma once

#include "conv_simt.cuh"

namespace dcb
{

struct TcPlan;

// Creates tensor-core state for the problems the kernels cover; *out stays
// null (and DCB_OK is returned) when none of them applies.  `fwd` is the
// forward geometry, `bwd` the forward-shaped geometry that computes backward
// data (only meaningful when bwd_is_fwd).
int32_t tc_plan_create(const ConvGeom& fwd, const ConvGeom& bwd,
                       bool bwd_is_fwd, int math_mode, TcPlan** out);
void tc_plan_destroy(TcPlan* p);
// which: 0 forward, 1 backward data, 2 backward filter
bool tc_supports(const TcPlan* p, int which);
// The kernel the plan prefers for that pass, as dcb_conv_plan_kernel_variant
// numbers them (1 row kernel fed by bulk copies, 2 row kernel whose converters
// fetch their own rows, 3 sweep, 4 multi-group sweep, 5 backward filter; 0 none).
int tc_variant(const TcPlan* p, int which);
// slot 0 runs the forward geometry, slot 1 the backward-data one.
int32_t tc_conv_fwd(TcPlan* p, int slot, float alpha, const float* x,
                    const float* w, float beta, float* y, cudaStream_t stream);
// Forward convolution (beta = 0) whose epilogue also returns, per filter, the sum
// and the sum of squares of the outputs.  DCB_UNSUPPORTED when the plan's
// kernel for this problem cannot do that; nothing has been launched then.
int32_t tc_conv_fwd_stats(TcPlan* p, float alpha, const float* x,
                          const float* w, float* y, float* sums,
                          float* sqsums, cudaStream_t stream);
// Device word that kernels set when a bounded wait expires (null if no plan).
int* tc_status_word(TcPlan* p);
int32_t tc_conv_bwd_filter(TcPlan* p, float alpha, const float* x,
                           const float* dy, float beta, float* dw,
                           cudaStream_t stream);

} // namespace dcb
