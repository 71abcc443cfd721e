// tcgen05 / TMEM convolution kernels.
#include "conv_tc.cuh"

namespace dcb
{

struct TcPlan
{
    int unused;
};

int32_t tc_plan_create(const ConvGeom&, const ConvGeom&, bool, int,
                       TcPlan** out)
{
    *out = nullptr;
    return DCB_OK;
}
void tc_plan_destroy(TcPlan* p)
{
    delete p;
}
bool tc_supports(const TcPlan*, int)
{
    return false;
}
int32_t tc_conv_fwd(TcPlan*, int, float, const float*, const float*, float,
                    float*, cudaStream_t)
{
    return DCB_UNSUPPORTED;
}
int32_t tc_conv_bwd_filter(TcPlan*, float, const float*, const float*, float,
                           float*, cudaStream_t)
{
    return DCB_UNSUPPORTED;
}

} // namespace dcb
