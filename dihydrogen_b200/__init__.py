"""B200-native implementation of DistConv's spatially-parallel layer path:
halo exchange, convolution forward / backward-data / backward-filter on the
halo-extended shard, distributed batch-normalisation.

The compute lives in libdistconv_b200.so (hand-written sm_100a kernels behind
the C ABI of include/dcb.h); this package is the Python host mirror of the
DistConv operator interface.  There is no CPU fallback.
"""
from .distconv import (  # noqa: F401
    LHS,
    RHS,
    Allreduce,
    BackendDNNLib,
    BatchNormalization,
    Convolution,
    Distribution,
    HaloExchange,
    LeakyReLU,
    Locale,
    Options,
    Pooling,
    Tensor,
    TensorShuffler,
    create_convolution_d_output_tensor,
    create_convolution_output_tensor,
    create_d_input_tensor,
    create_input_tensor,
    create_pooling_d_output_tensor,
    create_pooling_output_tensor,
    dump_local_tensor,
    dump_tensor,
    get_halo_sizes,
)
