// The MPI-facing constructors of distconv_b200.hpp, compiled against an mpi.h
// (here the thread-rank stand-in under oracle/mpi_shim, with two ranks as two
// host threads): tensor::LocaleMPI(MPI_Comm) (tensor_mpi.hpp:18-36) and
// DNNBackend(MPI_Comm, Handle_t, Stream_t, Options) (dnn_backend.hpp:661-665),
// then a partitioned tensor whose blobs travel through MPI_Allgather and a
// convolution set up with the reference's argument list.
//
// usage: shim_mpi_check   (prints "shim_mpi_check OK" and exits 0; needs a GPU)
#define DISTCONV_B200_HAS_MPI 1
#include "distconv_b200.hpp"

#include <cstdio>
#include <thread>
#include <vector>

using namespace distconv;

namespace
{
int g_fail = 0;

void rank_main(int rank)
{
    shim_mpi_set_rank(rank);
    cudaSetDevice(0);
    cudaStream_t st;
    cudaStreamCreate(&st);
    tensor::LocaleMPI loc(MPI_COMM_WORLD);
    if (loc.get_rank() != rank || loc.get_size() != 2)
        g_fail = 1;
    BackendDNNLib be(MPI_COMM_WORLD, /*handle=*/nullptr, st, backend::Options(false, true));
    if (be.get_comm() != MPI_COMM_WORLD || be.get_stream() != st || !be.deterministic())
        g_fail = 1;
    const int_vector shape{16, 8, 12, 2, 1}, grid{1, 1, 2, 1, 1}, f3{3, 3, 3}, ones{1, 1, 1}, fshape{3, 3, 3, 2, 4};
    TensorF x = create_input_tensor(shape, grid, f3, ones, ones, false, loc);
    TensorF y = create_convolution_output_tensor(x, fshape, ones, ones, ones);
    TensorF dx = create_d_input_tensor(x);
    TensorF dy = create_convolution_d_output_tensor(y, fshape, ones);
    const tensor::Shape fsh(std::vector<index_t>{3, 3, 3, 2, 4});
    const auto shared = tensor::Distribution::make_shared_distribution(tensor::Shape(std::vector<index_t>{1, 1, 2, 1, 1}));
    TensorF w(fsh, loc, shared), dw(fsh, loc, shared);
    for (TensorF* t : {&x, &y, &dx, &dy, &w, &dw})
        if (t->allocate())
            g_fail = 1;
    if (x.get_local_shape()[2] != 6 || x.get_local_real_shape()[2] != 8 || x.get_global_index()[2] != 6 * rank)
        g_fail = 1;
    // plans and halo plans are built; the exchanges' blobs went through MPI_Allgather
    Convolution<BackendDNNLib, float> conv(be, 5, HaloExchangeMethod::AL);
    conv.setup(x, w, y, dx, dw, dy, ones, ones, ones, 1, "DEFAULT", "DEFAULT", "DEFAULT", 0);
    if (conv.input_halo_exchange().find_peer_rank(2, rank == 0 ? RHS : LHS) != 1 - rank)
        g_fail = 1;
    cudaStreamSynchronize(st);
    MPI_Barrier(MPI_COMM_WORLD); // nobody unmaps while a peer still sets up
}
} // namespace

int main()
{
    shim_mpi_init_world(2);
    std::thread a(rank_main, 0), b(rank_main, 1);
    a.join();
    b.join();
    std::printf(g_fail ? "shim_mpi_check FAILED\n" : "shim_mpi_check OK\n");
    return g_fail;
}
