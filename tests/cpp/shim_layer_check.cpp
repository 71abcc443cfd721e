// Drives one spatially-partitioned conv + batch-norm layer (forward and the
// three backward passes of the convolution) and a max-pooling of the same input
// (forward, backward with the reverse SUM exchange) through the C++ classes of
// distconv_b200.hpp, with R ranks run as R host threads on one GPU, and checks
// every result against plain loops over the unpartitioned problem.
//
// Because all ranks share one device, a kernel that waits for a peer is only
// launched after the peer's kernel it waits for: each thread launches its
// "put" half, synchronises its stream, meets the others at a host barrier and
// only then launches the "wait" half.
//
// usage: shim_layer_check [ranks]   (prints "shim_layer_check OK" and exits 0)
#include "distconv_b200.hpp"

#include <unistd.h>

#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <mutex>
#include <thread>
#include <vector>

using namespace distconv;

namespace
{
struct Barrier
{
    explicit Barrier(int n) : n(n) {}
    void wait()
    {
        std::unique_lock<std::mutex> lk(m);
        const int gen = generation;
        if (++count == n)
        {
            count = 0;
            ++generation;
            cv.notify_all();
        }
        else
            cv.wait(lk, [&] { return gen != generation; });
    }
    int n, count = 0, generation = 0;
    std::mutex m;
    std::condition_variable cv;
};

// problem: W,H,D partitioned along D
constexpr int W = 20, H = 12, D = 16, C = 4, K = 8, N = 2, F = 3;
constexpr float EPS = 1e-5f, DECAY = 0.9f;

float synth(int64_t i, int salt)
{
    uint32_t h = (uint32_t) (i * 2654435761u) ^ (uint32_t) (salt * 40503u);
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    return (float) ((int) (h % 2001) - 1000) / 1000.f;
}
inline size_t gi(int n, int c, int d, int h, int w, int Cc)
{
    return ((((size_t) n * Cc + c) * D + d) * H + h) * W + w;
}

struct Global
{
    std::vector<float> x, w, dy, y, dx, dw, z; // z = batch-norm output
    std::vector<float> pdy, py, pdx;           // 3x3x3 max-pooling of x, stride 1, pad 1
    std::vector<float> mean, var;
};

void pool_reference(Global& g)
{
    const size_t nx = (size_t) N * C * D * H * W;
    g.py.assign(nx, 0.f);
    g.pdx.assign(nx, 0.f);
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
            for (int d = 0; d < D; ++d)
                for (int h = 0; h < H; ++h)
                    for (int w = 0; w < W; ++w)
                    {
                        float best = 0.f;
                        size_t at = 0;
                        bool any = false;
                        for (int kd = -1; kd <= 1; ++kd)
                            for (int kh = -1; kh <= 1; ++kh)
                                for (int kw = -1; kw <= 1; ++kw)
                                {
                                    const int dd = d + kd, hh = h + kh, ww = w + kw;
                                    if (dd < 0 || dd >= D || hh < 0 || hh >= H || ww < 0 || ww >= W)
                                        continue;
                                    const size_t i = gi(n, c, dd, hh, ww, C);
                                    if (!any || g.x[i] > best) // the first maximum keeps the gradient
                                    {
                                        best = g.x[i];
                                        at = i;
                                        any = true;
                                    }
                                }
                        const size_t o = gi(n, c, d, h, w, C);
                        g.py[o] = best;
                        g.pdx[at] += g.pdy[o];
                    }
}

void reference(Global& g)
{
    const size_t nx = (size_t) N * C * D * H * W, ny = (size_t) N * K * D * H * W;
    g.y.assign(ny, 0.f);
    g.dx.assign(nx, 0.f);
    g.dw.assign((size_t) K * C * F * F * F, 0.f);
    std::vector<double> dxa(nx, 0.0), dwa(g.dw.size(), 0.0);
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            for (int d = 0; d < D; ++d)
                for (int h = 0; h < H; ++h)
                    for (int w = 0; w < W; ++w)
                    {
                        double acc = 0;
                        const float dyv = g.dy[gi(n, k, d, h, w, K)];
                        for (int c = 0; c < C; ++c)
                            for (int fd = 0; fd < F; ++fd)
                                for (int fh = 0; fh < F; ++fh)
                                    for (int fw = 0; fw < F; ++fw)
                                    {
                                        const int id = d + fd - 1, ih = h + fh - 1, iw = w + fw - 1;
                                        if (id < 0 || id >= D || ih < 0 || ih >= H || iw < 0 || iw >= W)
                                            continue;
                                        const size_t wi = ((((size_t) k * C + c) * F + fd) * F + fh) * F + fw;
                                        const size_t xi = gi(n, c, id, ih, iw, C);
                                        acc += (double) g.x[xi] * g.w[wi];
                                        dxa[xi] += (double) dyv * g.w[wi];
                                        dwa[wi] += (double) dyv * g.x[xi];
                                    }
                        g.y[gi(n, k, d, h, w, K)] = (float) acc;
                    }
    for (size_t i = 0; i < nx; ++i)
        g.dx[i] = (float) dxa[i];
    for (size_t i = 0; i < dwa.size(); ++i)
        g.dw[i] = (float) dwa[i];
    // batch norm over y with unit scale / zero bias, unbiased variance
    g.z.assign(ny, 0.f);
    g.mean.assign(K, 0.f);
    g.var.assign(K, 0.f);
    const double cnt = (double) N * D * H * W;
    for (int k = 0; k < K; ++k)
    {
        double s = 0, q = 0;
        for (int n = 0; n < N; ++n)
            for (size_t i = 0; i < (size_t) D * H * W; ++i)
            {
                const double v = g.y[((size_t) n * K + k) * D * H * W + i];
                s += v;
                q += v * v;
            }
        const double m = s / cnt, var = (q / cnt - m * m) * cnt / (cnt - 1);
        g.mean[k] = (float) m;
        g.var[k] = (float) var;
        const double inv = 1.0 / std::sqrt(var + EPS);
        for (int n = 0; n < N; ++n)
            for (size_t i = 0; i < (size_t) D * H * W; ++i)
            {
                const size_t j = ((size_t) n * K + k) * D * H * W + i;
                g.z[j] = (float) ((g.y[j] - m) * inv);
            }
    }
}

// copies between a shard (halo-extended, device) and the global host array
void scatter(TensorF& t, const std::vector<float>& g, int Cc)
{
    const auto real = t.get_local_pitched_shape(); // rows carry padding up to the pitch
    const auto& loc = t.get_local_shape();
    const auto& off = t.get_global_index();
    const auto& ov = t.get_overlap();
    std::vector<float> host((size_t) real.get_size(), 0.f);
    for (int n = 0; n < loc[4]; ++n)
        for (int c = 0; c < loc[3]; ++c)
            for (int d = 0; d < loc[2]; ++d)
                for (int h = 0; h < loc[1]; ++h)
                    for (int w = 0; w < loc[0]; ++w)
                    {
                        const size_t li = ((((size_t) n * real[3] + c) * real[2] + d + ov[2]) * real[1] + h + ov[1])
                                              * real[0]
                                          + w + ov[0];
                        host[li] = g[gi(n + (int) off[4], c + (int) off[3], d + (int) off[2], h + (int) off[1],
                                        w + (int) off[0], Cc)];
                    }
    cudaMemcpy(t.get_buffer(), host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice);
}

double gather_err(TensorF& t, const std::vector<float>& g, int Cc)
{
    const auto real = t.get_local_pitched_shape(); // rows carry padding up to the pitch
    const auto& loc = t.get_local_shape();
    const auto& off = t.get_global_index();
    const auto& ov = t.get_overlap();
    std::vector<float> host((size_t) real.get_size());
    cudaMemcpy(host.data(), t.get_buffer(), host.size() * sizeof(float), cudaMemcpyDeviceToHost);
    double err = 0;
    for (int n = 0; n < loc[4]; ++n)
        for (int c = 0; c < loc[3]; ++c)
            for (int d = 0; d < loc[2]; ++d)
                for (int h = 0; h < loc[1]; ++h)
                    for (int w = 0; w < loc[0]; ++w)
                    {
                        const size_t li = ((((size_t) n * real[3] + c) * real[2] + d + ov[2]) * real[1] + h + ov[1])
                                              * real[0]
                                          + w + ov[0];
                        const float ref = g[gi(n + (int) off[4], c + (int) off[3], d + (int) off[2],
                                               h + (int) off[1], w + (int) off[0], Cc)];
                        err = std::max(err, (double) std::fabs(host[li] - ref) / (1.0 + std::fabs(ref)));
                    }
    return err;
}

struct Shared
{
    explicit Shared(int r) : bar(r), blobs((size_t) r * 256), fail(0) {}
    Barrier bar;
    std::vector<char> blobs;
    std::mutex m;
    int fail;
};

void rank_main(int rank, int R, Shared* sh, const Global* g)
{
    try
    {
        cudaSetDevice(0);
        cudaStream_t st;
        cudaStreamCreate(&st);
        auto ag = [sh, rank, R](const void* in, void* out, size_t n) {
            sh->bar.wait(); // everybody is done with the previous gather
            if (rank == 0)
                sh->blobs.resize((size_t) R * n);
            sh->bar.wait();
            std::memcpy(sh->blobs.data() + (size_t) rank * n, in, n);
            sh->bar.wait();
            std::memcpy(out, sh->blobs.data(), (size_t) R * n);
        };
        tensor::LocaleMPI loc(rank, R, ag);
        // the backend with the reference's option block (dnn_backend.hpp:46-63, 661-725)
        const Options opts(/*overlap_halo_exchange=*/false, /*deterministic=*/true, /*enable_profiling=*/true);
        BackendDNNLib be(loc, st, opts);
        if (be.get_stream() != st || !be.deterministic() || !be.profiling() || be.overlap_halo_exchange()
            || be.get_num_internal_comms() != 8
            || be.get_internal_comm(3)->get_stream() != be.get_internal_priority_stream(3)
            || be.get_al_comm().get_stream() != st || be.get_name() != "B200")
            throw std::runtime_error("backend accessors");
        const int_vector shape{W, H, D, C, N}, grid{1, 1, R, 1, 1}, fshape{F, F, F, C, K};
        const int_vector f3{F, F, F}, ones{1, 1, 1}, pads{1, 1, 1};
        TensorF x = create_input_tensor(shape, grid, f3, ones, ones, false, loc);
        TensorF dx = create_d_input_tensor(x);
        TensorF y = create_convolution_output_tensor(x, fshape, ones, pads, ones);
        TensorF dy = create_convolution_d_output_tensor(y, fshape, ones);
        TensorF z = create_convolution_output_tensor(x, fshape, ones, pads, ones);
        for (TensorF* t : {&x, &dx, &y, &dy, &z})
            if (t->allocate())
                throw std::runtime_error("allocate");
        scatter(x, g->x, C);
        scatter(dy, g->dy, K);
        const size_t wcount = (size_t) K * C * F * F * F;
        float *w = nullptr, *dw = nullptr, *stats = nullptr;
        cudaMalloc((void**) &w, wcount * 4);
        cudaMalloc((void**) &dw, wcount * 4);
        cudaMalloc((void**) &stats, 6 * K * 4); // mean|var|running mean|running var|scale|bias
        cudaMemcpy(w, g->w.data(), wcount * 4, cudaMemcpyHostToDevice);
        std::vector<float> init(6 * K, 0.f);
        for (int k = 0; k < K; ++k)
            init[3 * K + k] = init[4 * K + k] = 1.f; // running var, scale
        cudaMemcpy(stats, init.data(), init.size() * 4, cudaMemcpyHostToDevice);

        // filters as the reference passes them: tensors every rank holds whole
        const tensor::Shape fsh(std::vector<index_t>{F, F, F, C, K});
        const auto shared = tensor::Distribution::make_shared_distribution(tensor::Shape(std::vector<index_t>{1, 1, R, 1, 1}));
        TensorF wt(fsh, loc, shared), dwt(fsh, loc, shared);
        wt.set_view(w);
        dwt.set_view(dw);
        // the six-argument constructor (convolution.hpp:29-60)
        Convolution<BackendDNNLib, float> conv(be, 5, GetHaloExchangeMethod("P2P"), /*enable_overlap=*/false,
                                               /*enable_profiling=*/true, ChannelParallelismAlgorithm::NONE);
        conv.setup(x, wt, y, dx, dwt, dy, pads, ones, ones, 1, "DEFAULT", "DEFAULT", "DEFAULT", 0);
        BatchNormalization<BackendDNNLib, float> bn(be, 5, DECAY, EPS, true);

        auto phase = [&](auto put, auto wait) {
            put();
            cudaStreamSynchronize(st);
            sh->bar.wait();
            wait();
            cudaStreamSynchronize(st);
            sh->bar.wait();
        };
        // forward: halo exchange of x (D is the only partitioned dimension)
        x.clear_halo(2, st);
        phase([&] { conv.input_halo_exchange().pack_put(2, st); },
              [&] { conv.input_halo_exchange().wait_unpack(2, st); });
        if (R == 1)
        {
            // the reference's argument list (halo_exchange_cuda.hpp:107-113): one
            // communicator per dimension and side, the backend's internal ones
            BoundaryAttributesV<std::shared_ptr<BackendDNNLib::InternalCommType>> comms;
            int k = 0;
            apply_to_spatial_sides(5, [&](int i, Side side) { comms(i, side) = be.get_internal_comm(k++); });
            conv.input_halo_exchange().exchange(comms, st, /*rendezvous=*/false, /*sync_back=*/true,
                                                /*is_reverse=*/false, /*skip_unpack=*/false);
            conv.set_num_samples(N); // the extent the layer was set up with: nothing to rebuild
        }
        // the statistics come from the convolution's epilogue where its kernel has one
        const int fused = conv.forward_with_statistics(1.f, x, w, y, stats, stats + K, /*skip_halo_exchange=*/true);
        if (!fused)
            bn.forward_stage1(y, stats, stats + K);
        phase([&] { be.allreduce_push(stats, 2 * K); }, [&] { be.allreduce_pull(stats, 2 * K); });
        bn.forward_stage2(y, stats, stats + K, stats + 2 * K, stats + 3 * K, stats + 4 * K, stats + 5 * K, z);
        // backward of the convolution
        phase([&] { conv.d_output_halo_exchange().pack_put(2, st); },
              [&] { conv.d_output_halo_exchange().wait_unpack(2, st); });
        conv.backward_data(1.f, wt, dy, 0.f, dx, /*skip_halo_exchange=*/true);
        conv.backward_filter(1.f, x, dy, 0.f, dwt, /*reduce=*/false);
        phase([&] { be.allreduce_push(dw, (index_t) wcount); }, [&] { be.allreduce_pull(dw, (index_t) wcount); });
        if (conv.status() != DCB_OK)
            throw std::runtime_error("layer status");
        cudaStreamSynchronize(st);

        // max-pooling of x (its halos are still in place); the gradients a rank
        // computes for its neighbours' cells go back with the reverse SUM exchange
        TensorF py = create_pooling_output_tensor(x, f3, ones, pads);
        TensorF pdy = create_pooling_d_output_tensor(py);
        TensorF pdx = create_d_input_tensor(x);
        for (TensorF* t : {&py, &pdy, &pdx})
            if (t->allocate())
                throw std::runtime_error("allocate");
        scatter(pdy, g->pdy, C);
        Pooling<BackendDNNLib, float> pool(be, 5);
        pool.setup(x, py, pdx, pdy, f3, pads, ones, "MAX");
        pool.forward(1.f, x, 0.f, py, true, /*skip_halo_exchange=*/true);
        pool.backward(1.f, py, pdy, x, 0.f, pdx, /*skip_halo_exchange=*/true);
        phase([&] { pool.d_input_halo_exchange().pack_put(2, st, true, tensor::HaloExchangeAccumOp::SUM); },
              [&] { pool.d_input_halo_exchange().wait_unpack(2, st, true, tensor::HaloExchangeAccumOp::SUM); });
        const double e_py = gather_err(py, g->py, C), e_pdx = gather_err(pdx, g->pdx, C);

        // re-distribution: x (partitioned along D) -> sample-parallel where N divides, and back
        double e_shf = 0;
        if (N % R == 0)
        {
            const tensor::Shape gs(std::vector<index_t>{W, H, D, C, N});
            TensorF xs(gs, loc,
                       tensor::Distribution::make_overlapped_distribution(
                           tensor::Shape(std::vector<index_t>{1, 1, 1, 1, R}), tensor::IntVector(5, 0)));
            TensorF xb = create_d_input_tensor(x);
            if (xs.allocate() || xb.allocate())
                throw std::runtime_error("allocate");
            tensor::TensorMPICUDAShuffler<float> shf(x, xs);
            phase([&] { shf.put(true, x.get_buffer(), st); }, [&] { shf.wait_unpack(true, xs.get_buffer(), st); });
            phase([&] { shf.put(false, xs.get_buffer(), st); }, [&] { shf.wait_unpack(false, xb.get_buffer(), st); });
            if (shf.status(true, st) != DCB_OK || shf.status(false, st) != DCB_OK)
                throw std::runtime_error("shuffle status");
            e_shf = std::max(gather_err(xs, g->x, C), gather_err(xb, g->x, C));
        }

        std::vector<float> hdw(wcount), hstats(2 * K);
        cudaMemcpy(hdw.data(), dw, wcount * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(hstats.data(), stats, 2 * K * 4, cudaMemcpyDeviceToHost);
        double e_dw = 0, e_st = 0;
        for (size_t i = 0; i < wcount; ++i)
            e_dw = std::max(e_dw, (double) std::fabs(hdw[i] - g->dw[i]) / (1.0 + std::fabs(g->dw[i])));
        for (int k = 0; k < K; ++k)
        {
            e_st = std::max(e_st, (double) std::fabs(hstats[k] - g->mean[k]));
            e_st = std::max(e_st, (double) std::fabs(hstats[K + k] - g->var[k]) / (1.0 + g->var[k]));
        }
        const double e_y = gather_err(y, g->y, K), e_dx = gather_err(dx, g->dx, C), e_z = gather_err(z, g->z, K);
        // dump_tensor: rank 0 writes the global y as raw floats, W fastest (distconv.hpp:581-631)
        const std::string dump = "/tmp/shim_dump_" + std::to_string((long) getpid()) + "_" + std::to_string(R);
        dump_tensor(y, dump, true);
        double e_dump = 0;
        if (rank == 0)
        {
            std::vector<float> back(g->y.size());
            std::FILE* f = std::fopen((dump + ".out").c_str(), "rb");
            if (!f || std::fread(back.data(), sizeof(float), back.size(), f) != back.size())
                throw std::runtime_error("dump_tensor file");
            std::fclose(f);
            std::remove((dump + ".out").c_str());
            for (size_t i = 0; i < back.size(); ++i)
                e_dump = std::max(e_dump, (double) std::fabs(back[i] - g->y[i]) / (1.0 + std::fabs(g->y[i])));
        }
        std::printf("rank %d/%d: y %.2e  dx %.2e  dw %.2e  stats %.2e  bn %.2e  pool %.2e / %.2e  shuffle %.1e  (fwd "
                    "kernel kind %d, statistics %s)\n",
                    rank, R, e_y, e_dx, e_dw, e_st, e_z, e_py, e_pdx, e_shf, conv.kernel_kind(0),
                    fused ? "fused" : "separate");
        const bool ok = e_y < 2e-5 && e_dx < 2e-5 && e_dw < 5e-5 && e_st < 2e-5 && e_z < 1e-4 && e_py < 1e-6
                        && e_pdx < 2e-6 && e_shf == 0.0 && e_dump < 2e-5;
        if (!ok)
        {
            std::lock_guard<std::mutex> lk(sh->m);
            sh->fail = 1;
        }
        sh->bar.wait(); // nobody tears its windows down while a peer may still read them
        cudaFree(w);
        cudaFree(dw);
        cudaFree(stats);
    }
    catch (const std::exception& e)
    {
        std::fprintf(stderr, "rank %d: %s\n", rank, e.what());
        std::exit(2); // a rank that left would strand the others at the barrier
    }
}
} // namespace

// the vocabulary of base.hpp / tensor_base.hpp / memory.hpp, host side only
bool vocabulary_check()
{
    bool ok = GetHaloExchangeMethod("AL") == HaloExchangeMethod::AL
              && GetHaloExchangeMethod("HYBRID") == HaloExchangeMethod::HYBRID
              && GetBatchnormImpl("AL_NCCL") == BatchnormImpl::AL_NCCL && GetShuffleMethod("MPI") == ShuffleMethod::MPI
              && ~LHS == RHS;
    try
    {
        GetHaloExchangeMethod("carrier pigeon");
        ok = false;
    }
    catch (const std::invalid_argument&)
    {}
    int calls = 0;
    apply_to_sides<3>([&](int, Side) { ++calls; });
    apply_to_spatial_sides(5, [&](int, Side) { ++calls; });
    ok = ok && calls == 12;
    BoundaryAttributesV<int> attrs(7, 9);
    attrs(2, RHS) = 1;
    ok = ok && attrs(0, LHS) == 7 && attrs(1, RHS) == 9 && attrs(2, RHS) == 1;
    tensor::Array<3> a{4, 5, 6};
    ok = ok && a[-1] == 6 && a.get_size() == 120 && (a + tensor::Array<3>(1))[0] == 5;
    const tensor::Shape shape(std::vector<index_t>{4, 3, 2});
    ok = ok && tensor::get_strides(shape)[2] == 12 && tensor::get_offset(tensor::IndexVector(std::vector<index_t>{1, 2, 1}), shape) == 21;
    // a host tensor on the process locale, aliasing caller memory through View
    using HostTensor = tensor::Tensor<float, tensor::LocaleProcess, tensor::BaseAllocator>;
    HostTensor ht(shape, tensor::LocaleProcess(), tensor::Distribution::make_localized_distribution(3));
    std::vector<float> backing(24, 2.5f);
    tensor::View(ht, backing.data());
    ok = ok && ht.is_view() && ht.get_buffer() == backing.data() && ht.get_pitch() == 4;
    HostTensor owned(shape, tensor::LocaleProcess(), tensor::Distribution::make_localized_distribution(3));
    ok = ok && owned.allocate() == 0 && owned.get_buffer()[23] == 0.f && !owned.is_view();
    std::ostringstream os;
    os << HaloExchangeMethod::P2P << " " << BatchnormImpl::MPI << " " << RHS << " " << ChannelParallelismAlgorithm::AUTO;
    ok = ok && os.str() == "P2P MPI RHS AUTO";
    return ok;
}

int main(int argc, char** argv)
{
    const int R = argc > 1 ? std::atoi(argv[1]) : 2;
    if (!vocabulary_check())
    {
        std::printf("shim_layer_check FAILED (vocabulary)\n");
        return 1;
    }
    Global g;
    const size_t nx = (size_t) N * C * D * H * W, ny = (size_t) N * K * D * H * W;
    g.x.resize(nx);
    g.dy.resize(ny);
    g.w.resize((size_t) K * C * F * F * F);
    for (size_t i = 0; i < nx; ++i)
        g.x[i] = synth((int64_t) i, 1);
    for (size_t i = 0; i < ny; ++i)
        g.dy[i] = synth((int64_t) i, 2);
    for (size_t i = 0; i < g.w.size(); ++i)
        g.w[i] = 0.25f * synth((int64_t) i, 3);
    reference(g);
    g.pdy.resize(nx);
    for (size_t i = 0; i < nx; ++i)
        g.pdy[i] = synth((int64_t) i, 4);
    pool_reference(g);
    Shared sh(R);
    std::vector<std::thread> th;
    for (int r = 0; r < R; ++r)
        th.emplace_back(rank_main, r, R, &sh, &g);
    for (auto& t : th)
        t.join();
    if (sh.fail)
    {
        std::printf("shim_layer_check FAILED\n");
        return 1;
    }
    std::printf("shim_layer_check OK\n");
    return 0;
}
