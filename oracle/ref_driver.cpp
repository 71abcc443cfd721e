// TEST INFRASTRUCTURE ONLY -- never linked into or called by the shipped
// library.
//
// Drives the reference's own header-only CPU code (the tensor model of
// legacy/include/distconv/tensor/tensor_mpi.hpp, the geometry helpers of
// legacy/include/distconv/distconv.hpp and Convolution<ref::Backend,float> of
// legacy/include/distconv/ref/backend.hpp) with R in-process ranks, so that the
// restated oracle and the CUDA path can be compared with outputs of the
// reference itself.  The reference headers are compiled where they lie; no
// reference source is copied here.
//
//   ref_driver geom <nd> <shape...> <locale...> <filter...> <stride...> <pad> <K>
//       prints, per rank, the reference's local shape, halo-extended shape,
//       global offset, get_halo_sizes() result and the conv output's local
//       shape/offset (tensor_mpi.hpp:440-563, distconv.hpp:21-99,365-413).
//   ref_driver conv <dir>
//       4-D, stride 1 (all ref::Backend supports): reads spec.txt, x.bin,
//       w.bin, dy.bin from <dir>; halos of x and dy are filled by definition
//       (global value inside the domain, zero outside) because the reference
//       has no CPU halo exchange (ref/backend.hpp:257); writes y.bin, dx.bin,
//       dw.bin (global tensors, W fastest).
#include "distconv/distconv.hpp"
#include "distconv/ref/backend.hpp"

#include <chrono>
#include <fstream>
#include <iostream>
#include <sstream>
#include <thread>

using namespace distconv;
using TensorF = tensor::Tensor<float, tensor::LocaleMPI, tensor::BaseAllocator>;

namespace
{

std::vector<float> read_bin(const std::string& path, size_t n)
{
    std::vector<float> v(n);
    std::ifstream f(path, std::ios::binary);
    if (!f)
    {
        std::cerr << "cannot open " << path << "\n";
        std::exit(2);
    }
    f.read(reinterpret_cast<char*>(v.data()), n * sizeof(float));
    return v;
}

void write_bin(const std::string& path, const std::vector<float>& v)
{
    std::ofstream f(path, std::ios::binary);
    f.write(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(float));
}

size_t prod(const int_vector& v)
{
    size_t p = 1;
    for (auto x : v)
        p *= x;
    return p;
}

// Fill a local tensor (owned cells and halo cells) from a global array.
void fill_from_global(TensorF& t, const std::vector<float>& g)
{
    const int nd = t.get_num_dims();
    const auto real = t.get_local_real_shape();
    const auto shape = t.get_shape();
    const auto off = t.get_global_index();
    const auto ov = t.get_overlap();
    const size_t n = real.get_size();
    float* buf = t.get_buffer();
    for (size_t lin = 0; lin < n; ++lin)
    {
        size_t r = lin, goff = 0, gstride = 1;
        bool inside = true;
        for (int d = 0; d < nd; ++d)
        {
            long i = (long) (r % real[d]);
            r /= real[d];
            long gi = i - ov[d] + (long) off[d];
            if (gi < 0 || gi >= (long) shape[d])
                inside = false;
            goff += (size_t) (gi < 0 ? 0 : gi) * gstride;
            gstride *= shape[d];
        }
        buf[lin] = inside ? g[goff] : 0.f;
    }
}

// Scatter the owned cells of a local tensor into a global array.
void scatter_to_global(const TensorF& t, std::vector<float>& g)
{
    const int nd = t.get_num_dims();
    const auto loc = t.get_local_shape();
    const auto shape = t.get_shape();
    const auto off = t.get_global_index();
    const size_t n = loc.get_size();
    for (size_t lin = 0; lin < n; ++lin)
    {
        size_t r = lin, goff = 0, gstride = 1;
        IndexVector idx(nd, 0);
        for (int d = 0; d < nd; ++d)
        {
            idx[d] = r % loc[d];
            r /= loc[d];
            goff += (idx[d] + off[d]) * gstride;
            gstride *= shape[d];
        }
        g[goff] = t.get(idx);
    }
}

template <typename V>
std::string vec_str(const V& v, int n)
{
    std::ostringstream ss;
    for (int i = 0; i < n; ++i)
        ss << (i ? "," : "") << v[i];
    return ss.str();
}

struct Spec
{
    int nd = 4;
    int_vector shape, locale, filter, strides, dilations, pads;
    int K = 1;
    int pad = 1;
    int nranks() const { return (int) prod(locale); }
};

std::mutex g_print_mu;

void geom_rank(const Spec& s, int rank, std::vector<std::string>& out)
{
    shim_mpi_set_rank(rank);
    const int nsd = s.nd - 2;
    auto input = create_input_tensor<TensorF>(
        s.shape, s.locale, s.filter, s.strides, s.dilations, false,
        MPI_COMM_WORLD);
    auto filter = create_filter_tensor<TensorF>(
        s.locale, s.filter, input, s.shape[s.nd - 2], s.K, 1, MPI_COMM_WORLD,
        ChannelParallelismAlgorithm::NONE);
    auto output = create_convolution_output_tensor<TensorF>(
        input, filter, s.strides, s.pads, s.dilations, 1);
    auto d_output =
        create_convolution_d_output_tensor<TensorF>(output, filter, s.dilations);
    IntVector fs, bs, fr, br;
    internal::get_halo_sizes(input, IntVector(s.filter), IntVector(s.strides),
                             IntVector(s.dilations), fs, bs, fr, br,
                             s.pad != 0);
    std::ostringstream ss;
    ss << "rank " << rank << " local " << vec_str(input.get_local_shape(), s.nd)
       << " real " << vec_str(input.get_local_real_shape(), s.nd) << " offset "
       << vec_str(input.get_global_index(), s.nd) << " fwd_send "
       << vec_str(fs, nsd) << " bwd_send " << vec_str(bs, nsd) << " fwd_recv "
       << vec_str(fr, nsd) << " bwd_recv " << vec_str(br, nsd) << " out_shape "
       << vec_str(output.get_shape(), s.nd) << " out_local "
       << vec_str(output.get_local_shape(), s.nd) << " out_offset "
       << vec_str(output.get_global_index(), s.nd) << " dout_real "
       << vec_str(d_output.get_local_real_shape(), s.nd) << " split_root "
       << (input.is_split_root() ? 1 : 0);
    out[rank] = ss.str();
}

void conv_rank(const Spec& s, int rank, const std::vector<float>& gx,
               const std::vector<float>& gw, const std::vector<float>& gdy,
               std::vector<float>& gy, std::vector<float>& gdx,
               std::vector<float>& gdw, std::vector<double>& secs)
{
    shim_mpi_set_rank(rank);
    auto input = create_input_tensor<TensorF>(
        s.shape, s.locale, s.filter, s.strides, s.dilations, false,
        MPI_COMM_WORLD);
    auto d_input = create_d_input_tensor<TensorF>(input);
    auto filter = create_filter_tensor<TensorF>(
        s.locale, s.filter, input, s.shape[s.nd - 2], s.K, 1, MPI_COMM_WORLD,
        ChannelParallelismAlgorithm::NONE);
    auto d_filter = create_d_filter_tensor<TensorF>(filter);
    auto output = create_convolution_output_tensor<TensorF>(
        input, filter, s.strides, s.pads, s.dilations, 1);
    auto d_output =
        create_convolution_d_output_tensor<TensorF>(output, filter, s.dilations);
    for (TensorF* t : {&input, &d_input, &filter, &d_filter, &output, &d_output})
    {
        assert0(t->allocate());
        t->zero();
    }
    fill_from_global(input, gx);
    fill_from_global(d_output, gdy);
    std::memcpy(filter.get_buffer(), gw.data(), gw.size() * sizeof(float));

    ref::Backend be;
    Convolution<ref::Backend, float> conv(be, s.nd - 2);
    conv.setup(input, filter, output, d_input, d_filter, d_output, s.pads,
               s.strides, s.dilations, 1, "DEFAULT", "DEFAULT", "DEFAULT", 0);
    auto t0 = std::chrono::steady_clock::now();
    conv.forward(1.0f, input, filter, 0.0f, output);
    auto t1 = std::chrono::steady_clock::now();
    conv.backward_data(1.0f, filter, d_output, 0.0f, d_input);
    auto t2 = std::chrono::steady_clock::now();
    conv.backward_filter(1.0f, input, d_output, 0.0f, d_filter, true);
    auto t3 = std::chrono::steady_clock::now();
    secs[3 * rank + 0] = std::chrono::duration<double>(t1 - t0).count();
    secs[3 * rank + 1] = std::chrono::duration<double>(t2 - t1).count();
    secs[3 * rank + 2] = std::chrono::duration<double>(t3 - t2).count();

    {
        std::lock_guard<std::mutex> lk(g_print_mu);
        scatter_to_global(output, gy);
        scatter_to_global(d_input, gdx);
        if (rank == 0)
            std::memcpy(gdw.data(), d_filter.get_buffer(),
                        gdw.size() * sizeof(float));
    }
}

Spec parse_args(int argc, char** argv, int first)
{
    Spec s;
    int a = first;
    s.nd = std::atoi(argv[a++]);
    const int nsd = s.nd - 2;
    for (int i = 0; i < s.nd; ++i)
        s.shape.push_back(std::atoi(argv[a++]));
    for (int i = 0; i < s.nd; ++i)
        s.locale.push_back(std::atoi(argv[a++]));
    for (int i = 0; i < nsd; ++i)
        s.filter.push_back(std::atoi(argv[a++]));
    for (int i = 0; i < nsd; ++i)
        s.strides.push_back(std::atoi(argv[a++]));
    s.pad = std::atoi(argv[a++]);
    s.K = std::atoi(argv[a++]);
    (void) argc;
    s.dilations = int_vector(nsd, 1);
    for (int i = 0; i < nsd; ++i)
        s.pads.push_back(s.pad ? (s.filter[i] - 1) / 2 : 0);
    return s;
}

} // namespace

int main(int argc, char** argv)
{
    if (argc < 3)
    {
        std::cerr << "usage: ref_driver geom ... | conv <dir> | time <dir>\n";
        return 2;
    }
    const std::string mode = argv[1];
    if (mode == "geom")
    {
        Spec s = parse_args(argc, argv, 2);
        const int R = s.nranks();
        shim_mpi_init_world(R);
        std::vector<std::string> out(R);
        std::vector<std::thread> th;
        for (int r = 0; r < R; ++r)
            th.emplace_back(geom_rank, std::cref(s), r, std::ref(out));
        for (auto& t : th)
            t.join();
        for (auto& l : out)
            std::cout << l << "\n";
        return 0;
    }
    if (mode == "conv")
    {
        const std::string dir = argv[2];
        std::ifstream sp(dir + "/spec.txt");
        std::vector<std::string> toks{"ref_driver", "conv"};
        std::string tok;
        while (sp >> tok)
            toks.push_back(tok);
        std::vector<char*> av;
        for (auto& t : toks)
            av.push_back(const_cast<char*>(t.c_str()));
        Spec s = parse_args((int) av.size(), av.data(), 2);
        if (s.nd != 4)
        {
            std::cerr << "ref::Backend only handles 4-D tensors\n";
            return 2;
        }
        const int R = s.nranks();
        shim_mpi_init_world(R);
        const size_t nx = prod(s.shape);
        int_vector wshape = s.filter;
        wshape.push_back(s.shape[2]);
        wshape.push_back(s.K);
        const size_t nw = prod(wshape);
        // stride 1, pad = radius or 0
        int_vector yshape = s.shape;
        for (int i = 0; i < 2; ++i)
            yshape[i] = s.shape[i] + 2 * s.pads[i] - s.filter[i] + 1;
        yshape[2] = s.K;
        const size_t ny = prod(yshape);
        auto gx = read_bin(dir + "/x.bin", nx);
        auto gw = read_bin(dir + "/w.bin", nw);
        auto gdy = read_bin(dir + "/dy.bin", ny);
        std::vector<float> gy(ny, 0.f), gdx(nx, 0.f), gdw(nw, 0.f);
        std::vector<double> secs(3 * R, 0.0);
        std::vector<std::thread> th;
        for (int r = 0; r < R; ++r)
            th.emplace_back(conv_rank, std::cref(s), r, std::cref(gx),
                            std::cref(gw), std::cref(gdy), std::ref(gy),
                            std::ref(gdx), std::ref(gdw), std::ref(secs));
        for (auto& t : th)
            t.join();
        write_bin(dir + "/y.bin", gy);
        write_bin(dir + "/dx.bin", gdx);
        write_bin(dir + "/dw.bin", gdw);
        double mx[3] = {0, 0, 0};
        for (int r = 0; r < R; ++r)
            for (int k = 0; k < 3; ++k)
                mx[k] = std::max(mx[k], secs[3 * r + k]);
        std::cout << "ranks " << R << " fwd_s " << mx[0] << " bwd_data_s "
                  << mx[1] << " bwd_filter_s " << mx[2] << "\n";
        return 0;
    }
    std::cerr << "unknown mode " << mode << "\n";
    return 2;
}
