// TEST INFRASTRUCTURE ONLY — python module `_apr_ref`.
//
// Compiles the reference's own CPU operators (pyapr/aprnet/src/{conv,helpers,kernel,maxpool,
// upsample,APRNetImageBuffer}.hpp), unmodified and from where they lie in the reference checkout,
// against the small LibAPR stand-in under ref_shim/.  It is used to (1) generate the golden vectors
// under tests/golden/, (2) validate this project's own CPU restatement (apr_oracle.cpp) and
// (3) serve as the timed CPU baseline.  The product library never links or imports it.
#include <omp.h>
#include <torch/extension.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/numpy.h>

#include <data_structures/APR/APR.hpp>
#include <data_structures/APR/particles/ParticleData.hpp>
#include "conv.hpp"
#include "kernel.hpp"
#include "maxpool.hpp"
#include "upsample.hpp"

namespace py = pybind11;

static void fill_access(ShimAccess& a, int lmin, int lmax, const std::vector<std::vector<int>>& dims_zxy,
                        py::array_t<int64_t, py::array::c_style | py::array::forcecast> row_ptr,
                        py::array_t<uint16_t, py::array::c_style | py::array::forcecast> y) {
    std::vector<int> zn(lmax + 1), xn(lmax + 1), yn(lmax + 1);
    for (int l = 0; l <= lmax; ++l) { zn[l] = dims_zxy[l][0]; xn[l] = dims_zxy[l][1]; yn[l] = dims_zxy[l][2]; }
    a.init(lmin, lmax, zn, xn, yn);
    a.row_ptr.assign(row_ptr.data(), row_ptr.data() + row_ptr.size());
    a.y_vec.assign(y.data(), y.data() + y.size());
    if ((int64_t) a.row_ptr.size() != a.row_off[lmax + 1] + 1) throw std::invalid_argument("row_ptr size mismatch");
    if ((int64_t) a.y_vec.size() != a.row_ptr.back()) throw std::invalid_argument("y size mismatch");
}

static torch::Tensor ref_fill_tree_mean(APR& apr, torch::Tensor input, int level_delta) {
    const int cml = apr.level_max() - level_delta;
    auto tree_it = apr.tree_iterator();
    const int64_t T = tree_it.total_number_particles(cml - 1);
    auto out = torch::zeros({input.size(0), T}, input.dtype());
    AT_DISPATCH_FLOATING_TYPES(input.scalar_type(), "ref_fill_tree_mean", ([&] {
        auto in = input.accessor<scalar_t, 2>();
        auto o = out.accessor<scalar_t, 2>();
        for (int c = 0; c < input.size(0); ++c) {
            ParticleData<scalar_t> tree;
            helpers::fill_tree_mean<true, scalar_t>(apr, in[c], tree, cml);
            for (int64_t i = 0; i < T; ++i) o[c][i] = tree[i];
        }
    }));
    return out;
}

// grad_input (C, N) is updated in place from grad_tree (C, T), as the reference does at conv.hpp:478
static torch::Tensor ref_fill_tree_mean_backward(APR& apr, torch::Tensor grad_input, torch::Tensor grad_tree, int level_delta) {
    const int cml = apr.level_max() - level_delta;
    auto out = grad_input.clone();
    AT_DISPATCH_FLOATING_TYPES(out.scalar_type(), "ref_fill_tree_mean_backward", ([&] {
        auto gi = out.accessor<scalar_t, 2>();
        auto gt = grad_tree.accessor<scalar_t, 2>();
        for (int c = 0; c < out.size(0); ++c) {
            ParticleData<scalar_t> tree(grad_tree.size(1));
            for (int64_t i = 0; i < grad_tree.size(1); ++i) tree[i] = gt[c][i];
            helpers::fill_tree_mean_backward<true, scalar_t>(apr, gi[c], tree, cml);
        }
    }));
    return out;
}

PYBIND11_MODULE(_apr_ref, m) {
    m.doc() = "reference CPU operators of pyapr.aprnet compiled against a LibAPR stand-in (test oracle)";

    py::class_<APR>(m, "APR")
        .def(py::init([](std::vector<int> shape_zxy, int level_min, int level_max,
                         std::vector<std::vector<int>> dims_zxy,
                         py::array_t<int64_t, py::array::c_style | py::array::forcecast> row_ptr,
                         py::array_t<uint16_t, py::array::c_style | py::array::forcecast> y,
                         py::array_t<int64_t, py::array::c_style | py::array::forcecast> tree_row_ptr,
                         py::array_t<uint16_t, py::array::c_style | py::array::forcecast> tree_y) {
            auto apr = std::make_unique<APR>();
            apr->dims_yxz[0] = shape_zxy[2]; apr->dims_yxz[1] = shape_zxy[1]; apr->dims_yxz[2] = shape_zxy[0];
            fill_access(apr->parts, level_min, level_max, dims_zxy, row_ptr, y);
            std::vector<std::vector<int>> tdims(dims_zxy.begin(), dims_zxy.begin() + level_max);
            fill_access(apr->tree, level_min - 1, level_max - 1, tdims, tree_row_ptr, tree_y);
            return apr;
        }))
        .def("level_min", &APR::level_min)
        .def("level_max", &APR::level_max)
        .def("total_number_particles", &APR::total_number_particles)
        .def("total_number_tree_particles", &APR::total_number_tree_particles);

    m.def("number_parts", &helpers::number_parts);
    m.def("fill_tree_mean", &ref_fill_tree_mean);
    m.def("fill_tree_mean_backward", &ref_fill_tree_mean_backward);

    m.def("convolve333_forward", &Convolution<3, 3, 3>::forward);
    m.def("convolve333_backward", &Convolution<3, 3, 3>::backward);
    m.def("convolve111_forward", &Convolution<1, 1, 1>::forward);
    m.def("convolve111_backward", &Convolution<1, 1, 1>::backward);
    m.def("restrict_kernel333_forward", &RestrictKernel<3, 3, 3>::forward);
    m.def("restrict_kernel333_backward", &RestrictKernel<3, 3, 3>::backward);
    m.def("maxpool_forward", &MaxPool::forward);
    m.def("maxpool_backward", &MaxPool::backward);
    m.def("upsample_const_forward", &UpSampleConst::forward);
    m.def("upsample_const_backward", &UpSampleConst::backward);
    m.def("set_num_threads", [](int n) { omp_set_num_threads(n); });
    m.def("get_max_threads", []() { return omp_get_max_threads(); });
}
