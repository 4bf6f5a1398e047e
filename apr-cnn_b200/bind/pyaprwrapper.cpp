// Python module `_pyaprwrapper`: the host side of the drop-in boundary.
//
// Mirrors the part of the reference's extension module that the particle-domain CNN path uses
// (wrappers/pythonBind.cpp:63-184): `data_containers.APR` / `APRPtrVector`
// (pyapr/data_containers/src/BindAPR.hpp:44-133), `aprnet.utils.number_*`
// (pyapr/aprnet/src/utils.hpp:340-382) and the `aprnet.cuda.*` operator functions
// (wrappers/pythonBind.cpp:162-181) with the same names, keyword names, tensor conventions and error
// behaviour (pyapr/aprnet/cuda/src/wrap_*_gpu.hpp).  This layer owns tensor allocation, the batch
// loop and error -> exception translation; all arithmetic happens in libaprnet_b200 behind the C ABI
// declared in include/aprnet_b200.h.  There is no CPU implementation: a non-CUDA tensor is an error.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <pybind11/stl_bind.h>
#include <pybind11/numpy.h>

#include <cmath>
#include <cstdint>
#include <memory>
#include <sstream>
#include <string>
#include <array>
#include <vector>

#include "../../include/aprnet_b200.h"

namespace py = pybind11;

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) CHECK_CUDA(x); CHECK_CONTIGUOUS(x)

// ---------------------------------------------------------------------------------------------
// APR: host copy of the linear access arrays + the device handle created by init_cuda()
// ---------------------------------------------------------------------------------------------
class APR {
public:
    std::string name;
    int org_dims_[3] = {0, 0, 0};            // (y, x, z) as in the reference's APR::org_dims
    int level_min_ = 0, level_max_ = 0;
    std::vector<int> dims_zxy;               // 3 * (level_max + 1)
    std::vector<int64_t> row_ptr, tree_row_ptr;
    std::vector<uint16_t> y_vec, tree_y_vec;
    std::vector<int64_t> row_off, trow_off;  // first row of each level
    aprnet_apr* dev = nullptr;
    int dev_index = -1;
    bool initialized = false;

    APR() = default;
    APR(const APR&) = delete;
    APR& operator=(const APR&) = delete;
    ~APR() { if (dev) aprnet_apr_destroy(dev); }

    void init(int z, int x, int y, py::array_t<int64_t, py::array::c_style | py::array::forcecast> rp,
              py::array_t<uint16_t, py::array::c_style | py::array::forcecast> yv,
              py::array_t<int64_t, py::array::c_style | py::array::forcecast> trp,
              py::array_t<uint16_t, py::array::c_style | py::array::forcecast> tyv) {
        org_dims_[0] = y; org_dims_[1] = x; org_dims_[2] = z;
        const int mx = std::max(z, std::max(x, y));
        level_max_ = std::max(1, (int) std::ceil(std::log2((double) mx)));
        level_min_ = 1;
        dims_zxy.resize(3 * (level_max_ + 1));
        for (int l = 0; l <= level_max_; ++l) {
            const double s = std::pow(2.0, level_max_ - l);
            dims_zxy[3 * l] = (int) std::ceil(z / s);
            dims_zxy[3 * l + 1] = (int) std::ceil(x / s);
            dims_zxy[3 * l + 2] = (int) std::ceil(y / s);
        }
        row_off.assign(level_max_ + 2, 0);
        trow_off.assign(level_max_ + 2, 0);
        for (int l = 0; l <= level_max_; ++l) {
            const int64_t rows = (int64_t) dims_zxy[3 * l] * dims_zxy[3 * l + 1];
            row_off[l + 1] = row_off[l] + (l >= level_min_ ? rows : 0);
            trow_off[l + 1] = trow_off[l] + (l <= level_max_ - 1 ? rows : 0);
        }
        if (rp.size() != row_off[level_max_ + 1] + 1) throw std::invalid_argument("APR: row_ptr has the wrong length");
        if (trp.size() != trow_off[level_max_] + 1) throw std::invalid_argument("APR: tree_row_ptr has the wrong length");
        row_ptr.assign(rp.data(), rp.data() + rp.size());
        tree_row_ptr.assign(trp.data(), trp.data() + trp.size());
        if (yv.size() != row_ptr.back() || tyv.size() != tree_row_ptr.back())
            throw std::invalid_argument("APR: y arrays do not match the row pointers");
        y_vec.assign(yv.data(), yv.data() + yv.size());
        tree_y_vec.assign(tyv.data(), tyv.data() + tyv.size());
        if (dev) { aprnet_apr_destroy(dev); dev = nullptr; }
        initialized = true;
    }

    int level_min() const { return level_min_; }
    int level_max() const { return level_max_; }
    int z_num(int l) const { return dims_zxy.at(3 * l); }
    int x_num(int l) const { return dims_zxy.at(3 * l + 1); }
    int y_num(int l) const { return dims_zxy.at(3 * l + 2); }
    int org_dims(int d) const { return org_dims_[d]; }
    uint64_t total_number_particles() const { return y_vec.size(); }
    uint64_t total_number_tree_particles() const { return tree_y_vec.size(); }
    double computational_ratio() const {
        return (double) org_dims_[0] * org_dims_[1] * org_dims_[2] / (double) std::max<size_t>(y_vec.size(), 1);
    }

    int64_t particles_level_end(int l) const { return row_ptr[row_off[l + 1]]; }
    int64_t tree_level_begin(int l) const { return tree_row_ptr[trow_off[l]]; }
    int64_t tree_level_end(int l) const { return tree_row_ptr[trow_off[l + 1]]; }

    // pyapr/aprnet/src/helpers.hpp:86-101
    int64_t number_parts(int level_delta) const {
        const int cml = level_max_ - level_delta;
        if (cml < 0 || cml > level_max_) throw std::invalid_argument("level_delta out of range");
        int64_t n = particles_level_end(cml);
        if (cml <= level_max_ - 1) n += tree_level_end(cml) - tree_level_begin(cml);
        return n;
    }

    // copy access structures to the current CUDA device (the reference's APR::init_cuda)
    void init_cuda(bool with_tree) {
        (void) with_tree;
        if (!initialized) throw std::runtime_error("APR is not initialized");
        const int device = (int) c10::cuda::current_device();
        if (dev && dev_index == device) return;
        if (dev) { aprnet_apr_destroy(dev); dev = nullptr; }
        const int rc = aprnet_apr_create(&dev, level_min_, level_max_, dims_zxy.data(), row_ptr.data(), y_vec.data(),
                                         tree_row_ptr.data(), tree_y_vec.data(), device);
        if (rc != APRNET_OK) throw std::runtime_error(std::string("APR.init_cuda failed: ") + aprnet_last_error());
        dev_index = device;
    }

    aprnet_apr* handle(const torch::Tensor& like) const {
        TORCH_CHECK(dev != nullptr, "APR.init_cuda() must be called before using the CUDA operators");
        TORCH_CHECK(like.device().index() == dev_index, "APR access data lives on cuda:", dev_index, " but the tensor is on ", like.device());
        return dev;
    }
};

PYBIND11_MAKE_OPAQUE(std::vector<APR*>)

namespace {

// 0 = exact fp32/fp64 CUDA-core kernels; 1 = bf16 tensor-core path for float32 3x3x3 convolutions
int g_conv_mode = 0;

// arithmetic of one call: "" = the process-wide setting, "fp32" / "bf16" = this call only (per-module option)
inline int resolve_mode(const std::string& precision) {
    if (precision.empty()) return g_conv_mode;
    if (precision == "fp32") return 0;
    if (precision == "bf16") return 1;
    throw std::invalid_argument("precision must be '', 'fp32' or 'bf16'");
}

inline void check(int rc, const char* what) {
    TORCH_CHECK(rc == APRNET_OK, what, " failed (", rc, "): ", aprnet_last_error());
}

inline int dtype_id(const torch::Tensor& t) {
    if (t.scalar_type() == torch::kFloat32) return APRNET_F32;
    if (t.scalar_type() == torch::kFloat64) return APRNET_F64;
    TORCH_CHECK(false, "aprnet CUDA operators support float32 and float64 tensors, got ", t.scalar_type());
    return -1;
}

inline void* stream_of(const torch::Tensor& t) { return (void*) at::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

inline std::vector<int> read_level_delta(const torch::Tensor& level_delta, size_t batch) {
    TORCH_CHECK(!level_delta.device().is_cuda(), "level_delta must be a CPU tensor");
    TORCH_CHECK(level_delta.scalar_type() == torch::kInt32 && level_delta.dim() == 1, "level_delta must be a 1-D int32 tensor");
    TORCH_CHECK((size_t) level_delta.size(0) >= batch, "level_delta has fewer entries than the batch");
    auto acc = level_delta.accessor<int, 1>();
    std::vector<int> out(batch);
    for (size_t i = 0; i < batch; ++i) out[i] = acc[i];
    return out;
}

inline void check_batch(const std::vector<APR*>& aprs, const torch::Tensor& t) {
    TORCH_CHECK(t.dim() == 3, "expected a (batch, channels, particles) tensor");
    TORCH_CHECK((int64_t) aprs.size() == t.size(0), "number of APRs (", aprs.size(), ") does not match the batch size (", t.size(0), ")");
}

// pyapr/aprnet/cuda/src/common.hpp:17 (CHECK_LEVEL_DELTA against tree level_max + 1 = level_max)
inline void check_level_delta(const APR& apr, int dl) {
    TORCH_CHECK(dl >= 0 && apr.level_max() > dl, "level delta ", dl, " is too large for APR with maximum level ", apr.level_max());
}

inline size_t esize(const torch::Tensor& t) { return t.element_size(); }
inline char* row(const torch::Tensor& t, int64_t b) { return (char*) t.data_ptr() + b * t.stride(0) * (int64_t) esize(t); }

// zero the padding behind the valid entries of batch item b
inline void zero_padding(torch::Tensor& t, int64_t b, int64_t valid) {
    if (valid < t.size(2)) t.select(0, b).narrow(1, valid, t.size(2) - valid).zero_();
}

// ---- 3x3x3 convolution ------------------------------------------------------------------------
static std::vector<torch::Tensor> conv333_forward_impl(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights, torch::Tensor level_delta, bool keep_tree,
                                                       const std::string& precision = "") {
    CHECK_INPUT(input); CHECK_INPUT(weights);
    check_batch(aprs, input);
    TORCH_CHECK(weights.dim() == 6 && weights.size(3) == 3 && weights.size(4) == 3 && weights.size(5) == 3, "weights must be (levels, Cout, Cin, 3, 3, 3)");
    TORCH_CHECK(input.size(1) == weights.size(2), "input tensor shape does not match weights tensor");
    TORCH_CHECK(input.scalar_type() == weights.scalar_type(), "input and weights must have the same dtype");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_tree = 1;
    for (size_t i = 0; i < aprs.size(); ++i) {
        check_level_delta(*aprs[i], dl[i]);
        max_tree = std::max<int64_t>(max_tree, aprnet_tree_size(aprs[i]->handle(input), dl[i]));
        TORCH_CHECK(aprs[i]->number_parts(dl[i]) <= input.size(2), "input has fewer particles than the APR at this level delta");
    }
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2);
    auto output = torch::empty({input.size(0), cout, n}, input.options());
    // one tree buffer per batch item when the caller keeps it for the backward pass, else one shared scratch
    auto tree_all = torch::empty({keep_tree ? input.size(0) : 1, cin, max_tree}, input.options());
    const int dt = dtype_id(input);
    const bool tc = resolve_mode(precision) == 1 && dt == APRNET_F32;
    torch::Tensor ws;
    if (tc) {
        int64_t bytes = 256;
        for (size_t i = 0; i < aprs.size(); ++i)
            bytes = std::max<int64_t>(bytes, aprnet_conv333_tc_forward_workspace_bytes(aprs[i]->handle(input), dl[i], (int) cin, (int) cout, (int) weights.size(0)));
        ws = torch::empty({bytes}, input.options().dtype(torch::kUInt8));
    }
    for (int64_t b = 0; b < input.size(0); ++b) {
        auto tree = tree_all.select(0, keep_tree ? b : 0);
        if (tc)
            check(aprnet_conv333_forward_tc(aprs[b]->handle(input), dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                            (const float*) weights.data_ptr(), (float*) row(output, b), n, (float*) tree.data_ptr(), max_tree,
                                            ws.data_ptr(), stream_of(input)), "conv333_forward (tensor cores)");
        else
            check(aprnet_conv333_forward(aprs[b]->handle(input), dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n,
                                         weights.data_ptr(), row(output, b), n, tree.data_ptr(), max_tree, stream_of(input)),
                  "conv333_forward");
        zero_padding(output, b, aprs[b]->number_parts(dl[b]));
    }
    return {output, tree_all};
}

torch::Tensor conv333_forward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights, torch::Tensor level_delta) {
    return conv333_forward_impl(aprs, input, weights, level_delta, false)[0];
}

// same, but also returns the tree means (B, Cin, T) so that the backward pass need not recompute them
std::vector<torch::Tensor> conv333_forward_keep_tree(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights, torch::Tensor level_delta,
                                                     const std::string& precision) {
    return conv333_forward_impl(aprs, input, weights, level_delta, true, precision);
}

// Tensor-core forward that keeps the packed bf16 rows of the input (particles, tree means, zero row) for the
// backward pass instead of the fp32 input and the tree means: returns {output, rows (B, bytes) uint8}.
std::vector<torch::Tensor> conv333_forward_keep_rows(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights, torch::Tensor level_delta) {
    CHECK_INPUT(input); CHECK_INPUT(weights);
    check_batch(aprs, input);
    TORCH_CHECK(weights.dim() == 6 && weights.size(3) == 3 && weights.size(4) == 3 && weights.size(5) == 3, "weights must be (levels, Cout, Cin, 3, 3, 3)");
    TORCH_CHECK(input.size(1) == weights.size(2), "input tensor shape does not match weights tensor");
    TORCH_CHECK(input.scalar_type() == torch::kFloat32 && weights.scalar_type() == torch::kFloat32, "the tensor-core path takes float32 tensors");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2);
    int64_t max_tree = 1, rows_bytes = 256, w_bytes = 256;
    for (size_t i = 0; i < aprs.size(); ++i) {
        check_level_delta(*aprs[i], dl[i]);
        aprnet_apr* h = aprs[i]->handle(input);
        TORCH_CHECK(aprs[i]->number_parts(dl[i]) <= n, "input has fewer particles than the APR at this level delta");
        max_tree = std::max<int64_t>(max_tree, aprnet_tree_size(h, dl[i]));
        const int64_t rb = aprnet_conv333_tc_packed_rows_bytes(h, dl[i], (int) cin);
        rows_bytes = std::max(rows_bytes, rb);
        w_bytes = std::max(w_bytes, aprnet_conv333_tc_forward_workspace_bytes(h, dl[i], (int) cin, (int) cout, (int) weights.size(0)) - rb);
    }
    auto output = torch::empty({input.size(0), cout, n}, input.options());
    auto tree = torch::empty({cin, max_tree}, input.options());
    // per batch item: [packed rows | packed weights]; only the rows part is handed back (the view keeps the buffer)
    auto ws = torch::empty({input.size(0), rows_bytes + w_bytes}, input.options().dtype(torch::kUInt8));
    for (int64_t b = 0; b < input.size(0); ++b) {
        check(aprnet_conv333_forward_tc(aprs[b]->handle(input), dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                        (const float*) weights.data_ptr(), (float*) row(output, b), n, (float*) tree.data_ptr(), max_tree,
                                        row(ws, b), stream_of(input)), "conv333_forward (tensor cores)");
        zero_padding(output, b, aprs[b]->number_parts(dl[b]));
    }
    return {output, ws};
}

std::vector<torch::Tensor> conv333_backward_with_rows(std::vector<APR*>& aprs, torch::Tensor rows, torch::Tensor weights, torch::Tensor grad_output,
                                                      torch::Tensor level_delta, bool need_grad_input) {
    CHECK_INPUT(weights); CHECK_INPUT(grad_output); CHECK_INPUT(rows);
    check_batch(aprs, grad_output);
    TORCH_CHECK(rows.dim() == 2 && rows.size(0) == grad_output.size(0) && rows.scalar_type() == torch::kUInt8, "rows must be the (batch, bytes) buffer of conv333_forward_keep_rows");
    TORCH_CHECK(grad_output.dim() == 3 && grad_output.size(1) == weights.size(1) && grad_output.scalar_type() == torch::kFloat32, "grad_output shape does not match");
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = weights.size(2), cout = weights.size(1), n = grad_output.size(2);
    int64_t max_tree = 1, bytes = 256;
    for (size_t i = 0; i < aprs.size(); ++i) {
        check_level_delta(*aprs[i], dl[i]);
        aprnet_apr* h = aprs[i]->handle(grad_output);
        max_tree = std::max<int64_t>(max_tree, aprnet_tree_size(h, dl[i]));
        TORCH_CHECK(rows.size(1) >= aprnet_conv333_tc_packed_rows_bytes(h, dl[i], (int) cin), "rows buffer too small for this APR");
        bytes = std::max<int64_t>(bytes, aprnet_conv333_tc_workspace_bytes(h, dl[i], (int) cin, (int) cout, (int) weights.size(0)));
    }
    auto grad_tree = torch::empty({cin, max_tree}, grad_output.options());
    auto grad_input = need_grad_input ? torch::empty({grad_output.size(0), cin, n}, grad_output.options()) : torch::Tensor();
    auto grad_weights = torch::zeros_like(weights);
    auto ws = torch::empty({bytes}, grad_output.options().dtype(torch::kUInt8));
    auto partial = torch::empty({aprnet_conv333_tc_dw_partial_elems((int) cin, (int) cout)}, grad_output.options());
    for (int64_t b = 0; b < grad_output.size(0); ++b) {
        check(aprnet_conv333_backward_tc_rows(aprs[b]->handle(grad_output), dl[b], (int) cin, (int) cout, (int) weights.size(0), row(rows, b),
                                              (const float*) row(grad_output, b), n, (const float*) weights.data_ptr(),
                                              need_grad_input ? (float*) row(grad_input, b) : nullptr, n, (float*) grad_weights.data_ptr(),
                                              (float*) grad_tree.data_ptr(), max_tree, (float*) partial.data_ptr(), ws.data_ptr(), stream_of(grad_output)),
              "conv333_backward (tensor cores, packed rows)");
        if (need_grad_input) zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
    }
    return {grad_input, grad_weights};
}

static std::vector<torch::Tensor> conv333_backward_impl(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights,
                                            torch::Tensor grad_output, torch::Tensor level_delta, c10::optional<torch::Tensor> saved_tree,
                                            bool need_grad_input = true, const std::string& precision = "") {
    CHECK_INPUT(input); CHECK_INPUT(weights); CHECK_INPUT(grad_output);
    check_batch(aprs, input);
    TORCH_CHECK(grad_output.dim() == 3 && grad_output.size(0) == input.size(0) && grad_output.size(1) == weights.size(1) &&
                grad_output.size(2) == input.size(2), "grad_output shape does not match");
    TORCH_CHECK(input.size(1) == weights.size(2), "input tensor shape does not match weights tensor");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_tree = 1;
    for (size_t i = 0; i < aprs.size(); ++i) {
        check_level_delta(*aprs[i], dl[i]);
        max_tree = std::max<int64_t>(max_tree, aprnet_tree_size(aprs[i]->handle(input), dl[i]));
    }
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2);
    const int dt = dtype_id(input);
    void* st = stream_of(input);
    const bool tc = resolve_mode(precision) == 1 && dt == APRNET_F32;
    const bool skip_gin = tc && !need_grad_input;        // only the tensor-core driver can leave the input gradient out
    const bool have_tree = saved_tree.has_value() && saved_tree->defined() && saved_tree->dim() == 3 && saved_tree->size(0) == input.size(0) &&
                           saved_tree->size(1) == cin && saved_tree->size(2) == max_tree && saved_tree->is_contiguous() &&
                           saved_tree->scalar_type() == input.scalar_type();
    auto tree_all = have_tree ? *saved_tree : torch::empty({1, cin, max_tree}, input.options());
    auto grad_tree = torch::empty({cin, max_tree}, input.options());
    // the tensor-core path writes every valid entry of grad_input; the CUDA-core path accumulates into zeros
    auto grad_input = skip_gin ? torch::Tensor() : (tc ? torch::empty_like(input) : torch::zeros_like(input));
    auto grad_weights = torch::zeros_like(weights);
    torch::Tensor partial;
    if (!tc) partial = torch::empty({aprnet_conv333_partial_elems((int) cin, (int) cout)}, input.options());
    torch::Tensor ws;
    if (tc) {
        int64_t bytes = 256;
        for (size_t i = 0; i < aprs.size(); ++i)
            bytes = std::max<int64_t>(bytes, aprnet_conv333_tc_workspace_bytes(aprs[i]->handle(input), dl[i], (int) cin, (int) cout, (int) weights.size(0)));
        ws = torch::empty({bytes}, input.options().dtype(torch::kUInt8));
    }
    torch::Tensor partial_tc;
    if (tc) partial_tc = torch::empty({aprnet_conv333_tc_dw_partial_elems((int) cin, (int) cout)}, input.options());
    for (int64_t b = 0; b < input.size(0); ++b) {
        aprnet_apr* h = aprs[b]->handle(input);
        auto tree = tree_all.select(0, have_tree ? b : 0);
        if (tc) {
            check(aprnet_conv333_backward_tc(h, dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                             (const float*) row(grad_output, b), n, (const float*) weights.data_ptr(),
                                             skip_gin ? nullptr : (float*) row(grad_input, b), (float*) grad_weights.data_ptr(), (float*) tree.data_ptr(),
                                             have_tree ? 1 : 0, (float*) grad_tree.data_ptr(), max_tree, (float*) partial_tc.data_ptr(),
                                             ws.data_ptr(), st),
                  "conv333_backward (tensor cores)");
            if (!skip_gin) zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
            continue;
        }
        if (!have_tree)
        check(aprnet_fill_tree_mean_forward(h, dl[b], dt, (int) cin, row(input, b), n, tree.data_ptr(), max_tree, st), "fill_tree_mean");
        check(aprnet_conv333_backward_weights(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n,
                                              tree.data_ptr(), max_tree, row(grad_output, b), n, grad_weights.data_ptr(),
                                              partial.data_ptr(), st), "conv333_backward_weights");
        check(aprnet_conv333_backward_input(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(grad_output, b), n,
                                            weights.data_ptr(), row(grad_input, b), n, grad_tree.data_ptr(), max_tree, st),
              "conv333_backward_input");
    }
    return {grad_input, grad_weights};
}

std::vector<torch::Tensor> conv333_backward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights,
                                            torch::Tensor grad_output, torch::Tensor level_delta) {
    return conv333_backward_impl(aprs, input, weights, grad_output, level_delta, c10::nullopt);
}

std::vector<torch::Tensor> conv333_backward_with_tree(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights,
                                                      torch::Tensor grad_output, torch::Tensor level_delta, torch::Tensor tree,
                                                      bool need_grad_input, const std::string& precision) {
    return conv333_backward_impl(aprs, input, weights, grad_output, level_delta, tree, need_grad_input, precision);
}

// ---- 3x3x3 convolution, split forms for one z-slab of an APR per GPU (pyapr/aprnet/cuda/sharded.py) ----------
// forward with given tree means (B, Cin, T); returns {output, kept}: kept = packed bf16 rows (bf16 mode) or an empty tensor
std::vector<torch::Tensor> conv333_forward_pretree(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor tree, torch::Tensor weights,
                                                   torch::Tensor level_delta, const std::string& precision) {
    CHECK_INPUT(input); CHECK_INPUT(weights); CHECK_INPUT(tree);
    check_batch(aprs, input);
    TORCH_CHECK(weights.dim() == 6 && weights.size(3) == 3 && weights.size(4) == 3 && weights.size(5) == 3, "weights must be (levels, Cout, Cin, 3, 3, 3)");
    TORCH_CHECK(input.size(1) == weights.size(2), "input tensor shape does not match weights tensor");
    TORCH_CHECK(tree.dim() == 3 && tree.size(0) == input.size(0) && tree.size(1) == input.size(1) && tree.scalar_type() == input.scalar_type(),
                "tree must be (batch, Cin, tree nodes) of the input's dtype");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2), ldt = tree.size(2);
    const int dt = dtype_id(input);
    const bool tc = resolve_mode(precision) == 1 && dt == APRNET_F32;
    int64_t rows_bytes = 256, w_bytes = 256;
    for (size_t i = 0; i < aprs.size(); ++i) {
        check_level_delta(*aprs[i], dl[i]);
        aprnet_apr* h = aprs[i]->handle(input);
        TORCH_CHECK(aprs[i]->number_parts(dl[i]) <= n && aprnet_tree_size(h, dl[i]) <= ldt, "input or tree has fewer entries than the APR at this level delta");
        if (tc) {
            const int64_t rb = aprnet_conv333_tc_packed_rows_bytes(h, dl[i], (int) cin);
            rows_bytes = std::max(rows_bytes, rb);
            w_bytes = std::max(w_bytes, aprnet_conv333_tc_forward_workspace_bytes(h, dl[i], (int) cin, (int) cout, (int) weights.size(0)) - rb);
        }
    }
    auto output = torch::empty({input.size(0), cout, n}, input.options());
    torch::Tensor ws = tc ? torch::empty({input.size(0), rows_bytes + w_bytes}, input.options().dtype(torch::kUInt8)) : torch::Tensor();
    for (int64_t b = 0; b < input.size(0); ++b) {
        if (tc)
            check(aprnet_conv333_forward_tc_pretree(aprs[b]->handle(input), dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                                    (const float*) weights.data_ptr(), (float*) row(output, b), n, (const float*) row(tree, b), ldt,
                                                    row(ws, b), stream_of(input)), "conv333_forward_pretree (tensor cores)");
        else
            check(aprnet_conv333_forward_pretree(aprs[b]->handle(input), dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n,
                                                 weights.data_ptr(), row(output, b), n, row(tree, b), ldt, stream_of(input)), "conv333_forward_pretree");
        zero_padding(output, b, aprs[b]->number_parts(dl[b]));
    }
    return {output, tc ? ws : torch::empty({0}, input.options().dtype(torch::kUInt8))};
}

// backward without the tree adjoint: returns {grad_input (direct contributions), grad_tree (B, Cin, T), grad_weights}.
// bf16 mode: `kept` is the rows buffer of conv333_forward_pretree and `input` is not read; otherwise input and tree are used.
std::vector<torch::Tensor> conv333_backward_pretree(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor tree, torch::Tensor kept, torch::Tensor weights,
                                                    torch::Tensor grad_output, torch::Tensor level_delta, bool need_grad_input) {
    CHECK_INPUT(weights); CHECK_INPUT(grad_output); CHECK_INPUT(tree);
    check_batch(aprs, grad_output);
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = weights.size(2), cout = weights.size(1), n = grad_output.size(2), ldt = tree.size(2), B = grad_output.size(0);
    const int dt = dtype_id(grad_output);
    const bool tc = dt == APRNET_F32 && kept.numel() > 0;          // a rows buffer exists only when the forward call ran on the tensor cores
    TORCH_CHECK(grad_output.size(1) == cout && tree.dim() == 3 && tree.size(0) == B && tree.size(1) == cin, "shapes do not match");
    if (!tc) { CHECK_INPUT(input); TORCH_CHECK(input.dim() == 3 && input.size(1) == cin && input.size(2) == n, "input shape does not match"); }
    auto grad_tree = torch::zeros({B, cin, ldt}, grad_output.options());
    auto grad_weights = torch::zeros_like(weights);
    torch::Tensor grad_input;
    void* st = stream_of(grad_output);
    if (tc) {
        int64_t bytes = 256;
        for (size_t i = 0; i < aprs.size(); ++i) {
            check_level_delta(*aprs[i], dl[i]);
            aprnet_apr* h = aprs[i]->handle(grad_output);
            TORCH_CHECK(kept.dim() == 2 && kept.size(0) == B && kept.size(1) >= aprnet_conv333_tc_packed_rows_bytes(h, dl[i], (int) cin), "rows buffer too small for this APR");
            bytes = std::max<int64_t>(bytes, aprnet_conv333_tc_workspace_bytes(h, dl[i], (int) cin, (int) cout, (int) weights.size(0)));
        }
        if (need_grad_input) grad_input = torch::empty({B, cin, n}, grad_output.options());
        auto ws = torch::empty({bytes}, grad_output.options().dtype(torch::kUInt8));
        auto partial = torch::empty({aprnet_conv333_tc_dw_partial_elems((int) cin, (int) cout)}, grad_output.options());
        for (int64_t b = 0; b < B; ++b) {
            check(aprnet_conv333_backward_tc_rows_pretree(aprs[b]->handle(grad_output), dl[b], (int) cin, (int) cout, (int) weights.size(0), row(kept, b),
                                                          (const float*) row(grad_output, b), n, (const float*) weights.data_ptr(),
                                                          need_grad_input ? (float*) row(grad_input, b) : nullptr, n, (float*) grad_weights.data_ptr(),
                                                          (float*) row(grad_tree, b), ldt, (float*) partial.data_ptr(), ws.data_ptr(), st),
                  "conv333_backward_pretree (tensor cores)");
            if (need_grad_input) zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
        }
    } else {
        auto partial = torch::empty({aprnet_conv333_partial_elems((int) cin, (int) cout)}, grad_output.options());
        grad_input = torch::zeros({B, cin, n}, grad_output.options());
        for (int64_t b = 0; b < B; ++b) {
            check_level_delta(*aprs[b], dl[b]);
            aprnet_apr* h = aprs[b]->handle(grad_output);
            check(aprnet_conv333_backward_weights(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n, row(tree, b), ldt,
                                                  row(grad_output, b), n, grad_weights.data_ptr(), partial.data_ptr(), st), "conv333_backward_weights");
            if (need_grad_input)
                check(aprnet_conv333_backward_input_pretree(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(grad_output, b), n,
                                                            weights.data_ptr(), row(grad_input, b), n, row(grad_tree, b), ldt, st), "conv333_backward_input_pretree");
        }
    }
    return {grad_input, grad_tree, grad_weights};
}

// tree means of a batch (B, C, N) -> (B, C, T); and the adjoint applied in place to grad_input / grad_tree
torch::Tensor fill_tree_mean_batch(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor level_delta) {
    CHECK_INPUT(input);
    check_batch(aprs, input);
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_tree = 1;
    for (size_t i = 0; i < aprs.size(); ++i) { check_level_delta(*aprs[i], dl[i]); max_tree = std::max<int64_t>(max_tree, aprnet_tree_size(aprs[i]->handle(input), dl[i])); }
    auto tree = torch::zeros({input.size(0), input.size(1), max_tree}, input.options());
    for (int64_t b = 0; b < input.size(0); ++b)
        check(aprnet_fill_tree_mean_forward(aprs[b]->handle(input), dl[b], dtype_id(input), (int) input.size(1), row(input, b), input.size(2),
                                            row(tree, b), max_tree, stream_of(input)), "fill_tree_mean");
    return tree;
}

void fill_tree_mean_backward_inplace(std::vector<APR*>& aprs, torch::Tensor grad_input, torch::Tensor grad_tree, torch::Tensor level_delta) {
    CHECK_INPUT(grad_input); CHECK_INPUT(grad_tree);
    check_batch(aprs, grad_input);
    TORCH_CHECK(grad_tree.dim() == 3 && grad_tree.size(0) == grad_input.size(0) && grad_tree.size(1) == grad_input.size(1), "grad_tree must be (batch, channels, tree nodes)");
    c10::cuda::CUDAGuard guard(grad_input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    for (int64_t b = 0; b < grad_input.size(0); ++b) {
        check_level_delta(*aprs[b], dl[b]);
        TORCH_CHECK(aprnet_tree_size(aprs[b]->handle(grad_input), dl[b]) <= grad_tree.size(2), "grad_tree has fewer nodes than the APR at this level delta");
        check(aprnet_fill_tree_mean_backward(aprs[b]->handle(grad_input), dl[b], dtype_id(grad_input), (int) grad_input.size(1), row(grad_input, b), grad_input.size(2),
                                             row(grad_tree, b), grad_tree.size(2), stream_of(grad_input)), "fill_tree_mean_backward");
    }
}

// ---- 1x1x1 convolution ------------------------------------------------------------------------
torch::Tensor conv111_forward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights, torch::Tensor level_delta,
                              const std::string& precision) {
    CHECK_INPUT(input); CHECK_INPUT(weights);
    check_batch(aprs, input);
    TORCH_CHECK(weights.dim() == 6 && weights.size(3) == 1 && weights.size(4) == 1 && weights.size(5) == 1, "weights must be (stencils, Cout, Cin, 1, 1, 1)");
    TORCH_CHECK(input.size(1) == weights.size(2), "input tensor shape does not match weights tensor");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2);
    auto output = torch::empty({input.size(0), cout, n}, input.options());
    const int dt = dtype_id(input);
    const bool tc = resolve_mode(precision) == 1 && dt == APRNET_F32;
    for (int64_t b = 0; b < input.size(0); ++b) {
        check_level_delta(*aprs[b], dl[b]);
        // tensor cores where the layer asks for bf16 arithmetic and the weights fit shared memory; CUDA cores otherwise
        int rc = APRNET_ERR_UNSUPPORTED;
        if (tc) {
            rc = aprnet_conv111_forward_tc(aprs[b]->handle(input), dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                           (const float*) weights.data_ptr(), (float*) row(output, b), n, stream_of(input));
            if (rc != APRNET_ERR_UNSUPPORTED) check(rc, "conv111_forward (tensor cores)");
        }
        if (rc == APRNET_ERR_UNSUPPORTED)
        check(aprnet_conv111_forward(aprs[b]->handle(input), dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n,
                                     weights.data_ptr(), row(output, b), n, stream_of(input)), "conv111_forward");
        zero_padding(output, b, aprs[b]->number_parts(dl[b]));
    }
    return output;
}

std::vector<torch::Tensor> conv111_backward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor weights,
                                            torch::Tensor grad_output, torch::Tensor level_delta, const std::string& precision) {
    CHECK_INPUT(input); CHECK_INPUT(weights); CHECK_INPUT(grad_output);
    check_batch(aprs, input);
    TORCH_CHECK(grad_output.dim() == 3 && grad_output.size(1) == weights.size(1) && grad_output.size(2) == input.size(2), "grad_output shape does not match");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    const int64_t cin = input.size(1), cout = weights.size(1), n = input.size(2);
    auto grad_input = torch::empty_like(input);
    auto grad_weights = torch::zeros_like(weights);
    auto partial = torch::empty({aprnet_conv111_partial_elems((int) cin, (int) cout)}, input.options());
    const int dt = dtype_id(input);
    const bool tc = resolve_mode(precision) == 1 && dt == APRNET_F32;
    void* st = stream_of(input);
    for (int64_t b = 0; b < input.size(0); ++b) {
        check_level_delta(*aprs[b], dl[b]);
        aprnet_apr* h = aprs[b]->handle(input);
        int rc = APRNET_ERR_UNSUPPORTED;
        if (tc) {
            rc = aprnet_conv111_backward_input_tc(h, dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(grad_output, b), n,
                                                  (const float*) weights.data_ptr(), (float*) row(grad_input, b), n, st);
            if (rc != APRNET_ERR_UNSUPPORTED) check(rc, "conv111_backward_input (tensor cores)");
        }
        if (rc == APRNET_ERR_UNSUPPORTED)
        check(aprnet_conv111_backward_input(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(grad_output, b), n,
                                            weights.data_ptr(), row(grad_input, b), n, st), "conv111_backward_input");
        zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
        rc = APRNET_ERR_UNSUPPORTED;
        if (tc) {
            rc = aprnet_conv111_backward_weights_tc(h, dl[b], (int) cin, (int) cout, (int) weights.size(0), (const float*) row(input, b), n,
                                                    (const float*) row(grad_output, b), n, (float*) grad_weights.data_ptr(),
                                                    (float*) partial.data_ptr(), partial.numel(), st);
            if (rc != APRNET_ERR_UNSUPPORTED) check(rc, "conv111_backward_weights (tensor cores)");
        }
        if (rc == APRNET_ERR_UNSUPPORTED)
        check(aprnet_conv111_backward_weights(h, dl[b], dt, (int) cin, (int) cout, (int) weights.size(0), row(input, b), n,
                                              row(grad_output, b), n, grad_weights.data_ptr(), partial.data_ptr(), st),
              "conv111_backward_weights");
    }
    return {grad_input, grad_weights};
}

// ---- restriction --------------------------------------------------------------------------------
torch::Tensor restrict_kernel_333_forward(torch::Tensor weights, const int num_levels) {
    CHECK_INPUT(weights);
    TORCH_CHECK(weights.dim() == 6, "weights must be 6-dimensional");
    TORCH_CHECK(num_levels >= weights.size(0), "restrict_kernel_333_forward requires num_levels >= weights.shape[0]");
    c10::cuda::CUDAGuard guard(weights.device());
    auto output = torch::empty({num_levels, weights.size(1), weights.size(2), 3, 3, 3}, weights.options());
    check(aprnet_restrict333_forward(dtype_id(weights), (int) weights.size(0), num_levels, weights.size(1) * weights.size(2),
                                     weights.data_ptr(), output.data_ptr(), stream_of(weights)), "restrict_kernel333_forward");
    return output;
}

torch::Tensor restrict_kernel_333_backward(torch::Tensor grad_weights_expanded, const int num_levels) {
    CHECK_INPUT(grad_weights_expanded);
    TORCH_CHECK(num_levels <= grad_weights_expanded.size(0), "restrict_kernel_333_backward requires num_levels <= grad_weights_expanded.shape[0]");
    c10::cuda::CUDAGuard guard(grad_weights_expanded.device());
    auto g = grad_weights_expanded;
    auto output = torch::empty({num_levels, g.size(1), g.size(2), 3, 3, 3}, g.options());
    check(aprnet_restrict333_backward(dtype_id(g), num_levels, (int) g.size(0), g.size(1) * g.size(2), g.data_ptr(), output.data_ptr(),
                                      stream_of(g)), "restrict_kernel333_backward");
    return output;
}

// ---- max pooling --------------------------------------------------------------------------------
std::vector<torch::Tensor> maxpool_forward_cuda(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor level_delta) {
    CHECK_INPUT(input);
    check_batch(aprs, input);
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) {
        TORCH_CHECK(dl[i] >= 0 && aprs[i]->level_max() - dl[i] - 1 >= aprs[i]->level_min(), "level delta ", dl[i], " is too large to pool this APR");
        max_size = std::max(max_size, aprs[i]->number_parts(dl[i] + 1));
    }
    auto output = torch::empty({input.size(0), input.size(1), max_size}, input.options());
    auto max_indices = torch::zeros({input.size(0), input.size(1), max_size}, input.options().dtype(torch::kLong));
    const int dt = dtype_id(input);
    for (int64_t b = 0; b < input.size(0); ++b) {
        check(aprnet_maxpool_forward(aprs[b]->handle(input), dl[b], dt, (int) input.size(1), row(input, b), input.size(2), row(output, b),
                                     (int64_t*) row(max_indices, b), max_size, stream_of(input)), "maxpool_forward");
        zero_padding(output, b, aprs[b]->number_parts(dl[b] + 1));
    }
    return {output, max_indices};
}

torch::Tensor maxpool_backward_cuda(std::vector<APR*>& aprs, torch::Tensor grad_output, torch::Tensor max_indices, torch::Tensor level_delta) {
    CHECK_INPUT(grad_output); CHECK_INPUT(max_indices);
    check_batch(aprs, grad_output);
    TORCH_CHECK(max_indices.scalar_type() == torch::kLong && max_indices.sizes() == grad_output.sizes(), "max_indices must be int64 with the shape of grad_output");
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) max_size = std::max(max_size, aprs[i]->number_parts(dl[i]));
    auto grad_input = torch::zeros({grad_output.size(0), grad_output.size(1), max_size}, grad_output.options());
    const int dt = dtype_id(grad_output);
    for (int64_t b = 0; b < grad_output.size(0); ++b)
        check(aprnet_maxpool_backward(aprs[b]->handle(grad_output), dl[b], dt, (int) grad_output.size(1), row(grad_output, b),
                                      (const int64_t*) row(max_indices, b), grad_output.size(2), row(grad_input, b), max_size,
                                      stream_of(grad_output)), "maxpool_backward");
    return grad_input;
}

// ---- up-sampling --------------------------------------------------------------------------------
torch::Tensor upsample_const_forward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor level_delta) {
    CHECK_INPUT(input);
    check_batch(aprs, input);
    TORCH_CHECK(level_delta.min().item<int>() > 0, "upsample_const_forward assumes all inputs to have level_delta > 0");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) max_size = std::max(max_size, aprs[i]->number_parts(dl[i] - 1));
    auto output = torch::empty({input.size(0), input.size(1), max_size}, input.options());
    const int dt = dtype_id(input);
    for (int64_t b = 0; b < input.size(0); ++b) {
        check(aprnet_upsample_forward(aprs[b]->handle(input), dl[b], dt, (int) input.size(1), row(input, b), input.size(2), row(output, b),
                                      max_size, stream_of(input)), "upsample_const_forward");
        zero_padding(output, b, aprs[b]->number_parts(dl[b] - 1));
    }
    return output;
}

torch::Tensor upsample_const_backward(std::vector<APR*>& aprs, torch::Tensor grad_output, torch::Tensor level_delta) {
    CHECK_INPUT(grad_output);
    check_batch(aprs, grad_output);
    TORCH_CHECK(level_delta.min().item<int>() > 0, "upsample_const_backward assumes all inputs to have level_delta > 0");
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) max_size = std::max(max_size, aprs[i]->number_parts(dl[i]));
    auto grad_input = torch::empty({grad_output.size(0), grad_output.size(1), max_size}, grad_output.options());
    const int dt = dtype_id(grad_output);
    for (int64_t b = 0; b < grad_output.size(0); ++b) {
        check(aprnet_upsample_backward(aprs[b]->handle(grad_output), dl[b], dt, (int) grad_output.size(1), row(grad_output, b),
                                       grad_output.size(2), row(grad_input, b), max_size, stream_of(grad_output)), "upsample_const_backward");
        zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
    }
    return grad_input;
}

// ---- particles <-> dense image (wrap_reconstruct_gpu.hpp:29-98, wrap_sample_particles_gpu.hpp:29-98) ----
static std::array<int64_t, 3> image_extent(std::vector<APR*>& aprs, const std::vector<int>& dl, const torch::Tensor& like) {
    std::array<int64_t, 3> e = {0, 0, 0};
    for (size_t i = 0; i < aprs.size(); ++i) {
        int z, x, y;
        check(aprnet_image_dims(aprs[i]->handle(like), dl[i], &z, &x, &y), "image_dims");
        e[0] = std::max<int64_t>(e[0], z); e[1] = std::max<int64_t>(e[1], x); e[2] = std::max<int64_t>(e[2], y);
    }
    return e;
}

// the C functions take one image of exactly the APR's extents; a batch whose APRs differ in size is padded
static void check_same_extent(std::vector<APR*>& aprs, const std::vector<int>& dl, const torch::Tensor& like, const std::array<int64_t, 3>& e) {
    for (size_t i = 0; i < aprs.size(); ++i) {
        int z, x, y;
        check(aprnet_image_dims(aprs[i]->handle(like), dl[i], &z, &x, &y), "image_dims");
        TORCH_CHECK(z == e[0] && x == e[1] && y == e[2], "all APRs of a batch must have the same image extents at their level_delta");
    }
}

torch::Tensor reconstruct_forward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor level_delta) {
    CHECK_INPUT(input);
    check_batch(aprs, input);
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    for (size_t i = 0; i < aprs.size(); ++i) check_level_delta(*aprs[i], dl[i]);
    const auto e = image_extent(aprs, dl, input);
    check_same_extent(aprs, dl, input, e);
    auto output = torch::empty({input.size(0), input.size(1), e[0], e[1], e[2]}, input.options());
    for (int64_t b = 0; b < input.size(0); ++b)
        check(aprnet_reconstruct_forward(aprs[b]->handle(input), dl[b], dtype_id(input), (int) input.size(1), row(input, b), input.size(2),
                                         row(output, b), stream_of(input)), "reconstruct_forward");
    return output;
}

torch::Tensor reconstruct_backward(std::vector<APR*>& aprs, torch::Tensor grad_output, torch::Tensor level_delta) {
    CHECK_INPUT(grad_output);
    TORCH_CHECK(grad_output.dim() == 5 && (size_t) grad_output.size(0) == aprs.size(), "expected (batch, channels, z, x, y)");
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) { check_level_delta(*aprs[i], dl[i]); max_size = std::max(max_size, aprs[i]->number_parts(dl[i])); }
    check_same_extent(aprs, dl, grad_output, {grad_output.size(2), grad_output.size(3), grad_output.size(4)});
    auto grad_input = torch::empty({grad_output.size(0), grad_output.size(1), max_size}, grad_output.options());
    for (int64_t b = 0; b < grad_output.size(0); ++b) {
        check(aprnet_reconstruct_backward(aprs[b]->handle(grad_output), dl[b], dtype_id(grad_output), (int) grad_output.size(1), row(grad_output, b),
                                          row(grad_input, b), max_size, stream_of(grad_output)), "reconstruct_backward");
        zero_padding(grad_input, b, aprs[b]->number_parts(dl[b]));
    }
    return grad_input;
}

torch::Tensor sample_particles_forward(std::vector<APR*>& aprs, torch::Tensor input, torch::Tensor level_delta) {
    CHECK_INPUT(input);
    TORCH_CHECK(input.dim() == 5 && (size_t) input.size(0) == aprs.size(), "expected (batch, channels, z, x, y)");
    c10::cuda::CUDAGuard guard(input.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    int64_t max_size = 0;
    for (size_t i = 0; i < aprs.size(); ++i) { check_level_delta(*aprs[i], dl[i]); max_size = std::max(max_size, aprs[i]->number_parts(dl[i])); }
    check_same_extent(aprs, dl, input, {input.size(2), input.size(3), input.size(4)});
    auto output = torch::empty({input.size(0), input.size(1), max_size}, input.options());
    for (int64_t b = 0; b < input.size(0); ++b) {
        check(aprnet_sample_particles_forward(aprs[b]->handle(input), dl[b], dtype_id(input), (int) input.size(1), row(input, b),
                                              row(output, b), max_size, stream_of(input)), "sample_particles_forward");
        zero_padding(output, b, aprs[b]->number_parts(dl[b]));
    }
    return output;
}

torch::Tensor sample_particles_backward(std::vector<APR*>& aprs, torch::Tensor grad_output, torch::Tensor level_delta) {
    CHECK_INPUT(grad_output);
    check_batch(aprs, grad_output);
    c10::cuda::CUDAGuard guard(grad_output.device());
    const auto dl = read_level_delta(level_delta, aprs.size());
    for (size_t i = 0; i < aprs.size(); ++i) check_level_delta(*aprs[i], dl[i]);
    const auto e = image_extent(aprs, dl, grad_output);
    check_same_extent(aprs, dl, grad_output, e);
    auto grad_input = torch::empty({grad_output.size(0), grad_output.size(1), e[0], e[1], e[2]}, grad_output.options());
    for (int64_t b = 0; b < grad_output.size(0); ++b)
        check(aprnet_sample_particles_backward(aprs[b]->handle(grad_output), dl[b], dtype_id(grad_output), (int) grad_output.size(1),
                                               row(grad_output, b), grad_output.size(2), row(grad_input, b), stream_of(grad_output)),
              "sample_particles_backward");
    return grad_input;
}

// ---- fused GroupNorm + ReLU ---------------------------------------------------------------------------
std::vector<torch::Tensor> groupnorm_relu_forward(torch::Tensor x, c10::optional<torch::Tensor> gamma, c10::optional<torch::Tensor> beta,
                                                  int64_t groups, double eps, bool relu) {
    CHECK_INPUT(x);
    TORCH_CHECK(x.dim() == 3 && x.size(1) % groups == 0, "expected (batch, channels, n) with channels divisible by groups");
    c10::cuda::CUDAGuard guard(x.device());
    auto y = torch::empty_like(x);
    auto mean = torch::empty({x.size(0) * groups}, x.options());
    auto rstd = torch::empty({x.size(0) * groups}, x.options());
    auto ws = torch::empty({aprnet_groupnorm_workspace_bytes((int) x.size(0), (int) x.size(1), (int) groups)}, x.options().dtype(torch::kUInt8));
    const void* g = gamma.has_value() && gamma->defined() ? gamma->contiguous().data_ptr() : nullptr;
    const void* b = beta.has_value() && beta->defined() ? beta->contiguous().data_ptr() : nullptr;
    check(aprnet_groupnorm_relu_forward(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), (int) groups, x.data_ptr(), g, b, eps,
                                        y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), ws.data_ptr(), relu ? 1 : 0, stream_of(x)), "groupnorm_relu_forward");
    return {y, mean, rstd};
}

std::vector<torch::Tensor> groupnorm_relu_backward(torch::Tensor x, torch::Tensor grad_y, c10::optional<torch::Tensor> gamma,
                                                   c10::optional<torch::Tensor> beta, torch::Tensor mean, torch::Tensor rstd,
                                                   int64_t groups, bool relu) {
    CHECK_INPUT(x); CHECK_INPUT(grad_y); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    TORCH_CHECK(x.sizes() == grad_y.sizes(), "grad_y must have the shape of x");
    c10::cuda::CUDAGuard guard(x.device());
    auto dx = torch::empty_like(x);
    auto dgamma = torch::empty({x.size(1)}, x.options());
    auto dbeta = torch::empty({x.size(1)}, x.options());
    auto ws = torch::empty({aprnet_groupnorm_workspace_bytes((int) x.size(0), (int) x.size(1), (int) groups)}, x.options().dtype(torch::kUInt8));
    const void* g = gamma.has_value() && gamma->defined() ? gamma->contiguous().data_ptr() : nullptr;
    const void* b = beta.has_value() && beta->defined() ? beta->contiguous().data_ptr() : nullptr;
    check(aprnet_groupnorm_relu_backward(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), (int) groups, x.data_ptr(), grad_y.data_ptr(), g, b,
                                         mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), ws.data_ptr(),
                                         relu ? 1 : 0, stream_of(x)), "groupnorm_relu_backward");
    return {dx, dgamma, dbeta};
}

// split forms of GroupNorm + ReLU (sums on this device, statistics from the caller)
torch::Tensor groupnorm_row_sums(torch::Tensor x) {
    CHECK_INPUT(x);
    TORCH_CHECK(x.dim() == 3, "expected (batch, channels, n)");
    c10::cuda::CUDAGuard guard(x.device());
    auto sums = torch::empty({x.size(0) * x.size(1), 2}, x.options().dtype(torch::kFloat64));
    auto ws = torch::empty({aprnet_groupnorm_workspace_bytes((int) x.size(0), (int) x.size(1), 1)}, x.options().dtype(torch::kUInt8));
    check(aprnet_groupnorm_row_sums(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), x.data_ptr(), ws.data_ptr(), sums.data_ptr<double>(), stream_of(x)), "groupnorm_row_sums");
    return sums;
}

torch::Tensor groupnorm_relu_apply(torch::Tensor x, c10::optional<torch::Tensor> gamma, c10::optional<torch::Tensor> beta, torch::Tensor mean, torch::Tensor rstd,
                                   int64_t groups, bool relu) {
    CHECK_INPUT(x); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    TORCH_CHECK(x.dim() == 3 && x.size(1) % groups == 0 && mean.numel() == x.size(0) * groups && rstd.numel() == mean.numel() &&
                mean.scalar_type() == x.scalar_type() && rstd.scalar_type() == x.scalar_type(), "statistics do not match the input");
    c10::cuda::CUDAGuard guard(x.device());
    auto y = torch::empty_like(x);
    const void* g = gamma.has_value() && gamma->defined() ? gamma->contiguous().data_ptr() : nullptr;
    const void* b = beta.has_value() && beta->defined() ? beta->contiguous().data_ptr() : nullptr;
    check(aprnet_groupnorm_relu_apply(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), (int) groups, x.data_ptr(), g, b, mean.data_ptr(), rstd.data_ptr(),
                                      y.data_ptr(), relu ? 1 : 0, stream_of(x)), "groupnorm_relu_apply");
    return y;
}

torch::Tensor groupnorm_backward_row_sums(torch::Tensor x, torch::Tensor grad_y, c10::optional<torch::Tensor> gamma, c10::optional<torch::Tensor> beta,
                                          torch::Tensor mean, torch::Tensor rstd, int64_t groups, bool relu) {
    CHECK_INPUT(x); CHECK_INPUT(grad_y); CHECK_INPUT(mean); CHECK_INPUT(rstd);
    TORCH_CHECK(x.sizes() == grad_y.sizes() && x.dim() == 3 && x.size(1) % groups == 0, "grad_y must have the shape of x");
    c10::cuda::CUDAGuard guard(x.device());
    auto sums = torch::empty({x.size(0) * x.size(1), 2}, x.options().dtype(torch::kFloat64));
    auto ws = torch::empty({aprnet_groupnorm_workspace_bytes((int) x.size(0), (int) x.size(1), (int) groups)}, x.options().dtype(torch::kUInt8));
    const void* g = gamma.has_value() && gamma->defined() ? gamma->contiguous().data_ptr() : nullptr;
    const void* b = beta.has_value() && beta->defined() ? beta->contiguous().data_ptr() : nullptr;
    check(aprnet_groupnorm_backward_row_sums(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), (int) groups, x.data_ptr(), grad_y.data_ptr(), g, b,
                                             mean.data_ptr(), rstd.data_ptr(), ws.data_ptr(), sums.data_ptr<double>(), relu ? 1 : 0, stream_of(x)), "groupnorm_backward_row_sums");
    return sums;
}

torch::Tensor groupnorm_backward_apply(torch::Tensor x, torch::Tensor grad_y, c10::optional<torch::Tensor> gamma, c10::optional<torch::Tensor> beta,
                                       torch::Tensor mean, torch::Tensor rstd, torch::Tensor group_terms, int64_t groups, bool relu) {
    CHECK_INPUT(x); CHECK_INPUT(grad_y); CHECK_INPUT(mean); CHECK_INPUT(rstd); CHECK_INPUT(group_terms);
    TORCH_CHECK(x.sizes() == grad_y.sizes() && x.dim() == 3 && x.size(1) % groups == 0 && group_terms.numel() == 2 * x.size(0) * groups &&
                group_terms.scalar_type() == x.scalar_type(), "arguments do not match the input");
    c10::cuda::CUDAGuard guard(x.device());
    auto dx = torch::empty_like(x);
    const void* g = gamma.has_value() && gamma->defined() ? gamma->contiguous().data_ptr() : nullptr;
    const void* b = beta.has_value() && beta->defined() ? beta->contiguous().data_ptr() : nullptr;
    check(aprnet_groupnorm_backward_apply(dtype_id(x), (int) x.size(0), (int) x.size(1), x.size(2), (int) groups, x.data_ptr(), grad_y.data_ptr(), g, b,
                                          mean.data_ptr(), rstd.data_ptr(), group_terms.data_ptr(), dx.data_ptr(), relu ? 1 : 0, stream_of(x)), "groupnorm_backward_apply");
    return dx;
}

// ---- tree fill on (C, N) tensors -------------------------------------------------------------------
torch::Tensor fill_tree(APR& apr, torch::Tensor input, bool use_max) {
    CHECK_INPUT(input);
    TORCH_CHECK(input.dim() == 2 && input.size(1) >= (int64_t) apr.total_number_particles(), "expected a (channels, particles) tensor");
    c10::cuda::CUDAGuard guard(input.device());
    const int64_t t = std::max<int64_t>(1, (int64_t) apr.total_number_tree_particles());
    auto tree = torch::empty({input.size(0), t}, input.options());
    if (use_max)
        check(aprnet_fill_tree_max(apr.handle(input), dtype_id(input), (int) input.size(0), input.data_ptr(), input.size(1), tree.data_ptr(), t, stream_of(input)), "fill_tree_max");
    else
        check(aprnet_fill_tree_mean_full(apr.handle(input), dtype_id(input), (int) input.size(0), input.data_ptr(), input.size(1), tree.data_ptr(), t, stream_of(input)), "fill_tree_mean");
    return tree.narrow(1, 0, (int64_t) apr.total_number_tree_particles());
}

torch::Tensor fill_tree_mean_dl(APR& apr, torch::Tensor input, int level_delta) {
    CHECK_INPUT(input);
    check_level_delta(apr, level_delta);
    c10::cuda::CUDAGuard guard(input.device());
    const int64_t ts = aprnet_tree_size(apr.handle(input), level_delta);
    auto tree = torch::empty({input.size(0), std::max<int64_t>(ts, 1)}, input.options());
    check(aprnet_fill_tree_mean_forward(apr.handle(input), level_delta, dtype_id(input), (int) input.size(0), input.data_ptr(), input.size(1),
                                        tree.data_ptr(), std::max<int64_t>(ts, 1), stream_of(input)), "fill_tree_mean");
    return tree.narrow(1, 0, ts);
}

torch::Tensor fill_tree_mean_dl_backward(APR& apr, torch::Tensor grad_input, torch::Tensor grad_tree, int level_delta) {
    CHECK_INPUT(grad_input); CHECK_INPUT(grad_tree);
    check_level_delta(apr, level_delta);
    c10::cuda::CUDAGuard guard(grad_input.device());
    auto gi = grad_input.clone();
    auto gt = grad_tree.clone();
    check(aprnet_fill_tree_mean_backward(apr.handle(gi), level_delta, dtype_id(gi), (int) gi.size(0), gi.data_ptr(), gi.size(1), gt.data_ptr(),
                                         gt.size(1), stream_of(gi)), "fill_tree_mean_backward");
    return gi;
}

py::array_t<int32_t> plan_nbr_table(APR& apr, int level_delta) {
    TORCH_CHECK(apr.dev != nullptr, "APR.init_cuda() must be called first");
    py::array_t<int32_t> out({(py::ssize_t) 27, (py::ssize_t) apr.number_parts(level_delta)});
    check(aprnet_plan_copy_nbr_table(apr.dev, level_delta, out.mutable_data()), "plan_nbr_table");
    return out;
}

py::array_t<int32_t> child_table(APR& apr) {
    TORCH_CHECK(apr.dev != nullptr, "APR.init_cuda() must be called first");
    py::array_t<int32_t> out({(py::ssize_t) 8, (py::ssize_t) apr.total_number_tree_particles()});
    check(aprnet_copy_child_table(apr.dev, out.mutable_data()), "child_table");
    return out;
}

template<typename T>
py::array_t<T> to_array(const std::vector<T>& v) { return py::array_t<T>((py::ssize_t) v.size(), v.data()); }

} // namespace

PYBIND11_MODULE(_pyaprwrapper, m) {
    using namespace pybind11::literals;
    m.doc() = "B200-native particle-domain CNN operators behind the pyapr extension-module interface";
    m.attr("__version__") = py::str("aprnet-b200-0.1");
    m.attr("__cuda_build__") = true;

    py::module data_containers = m.def_submodule("data_containers");
    py::class_<APR>(data_containers, "APR")
        .def(py::init())
        .def("__repr__", [](APR& a) {
            return "APR(shape [" + std::to_string(a.org_dims(2)) + ", " + std::to_string(a.org_dims(1)) + ", " +
                   std::to_string(a.org_dims(0)) + "], " + std::to_string(a.total_number_particles()) + " particles)"; })
        .def_readwrite("name", &APR::name)
        .def("init_from_arrays", &APR::init, "shape_z"_a, "shape_x"_a, "shape_y"_a, "row_ptr"_a, "y"_a, "tree_row_ptr"_a, "tree_y"_a,
             "Set the linear access arrays (CSR row pointers and y coordinates of particles and tree nodes)")
        .def("total_number_particles", &APR::total_number_particles, "return number of particles")
        .def("total_number_tree_particles", &APR::total_number_tree_particles, "return number of interior tree particles")
        .def("level_min", &APR::level_min, "return the minimum resolution level")
        .def("level_max", &APR::level_max, "return the maximum resolution level")
        .def("x_num", &APR::x_num, "level"_a)
        .def("y_num", &APR::y_num, "level"_a)
        .def("z_num", &APR::z_num, "level"_a)
        .def("org_dims", &APR::org_dims, "returns the original image size in a specified dimension (y, x, z)", "dim"_a)
        .def("shape", [](APR& self) { return py::make_tuple(self.org_dims(2), self.org_dims(1), self.org_dims(0)); })
        .def("init_cuda", &APR::init_cuda, "copy access structures to GPU device", "with_tree"_a = true)
        .def("cuda_device_bytes", [](APR& a) { return a.dev ? aprnet_device_bytes(a.dev) : (int64_t) 0; })
        .def("plan", [](APR& a, int dl) { TORCH_CHECK(a.dev, "APR.init_cuda() must be called first");
                                          c10::cuda::CUDAGuard guard((c10::DeviceIndex) a.dev_index);      // the tables live on the APR's device
                                          check(aprnet_plan_build(a.dev, dl, nullptr), "plan");
                                          if (g_conv_mode == 1) check(aprnet_edge_plan_build(a.dev, dl, nullptr), "edge plan"); }, "level_delta"_a,
             "Build (and cache) the neighbour table of a level delta ahead of the first convolution")
        .def("computational_ratio", &APR::computational_ratio)
        .def(py::pickle(
            [](APR& a) {
                if (!a.initialized) throw std::runtime_error("Invalid state - APR not initialized");
                return py::make_tuple(a.org_dims(0), a.org_dims(1), a.org_dims(2), a.name, to_array(a.row_ptr), to_array(a.y_vec),
                                      to_array(a.tree_row_ptr), to_array(a.tree_y_vec));
            },
            [](py::tuple t) {
                if (t.size() != 8) throw std::runtime_error("Error unpickling APR object - invalid state size");
                auto a = std::make_unique<APR>();
                a->init(t[2].cast<int>(), t[1].cast<int>(), t[0].cast<int>(), t[4].cast<py::array_t<int64_t>>(),
                        t[5].cast<py::array_t<uint16_t>>(), t[6].cast<py::array_t<int64_t>>(), t[7].cast<py::array_t<uint16_t>>());
                a->name = t[3].cast<std::string>();
                return a;
            }));
    py::bind_vector<std::vector<APR*>>(data_containers, "APRPtrVector", py::module_local(false));

    py::module aprnet = m.def_submodule("aprnet");
    py::module utils = aprnet.def_submodule("utils");
    utils.def("number_particles", [](APR& a, int dl) { return a.number_parts(dl); }, "apr"_a, "level_delta"_a);
    utils.def("number_particles_after_pooling", [](APR& a, int dl) { return a.number_parts(dl + 1); }, "apr"_a, "level_delta"_a);
    utils.def("number_particles_after_upsampling", [](APR& a, int dl) { return a.number_parts(dl - 1); }, "apr"_a, "level_delta"_a);
    utils.def("number_parts", [](APR& a, int dl) { return a.number_parts(dl); }, "apr"_a, "level_delta"_a);

    py::module cuda = aprnet.def_submodule("cuda");
    cuda.def("maxpool_forward_cuda", &maxpool_forward_cuda, "aprs"_a, "input"_a, "level_delta"_a);
    cuda.def("maxpool_backward_cuda", &maxpool_backward_cuda, "aprs"_a, "grad_output"_a, "max_indices"_a, "level_delta"_a);
    cuda.def("conv111_forward", &conv111_forward, "aprs"_a, "input"_a, "weights"_a, "level_delta"_a, "precision"_a = "");
    cuda.def("conv111_backward", &conv111_backward, "aprs"_a, "input"_a, "weights"_a, "grad_output"_a, "level_delta"_a, "precision"_a = "");
    cuda.def("conv333_forward", &conv333_forward, "aprs"_a, "input"_a, "weights"_a, "level_delta"_a);
    cuda.def("conv333_backward", &conv333_backward, "aprs"_a, "input"_a, "weights"_a, "grad_output"_a, "level_delta"_a);
    // extensions: keep the tree means of the forward pass for the backward pass
    cuda.def("conv333_forward_keep_tree", &conv333_forward_keep_tree, "aprs"_a, "input"_a, "weights"_a, "level_delta"_a, "precision"_a = "");
    cuda.def("conv333_backward_with_tree", &conv333_backward_with_tree, "aprs"_a, "input"_a, "weights"_a, "grad_output"_a, "level_delta"_a, "tree"_a, "need_grad_input"_a = true,
             "precision"_a = "");
    cuda.def("conv333_forward_keep_rows", &conv333_forward_keep_rows, "aprs"_a, "input"_a, "weights"_a, "level_delta"_a);
    cuda.def("conv333_backward_with_rows", &conv333_backward_with_rows, "aprs"_a, "rows"_a, "weights"_a, "grad_output"_a, "level_delta"_a, "need_grad_input"_a = true);
    cuda.def("upsample_const_forward", &upsample_const_forward, "aprs"_a, "input"_a, "level_delta"_a);
    cuda.def("upsample_const_backward", &upsample_const_backward, "aprs"_a, "grad_output"_a, "level_delta"_a);
    cuda.def("reconstruct_forward", &reconstruct_forward, "aprs"_a, "input"_a, "level_delta"_a);
    cuda.def("reconstruct_backward", &reconstruct_backward, "aprs"_a, "grad_output"_a, "level_delta"_a);
    cuda.def("sample_particles_forward", &sample_particles_forward, "aprs"_a, "input"_a, "level_delta"_a);
    cuda.def("sample_particles_backward", &sample_particles_backward, "aprs"_a, "grad_output"_a, "level_delta"_a);
    cuda.def("restrict_kernel333_forward", &restrict_kernel_333_forward, "weights"_a, "num_levels"_a);
    cuda.def("restrict_kernel333_backward", &restrict_kernel_333_backward, "grad_weights_expanded"_a, "num_levels"_a);
    cuda.def("groupnorm_relu_forward", &groupnorm_relu_forward, "x"_a, "gamma"_a, "beta"_a, "groups"_a, "eps"_a, "relu"_a);
    cuda.def("groupnorm_relu_backward", &groupnorm_relu_backward, "x"_a, "grad_y"_a, "gamma"_a, "beta"_a, "mean"_a, "rstd"_a, "groups"_a, "relu"_a);
    // split forms for one z-slab of an APR per GPU (halo exchange between the steps, pyapr/aprnet/cuda/sharded.py)
    cuda.def("conv333_forward_pretree", &conv333_forward_pretree, "aprs"_a, "input"_a, "tree"_a, "weights"_a, "level_delta"_a, "precision"_a = "");
    cuda.def("conv333_backward_pretree", &conv333_backward_pretree, "aprs"_a, "input"_a, "tree"_a, "kept"_a, "weights"_a, "grad_output"_a, "level_delta"_a, "need_grad_input"_a = true);
    cuda.def("fill_tree_mean_batch", &fill_tree_mean_batch, "aprs"_a, "input"_a, "level_delta"_a);
    cuda.def("fill_tree_mean_backward_inplace", &fill_tree_mean_backward_inplace, "aprs"_a, "grad_input"_a, "grad_tree"_a, "level_delta"_a);
    cuda.def("groupnorm_row_sums", &groupnorm_row_sums, "x"_a);
    cuda.def("groupnorm_relu_apply", &groupnorm_relu_apply, "x"_a, "gamma"_a, "beta"_a, "mean"_a, "rstd"_a, "groups"_a, "relu"_a);
    cuda.def("groupnorm_backward_row_sums", &groupnorm_backward_row_sums, "x"_a, "grad_y"_a, "gamma"_a, "beta"_a, "mean"_a, "rstd"_a, "groups"_a, "relu"_a);
    cuda.def("groupnorm_backward_apply", &groupnorm_backward_apply, "x"_a, "grad_y"_a, "gamma"_a, "beta"_a, "mean"_a, "rstd"_a, "group_terms"_a, "groups"_a, "relu"_a);
    // test / inspection hooks (not part of the reference interface)
    cuda.def("fill_tree_mean", &fill_tree_mean_dl, "apr"_a, "input"_a, "level_delta"_a);
    cuda.def("fill_tree_mean_backward", &fill_tree_mean_dl_backward, "apr"_a, "grad_input"_a, "grad_tree"_a, "level_delta"_a);
    cuda.def("plan_nbr_table", &plan_nbr_table, "apr"_a, "level_delta"_a);
    cuda.def("child_table", &child_table, "apr"_a);
    cuda.def("set_conv_precision", [](const std::string& mode) {
        if (mode == "fp32") g_conv_mode = 0;
        else if (mode == "bf16") g_conv_mode = 1;
        else throw std::invalid_argument("conv precision must be 'fp32' or 'bf16'");
    }, "mode"_a, "'fp32': exact CUDA-core kernels (default); 'bf16': tensor-core path for float32 3x3x3 convolutions (bf16 operands, fp32 accumulation)");
    cuda.def("get_conv_precision", []() { return std::string(g_conv_mode == 1 ? "bf16" : "fp32"); });
    cuda.def("tc_error_flag", []() { return aprnet_tc_error_flag(); });
    cuda.def("tc_error_reset", []() { aprnet_tc_error_reset(); }, "Clear the flag that a tensor-core kernel raises when one of its bounded waits runs out");
    cuda.def("tc_selftest_wait_timeout", [](int max_polls) {
        check(aprnet_tc_selftest_wait_timeout(max_polls, (void*) at::cuda::getCurrentCUDAStream().stream()), "tc_selftest_wait_timeout");
    }, "max_polls"_a = 1000, "Test hook: a kernel whose bounded wait runs out and raises the tensor-core error flag");
    cuda.def("tc_set_option", [](const std::string& name, int value) { check(aprnet_tc_set_option(name.c_str(), value), "tc_set_option"); },
             "name"_a, "value"_a, "Measurement switches of the tensor-core gather kernel ('taps', 'wps', 'ks'; 0 = automatic)");
    cuda.def("measure_fp32_fma_tflops", [](int repeats) {
        double v = 0.0;
        check(aprnet_measure_fp32_fma_tflops(repeats, &v, (void*) at::cuda::getCurrentCUDAStream().stream()), "measure_fp32_fma_tflops");
        return v;
    }, "repeats"_a = 5, "Measured fp32 FMA throughput of the current device in TFLOP/s (register-only FMA chains)");
    cuda.def("profile_enable", [](bool on) { aprnet_profile_enable(on ? 1 : 0); }, "on"_a,
             "Bracket every kernel launch of the library with CUDA events (benchmark use)");
    cuda.def("profile_read", []() {
        std::string buf((size_t) 1 << 16, '\0');
        aprnet_profile_read(&buf[0], (int64_t) buf.size());
        py::dict out;
        std::istringstream is(buf.c_str());
        std::string name; long long calls; double ms;
        while (is >> name >> calls >> ms) out[py::str(name)] = py::make_tuple(calls, ms);
        return out;
    }, "Return {kernel name: (launches, total milliseconds)} since the last read and clear the records");

    py::module tree = m.def_submodule("tree");
    tree.def("fill_tree_mean", [](APR& a, torch::Tensor x) { return fill_tree(a, x, false); }, "apr"_a, "parts"_a);
    tree.def("fill_tree_max", [](APR& a, torch::Tensor x) { return fill_tree(a, x, true); }, "apr"_a, "parts"_a);
}
