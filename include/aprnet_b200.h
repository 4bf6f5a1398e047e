/*
 * aprnet_b200 — C ABI of the B200 (sm_100a) particle-domain CNN operators.
 *
 * Drop-in boundary for the operator set that AdaptiveParticles/APR-CNN exposes to Python as
 * `_pyaprwrapper.aprnet.cuda` (wrappers/pythonBind.cpp:162-181).  Every entry point takes plain
 * pointers and sizes, returns 0 on success or a negative status (never aborts), launches on the
 * stream it is given and performs no device-wide synchronisation and no allocation on the hot path:
 * outputs and scratch buffers are owned by the caller.
 *
 * Conventions
 *   - feature tensors are channel-major: element (c, p) of a tensor lives at base[c * ld + p], with
 *     `ld` >= number of valid entries (the reference pads a batch to its largest APR,
 *     pyapr/aprnet/cuda/src/wrap_conv_gpu.hpp:51);
 *   - `level_delta` = number of poolings applied; the valid entries of a feature tensor are the APR
 *     particles of levels <= level_max - level_delta followed by the tree nodes of that level
 *     (pyapr/aprnet/src/helpers.hpp:86-101);
 *   - `dtype` selects the arithmetic: APRNET_F32 or APRNET_F64 (the reference dispatches both,
 *     wrap_conv_gpu.hpp:54);
 *   - `stream` is a cudaStream_t passed as void*.
 *   - all data pointers are DEVICE pointers unless the parameter name starts with `host_`.
 */
#ifndef APRNET_B200_H
#define APRNET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define APRNET_F32 0
#define APRNET_F64 1

#define APRNET_OK 0
#define APRNET_ERR_ARG (-1)      /* bad argument (null pointer, level_delta out of range, size mismatch) */
#define APRNET_ERR_CUDA (-2)     /* a CUDA runtime call failed; aprnet_last_error() has the text */
#define APRNET_ERR_UNSUPPORTED (-3)

typedef struct aprnet_apr aprnet_apr;

/* Text of the last error raised on the calling thread. */
const char* aprnet_last_error(void);

/* Optional per-kernel timing.  While enabled, every kernel launch made by this library is bracketed
 * by two CUDA events on its stream.  aprnet_profile_read() waits for the recorded events, writes one
 * line "name launches total_ms" per kernel into buf (NUL-terminated, truncated to buflen), clears the
 * records and returns the untruncated length.  Not thread-safe; meant for benchmarks. */
void aprnet_profile_enable(int on);
int64_t aprnet_profile_read(char* buf, int64_t buflen);
/* Measured fp32 multiply-add throughput of the current device in TFLOP/s (best of `repeats` short runs of
 * register-only FMA chains, timed with CUDA events): the denominator of the roofline of the fp32 CUDA-core
 * convolution path.  No counterpart in the reference. */
int aprnet_measure_fp32_fma_tflops(int repeats, double* tflops_out, void* stream);

/* ---- access structure ------------------------------------------------------------------------
 * Replaces LibAPR's APR::init_cuda / gpuAPRHelper / gpuTreeHelper as used at
 * pyapr/aprnet/cuda/src/wrap_conv_gpu.hpp:23-28 (device copies of level_xz_vec / xz_end_vec / y_vec
 * for particles and tree).  Rows are numbered level-major, then z, then x; particles of row r are
 * [row_ptr[r], row_ptr[r+1]) and `y` holds their ascending y coordinates.  `dims_zxy` holds
 * (z_num, x_num, y_num) for levels 0..level_max.  Particle rows cover levels
 * level_min..level_max, tree rows cover level_min-1..level_max-1.  All arguments are HOST arrays;
 * they are copied to `device`.  Also builds the child table of the tree (cached). */
int aprnet_apr_create(aprnet_apr** out, int level_min, int level_max, const int* host_dims_zxy,
                      const int64_t* host_row_ptr, const uint16_t* host_y,
                      const int64_t* host_tree_row_ptr, const uint16_t* host_tree_y, int device);
void aprnet_apr_destroy(aprnet_apr* apr);

/* pyapr/aprnet/src/helpers.hpp:86-110 (number_parts, number_parts_after_pooling/upsampling) */
int64_t aprnet_number_parts(const aprnet_apr* apr, int level_delta);
/* number of tree nodes of levels <= level_max - level_delta - 1: rows of the tree scratch that
 * conv333 needs (pyapr/aprnet/cuda/src/wrap_conv_gpu.hpp:42-52) */
int64_t aprnet_tree_size(const aprnet_apr* apr, int level_delta);
int64_t aprnet_total_tree_nodes(const aprnet_apr* apr);
/* bytes of device memory held by the handle (access arrays, child table, cached plans) */
int64_t aprnet_device_bytes(const aprnet_apr* apr);

/* Builds (once; cached in the handle) the neighbour table of `level_delta`: for each output
 * location and each of the 27 stencil taps, which value fills that cell.  Replaces the per-call
 * non-empty-row enumeration and dense-patch staging of the reference
 * (pyapr/aprnet/cuda/src/nonempty_rows.cu:26-230, conv333_gpu.cu:63-118).  Called implicitly by the
 * conv333 entry points; call it up front to keep allocation out of timed regions. */
int aprnet_plan_build(aprnet_apr* apr, int level_delta, void* stream);
/* Test hooks: copy the cached tables to host memory.  nbr: int32[27][N]; child: int32[8][T]. */
int aprnet_plan_copy_nbr_table(aprnet_apr* apr, int level_delta, int32_t* host_out);
int aprnet_copy_child_table(aprnet_apr* apr, int32_t* host_out);

/* ---- tree fill -------------------------------------------------------------------------------
 * pyapr/aprnet/cuda/src/fill_tree_gpu.hpp:15-32 (apply_fill_tree_mean / _backward); arithmetic of
 * pyapr/aprnet/src/helpers.hpp:156-350.  tree is (C, ld_tree) with aprnet_tree_size() valid entries. */
int aprnet_fill_tree_mean_forward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                                  const void* input, int64_t ld_in, void* tree, int64_t ld_tree, void* stream);
/* grad_input += adjoint(grad_tree); grad_tree is used as workspace (root-to-leaf accumulation). */
int aprnet_fill_tree_mean_backward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                                   void* grad_input, int64_t ld_in, void* grad_tree, int64_t ld_tree, void* stream);
/* pyapr/tree/fill_tree.py:46-71 (fill_tree_max): every tree node = max over its descendants,
 * level_delta 0, tree is (C, ld_tree) with aprnet_total_tree_nodes() valid entries. */
int aprnet_fill_tree_max(const aprnet_apr* apr, int dtype, int channels, const void* input, int64_t ld_in,
                         void* tree, int64_t ld_tree, void* stream);
/* pyapr/tree/fill_tree.py:20-43 (fill_tree_mean): all tree nodes from the particles, level_delta 0 */
int aprnet_fill_tree_mean_full(const aprnet_apr* apr, int dtype, int channels, const void* input, int64_t ld_in,
                               void* tree, int64_t ld_tree, void* stream);

/* ---- stencil restriction ---------------------------------------------------------------------
 * pyapr/aprnet/cuda/src/restrict_gpu.hpp:25-32 (apply_restrict_kernel_333 / _backward).
 * weights (S, Cout, Cin, 3,3,3) -> expanded (L, Cout, Cin, 3,3,3); backward is the transpose. */
int aprnet_restrict333_forward(int dtype, int num_stencils, int num_levels, int64_t filters,
                               const void* weights, void* expanded, void* stream);
int aprnet_restrict333_backward(int dtype, int num_stencils, int num_levels, int64_t filters,
                                const void* grad_expanded, void* grad_weights, void* stream);

/* ---- 3x3x3 convolution -----------------------------------------------------------------------
 * pyapr/aprnet/cuda/src/conv_gpu.hpp:74-96 (apply_conv333, apply_conv333_backward).
 * weights: (num_slots, Cout, Cin, 27), level l uses slot min(cml - l, num_slots - 1).
 * tree_scratch: (Cin, ld_tree) workspace, overwritten with fill_tree_mean(input). */
int aprnet_conv333_forward(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                           const void* input, int64_t ld_in, const void* weights,
                           void* output, int64_t ld_out, void* tree_scratch, int64_t ld_tree, void* stream);
/* grad_input (Cin, ld_in) must be zero-filled by the caller; grad_tree_scratch (Cin, ld_tree) is
 * zero-filled by the call.  grad_output is (Cout, ld_out). */
int aprnet_conv333_backward_input(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                                  const void* grad_output, int64_t ld_out, const void* weights,
                                  void* grad_input, int64_t ld_in, void* grad_tree_scratch, int64_t ld_tree,
                                  void* stream);
/* grad_weights (num_slots, Cout, Cin, 27) is ACCUMULATED into (so a batch loop sums, as the reference
 * does).  tree_scratch must hold fill_tree_mean(input) (as left by the forward call, or recomputed with
 * aprnet_fill_tree_mean_forward).  partial: workspace of aprnet_conv333_partial_elems() elements;
 * block-local sums are written there and reduced in a fixed order (deterministic). */
int64_t aprnet_conv333_partial_elems(int cin, int cout);
int aprnet_conv333_backward_weights(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                                    const void* input, int64_t ld_in, const void* tree_scratch, int64_t ld_tree,
                                    const void* grad_output, int64_t ld_out, void* grad_weights,
                                    void* partial, void* stream);

/* Split forms for a caller that exchanges values between the tree fill and the gather -- one z-slab of an
 * APR per GPU with halo rows from the neighbouring slabs (the reference has no multi-GPU path; the stencil
 * reach that fixes the halo is pyapr/aprnet/cuda/src/conv333_gpu.cu:65-72,239-246).  Forward: `tree` holds
 * the tree means (aprnet_fill_tree_mean_forward, then the halo entries from their owners) and is only
 * read.  Backward: grad_input receives the direct contributions only and grad_tree the gradient of the
 * tree means; the caller adds the halo parts at their owners and then folds grad_tree into grad_input with
 * aprnet_fill_tree_mean_backward.  Same argument conventions as the calls above. */
int aprnet_conv333_forward_pretree(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                                   const void* input, int64_t ld_in, const void* weights,
                                   void* output, int64_t ld_out, const void* tree, int64_t ld_tree, void* stream);
int aprnet_conv333_backward_input_pretree(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                                          const void* grad_output, int64_t ld_out, const void* weights,
                                          void* grad_input, int64_t ld_in, void* grad_tree, int64_t ld_tree,
                                          void* stream);

/* ---- 3x3x3 convolution on the tensor cores (bf16 operands, fp32 accumulation) ------------------
 * No counterpart in the reference (its kernels are CUDA-core only).  Same contract as
 * aprnet_conv333_forward for float32 tensors; results differ by the bf16 rounding of inputs and
 * weights (relative error <= 2e-2).  `workspace` needs aprnet_conv333_tc_workspace_bytes() bytes,
 * 256-byte aligned.  Waits inside the kernels are bounded; aprnet_tc_error_flag() becomes non-zero
 * if one ever expired, and later calls then fail with APRNET_ERR_CUDA. */
int64_t aprnet_conv333_tc_workspace_bytes(const aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots);          /* backward (and forward) */
int64_t aprnet_conv333_tc_forward_workspace_bytes(const aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots);  /* forward only */
int aprnet_conv333_forward_tc(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                              const float* input, int64_t ld_in, const float* weights, float* output, int64_t ld_out,
                              float* tree_scratch, int64_t ld_tree, void* workspace, void* stream);
/* Complete backward pass with the contractions on the tensor cores.  grad_weights
 * (num_slots, Cout, Cin, 27) is accumulated into (deterministic block partials + fixed-order second
 * pass); grad_input (Cin, ld_in) is written (pass NULL to skip the input gradient).  Steps: tree means of the input -> bf16 channels-last
 * copies of input and grad_output -> weight gradient -> same-level part of the input gradient (a
 * gather) -> cross-level part (edge-list GEMM + deterministic per-target sums) and tree adjoint.
 * tree / grad_tree: (Cin, ld_tree) float scratch (pass tree_scratch_is_valid = 1 when tree_scratch still
 * holds the tree means that the forward call left there: the fill is then skipped); partial: aprnet_conv333_tc_dw_partial_elems()
 * floats; workspace: aprnet_conv333_tc_workspace_bytes() bytes. */
int64_t aprnet_conv333_tc_dw_partial_elems(int cin, int cout);
int aprnet_conv333_backward_tc(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                               const float* input, int64_t ld_in, const float* grad_output, int64_t ld_out,
                               const float* weights, float* grad_input, float* grad_weights,
                               float* tree_scratch, int tree_scratch_is_valid, float* grad_tree_scratch, int64_t ld_tree,
                               float* partial, void* workspace, void* stream);
/* The same backward pass from the packed bf16 rows of the input that aprnet_conv333_forward_tc left in
 * the first aprnet_conv333_tc_packed_rows_bytes() bytes of its workspace (keep that buffer instead of the
 * fp32 input and the tree means: half the bytes, and no second packing pass).  grad_input may be NULL. */
int64_t aprnet_conv333_tc_packed_rows_bytes(const aprnet_apr* apr, int level_delta, int cin);
int aprnet_conv333_backward_tc_rows(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                                    const void* packed_input_rows, const float* grad_output, int64_t ld_out,
                                    const float* weights, float* grad_input, int64_t ld_in, float* grad_weights,
                                    float* grad_tree_scratch, int64_t ld_tree, float* partial, void* workspace, void* stream);
/* Split forms on the tensor cores (see aprnet_conv333_forward_pretree). */
int aprnet_conv333_forward_tc_pretree(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                                      const float* input, int64_t ld_in, const float* weights, float* output, int64_t ld_out,
                                      const float* tree, int64_t ld_tree, void* workspace, void* stream);
int aprnet_conv333_backward_tc_rows_pretree(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                                            const void* packed_input_rows, const float* grad_output, int64_t ld_out,
                                            const float* weights, float* grad_input, int64_t ld_in, float* grad_weights,
                                            float* grad_tree, int64_t ld_tree, float* partial, void* workspace, void* stream);
/* Building blocks of the above, exported for callers that keep the packed copies around. */
int aprnet_conv333_backward_weights_tc(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                                       const void* packed_input_rows, int input_row_width,
                                       const void* packed_grad_output_rows, int grad_output_row_width,
                                       float* grad_weights, float* partial, void* stream);
int aprnet_conv333_backward_input_cross_level(aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_slots,
                                              const void* grad_output, int64_t ld_out, const void* weights,
                                              void* grad_input, int64_t ld_in, void* grad_tree_scratch, int64_t ld_tree,
                                              void* stream);
/* Cross-level part of the input gradient without atomics: an edge-list GEMM on the tensor cores plus a
 * per-target pull (deterministic).  The edge lists of a level delta are built once and cached
 * (aprnet_edge_plan_build allocates; call it up front).  edge_ws: aprnet_edge_workspace_bytes() bytes.
 * Limit: 27 * N(level_delta) < 2^31, i.e. up to 79.5 M locations (32-bit edge ids); beyond it
 * aprnet_conv333_backward_tc(_rows) falls back to aprnet_conv333_backward_input_cross_level (atomic adds). */
int aprnet_edge_plan_build(aprnet_apr* apr, int level_delta, void* stream);
int64_t aprnet_edge_workspace_bytes(const aprnet_apr* apr, int level_delta, int cout);
int aprnet_conv333_backward_input_cross_level_tc(aprnet_apr* apr, int level_delta, int cin, int cout, int num_slots,
                                                 const void* packed_grad_output_rows, int grad_output_row_width,
                                                 const float* weights, float* grad_input, int64_t ld_in,
                                                 float* grad_tree_scratch, int64_t ld_tree, void* packed_weight_ws,
                                                 void* edge_ws, int64_t edge_ws_bytes, void* stream);
int aprnet_tc_error_flag(void);
/* Clears the flag above so that the tensor-core entry points accept calls again after a wait ran out. */
void aprnet_tc_error_reset(void);
/* Test hook for the error path: launches one small kernel whose bounded wait (max_polls polls) is on a barrier
 * that nothing arrives at; the wait runs out, the kernel raises the flag above and returns (nothing hangs). */
int aprnet_tc_selftest_wait_timeout(int max_polls, void* stream);
/* Measurement switches of the tensor-core gather kernel (0 = automatic): "taps" = taps of the 27 per shared-memory
 * stage, "wps" = producer warps that fill one stage together (both must be set, and the pair must be a compiled
 * shape whose ring fits shared memory, else the automatic choice stays), "tma_taps" = how many of a stage's taps the TMA
 * unit fetches (tile::gather4) instead of cp.async (with "taps" and "wps"), "ks" = channels per stage (16, 32, 64),
 * "dw_waves" = waves of blocks of the weight-gradient kernel. */
int aprnet_tc_set_option(const char* name, int value);

/* ---- 1x1x1 convolution -----------------------------------------------------------------------
 * pyapr/aprnet/cuda/src/conv_gpu.hpp:98-120 (apply_conv111 / _backward).  weights (S, Cout, Cin);
 * level l uses stencil min(cml - l, S - 1), upgraded tree nodes use stencil 0. */
int aprnet_conv111_forward(const aprnet_apr* apr, int level_delta, int dtype, int cin, int cout, int num_stencils,
                           const void* input, int64_t ld_in, const void* weights, void* output, int64_t ld_out,
                           void* stream);
int aprnet_conv111_backward_input(const aprnet_apr* apr, int level_delta, int dtype, int cin, int cout,
                                  int num_stencils, const void* grad_output, int64_t ld_out, const void* weights,
                                  void* grad_input, int64_t ld_in, void* stream);
/* The same two products with bf16 operands and fp32 accumulation on the tensor cores (float32 tensors, the layer's
 * precision "bf16"): replaces the same launchers, conv111_gpu.cu:175-232.  APRNET_ERR_UNSUPPORTED when a channel count
 * exceeds 256 or is below 8, or the level's weights plus two operand stages do not fit shared memory: call the entry
 * above then. */
int aprnet_conv111_forward_tc(const aprnet_apr* apr, int level_delta, int cin, int cout, int num_stencils,
                              const float* input, int64_t ld_in, const float* weights, float* output, int64_t ld_out, void* stream);
int aprnet_conv111_backward_input_tc(const aprnet_apr* apr, int level_delta, int cin, int cout, int num_stencils,
                                     const float* grad_output, int64_t ld_out, const float* weights, float* grad_input, int64_t ld_in,
                                     void* stream);
/* Weight gradient of the 1x1x1 convolution with bf16 operands on the tensor cores (accumulated into grad_weights, float32
 * (num_stencils, Cout, Cin)); partial: aprnet_conv111_partial_elems() floats, partial_elems its size.
 * APRNET_ERR_UNSUPPORTED above 256 channels (call aprnet_conv111_backward_weights then). */
int aprnet_conv111_backward_weights_tc(const aprnet_apr* apr, int level_delta, int cin, int cout, int num_stencils,
                                       const float* input, int64_t ld_in, const float* grad_output, int64_t ld_out,
                                       float* grad_weights, float* partial, int64_t partial_elems, void* stream);
int64_t aprnet_conv111_partial_elems(int cin, int cout);
int aprnet_conv111_backward_weights(const aprnet_apr* apr, int level_delta, int dtype, int cin, int cout,
                                    int num_stencils, const void* input, int64_t ld_in, const void* grad_output,
                                    int64_t ld_out, void* grad_weights, void* partial, void* stream);

/* No counterpart in the reference.  Same result as aprnet_conv111_backward_weights (float32 only,
 * grad_weights (S, Cout, Cin) is accumulated into), for callers that cannot allocate device memory
 * where they call this library — e.g. a host whose own arena owns the whole GPU, or a loop that cannot
 * afford an allocation's device-wide synchronisation.  The block-partial sums live in a fixed 4 MiB
 * array inside the library image (held by every GPU that loads the library until the process exits)
 * instead of a caller workspace.  Limits and rules: cin * cout <= 262144, otherwise
 * APRNET_ERR_UNSUPPORTED; calls that overlap on one GPU race on the shared array, so serialise them;
 * the array keeps the previous call's contents (the call overwrites all it reads).  The first call on
 * each device looks up the array's device address (with that device current); make that first call
 * before starting any stream capture, and before a host arena claims the rest of the GPU: with lazy
 * module loading the CUDA runtime places the library image, the 4 MiB array included, on the device at
 * that first use, which can fail with an out-of-memory error on a GPU that is already full.  Every later
 * call allocates nothing. */
int aprnet_conv111_backward_weights_static(const aprnet_apr* apr, int level_delta, int cin, int cout,
                                           int num_stencils, const float* input, int64_t ld_in,
                                           const float* grad_output, int64_t ld_out, float* grad_weights,
                                           void* stream);
int64_t aprnet_static_scratch_bytes(void);

/* ---- GroupNorm (+ ReLU) over (batch, channels, n) tensors ------------------------------------------
 * No counterpart among the reference's own kernels: its network blocks call torch.nn.GroupNorm and
 * ReLU (apr_models/apr_models/unet/unet_parts.py:18-26).  Same arithmetic (biased variance, eps inside
 * the root, statistics over the whole particle axis of each (batch item, group)), fused into one
 * statistics pass + one apply pass forward and one reduction pass + one apply pass backward.
 * x, y, grad tensors are contiguous (batch, channels, n); mean / rstd are (batch * groups); gamma, beta
 * and their gradients are (channels) or NULL.  relu != 0 fuses max(., 0).
 * workspace: aprnet_groupnorm_workspace_bytes() bytes. */
int64_t aprnet_groupnorm_workspace_bytes(int batch, int channels, int groups);
int aprnet_groupnorm_relu_forward(int dtype, int batch, int channels, int64_t n, int groups, const void* x,
                                  const void* gamma, const void* beta, double eps, void* y, void* mean, void* rstd,
                                  void* workspace, int relu, void* stream);
int aprnet_groupnorm_relu_backward(int dtype, int batch, int channels, int64_t n, int groups, const void* x,
                                   const void* grad_y, const void* gamma, const void* beta, const void* mean,
                                   const void* rstd, void* grad_x, void* grad_gamma, void* grad_beta,
                                   void* workspace, int relu, void* stream);

/* Split forms of the two passes above for one z-slab of an APR per GPU: every rank reduces over the
 * particles it owns into row_sums (double, (batch * channels, 2): sum x and sum x^2 forward; sum dy_eff and
 * sum dy_eff * xhat backward), the caller all-reduces the sums, derives mean / rstd / the two group terms
 * (means of gamma * dy_eff and of gamma * dy_eff * xhat over the group) and applies them.  No counterpart in
 * the reference (it has no multi-GPU path). */
int aprnet_groupnorm_row_sums(int dtype, int batch, int channels, int64_t n, const void* x, void* workspace,
                              double* row_sums, void* stream);
int aprnet_groupnorm_relu_apply(int dtype, int batch, int channels, int64_t n, int groups, const void* x,
                                const void* gamma, const void* beta, const void* mean, const void* rstd, void* y,
                                int relu, void* stream);
int aprnet_groupnorm_backward_row_sums(int dtype, int batch, int channels, int64_t n, int groups, const void* x,
                                       const void* grad_y, const void* gamma, const void* beta, const void* mean,
                                       const void* rstd, void* workspace, double* row_sums, int relu, void* stream);
int aprnet_groupnorm_backward_apply(int dtype, int batch, int channels, int64_t n, int groups, const void* x,
                                    const void* grad_y, const void* gamma, const void* beta, const void* mean,
                                    const void* rstd, const void* group_terms, void* grad_x, int relu, void* stream);

/* ---- max pooling / constant up-sampling --------------------------------------------------------
 * pyapr/aprnet/cuda/src/maxpool_gpu.hpp:24-40, upsample_constant_gpu.hpp:17-31.
 * maxpool: level_delta -> level_delta + 1; max_indices are int64 positions in the input's particle
 * axis; first maximum in the reference CPU's visiting order wins (pyapr/aprnet/src/maxpool.hpp:105-142). */
int aprnet_maxpool_forward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                           const void* input, int64_t ld_in, void* output, int64_t* max_indices, int64_t ld_out,
                           void* stream);
/* grad_input must be zero-filled by the caller (only the kept particles and the arg-max positions are written). */
int aprnet_maxpool_backward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                            const void* grad_output, const int64_t* max_indices, int64_t ld_out,
                            void* grad_input, int64_t ld_in, void* stream);
/* upsample: level_delta -> level_delta - 1 (level_delta must be > 0,
 * pyapr/aprnet/cuda/src/wrap_upsample_const_gpu.hpp:36). */
int aprnet_upsample_forward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                            const void* input, int64_t ld_in, void* output, int64_t ld_out, void* stream);
int aprnet_upsample_backward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                             const void* grad_output, int64_t ld_out, void* grad_input, int64_t ld_in,
                             void* stream);

/* ---- particles <-> dense image at level_max - level_delta -------------------------------------
 * Replace apply_reconstruct / apply_reconstruct_backward (pyapr/aprnet/cuda/src/reconstruct_gpu.cu:159-225)
 * and apply_sample_particles / _backward (sample_particles_gpu.cu:172-246).  image: (channels, Z, X, Y)
 * contiguous with the extents of aprnet_image_dims(); particle tensors: (channels, ld).
 * reconstruct: piecewise-constant image from particle values; its backward sums the image gradient over
 * each particle's cell.  sample_particles: mean of the image over each particle's cell (cells are clipped
 * at the volume border); its backward spreads value / cell volume over the cell.  Every output element
 * has exactly one writer (no atomics). */
int aprnet_image_dims(const aprnet_apr* apr, int level_delta, int* z_num, int* x_num, int* y_num);
int aprnet_reconstruct_forward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                               const void* input, int64_t ld_in, void* image, void* stream);
int aprnet_reconstruct_backward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                                const void* grad_image, void* grad_input, int64_t ld_in, void* stream);
int aprnet_sample_particles_forward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                                    const void* image, void* output, int64_t ld_out, void* stream);
int aprnet_sample_particles_backward(const aprnet_apr* apr, int level_delta, int dtype, int channels,
                                     const void* grad_output, int64_t ld_out, void* grad_image, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* APRNET_B200_H */
