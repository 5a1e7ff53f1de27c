/*
 * sortnet_b200 — C ABI of the B200 (sm_100a) norm-distance neuron kernels.
 *
 * Drop-in boundary: these entry points are what a binding for the `norm_dist_cuda`
 * extension module of zbh2047/SortNet (core/cuda/norm_dist.cpp:294-318) calls instead of
 * the static launchers declared in core/cuda/norm_dist.h:4-60.  Argument order follows
 * those launchers: inputs, sizes (B, CO, CI, G, HW), outputs, optional index lists with the
 * full weight shape (W_CO, W_CI); a CUDA stream handle is appended.
 *
 * Conventions
 *   - All pointers are device pointers to contiguous fp32 / int32 arrays owned by the
 *     caller; the 2-D shapes (G == 1, HW == 1) allocate and free nothing.  Outputs are overwritten; gradient
 *     buffers are zero-filled by the backward entry points before they scatter into them
 *     (the reference launchers do the same, e.g. inf_dist_cuda.cu:332,348-349).
 *   - Shapes: x [B, CI, HW], w [W_CO, W_CI / G], y [B, CO, HW]; CO, CI, W_CO and W_CI are totals
 *     over the G groups (W_CI = columns of w times G, as core/cuda/norm_dist.cpp:139-143 passes
 *     it).  Group g of the outputs sees input channels g*CI/G .. (g+1)*CI/G - 1 and rows
 *     g*W_CO/G .. of w; the HW positions of a row are independent samples that share the row's
 *     sub-batch (inf_dist_cuda.cu:112-123,152-171).  G == 1 and HW == 1 (every fully connected
 *     SortNet layer) run the tiled kernels directly.  Any other G >= 1, HW >= 1 is served by
 *     repacking the operands into G row-major 2-D problems, running the same kernels on each and
 *     scattering the results back; that path takes its scratch from the stream-ordered allocator
 *     (a memory pool of the library's own, cudaMallocFromPoolAsync / cudaFreeAsync on `stream`), about
 *     two copies of the operands.
 *   - Index lists (`w_index_ci` [S, G, CI / G], `w_index_co` [S, G, CO / G], S = ceil(B / 32),
 *     int32, may be NULL) select, for each 32-row sub-batch, the columns / rows of w that the
 *     compact x / y correspond to (core/models/norm_dist.py:14-17; inf_dist_cuda.cu:123,166-169).
 *   - `stream` is a cudaStream_t (NULL = legacy default stream).  Work is enqueued on it and
 *     the call returns without synchronising.  Entry points are re-entrant and keep no
 *     mutable global state besides cached device attributes.
 *   - Return value: 0 on success, otherwise one of the SNB_STATUS_* codes below;
 *     snb_status_string() describes it and snb_last_cuda_error() gives the CUDA runtime
 *     message after SNB_STATUS_CUDA.  The reference launchers return void and check nothing.
 */
#ifndef SORTNET_B200_H
#define SORTNET_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SNB_STATUS_OK 0
#define SNB_STATUS_NULL_POINTER 1
#define SNB_STATUS_BAD_SHAPE 2
#define SNB_STATUS_UNSUPPORTED 3
#define SNB_STATUS_TOO_LARGE 4
#define SNB_STATUS_CUDA 5
#define SNB_STATUS_ALIGNMENT 6
#define SNB_STATUS_STATIC_CAPACITY 7
#define SNB_STATUS_INDEX_RANGE 8

const char* snb_status_string(int status);
const char* snb_last_cuda_error(void);
int snb_version(void);

/* 1 if a bounded device-side wait (the mbarrier waits of the TMA-staged kernels) ever gave up on the
 * current device, 0 if not, -1 on a CUDA error; synchronises the device.  No counterpart in the
 * reference. */
int snb_device_wait_failed(void);

/* Runs a register-only FMA chain (no counterpart in the reference); *flops = operations done.
 * The benchmark times it to get the FP32 CUDA-core peak used in its roofline fractions.
 * scratch: at least 4 bytes of device memory. */
int snb_probe_fp32(float* scratch, int iters, double* flops, void* stream);

/* ---- l-infinity distance ---------------------------------------------------------------- */

/* y[b,j] = max(1e-10, max_c |x[b,c] - w[co[s][j], ci[s][c]]|), pos[b,j] = lowest such c, bit 31
 * set when x - w < 0; pos = 0 when nothing exceeds 1e-10.
 * Replaces inf_dist::forward (norm_dist.h:24-26; inf_dist_cuda.cu:306-323). */
int snb_inf_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                         float* y, int* pos, const int* w_index_ci, const int* w_index_co,
                         int W_CO, int W_CI, void* stream);

/* The same operation with caller-provided scratch memory.  The kernel can then share output
 * tiles between thread blocks along the reduction axis (every SM gets the same amount of work
 * whatever the shape and mask sizes) and merge the partial (value, position) pairs with 64-bit
 * atomics in `workspace`; when workspace is NULL or smaller than
 * snb_inf_dist_forward_workspace_bytes(B, CO) = 8 * B * CO bytes, it behaves exactly like
 * snb_inf_dist_forward.  The workspace needs 8-byte alignment, may hold anything on entry and holds
 * nothing of value on return; results are bit-identical to snb_inf_dist_forward.
 * No counterpart in the reference (its launcher has no scratch argument). */
size_t snb_inf_dist_forward_workspace_bytes(int B, int CO);
int snb_inf_dist_forward_ws(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                            float* y, int* pos, const int* w_index_ci, const int* w_index_co,
                            int W_CO, int W_CI, void* workspace, size_t workspace_bytes, void* stream);

/* snb_inf_dist_forward_ws for index lists in ascending order (every list strictly increasing), the
 * order in which the sampler (snb_sample_mask) and the reference's sample_mask
 * (core/models/norm_dist.py:14-17, which ends with torch.sort) produce them.  With a 16-byte aligned
 * workspace of snb_inf_dist_forward_sorted_workspace_bytes(B, CO, W_CI) bytes (merge keys, a
 * [B, W_CI] copy of x with NaN in the dropped columns, inverse lists), W_CI a multiple of 4, a 16-byte
 * aligned w and at least 3/4 of the columns kept, W is read along whole rows with 16-byte copies: a
 * NaN difference never enters the maximum, and full-column order is list order, so y and pos are
 * bit-identical to snb_inf_dist_forward.  Otherwise it forwards to snb_inf_dist_forward_ws.  Lists
 * in another order still give exact y, but ties for the maximum may then resolve to another of the
 * tied positions.  No counterpart in the reference. */
size_t snb_inf_dist_forward_sorted_workspace_bytes(int B, int CO, int W_CI);
int snb_inf_dist_forward_sorted_ws(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                                   float* y, int* pos, const int* w_index_ci, const int* w_index_co,
                                   int W_CO, int W_CI, void* workspace, size_t workspace_bytes, void* stream);

/* Unmasked snb_inf_dist_forward for callers that must not allocate device memory.  It has no
 * counterpart in the reference.  Who needs it: a host that binds this C ABI directly — a C or C++
 * serving loop, a plugin inside another runtime — has no tensor library to hand it cached scratch,
 * and calling cudaMalloc / cudaFree around every forward is not an option for it: those calls
 * synchronise the whole device, can fail when memory is fragmented or budgeted by the embedding
 * application, and are forbidden in code paths that only enqueue work.  This variant runs the
 * same k-split kernel as snb_inf_dist_forward_ws, but its merge scratch is an 8 MiB array that
 * is part of the library image on every GPU that loads it; the function calls no allocator of
 * any kind (no cudaMalloc, no cudaFree, no library routine that allocates).
 *   - Limit: B * CO <= snb_inf_dist_forward_noalloc_max_outputs() = 1048576 (e.g. 128 x 5120);
 *     larger problems return SNB_STATUS_STATIC_CAPACITY and must use the other two entry points.
 *   - The first call on each device looks up the array's device address (a one-off set-up step
 *     done with that device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array: the part a call uses is cleared on `stream`
 *     before the kernel runs, and whatever the previous call left there is ignored, but two calls
 *     whose GPU work overlaps in time (different streams, different host threads) race on it.
 *     Serialise them, or give concurrent callers snb_inf_dist_forward_ws with their own scratch.
 *   - Results are bit-identical to snb_inf_dist_forward. */
int snb_inf_dist_forward_noalloc(const float* x, const float* w, int B, int CO, int CI, int G,
                                 int HW, float* y, int* pos, void* stream);
int snb_inf_dist_forward_noalloc_max_outputs(void);

/* Same y without pos, unmasked.  Replaces inf_dist::forward_nograd (norm_dist.h:22-23;
 * inf_dist_cuda.cu:277-304). */
int snb_inf_dist_forward_nograd(const float* x, const float* w, int B, int CO, int CI, int G,
                                int HW, float* y, void* stream);

/* grad_input[b, idx] += s * grad_output[b,j] with (idx, s) decoded from pos.
 * Replaces inf_dist::backward_input (norm_dist.h:27-28; inf_dist_cuda.cu:325-336). */
int snb_inf_dist_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI,
                                int G, int HW, float* grad_input, void* stream);

/* As above plus grad_weight[co[s][j], ci[s][idx]] -= s * grad_output[b,j]; grad_weight is the
 * full [W_CO, W_CI] matrix.  Replaces inf_dist::backward_input_weight (norm_dist.h:29-31;
 * inf_dist_cuda.cu:338-354). */
int snb_inf_dist_backward_input_weight(const float* grad_output, const int* pos, int B, int CO,
                                       int CI, int G, int HW, float* grad_input,
                                       float* grad_weight, const int* w_index_ci,
                                       const int* w_index_co, int W_CO, int W_CI, void* stream);

/* ---- l-p distance, finite p ----------------------------------------------------------------- */

/* p <= 10: y = max(sum_c |t|^p, FLT_MIN)^(1/p); p > 10: y = M (sum_c (|t|/M)^p + (1e-10/M)^p)^(1/p)
 * with M = max(1e-10, max_c |t|), t = x - w.  Integer p in [1, 8] uses multiply chains.
 * Replaces norm_dist<ip>::forward and ::forward_with_max(max_output = NULL) behind the p
 * dispatch of core/cuda/norm_dist.cpp:43-65 (norm_dist.h:5-10; norm_dist_cuda.cu:511-551). */
int snb_norm_dist_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                          float* y, float p, const int* w_index_ci, const int* w_index_co,
                          int W_CO, int W_CI, void* stream);

/* The same operation with caller-provided scratch memory for p > 10: the maxima M then live in
 * `workspace` (snb_norm_dist_forward_workspace_bytes(B, CO, p) = 4 * B * CO bytes, 16-byte aligned,
 * any content on entry) instead of y, which frees y to collect partial sums, so that thread blocks
 * can share output tiles along the reduction axis and every SM gets the same amount of work
 * whatever the shape and mask sizes.  For p <= 10 no scratch is needed (the function returns 0
 * bytes) and both entry points behave alike; with workspace NULL or too small the p > 10 case runs
 * one thread block per output tile.  Partial sums merge with floating-point atomics, so results
 * of the two entry points (and of repeated calls) can differ in the last bits.
 * No counterpart in the reference (its launcher has no scratch argument). */
size_t snb_norm_dist_forward_workspace_bytes(int B, int CO, float p);
int snb_norm_dist_forward_ws(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                             float* y, float p, const int* w_index_ci, const int* w_index_co,
                             int W_CO, int W_CI, void* workspace, size_t workspace_bytes, void* stream);

/* grad_input[b,c] = sum_j g[b,j] sgn(t) (|t| / y[b,j])^(p-1).
 * Replaces norm_dist<ip>::backward_input (norm_dist.h:11-13; norm_dist_cuda.cu:553-572). */
int snb_norm_dist_backward_input(const float* grad_output, const float* x, const float* w,
                                 const float* y, int B, int CO, int CI, int G, int HW,
                                 float* grad_input, float p, const int* w_index_ci,
                                 const int* w_index_co, int W_CO, int W_CI, void* stream);

/* As above plus grad_weight[co[s][j], ci[s][c]] -= the same terms summed over the sub-batch.
 * Replaces norm_dist<ip>::backward_input_weight (norm_dist.h:14-18; norm_dist_cuda.cu:574-594). */
int snb_norm_dist_backward_input_weight(const float* grad_output, const float* x, const float* w,
                                        const float* y, int B, int CO, int CI, int G, int HW,
                                        float* grad_input, float* grad_weight, float p,
                                        const int* w_index_ci, const int* w_index_co, int W_CO,
                                        int W_CI, void* stream);

/* ---- interval bounds through an l-infinity layer ------------------------------------------- */

/* yL = -min(-1e-10, min_c min(w - xL, xU - w)), yU = max(1e-10, max_c max(w - xL, xU - w)); an
 * inverted interval (xL > xU) is replaced by its midpoint.
 * Replaces bound_inf_dist::forward_nograd (norm_dist.h:35-36; bound_inf_dist_cuda.cu:314-328). */
int snb_bound_inf_dist_forward_nograd(const float* xl, const float* xu, const float* w, int B,
                                      int CO, int CI, int G, int HW, float* yl, float* yu,
                                      void* stream);

/* Same bounds plus the words of the coordinates that set them: c | (bit 31 when w - xL > xU - w);
 * posL = 0xffffffff when the lower bound stayed at its floor (no gradient), posU defaults to 0.
 * Replaces bound_inf_dist::forward (norm_dist.h:37-38; bound_inf_dist_cuda.cu:330-345). */
int snb_bound_inf_dist_forward(const float* xl, const float* xu, const float* w, int B, int CO,
                               int CI, int G, int HW, float* yl, float* yu, int* posl, int* posu,
                               void* stream);

/* Sparse backward of the bounds.  Replaces bound_inf_dist::backward_input and
 * ::backward_input_weight (norm_dist.h:39-44; bound_inf_dist_cuda.cu:362-383). */
int snb_bound_inf_dist_backward_input(const float* grad_yl, const float* grad_yu, const int* posl,
                                      const int* posu, int B, int CO, int CI, int G, int HW,
                                      float* grad_xl, float* grad_xu, void* stream);
int snb_bound_inf_dist_backward_input_weight(const float* grad_yl, const float* grad_yu,
                                             const int* posl, const int* posu, int B, int CO, int CI,
                                             int G, int HW, float* grad_xl, float* grad_xu,
                                             float* grad_w, void* stream);

/* ---- sort neuron (evaluation-time form of the masked l-infinity neuron) -------------------- */

/* y[b,j] = (1e-10 + sum_{r<K} q (1-q)^r * r-th largest |x[b,c] - w[j,c]|) / (1 - (1-q)^K),
 * 2 <= K <= 25, 0 < q < 1.  Replaces sort_neuron::forward_nograd (norm_dist.h:48-49;
 * sort_neuron.cu:403-435). */
int snb_sort_neuron_forward_nograd(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                                   float* y, float q, int K, void* stream);

/* Same value plus pos [K, B, CO, HW]: word of the r-th largest element (index | bit 31 when
 * x - w < 0); of equal values the later index ranks higher; unfilled ranks hold word 0.
 * Replaces sort_neuron::forward (norm_dist.h:50-51; sort_neuron.cu:453-485). */
int snb_sort_neuron_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW,
                            float* y, int* pos, float q, int K, void* stream);

/* Interval bounds of the sort neuron over the box [xL, xU].
 * Replaces bound_sort_neuron_forward_cuda (norm_dist.h:58-59; sort_neuron.cu:502-534). */
int snb_bound_sort_neuron_forward(const float* xl, const float* xu, const float* w, int B, int CO, int CI,
                                  int G, int HW, float* yl, float* yu, float q, int K, void* stream);

/* Sparse backward through the K recorded positions.  Replaces sort_neuron::backward_input and
 * ::backward_input_weight (norm_dist.h:52-56; sort_neuron.cu:536-562). */
int snb_sort_neuron_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI, int G,
                                   int HW, float* grad_input, float q, int K, void* stream);
int snb_sort_neuron_backward_input_weight(const float* grad_output, const int* pos, int B, int CO, int CI,
                                          int G, int HW, float* grad_input, float* grad_weight, float q,
                                          int K, void* stream);

/* ---- mean shift ------------------------------------------------------------------------------ */

/* mean[c] (c < C_full) = mean of x[b, slot(c)] over the rows whose sub-batch kept channel c
 * (index [S, C] sorted int32, NULL = all channels, then C_full == C); 0 for never-kept channels.
 * When running_mean is not NULL it is updated as (1 - momentum) * running_mean + momentum * mean.
 * Replaces the training branch of MeanShiftDropout.forward
 * (core/models/bound_basic_module.py:125-144), which is PyTorch code in the reference. */
int snb_mean_shift_stats(const float* x, const int* index, int B, int C, int C_full, float* mean,
                         float* running_mean, float momentum, void* stream);

/* y[b,j] = x[b,j] - mean[index[s_b][j]] (index NULL = identity); y may alias x.
 * Replaces core/models/bound_basic_module.py:149-157. */
int snb_mean_shift_apply(const float* x, const float* mean, const int* index, int B, int C,
                         float* y, void* stream);

/* ---- mask sampling ---------------------------------------------------------------------------- */

/* out [lists, count] int32: for each list an independent, uniformly random subset of
 * {0 .. channels-1} with exactly `count` elements, ascending.  Deterministic in (seed, lists,
 * channels, count).  channels <= 51200.  Replaces sample_mask (core/models/norm_dist.py:14-17:
 * uniform scores + top-k + sort in PyTorch); the caller draws `count` ~ Binomial(channels, keep rate) itself because it fixes the
 * tensor shapes. */
int snb_sample_mask(int* out, int lists, int channels, int count, unsigned long long seed, void* stream);

/* `jobs` (<= 16) calls of snb_sample_mask in one launch, e.g. the masks of every layer of a model for
 * one training step: outs[j] [lists, counts[j]] receives the lists that
 * snb_sample_mask(outs[j], lists, channels[j], counts[j], seeds[j]) would write.  outs, channels,
 * counts and seeds are host arrays of `jobs` entries.  No counterpart in the reference. */
int snb_sample_mask_batch(int jobs, int* const* outs, const int* channels, const int* counts,
                          const unsigned long long* seeds, int lists, void* stream);

/* Debug aid: checks caller-made index lists (index [lists, count] int32, i.e. the [S, G, count] lists
 * of one operand) before they are handed to the kernels, which read w through them unchecked like
 * the reference's (inf_dist_cuda.cu:163-172).  Returns SNB_STATUS_INDEX_RANGE when an entry lies
 * outside [0, channels); *flags (host pointer, may be NULL) receives bit 0 = out of range, bit 1 =
 * some list is not strictly ascending (legal, but the kernels gather fastest from ascending lists
 * and the argmax tie rule "lowest compact index" then means "lowest channel").  Runs a small kernel
 * and synchronises `stream`: not for the training loop.  sortnet_b200.norm_dist_cuda calls it for
 * every index list when SORTNET_B200_DEBUG=1.  No counterpart in the reference. */
int snb_check_index_lists(const int* index, int lists, int count, int channels, int* flags, void* stream);

/* Hands the scratch that grouped / spatial calls (G > 1 or HW > 1) left in the library's memory pool of
 * the current device back to the driver; the pool otherwise keeps up to 2 GiB of it for reuse.
 * No counterpart in the reference. */
int snb_trim_scratch(void);

/* ---- whole layers and the model head (G = 1, HW = 1) ---------------------------------------- */

/* One fully connected norm-distance layer of the training / plain forward in one call: the distance
 * (p = inf: snb_inf_dist_forward_sorted_ws when pos is given - index lists must be ascending -,
 * snb_inf_dist_forward_nograd when pos is NULL and there are no index lists; finite p:
 * snb_norm_dist_forward_ws) into y_dist, then, when `mean`
 * is not NULL, the batch mean per channel into mean [W_CO] with the momentum update of running_mean
 * (may be NULL), and out[b, j] = (y_dist[b, j] - mean[c]) + bias[c] with c = w_index_co[s_b][j] (mean
 * and bias optional; out may be y_dist).  workspace as in the _ws entry points (may be NULL).
 * Replaces the chain norm_dist_dropout / norm_dist -> MeanShiftDropout.forward -> bias add of
 * NormDistBase.forward (core/models/norm_dist.py:85-103; core/models/bound_basic_module.py:123-157). */
int snb_layer_forward(const float* x, const float* w, int B, int CO, int CI, float p, const int* w_index_ci,
                      const int* w_index_co, int W_CO, int W_CI, float* y_dist, int* pos, void* workspace,
                      size_t workspace_bytes, float* running_mean, float momentum, float* mean, const float* bias,
                      float* out, void* stream);

/* Backward of snb_layer_forward: grad_bias [W_CO] (optional) = column sums of grad_out over the rows
 * that kept each channel; with mean_shift != 0 the gradient is centred like the activations were
 * (mean [W_CO] and grad_centred [B, CO] are scratch); then the distance backward into grad_x
 * [B, CI] (NULL: stop after the bias gradient) and grad_w [W_CO, W_CI] (optional, zero-filled here).
 * pos is needed for p = inf, x / w / y_dist for finite p.
 * Replaces the autograd chain of the same Python code (core/norm_dist.py:75-99 for the operator). */
int snb_layer_backward(const float* grad_out, const float* x, const float* w, const float* y_dist, const int* pos,
                       int B, int CO, int CI, float p, const int* w_index_ci, const int* w_index_co, int W_CO,
                       int W_CI, int mean_shift, float* mean, float* grad_centred, float* grad_bias, float* grad_x,
                       float* grad_w, void* stream);

/* One layer of the evaluation-mode l-inf interval-bound pass: y = l-inf distance of the point value x
 * (x may be NULL), (yl, yu) = interval bounds of the box (xl, xu) (may be NULL), then running_mean
 * subtracted from and bias added to all three (each optional).
 * Replaces NormDistBase.forward in evaluation mode without a keep rate
 * (core/models/norm_dist.py:93-103) and MeanShiftDropout's evaluation branch. */
int snb_layer_bound_forward(const float* x, const float* xl, const float* xu, const float* w, int B, int CO, int CI,
                            const float* running_mean, const float* bias, float* y, float* yl, float* yu,
                            void* stream);

/* xl = max(x - eps, down), xu = min(x + eps, up) over n values: the input box of the certification
 * forward for scalar bounds.  Replaces ell_inf_models.py:35-36. */
int snb_input_box(const float* x, float eps, float down, float up, long long n, float* xl, float* xu, void* stream);

/* Head of the training step on the last layer's outputs d [B, K] with int64 targets:
 * margin[b, c] = ((d[b, t] + eps) - (d[b, c] - eps)) / (2 eps), 0 at c = t (written when margin is
 * not NULL); loss = mean_b (max_c clamp(margin, 0, clip) + lam * cross_entropy(-scale * d[b, :], t));
 * grad_d [B, K] (optional) = d loss / d d.  row_loss [B] is scratch; *loss is a device float.
 * Replaces ell_inf_models.py:45-50 and the `mixture` loss of main.py:357-364 with their autograd
 * backward. */
int snb_margin_loss(const float* d, const long long* target, int B, int K, float eps, float clip, float lam,
                    float scale, float* margin, float* row_loss, float* loss, float* grad_d, void* stream);

/* *fraction (device float) = share of rows b with max_{c != t} (yu[b, t] - yl[b, c]) < 0, i.e. whose
 * worst-case margin from the bounds (yl, yu) [B, K] of the last layer is negative for every wrong
 * class; row_flag [B] is scratch.  Replaces ell_inf_models.py:45-50 on the bounds plus the
 * certified-accuracy count of main.py:225-227. */
int snb_certified_fraction(const float* yl, const float* yu, const long long* target, int B, int K, float* row_flag,
                           float* fraction, void* stream);

/* ---- optimiser ------------------------------------------------------------------------------- */

/* One AdamW step over flat buffers of n fp32 values (n a multiple of 4, 16-byte aligned), with the
 * arithmetic of torch.optim.AdamW; g is multiplied by grad_scale first; step counts from 1.
 * Replaces the optimizer.step() of the reference's training loop (main.py:95,429-432), which is
 * PyTorch code there. */
int snb_adamw_step(float* w, const float* g, float* m, float* v, long long n, float lr, float beta1,
                   float beta2, float eps, float weight_decay, int step, float grad_scale, void* stream);

/* snb_adamw_step with the gradient given as `parts` (<= 16) partial buffers of n values each (a host
 * array of device pointers; summed in index order, then multiplied by grad_scale) and the new values
 * written to w_dst (may equal w_src).  It is the local part of a data-parallel step whose
 * reduce-scatter and all-gather are device-to-device copies that run beside other kernels; the
 * two parameter buffers let those kernels keep reading the old values meanwhile.
 * Replaces DistributedDataParallel's all-reduce plus optimizer.step() (main.py:402,95) together
 * with the copies. */
int snb_adamw_reduce_step(const float* w_src, float* w_dst, const void* const* grad_parts, int parts, float* m,
                          float* v, long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                          int step, float grad_scale, void* stream);

/* Data-parallel AdamW step fused with the gradient exchange: this rank sums elements [lo, hi) of
 * the flat gradient buffers of all `world` ranks (peer pointers of one NVLink node, entry `rank`
 * its own), divides by world, applies AdamW with its shard-sized moments m, v and stores the new
 * parameter values into every rank's flat parameter buffer.  lo, hi multiples of 4; all pointers
 * 16-byte aligned; world <= 16.  The caller orders ranks with barriers (snb_peer_barrier) before and
 * after.
 * Replaces DistributedDataParallel's all-reduce plus optimizer.step() (main.py:402,95). */
int snb_dp_adamw_step(const void* const* grad_ptrs, void* const* param_ptrs, float* m, float* v, int rank,
                      int world, long long lo, long long hi, float lr, float beta1, float beta2, float eps,
                      float weight_decay, int step, void* stream);

/* Stream-ordered barrier between the `world` (<= 16) ranks of one NVLink node, one process per GPU:
 * enqueues one small kernel that stores `epoch` into every peer's flag word for this rank (release,
 * system scope) and waits until this rank's own flag words hold `epoch` or later.  flag_ptrs: host
 * array of `world` pointers to the ranks' flag arrays (`world` 32-bit words each, zero-initialised,
 * mapped into this process; entry `rank` is this GPU's own).  Every barrier on the same flags
 * passes the next epoch (1, 2, 3, ...), the same on all ranks.  The wait is bounded: after
 * timeout_ns nanoseconds the kernel writes 1 + (rank it gave up on) into *status (any
 * device-accessible int, e.g. pinned host memory, 0 on entry) and returns; nothing traps or hangs,
 * and the host reads *status when it next synchronises.  What ran after a failed barrier read
 * stale data and must be discarded.
 * Replaces the ordering DistributedDataParallel gets from NCCL (main.py:402); the reference has
 * no time-out (a missing rank hangs it). */
int snb_peer_barrier(void* const* flag_ptrs, int rank, int world, unsigned int epoch,
                     unsigned long long timeout_ns, int* status, void* stream);

/* The two halves of snb_peer_barrier as separate stream-ordered operations with the same arguments:
 * snb_peer_signal stores `epoch` into every peer's flag word for this rank, snb_peer_wait waits
 * (bounded, as above) until this rank's flag words hold `epoch` or later.  A kernel that waits on
 * the GPU costs the kernels running beside it about half of the time it waits (measured on B200),
 * so a caller with work to overlap signals as early and waits as late as its data flow allows: by
 * then the peers have signalled and the wait returns at once.  No counterpart in the reference. */
int snb_peer_signal(void* const* flag_ptrs, int rank, int world, unsigned int epoch, void* stream);
int snb_peer_wait(void* const* flag_ptrs, int rank, int world, unsigned int epoch, unsigned long long timeout_ns,
                  int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SORTNET_B200_H */
