/*
 * b200loss.h — C ABI of libb200loss.so: fused per-pixel losses for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes only.  All pointers named
 * "logits", "labels", "losses", "grad*", "out", "jacc" and "workspace" are DEVICE
 * pointers owned by the caller; the library never allocates, frees or keeps a
 * pointer after it returns.
 * Work is enqueued on `stream` (a cudaStream_t passed as void*) and the call
 * returns without synchronising.  Return value: 0 on success, otherwise one of
 * the B200_ERR_* codes; b200_last_error() gives the message of the calling
 * thread's last failure.  Nothing throws across this boundary.
 *
 * Shapes follow the reference project (CoinCheung/pytorch-loss): logits are
 * [N, C, M] row-major with M = product of the trailing (spatial) dims, labels
 * are int64 [N, M] (focal: same dtype and shape as the logits).
 *
 * dtype codes: B200_F32 (float), B200_F16 (__half), B200_BF16 (__nv_bfloat16): the storage type of
 * logits, per-pixel losses and gradients; arithmetic is fp32.  B200_F64 (double, arithmetic in double)
 * is accepted by b200_{lsr,lmargin}_{forward,backward} and b200_focal_{forward,backward,forward_backward}.
 *
 * Reduction record ("out", 32 bytes, 8-byte aligned), written by the forward
 * kernels when `out` is non-NULL:
 *     double sum;     // sum of the per-pixel losses of valid pixels
 *     double count;   // number of valid (non-ignored) pixels / elements
 *     float  mean;    // (float)(sum / count)      (NaN when count == 0)
 *     float  sum32;   // (float)sum
 *     float  pad[2];
 *
 * Workspace: every op that reduces needs `b200_reduce_workspace_bytes()` bytes
 * of device memory whose first 64 bytes are ZERO before its first use; the
 * kernels leave them zero again, so one zero-initialised buffer per stream can
 * be reused forever.  Two calls that overlap on the GPU must not share one.
 * Byte 4..7 of the workspace is a status word: non-zero after a kernel gave up
 * a bounded wait (see b200_read_status).  Bytes 8..15 hold the optional exchange
 * context pointer (b200_reduce_attach_exchange; zero = none).
 */
#ifndef B200LOSS_H_
#define B200LOSS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK               0
#define B200_ERR_ARG          1   /* null pointer, bad size, bad dtype, misaligned buffer */
#define B200_ERR_UNSUPPORTED  2   /* shape outside what the kernels cover */
#define B200_ERR_LAUNCH       3   /* CUDA runtime reported an error at launch */
#define B200_ERR_STATUS       4   /* device status word set (a bounded wait ran out) */
#define B200_ERR_WORKSPACE    5   /* workspace too small */

#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2
#define B200_F64 3   /* double: per-pixel forward/backward entry points of label smooth, large margin, focal */

/* Version of this ABI (bumped on any signature change). */
int b200_abi_version(void);

/* Message of the calling thread's last failed call ("" if none). */
const char *b200_last_error(void);

/* Number of kernels this library has launched in this process so far (all threads,
 * all devices); a monotonically increasing diagnostic counter. */
uint64_t b200_kernel_launch_count(void);

/* Bytes of workspace the reducing forward kernels need (constant). */
size_t b200_reduce_workspace_bytes(void);

/* Synchronises `stream`, reads the workspace's status word, clears it, and returns
 * B200_OK or B200_ERR_STATUS.  For tests and debugging; never needed for results. */
int b200_read_status(void *workspace, void *stream);

/* ---------------------------------------------------- fused training step ---
 * The reference fuses forward and backward of the focal loss in
 * focal_cpp.focalloss_forward_backward (csrc/focal_kernel.cu:246-297, unscaled gradient, then a
 * `grads * grad_output` pass in Python, focal_loss.py:169).  For a REDUCED loss the final
 * gradient can be written directly:
 *   b200_focal_forward_backward_reduced: one pass; out = reduction record, grad_logits =
 *       dloss/dlogits * grad_scale / *denom (denom: optional device double, e.g. the global
 *       element count from b200_exchange_count; grad_scale: e.g. 1/E for 'mean').
 *   b200_focal_forward_backward_predicted: the same for a 'mean' over a batch sharded across
 *       GPUs, without a count exchange before it: the gradient is divided by *denom_state (device
 *       double: the global count the previous call found; initialise with b200_exchange_count),
 *       and after its cross-GPU sum the kernel stores predicted/actual count in *correction
 *       (device float; exactly 1 while shapes do not change) and the actual count in *denom_state.
 *   b200_rescale_gradient: grad *= *grad_out * *correction in place (device floats; correction
 *       may be null); every block leaves at once when the product is 1, as it is for
 *       `loss.backward()` in the steady state.
 *   b200_exchange_count: out->count = count summed over the ranks attached to the workspace
 *       (cross-GPU sum below); with nothing attached, out->count = count.
 */
int b200_focal_forward_backward_reduced(const void *logits, const void *labels, void *grad_logits,
                                        void *out, void *workspace, size_t workspace_bytes,
                                        const void *denom, float grad_scale, int64_t E, int dtype,
                                        float gamma, float alpha, int defer, void *stream);
int b200_focal_forward_backward_predicted(const void *logits, const void *labels, void *grad_logits,
                                          void *out, void *workspace, size_t workspace_bytes,
                                          void *denom_state, float *correction, int64_t E, int dtype,
                                          float gamma, float alpha, int defer, void *stream);
int b200_rescale_gradient(void *grad, const float *grad_out, const float *correction, int64_t E, int dtype,
                          void *stream);
/* Bits of the `defer` argument of the fused steps. */
#define B200_STEP_DEFER 1        /* post the sums to the peers, collect later (below) */
#define B200_STEP_AFTER_COUNT 2  /* softmax steps with a `denom`: b200_count_valid wrote it and is the
                                  * operation directly in front of this call on the stream, so the step's
                                  * kernel may start under the count's tail (programmatic dependent launch:
                                  * it fills its pipeline from the logits, which the count does not write,
                                  * and waits for the count before it reads *denom).  Do not set it when
                                  * anything else was enqueued in between. */
/* `defer` bit B200_STEP_DEFER (fused steps; only acts on a workspace with ranks attached, see "cross-GPU sum"): the
 * kernel posts this rank's [sum, count] to the peers and returns without waiting for theirs; the
 * record's float fields stay NaN (and *correction unwritten) until a later call on the same
 * stream completes it:
 *   b200_rescale_gradient_finish: what b200_rescale_gradient does, after collecting the ranks'
 *       sums into `out` (block 0; `correction` and `denom_state` as given to the _predicted step,
 *       else NULL) -- the wait for the slowest rank and the link overlaps the launch in between;
 *   b200_exchange_finish: only completes `out` (a loss that is read before or without backward).
 * Both do nothing extra when the record is complete already.  One record per workspace may be
 * pending at a time; complete it before the next reducing call on that workspace. */
int b200_rescale_gradient_finish(void *grad, const float *grad_out, float *correction, int64_t E, int dtype,
                                 void *workspace, void *out, void *denom_state, void *stream);
int b200_exchange_finish(void *workspace, void *out, void *denom_state, float *correction, void *stream);
int b200_exchange_count(double count, void *out, void *workspace, size_t workspace_bytes, void *stream);

/* The same fusion for the two softmax losses (no counterpart in the reference, whose
 * LSR_forward/LSR_backward, csrc/lsr_kernel.cu:191-318, and large-margin pair,
 * csrc/large_margin_kernel.cu:354-481, always read the logits twice per step):
 *   b200_softmax_fused_step_path: 1 when the layout has a fused step (channel columns of a
 *       pixel tile fit in shared memory, 16-byte aligned rows), else 0.
 *   b200_count_valid: out->count = number of labels != ignore_index (summed over attached
 *       ranks): the 'mean' divisor, needed on the device before gradients are written.
 *   b200_{lsr,lmargin}_forward_backward_reduced: one pass over the logits; out = reduction
 *       record of the loss, grad_logits = dloss/dlogits / *denom (denom: optional device double).
 *       B200_ERR_UNSUPPORTED when b200_softmax_fused_step_path says 0.
 * Backward of the step is b200_rescale_gradient. */
int b200_softmax_fused_step_path(const void *logits, const int64_t *labels, const void *grad_logits,
                                 int64_t N, int64_t C, int64_t M, int dtype);
int b200_count_valid(const int64_t *labels, int64_t P, int64_t ignore_index, void *out,
                     void *workspace, size_t workspace_bytes, void *stream);
int b200_lsr_forward_backward_reduced(const void *logits, const int64_t *labels, void *grad_logits,
                                      void *out, void *workspace, size_t workspace_bytes,
                                      const void *denom, int64_t N, int64_t C, int64_t M, int dtype,
                                      int64_t ignore_index, float smooth, int defer, void *stream);
int b200_lmargin_forward_backward_reduced(const void *logits, const int64_t *labels, void *grad_logits,
                                          void *out, void *workspace, size_t workspace_bytes,
                                          const void *denom, int64_t N, int64_t C, int64_t M, int dtype,
                                          int64_t ignore_index, float lam, int defer, void *stream);

/* ------------------------------------------------- cross-GPU sum (optional) ---
 * No counterpart in the reference (it has no multi-GPU path for these losses).
 * With one process per GPU and the batch sharded over the ranks, reduction 'mean'
 * needs the global [sum, count].  Instead of a collective call between the forward
 * and the backward kernel, the reducing forward kernel can exchange the pair
 * itself: attach an exchange context to a reduction workspace, and every reducing
 * forward that uses that workspace writes the GLOBAL sums into its record (all
 * ranks get identical bits; rank order summation).  All ranks must then make the
 * same sequence of reducing calls on their attached workspaces, like a collective.
 *
 * The context is `b200_exchange_ctx_bytes()` bytes of device memory laid out as
 *     int32 world; int32 rank; uint32 poll_limit; uint32 reserved;
 *     uint64 *seq;              // eight zero-initialised uint64 in this rank's memory (call
 *                               // counter; sequence number of a deferred sum)
 *     void  *slots[16];         // slots[p]: rank p's slot array as mapped in THIS
 *                               // process (p == rank: the local array); each array is
 *                               // b200_exchange_slot_bytes(world) bytes, zero-initialised
 * The peers' arrays are ordinary device allocations opened through CUDA IPC (or any
 * other peer mapping); the kernel only STORES to them and polls its own array.  Messages
 * are 8-byte words that carry their own flag (no fence between data and flag) and a tag
 * (count / loss sum).  A wait that exceeds poll_limit polls sets status bit 0x100, a message
 * with a foreign tag (the ranks' call sequences differ) sets 0x200 (b200_read_status); in
 * both cases the record's sum, count and mean are NaN, never a silently local or stale
 * number.  exchange_ctx == NULL detaches.
 */
/* Lets kernels of the calling thread's current device store into `peer_device`'s memory
 * (cudaDeviceEnablePeerAccess; already enabled counts as success). */
int b200_enable_peer_access(int peer_device);
/* CUDA IPC helpers for the slot arrays (each rank exports its array, every peer opens it
 * with its own device current, which maps it for that device's kernels).
 *   export: 64-byte handle of the allocation that contains dev_ptr + dev_ptr's offset in it
 *   open  : the peer's dev_ptr as mapped in this process (lazy peer access enabled)
 *   close : unmaps (pass the same offset) */
int b200_ipc_export(const void *dev_ptr, void *handle64, uint64_t *offset);
int b200_ipc_open(const void *handle64, uint64_t offset, void **mapped);
int b200_ipc_close(void *mapped, uint64_t offset);
size_t b200_exchange_ctx_bytes(void);
size_t b200_exchange_slot_bytes(int world);
int b200_reduce_attach_exchange(void *workspace, const void *exchange_ctx, void *stream);

/* ------------------------------------------------------------------ focal ---
 * Sigmoid focal loss, elementwise over E elements.
 * Replaces focal_cpp.focalloss_forward / focalloss_backward /
 * focalloss_forward_backward (reference csrc/focal_kernel.cu:301-341; math at
 * :30-118).  `labels` has the dtype of `logits` (soft labels allowed).
 *
 * forward:  losses (E elements, dtype) may be NULL; out (reduction record) may be
 *           NULL; at least one must be given.  workspace is required iff out != NULL.
 * backward: grad_logits[i] = dloss_i/dlogit_i * g, where g is
 *             grad_mode 0: 1
 *             grad_mode 1: *(const float*)grad_out            (one device scalar)
 *             grad_mode 2: ((const dtype*)grad_out)[i]        (elementwise)
 *           and, when denom != NULL, additionally divided by ((const double*)denom)[0]
 *           read on the device (the element count for reduction='mean', e.g. the
 *           `count` field of the reduction record, possibly all-reduced).
 * forward_backward: writes losses and unscaled gradients in one pass.
 */
int b200_focal_forward(const void *logits, const void *labels, void *losses, void *out,
                       void *workspace, size_t workspace_bytes, int64_t E, int dtype,
                       float gamma, float alpha, void *stream);
int b200_focal_backward(const void *logits, const void *labels, const void *grad_out,
                        int grad_mode, const void *denom, void *grad_logits, int64_t E,
                        int dtype, float gamma, float alpha, void *stream);
int b200_focal_forward_backward(const void *logits, const void *labels, void *losses,
                                void *grad_logits, int64_t E, int dtype, float gamma,
                                float alpha, void *stream);

/* Reducing focal forward that needs no workspace and allocates nothing.
 * This entry point has no counterpart in the reference.  It is for callers that cannot
 * provide device memory beyond inputs and outputs: a host that handed every byte of the GPU
 * to its own pool at start-up, or a bare FFI caller with no allocator that must not cause a
 * device-wide stall inside a hot loop.  The scratch of the reduction (64-byte header + one
 * 16-byte partial per block, 16 448 bytes in total) is a fixed array inside the library's
 * device image; every GPU that loads the library holds it until the process exits.
 *   - `out` (the 32-byte reduction record) is required, `losses` (E elements) is optional;
 *     both, like the inputs, are the caller's device memory.
 *   - E may be at most 2^28 = 268 435 456 elements; larger inputs are refused with
 *     B200_ERR_UNSUPPORTED (use b200_focal_forward with your own workspace instead).
 *   - The first call on each device looks up the array's device address (the device that
 *     is current at that moment must be the one the pointers live on).  Make that first
 *     call before any stream capture begins.
 *   - All calls on a device share the one array and each call re-arms its header on
 *     `stream` first.  Two calls that overlap on the GPU (different streams or threads)
 *     race on it: serialise them.
 * Neither this function nor anything it calls uses cudaMalloc, cudaFree or an allocating
 * library routine.  Per-element losses are bit-identical to b200_focal_forward's; the sum,
 * count and mean agree with it to the rounding of the reduction (another grid, so another
 * summation order: ~1e-7 relative, the count exactly). */
int b200_focal_forward_noalloc(const void *logits, const void *labels, void *losses, void *out,
                               int64_t E, int dtype, float gamma, float alpha, void *stream);

/* -------------------------------------------------- label-smooth softmax CE ---
 * Replaces lsr_cpp.lsr_forward / lsr_backward (reference csrc/lsr_kernel.cu:296-322;
 * math at :66-185) including the ATen log_softmax/softmax calls and the Python-side
 * `grad.mul_(grad_output.unsqueeze(1))`, `(labels != ignore).sum()` and
 * `losses.sum()` passes (reference pytorch_loss/label_smooth.py:144,169-170).
 *
 * forward:  losses ([N, M], dtype) may be NULL; out may be NULL; one must be given.
 * backward: grad_logits [N, C, M] = (sumy * softmax - y) * g, zero at ignored
 *           pixels, with g:
 *             grad_mode 0: 1
 *             grad_mode 1: *(const float*)grad_out
 *             grad_mode 2: ((const dtype*)grad_out)[n*M + m]   (per pixel)
 *           and, when denom != NULL, additionally divided by ((const double*)denom)[0]
 *           read on the device (the valid-pixel count, possibly all-reduced).
 */
int b200_lsr_forward(const void *logits, const int64_t *labels, void *losses, void *out,
                     void *workspace, size_t workspace_bytes, int64_t N, int64_t C,
                     int64_t M, int dtype, int64_t ignore_index, float smooth, void *stream);
int b200_lsr_backward(const void *logits, const int64_t *labels, const void *grad_out,
                      int grad_mode, const void *denom, void *grad_logits, int64_t N,
                      int64_t C, int64_t M, int dtype, int64_t ignore_index, float smooth,
                      void *stream);

/* ------------------------------------------------------ large-margin softmax ---
 * Replaces large_margin_cpp.l_margin_forward / l_margin_backward /
 * l_margin_forward_backward (reference csrc/large_margin_kernel.cu:796-838; math at
 * :388-481) and the Python-side scaling / counting passes (reference
 * large_margin_softmax.py:167,191,221-226).  Same argument conventions as LSR.
 */
int b200_lmargin_forward(const void *logits, const int64_t *labels, void *losses, void *out,
                         void *workspace, size_t workspace_bytes, int64_t N, int64_t C,
                         int64_t M, int dtype, int64_t ignore_index, float lam, void *stream);
int b200_lmargin_backward(const void *logits, const int64_t *labels, const void *grad_out,
                          int grad_mode, const void *denom, void *grad_logits, int64_t N,
                          int64_t C, int64_t M, int dtype, int64_t ignore_index, float lam,
                          void *stream);

/* ------------------------------------------------------------ Lovasz softmax ---
 * Replaces lovasz_softmax_cpp.lovasz_softmax_forward / lovasz_softmax_backward
 * (reference csrc/lovasz_softmax.cu:778-802; pipeline at :495-773, scan in
 * csrc/cumsum.hpp:113-150).
 *
 * Groups: per_image == 0 -> one group holding all N*M pixels (the reference's
 * behaviour); per_image != 0 -> every image is its own group.  G = number of groups,
 * L = pixels per group.  Segments are (group, class) pairs.
 *
 * forward:  loss  float[G*C]      per-segment Lovasz loss
 *           jacc  float[G*C*L]    Jaccard-gradient of every pixel, segment-major,
 *                                 pixel order inside the group (what backward needs)
 *           workspace: b200_lovasz_workspace_bytes(...) bytes, 256-byte aligned; no
 *           zero-initialisation required.
 * backward: grad float32 [G*C] upstream gradient per segment;
 *           grad_logits [N, C, M] (dtype).
 */
size_t b200_lovasz_workspace_bytes(int64_t N, int64_t C, int64_t M, int per_image);
int b200_lovasz_forward(const void *logits, const int64_t *labels, float *loss, float *jacc,
                        void *workspace, size_t workspace_bytes, int64_t N, int64_t C,
                        int64_t M, int dtype, int64_t ignore_index, int per_image,
                        void *stream);
int b200_lovasz_backward(const float *grad, const void *logits, const int64_t *labels,
                         const float *jacc, void *grad_logits, int64_t N, int64_t C,
                         int64_t M, int dtype, int64_t ignore_index, int per_image,
                         void *stream);

/* ---------------------------------- label smooth / large margin with statistics ---
 * No counterpart in the reference (its backward recomputes the softmax from scratch).
 * For many classes the forward kernel can leave 16 bytes of statistics per pixel
 * (maximum, 1 / sum, and for large margin two gradient coefficients) from which the
 * backward kernel produces every gradient element in one streaming pass.
 *   b200_softmax_stats_path(...) == 1 : the layout takes that path (more classes than a
 *       512-pixel resident tile holds, M >= 512, 16-byte aligned rows and pointers);
 *       pass grad_logits = NULL when asking on behalf of the forward.
 *   *_forward_ex : as *_forward, plus `stats` (float[N*M][4], 16-byte aligned, may be NULL);
 *       written only when the path applies to (logits, labels).
 *   *_backward_ex: as *_backward, plus the `stats` of the forward of the same inputs; used only
 *       when the path applies to (logits, labels, grad_logits), else the gradient is
 *       recomputed as in *_backward.  Pass stats only if the forward's query returned 1.
 */
int b200_softmax_stats_path(const void *logits, const int64_t *labels, const void *grad_logits,
                            int64_t N, int64_t C, int64_t M, int dtype);
int b200_lsr_forward_ex(const void *logits, const int64_t *labels, void *losses, void *out,
                        void *workspace, size_t workspace_bytes, void *stats, int64_t N, int64_t C,
                        int64_t M, int dtype, int64_t ignore_index, float smooth, void *stream);
int b200_lsr_backward_ex(const void *logits, const int64_t *labels, const void *stats,
                         const void *grad_out, int grad_mode, const void *denom, void *grad_logits,
                         int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index,
                         float smooth, void *stream);
int b200_lmargin_forward_ex(const void *logits, const int64_t *labels, void *losses, void *out,
                            void *workspace, size_t workspace_bytes, void *stats, int64_t N,
                            int64_t C, int64_t M, int dtype, int64_t ignore_index, float lam,
                            void *stream);
int b200_lmargin_backward_ex(const void *logits, const int64_t *labels, const void *stats,
                             const void *grad_out, int grad_mode, const void *denom,
                             void *grad_logits, int64_t N, int64_t C, int64_t M, int dtype,
                             int64_t ignore_index, float lam, void *stream);

/* ------------------------------------------------------------------- OHEM ---
 * Online hard example mining by score: the relabelling step in front of a
 * cross-entropy / large-margin loss.  Replaces ohem_cpp.score_ohem_label
 * (reference csrc/ohem_label_kernel.cu:179-262, :265-281; kernels :53-176; callers
 * pytorch_loss/ohem_loss.py:22-27,41-46).
 *   score_i = softmax(logits_i)[labels_i]   (1 for ignored pixels)
 *   out_i   = ignore_index  if score_i > max(score_thresh, t),  else labels_i,
 * where t is the n_min-th smallest score: the n_min hardest pixels and every pixel
 * scoring at most the threshold keep their label.  n_min >= N*M copies the labels;
 * n_min <= 0 lets the threshold alone decide.  Pixels tied with t all stay (the
 * reference's unstable sort keeps an unspecified subset of them).
 * out_labels may alias labels.  workspace: b200_ohem_workspace_bytes(N, M) bytes,
 * 256-byte aligned, contents irrelevant on entry.  At most 2^32 - 1 pixels.
 */
size_t b200_ohem_workspace_bytes(int64_t N, int64_t M);
int b200_ohem_label(const void *logits, const int64_t *labels, int64_t *out_labels,
                    void *workspace, size_t workspace_bytes, int64_t N, int64_t C, int64_t M,
                    int dtype, int64_t ignore_index, float score_thresh, int64_t n_min,
                    void *stream);

/* ---------------------------------------------------------- Taylor softmax ---
 * Softmax with e^x replaced by its Taylor polynomial of even order n,
 * f(x) = sum_{i<=n} x^i / i!, over the middle dimension of feat viewed as [N, C, M]:
 * out = f / sum_C f (use_log: its logarithm).  Replaces
 * taylor_softmax_cpp.taylor_softmax_forward / taylor_softmax_backward (reference
 * csrc/taylor_softmax.cu:391-421; kernels :50-265).  2 <= n <= 16, n even.
 * backward: grad_feat = d sum(out * grad) / d feat; grad has the shape and dtype of feat.
 */
int b200_taylor_softmax_forward(const void *feat, void *out, int64_t N, int64_t C, int64_t M,
                                int dtype, int n, int use_log, void *stream);
int b200_taylor_softmax_backward(const void *grad, const void *feat, void *grad_feat, int64_t N,
                                 int64_t C, int64_t M, int dtype, int n, int use_log,
                                 void *stream);

/* -------------------------------------------------- PC softmax cross entropy ---
 * Replaces the tensor-op chain of PCSoftmaxCrossEntropyV1 / PCSoftmaxCrossEntropyFunction
 * (reference pc_softmax.py:35-49, :52-97; the reference has no native kernel for it): with class
 * proportions weight[C] (device floats),
 *   losses[n, m]     = -(x_lb - max - log sum_j weight_j e^{x_j - max}), 0 at ignored pixels
 *   grad_logits[n,j,m] = weight_j e^{x_j - max} / sum_k weight_k e^{x_k - max} - 1[j == lb], 0 at
 *                        ignored pixels (the derivative of the loss above; the reference's V2
 *                        backward, pc_softmax.py:104-106, scales every channel by weight_lb instead)
 * in ONE launch; either output may be NULL.  Reduction and upstream gradient are the caller's. */
int b200_pc_softmax_ce(const void *logits, const int64_t *labels, const float *weight, void *losses,
                       void *grad_logits, int64_t N, int64_t C, int64_t M, int dtype,
                       int64_t ignore_index, void *stream);
/* The 'mean' / 'sum' TRAINING STEP of the same loss on the tile pipeline of the label-smooth step
 * (b200_lsr_forward_backward_reduced with smoothing 0 and the class weights inside the
 * exponentials): out = reduction record of the loss over the valid pixels, grad_logits =
 * d(loss sum)/d(logits) / *denom (denom: optional device double, e.g. the count of
 * b200_count_valid), ONE read of the logits.  b200_pc_softmax_step_path: 1 when the layout has
 * this step (M > 1, 16-byte aligned rows, at most 256 classes), else 0 -> use b200_pc_softmax_ce.
 * `flags`: B200_STEP_AFTER_COUNT as for the label-smooth step.  Backward: b200_rescale_gradient. */
int b200_pc_softmax_step_path(const void *logits, const int64_t *labels, const void *grad_logits,
                              int64_t N, int64_t C, int64_t M, int dtype);
int b200_pc_softmax_step(const void *logits, const int64_t *labels, const float *weight,
                         void *grad_logits, void *out, void *workspace, size_t workspace_bytes,
                         const void *denom, int64_t N, int64_t C, int64_t M, int dtype,
                         int64_t ignore_index, int flags, void *stream);
/* The same with the gradient divided by *denom (a device double, e.g. the count written by
 * b200_count_valid; NULL: not divided): what 'mean' needs, so that the caller's backward has
 * nothing left to do for an upstream gradient of 1 (the division the reference's backward
 * makes with a tensor op, pc_softmax.py:108-110). */
int b200_pc_softmax_ce_scaled(const void *logits, const int64_t *labels, const float *weight,
                              void *losses, void *grad_logits, const void *denom, int64_t N,
                              int64_t C, int64_t M, int dtype, int64_t ignore_index, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200LOSS_H_ */
