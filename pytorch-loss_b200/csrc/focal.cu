// Sigmoid focal loss for sm_100a: one streaming kernel family.
//
// Math follows the reference's elementwise kernels (csrc/focal_kernel.cu:30-118):
//   p = sigmoid(x), log p = x >= 0 ? -log1p(e^-x) : x - log1p(e^x), log(1-p) = log p - x
//   ce = y*a*log p + (1-y)*(1-a)*log(1-p);  coeff = -|y-p|^g;  loss = coeff*ce
//   d_ce = y*a - p*(1 - y - a + 2*y*a);  d_coeff = g*|y-p|^(g-1)*p*(1-p), negated if y < p
//   grad = d_coeff*ce + d_ce*coeff
// One exp and one log per element serve both branches (e = e^-|x|), on the special-function
// unit's approximate instructions: the full-precision expf/log1pf/division sequences cost
// ~110 issue slots per element, which made the kernel instruction-bound at half of HBM speed.
//
// Data movement: 16-byte loads/stores, two vectors in flight per thread per array,
// persistent grid of kBlocksPerSM blocks per SM; the 'mean'/'sum' forward writes no
// per-element loss at all (8 B/element), the backward recomputes (12 B/element).
#include "common.cuh"

#include <mutex>
#include <stdlib.h>

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerSM = 4;

enum FocalMode { kFwd = 0, kBwd = 1, kFwdBwd = 2 };

struct FocalParams {
    const void *logits;
    const void *labels;
    void *losses;        // may be null (kFwd with reduce only)
    void *grads;         // kBwd / kFwdBwd
    const void *grad_out;
    int grad_mode;       // 0 none, 1 device float scalar, 2 elementwise (dtype)
    const double *denom; // optional device divisor
    void *workspace;     // reduce
    ReduceRecord *out;   // reduce
    int64_t E;
    float gamma, alpha;
    float host_scale;    // extra factor on the gradient (0 is read as 1): 1/E of a fused 'mean' step
    double *denom_state; // optional: predicted divisor, replaced by the reduced count after the sum
    float *correction;   // with denom_state: predicted / actual divisor of this call
    int defer;           // cross-GPU sum: post only; b200_exchange_finish / b200_rescale_gradient_finish collect
};

// The fused step of a batch sharded over GPUs divides by the GLOBAL element count, which the
// kernel only knows after its own cross-GPU sum.  It therefore divides by the count the previous
// call found (*denom_state), and the thread that writes the record stores predicted / actual for
// the rescale kernel and the actual count for the next call.  With unchanged shapes the
// correction is exactly 1.  Every block has read *denom_state before it took its ticket, so
// the overwrite cannot be seen by this launch.
__device__ __forceinline__ void publish_denominator(double *denom_state, float *correction, const ReduceRecord *out) {
    if (!denom_state) return;
    const double used = *denom_state, actual = out->count;
    *correction = static_cast<float>(used / actual);
    *denom_state = actual;
}
__device__ __forceinline__ void publish_denominator(const FocalParams &prm) {
    publish_denominator(prm.denom_state, prm.correction, prm.out);
}

template <bool GAMMA2>
__device__ __forceinline__ void focal_core(float x, float y, float gamma, float alpha, float &loss,
                                           float &grad, bool want_grad) {
    // e in (0, 1]: one ex2.approx, one rcp.approx, one lg2.approx.  log1p(e) = log(1 + e) is
    // taken at an argument in (1, 2], where the absolute error of lg2.approx (2^-22) plus the
    // rounding of 1 + e stays below 3e-7 -- two orders below the gradient tolerance and, being
    // unbiased over elements, far below the relative tolerance of the reduced loss.
    const float e = __expf(-fabsf(x));
    const float inv = __fdividef(1.f, 1.f + e);
    const float p = x >= 0.f ? inv : e * inv;
    const float l1p = __logf(1.f + e);
    const float log_p = x >= 0.f ? -l1p : x - l1p;
    const float ce = y * alpha * log_p + (1.f - y) * (1.f - alpha) * (log_p - x);
    const float d = fabsf(y - p);
    const float coeff = GAMMA2 ? -(d * d) : -powf(d, gamma);
    loss = coeff * ce;
    if (want_grad) {
        const float d_ce = y * alpha - p * (1.f - y - alpha + 2.f * y * alpha);
        float d_coeff = (GAMMA2 ? 2.f * d : gamma * powf(d, gamma - 1.f)) * p * (1.f - p);
        if (y < p) d_coeff = -d_coeff;
        grad = d_coeff * ce + d_ce * coeff;
    }
}

template <typename T, int MODE, bool GAMMA2, bool REDUCE, int UNROLL = 2>
__global__ void __launch_bounds__(kThreads) focal_kernel(const FocalParams prm) {
    using V = Vec16<T>;
    constexpr int VN = V::N;
    const T *__restrict__ logits = static_cast<const T *>(prm.logits);
    const T *__restrict__ labels = static_cast<const T *>(prm.labels);
    T *__restrict__ losses = static_cast<T *>(prm.losses);
    T *__restrict__ grads = static_cast<T *>(prm.grads);
    const T *__restrict__ gout = static_cast<const T *>(prm.grad_out);
    const float gamma = prm.gamma, alpha = prm.alpha;
    constexpr bool kGrad = MODE != kFwd;
    constexpr bool kLoss = MODE != kBwd;

    float gscale = 1.f;
    if (MODE == kBwd && prm.grad_mode == 1) gscale = *static_cast<const float *>(prm.grad_out);
    if (MODE != kFwd && prm.denom) gscale = static_cast<float>(double(gscale) / *prm.denom);
    if (MODE != kFwd && prm.host_scale != 0.f) gscale *= prm.host_scale;
    const bool per_elem = (MODE == kBwd) && prm.grad_mode == 2;

    double acc = 0.0;
    const int64_t nvec = prm.E / VN;
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x;

    auto do_vec = [&](int64_t vi, const V &xv, const V &yv) {
        V lv, gv, sv;
        if (per_elem) sv = ld_stream16<V>(gout + vi * VN);
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < VN; ++k) {
            float loss, grad = 0.f;
            focal_core<GAMMA2>(to_f32(xv.v[k]), to_f32(yv.v[k]), gamma, alpha, loss, grad, kGrad);
            if (kLoss) {
                part += loss;
                lv.v[k] = from_f32<T>(loss);
            }
            if (kGrad) {
                const float s = per_elem ? gscale * to_f32(sv.v[k]) : gscale;
                gv.v[k] = from_f32<T>(grad * s);
            }
        }
        if (kLoss && losses) st_stream16(losses + vi * VN, lv);
        if (kGrad) st_stream16(grads + vi * VN, gv);
        if (REDUCE) acc += double(part);
    };

    // UNROLL vectors per array in flight per thread
    for (; i + (UNROLL - 1) * stride < nvec; i += UNROLL * stride) {
        V xs[UNROLL], ys[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            xs[u] = ld_stream16<V>(logits + (i + u * stride) * VN);
            ys[u] = ld_stream16<V>(labels + (i + u * stride) * VN);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) do_vec(i + u * stride, xs[u], ys[u]);
    }
    for (; i < nvec; i += stride) {
        const V x0 = ld_stream16<V>(logits + i * VN);
        const V y0 = ld_stream16<V>(labels + i * VN);
        do_vec(i, x0, y0);
    }
    // scalar tail (E not a multiple of the vector width)
    if (blockIdx.x == 0) {
        for (int64_t j = nvec * VN + threadIdx.x; j < prm.E; j += kThreads) {
            float loss, grad = 0.f;
            focal_core<GAMMA2>(to_f32(logits[j]), to_f32(labels[j]), gamma, alpha, loss, grad, kGrad);
            if (kLoss && losses) losses[j] = from_f32<T>(loss);
            if (kGrad) {
                const float s = per_elem ? gscale * to_f32(gout[j]) : gscale;
                grads[j] = from_f32<T>(grad * s);
            }
            if (REDUCE) acc += double(loss);
        }
    }
    if (REDUCE) {
        __shared__ double sh[64];
        const double cnt = (blockIdx.x == 0 && threadIdx.x == 0) ? double(prm.E) : 0.0;
        if (grid_reduce_finish(acc, cnt, prm.workspace, prm.out, sh, kTagSum, prm.defer != 0)) publish_denominator(prm);
    }
}

// Bulk-copy ring variant.  Plain 128-bit loads top out near 4 TB/s of reads on B200 (the SM's
// outstanding-load capacity divided by the loaded latency), whatever the unrolling or the
// number of blocks; bulk-async copies do not go through that path.  One thread of an extra
// warp streams chunks of logits and labels into a ring of shared-memory stages, the compute
// warps read them back with 16-byte shared loads, gradients/losses leave with plain 128-bit
// stores (stores are not the limiter).  Hand-offs: full[s] (copy bytes landed), empty[s]
// (one arrival per compute warp).  Every wait is bounded.
constexpr int kRingStages = 4;
constexpr int kRingChunkBytes = 8192;             // per array and stage
constexpr int kRingBlock = kThreads + 32;

template <typename T, int MODE, bool GAMMA2, bool REDUCE>
__global__ void __launch_bounds__(kRingBlock) focal_ring_kernel(const FocalParams prm) {
    using V = Vec16<T>;
    constexpr int VN = V::N;
    constexpr int kChunkElems = kRingChunkBytes / int(sizeof(T));
    constexpr int kVecPerThread = kChunkElems / VN / kThreads;
    static_assert(kVecPerThread >= 1, "chunk too small for the block");
    extern __shared__ unsigned char ring_raw[];
    unsigned char(*stage_mem)[2][kRingChunkBytes] = reinterpret_cast<unsigned char(*)[2][kRingChunkBytes]>(
        ring_raw + ((128u - (smem_u32(ring_raw) & 127u)) & 127u));
    __shared__ __align__(8) uint64_t full[kRingStages], empty[kRingStages];
    __shared__ double sh[64];

    const T *__restrict__ logits = static_cast<const T *>(prm.logits);
    const T *__restrict__ labels = static_cast<const T *>(prm.labels);
    T *__restrict__ losses = static_cast<T *>(prm.losses);
    T *__restrict__ grads = static_cast<T *>(prm.grads);
    const T *__restrict__ gout = static_cast<const T *>(prm.grad_out);
    const float gamma = prm.gamma, alpha = prm.alpha;
    constexpr bool kGrad = MODE != kFwd;
    constexpr bool kLoss = MODE != kBwd;
    const int tid = threadIdx.x;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;

    if (tid == 0) {
        for (int s = 0; s < kRingStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kThreads / 32);
        }
        fence_mbar_init();
    }
    __syncthreads();

    const int64_t nvec = prm.E / VN;                        // whole vectors
    const int64_t nchunks = (nvec * VN + kChunkElems - 1) / kChunkElems;
    double acc = 0.0;

    if (tid == kThreads) {
        int k = 0;
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++k) {
            const int s = k % kRingStages;
            if (k >= kRingStages && !mbar_wait_bounded(&empty[s], ((k / kRingStages) - 1) & 1, status)) break;
            const int64_t e0 = c * kChunkElems;
            int64_t ne = nvec * VN - e0;
            if (ne > kChunkElems) ne = kChunkElems;
            const uint32_t bytes = uint32_t(ne) * sizeof(T);   // multiple of 16
            mbar_expect_tx(&full[s], 2 * bytes);
            bulk_load_1d(stage_mem[s][0], logits + e0, bytes, &full[s]);
            bulk_load_1d(stage_mem[s][1], labels + e0, bytes, &full[s]);
        }
    } else if (tid < kThreads) {
        float gscale = 1.f;
        if (MODE == kBwd && prm.grad_mode == 1) gscale = *static_cast<const float *>(prm.grad_out);
        if (MODE != kFwd && prm.denom) gscale = static_cast<float>(double(gscale) / *prm.denom);
    if (MODE != kFwd && prm.host_scale != 0.f) gscale *= prm.host_scale;
        const bool per_elem = (MODE == kBwd) && prm.grad_mode == 2;
        const int lane = tid & 31;
        int k = 0;
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++k) {
            const int s = k % kRingStages;
            const int64_t v0 = c * (kChunkElems / VN);          // first vector of the chunk
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&full[s], (k / kRingStages) & 1, status);
            if (!compute_all(ok, kThreads)) break;
            const V *sx = reinterpret_cast<const V *>(stage_mem[s][0]);
            const V *sy = reinterpret_cast<const V *>(stage_mem[s][1]);
            float part = 0.f;
#pragma unroll
            for (int u = 0; u < kVecPerThread; ++u) {
                const int lv = u * kThreads + tid;
                const int64_t vi = v0 + lv;
                if (vi < nvec) {
                    const V xv = sx[lv], yv = sy[lv];
                    V lvv, gv, sv;
                    if (per_elem) sv = ld_stream16<V>(gout + vi * VN);
#pragma unroll
                    for (int q = 0; q < VN; ++q) {
                        float loss, grad = 0.f;
                        focal_core<GAMMA2>(to_f32(xv.v[q]), to_f32(yv.v[q]), gamma, alpha, loss, grad, kGrad);
                        if (kLoss) {
                            part += loss;
                            lvv.v[q] = from_f32<T>(loss);
                        }
                        if (kGrad) {
                            const float sc = per_elem ? gscale * to_f32(sv.v[q]) : gscale;
                            gv.v[q] = from_f32<T>(grad * sc);
                        }
                    }
                    if (kLoss && losses) st_stream16(losses + vi * VN, lvv);
                    if (kGrad) st_stream16(grads + vi * VN, gv);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (REDUCE) acc += double(part);
        }
        // scalar tail (E not a multiple of the vector width)
        if (blockIdx.x == 0) {
            for (int64_t j = nvec * VN + tid; j < prm.E; j += kThreads) {
                float loss, grad = 0.f;
                focal_core<GAMMA2>(to_f32(logits[j]), to_f32(labels[j]), gamma, alpha, loss, grad, kGrad);
                if (kLoss && losses) losses[j] = from_f32<T>(loss);
                if (kGrad) {
                    const float sc = per_elem ? gscale * to_f32(gout[j]) : gscale;
                    grads[j] = from_f32<T>(grad * sc);
                }
                if (REDUCE) acc += double(loss);
            }
        }
    }
    if (REDUCE) {
        const double cnt = (blockIdx.x == 0 && tid == 0) ? double(prm.E) : 0.0;
        if (grid_reduce_finish(acc, cnt, prm.workspace, prm.out, sh, kTagSum, prm.defer != 0)) publish_denominator(prm);
    }
}

// Scalar-only variant for buffers that are not 16-byte aligned.
template <typename T, int MODE, bool REDUCE>
__global__ void __launch_bounds__(kThreads) focal_kernel_unaligned(const FocalParams prm) {
    const T *logits = static_cast<const T *>(prm.logits);
    const T *labels = static_cast<const T *>(prm.labels);
    T *losses = static_cast<T *>(prm.losses);
    T *grads = static_cast<T *>(prm.grads);
    const T *gout = static_cast<const T *>(prm.grad_out);
    constexpr bool kGrad = MODE != kFwd;
    constexpr bool kLoss = MODE != kBwd;
    float gscale = 1.f;
    if (MODE == kBwd && prm.grad_mode == 1) gscale = *static_cast<const float *>(prm.grad_out);
    if (MODE != kFwd && prm.denom) gscale = static_cast<float>(double(gscale) / *prm.denom);
    if (MODE != kFwd && prm.host_scale != 0.f) gscale *= prm.host_scale;
    const bool per_elem = (MODE == kBwd) && prm.grad_mode == 2;
    double acc = 0.0;
    for (int64_t j = int64_t(blockIdx.x) * kThreads + threadIdx.x; j < prm.E;
         j += int64_t(gridDim.x) * kThreads) {
        float loss, grad = 0.f;
        focal_core<false>(to_f32(logits[j]), to_f32(labels[j]), prm.gamma, prm.alpha, loss, grad, kGrad);
        if (kLoss && losses) losses[j] = from_f32<T>(loss);
        if (kGrad) {
            const float s = per_elem ? gscale * to_f32(gout[j]) : gscale;
            grads[j] = from_f32<T>(grad * s);
        }
        if (REDUCE) acc += double(loss);
    }
    if (REDUCE) {
        __shared__ double sh[64];
        const double cnt = (blockIdx.x == 0 && threadIdx.x == 0) ? double(prm.E) : 0.0;
        if (grid_reduce_finish(acc, cnt, prm.workspace, prm.out, sh, kTagSum, prm.defer != 0)) publish_denominator(prm);
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int MODE, bool REDUCE>
int launch_focal(const FocalParams &prm, cudaStream_t stream) {
    const int vn = Vec16<T>::N;
    int64_t want = (prm.E / vn + kThreads - 1) / kThreads;
    // the fused step (loss sum + gradient) runs best with all eight blocks of an SM resident and
    // one vector per array in flight per thread: 38.8 us against 43.2 us at 16.7 M elements
    constexpr bool kFusedStep = MODE == kFwdBwd && REDUCE;
    constexpr int bps = kFusedStep ? 8 : kBlocksPerSM;
    int64_t cap = int64_t(sm_count()) * bps;
    if (REDUCE && cap > kMaxPartials) cap = kMaxPartials;      // one partial slot per block
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    const dim3 grid(static_cast<unsigned>(want));
    const bool al = aligned16(prm.logits) && aligned16(prm.labels) &&
                    (!prm.losses || aligned16(prm.losses)) && (!prm.grads || aligned16(prm.grads)) &&
                    (prm.grad_mode != 2 || aligned16(prm.grad_out));
    // the ring wins for the read-only forward (8% at the 16.7 M-element size); with a gradient
    // stream to write, plain loads + stores are as fast and simpler (fused step: ring 40.1 us at
    // its best geometry, plain 39.1 us)
    if (al && MODE == kFwd) {
        constexpr size_t smem = 128 + size_t(kRingStages) * 2 * kRingChunkBytes;
        const int per_sm = int((220 * 1024) / (smem + 1024));
        const int64_t chunk_elems = kRingChunkBytes / sizeof(T);
        int64_t g = (prm.E + chunk_elems - 1) / chunk_elems;
        if (g > int64_t(sm_count()) * per_sm) g = int64_t(sm_count()) * per_sm;
        if (REDUCE && g > kMaxPartials) g = kMaxPartials;
        if (g < 1) g = 1;
        auto go = [&](auto kern) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            kern<<<dim3(unsigned(g)), kRingBlock, smem, stream>>>(prm);
        };
        if (prm.gamma == 2.f) go(focal_ring_kernel<T, MODE, true, REDUCE>);
        else go(focal_ring_kernel<T, MODE, false, REDUCE>);
        return launch_status("focal ring kernel launch");
    }
    if (!al) {
        focal_kernel_unaligned<T, MODE, REDUCE><<<grid, kThreads, 0, stream>>>(prm);
    } else if (prm.gamma == 2.f && kFusedStep) {
        focal_kernel<T, MODE, true, REDUCE, 1><<<grid, kThreads, 0, stream>>>(prm);
    } else if (prm.gamma == 2.f) {
        focal_kernel<T, MODE, true, REDUCE><<<grid, kThreads, 0, stream>>>(prm);
    } else {
        focal_kernel<T, MODE, false, REDUCE><<<grid, kThreads, 0, stream>>>(prm);
    }
    return launch_status("focal kernel launch");
}

template <int MODE, bool REDUCE>
int dispatch_focal(const FocalParams &prm, int dtype, cudaStream_t stream) {
    if (dtype == B200_F32) return launch_focal<float, MODE, REDUCE>(prm, stream);
    if (dtype == B200_F16) return launch_focal<__half, MODE, REDUCE>(prm, stream);
    if (dtype == B200_BF16) return launch_focal<__nv_bfloat16, MODE, REDUCE>(prm, stream);
    set_error("focal: unknown dtype code %d", dtype);
    return B200_ERR_ARG;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_focal_forward(const void *logits, const void *labels, void *losses, void *out,
                                  void *workspace, size_t workspace_bytes, int64_t E, int dtype,
                                  float gamma, float alpha, void *stream) {
    if (E == 0 && !out) return B200_OK;   // empty input, nothing to write
    if (E < 0 || (!losses && !out)) {
        set_error("b200_focal_forward: need E >= 0 and at least one of losses/out");
        return B200_ERR_ARG;
    }
    if (E > 0 && (!logits || !labels)) {
        set_error("b200_focal_forward: null input pointer");
        return B200_ERR_ARG;
    }
    if (out && (!workspace || workspace_bytes < kReduceWorkspaceBytes)) {
        set_error("b200_focal_forward: workspace of %zu bytes required, got %zu",
                  kReduceWorkspaceBytes, workspace ? workspace_bytes : size_t(0));
        return B200_ERR_WORKSPACE;
    }
    if (E == 0 && !out) return B200_OK;
    if (dtype == B200_F64)
        return f64_focal(logits, labels, losses, nullptr, nullptr, 0, nullptr, out, workspace, E, gamma, alpha, stream);
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.losses = losses;
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return out ? dispatch_focal<kFwd, true>(prm, dtype, s) : dispatch_focal<kFwd, false>(prm, dtype, s);
}

extern "C" int b200_focal_backward(const void *logits, const void *labels, const void *grad_out,
                                   int grad_mode, const void *denom, void *grad_logits, int64_t E,
                                   int dtype, float gamma, float alpha, void *stream) {
    if (E < 0 || grad_mode < 0 || grad_mode > 2 || (grad_mode != 0 && !grad_out)) {
        set_error("b200_focal_backward: bad E / grad_mode / grad_out");
        return B200_ERR_ARG;
    }
    if (E == 0) return B200_OK;
    if (!logits || !labels || !grad_logits) {
        set_error("b200_focal_backward: null pointer");
        return B200_ERR_ARG;
    }
    if (dtype == B200_F64)
        return f64_focal(logits, labels, nullptr, grad_logits, grad_out, grad_mode, denom, nullptr, nullptr, E, gamma,
                         alpha, stream);
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.grad_out = grad_out;
    prm.grad_mode = grad_mode;
    prm.denom = static_cast<const double *>(denom);
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    return dispatch_focal<kBwd, false>(prm, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_focal_forward_backward(const void *logits, const void *labels, void *losses,
                                           void *grad_logits, int64_t E, int dtype, float gamma,
                                           float alpha, void *stream) {
    if (E < 0) {
        set_error("b200_focal_forward_backward: E < 0");
        return B200_ERR_ARG;
    }
    if (E == 0) return B200_OK;
    if (!logits || !labels || !losses || !grad_logits) {
        set_error("b200_focal_forward_backward: null pointer");
        return B200_ERR_ARG;
    }
    if (dtype == B200_F64)
        return f64_focal(logits, labels, losses, grad_logits, nullptr, 0, nullptr, nullptr, nullptr, E, gamma, alpha,
                         stream);
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.losses = losses;
    prm.grads = grad_logits;
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    return dispatch_focal<kFwdBwd, false>(prm, dtype, static_cast<cudaStream_t>(stream));
}

// Loss sum and FINAL gradient of a reduced focal loss in one pass over the inputs: the fused
// training step (reads logits and labels once, writes the gradient once).  The gradient is
// scaled by grad_scale / *denom (denom: optional device double, e.g. the global element count
// of a batch sharded over several GPUs; grad_scale: e.g. 1/E for 'mean').
extern "C" int b200_focal_forward_backward_reduced(const void *logits, const void *labels, void *grad_logits,
                                                   void *out, void *workspace, size_t workspace_bytes,
                                                   const void *denom, float grad_scale, int64_t E, int dtype,
                                                   float gamma, float alpha, int defer, void *stream) {
    if (E < 0 || !out) {
        set_error("b200_focal_forward_backward_reduced: need E >= 0 and out");
        return B200_ERR_ARG;
    }
    if (!workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("b200_focal_forward_backward_reduced: workspace of %zu bytes required", kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    if (E > 0 && (!logits || !labels || !grad_logits)) {
        set_error("b200_focal_forward_backward_reduced: null pointer");
        return B200_ERR_ARG;
    }
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.denom = static_cast<const double *>(denom);
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    prm.host_scale = grad_scale;
    prm.defer = defer & B200_STEP_DEFER;
    return dispatch_focal<kFwdBwd, true>(prm, dtype, static_cast<cudaStream_t>(stream));
}

// The same step for a 'mean' over a batch sharded across GPUs (workspace with an exchange
// attached).  The gradient is divided by *denom_state, the global element count the previous call
// found (initialise it with b200_exchange_count); after the cross-GPU sum the kernel stores
// predicted / actual count in *correction (1 while the shapes do not change; pass it to
// b200_rescale_gradient) and the actual count in *denom_state.
extern "C" int b200_focal_forward_backward_predicted(const void *logits, const void *labels, void *grad_logits,
                                                     void *out, void *workspace, size_t workspace_bytes,
                                                     void *denom_state, float *correction, int64_t E, int dtype,
                                                     float gamma, float alpha, int defer, void *stream) {
    if (E < 0 || !out || !denom_state || !correction) {
        set_error("b200_focal_forward_backward_predicted: need E >= 0, out, denom_state and correction");
        return B200_ERR_ARG;
    }
    if (!workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("b200_focal_forward_backward_predicted: workspace of %zu bytes required", kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    if (E > 0 && (!logits || !labels || !grad_logits)) {
        set_error("b200_focal_forward_backward_predicted: null pointer");
        return B200_ERR_ARG;
    }
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.denom = static_cast<const double *>(denom_state);
    prm.denom_state = static_cast<double *>(denom_state);
    prm.correction = correction;
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    prm.defer = defer & B200_STEP_DEFER;
    return dispatch_focal<kFwdBwd, true>(prm, dtype, static_cast<cudaStream_t>(stream));
}

namespace b200 {
namespace {
// grad *= *g unless *g == 1 (the usual upstream gradient of a scalar loss): then every block
// leaves at once and the stored gradient is already the answer.
constexpr int kRescaleThreads = 1024;
// With `workspace`: a loss sum of this stream may be posted to the other GPUs but not collected
// yet (grid_reduce_finish<defer>).  Warp 0 of block 0 collects it and completes the record `out`
// (and, for the focal step that divided by a predicted count, the correction and the count for
// the next call) before anything else; blocks that need the correction wait for that (bounded).
// E == 0: only that.
template <typename T>
__global__ void __launch_bounds__(kRescaleThreads) rescale_kernel(T *grad, const float *g, float *corr, int64_t E,
                                                                  void *workspace, ReduceRecord *out,
                                                                  double *denom_state) {
    if (workspace) {
        volatile float *done = &out->pad[0];
        if (blockIdx.x == 0 && threadIdx.x < 32) {
            if (exchange_finish_pending(workspace, out)) publish_denominator(denom_state, corr, out);
            if (threadIdx.x == 0) {
                __threadfence();
                *done = 1.f;
            }
        }
        if (corr && E > 0) {
            if (threadIdx.x == 0) {                      // one poller per block
                const ExchangeCtx *ex = exchange_of(workspace);
                const unsigned limit = ex ? ex->poll_limit : (1u << 20);
                unsigned polls = 0;
                while (*done != 1.f) {
                    if (++polls > limit) {
                        atomicOr(reinterpret_cast<unsigned *>(workspace) + 1, 0x100u);
                        break;
                    }
                    __nanosleep(32);
                }
                __threadfence();
            }
            __syncthreads();
        }
    }
    if (E == 0) return;
    const float f = corr ? *g * *static_cast<volatile float *>(corr) : *g;
    if (f == 1.f) return;
    constexpr int V = 16 / int(sizeof(T));                 // elements per 16-byte access
    const bool aligned = (reinterpret_cast<uintptr_t>(grad) & 15) == 0;
    const int64_t nvec = aligned ? E / V : 0;
    const int64_t stride = int64_t(gridDim.x) * kRescaleThreads;
    int64_t i = int64_t(blockIdx.x) * kRescaleThreads + threadIdx.x;
    uint4 *g4 = reinterpret_cast<uint4 *>(grad);
    for (; i + 3 * stride < nvec; i += 4 * stride) {        // four independent accesses in flight
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = g4[i + u * stride];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            T *e = reinterpret_cast<T *>(&v[u]);
#pragma unroll
            for (int k = 0; k < V; ++k) e[k] = from_f32<T>(to_f32(e[k]) * f);
            g4[i + u * stride] = v[u];
        }
    }
    for (; i < nvec; i += stride) {
        uint4 v = g4[i];
        T *e = reinterpret_cast<T *>(&v);
#pragma unroll
        for (int k = 0; k < V; ++k) e[k] = from_f32<T>(to_f32(e[k]) * f);
        g4[i] = v;
    }
    for (int64_t j = nvec * V + int64_t(blockIdx.x) * kRescaleThreads + threadIdx.x; j < E; j += stride)
        grad[j] = from_f32<T>(to_f32(grad[j]) * f);
}
__global__ void count_exchange_kernel(double count, void *workspace, ReduceRecord *out) {
    __shared__ double sh[64];
    grid_reduce_finish(0.0, threadIdx.x == 0 ? count : 0.0, workspace, out, sh, kTagCount);
}
}  // namespace
}  // namespace b200

namespace {
int launch_rescale(void *grad, const float *grad_out, float *correction, int64_t E, int dtype, void *workspace,
                   void *out, void *denom_state, void *stream) {
    // one block of 1024 threads per SM at most: the usual call (upstream gradient 1) only has to
    // start and leave, and 148 x 1024 threads x 4 vectors in flight still cover the memory latency
    int64_t grid = (E + kRescaleThreads * 16 - 1) / (kRescaleThreads * 16);
    const int64_t cap = int64_t(sm_count());
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ReduceRecord *rec = static_cast<ReduceRecord *>(out);
    double *ds = static_cast<double *>(denom_state);
    if (dtype == B200_F32)
        rescale_kernel<float><<<unsigned(grid), E > 0 ? kRescaleThreads : 32, 0, s>>>(static_cast<float *>(grad), grad_out,
                                                                                     correction, E, workspace, rec, ds);
    else if (dtype == B200_F16)
        rescale_kernel<__half><<<unsigned(grid), kRescaleThreads, 0, s>>>(static_cast<__half *>(grad), grad_out,
                                                                          correction, E, workspace, rec, ds);
    else if (dtype == B200_BF16)
        rescale_kernel<__nv_bfloat16><<<unsigned(grid), kRescaleThreads, 0, s>>>(
            static_cast<__nv_bfloat16 *>(grad), grad_out, correction, E, workspace, rec, ds);
    else {
        set_error("rescale: unknown dtype code %d", dtype);
        return B200_ERR_ARG;
    }
    return launch_status("gradient rescale kernel launch");
}
}  // namespace

// In place: grad[i] *= *grad_out * *correction (floats in device memory; correction may be
// null = 1); a no-op kernel when the product is 1.
extern "C" int b200_rescale_gradient(void *grad, const float *grad_out, const float *correction, int64_t E,
                                     int dtype, void *stream) {
    if (E < 0 || (E > 0 && (!grad || !grad_out))) {
        set_error("b200_rescale_gradient: bad arguments");
        return B200_ERR_ARG;
    }
    if (E == 0) return B200_OK;
    return launch_rescale(grad, grad_out, const_cast<float *>(correction), E, dtype, nullptr, nullptr, nullptr, stream);
}

// The same, after completing a reduction record whose cross-GPU sum was deferred (`defer` of the
// fused steps): the kernel first collects the ranks' sums into `out` (and writes `correction` and
// `denom_state` for the focal step with a predicted count; both may be null otherwise).
extern "C" int b200_rescale_gradient_finish(void *grad, const float *grad_out, float *correction, int64_t E, int dtype,
                                            void *workspace, void *out, void *denom_state, void *stream) {
    if (E < 0 || (E > 0 && (!grad || !grad_out)) || !workspace || !out) {
        set_error("b200_rescale_gradient_finish: bad arguments");
        return B200_ERR_ARG;
    }
    return launch_rescale(grad, grad_out, correction, E, dtype, workspace, out, denom_state, stream);
}

// Completes a deferred record without a gradient to rescale (a loss that is read before, or
// without, backward).  Does nothing when the record is complete already.
extern "C" int b200_exchange_finish(void *workspace, void *out, void *denom_state, float *correction, void *stream) {
    if (!workspace || !out) {
        set_error("b200_exchange_finish: workspace and out are required");
        return B200_ERR_ARG;
    }
    return launch_rescale(nullptr, nullptr, correction, 0, B200_F32, workspace, out, denom_state, stream);
}

// out->count = `count` added over the ranks attached to `workspace` (out->sum = 0): the global
// divisor of a sharded batch, known before the fused step writes its gradients.
extern "C" int b200_exchange_count(double count, void *out, void *workspace, size_t workspace_bytes, void *stream) {
    if (!out || !workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("b200_exchange_count: out and a reduction workspace are required");
        return B200_ERR_ARG;
    }
    count_exchange_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(count, workspace,
                                                                          static_cast<ReduceRecord *>(out));
    return launch_status("count exchange kernel launch");
}

// ------------------------------------------------- focal forward without any allocation
//
// Some users of this library cannot hand it a workspace: a host that gave all device
// memory to its own pool at start-up (a later cudaMalloc would fail or stall the device), or
// a plain-FFI caller that has no allocator of its own and must not trigger one inside a
// latency-critical loop.  For them the reducing focal forward also exists with its scratch
// (ticket, status word, one partial per block) in a fixed array that lives in the library's
// device image: kFocalNoAllocScratchBytes bytes on every GPU that loads the library, for
// the life of the process.
//
// The array's name is only a host-side handle; the device address is looked up once per
// device with cudaGetSymbolAddress while that device is current, and that address is what
// the kernel receives.  All calls on a device share the array: calls that overlap on the
// GPU (two streams, two threads) race on it and must be serialised by the caller.
static __device__ __align__(256) unsigned char b200_focal_noalloc_scratch[b200::kPartialsOffset + 1024 * 16];

namespace b200 {
namespace {

constexpr int kFocalNoAllocMaxBlocks = 1024;
static_assert(sizeof(b200_focal_noalloc_scratch) == kPartialsOffset + size_t(kFocalNoAllocMaxBlocks) * 16,
              "the scratch array holds the header and one partial per block");
constexpr int64_t kFocalNoAllocMaxElems = int64_t(1) << 28;
constexpr int kMaxDevices = 64;

// Device address of the scratch array on the current device (set up on first use).
int focal_noalloc_scratch(void **out) {
    static void *ptrs[kMaxDevices] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("b200_focal_forward_noalloc: cannot identify the current device");
        return B200_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, b200_focal_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            set_error("b200_focal_forward_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return B200_ERR_LAUNCH;
        }
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return B200_OK;
}

template <typename T>
int launch_focal_noalloc(const FocalParams &prm, cudaStream_t stream) {
    const int vn = Vec16<T>::N;
    int64_t want = (prm.E / vn + kThreads - 1) / kThreads;
    int64_t cap = int64_t(sm_count()) * kBlocksPerSM;
    if (cap > kFocalNoAllocMaxBlocks) cap = kFocalNoAllocMaxBlocks;   // one partial slot per block
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    const dim3 grid(static_cast<unsigned>(want));
    const bool al = aligned16(prm.logits) && aligned16(prm.labels) && (!prm.losses || aligned16(prm.losses));
    if (!al) {
        focal_kernel_unaligned<T, kFwd, true><<<grid, kThreads, 0, stream>>>(prm);
    } else if (prm.gamma == 2.f) {
        focal_kernel<T, kFwd, true, true><<<grid, kThreads, 0, stream>>>(prm);
    } else {
        focal_kernel<T, kFwd, false, true><<<grid, kThreads, 0, stream>>>(prm);
    }
    return launch_status("focal no-alloc kernel launch");
}

}  // namespace
}  // namespace b200

extern "C" int b200_focal_forward_noalloc(const void *logits, const void *labels, void *losses,
                                          void *out, int64_t E, int dtype, float gamma, float alpha,
                                          void *stream) {
    if (E < 0 || !out) {
        set_error("b200_focal_forward_noalloc: need E >= 0 and an output record");
        return B200_ERR_ARG;
    }
    if (E > kFocalNoAllocMaxElems) {
        set_error("b200_focal_forward_noalloc: E=%lld exceeds the maximum of %lld elements of this entry point; "
                  "use b200_focal_forward with a caller-provided workspace",
                  (long long)E, (long long)kFocalNoAllocMaxElems);
        return B200_ERR_UNSUPPORTED;
    }
    if (E > 0 && (!logits || !labels)) {
        set_error("b200_focal_forward_noalloc: null input pointer");
        return B200_ERR_ARG;
    }
    if (!dtype_known(dtype)) {
        set_error("b200_focal_forward_noalloc: unknown dtype code %d", dtype);
        return B200_ERR_ARG;
    }
    void *scratch = nullptr;
    const int rc = focal_noalloc_scratch(&scratch);
    if (rc != B200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps whatever the previous call left: re-arm ticket and status word
    if (cudaMemsetAsync(scratch, 0, kPartialsOffset, s) != cudaSuccess)
        return launch_status("b200_focal_forward_noalloc: clearing the scratch header");
    FocalParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.losses = losses;
    prm.workspace = scratch;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.E = E;
    prm.gamma = gamma;
    prm.alpha = alpha;
    if (dtype == B200_BF16) return launch_focal_noalloc<__nv_bfloat16>(prm, s);
    return dtype == B200_F32 ? launch_focal_noalloc<float>(prm, s) : launch_focal_noalloc<__half>(prm, s);
}
