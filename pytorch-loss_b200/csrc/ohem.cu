// Online hard example mining by score: which pixels keep their label (sm_100a).
//
// What is computed (reference csrc/ohem_label_kernel.cu:53-176, host side :179-262, called from
// pytorch_loss/ohem_loss.py:22-27,41-46):
//   score_i = softmax(x_i)[label_i]            (ignored pixels: 1)
//   sort the scores ascending; every pixel at sorted position >= n_min whose score exceeds
//   score_thresh gets the ignore label; n_min >= number of pixels returns the labels unchanged.
// In other words the n_min hardest pixels always stay, and so does every pixel whose score
// is at most the threshold.  With t = the n_min-th smallest score this is
//   out_i = (score_i > max(score_thresh, t)) ? ignore : label_i
// so no sort is needed, only a selection.  Pixels whose score EQUALS t all stay here; the
// reference keeps whichever of them its (unstable) sort happens to place first.
//
// How:
//   score    one pass over the logits: online softmax per pixel (4 adjacent pixels per thread
//            from 16-byte loads when the layout allows), score out, and a histogram of the
//            score's bits 20..30 (non-negative floats order like their bit patterns)
//   select   radix select of the n_min-th smallest score, 11 + 11 + 9 bits: two more
//            histogram passes over the scores (only those that match the prefix found so far
//            count).  The block that finishes a histogram last picks the digit, so a pass is
//            one launch and nothing waits.
//   relabel  one pass over labels and scores.
#include "common.cuh"

#include <cfloat>
#include <cstring>

namespace b200 {
namespace {

constexpr int kOhemThreads = 256;
constexpr int kBinsPerPass = 2048;
constexpr float kOhemLog2e = 1.4426950408889634f;

// Device-side state of one call, at the start of the workspace (256 bytes, zeroed per call).
struct OhemState {
    unsigned ticket[3];   // one per histogram pass
    uint32_t prefix;      // bits of the selected value found so far
    uint32_t k_rem;       // 1-based rank still to find inside the current prefix
    uint32_t t_bits;      // the n_min-th smallest score (after the last pass)
    uint32_t done;        // set once t is known well enough: the remaining passes return at once
};

struct OhemWorkspace {
    OhemState *state;
    uint32_t *hist;       // [3][kBinsPerPass]
    float *scores;        // [P]
    size_t bytes;
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

OhemWorkspace carve(void *base, int64_t P) {
    OhemWorkspace w{};
    char *p = static_cast<char *>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *r = p ? p + off : nullptr;
        off += align256(bytes);
        return r;
    };
    w.state = reinterpret_cast<OhemState *>(take(256));
    w.hist = reinterpret_cast<uint32_t *>(take(size_t(3) * kBinsPerPass * 4));
    w.scores = reinterpret_cast<float *>(take(size_t(P) * 4));
    w.bytes = off;
    return w;
}

// Shared-memory histogram of a block: a warp whose lanes all hit one bin adds once.
__device__ __forceinline__ void hist_add(uint32_t *sh, uint32_t bin, bool active) {
    const uint32_t mask = __ballot_sync(0xffffffffu, active);
    if (mask == 0u) return;
    const int leader = __ffs(mask) - 1;
    const uint32_t b0 = __shfl_sync(0xffffffffu, bin, leader);
    if (__all_sync(0xffffffffu, !active || bin == b0)) {
        if ((threadIdx.x & 31) == leader) atomicAdd(&sh[b0], uint32_t(__popc(mask)));
    } else if (active) {
        atomicAdd(&sh[bin], 1u);
    }
}

// End of a histogram pass.  Every block adds its shared-memory histogram to the global one
// and takes a ticket; the block with the last ticket finds the bin that holds rank k_rem
// and extends the prefix.  `shift`: position of this pass's digit; last pass: shift == 0.
// thresh_bits: bits of score_thresh.  When the digits found so far already place t below the
// threshold's own prefix, t < score_thresh, the cut is the threshold, and the finer passes are
// not needed (the usual case early in training, when most pixels are still hard).
__device__ __forceinline__ void finish_pass(uint32_t *sh, uint32_t *__restrict__ ghist, OhemState *st, int pass,
                                            int shift, uint32_t k_first, uint32_t thresh_bits) {
    __shared__ unsigned s_last;
    __shared__ uint32_t s_scan[kOhemThreads / 32];
    __syncthreads();
    for (int b = threadIdx.x; b < kBinsPerPass; b += kOhemThreads)
        if (sh[b]) atomicAdd(&ghist[b], sh[b]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&st->ticket[pass], 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // inclusive scan of the 2048 bins, 8 consecutive bins per thread
    constexpr int BPT = kBinsPerPass / kOhemThreads;
    uint32_t c[BPT], mine = 0;
#pragma unroll
    for (int q = 0; q < BPT; ++q) {
        c[q] = __ldcg(&ghist[threadIdx.x * BPT + q]);
        mine += c[q];
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    uint32_t before = incl - mine;
    for (int w = 0; w < warp; ++w) before += s_scan[w];
    const uint32_t k = pass == 0 ? k_first : *reinterpret_cast<volatile uint32_t *>(&st->k_rem);
    // the thread whose 8 bins straddle rank k (k is 1-based; the total is >= k by construction)
    if (before < k && k <= before + mine) {
        uint32_t run = before;
        int q = 0;
        for (; q < BPT - 1; ++q) {
            if (k <= run + c[q]) break;
            run += c[q];
        }
        const uint32_t bin = uint32_t(threadIdx.x * BPT + q);
        const uint32_t prefix = (pass == 0 ? 0u : st->prefix) | (bin << shift);
        st->prefix = prefix;
        st->k_rem = k - run;
        if (shift == 0) st->t_bits = prefix;
        else if ((prefix >> shift) < (thresh_bits >> shift)) {
            st->t_bits = prefix;          // a lower bound of t, itself below the threshold
            st->done = 1u;
        }
    }
}

// Online softmax of VEC adjacent pixels; the label channel's logit is picked up on the way.
template <typename T, int VEC>
__global__ void __launch_bounds__(kOhemThreads, 3)
ohem_score_kernel(const T *__restrict__ logits, const int64_t *__restrict__ labels, float *__restrict__ scores,
                  uint32_t *__restrict__ ghist, OhemState *st, int64_t N, int C, int64_t M, int64_t ignore,
                  uint32_t k_first, uint32_t thresh_bits) {
    __shared__ uint32_t sh[kBinsPerPass];
    for (int b = threadIdx.x; b < kBinsPerPass; b += kOhemThreads) sh[b] = 0u;
    __syncthreads();
    const int64_t groups_per_image = M / VEC;               // VEC > 1 only when M % VEC == 0
    const int64_t groups = N * groups_per_image;
    const int64_t stride = int64_t(gridDim.x) * kOhemThreads;
    // every lane of a warp runs the same number of iterations (the histogram votes are warp-wide)
    const int64_t rounds = (groups + stride - 1) / stride;
    for (int64_t it = 0; it < rounds; ++it) {
        const int64_t gidx = it * stride + int64_t(blockIdx.x) * kOhemThreads + threadIdx.x;
        const bool live = gidx < groups;
        float sc[VEC];
        if (live) {
            const int64_t n = gidx / groups_per_image, m0 = (gidx % groups_per_image) * VEC;
            int lb[VEC];                    // -1: ignored, -2: outside [0, C) (scores 0: counts as hard)
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const int64_t l = __ldg(labels + n * M + m0 + v);
                lb[v] = l == ignore ? -1 : ((l >= 0 && l < C) ? int(l) : -2);
            }
            float mx[VEC], sum[VEC], xl[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                mx[v] = -FLT_MAX;
                sum[v] = 0.f;
                xl[v] = -FLT_MAX;
            }
            const T *col = logits + n * C * M + m0;
            // channels in chunks of kChunk: the running maximum moves once per chunk, so an element
            // costs one exponential plus 1/kChunk of the rescaling one
            constexpr int kChunk = 8;
            for (int j0 = 0; j0 < C; j0 += kChunk) {
                float x[kChunk][VEC];
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    const int j = j0 + q;
                    if (j < C) {
                        if constexpr (VEC == 4 && sizeof(T) == 4) {
                            const float4 f = __ldcs(reinterpret_cast<const float4 *>(col + int64_t(j) * M));
                            x[q][0] = f.x; x[q][1] = f.y; x[q][2] = f.z; x[q][3] = f.w;
                        } else {
#pragma unroll
                            for (int v = 0; v < VEC; ++v) x[q][v] = to_f32(col[int64_t(j) * M + v]);
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < VEC; ++v) x[q][v] = -FLT_MAX;
                    }
                }
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float mn = mx[v];
#pragma unroll
                    for (int q = 0; q < kChunk; ++q) mn = fmaxf(mn, x[q][v]);
                    float acc = sum[v] * exp2f((mx[v] - mn) * kOhemLog2e);
                    const float off = -mn * kOhemLog2e;
#pragma unroll
                    for (int q = 0; q < kChunk; ++q) {
                        // (padding channels hold -FLT_MAX: their term underflows to 0)
                        acc += exp2f(fmaf(x[q][v], kOhemLog2e, off));
                        if (lb[v] == j0 + q) xl[v] = x[q][v];
                    }
                    sum[v] = acc;
                    mx[v] = mn;
                }
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v)
                sc[v] = lb[v] == -1 ? 1.f : __fdividef(exp2f((xl[v] - mx[v]) * kOhemLog2e), sum[v]);
            if constexpr (VEC == 4) {
                *reinterpret_cast<float4 *>(scores + n * M + m0) = make_float4(sc[0], sc[1], sc[2], sc[3]);
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) scores[n * M + m0 + v] = sc[v];
            }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const uint32_t bin = min(__float_as_uint(live ? sc[v] : 0.f) >> 20, uint32_t(kBinsPerPass - 1));
            hist_add(sh, bin, live);
        }
    }
    finish_pass(sh, ghist, st, 0, 20, k_first, thresh_bits);
}

// Histogram of the next digit over the scores that match the prefix found so far.
__global__ void __launch_bounds__(kOhemThreads)
ohem_hist_kernel(const float *__restrict__ scores, uint32_t *__restrict__ ghist, OhemState *st, int64_t P, int pass,
                 int match_shift, int shift, uint32_t mask, uint32_t thresh_bits) {
    __shared__ uint32_t sh[kBinsPerPass];
    if (*reinterpret_cast<volatile uint32_t *>(&st->done)) return;
    for (int b = threadIdx.x; b < kBinsPerPass; b += kOhemThreads) sh[b] = 0u;
    __syncthreads();
    const uint32_t want = st->prefix >> match_shift;
    // 4 x 4 scores per thread and round: the four 16-byte loads (the workspace is 256-byte aligned)
    // are all in flight before the first warp vote
    constexpr int kQ = 4;
    const int64_t quads = (P + 3) / 4;
    const int64_t stride = int64_t(gridDim.x) * kOhemThreads;
    const int64_t rounds = (quads + stride * kQ - 1) / (stride * kQ);
    for (int64_t it = 0; it < rounds; ++it) {
        uint32_t bits[kQ][4];
#pragma unroll
        for (int u = 0; u < kQ; ++u) {
            const int64_t q = (it * kQ + u) * stride + int64_t(blockIdx.x) * kOhemThreads + threadIdx.x;
            bits[u][0] = bits[u][1] = bits[u][2] = bits[u][3] = 0xFFFFFFFFu;
            if (q * 4 + 3 < P) {
                const uint4 w4 = __ldg(reinterpret_cast<const uint4 *>(scores) + q);
                bits[u][0] = w4.x; bits[u][1] = w4.y; bits[u][2] = w4.z; bits[u][3] = w4.w;
            } else {
                for (int v = 0; v < 4; ++v)
                    if (q * 4 + v < P) bits[u][v] = __float_as_uint(__ldg(scores + q * 4 + v));
            }
        }
#pragma unroll
        for (int u = 0; u < kQ; ++u) {
            const int64_t q = (it * kQ + u) * stride + int64_t(blockIdx.x) * kOhemThreads + threadIdx.x;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const bool hit = q * 4 + v < P && (bits[u][v] >> match_shift) == want;
                if (__any_sync(0xffffffffu, hit)) hist_add(sh, (bits[u][v] >> shift) & mask, hit);
            }
        }
    }
    finish_pass(sh, ghist, st, pass, shift, 0u, thresh_bits);
}

__global__ void __launch_bounds__(kOhemThreads)
ohem_relabel_kernel(const int64_t *__restrict__ labels, const float *__restrict__ scores,
                    int64_t *__restrict__ out, const OhemState *__restrict__ st, int64_t P, int64_t ignore,
                    float thresh, int use_select) {
    float cut = thresh;
    if (use_select) cut = fmaxf(thresh, __uint_as_float(st->t_bits));
    const int64_t stride = int64_t(gridDim.x) * kOhemThreads;
    for (int64_t i = int64_t(blockIdx.x) * kOhemThreads + threadIdx.x; i < P; i += stride) {
        const int64_t lb = __ldg(labels + i);
        out[i] = __ldg(scores + i) > cut ? ignore : lb;
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200_ohem_workspace_bytes(int64_t N, int64_t M) {
    if (N <= 0 || M <= 0) return 256;
    return carve(nullptr, N * M).bytes;
}

extern "C" int b200_ohem_label(const void *logits, const int64_t *labels, int64_t *out_labels, void *workspace,
                               size_t workspace_bytes, int64_t N, int64_t C, int64_t M, int dtype,
                               int64_t ignore_index, float score_thresh, int64_t n_min, void *stream) {
    if (N < 0 || C < 1 || M < 0 || C >= (int64_t(1) << 31)) {
        set_error("b200_ohem_label: bad shape N=%lld C=%lld M=%lld", (long long)N, (long long)C, (long long)M);
        return B200_ERR_ARG;
    }
    if (!dtype_known(dtype)) {
        set_error("b200_ohem_label: unknown dtype code %d", dtype);
        return B200_ERR_ARG;
    }
    const int64_t P = N * M;
    if (P == 0) return B200_OK;
    if (P >= (int64_t(1) << 32)) {
        set_error("b200_ohem_label: more than 2^32 pixels");
        return B200_ERR_UNSUPPORTED;
    }
    if (!logits || !labels || !out_labels || !workspace) {
        set_error("b200_ohem_label: null pointer");
        return B200_ERR_ARG;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // reference :193: nothing can be dropped
    if (n_min >= P) {
        if (out_labels != labels &&
            cudaMemcpyAsync(out_labels, labels, size_t(P) * 8, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            return launch_status("ohem label copy");
        return B200_OK;
    }
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) {
        set_error("b200_ohem_label: workspace must be 256-byte aligned");
        return B200_ERR_ARG;
    }
    OhemWorkspace w = carve(workspace, P);
    if (workspace_bytes < w.bytes) {
        set_error("b200_ohem_label: workspace of %zu bytes required, got %zu", w.bytes, workspace_bytes);
        return B200_ERR_WORKSPACE;
    }
    if (cudaMemsetAsync(w.state, 0, reinterpret_cast<char *>(w.scores) - reinterpret_cast<char *>(w.state), s) !=
        cudaSuccess)
        return launch_status("ohem workspace memset");
    const int use_select = n_min > 0 ? 1 : 0;      // n_min <= 0: the threshold alone decides
    const uint32_t k_first = use_select ? uint32_t(n_min) : 1u;
    // bits of the threshold as the kernels compare them (negative or NaN thresholds: no shortcut)
    uint32_t thresh_bits = 0u;
    if (score_thresh > 0.f) std::memcpy(&thresh_bits, &score_thresh, 4);
    int rc;
    const bool vec4 = dtype == B200_F32 && M % 4 == 0 && aligned16(logits);
    const int64_t groups = vec4 ? P / 4 : P;
    int64_t grid = (groups + kOhemThreads - 1) / kOhemThreads;
    const int64_t cap = int64_t(sm_count()) * 8;
    if (grid > cap) grid = cap;
    const int Ci = int(C);
    if (vec4)
        ohem_score_kernel<float, 4><<<unsigned(grid), kOhemThreads, 0, s>>>(
            static_cast<const float *>(logits), labels, w.scores, w.hist, w.state, N, Ci, M, ignore_index, k_first, thresh_bits);
    else if (dtype == B200_F32)
        ohem_score_kernel<float, 1><<<unsigned(grid), kOhemThreads, 0, s>>>(
            static_cast<const float *>(logits), labels, w.scores, w.hist, w.state, N, Ci, M, ignore_index, k_first, thresh_bits);
    else if (dtype == B200_F16)
        ohem_score_kernel<__half, 1><<<unsigned(grid), kOhemThreads, 0, s>>>(
            static_cast<const __half *>(logits), labels, w.scores, w.hist, w.state, N, Ci, M, ignore_index, k_first, thresh_bits);
    else
        ohem_score_kernel<__nv_bfloat16, 1><<<unsigned(grid), kOhemThreads, 0, s>>>(
            static_cast<const __nv_bfloat16 *>(logits), labels, w.scores, w.hist, w.state, N, Ci, M, ignore_index, k_first, thresh_bits);
    if ((rc = launch_status("ohem score kernel launch")) != B200_OK) return rc;
    int64_t pgrid = (P + kOhemThreads - 1) / kOhemThreads;
    if (pgrid > cap) pgrid = cap;
    if (use_select) {
        // the select passes read 4 bytes per pixel: two blocks per SM (every block pays for a
        // histogram flush and a ticket), 64 bytes per thread in flight
        int64_t hgrid = (P / 4 + kOhemThreads - 1) / kOhemThreads;
        if (hgrid > int64_t(sm_count()) * 2) hgrid = int64_t(sm_count()) * 2;
        if (hgrid < 1) hgrid = 1;
        ohem_hist_kernel<<<unsigned(hgrid), kOhemThreads, 0, s>>>(w.scores, w.hist + kBinsPerPass, w.state, P, 1, 20, 9,
                                                                  0x7FFu, thresh_bits);
        if ((rc = launch_status("ohem select pass 2 launch")) != B200_OK) return rc;
        ohem_hist_kernel<<<unsigned(hgrid), kOhemThreads, 0, s>>>(w.scores, w.hist + 2 * kBinsPerPass, w.state, P, 2, 9,
                                                                  0, 0x1FFu, thresh_bits);
        if ((rc = launch_status("ohem select pass 3 launch")) != B200_OK) return rc;
    }
    ohem_relabel_kernel<<<unsigned(pgrid), kOhemThreads, 0, s>>>(labels, w.scores, out_labels, w.state, P, ignore_index,
                                                                 score_thresh, use_select);
    return launch_status("ohem relabel kernel launch");
}
