// Proportion-corrected softmax cross entropy (PC softmax, arXiv 1911.10688) for sm_100a.
//
// What is computed (reference pc_softmax.py:35-49 forward, :52-97 the same as a Function): with
// class proportions W_j,
//   loss  = -(x_lb - m - log sum_j W_j e^{x_j - m}),   m = max_j x_j;   0 at ignored pixels
//   grad_j = W_j e^{x_j - m} / sum_k W_k e^{x_k - m} - 1[j == lb];      0 at ignored pixels
// The gradient is the derivative of that loss (what autograd gives for the reference's V1
// class).  The hand-written backward of the reference's V2 Function multiplies every channel
// by W_lb instead of W_j (pc_softmax.py:104-106), which is not the derivative of its own
// forward; that is not reproduced.
//
// How: one kernel, forward and gradient in one launch.  The logits are viewed as [N, C, M].
//   M > 1   a thread owns 4 adjacent pixels (16-byte accesses when M % 4 == 0 and the
//           pointers allow, else one pixel) and walks the channels twice: online maximum and
//           weighted sum first, gradients second (the second walk finds its lines in L1/L2).
//   M == 1  a warp owns a row: lanes stride over the channels, shuffles combine.
//   M > 1, at most 32 channels, float32, M even: a thread owns 2 adjacent pixels and keeps all
//           their channels in registers, so the logits cross HBM once (8-byte accesses).  (A
//           second 4-byte store for the label channel's "- 1" instead of a compare per channel
//           was tried: it costs partial-sector writes and measured slower.)
// Per-pixel losses and gradients leave in the logits' dtype.  The gradient is divided by
// *denom when one is given (a device double: the number of valid pixels for 'mean', counted
// beforehand), so that what leaves is final for an upstream gradient of 1; the sum over the
// per-pixel losses is the caller's.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kPcThreads = 256;

struct PcParams {
    const void *logits;
    const int64_t *labels;
    const float *weight;     // [C]
    void *losses;            // [N, M] or null
    void *grads;             // [N, C, M] or null
    int64_t N, C, M, ignore;
    const double *denom;     // gradient divisor in device memory, or null
};

__device__ __forceinline__ float exp2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ float grad_scale(const PcParams &p) {
    return p.denom ? float(1.0 / *p.denom) : 1.f;
}

template <typename T, int VEC> struct PcPack;
template <> struct PcPack<float, 4> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <typename T> struct PcPack<T, 1> {
    static __device__ __forceinline__ void load(const T *p, float (&v)[1]) { v[0] = to_f32(*p); }
    static __device__ __forceinline__ void store(T *p, const float (&v)[1]) { *p = from_f32<T>(v[0]); }
};

template <typename T, int VEC>
__global__ void __launch_bounds__(kPcThreads) pc_spatial_kernel(const PcParams p) {
    const T *x = static_cast<const T *>(p.logits);
    T *losses = static_cast<T *>(p.losses);
    T *grads = static_cast<T *>(p.grads);
    const int64_t groups_per_row = p.M / VEC;
    const int64_t groups = p.N * groups_per_row;
    const int64_t stride = int64_t(gridDim.x) * kPcThreads;
    const float gs = grad_scale(p);
    for (int64_t gi = int64_t(blockIdx.x) * kPcThreads + threadIdx.x; gi < groups; gi += stride) {
        const int64_t n = gi / groups_per_row, m0 = (gi % groups_per_row) * VEC;
        const int64_t base = n * p.C * p.M + m0;
        int64_t lb[VEC];
        float m[VEC], s[VEC], xl[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            lb[v] = p.labels[n * p.M + m0 + v];
            m[v] = -INFINITY;
            s[v] = 0.f;
            xl[v] = 0.f;
        }
#pragma unroll 4
        for (int64_t j = 0; j < p.C; ++j) {
            float xv[VEC];
            PcPack<T, VEC>::load(x + base + j * p.M, xv);
            const float w = __ldg(p.weight + j);
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float mn = fmaxf(m[v], xv[v]);
                s[v] = s[v] * __expf(m[v] - mn) + w * __expf(xv[v] - mn);
                m[v] = mn;
                if (j == lb[v]) xl[v] = xv[v];
            }
        }
        float inv[VEC];
        bool valid[VEC];
        float lv[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            valid[v] = lb[v] != p.ignore;
            inv[v] = valid[v] ? __fdividef(gs, s[v]) : 0.f;
            lv[v] = valid[v] ? (m[v] + __logf(s[v])) - xl[v] : 0.f;
        }
        if (losses) PcPack<T, VEC>::store(losses + n * p.M + m0, lv);
        if (!grads) continue;
#pragma unroll 4
        for (int64_t j = 0; j < p.C; ++j) {
            float xv[VEC], gv[VEC];
            PcPack<T, VEC>::load(x + base + j * p.M, xv);
            const float w = __ldg(p.weight + j);
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float g = w * __expf(xv[v] - m[v]) * inv[v];
                if (valid[v] && j == lb[v]) g -= gs;
                gv[v] = g;
            }
            PcPack<T, VEC>::store(grads + base + j * p.M, gv);
        }
    }
}

// M > 1, C <= CMAX, float32, M even, 8-byte aligned pointers, C * M < 2^31: all channels of a
// pixel pair in registers; channel offsets are 32-bit; the class weights wait in shared memory.
template <int CMAX>
__global__ void __launch_bounds__(kPcThreads, CMAX <= 20 ? 3 : 2) pc_resident_kernel(const PcParams p) {
    __shared__ float sw[CMAX];
    const float *x = static_cast<const float *>(p.logits);
    float *losses = static_cast<float *>(p.losses);
    float *grads = static_cast<float *>(p.grads);
    const int C = int(p.C);
    const int M = int(p.M);
    if (threadIdx.x < CMAX) sw[threadIdx.x] = threadIdx.x < C ? __ldg(p.weight + threadIdx.x) : 0.f;
    __syncthreads();
    const int64_t groups_per_row = p.M / 2;
    const int64_t groups = p.N * groups_per_row;
    const int64_t stride = int64_t(gridDim.x) * kPcThreads;
    const float gs = grad_scale(p);
    constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
    for (int64_t gi = int64_t(blockIdx.x) * kPcThreads + threadIdx.x; gi < groups; gi += stride) {
        const int64_t n = gi / groups_per_row, m0 = (gi % groups_per_row) * 2;
        const int64_t base = n * p.C * p.M + m0;
        const float *xb = x + base;
        float2 xv[CMAX];
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) xv[j] = __ldcs(reinterpret_cast<const float2 *>(xb + j * M));
        const longlong2 lb2 = __ldcs(reinterpret_cast<const longlong2 *>(p.labels + n * p.M + m0));
        const bool v0 = lb2.x != p.ignore, v1 = lb2.y != p.ignore;
        // (labels outside [0, C) that are not the ignore value are undefined in the reference too;
        // here no channel takes the target term)
        const int l0 = v0 ? int(lb2.x) : -1, l1 = v1 ? int(lb2.y) : -1;
        float2 mx = make_float2(-INFINITY, -INFINITY);
        float xl0 = 0.f, xl1 = 0.f;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) {
                mx.x = fmaxf(mx.x, xv[j].x);
                mx.y = fmaxf(mx.y, xv[j].y);
                if (j == l0) xl0 = xv[j].x;
                if (j == l1) xl1 = xv[j].y;
            }
        const float2 nm2 = make_float2(-mx.x * kLog2e, -mx.y * kLog2e);
        float2 s = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) {
                const float w = sw[j];
                xv[j].x = w * exp2_approx(fmaf(xv[j].x, kLog2e, nm2.x));     // the weighted exponential takes x's place
                xv[j].y = w * exp2_approx(fmaf(xv[j].y, kLog2e, nm2.y));
                s.x += xv[j].x;
                s.y += xv[j].y;
            }
        if (losses) {
            float2 l;
            l.x = v0 ? fmaf(__log2f(s.x), kLn2, mx.x) - xl0 : 0.f;
            l.y = v1 ? fmaf(__log2f(s.y), kLn2, mx.y) - xl1 : 0.f;
            __stcs(reinterpret_cast<float2 *>(losses + n * p.M + m0), l);
        }
        if (!grads) continue;
        const float2 inv = make_float2(v0 ? __fdividef(gs, s.x) : 0.f, v1 ? __fdividef(gs, s.y) : 0.f);
        float *gb = grads + base;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) {
                float2 g = make_float2(xv[j].x * inv.x, xv[j].y * inv.y);
                if (j == l0) g.x -= gs;
                if (j == l1) g.y -= gs;
                __stcs(reinterpret_cast<float2 *>(gb + j * M), g);
            }
    }
}

// M == 1: one warp per row.
template <typename T>
__global__ void __launch_bounds__(kPcThreads) pc_rows_kernel(const PcParams p) {
    const T *x = static_cast<const T *>(p.logits);
    T *losses = static_cast<T *>(p.losses);
    T *grads = static_cast<T *>(p.grads);
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (kPcThreads / 32);
    const float gs = grad_scale(p);
    for (int64_t r = int64_t(blockIdx.x) * (kPcThreads / 32) + (threadIdx.x >> 5); r < p.N; r += warps) {
        const T *row = x + r * p.C;
        const int64_t lb = p.labels[r];
        float m = -INFINITY, s = 0.f;
        for (int64_t j = lane; j < p.C; j += 32) {
            const float xv = to_f32(row[j]);
            const float mn = fmaxf(m, xv);
            s = s * __expf(m - mn) + __ldg(p.weight + j) * __expf(xv - mn);
            m = mn;
        }
        const float mw = warp_max(m);
        s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - mw));
        const bool valid = lb != p.ignore;
        const float inv = valid ? __fdividef(gs, s) : 0.f;
        if (lane == 0 && losses) {
            const float xl = (valid && lb >= 0 && lb < p.C) ? to_f32(row[lb]) : 0.f;
            losses[r] = from_f32<T>(valid ? (mw + __logf(s)) - xl : 0.f);
        }
        if (!grads) continue;
        T *grow = grads + r * p.C;
        for (int64_t j = lane; j < p.C; j += 32) {
            float g = __ldg(p.weight + j) * __expf(to_f32(row[j]) - mw) * inv;
            if (valid && j == lb) g -= gs;
            grow[j] = from_f32<T>(g);
        }
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
int launch_pc(const PcParams &p, cudaStream_t stream) {
    const int sms = sm_count();
    if (p.M == 1) {
        int64_t grid = (p.N + (kPcThreads / 32) - 1) / (kPcThreads / 32);
        if (grid > int64_t(sms) * 8) grid = int64_t(sms) * 8;
        pc_rows_kernel<T><<<unsigned(grid), kPcThreads, 0, stream>>>(p);
        return launch_status("pc softmax rows kernel launch");
    }
    if constexpr (sizeof(T) == 4) {
        auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7u) == 0; };
        if (p.M % 2 == 0 && p.C <= 32 && p.C * p.M < (int64_t(1) << 31) && al8(p.logits) && (!p.grads || al8(p.grads)) && (!p.losses || al8(p.losses)) &&
            aligned16(p.labels)) {
            const int64_t groups2 = p.N * (p.M / 2);
            int64_t grid2 = (groups2 + kPcThreads - 1) / kPcThreads;
            if (grid2 > int64_t(sms) * 16) grid2 = int64_t(sms) * 16;     // (2 blocks per SM and 4 x SMs blocks measured 50 % slower)
            if (p.C <= 8) pc_resident_kernel<8><<<unsigned(grid2), kPcThreads, 0, stream>>>(p);
            else if (p.C <= 20) pc_resident_kernel<20><<<unsigned(grid2), kPcThreads, 0, stream>>>(p);
            else pc_resident_kernel<32><<<unsigned(grid2), kPcThreads, 0, stream>>>(p);
            return launch_status("pc softmax resident kernel launch");
        }
    }
    const bool vec = sizeof(T) == 4 && p.M % 4 == 0 && aligned16(p.logits) && (!p.grads || aligned16(p.grads)) &&
                     (!p.losses || aligned16(p.losses));
    const int64_t groups = p.N * (vec ? p.M / 4 : p.M);
    int64_t grid = (groups + kPcThreads - 1) / kPcThreads;
    if (grid > int64_t(sms) * 8) grid = int64_t(sms) * 8;
    if (grid < 1) grid = 1;
    if constexpr (sizeof(T) == 4) {
        if (vec) {
            pc_spatial_kernel<T, 4><<<unsigned(grid), kPcThreads, 0, stream>>>(p);
            return launch_status("pc softmax kernel launch");
        }
    }
    pc_spatial_kernel<T, 1><<<unsigned(grid), kPcThreads, 0, stream>>>(p);
    return launch_status("pc softmax kernel launch");
}

}  // namespace
}  // namespace b200

using namespace b200;

namespace {
int pc_entry(const void *logits, const int64_t *labels, const float *weight, void *losses, void *grad_logits,
             const void *denom, int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index, void *stream);
}

extern "C" int b200_pc_softmax_ce(const void *logits, const int64_t *labels, const float *weight, void *losses,
                                  void *grad_logits, int64_t N, int64_t C, int64_t M, int dtype,
                                  int64_t ignore_index, void *stream) {
    return pc_entry(logits, labels, weight, losses, grad_logits, nullptr, N, C, M, dtype, ignore_index, stream);
}

// The same with the gradient divided by *denom (device double, e.g. the count of b200_count_valid).
extern "C" int b200_pc_softmax_ce_scaled(const void *logits, const int64_t *labels, const float *weight, void *losses,
                                         void *grad_logits, const void *denom, int64_t N, int64_t C, int64_t M,
                                         int dtype, int64_t ignore_index, void *stream) {
    return pc_entry(logits, labels, weight, losses, grad_logits, denom, N, C, M, dtype, ignore_index, stream);
}

namespace {
int pc_entry(const void *logits, const int64_t *labels, const float *weight, void *losses, void *grad_logits,
             const void *denom, int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index, void *stream) {
    if (N < 0 || C < 1 || M < 0) {
        set_error("b200_pc_softmax_ce: bad shape N=%lld C=%lld M=%lld", (long long)N, (long long)C, (long long)M);
        return B200_ERR_ARG;
    }
    if (N * M == 0) return B200_OK;
    if (!logits || !labels || !weight || (!losses && !grad_logits)) {
        set_error("b200_pc_softmax_ce: null pointer");
        return B200_ERR_ARG;
    }
    PcParams p{logits, labels, weight, losses, grad_logits, N, C, M, ignore_index, static_cast<const double *>(denom)};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == B200_F32) return launch_pc<float>(p, s);
    if (dtype == B200_F16) return launch_pc<__half>(p, s);
    if (dtype == B200_BF16) return launch_pc<__nv_bfloat16>(p, s);
    set_error("b200_pc_softmax_ce: unknown dtype code %d", dtype);
    return B200_ERR_ARG;
}
}  // namespace
