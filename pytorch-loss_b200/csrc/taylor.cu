// Taylor softmax / log-Taylor softmax over one dimension of a tensor (sm_100a).
//
// What is computed (reference csrc/taylor_softmax.cu:50-265, host side :268-417; Python
// taylor_softmax.py:15-50): with f(x) = sum_{i=0..n} x^i / i!  (n even, so f > 0),
//   forward   out_j = f(x_j) / S,  S = sum_j f(x_j)           (use_log: log f(x_j) - log S)
//   backward  softmax: dx_k = f'(x_k)/S * (g_k - sum_j g_j out_j)
//             log    : dx_k = f'(x_k) * (g_k / f(x_k) - (sum_j g_j) / S),   f' = sum_{i<n} x^i/i!
// over the dimension `dim` of a tensor viewed as [N, C, M] (N = product of the leading
// sizes, C = size(dim), M = product of the trailing sizes).
//
// How: the op streams x (and g) once from HBM and writes once; there is no exponential.  The
// log form takes the hardware logarithm (lg2.approx, a few ulp) per element and the library
// one per position for log S.
//   M > 1   few channels (<= 32 forward, <= 20 backward, float32): a thread owns 2 adjacent
//           positions (1 when M is odd or the pointers are not 8-byte aligned) and keeps all their
//           channels in registers -- one read, one write;
//           33..320 channels (float32): channel slices over the threads of a block, each thread's
//           share in registers, partial sums through shared memory -- again one read, one write;
//           otherwise a thread owns 4 adjacent positions along M (16-byte accesses when the layout
//           allows, else one position) and walks the C channels twice: sums first, outputs
//           second; the second walk finds its lines in L1/L2 (a block's working set is C x 4 KB).
//   M == 1  a warp owns a row: lanes stride over the channels, warp-shuffle sums; rows of 64..1024
//           floats stay in the warp's registers between the sum and the output (one read).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kTaylorThreads = 256;
constexpr int kMaxOrder = 16;

struct TaylorParams {
    const void *x;
    const void *g;        // backward only
    void *out;
    int64_t N, C, M;
    int order;            // n
};

// f (degree n) and, if wanted, f' (degree n - 1) by Horner's rule.  ORDER > 0: compile-time
// order (the loops unroll and 1/i become immediates); ORDER == 0: the order comes from p.
template <int ORDER, bool WANT_D>
__device__ __forceinline__ void taylor_poly(float x, const TaylorParams &p, float &f, float &d) {
    if constexpr (ORDER > 0) {
        float a = 1.f;
#pragma unroll
        for (int i = ORDER; i >= 1; --i) a = fmaf(a, x * (1.f / float(i)), 1.f);
        f = a;
        if (WANT_D) {
            float b = 1.f;
#pragma unroll
            for (int i = ORDER - 1; i >= 1; --i) b = fmaf(b, x * (1.f / float(i)), 1.f);
            d = b;
        }
    } else {
        float a = 1.f;
        for (int i = p.order; i >= 1; --i) a = fmaf(a, x * __frcp_rn(float(i)), 1.f);
        f = a;
        if (WANT_D) {
            float b = 1.f;
            for (int i = p.order - 1; i >= 1; --i) b = fmaf(b, x * __frcp_rn(float(i)), 1.f);
            d = b;
        }
    }
}

template <typename T, int VEC> struct Pack;
template <> struct Pack<float, 4> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <typename T> struct Pack<T, 1> {
    static __device__ __forceinline__ void load(const T *p, float (&v)[1]) { v[0] = to_f32(*p); }
    static __device__ __forceinline__ void store(T *p, const float (&v)[1]) { *p = from_f32<T>(v[0]); }
};

// M > 1: VEC adjacent positions per thread, two walks over the channels.
template <typename T, int VEC, bool BWD, bool LOG, int ORDER>
__global__ void __launch_bounds__(kTaylorThreads)
taylor_spatial_kernel(const TaylorParams p) {
    const T *x = static_cast<const T *>(p.x);
    const T *g = static_cast<const T *>(p.g);
    T *out = static_cast<T *>(p.out);
    const int64_t groups_per_row = p.M / VEC;          // VEC > 1 only when M % VEC == 0
    const int64_t groups = p.N * groups_per_row;
    const int64_t stride = int64_t(gridDim.x) * kTaylorThreads;
    for (int64_t gi = int64_t(blockIdx.x) * kTaylorThreads + threadIdx.x; gi < groups; gi += stride) {
        const int64_t n = gi / groups_per_row, m0 = (gi % groups_per_row) * VEC;
        const int64_t base = n * p.C * p.M + m0;
        float S[VEC], A[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) S[v] = A[v] = 0.f;
#pragma unroll 4
        for (int64_t j = 0; j < p.C; ++j) {
            float xv[VEC], gv[VEC];
            Pack<T, VEC>::load(x + base + j * p.M, xv);
            if (BWD) Pack<T, VEC>::load(g + base + j * p.M, gv);
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float f, d;
                taylor_poly<ORDER, false>(xv[v], p, f, d);
                S[v] += f;
                if (BWD) A[v] += LOG ? gv[v] : gv[v] * f;      // log: sum g;  softmax: sum g f
            }
        }
        float invS[VEC], logS[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            invS[v] = 1.f / S[v];
            logS[v] = LOG && !BWD ? logf(S[v]) : 0.f;
        }
#pragma unroll 4
        for (int64_t j = 0; j < p.C; ++j) {
            float xv[VEC], gv[VEC], ov[VEC];
            Pack<T, VEC>::load(x + base + j * p.M, xv);
            if (BWD) Pack<T, VEC>::load(g + base + j * p.M, gv);
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float f, d;
                taylor_poly<ORDER, BWD>(xv[v], p, f, d);
                if (!BWD) ov[v] = LOG ? __logf(f) - logS[v] : f * invS[v];
                else if (LOG) ov[v] = d * (gv[v] / f - A[v] * invS[v]);
                else ov[v] = d * invS[v] * (gv[v] - A[v] * invS[v]);
            }
            Pack<T, VEC>::store(out + base + j * p.M, ov);
        }
    }
}

// M > 1, few channels (C <= CMAX), float32: a thread owns VEC adjacent positions (2: 8-byte
// accesses, 256 B per warp and channel, M even and 8-byte aligned pointers; 1: any M, any
// alignment) and keeps all their channels in registers, so x (and g) are read once.
template <bool BWD, bool LOG, int ORDER, int CMAX, int VEC>
__global__ void __launch_bounds__(kTaylorThreads, (!BWD && CMAX <= 20) || VEC == 1 ? 3 : 2)
taylor_resident_kernel(const TaylorParams p) {
    const float *x = static_cast<const float *>(p.x);
    const float *g = static_cast<const float *>(p.g);
    float *out = static_cast<float *>(p.out);
    const int C = int(p.C);
    const int64_t groups_per_row = p.M / VEC;
    const int64_t groups = p.N * groups_per_row;
    const int64_t stride = int64_t(gridDim.x) * kTaylorThreads;
    struct Vals { float v[VEC]; };
    auto load = [](const float *q) {
        Vals r;
        if constexpr (VEC == 2) {
            const float2 f = __ldcs(reinterpret_cast<const float2 *>(q));
            r.v[0] = f.x;
            r.v[1] = f.y;
        } else {
            r.v[0] = __ldcs(q);
        }
        return r;
    };
    for (int64_t gi = int64_t(blockIdx.x) * kTaylorThreads + threadIdx.x; gi < groups; gi += stride) {
        const int64_t n = gi / groups_per_row, m0 = (gi % groups_per_row) * VEC;
        const int64_t base = n * p.C * p.M + m0;
        Vals xv[CMAX], gv[BWD ? CMAX : 1];
#pragma unroll
        for (int j = 0; j < CMAX; ++j) {
            if (j < C) {
                xv[j] = load(x + base + j * p.M);
                if (BWD) gv[j] = load(g + base + j * p.M);
            }
        }
        float S[VEC], A[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) S[v] = A[v] = 0.f;
#pragma unroll
        for (int j = 0; j < CMAX; ++j) {
            if (j < C) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float f, d;
                    taylor_poly<ORDER, false>(xv[j].v[v], p, f, d);
                    S[v] += f;
                    if (BWD) A[v] += LOG ? gv[j].v[v] : gv[j].v[v] * f;
                    else xv[j].v[v] = f;          // forward: f(x) takes x's place; backward recomputes it with f'
                }
            }
        }
        float invS[VEC], logS[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            invS[v] = 1.f / S[v];
            logS[v] = LOG && !BWD ? logf(S[v]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < CMAX; ++j) {
            if (j < C) {
                float o[VEC];
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    if constexpr (!BWD) {
                        o[v] = LOG ? __logf(xv[j].v[v]) - logS[v] : xv[j].v[v] * invS[v];
                    } else {
                        float f, d;
                        taylor_poly<ORDER, true>(xv[j].v[v], p, f, d);
                        o[v] = LOG ? d * (gv[j].v[v] / f - A[v] * invS[v]) : d * invS[v] * (gv[j].v[v] - A[v] * invS[v]);
                    }
                }
                if constexpr (VEC == 2) __stcs(reinterpret_cast<float2 *>(out + base + j * p.M), make_float2(o[0], o[1]));
                else __stcs(out + base + j * p.M, o[0]);
            }
        }
    }
}

// M > 1, more channels than one thread can hold (float32, M even, 8-byte aligned): the 256
// threads of a block are KS channel slices x (256 / KS) adjacent position PAIRS; a thread keeps
// its slice's channels (every KS-th, at most CPT of them) of one pair in registers -- a warp
// reads 256 contiguous bytes per channel -- and the slices add their partial sums through shared
// memory (two buffers, one block barrier per group of positions).  x and g are read once.
template <bool BWD, bool LOG, int ORDER, int KS, int CPT>
__global__ void __launch_bounds__(kTaylorThreads, 2)
taylor_sliced_kernel(const TaylorParams p) {
    constexpr int PX = kTaylorThreads / KS;            // position pairs per block and round
    __shared__ float2 part[2][2][KS][PX];              // [round parity][S, A][slice][pair]
    const float *x = static_cast<const float *>(p.x);
    const float *g = static_cast<const float *>(p.g);
    float *out = static_cast<float *>(p.out);
    const int C = int(p.C);
    const int M = int(p.M);                            // C * M < 2^31 (host check): 32-bit channel offsets
    const int px = threadIdx.x % PX, ks = threadIdx.x / PX;
    const int64_t groups_per_row = (p.M / 2 + PX - 1) / PX;
    const int64_t groups = p.N * groups_per_row;
    int par = 0;
    for (int64_t gi = blockIdx.x; gi < groups; gi += gridDim.x, par ^= 1) {
        const int64_t n = gi / groups_per_row;
        const int m = (int(gi % groups_per_row) * PX + px) * 2;
        const bool live = m < M;
        const int64_t base = n * p.C * p.M + (live ? m : 0);
        const float *xb = x + base;
        const float *gb = BWD ? g + base : nullptr;
        float2 xv[CPT], gv[BWD ? CPT : 1];
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int j = ks + i * KS;
            if (live && j < C) {
                xv[i] = __ldcs(reinterpret_cast<const float2 *>(xb + j * M));
                if (BWD) gv[i] = __ldcs(reinterpret_cast<const float2 *>(gb + j * M));
            }
        }
        float2 S = make_float2(0.f, 0.f), A = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            if (ks + i * KS < C) {
                float d;
                float2 f;
                taylor_poly<ORDER, false>(xv[i].x, p, f.x, d);
                taylor_poly<ORDER, false>(xv[i].y, p, f.y, d);
                S.x += f.x;
                S.y += f.y;
                if (BWD) {
                    A.x += LOG ? gv[i].x : gv[i].x * f.x;
                    A.y += LOG ? gv[i].y : gv[i].y * f.y;
                } else {
                    xv[i] = f;                        // forward: f(x) takes x's place
                }
            }
        }
        part[par][0][ks][px] = S;
        if (BWD) part[par][1][ks][px] = A;
        __syncthreads();
        S = make_float2(0.f, 0.f);
        A = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < KS; ++q) {
            const float2 s = part[par][0][q][px];
            S.x += s.x;
            S.y += s.y;
            if (BWD) {
                const float2 a = part[par][1][q][px];
                A.x += a.x;
                A.y += a.y;
            }
        }
        if (!live) continue;
        const float2 invS = make_float2(1.f / S.x, 1.f / S.y);
        const float2 logS = LOG && !BWD ? make_float2(logf(S.x), logf(S.y)) : make_float2(0.f, 0.f);
        float *ob = out + base;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int j = ks + i * KS;
            if (j < C) {
                float2 o;
                if constexpr (!BWD) {
                    o.x = LOG ? __logf(xv[i].x) - logS.x : xv[i].x * invS.x;
                    o.y = LOG ? __logf(xv[i].y) - logS.y : xv[i].y * invS.y;
                } else {
                    float fx, fy, dx, dy;
                    taylor_poly<ORDER, true>(xv[i].x, p, fx, dx);
                    taylor_poly<ORDER, true>(xv[i].y, p, fy, dy);
                    if (LOG) {
                        o.x = dx * (gv[i].x / fx - A.x * invS.x);
                        o.y = dy * (gv[i].y / fy - A.y * invS.y);
                    } else {
                        o.x = dx * invS.x * (gv[i].x - A.x * invS.x);
                        o.y = dy * invS.y * (gv[i].y - A.y * invS.y);
                    }
                }
                __stcs(reinterpret_cast<float2 *>(ob + j * M), o);
            }
        }
    }
}

// M == 1: one warp per row.
template <typename T, bool BWD, bool LOG, int ORDER>
__global__ void __launch_bounds__(kTaylorThreads)
taylor_rows_kernel(const TaylorParams p) {
    const T *x = static_cast<const T *>(p.x);
    const T *g = static_cast<const T *>(p.g);
    T *out = static_cast<T *>(p.out);
    const int lane = threadIdx.x & 31;
    const int64_t warps = int64_t(gridDim.x) * (kTaylorThreads / 32);
    for (int64_t r = int64_t(blockIdx.x) * (kTaylorThreads / 32) + (threadIdx.x >> 5); r < p.N; r += warps) {
        const T *xr = x + r * p.C;
        const T *gr = BWD ? g + r * p.C : nullptr;
        float S = 0.f, A = 0.f;
#pragma unroll 8
        for (int64_t j = lane; j < p.C; j += 32) {
            float f, d;
            taylor_poly<ORDER, false>(to_f32(xr[j]), p, f, d);
            S += f;
            if (BWD) A += LOG ? to_f32(gr[j]) : to_f32(gr[j]) * f;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            S += __shfl_xor_sync(0xffffffffu, S, o);
            A += __shfl_xor_sync(0xffffffffu, A, o);
        }
        const float invS = 1.f / S, logS = LOG && !BWD ? logf(S) : 0.f;
#pragma unroll 8
        for (int64_t j = lane; j < p.C; j += 32) {
            float f, d;
            taylor_poly<ORDER, BWD>(to_f32(xr[j]), p, f, d);
            float o;
            if (!BWD) o = LOG ? __logf(f) - logS : f * invS;
            else if (LOG) o = d * (to_f32(gr[j]) / f - A * invS);
            else o = d * invS * (to_f32(gr[j]) - A * invS);
            out[r * p.C + j] = from_f32<T>(o);
        }
    }
}

// M == 1, rows of up to 32 * NV * 4 floats (float32, C a multiple of 4, 16-byte aligned pointers):
// a warp owns a row and keeps it in registers -- NV 16-byte vectors per lane, all loads of a lane
// in flight together -- so x (and g) are read once; sums by warp shuffles.
template <bool BWD, bool LOG, int ORDER, int NV>
__global__ void __launch_bounds__(kTaylorThreads, BWD ? 2 : 3)
taylor_rows_resident_kernel(const TaylorParams p) {
    const float4 *x = static_cast<const float4 *>(p.x);
    const float4 *g = static_cast<const float4 *>(p.g);
    float4 *out = static_cast<float4 *>(p.out);
    const int lane = threadIdx.x & 31;
    const int nvec = int(p.C) >> 2;                     // 16-byte vectors per row
    const int64_t warps = int64_t(gridDim.x) * (kTaylorThreads / 32);
    for (int64_t r = int64_t(blockIdx.x) * (kTaylorThreads / 32) + (threadIdx.x >> 5); r < p.N; r += warps) {
        const float4 *xr = x + r * nvec;
        const float4 *gr = BWD ? g + r * nvec : nullptr;
        float4 xv[NV], gv[BWD ? NV : 1];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                xv[i] = __ldcs(xr + v);
                if (BWD) gv[i] = __ldcs(gr + v);
            }
        }
        float S = 0.f, A = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32 * i < nvec) {
                float *xe = reinterpret_cast<float *>(&xv[i]);
                const float *ge = reinterpret_cast<const float *>(&gv[BWD ? i : 0]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float f, d;
                    taylor_poly<ORDER, false>(xe[e], p, f, d);
                    S += f;
                    if (BWD) A += LOG ? ge[e] : ge[e] * f;
                    else xe[e] = f;                     // forward: f(x) takes x's place
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            S += __shfl_xor_sync(0xffffffffu, S, o);
            if (BWD) A += __shfl_xor_sync(0xffffffffu, A, o);
        }
        const float invS = 1.f / S, logS = LOG && !BWD ? logf(S) : 0.f;
        float4 *orow = out + r * nvec;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float4 o4;
                float *oe = reinterpret_cast<float *>(&o4);
                const float *xe = reinterpret_cast<const float *>(&xv[i]);
                const float *ge = reinterpret_cast<const float *>(&gv[BWD ? i : 0]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if constexpr (!BWD) {
                        oe[e] = LOG ? __logf(xe[e]) - logS : xe[e] * invS;
                    } else {
                        float f, d;
                        taylor_poly<ORDER, true>(xe[e], p, f, d);
                        oe[e] = LOG ? d * (ge[e] / f - A * invS) : d * invS * (ge[e] - A * invS);
                    }
                }
                __stcs(orow + v, o4);
            }
        }
    }
}

inline bool aligned16(const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

template <typename T, bool BWD, bool LOG, int ORDER>
int launch_taylor(const TaylorParams &p, cudaStream_t stream) {
    if (p.M == 1) {
        int64_t grid = (p.N + kTaylorThreads / 32 - 1) / (kTaylorThreads / 32);
        const int64_t cap = int64_t(sm_count()) * 8;
        if (grid > cap) grid = cap;
        if constexpr (sizeof(T) == 4 && ORDER > 0) {
            // classification-sized rows: the row stays in the warp's registers (one read)
            if (p.C % 4 == 0 && p.C >= 64 && p.C <= 1024 && aligned16(p.x) && aligned16(p.out) && (!BWD || aligned16(p.g))) {
                if (p.C <= 256)
                    taylor_rows_resident_kernel<BWD, LOG, ORDER, 2><<<unsigned(grid), kTaylorThreads, 0, stream>>>(p);
                else
                    taylor_rows_resident_kernel<BWD, LOG, ORDER, 8><<<unsigned(grid), kTaylorThreads, 0, stream>>>(p);
                return launch_status("taylor softmax resident rows kernel launch");
            }
        }
        taylor_rows_kernel<T, BWD, LOG, ORDER><<<unsigned(grid), kTaylorThreads, 0, stream>>>(p);
        return launch_status("taylor softmax rows kernel launch");
    }
    if constexpr (sizeof(T) == 4) {
        // few channels: everything a thread needs stays in its registers, one read of x (and g)
        const bool al8 = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out) |
                           (BWD ? reinterpret_cast<uintptr_t>(p.g) : 0)) & 7u) == 0;
        constexpr int kSmall = BWD ? 20 : 32;
        if (p.C <= kSmall) {
            const bool pairs = p.M % 2 == 0 && al8;        // else one position per thread: any M, any alignment
            const int64_t groups2 = p.N * (pairs ? p.M / 2 : p.M);
            int64_t grid2 = (groups2 + kTaylorThreads - 1) / kTaylorThreads;
            const int64_t cap2 = int64_t(sm_count()) * 2 * 8;
            if (grid2 > cap2) grid2 = cap2;
            const unsigned g2 = unsigned(grid2);
            if (pairs) {
                if (p.C <= 8) taylor_resident_kernel<BWD, LOG, ORDER, 8, 2><<<g2, kTaylorThreads, 0, stream>>>(p);
                else if (!BWD && p.C <= 20) taylor_resident_kernel<false, LOG, ORDER, 20, 2><<<g2, kTaylorThreads, 0, stream>>>(p);
                else taylor_resident_kernel<BWD, LOG, ORDER, kSmall, 2><<<g2, kTaylorThreads, 0, stream>>>(p);
            } else {
                if (p.C <= 8) taylor_resident_kernel<BWD, LOG, ORDER, 8, 1><<<g2, kTaylorThreads, 0, stream>>>(p);
                else taylor_resident_kernel<BWD, LOG, ORDER, kSmall, 1><<<g2, kTaylorThreads, 0, stream>>>(p);
            }
            return launch_status("taylor softmax resident kernel launch");
        }
    }
    if constexpr (sizeof(T) == 4 && ORDER > 0) {
        // 33..320 channels: sliced register-resident kernel (forward: 40 channels per thread in 4
        // or 8 slices; backward holds x and g: 20 channels per thread in 8 or 16 slices)
        const bool al8s = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out) |
                            (BWD ? reinterpret_cast<uintptr_t>(p.g) : 0)) & 7u) == 0;
        // (measured at [16,64,512,512] / [16,40,512,512]: the forward ties with or loses to the two
        // walks below up to ~96 channels, 0.58 / 0.59 against 0.61 / 0.68 of peak; the backward wins from
        // 33 on, 0.90 / 0.69 against 0.62 / 0.63; at 150 channels 0.83 / 1.00 against 0.60 / 0.61)
        if (p.C > (BWD ? 32 : 96) && p.C <= 320 && p.C * p.M < (int64_t(1) << 31) && p.M >= 64 && p.M % 2 == 0 && al8s) {
            // slices so that a thread holds 20..48 channels: few channels per thread leave too few
            // bytes in flight between two block barriers (C = 40 in 4 slices: 0.46 of peak)
            constexpr int KS0 = BWD ? 4 : 2, KS1 = BWD ? 8 : 4, KS2 = BWD ? 16 : 8;
            constexpr int CPT0 = BWD ? 24 : 48, CPT = BWD ? 20 : 40;
            const int ks = p.C <= 96 ? KS0 : (p.C <= 160 ? KS1 : KS2);
            const int px = kTaylorThreads / ks;
            const int64_t rounds = p.N * ((p.M / 2 + px - 1) / px);
            int64_t grid3 = int64_t(sm_count()) * 2;
            if (grid3 > rounds) grid3 = rounds;
            const unsigned g3 = unsigned(grid3);
            if (ks == KS0) taylor_sliced_kernel<BWD, LOG, ORDER, KS0, CPT0><<<g3, kTaylorThreads, 0, stream>>>(p);
            else if (ks == KS1) taylor_sliced_kernel<BWD, LOG, ORDER, KS1, CPT><<<g3, kTaylorThreads, 0, stream>>>(p);
            else taylor_sliced_kernel<BWD, LOG, ORDER, KS2, CPT><<<g3, kTaylorThreads, 0, stream>>>(p);
            return launch_status("taylor softmax sliced kernel launch");
        }
    }
    const bool vec4 = sizeof(T) == 4 && p.M % 4 == 0 && aligned16(p.x) && aligned16(p.out) && (!BWD || aligned16(p.g));
    const int64_t groups = p.N * (vec4 ? p.M / 4 : p.M);
    int64_t grid = (groups + kTaylorThreads - 1) / kTaylorThreads;
    // few resident blocks: the second walk over the channels should find the first walk's lines
    // in L1 (a block's working set is C x 4 KB (x 2 in backward))
    const int64_t cap = int64_t(sm_count()) * 3;
    if (grid > cap) grid = cap;
    if constexpr (sizeof(T) == 4) {
        if (vec4) {
            taylor_spatial_kernel<T, 4, BWD, LOG, ORDER><<<unsigned(grid), kTaylorThreads, 0, stream>>>(p);
            return launch_status("taylor softmax kernel launch");
        }
    }
    taylor_spatial_kernel<T, 1, BWD, LOG, ORDER><<<unsigned(grid), kTaylorThreads, 0, stream>>>(p);
    return launch_status("taylor softmax kernel launch");
}

template <typename T, bool BWD, bool LOG>
int launch_taylor_order(const TaylorParams &p, cudaStream_t stream) {
    switch (p.order) {
        case 2: return launch_taylor<T, BWD, LOG, 2>(p, stream);
        case 4: return launch_taylor<T, BWD, LOG, 4>(p, stream);
        case 6: return launch_taylor<T, BWD, LOG, 6>(p, stream);
        default: return launch_taylor<T, BWD, LOG, 0>(p, stream);
    }
}

template <bool BWD>
int dispatch_taylor(TaylorParams &p, int dtype, int order, int use_log, const char *who, cudaStream_t stream) {
    if (p.N < 0 || p.C < 1 || p.M < 0) {
        set_error("%s: bad shape N=%lld C=%lld M=%lld", who, (long long)p.N, (long long)p.C, (long long)p.M);
        return B200_ERR_ARG;
    }
    if (order < 2 || order > kMaxOrder || (order & 1)) {
        set_error("%s: n must be even, 2 <= n <= %d (got %d)", who, kMaxOrder, order);
        return B200_ERR_ARG;
    }
    if (p.N * p.M == 0) return B200_OK;
    if (!p.x || !p.out || (BWD && !p.g)) {
        set_error("%s: null pointer", who);
        return B200_ERR_ARG;
    }
    p.order = order;
    if (dtype == B200_F32)
        return use_log ? launch_taylor_order<float, BWD, true>(p, stream) : launch_taylor_order<float, BWD, false>(p, stream);
    if (dtype == B200_F16)
        return use_log ? launch_taylor_order<__half, BWD, true>(p, stream)
                       : launch_taylor_order<__half, BWD, false>(p, stream);
    if (dtype == B200_BF16)
        return use_log ? launch_taylor_order<__nv_bfloat16, BWD, true>(p, stream)
                       : launch_taylor_order<__nv_bfloat16, BWD, false>(p, stream);
    set_error("%s: unknown dtype code %d", who, dtype);
    return B200_ERR_ARG;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_taylor_softmax_forward(const void *feat, void *out, int64_t N, int64_t C, int64_t M, int dtype,
                                           int n, int use_log, void *stream) {
    TaylorParams p{};
    p.x = feat;
    p.out = out;
    p.N = N; p.C = C; p.M = M;
    return dispatch_taylor<false>(p, dtype, n, use_log, "b200_taylor_softmax_forward", static_cast<cudaStream_t>(stream));
}

extern "C" int b200_taylor_softmax_backward(const void *grad, const void *feat, void *grad_feat, int64_t N, int64_t C,
                                            int64_t M, int dtype, int n, int use_log, void *stream) {
    TaylorParams p{};
    p.x = feat;
    p.g = grad;
    p.out = grad_feat;
    p.N = N; p.C = C; p.M = M;
    return dispatch_taylor<true>(p, dtype, n, use_log, "b200_taylor_softmax_backward", static_cast<cudaStream_t>(stream));
}
