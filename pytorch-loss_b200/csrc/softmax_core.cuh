// Per-pixel math of the two softmax-family losses, written once and used by every
// access regime (pixel tiles in shared memory, rows in shared memory, strided
// global sweeps).  A "pixel" is one channel vector x[0..C) with a label.
//
// The regimes feed the math through three phases, each a loop over (part of) the
// channels followed by a combine across the threads that share the pixel:
//   phase 1  running maxima                     -> Stat1
//   phase 2  sums relative to the maxima        -> Stat2
//   phase 3  gradient of channel j from x_j     (needs Stat1, Stat2 finalised)
//
// Label-smooth CE (reference csrc/lsr_kernel.cu:83-84,123-125 for the constants):
//   y_lb = 1-eps, y_j = eps/C, sumy = eps/C*(C-1) + 1-eps
//   loss = sumy*(m + log s) - eps/C * sum_j x_j - (1-eps-eps/C) * x_lb
//   grad_j = sumy * e^{x_j-m}/s - y_j
//
// Large-margin softmax (reference csrc/large_margin_kernel.cu:425-471), with
// m' = max_{j!=lb} x_j, d_j = x_j - m', s' = sum_{j!=lb} e^{d_j}, q_j = e^{d_j}/s',
// a = 1/(C-1), Sqx = sum_{j!=lb} q_j d_j, Sx = sum_{j!=lb} d_j:
//   loss = log(sum_j e^{x_j}) - x_lb + lam/2 * (Sqx - a*Sx)      (log s' cancels)
//   grad_lb = p_lb - 1;  grad_j = r*q_j + lam/2 * (q_j*(d_j + 1 - Sqx) - a),  r = 1 - p_lb
// Using the off-target maximum keeps q finite when the target logit dominates.
#pragma once

#include "common.cuh"

namespace b200 {

// kPC: proportion-corrected softmax cross entropy = label smooth with smoothing 0 and a class
// weight inside every exponential; only the resident-tile fused step is instantiated for it.
enum LossKind { kLSR = 0, kLMargin = 1, kPC = 2 };

struct LossConsts {
    // LSR
    float lb_pos, lb_neg, sumy;
    // LMargin
    float half_lam, a;
    int C;
};

__host__ __device__ inline LossConsts make_consts(int kind, int64_t C, float hp) {
    LossConsts k{};
    k.C = static_cast<int>(C);
    if (kind == kLSR) {
        k.lb_pos = 1.f - hp;
        k.lb_neg = hp / static_cast<float>(C);
        k.sumy = k.lb_neg * static_cast<float>(C - 1) + k.lb_pos;
    } else {
        k.half_lam = hp * 0.5f;
        k.a = 1.f / static_cast<float>(C - 1);
    }
    return k;
}

constexpr float kNegInf = -3.402823466e38f;   // finite stand-in: (-FLT_MAX) - x stays finite

template <int KIND> struct Stat1;
template <int KIND> struct Stat2;

// ------------------------------------------------------------------- LSR
template <> struct Stat1<kLSR> {
    float m;
    __device__ __forceinline__ void init() { m = kNegInf; }
    __device__ __forceinline__ void add(float x, bool /*is_lb*/) { m = fmaxf(m, x); }
    __device__ __forceinline__ void merge(const Stat1 &o) { m = fmaxf(m, o.m); }
    static constexpr int kWords = 1;
    __device__ __forceinline__ void store(float *p, int stride) const { p[0] = m; }
    __device__ __forceinline__ void load(const float *p, int stride) { m = p[0]; }
};
template <> struct Stat2<kLSR> {
    float s, sx, xl;
    __device__ __forceinline__ void init() { s = 0.f; sx = 0.f; xl = 0.f; }
    __device__ __forceinline__ void add(float x, bool is_lb, const Stat1<kLSR> &a) {
        s += exp_fast(x - a.m);
        sx += x;
        if (is_lb) xl = x;
    }
    __device__ __forceinline__ void merge(const Stat2 &o) { s += o.s; sx += o.sx; xl += o.xl; }
    static constexpr int kWords = 3;
    __device__ __forceinline__ void store(float *p, int stride) const {
        p[0] = s; p[stride] = sx; p[2 * stride] = xl;
    }
    __device__ __forceinline__ void load(const float *p, int stride) {
        s = p[0]; sx = p[stride]; xl = p[2 * stride];
    }
};

// --------------------------------------------------------------- LMargin
template <> struct Stat1<kLMargin> {
    float m_no;   // max over j != lb
    float xl;     // x_lb (others contribute -FLT_MAX)
    __device__ __forceinline__ void init() { m_no = kNegInf; xl = kNegInf; }
    __device__ __forceinline__ void add(float x, bool is_lb) {
        if (is_lb) xl = x; else m_no = fmaxf(m_no, x);
    }
    __device__ __forceinline__ void merge(const Stat1 &o) { m_no = fmaxf(m_no, o.m_no); xl = fmaxf(xl, o.xl); }
    static constexpr int kWords = 2;
    __device__ __forceinline__ void store(float *p, int stride) const { p[0] = m_no; p[stride] = xl; }
    __device__ __forceinline__ void load(const float *p, int stride) { m_no = p[0]; xl = p[stride]; }
};
template <> struct Stat2<kLMargin> {
    float s_no, sde, sd;   // sum e^d, sum d*e^d, sum d   over j != lb
    __device__ __forceinline__ void init() { s_no = 0.f; sde = 0.f; sd = 0.f; }
    __device__ __forceinline__ void add(float x, bool is_lb, const Stat1<kLMargin> &a) {
        if (!is_lb) {
            const float d = x - a.m_no;
            const float e = exp_fast(d);
            s_no += e;
            sde += d * e;
            sd += d;
        }
    }
    __device__ __forceinline__ void merge(const Stat2 &o) { s_no += o.s_no; sde += o.sde; sd += o.sd; }
    static constexpr int kWords = 3;
    __device__ __forceinline__ void store(float *p, int stride) const {
        p[0] = s_no; p[stride] = sde; p[2 * stride] = sd;
    }
    __device__ __forceinline__ void load(const float *p, int stride) {
        s_no = p[0]; sde = p[stride]; sd = p[2 * stride];
    }
};

// Finalised per-pixel quantities: loss value and what phase 3 needs.  Sums lie in [1, C], where
// lg2.approx / rcp.approx are accurate to ~1e-7 relative; the per-pixel epilogue then costs a
// dozen instructions instead of the ~60 of the IEEE-rounded logf / division sequences.
template <int KIND> struct PixelFinal;

template <> struct PixelFinal<kLSR> {
    float m, inv_s, loss;
    __device__ __forceinline__ void finish(const Stat1<kLSR> &a, const Stat2<kLSR> &b,
                                           const LossConsts &k) {
        m = a.m;
        inv_s = __fdividef(1.f, b.s);
        loss = k.sumy * (a.m + __logf(b.s)) - k.lb_neg * b.sx - (k.lb_pos - k.lb_neg) * b.xl;
    }
    __device__ __forceinline__ float grad(float x, bool is_lb, const LossConsts &k) const {
        return k.sumy * exp_fast(x - m) * inv_s - (is_lb ? k.lb_pos : k.lb_neg);
    }
    // Gradient from e = e^{x-m} kept from phase 2 (saves the second exponential).
    __device__ __forceinline__ float grad_from_exp(float e, bool is_lb, const LossConsts &k) const {
        return k.sumy * e * inv_s - (is_lb ? k.lb_pos : k.lb_neg);
    }
};

template <> struct PixelFinal<kLMargin> {
    float m_no, inv_s_no, r, sqx, g_lb, loss;
    __device__ __forceinline__ void finish(const Stat1<kLMargin> &a, const Stat2<kLMargin> &b,
                                           const LossConsts &k) {
        m_no = a.m_no;
        inv_s_no = __fdividef(1.f, b.s_no);
        sqx = b.sde * inv_s_no;
        // softmax over all channels from the off-target sum and the target logit
        const float m = fmaxf(a.m_no, a.xl);
        const float e_no = b.s_no * __expf(a.m_no - m);
        const float e_lb = __expf(a.xl - m);
        const float s_all = e_no + e_lb;
        r = __fdividef(e_no, s_all);
        g_lb = -r;                                 // p_lb - 1 = -(1 - p_lb)
        loss = (m + __logf(s_all)) - a.xl + k.half_lam * (sqx - k.a * b.sd);
    }
    __device__ __forceinline__ float grad(float x, bool is_lb, const LossConsts &k) const {
        if (is_lb) return g_lb;
        const float d = x - m_no;
        const float q = exp_fast(d) * inv_s_no;
        return r * q + k.half_lam * (q * (d + 1.f - sqx) - k.a);
    }
};

// Helpers of the kernels that keep e^{x-m} in shared memory between phases 2 and 3 (LSR only;
// the large-margin gradient needs x itself again).
__device__ __forceinline__ float s1_max(const Stat1<kLSR> &a) { return a.m; }
__device__ __forceinline__ void s2_add_with_exp(Stat2<kLSR> &b, float x, float e, bool is_lb) {
    b.s += e;
    b.sx += x;
    if (is_lb) b.xl = x;
}
// Phase-3 gradient from what the tile holds: e^{x-m} for LSR, x for large margin.
template <int KIND>
__device__ __forceinline__ float grad_phase3(const PixelFinal<KIND> &fin, float v, bool is_lb,
                                             const LossConsts &k) {
    if constexpr (KIND == kLSR) return fin.grad_from_exp(v, is_lb, k);
    else return fin.grad(v, is_lb, k);
}

// Upstream-gradient scale shared by all backward kernels: grad_mode 1 reads one device
// float, denom (optional) is a device double; mode 2 multiplies per pixel later.
__device__ __forceinline__ float uniform_grad_scale(const void *grad_out, int grad_mode,
                                                    const double *denom) {
    double g = 1.0;
    if (grad_mode == 1) g = double(*static_cast<const float *>(grad_out));
    if (denom) g /= *denom;
    return static_cast<float>(g);
}

}  // namespace b200
