// float64 instantiations of the label-smooth, large-margin and focal losses (sm_100a).
//
// The reference dispatches its kernels over double as well (AT_DISPATCH_FLOATING_TYPES,
// csrc/lsr_kernel.cu:218,239,283, csrc/focal_kernel.cu:192,232,268,
// csrc/large_margin_kernel.cu:628-710); callers use it for gradient checks and as a numerical
// yardstick, not for speed.  These kernels compute in double throughout with the plain library
// functions (exp, log, log1p, pow): one thread per pixel walking the channels in three strided
// sweeps (maximum, sums, gradients), one thread per element for focal.  Same entry points, same
// argument meaning as the float kernels (dtype code B200_F64); hyper-parameters still cross the
// boundary as float, as in the reference (csrc/lsr_kernel.cu:299).
#include "common.cuh"
#include "softmax_core.cuh"

namespace b200 {
namespace {

constexpr int kF64Threads = 256;

struct Softmax64Params {
    const double *x;
    const int64_t *labels;
    double *losses;          // [N, M] or null
    double *grads;           // [N, C, M] (backward)
    const void *grad_out;    // mode 1: device float; mode 2: double [N, M]
    int grad_mode;
    const double *denom;
    void *workspace;
    ReduceRecord *out;
    int64_t N, C, M, ignore;
    double hp;               // smoothing / lambda
};

template <int KIND, bool BWD, bool REDUCE>
__global__ void __launch_bounds__(kF64Threads) softmax64_kernel(const Softmax64Params p) {
    __shared__ double sh[64];
    const int64_t P = p.N * p.M;
    const int64_t C = p.C;
    double gscale = 1.0;
    if (BWD && p.grad_mode == 1) gscale = double(*static_cast<const float *>(p.grad_out));
    if (BWD && p.denom) gscale /= *p.denom;
    double acc = 0.0, cnt = 0.0;
    for (int64_t i = int64_t(blockIdx.x) * kF64Threads + threadIdx.x; i < P; i += int64_t(gridDim.x) * kF64Threads) {
        const int64_t n = i / p.M, m = i % p.M;
        const double *x = p.x + n * C * p.M + m;
        const int64_t lb = p.labels[i];
        const bool valid = lb != p.ignore;
        double *g = BWD ? p.grads + n * C * p.M + m : nullptr;
        if (!valid) {
            if (!BWD && p.losses) p.losses[i] = 0.0;
            if (BWD)
                for (int64_t j = 0; j < C; ++j) g[j * p.M] = 0.0;
            continue;
        }
        double sc = gscale;
        if (BWD && p.grad_mode == 2) sc *= static_cast<const double *>(p.grad_out)[i];
        // maximum over all channels, and over all but the target
        double mx = -INFINITY, mo = -INFINITY;
        for (int64_t j = 0; j < C; ++j) {
            const double v = x[j * p.M];
            mx = fmax(mx, v);
            if (j != lb) mo = fmax(mo, v);
        }
        const double xl = (lb >= 0 && lb < C) ? x[lb * p.M] : 0.0;
        if (KIND == kLSR) {
            const double lb_pos = 1.0 - p.hp, lb_neg = p.hp / double(C);
            const double sumy = lb_neg * double(C - 1) + lb_pos;
            double s = 0.0, sx = 0.0;
            for (int64_t j = 0; j < C; ++j) {
                const double v = x[j * p.M];
                s += exp(v - mx);
                sx += v;
            }
            if (!BWD) {
                const double l = sumy * (mx + log(s)) - lb_neg * sx - (lb_pos - lb_neg) * xl;
                if (p.losses) p.losses[i] = l;
                acc += l;
                cnt += 1.0;
            } else {
                const double inv = 1.0 / s;
                for (int64_t j = 0; j < C; ++j) {
                    const double pj = exp(x[j * p.M] - mx) * inv;
                    g[j * p.M] = (sumy * pj - (j == lb ? lb_pos : lb_neg)) * sc;
                }
            }
        } else {
            // q = softmax over the channels other than the target, a = 1 / (C - 1)
            const double half_lam = 0.5 * p.hp, a = 1.0 / double(C - 1);
            double so = 0.0, sqd = 0.0, sd = 0.0;          // sum e^{d}, sum d e^{d}, sum d   (d = x - mo, j != lb)
            for (int64_t j = 0; j < C; ++j) {
                if (j == lb) continue;
                const double d = x[j * p.M] - mo;
                const double e = exp(d);
                so += e;
                sqd += d * e;
                sd += d;
            }
            const double log_so = log(so);
            const double qd = sqd / so;                    // sum_j q_j d_j
            // all-channel softmax relative to mx
            const double s_all = so * exp(mo - mx) + exp(xl - mx);
            if (!BWD) {
                // sum_{j != lb} (q_j - a) log q_j with log q_j = d_j - log so
                const double margin = (qd - log_so) - a * (sd - double(C - 1) * log_so);
                const double l = (mx + log(s_all)) - xl + half_lam * margin;
                if (p.losses) p.losses[i] = l;
                acc += l;
                cnt += 1.0;
            } else {
                const double inv_all = 1.0 / s_all, inv_o = 1.0 / so;
                for (int64_t j = 0; j < C; ++j) {
                    const double v = x[j * p.M];
                    const double pj = exp(v - mx) * inv_all;
                    double gj;
                    if (j == lb) gj = pj - 1.0;
                    else {
                        const double d = v - mo;
                        const double q = exp(d) * inv_o;
                        gj = pj + half_lam * (q * (d + 1.0 - qd) - a);
                    }
                    g[j * p.M] = gj * sc;
                }
            }
        }
    }
    if (REDUCE) grid_reduce_finish(acc, cnt, p.workspace, p.out, sh);
}

struct Focal64Params {
    const double *x, *y;
    double *losses, *grads;
    const void *grad_out;
    int grad_mode;
    const double *denom;
    void *workspace;
    ReduceRecord *out;
    int64_t E;
    double gamma, alpha;
};

// reference csrc/focal_kernel.cu:43-50 (forward), :76-82 (gradient)
template <bool LOSS, bool GRAD, bool REDUCE>
__global__ void __launch_bounds__(kF64Threads) focal64_kernel(const Focal64Params p) {
    __shared__ double sh[64];
    double gscale = 1.0;
    if (GRAD && p.grad_mode == 1) gscale = double(*static_cast<const float *>(p.grad_out));
    if (GRAD && p.denom) gscale /= *p.denom;
    double acc = 0.0;
    for (int64_t i = int64_t(blockIdx.x) * kF64Threads + threadIdx.x; i < p.E; i += int64_t(gridDim.x) * kF64Threads) {
        const double x = p.x[i], y = p.y[i];
        const double e = exp(-fabs(x));
        const double l1p = log1p(e);
        const double prob = x >= 0.0 ? 1.0 / (1.0 + e) : e / (1.0 + e);
        const double log_p = x >= 0.0 ? -l1p : x - l1p;
        const double ce = y * p.alpha * log_p + (1.0 - y) * (1.0 - p.alpha) * (log_p - x);
        const double d = fabs(y - prob);
        const double coeff = -pow(d, p.gamma);
        if (LOSS) {
            const double l = coeff * ce;
            if (p.losses) p.losses[i] = l;
            acc += l;
        }
        if (GRAD) {
            const double d_ce = y * p.alpha - prob * (1.0 - y - p.alpha + 2.0 * y * p.alpha);
            double d_coeff = p.gamma * pow(d, p.gamma - 1.0) * prob * (1.0 - prob);
            if (y < prob) d_coeff = -d_coeff;
            double sc = gscale;
            if (p.grad_mode == 2) sc *= static_cast<const double *>(p.grad_out)[i];
            p.grads[i] = (d_coeff * ce + d_ce * coeff) * sc;
        }
    }
    if (REDUCE) {
        double cnt = 0.0;
        // every element counts: the grid-stride loop above visited ceil((E - first) / stride) of them
        for (int64_t i = int64_t(blockIdx.x) * kF64Threads + threadIdx.x; i < p.E; i += int64_t(gridDim.x) * kF64Threads)
            cnt += 1.0;
        grid_reduce_finish(acc, cnt, p.workspace, p.out, sh);
    }
}

unsigned grid_for(int64_t work) {
    int64_t g = (work + kF64Threads - 1) / kF64Threads;
    const int64_t cap = int64_t(sm_count()) * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return unsigned(g);
}

}  // namespace

int f64_softmax_forward(int kind, const void *logits, const int64_t *labels, void *losses, void *out, void *workspace,
                        int64_t N, int64_t C, int64_t M, int64_t ignore_index, float hp, void *stream) {
    Softmax64Params p{};
    p.x = static_cast<const double *>(logits);
    p.labels = labels;
    p.losses = static_cast<double *>(losses);
    p.workspace = workspace;
    p.out = static_cast<ReduceRecord *>(out);
    p.N = N; p.C = C; p.M = M; p.ignore = ignore_index;
    p.hp = double(hp);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = grid_for(N * M);
    if (kind == kLSR) {
        if (out) softmax64_kernel<kLSR, false, true><<<grid, kF64Threads, 0, s>>>(p);
        else softmax64_kernel<kLSR, false, false><<<grid, kF64Threads, 0, s>>>(p);
    } else {
        if (out) softmax64_kernel<kLMargin, false, true><<<grid, kF64Threads, 0, s>>>(p);
        else softmax64_kernel<kLMargin, false, false><<<grid, kF64Threads, 0, s>>>(p);
    }
    return launch_status("float64 softmax loss forward launch");
}

int f64_softmax_backward(int kind, const void *logits, const int64_t *labels, const void *grad_out, int grad_mode,
                         const void *denom, void *grad_logits, int64_t N, int64_t C, int64_t M,
                         int64_t ignore_index, float hp, void *stream) {
    Softmax64Params p{};
    p.x = static_cast<const double *>(logits);
    p.labels = labels;
    p.grads = static_cast<double *>(grad_logits);
    p.grad_out = grad_out;
    p.grad_mode = grad_mode;
    p.denom = static_cast<const double *>(denom);
    p.N = N; p.C = C; p.M = M; p.ignore = ignore_index;
    p.hp = double(hp);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = grid_for(N * M);
    if (kind == kLSR) softmax64_kernel<kLSR, true, false><<<grid, kF64Threads, 0, s>>>(p);
    else softmax64_kernel<kLMargin, true, false><<<grid, kF64Threads, 0, s>>>(p);
    return launch_status("float64 softmax loss backward launch");
}

int f64_focal(const void *logits, const void *labels, void *losses, void *grads, const void *grad_out, int grad_mode,
              const void *denom, void *out, void *workspace, int64_t E, float gamma, float alpha, void *stream) {
    Focal64Params p{};
    p.x = static_cast<const double *>(logits);
    p.y = static_cast<const double *>(labels);
    p.losses = static_cast<double *>(losses);
    p.grads = static_cast<double *>(grads);
    p.grad_out = grad_out;
    p.grad_mode = grad_mode;
    p.denom = static_cast<const double *>(denom);
    p.out = static_cast<ReduceRecord *>(out);
    p.workspace = workspace;
    p.E = E;
    p.gamma = double(gamma);
    p.alpha = double(alpha);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = grid_for(E);
    const bool want_loss = losses != nullptr || out != nullptr;
    if (grads && want_loss) focal64_kernel<true, true, false><<<grid, kF64Threads, 0, s>>>(p);
    else if (grads) focal64_kernel<false, true, false><<<grid, kF64Threads, 0, s>>>(p);
    else if (out) focal64_kernel<true, false, true><<<grid, kF64Threads, 0, s>>>(p);
    else focal64_kernel<true, false, false><<<grid, kF64Threads, 0, s>>>(p);
    return launch_status("float64 focal launch");
}

}  // namespace b200
