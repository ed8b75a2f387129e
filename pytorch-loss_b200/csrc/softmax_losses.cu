// Label-smooth CE and large-margin softmax for sm_100a: three access regimes around
// one math core (softmax_core.cuh).
//
//  tile   M > 1 (pixels contiguous): a CTA stages a [C x TP] tile of logits in shared
//         memory with ONE tiled bulk-async (TMA) load per <=256 channels, 256 threads work
//         on it as TP pixels x KS channel slices (lanes along pixels: bank-conflict-free),
//         the backward overwrites the tile with gradients and one TMA store returns it.
//         Logits cross HBM exactly once per pass, every access is a full 32-byte sector
//         whatever C is.  Several CTAs per SM overlap one tile's copy with another's math.
//         Falls back to cooperative loads/stores into the same tile when the tensor is
//         not 16-byte aligned along M.
//  rows   M == 1 (channels contiguous, e.g. [rows, 32768] classification): a CTA stages
//         one row with an untiled bulk-async copy, reduces it with warp shuffles, writes
//         gradients into the same buffer and bulk-stores it.
//  sweep  anything else (tiny C with M == 1, tiles or rows too large for shared memory):
//         one thread per pixel, two strided sweeps over global memory.
//
// Forward kernels either write per-pixel losses, or only the [sum, count] record
// (deterministic last-block reduction), or both.  Backward kernels recompute the softmax
// and scale by the upstream gradient and the (device-resident) valid count.
#include "softmax_core.cuh"
#include "pipeline.cuh"

#include <stdlib.h>

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr size_t kTileTargetBytes = 48 * 1024;
constexpr size_t kSmemLimit = 200 * 1024;

constexpr int kPcMaxC = 256;     // classes the kPC fused step holds weights for

struct SoftmaxParams {
    const void *logits;
    const int64_t *labels;
    void *losses;            // [N, M] dtype or null
    void *grads;             // [N, C, M] dtype (backward)
    const void *grad_out;    // see grad_mode
    int grad_mode;
    const double *denom;
    void *workspace;
    ReduceRecord *out;
    float4 *stats;           // [N*M] per-pixel statistics: written by the chunked forward, read by
                             // the chunked backward (null: not wanted / not available)
    int64_t N, C, M;
    int64_t ignore;
    LossConsts k;
    // tile geometry
    int TP, KS, CB, nbox, rows;
    int nbx;                 // boxes of TP pixels per tile (pair kernel)
    int stages;              // ring depth of the pipelined kernels
    int64_t tiles_per_image, total_tiles;
    int defer;               // cross-GPU sum of the fused step: post only (see grid_reduce_finish)
    int after_count;         // fused step launched as a programmatic dependent of the label count
    const float *chan_w;     // kPC: class weights [C] (device)
};

// ------------------------------------------------------------------ tile regime

template <typename T, int KIND, bool BWD, bool REDUCE, bool TMA>
__global__ void __launch_bounds__(kThreads)
tile_kernel(const SoftmaxParams prm, const __grid_constant__ CUtensorMap map_in,
            const __grid_constant__ CUtensorMap map_out) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ double sh_red[64];

    const int TP = prm.TP, KS = prm.KS, C = static_cast<int>(prm.C);
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    T *tile = reinterpret_cast<T *>(base);
    float *red = reinterpret_cast<float *>(base + ((size_t(prm.rows) * TP * sizeof(T) + 127) & ~size_t(127)));
    // red: [6][KS*TP] floats

    const int tid = threadIdx.x;
    const int p = tid % TP, ks = tid / TP;
    const int slab = KS * TP;
    unsigned *status = reinterpret_cast<unsigned *>(prm.workspace) + 1;

    const T *logits = static_cast<const T *>(prm.logits);
    T *grads = static_cast<T *>(prm.grads);
    T *losses = static_cast<T *>(prm.losses);
    const T *gout = static_cast<const T *>(prm.grad_out);

    if (TMA && tid == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();

    float gscale = 1.f;
    if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);

    double acc_loss = 0.0, acc_cnt = 0.0;
    uint32_t phase = 0;
    const uint32_t tile_bytes = uint32_t(prm.nbox) * prm.CB * TP * sizeof(T);

    for (int64_t t = blockIdx.x; t < prm.total_tiles; t += gridDim.x) {
        const int64_t n = t / prm.tiles_per_image;
        const int64_t p0 = (t % prm.tiles_per_image) * TP;
        const int64_t img_base = n * prm.C * prm.M;

        if (TMA) {
            if (tid == 0) {
                mbar_expect_tx(&bar, tile_bytes);
                for (int b = 0; b < prm.nbox; ++b)
                    tma_load_3d(tile + size_t(b) * prm.CB * TP, &map_in, int(p0), b * prm.CB, int(n), &bar);
            }
        } else {
            for (int idx = tid; idx < C * TP; idx += kThreads) {
                const int j = idx / TP, pp = idx % TP;
                const int64_t px = p0 + pp;
                tile[idx] = px < prm.M ? logits[img_base + int64_t(j) * prm.M + px] : from_f32<T>(0.f);
            }
        }
        const int64_t pix = p0 + p;
        const bool inb = pix < prm.M;
        const int64_t lb = inb ? prm.labels[n * prm.M + pix] : prm.ignore;
        const bool valid = inb && lb != prm.ignore;
        float pscale = gscale;
        if (BWD && prm.grad_mode == 2 && inb) pscale *= to_f32(gout[n * prm.M + pix]);

        if (TMA) {
            const bool ok = mbar_wait_bounded(&bar, phase, prm.workspace ? status : nullptr);
            if (!__syncthreads_and(ok)) break;   // uniform decision: no thread is left behind
            phase ^= 1;
        } else {
            __syncthreads();
        }

        const T *col = tile + p;
        // phase 1
        Stat1<KIND> s1;
        s1.init();
        for (int j = ks; j < C; j += KS) s1.add(to_f32(col[j * TP]), j == lb);
        if (KS > 1) {
            s1.store(red + tid, slab);
            __syncthreads();
            s1.init();
            for (int q = 0; q < KS; ++q) {
                Stat1<KIND> o;
                o.load(red + q * TP + p, slab);
                s1.merge(o);
            }
        }
        // phase 2
        Stat2<KIND> s2;
        s2.init();
        for (int j = ks; j < C; j += KS) s2.add(to_f32(col[j * TP]), j == lb, s1);
        if (KS > 1) {
            float *r2 = red + 2 * slab;
            s2.store(r2 + tid, slab);
            __syncthreads();
            s2.init();
            for (int q = 0; q < KS; ++q) {
                Stat2<KIND> o;
                o.load(r2 + q * TP + p, slab);
                s2.merge(o);
            }
        }
        PixelFinal<KIND> fin;
        fin.finish(s1, s2, prm.k);

        if (!BWD) {
            if (ks == 0 && inb) {
                const float l = valid ? fin.loss : 0.f;
                if (losses) losses[n * prm.M + pix] = from_f32<T>(l);
                if (REDUCE && valid) {
                    acc_loss += double(l);
                    acc_cnt += 1.0;
                }
            }
            if (!TMA || KS == 1) __syncthreads();   // tile (and red) free before the next load
        } else {
            T *wcol = tile + p;
            if (valid) {
                for (int j = ks; j < C; j += KS)
                    wcol[j * TP] = from_f32<T>(fin.grad(to_f32(wcol[j * TP]), j == lb, prm.k) * pscale);
            } else {
                for (int j = ks; j < C; j += KS) wcol[j * TP] = from_f32<T>(0.f);
            }
            if (TMA) {
                fence_proxy_async_smem();
                __syncthreads();
                if (tid == 0) {
                    for (int b = 0; b < prm.nbox; ++b)
                        tma_store_3d(&map_out, int(p0), b * prm.CB, int(n), tile + size_t(b) * prm.CB * TP);
                    bulk_commit();
                    bulk_wait_read_all();
                }
            } else {
                __syncthreads();
                for (int idx = tid; idx < C * TP; idx += kThreads) {
                    const int j = idx / TP, pp = idx % TP;
                    const int64_t px = p0 + pp;
                    if (px < prm.M) grads[img_base + int64_t(j) * prm.M + px] = tile[idx];
                }
                __syncthreads();
            }
        }
    }
    if (TMA && BWD && tid == 0) bulk_wait_all();
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// ------------------------------------------------------------------ rows regime
// One CTA per row of C contiguous values (M == 1).

template <int KIND> struct BlockStats {
    // Combines per-thread stats across the block through shared memory (32 warps max).
    template <typename S>
    __device__ static void combine(S &s, float *sh /* [32 * S::kWords] */) {
        // warp level: butterfly so every lane holds the warp's result
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            S other = s;
            float *w = reinterpret_cast<float *>(&other);
#pragma unroll
            for (int i = 0; i < S::kWords; ++i) w[i] = __shfl_xor_sync(0xffffffffu, w[i], o);
            s.merge(other);
        }
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        __syncthreads();
        if (lane == 0) s.store(sh + warp, 32);
        __syncthreads();
        S tot;
        tot.load(sh, 32);
        for (int w = 1; w < nwarp; ++w) {
            S o;
            o.load(sh + w, 32);
            tot.merge(o);
        }
        s = tot;
    }
};

template <typename T, int KIND, bool BWD, bool REDUCE, bool BULK>
__global__ void __launch_bounds__(kThreads)
rows_kernel(const SoftmaxParams prm) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ double sh_red[64];
    __shared__ float sh_stat[32 * 3];

    const int C = static_cast<int>(prm.C);
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    T *row = reinterpret_cast<T *>(base);
    const int tid = threadIdx.x;
    unsigned *status = reinterpret_cast<unsigned *>(prm.workspace) + 1;
    const T *logits = static_cast<const T *>(prm.logits);
    T *grads = static_cast<T *>(prm.grads);
    T *losses = static_cast<T *>(prm.losses);
    const T *gout = static_cast<const T *>(prm.grad_out);
    using V = Vec16<T>;
    constexpr int VN = V::N;
    const int nvec = C / VN;   // BULK guarantees C % VN == 0; otherwise a scalar tail follows

    if (BULK && tid == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    float gscale = 1.f;
    if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
    double acc_loss = 0.0, acc_cnt = 0.0;
    uint32_t phase = 0;
    const uint32_t row_bytes = uint32_t(C) * sizeof(T);

    for (int64_t r = blockIdx.x; r < prm.N; r += gridDim.x) {
        const T *src = logits + r * prm.C;
        if (BULK) {
            if (tid == 0) {
                mbar_expect_tx(&bar, row_bytes);
                // copies of at most 64 KiB each
                for (uint32_t off = 0; off < row_bytes; off += 65536u) {
                    const uint32_t nb = row_bytes - off < 65536u ? row_bytes - off : 65536u;
                    bulk_load_1d(reinterpret_cast<unsigned char *>(row) + off,
                                 reinterpret_cast<const unsigned char *>(src) + off, nb, &bar);
                }
            }
        } else {
            for (int j = tid; j < C; j += kThreads) row[j] = src[j];
        }
        const int64_t lb = prm.labels[r];
        const bool valid = lb != prm.ignore;
        float pscale = gscale;
        if (BWD && prm.grad_mode == 2) pscale *= to_f32(gout[r]);
        if (BULK) {
            const bool ok = mbar_wait_bounded(&bar, phase, prm.workspace ? status : nullptr);
            if (!__syncthreads_and(ok)) break;   // uniform decision: no thread is left behind
            phase ^= 1;
        } else {
            __syncthreads();
        }

        Stat1<KIND> s1;
        s1.init();
        for (int v = tid; v < nvec; v += kThreads) {
            const V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
            for (int i = 0; i < VN; ++i) s1.add(to_f32(xv.v[i]), v * VN + i == lb);
        }
        for (int j = nvec * VN + tid; j < C; j += kThreads) s1.add(to_f32(row[j]), j == lb);
        BlockStats<KIND>::combine(s1, sh_stat);

        Stat2<KIND> s2;
        s2.init();
        for (int v = tid; v < nvec; v += kThreads) {
            const V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
            for (int i = 0; i < VN; ++i) s2.add(to_f32(xv.v[i]), v * VN + i == lb, s1);
        }
        for (int j = nvec * VN + tid; j < C; j += kThreads) s2.add(to_f32(row[j]), j == lb, s1);
        BlockStats<KIND>::combine(s2, sh_stat);

        PixelFinal<KIND> fin;
        fin.finish(s1, s2, prm.k);

        if (!BWD) {
            if (tid == 0) {
                const float l = valid ? fin.loss : 0.f;
                if (losses) losses[r] = from_f32<T>(l);
                if (REDUCE && valid) {
                    acc_loss += double(l);
                    acc_cnt += 1.0;
                }
            }
            __syncthreads();   // row buffer free before the next copy lands
        } else {
            for (int v = tid; v < nvec; v += kThreads) {
                V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                for (int i = 0; i < VN; ++i)
                    xv.v[i] = from_f32<T>(valid ? fin.grad(to_f32(xv.v[i]), v * VN + i == lb, prm.k) * pscale : 0.f);
                *reinterpret_cast<V *>(row + v * VN) = xv;
            }
            for (int j = nvec * VN + tid; j < C; j += kThreads)
                row[j] = from_f32<T>(valid ? fin.grad(to_f32(row[j]), j == lb, prm.k) * pscale : 0.f);
            T *dst = grads + r * prm.C;
            if (BULK) {
                fence_proxy_async_smem();
                __syncthreads();
                if (tid == 0) {
                    for (uint32_t off = 0; off < row_bytes; off += 65536u) {
                        const uint32_t nb = row_bytes - off < 65536u ? row_bytes - off : 65536u;
                        bulk_store_1d(reinterpret_cast<unsigned char *>(dst) + off,
                                      reinterpret_cast<unsigned char *>(row) + off, nb);
                    }
                    bulk_commit();
                    bulk_wait_read_all();
                }
                __syncthreads();   // nobody may touch the row until the store has read it
            } else {
                __syncthreads();
                for (int j = tid; j < C; j += kThreads) dst[j] = row[j];
                __syncthreads();
            }
        }
    }
    if (BULK && BWD && tid == 0) bulk_wait_all();
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// ----------------------------------------------------------------- sweep regime
// One thread per pixel; channels are M elements apart.  Correct for every shape.

template <typename T, int KIND, bool BWD, bool REDUCE>
__global__ void __launch_bounds__(kThreads) sweep_kernel(const SoftmaxParams prm) {
    __shared__ double sh_red[64];
    const T *logits = static_cast<const T *>(prm.logits);
    T *grads = static_cast<T *>(prm.grads);
    T *losses = static_cast<T *>(prm.losses);
    const T *gout = static_cast<const T *>(prm.grad_out);
    const int C = static_cast<int>(prm.C);
    float gscale = 1.f;
    if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
    double acc_loss = 0.0, acc_cnt = 0.0;
    const int64_t P = prm.N * prm.M;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < P;
         i += int64_t(gridDim.x) * kThreads) {
        const int64_t n = i / prm.M, m = i % prm.M;
        const T *x = logits + n * prm.C * prm.M + m;
        const int64_t lb = prm.labels[i];
        const bool valid = lb != prm.ignore;
        if (!valid) {
            if (!BWD && losses) losses[i] = from_f32<T>(0.f);
            if (BWD) {
                T *g = grads + n * prm.C * prm.M + m;
                for (int j = 0; j < C; ++j) g[int64_t(j) * prm.M] = from_f32<T>(0.f);
            }
            continue;
        }
        Stat1<KIND> s1;
        s1.init();
        for (int j = 0; j < C; ++j) s1.add(to_f32(x[int64_t(j) * prm.M]), j == lb);
        Stat2<KIND> s2;
        s2.init();
        for (int j = 0; j < C; ++j) s2.add(to_f32(x[int64_t(j) * prm.M]), j == lb, s1);
        PixelFinal<KIND> fin;
        fin.finish(s1, s2, prm.k);
        if (!BWD) {
            if (losses) losses[i] = from_f32<T>(fin.loss);
            if (REDUCE) {
                acc_loss += double(fin.loss);
                acc_cnt += 1.0;
            }
        } else {
            float pscale = gscale;
            if (prm.grad_mode == 2) pscale *= to_f32(gout[i]);
            T *g = grads + n * prm.C * prm.M + m;
            for (int j = 0; j < C; ++j)
                g[int64_t(j) * prm.M] = from_f32<T>(fin.grad(to_f32(x[int64_t(j) * prm.M]), j == lb, prm.k) * pscale);
        }
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}


// Combine one float2 statistic across the KS channel slices of a tile (sum or max).
template <bool IS_MAX>
__device__ __forceinline__ float2 slice_combine(float2 v, float *area, int ks, int KS, int TP, int pix) {
    st_pair(area + ks * TP + pix, v);
    compute_sync(kTileCompute);
    float2 r = ld_pair(area + pix);
    for (int q = 1; q < KS; ++q) {
        const float2 o = ld_pair(area + q * TP + pix);
        r = IS_MAX ? max2(r, o) : add2(r, o);
    }
    return r;
}

// The first exchange of a tile also carries the slices' decision on the tile's arrival: its
// barrier is the AND-reducing one, so a timed-out wait is decided by all slices together
// without a barrier of its own.  `ok` comes back as the common decision.
__device__ __forceinline__ float2 slice_combine_max_first(float2 v, float *area, int ks, int KS, int TP, int pix,
                                                          bool &ok) {
    st_pair(area + ks * TP + pix, v);
    ok = compute_all(ok, kTileCompute);
    float2 r = ld_pair(area + pix);
    for (int q = 1; q < KS; ++q) r = max2(r, ld_pair(area + q * TP + pix));
    return r;
}

// Sums of two / three statistics across the slices with ONE barrier.
__device__ __forceinline__ void slice_sum2(float2 &a, float2 &b, float *area, int plane, int ks, int KS,
                                           int TP, int pix) {
    st_pair(area + ks * TP + pix, a);
    st_pair(area + plane + ks * TP + pix, b);
    compute_sync(kTileCompute);
    a = ld_pair(area + pix);
    b = ld_pair(area + plane + pix);
    for (int q = 1; q < KS; ++q) {
        a = add2(a, ld_pair(area + q * TP + pix));
        b = add2(b, ld_pair(area + plane + q * TP + pix));
    }
}
__device__ __forceinline__ void slice_sum3(float2 &a, float2 &b, float2 &c, float *area, int plane, int ks,
                                           int KS, int TP, int pix) {
    st_pair(area + ks * TP + pix, a);
    st_pair(area + plane + ks * TP + pix, b);
    st_pair(area + 2 * plane + ks * TP + pix, c);
    compute_sync(kTileCompute);
    a = ld_pair(area + pix);
    b = ld_pair(area + plane + pix);
    c = ld_pair(area + 2 * plane + pix);
    for (int q = 1; q < KS; ++q) {
        a = add2(a, ld_pair(area + q * TP + pix));
        b = add2(b, ld_pair(area + plane + q * TP + pix));
        c = add2(c, ld_pair(area + 2 * plane + q * TP + pix));
    }
}

template <typename T, int KIND, bool BWD, bool REDUCE>
__global__ void __launch_bounds__(kTileBlock)
tile_pair_kernel(const SoftmaxParams prm, const __grid_constant__ CUtensorMap map_in,
                 const __grid_constant__ CUtensorMap map_out) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    __shared__ double sh_red[64];
    __shared__ float s_lw2[KIND == kPC ? kPcMaxC : 1];    // kPC: log2 of the class weights

    const int TP = prm.TP, C = static_cast<int>(prm.C), NS = prm.stages;
    if constexpr (KIND == kPC) {
        // (a weight of 0 gives -inf: that class's exponential is 0, as w * e^x would be)
        for (int j = threadIdx.x; j < C; j += kTileBlock) s_lw2[j] = __log2f(__ldg(prm.chan_w + j));
    }
    const int NBX = prm.nbx, TPT = TP * NBX;        // a tile is NBX boxes of TP pixels side by side
    const int box_elems = prm.rows * TP;            // elements of one box in shared memory
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    // a stage = the logits tile followed by the tile's TP labels (both arrive by bulk copy) and
    // the tile's coordinates (image, first pixel), which the loader writes: the compute threads
    // then need no 64-bit division per tile
    const size_t label_off = (size_t(prm.rows) * TPT * sizeof(T) + 127) & ~size_t(127);
    const size_t coord_off = label_off + size_t(TPT) * sizeof(int64_t);
    const size_t stage_bytes = coord_off + 128;          // keeps every stage 128-byte aligned
    float *red = reinterpret_cast<float *>(base + NS * stage_bytes);   // [5 words][slices][TP]
    const int tid = threadIdx.x;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;
    const uint32_t box_bytes = uint32_t(prm.nbox) * prm.CB * TP * sizeof(T);   // one column of boxes

    pipe_init<kTileCompute, BWD>(bars, NS);
    const int64_t first = blockIdx.x, stride = gridDim.x;
    double acc_loss = 0.0, acc_cnt = 0.0;

    if (tid == kTileCompute) {
        int k = 0;
        for (int64_t t = first; t < prm.total_tiles; t += stride, ++k) {
            const int s = k % NS;
            if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, status)) break;
            const int64_t n = t / prm.tiles_per_image;
            const int64_t p0 = (t % prm.tiles_per_image) * TPT;
            T *stage = reinterpret_cast<T *>(base + s * stage_bytes);
            int64_t npix = prm.M - p0;
            if (npix > TPT) npix = TPT;
            const int nbx = int((npix + TP - 1) / TP);                       // boxes that hold pixels
            const uint32_t label_bytes = uint32_t(npix) * sizeof(int64_t);   // M % 4 == 0: multiple of 16
            *reinterpret_cast<int2 *>(base + s * stage_bytes + coord_off) = make_int2(int(n), int(p0));
            mbar_expect_tx(&bars.full[s], nbx * box_bytes + label_bytes);
            for (int bx = 0; bx < nbx; ++bx)
                for (int b = 0; b < prm.nbox; ++b)
                    tma_load_3d(stage + size_t(bx) * box_elems + size_t(b) * prm.CB * TP, &map_in,
                                int(p0) + bx * TP, b * prm.CB, int(n), &bars.full[s]);
            bulk_load_1d(base + s * stage_bytes + label_off, prm.labels + n * prm.M + p0, label_bytes, &bars.full[s]);
        }
    } else if (BWD && tid == kTileCompute + 32) {
        int k = 0;
        for (int64_t t = first; t < prm.total_tiles; t += stride, ++k) {
            const int s = k % NS;
            if (!mbar_wait_bounded(&bars.ready[s], (k / NS) & 1, status)) break;
            const int64_t n = t / prm.tiles_per_image;
            const int64_t p0 = (t % prm.tiles_per_image) * TPT;
            const T *stage = reinterpret_cast<const T *>(base + s * stage_bytes);
            int64_t npix = prm.M - p0;
            if (npix > TPT) npix = TPT;
            const int nbx = int((npix + TP - 1) / TP);
            for (int bx = 0; bx < nbx; ++bx)
                for (int b = 0; b < prm.nbox; ++b)
                    tma_store_3d(&map_out, int(p0) + bx * TP, b * prm.CB, int(n),
                                 stage + size_t(bx) * box_elems + size_t(b) * prm.CB * TP);
            bulk_commit();
            bulk_wait_read_all();
            mbar_arrive(&bars.empty[s]);
        }
        bulk_wait_all();
    } else if (tid < kTileCompute) {
        const int TPV = TPT >> 1;                     // pixel pairs per tile
        const int pg = tid % TPV, ks = tid / TPV, lane = tid & 31;
        const int KS = kTileCompute / TPV;
        const int pix = pg * 2;                       // first pixel of my pair inside the tile
        const int plane = KS * TPT;                   // floats per statistic word
        const int bxo = (pix / TP) * box_elems + (pix % TP);   // my pair's offset inside channel 0
        const int step = KS * TP;                     // tile elements between my channels
        const T *gout = static_cast<const T *>(prm.grad_out);
        T *losses = static_cast<T *>(prm.losses);
        const LossConsts kc = prm.k;
        float gscale = 1.f;
        // fused step: the divisor comes from the label count, which may still be running (the
        // loader warp above is already filling the ring)
        if (BWD && REDUCE) pdl_wait();
        if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
        float acc32 = 0.f;
        int cnt32 = 0;
        int k = 0;
        for (int64_t t = first; t < prm.total_tiles; t += stride, ++k) {
            const int s = k % NS;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, status);
            // A warp that owns whole pixel columns decides for itself.  Slices that exchange
            // statistics must give up together (their named barriers have no time limit): they
            // agree at the tile's first exchange, whose barrier carries the decision.
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (KS == 1 && !ok) break;
            const int2 coord = *reinterpret_cast<const int2 *>(base + s * stage_bytes + coord_off);
            const int64_t n = coord.x;
            const int64_t px0 = int64_t(coord.y) + pix;

            const int64_t *tile_labels = reinterpret_cast<const int64_t *>(base + s * stage_bytes + label_off);
            int lbi[2];
            bool inb[2];
            float2 psc = splat2(gscale);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                inb[i] = px0 + i < prm.M;
                const int64_t lb = inb[i] ? tile_labels[pix + i] : prm.ignore;
                const bool valid = inb[i] && lb != prm.ignore;
                lbi[i] = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
                if (BWD && prm.grad_mode == 2 && inb[i]) {
                    const float g = to_f32(gout[n * prm.M + px0 + i]);
                    if (i == 0) psc.x *= g; else psc.y *= g;
                }
            }
            // KS is a power of two: I visit the label channel of pixel i iff its low bits are ks
            const bool own0 = lbi[0] >= 0 && (lbi[0] & (KS - 1)) == ks;
            const bool own1 = lbi[1] >= 0 && (lbi[1] & (KS - 1)) == ks;

            T *tile = reinterpret_cast<T *>(base + s * stage_bytes);
            T *mine = tile + bxo + ks * TP;           // my first channel, my pixel pair

            if constexpr (KIND != kLMargin) {
                // ---- phase 1: max
                float2 m = splat2(kNegInf);
                {
                    const T *q = mine;
#pragma unroll 4
                    for (int j = ks; j < C; j += KS, q += step) m = max2(m, ld_pair(q));
                }
                if (KS > 1) {
                    m = slice_combine_max_first(m, red, ks, KS, TPT, pix, ok);
                    if (!ok) break;
                }
                // target logits.  Forward: slice 0 reads them (nobody writes the tile).  Backward
                // overwrites the tile with e^{x-m}, so the fused step (backward + loss sum) lets the
                // slice that owns the label channel read its logit ahead of its own sweep.
                float2 xl = splat2(0.f);
                if (!BWD && ks == 0) {
                    if (lbi[0] >= 0) xl.x = to_f32(tile[bxo + lbi[0] * TP]);
                    if (lbi[1] >= 0) xl.y = to_f32(tile[bxo + lbi[1] * TP + 1]);
                }
                if (BWD && REDUCE) {
                    if (own0) xl.x = to_f32(tile[bxo + lbi[0] * TP]);
                    if (own1) xl.y = to_f32(tile[bxo + lbi[1] * TP + 1]);
                }
                // ---- phase 2: sum of exponentials, sum of logits
                float2 sum, sx;
                {
                    const pk_t nml = pk2(mul2(m, splat2(-kLog2e))), l2e = psplat(kLog2e);
                    pk_t psum = psplat(0.f), psx = psplat(0.f);
                    T *q = mine;
#pragma unroll 4
                    for (int j = ks; j < C; j += KS, q += step) {
                        const pk_t x = ld_pk(q);
                        pk_t e;
                        if constexpr (KIND == kPC) e = pex2(pfma(x, l2e, padd(nml, psplat(s_lw2[j]))));   // w_j e^{x - m}
                        else e = pex2(pfma(x, l2e, nml));
                        psum = padd(psum, e);
                        if (KIND != kPC && (!BWD || REDUCE)) psx = padd(psx, x);    // (kPC: lb_neg = 0, the sum of logits is not used)
                        if (BWD) st_pk(q, e);
                    }
                    sum = upk2(psum);
                    sx = upk2(psx);
                }
                if (KS > 1) {
                    if (BWD && !REDUCE) sum = slice_combine<false>(sum, red + plane, ks, KS, TPT, pix);
                    else slice_sum2(sum, sx, red + plane, plane, ks, KS, TPT, pix);
                }
                if (!BWD) {
                    if (ks == 0) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (inb[i]) {
                                const float si = i ? sum.y : sum.x, mi = i ? m.y : m.x;
                                const float sxi = i ? sx.y : sx.x, xli = i ? xl.y : xl.x;
                                float l = 0.f;
                                if (lbi[i] != -1)
                                    l = kc.sumy * (mi + __logf(si)) - kc.lb_neg * sxi - (kc.lb_pos - kc.lb_neg) * xli;
                                if (losses) losses[n * prm.M + px0 + i] = from_f32<T>(l);
                                if (REDUCE && lbi[i] != -1) {
                                    acc32 += l;
                                    cnt32 += 1;
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.empty[s]);
                } else {
                    if (REDUCE) {
                        // fused step: the loss is a sum of terms, so slice 0 adds the softmax part
                        // and the label's owner the target part
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (ks == 0 && lbi[i] != -1) {
                                const float si = i ? sum.y : sum.x, mi = i ? m.y : m.x, sxi = i ? sx.y : sx.x;
                                acc32 += kc.sumy * (mi + __logf(si)) - kc.lb_neg * sxi;
                                cnt32 += 1;
                            }
                            if (i ? own1 : own0) acc32 -= (kc.lb_pos - kc.lb_neg) * (i ? xl.y : xl.x);
                        }
                    }
                    // ---- phase 3: g = (sumy * e / s - eps/C) * scale, then the target term
                    float2 a, b;
                    a.x = lbi[0] != -1 ? kc.sumy * __fdividef(psc.x, sum.x) : 0.f;
                    a.y = lbi[1] != -1 ? kc.sumy * __fdividef(psc.y, sum.y) : 0.f;
                    b.x = lbi[0] != -1 ? -kc.lb_neg * psc.x : 0.f;
                    b.y = lbi[1] != -1 ? -kc.lb_neg * psc.y : 0.f;
                    {
                        const pk_t pa = pk2(a), pb = pk2(b);
                        T *q = mine;
#pragma unroll 4
                        for (int j = ks; j < C; j += KS, q += step) st_pk(q, pfma(ld_pk(q), pa, pb));
                    }
                    const float dt = -(kc.lb_pos - kc.lb_neg);
                    if (own0) {
                        T *e = tile + bxo + lbi[0] * TP;
                        *e = from_f32<T>(to_f32(*e) + dt * psc.x);
                    }
                    if (own1) {
                        T *e = tile + bxo + lbi[1] * TP + 1;
                        *e = from_f32<T>(to_f32(*e) + dt * psc.y);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.ready[s]);
                }
            } else {
                // =============================== large margin ===============================
                // park the target logit out of the way of the max sweep
                float2 xl = splat2(0.f);
                if (own0) {
                    T *e = tile + bxo + lbi[0] * TP;
                    xl.x = to_f32(*e);
                    *e = from_f32<T>(sizeof(T) == 2 ? -65504.f : kNegInf);
                }
                if (own1) {
                    T *e = tile + bxo + lbi[1] * TP + 1;
                    xl.y = to_f32(*e);
                    *e = from_f32<T>(sizeof(T) == 2 ? -65504.f : kNegInf);
                }
                float2 m = splat2(kNegInf);       // max over j != lb
                {
                    const T *q = mine;
#pragma unroll 4
                    for (int j = ks; j < C; j += KS, q += step) m = max2(m, ld_pair(q));
                }
                if (KS > 1) {
                    // the owner publishes x_lb ahead of the max exchange's barrier; all read it after
                    if (own0) red[plane + pix] = xl.x;
                    if (own1) red[plane + pix + 1] = xl.y;
                    m = slice_combine_max_first(m, red, ks, KS, TPT, pix, ok);
                    if (!ok) break;
                    xl.x = lbi[0] >= 0 ? red[plane + pix] : 0.f;
                    xl.y = lbi[1] >= 0 ? red[plane + pix + 1] : 0.f;
                }
                // the target re-enters the sum sweep clamped to the off-target maximum
                const float2 cl = make_float2(fminf(xl.x, m.x), fminf(xl.y, m.y));
                if (own0) tile[bxo + lbi[0] * TP] = from_f32<T>(cl.x);
                if (own1) tile[bxo + lbi[1] * TP + 1] = from_f32<T>(cl.y);
                const float2 negm = make_float2(-m.x, -m.y);
                float2 sum, sde, sx;
                {
                    const pk_t pnegm = pk2(negm), l2e = psplat(kLog2e);
                    pk_t psum = psplat(0.f), psde = psplat(0.f), psx = psplat(0.f);
                    const T *q = mine;
#pragma unroll 4
                    for (int j = ks; j < C; j += KS, q += step) {
                        const pk_t x = ld_pk(q);
                        const pk_t d = padd(x, pnegm);
                        const pk_t e = pex2(pmul(d, l2e));
                        psum = padd(psum, e);
                        psde = pfma(d, e, psde);
                        psx = padd(psx, x);
                    }
                    sum = upk2(psum);
                    sde = upk2(psde);
                    sx = upk2(psx);
                }
                if (KS > 1) {
                    slice_sum3(sum, sde, sx, red + 2 * plane, plane, ks, KS, TPT, pix);
                }
                // per pixel: take the clamped target back out, then the closed forms
                float inv_s[2], rr[2], sqx[2], loss[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float mi = i ? m.y : m.x, xli = i ? xl.y : xl.x, ci = i ? cl.y : cl.x;
                    const float dc = ci - mi;
                    const float ec = ex2f(dc * kLog2e);
                    const float s_no = (i ? sum.y : sum.x) - ec;
                    const float sde_no = (i ? sde.y : sde.x) - dc * ec;
                    const float sd = ((i ? sx.y : sx.x) - ci) - float(C - 1) * mi;
                    inv_s[i] = __fdividef(1.f, s_no);
                    sqx[i] = sde_no * inv_s[i];
                    const float mm = fmaxf(mi, xli);
                    const float e_no = s_no * ex2f((mi - mm) * kLog2e);
                    const float e_lb = ex2f((xli - mm) * kLog2e);
                    const float s_all = e_no + e_lb;
                    rr[i] = __fdividef(e_no, s_all);
                    loss[i] = (mm + __logf(s_all)) - xli + kc.half_lam * (sqx[i] - kc.a * sd);
                }
                if (!BWD) {
                    if (ks == 0) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (inb[i]) {
                                const float l = lbi[i] != -1 ? loss[i] : 0.f;
                                if (losses) losses[n * prm.M + px0 + i] = from_f32<T>(l);
                                if (REDUCE && lbi[i] != -1) {
                                    acc32 += l;
                                    cnt32 += 1;
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.empty[s]);
                } else {
                    if (REDUCE && ks == 0) {          // fused step: every slice holds the same loss
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            if (lbi[i] != -1) {
                                acc32 += loss[i];
                                cnt32 += 1;
                            }
                        }
                    }
                    // g_j = scale * ( r*q + lam/2 * (q*(d + 1 - Sqx) - a) ),  q = e^d / s'
                    //     = q * (A + B*d) + Cc     with per-pixel A, B, Cc
                    float2 qa, qb, cc, qs;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const bool v = lbi[i] != -1;
                        const float sc = v ? (i ? psc.y : psc.x) : 0.f;
                        const float A = (rr[i] + kc.half_lam * (1.f - sqx[i])) * sc;
                        const float B = kc.half_lam * sc;
                        const float Cc = -kc.half_lam * kc.a * sc;
                        const float Q = v ? inv_s[i] : 0.f;
                        if (i == 0) { qa.x = A; qb.x = B; cc.x = Cc; qs.x = Q; }
                        else { qa.y = A; qb.y = B; cc.y = Cc; qs.y = Q; }
                    }
                    {
                        const pk_t pnegm = pk2(negm), l2e = psplat(kLog2e);
                        const pk_t pqa = pk2(qa), pqb = pk2(qb), pcc = pk2(cc), pqs = pk2(qs);
                        T *q = mine;
#pragma unroll 4
                        for (int j = ks; j < C; j += KS, q += step) {
                            const pk_t d = padd(ld_pk(q), pnegm);
                            const pk_t qq = pmul(pex2(pmul(d, l2e)), pqs);
                            st_pk(q, pfma(qq, pfma(pqb, d, pqa), pcc));
                        }
                    }
                    if (own0) tile[bxo + lbi[0] * TP] = from_f32<T>(-rr[0] * psc.x);
                    if (own1) tile[bxo + lbi[1] * TP + 1] = from_f32<T>(-rr[1] * psc.y);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.ready[s]);
                }
            }
            if (REDUCE && (k & 31) == 31) {
                acc_loss += double(acc32);
                acc_cnt += double(cnt32);
                acc32 = 0.f;
                cnt32 = 0;
            }
        }
        acc_loss += double(acc32);
        acc_cnt += double(cnt32);
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// ---------------------------------------------------- many channels, forward: chunked sweep
//
// Forward for class counts whose full tile does not fit beside a second one in shared memory
// (where tile_pair_kernel has to split the channels over warps and exchange statistics at
// block barriers).  Here a tile is 512 pixels wide and streams through the ring in chunks of
// kChunkCh channels; a thread owns two adjacent pixels over ALL channels and carries their
// running statistics in registers (online softmax: when the maximum moves, the sums are
// rescaled once per group of 8 channels), so there is no inter-warp exchange, no block
// barrier, and every element is read from shared memory once.
// Large margin leaves the target out of its sums: when the chunk with a pixel's label channel
// arrives, the thread saves that logit and overwrites it with a copy of another channel
// (channel 0, or 1 when the label is 0); the copy's terms are subtracted at the end, which
// cannot cancel (s' contains that channel's own term, and all d*e terms have one sign).
constexpr int kChunkCh = 16;
constexpr int kChunkGroup = 8;
constexpr int kChunkTP = 256;
constexpr int kChunkTile = 2 * kChunkTP;

struct ChunkLayout {
    uint32_t box_elems;     // elements of one box (kChunkCh x 256)
    uint32_t label_off, coord_off, stage_bytes;
};
template <typename T> __host__ __device__ inline ChunkLayout chunk_layout() {
    ChunkLayout l;
    l.box_elems = kChunkCh * kChunkTP;
    l.label_off = 2u * l.box_elems * uint32_t(sizeof(T));       // a multiple of 128
    l.coord_off = l.label_off + kChunkTile * 8u;
    l.stage_bytes = l.coord_off + 128u;
    return l;
}

template <typename T, int KIND, bool REDUCE>
__global__ void __launch_bounds__(kTileBlock)
tile_chunk_fwd_kernel(const SoftmaxParams prm, const __grid_constant__ CUtensorMap map_in) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    __shared__ double sh_red[64];
    const int C = static_cast<int>(prm.C), NS = prm.stages;
    const ChunkLayout lay = chunk_layout<T>();
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int tid = threadIdx.x;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;
    const int nchunks = (C + kChunkCh - 1) / kChunkCh;
    const int64_t tiles_per_image = (prm.M + kChunkTile - 1) / kChunkTile;
    const int64_t total_tiles = prm.N * tiles_per_image;
    const int64_t first = blockIdx.x, stride = gridDim.x;
    double acc_loss = 0.0, acc_cnt = 0.0;

    pipe_init<kTileCompute, false>(bars, NS);

    if (tid == kTileCompute) {
        int k = 0;
        for (int64_t t = first; t < total_tiles; t += stride) {
            const int64_t n = t / tiles_per_image;
            const int64_t p0 = (t % tiles_per_image) * kChunkTile;
            int64_t npix = prm.M - p0;
            if (npix > kChunkTile) npix = kChunkTile;
            const int nbx = int((npix + kChunkTP - 1) / kChunkTP);
            const uint32_t label_bytes = uint32_t(npix) * 8u;       // M % 4 == 0: a multiple of 16
            bool alive = true;
            for (int c = 0; c < nchunks && alive; ++c, ++k) {
                const int s = k % NS;
                if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, status)) {
                    alive = false;
                    break;
                }
                unsigned char *stage = base + size_t(s) * lay.stage_bytes;
                *reinterpret_cast<int4 *>(stage + lay.coord_off) = make_int4(int(n), int(p0), c, 0);
                mbar_expect_tx(&bars.full[s],
                               uint32_t(nbx) * lay.box_elems * uint32_t(sizeof(T)) + (c == 0 ? label_bytes : 0u));
                for (int bx = 0; bx < nbx; ++bx)
                    tma_load_3d(reinterpret_cast<T *>(stage) + size_t(bx) * lay.box_elems, &map_in,
                                int(p0) + bx * kChunkTP, c * kChunkCh, int(n), &bars.full[s]);
                if (c == 0) bulk_load_1d(stage + lay.label_off, prm.labels + n * prm.M + p0, label_bytes, &bars.full[s]);
            }
            if (!alive) break;
        }
    } else if (tid < kTileCompute) {
        const int lane = tid & 31;
        const int pix = tid * 2;
        const int bxo = (pix / kChunkTP) * int(lay.box_elems) + (pix % kChunkTP);
        T *losses = static_cast<T *>(prm.losses);
        const LossConsts kc = prm.k;
        float acc32 = 0.f;
        int cnt32 = 0;
        int k = 0;
        bool alive = true;
        for (int64_t t = first; t < total_tiles && alive; t += stride) {
            int lbi[2] = {-1, -1};
            bool inb[2] = {false, false};
            int64_t n = 0, px0 = 0;
            float2 m = splat2(kNegInf), sum = splat2(0.f), sde = splat2(0.f), sx = splat2(0.f);
            float2 xl = splat2(0.f), xo = splat2(0.f);
            for (int c = 0; c < nchunks; ++c, ++k) {
                const int s = k % NS;
                bool ok = true;
                if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, status);
                if (!__shfl_sync(0xffffffffu, ok, 0)) {
                    alive = false;
                    break;
                }
                unsigned char *stage = base + size_t(s) * lay.stage_bytes;
                T *mine = reinterpret_cast<T *>(stage) + bxo;
                const int c0 = c * kChunkCh;
                const int nch = min(kChunkCh, C - c0);
                if (c == 0) {
                    const int4 coord = *reinterpret_cast<const int4 *>(stage + lay.coord_off);
                    n = coord.x;
                    px0 = int64_t(coord.y) + pix;
                    const int64_t *tile_labels = reinterpret_cast<const int64_t *>(stage + lay.label_off);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        inb[i] = px0 + i < prm.M;
                        const int64_t lb = inb[i] ? tile_labels[pix + i] : prm.ignore;
                        const bool valid = inb[i] && lb != prm.ignore;
                        lbi[i] = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
                    }
                    if (KIND == kLMargin) {
                        // the stand-in for the target: channel 0, or 1 when the label is 0
                        xo.x = to_f32(mine[(lbi[0] == 0 ? 1 : 0) * kChunkTP]);
                        xo.y = to_f32(mine[(lbi[1] == 0 ? 1 : 0) * kChunkTP + 1]);
                    }
                }
                // the label channel of my pixels, if it is in this chunk
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j = lbi[i] - c0;
                    if (lbi[i] >= 0 && j >= 0 && j < kChunkCh) {
                        T *e = mine + j * kChunkTP + i;
                        if (i == 0) xl.x = to_f32(*e); else xl.y = to_f32(*e);
                        if (KIND == kLMargin) *e = from_f32<T>(i == 0 ? xo.x : xo.y);
                    }
                }
                for (int g0 = 0; g0 < nch; g0 += kChunkGroup) {
                    const int ng = min(kChunkGroup, nch - g0);
                    pk_t x[kChunkGroup];
                    float2 mn = m;
#pragma unroll
                    for (int q = 0; q < kChunkGroup; ++q) {
                        // (channels past the end of the group repeat its first one: harmless for
                        // the maximum, and the sums below stop at ng)
                        x[q] = ld_pk(mine + (g0 + (q < ng ? q : 0)) * kChunkTP);
                        mn = max2(mn, upk2(x[q]));
                    }
                    // rescale what has been summed so far to the new maximum
                    const float2 dm = make_float2(m.x - mn.x, m.y - mn.y);
                    const float2 r = ex2_2(mul2(dm, splat2(kLog2e)));
                    if (KIND == kLMargin) sde = mul2(r, fma2(dm, sum, sde));
                    sum = mul2(sum, r);
                    m = mn;
                    const pk_t nml = pk2(mul2(mn, splat2(-kLog2e))), l2e = psplat(kLog2e), negm = pk2(make_float2(-mn.x, -mn.y));
                    pk_t psum = pk2(sum), psde = pk2(sde), psx = pk2(sx);
#pragma unroll
                    for (int q = 0; q < kChunkGroup; ++q) {
                        if (q < ng) {
                            const pk_t e = pex2(pfma(x[q], l2e, nml));
                            psum = padd(psum, e);
                            if (KIND == kLMargin) psde = pfma(padd(x[q], negm), e, psde);
                            psx = padd(psx, x[q]);
                        }
                    }
                    sum = upk2(psum);
                    sde = upk2(psde);
                    sx = upk2(psx);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.empty[s]);
            }
            if (!alive) break;
            // ---- per pixel: closed forms
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (!inb[i]) continue;
                const float mi = i ? m.y : m.x, si = i ? sum.y : sum.x, sxi = i ? sx.y : sx.x;
                const float xli = lbi[i] >= 0 ? (i ? xl.y : xl.x) : 0.f;
                float l = 0.f;
                float4 st = make_float4(mi, 0.f, 0.f, 0.f);
                if (lbi[i] != -1) {
                    if (KIND == kLSR) {
                        l = kc.sumy * (mi + __logf(si)) - kc.lb_neg * sxi - (kc.lb_pos - kc.lb_neg) * xli;
                        st.y = __fdividef(1.f, si);
                    } else {
                        // take the stand-in's terms back out (no label channel: nothing was replaced)
                        const bool repl = lbi[i] >= 0;
                        const float ci = i ? xo.y : xo.x;
                        const float dc = ci - mi;
                        const float ec = repl ? ex2f(dc * kLog2e) : 0.f;
                        const float s_no = si - ec;
                        const float sde_no = (i ? sde.y : sde.x) - (repl ? dc * ec : 0.f);
                        const float nother = repl ? float(C - 1) : float(C);
                        const float sd = (sxi - (repl ? ci : 0.f)) - nother * mi;
                        const float inv_s = __fdividef(1.f, s_no);
                        const float sqx = sde_no * inv_s;
                        const float mm = fmaxf(mi, xli);
                        const float e_no = s_no * ex2f((mi - mm) * kLog2e);
                        const float e_lb = repl ? ex2f((xli - mm) * kLog2e) : 0.f;
                        const float s_all = e_no + e_lb;
                        l = (mm + __logf(s_all)) - xli + kc.half_lam * (sqx - kc.a * sd);
                        const float rr = __fdividef(e_no, s_all);
                        st.y = inv_s;
                        st.z = rr + kc.half_lam * (1.f - sqx);
                        st.w = rr;
                    }
                }
                if (prm.stats) prm.stats[n * prm.M + px0 + i] = st;
                if (losses) losses[n * prm.M + px0 + i] = from_f32<T>(l);
                if (REDUCE && lbi[i] != -1) {
                    acc32 += l;
                    cnt32 += 1;
                }
            }
            if (REDUCE && cnt32 >= 32) {
                acc_loss += double(acc32);
                acc_cnt += double(cnt32);
                acc32 = 0.f;
                cnt32 = 0;
            }
        }
        acc_loss += double(acc32);
        acc_cnt += double(cnt32);
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// ---------------------------------------------- many channels, backward from saved statistics
//
// The chunked forward leaves four floats per pixel (maximum, 1 / sum and, for large margin, the
// two per-pixel coefficients of its gradient).  With them every gradient element depends on its
// own logit only, so backward is one more streaming pass in the same chunks: TMA in, gradient
// in place, TMA out -- no resident tile, no slices, no block barrier.
//   label smooth : g_j = (sumy * e^{x_j - m} / s - eps/C) * sc,            target: - (1 - eps - eps/C) * sc
//   large margin : g_j = q_j * (A + lam/2 * d_j) * sc - lam/2 * a * sc,    target: - r * sc
//                  q_j = e^{d_j} / s',  d_j = x_j - m',  A = r + lam/2 * (1 - sum q d)
struct ChunkBwdLayout {
    uint32_t box_elems, label_off, stats_off, coord_off, stage_bytes;
};
template <typename T> __host__ __device__ inline ChunkBwdLayout chunk_bwd_layout() {
    ChunkBwdLayout l;
    l.box_elems = kChunkCh * kChunkTP;
    l.label_off = 2u * l.box_elems * uint32_t(sizeof(T));
    l.stats_off = l.label_off + kChunkTile * 8u;
    l.coord_off = l.stats_off + kChunkTile * 16u;
    l.stage_bytes = l.coord_off + 128u;
    return l;
}

template <typename T, int KIND>
__global__ void __launch_bounds__(kTileBlock)
tile_chunk_bwd_kernel(const SoftmaxParams prm, const __grid_constant__ CUtensorMap map_in,
                      const __grid_constant__ CUtensorMap map_out) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    const int C = static_cast<int>(prm.C), NS = prm.stages;
    const ChunkBwdLayout lay = chunk_bwd_layout<T>();
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int tid = threadIdx.x;
    unsigned *status = nullptr;                       // backward has no workspace: waits are bounded only
    const int nchunks = (C + kChunkCh - 1) / kChunkCh;
    const int64_t tiles_per_image = (prm.M + kChunkTile - 1) / kChunkTile;
    const int64_t total_tiles = prm.N * tiles_per_image;
    const int64_t first = blockIdx.x, stride = gridDim.x;

    pipe_init<kTileCompute, true>(bars, NS);

    if (tid == kTileCompute) {
        int k = 0;
        bool alive = true;
        for (int64_t t = first; t < total_tiles && alive; t += stride) {
            const int64_t n = t / tiles_per_image;
            const int64_t p0 = (t % tiles_per_image) * kChunkTile;
            int64_t npix = prm.M - p0;
            if (npix > kChunkTile) npix = kChunkTile;
            const int nbx = int((npix + kChunkTP - 1) / kChunkTP);
            const uint32_t label_bytes = uint32_t(npix) * 8u, stats_bytes = uint32_t(npix) * 16u;
            for (int c = 0; c < nchunks; ++c, ++k) {
                const int s = k % NS;
                if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, status)) {
                    alive = false;
                    break;
                }
                unsigned char *stage = base + size_t(s) * lay.stage_bytes;
                *reinterpret_cast<int4 *>(stage + lay.coord_off) = make_int4(int(n), int(p0), c, nbx);
                mbar_expect_tx(&bars.full[s], uint32_t(nbx) * lay.box_elems * uint32_t(sizeof(T)) +
                                                  (c == 0 ? label_bytes + stats_bytes : 0u));
                for (int bx = 0; bx < nbx; ++bx)
                    tma_load_3d(reinterpret_cast<T *>(stage) + size_t(bx) * lay.box_elems, &map_in,
                                int(p0) + bx * kChunkTP, c * kChunkCh, int(n), &bars.full[s]);
                if (c == 0) {
                    bulk_load_1d(stage + lay.label_off, prm.labels + n * prm.M + p0, label_bytes, &bars.full[s]);
                    bulk_load_1d(stage + lay.stats_off, prm.stats + n * prm.M + p0, stats_bytes, &bars.full[s]);
                }
            }
        }
    } else if (tid == kTileCompute + 32) {
        const int64_t total_chunks = ((total_tiles - first + stride - 1) / stride) * nchunks;
        for (int64_t k = 0; k < total_chunks; ++k) {
            const int s = int(k % NS);
            if (!mbar_wait_bounded(&bars.ready[s], uint32_t(k / NS) & 1u, status)) break;
            const unsigned char *stage = base + size_t(s) * lay.stage_bytes;
            const int4 coord = *reinterpret_cast<const int4 *>(stage + lay.coord_off);
            for (int bx = 0; bx < coord.w; ++bx)
                tma_store_3d(&map_out, coord.y + bx * kChunkTP, coord.z * kChunkCh, coord.x,
                             reinterpret_cast<const T *>(stage) + size_t(bx) * lay.box_elems);
            bulk_commit();
            bulk_wait_read_all();
            mbar_arrive(&bars.empty[s]);
        }
        bulk_wait_all();
    } else if (tid < kTileCompute) {
        const int lane = tid & 31;
        const int pix = tid * 2;
        const int bxo = (pix / kChunkTP) * int(lay.box_elems) + (pix % kChunkTP);
        const T *gout = static_cast<const T *>(prm.grad_out);
        const LossConsts kc = prm.k;
        const float gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
        int k = 0;
        bool alive = true;
        for (int64_t t = first; t < total_tiles && alive; t += stride) {
            int lbi[2] = {-1, -1};
            pk_t pa = 0, pb = 0, pc = 0, pm = 0;       // per-pixel coefficients, packed
            float tgt[2] = {0.f, 0.f};                 // value of the target element
            for (int c = 0; c < nchunks; ++c, ++k) {
                const int s = k % NS;
                bool ok = true;
                if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, status);
                if (!__shfl_sync(0xffffffffu, ok, 0)) {
                    alive = false;
                    break;
                }
                unsigned char *stage = base + size_t(s) * lay.stage_bytes;
                T *mine = reinterpret_cast<T *>(stage) + bxo;
                const int c0 = c * kChunkCh;
                const int nch = min(kChunkCh, C - c0);
                if (c == 0) {
                    const int4 coord = *reinterpret_cast<const int4 *>(stage + lay.coord_off);
                    const int64_t n = coord.x, px0 = int64_t(coord.y) + pix;
                    const int64_t *tile_labels = reinterpret_cast<const int64_t *>(stage + lay.label_off);
                    const float4 *tile_stats = reinterpret_cast<const float4 *>(stage + lay.stats_off);
                    float a2[2], b2[2], c2[2], m2[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const bool inb = px0 + i < prm.M;
                        const int64_t lb = inb ? tile_labels[pix + i] : prm.ignore;
                        const bool valid = inb && lb != prm.ignore;
                        lbi[i] = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
                        float sc = valid ? gscale : 0.f;
                        if (valid && prm.grad_mode == 2) sc *= to_f32(gout[n * prm.M + px0 + i]);
                        const float4 st = inb ? tile_stats[pix + i] : make_float4(0.f, 0.f, 0.f, 0.f);
                        m2[i] = st.x;
                        if (KIND == kLSR) {
                            // g = e * (sumy * sc / s) - eps/C * sc
                            a2[i] = kc.sumy * sc * st.y;
                            b2[i] = -kc.lb_neg * sc;
                            c2[i] = 0.f;
                            tgt[i] = -(kc.lb_pos - kc.lb_neg) * sc;            // added to the target element
                        } else {
                            // g = (e / s') * (A sc + lam/2 sc d) - lam/2 a sc
                            a2[i] = st.z * sc * st.y;
                            b2[i] = kc.half_lam * sc * st.y;
                            c2[i] = -kc.half_lam * kc.a * sc;
                            tgt[i] = -st.w * sc;                               // replaces the target element
                        }
                    }
                    pa = pk2(make_float2(a2[0], a2[1]));
                    pb = pk2(make_float2(b2[0], b2[1]));
                    pc = pk2(make_float2(c2[0], c2[1]));
                    pm = pk2(make_float2(m2[0], m2[1]));
                }
                {
                    const pk_t l2e = psplat(kLog2e);
                    const pk_t nml = pmul(pm, psplat(-kLog2e)), negm = pmul(pm, psplat(-1.f));
                    T *q = mine;
#pragma unroll 4
                    for (int j = 0; j < nch; ++j, q += kChunkTP) {
                        const pk_t x = ld_pk(q);
                        const pk_t e = pex2(pfma(x, l2e, nml));
                        if (KIND == kLSR) st_pk(q, pfma(e, pa, pb));
                        else st_pk(q, pfma(e, pfma(pb, padd(x, negm), pa), pc));
                    }
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j = lbi[i] - c0;
                    if (lbi[i] >= 0 && j >= 0 && j < kChunkCh) {
                        T *e = mine + j * kChunkTP + i;
                        *e = from_f32<T>(KIND == kLSR ? to_f32(*e) + tgt[i] : tgt[i]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.ready[s]);
            }
        }
    }
}

// Pair q of a 16-byte register vector as two floats, and back.
__device__ __forceinline__ float2 pair_of(const Vec16<float> &v, int q) { return make_float2(v.v[2 * q], v.v[2 * q + 1]); }
__device__ __forceinline__ float2 pair_of(const Vec16<__half> &v, int q) {
    return __half22float2(__halves2half2(v.v[2 * q], v.v[2 * q + 1]));
}
__device__ __forceinline__ float2 pair_of(const Vec16<__nv_bfloat16> &v, int q) {
    return make_float2(__bfloat162float(v.v[2 * q]), __bfloat162float(v.v[2 * q + 1]));
}
__device__ __forceinline__ void set_pair(Vec16<float> &v, int q, float2 f) {
    v.v[2 * q] = f.x;
    v.v[2 * q + 1] = f.y;
}
__device__ __forceinline__ void set_pair(Vec16<__half> &v, int q, float2 f) {
    const __half2 h = __float22half2_rn(f);
    v.v[2 * q] = __low2half(h);
    v.v[2 * q + 1] = __high2half(h);
}
__device__ __forceinline__ void set_pair(Vec16<__nv_bfloat16> &v, int q, float2 f) {
    v.v[2 * q] = __float2bfloat16_rn(f.x);
    v.v[2 * q + 1] = __float2bfloat16_rn(f.y);
}

// Reduce two values over the first n threads of the block (sum or max); every thread gets
// the result.  sh holds 2 floats per warp.  Two named-barrier syncs.
template <bool IS_MAX>
__device__ __forceinline__ void block_reduce2(float &a, float &b, float *sh, int n) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        a = IS_MAX ? fmaxf(a, oa) : a + oa;
        b = IS_MAX ? fmaxf(b, ob) : b + ob;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = n >> 5;
    compute_sync(n);                     // previous readers of sh are done
    if (lane == 0) {
        sh[2 * warp] = a;
        sh[2 * warp + 1] = b;
    }
    compute_sync(n);
    a = sh[0];
    b = sh[1];
    for (int w = 1; w < nwarp; ++w) {
        a = IS_MAX ? fmaxf(a, sh[2 * w]) : a + sh[2 * w];
        b = IS_MAX ? fmaxf(b, sh[2 * w + 1]) : b + sh[2 * w + 1];
    }
}

constexpr int kRowsCompute = 448;   // 14 compute warps + loader + storer = 16 warps: three blocks per SM at 40 registers
constexpr int kRowsBlock = kRowsCompute + 64;

// (register cap = the blocks per SM the launch asks for: backward and the fused step, BWD && REDUCE,
// run three per SM; uncapped, the fused step took 56 registers and fell to two blocks)
template <typename T, int KIND, bool BWD, bool REDUCE>
__global__ void __launch_bounds__(kRowsBlock, BWD ? 3 : 2)
rows_pipe_kernel(const SoftmaxParams prm) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    __shared__ double sh_red[64];
    __shared__ float sh_stat[32 * 3];
    // fused step: the loss sums live in shared memory (thread 0 alone touches them) and the label's
    // owner hands its logit to thread 0 through sh_xl, so the row loop carries no extra registers
    __shared__ double sh_acc[2];
    __shared__ float sh_xl;

    const int C = static_cast<int>(prm.C), NS = prm.stages;
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const size_t stage_bytes = (size_t(C) * sizeof(T) + 127) & ~size_t(127);
    if (BWD && REDUCE && threadIdx.x == 0) {
        sh_acc[0] = 0.0;
        sh_acc[1] = 0.0;
    }
    const int tid = threadIdx.x;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;
    const uint32_t row_bytes = uint32_t(C) * sizeof(T);
    using V = Vec16<T>;
    constexpr int VN = V::N;
    const int nvec = C / VN;

    pipe_init<kRowsCompute, BWD>(bars, NS);
    const int64_t first = blockIdx.x, stride = gridDim.x;
    double acc_loss = 0.0, acc_cnt = 0.0;

    if (tid == kRowsCompute) {
        int k = 0;
        for (int64_t r = first; r < prm.N; r += stride, ++k) {
            const int s = k % NS;
            if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, status)) break;
            unsigned char *stage = base + s * stage_bytes;
            const unsigned char *src = static_cast<const unsigned char *>(prm.logits) + r * prm.C * sizeof(T);
            mbar_expect_tx(&bars.full[s], row_bytes);
            for (uint32_t off = 0; off < row_bytes; off += 65536u) {
                const uint32_t nb = row_bytes - off < 65536u ? row_bytes - off : 65536u;
                bulk_load_1d(stage + off, src + off, nb, &bars.full[s]);
            }
        }
    } else if (BWD && tid == kRowsCompute + 32) {
        int k = 0;
        for (int64_t r = first; r < prm.N; r += stride, ++k) {
            const int s = k % NS;
            if (!mbar_wait_bounded(&bars.ready[s], (k / NS) & 1, status)) break;
            const unsigned char *stage = base + s * stage_bytes;
            unsigned char *dst = static_cast<unsigned char *>(prm.grads) + r * prm.C * sizeof(T);
            for (uint32_t off = 0; off < row_bytes; off += 65536u) {
                const uint32_t nb = row_bytes - off < 65536u ? row_bytes - off : 65536u;
                bulk_store_1d(dst + off, stage + off, nb);
            }
            bulk_commit();
            bulk_wait_read_all();
            mbar_arrive(&bars.empty[s]);
        }
        bulk_wait_all();
    } else if (tid < kRowsCompute) {
        // ---- compute: 16-byte shared loads, pairs of elements through packed fp32x2 math, no
        // per-element label compare (the thread that owns the label's vector edits that element).
        constexpr int NP = VN / 2;                    // pairs per 16-byte vector
        const int lane = tid & 31;
        const T *gout = static_cast<const T *>(prm.grad_out);
        T *losses = static_cast<T *>(prm.losses);
        const LossConsts kc = prm.k;
        float gscale = 1.f;
        if (BWD && REDUCE) pdl_wait();          // (see tile_pair_kernel)
        if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
        int k = 0;
        for (int64_t r = first; r < prm.N; r += stride, ++k) {
            const int s = k % NS;
            const int64_t lb = __ldg(prm.labels + r);
            const bool valid = lb != prm.ignore;
            const int lbi = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
            float psc = gscale;
            if (BWD && prm.grad_mode == 2) psc *= to_f32(gout[r]);
            const bool own = lbi >= 0 && (lbi / VN) % kRowsCompute == tid;   // my loop visits element lbi
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, status);
            if (!compute_all(ok, kRowsCompute)) break;
            T *row = reinterpret_cast<T *>(base + s * stage_bytes);

            float xl = KIND == kLMargin ? kNegInf : 0.f;
            if (KIND == kLMargin) {
                // park the target logit out of the way of the max sweep
                if (own) {
                    xl = to_f32(row[lbi]);
                    row[lbi] = from_f32<T>(sizeof(T) == 2 ? -65504.f : kNegInf);
                }
            } else if (!BWD && tid == 0 && lbi >= 0) {
                xl = to_f32(row[lbi]);
            } else if (BWD && REDUCE && own) {
                sh_xl = to_f32(row[lbi]);    // fused step: read by the thread that will overwrite it
            }
            // ---- phase 1: maximum (half rows: on the packed halves, exact and four values per
            // instruction-pair instead of a conversion and a compare each)
            float2 m2 = splat2(kNegInf);
            if constexpr (std::is_same<T, __half>::value) {
                __half2 hm = __float2half2_rn(-65504.f);
                for (int v = tid; v < nvec; v += kRowsCompute) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(row + v * VN);
                    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
                    hm = __hmax2(__hmax2(hm, h[0]), __hmax2(h[1], __hmax2(h[2], h[3])));
                }
                m2 = __half22float2(hm);
            } else {
                for (int v = tid; v < nvec; v += kRowsCompute) {
                    const V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                    for (int q = 0; q < NP; ++q) m2 = max2(m2, pair_of(xv, q));
                }
            }
            float red1[2] = {fmaxf(m2.x, m2.y), xl};
            if (KIND == kLMargin) {
                // max and the owner's x_lb (others hold 0) in one exchange
                block_reduce2<true>(red1[0], red1[1], sh_stat, kRowsCompute);
                xl = lbi >= 0 ? red1[1] : 0.f;
            } else {
                float dummy = 0.f;
                block_reduce2<true>(red1[0], dummy, sh_stat, kRowsCompute);
                // after that exchange's barrier, and before the next one lets an owner write again
                if (BWD && REDUCE && tid == 0 && lbi >= 0) xl = sh_xl;
            }
            const float m = red1[0];

            if constexpr (KIND == kLSR) {
                // ---- phase 2: sum of exponentials (kept in the row for backward), sum of logits
                const float2 nml = splat2(-m * kLog2e);
                float2 sum2 = splat2(0.f), sx2 = splat2(0.f);
                for (int v = tid; v < nvec; v += kRowsCompute) {
                    V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        const float2 x = pair_of(xv, q);
                        const float2 e = ex2_2(fma2(x, splat2(kLog2e), nml));
                        sum2 = add2(sum2, e);
                        if (!BWD || REDUCE) sx2 = add2(sx2, x);
                        if (BWD) set_pair(xv, q, e);
                    }
                    if (BWD) *reinterpret_cast<V *>(row + v * VN) = xv;
                }
                float ssum = sum2.x + sum2.y, ssx = sx2.x + sx2.y;
                block_reduce2<false>(ssum, ssx, sh_stat, kRowsCompute);
                if (!BWD) {
                    if (tid == 0) {
                        float l = 0.f;
                        if (lbi != -1)
                            l = kc.sumy * (m + __logf(ssum)) - kc.lb_neg * ssx - (kc.lb_pos - kc.lb_neg) * xl;
                        if (losses) losses[r] = from_f32<T>(l);
                        if (REDUCE && lbi != -1) {
                            acc_loss += double(l);
                            acc_cnt += 1.0;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.empty[s]);
                } else {
                    if (REDUCE) {
                        // fused step
                        if (tid == 0 && lbi != -1) {
                            sh_acc[0] += double(kc.sumy * (m + __logf(ssum)) - kc.lb_neg * ssx -
                                                (kc.lb_pos - kc.lb_neg) * xl);
                            sh_acc[1] += 1.0;
                        }
                    }
                    const float2 a = splat2(lbi != -1 ? kc.sumy * __fdividef(psc, ssum) : 0.f);
                    const float2 b = splat2(lbi != -1 ? -kc.lb_neg * psc : 0.f);
                    for (int v = tid; v < nvec; v += kRowsCompute) {
                        V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                        for (int q = 0; q < NP; ++q) set_pair(xv, q, fma2(pair_of(xv, q), a, b));
                        *reinterpret_cast<V *>(row + v * VN) = xv;
                    }
                    if (own) row[lbi] = from_f32<T>(to_f32(row[lbi]) - (kc.lb_pos - kc.lb_neg) * psc);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.ready[s]);
                }
            } else {
                // =============================== large margin ===============================
                // the target re-enters the sum sweep clamped to the off-target maximum
                const float cl = fminf(xl, m);
                if (own) row[lbi] = from_f32<T>(cl);
                const float2 negm = splat2(-m);
                float2 sum2 = splat2(0.f), sde2 = splat2(0.f), sx2 = splat2(0.f);
                for (int v = tid; v < nvec; v += kRowsCompute) {
                    const V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        const float2 x = pair_of(xv, q);
                        const float2 d = add2(x, negm);
                        const float2 e = ex2_2(mul2(d, splat2(kLog2e)));
                        sum2 = add2(sum2, e);
                        sde2 = fma2(d, e, sde2);
                        sx2 = add2(sx2, x);
                    }
                }
                float ssum = sum2.x + sum2.y, ssde = sde2.x + sde2.y, ssx = sx2.x + sx2.y;
                block_reduce2<false>(ssum, ssde, sh_stat, kRowsCompute);
                float dummy = 0.f;
                block_reduce2<false>(ssx, dummy, sh_stat, kRowsCompute);
                // take the clamped target back out, then the closed forms
                const float dc = cl - m;
                const float ec = ex2f(dc * kLog2e);
                const float s_no = ssum - ec;
                const float sde_no = ssde - dc * ec;
                const float sd = (ssx - cl) - float(C - 1) * m;
                const float inv_s = __fdividef(1.f, s_no);
                const float sqx = sde_no * inv_s;
                const float mm = fmaxf(m, xl);
                const float e_no = s_no * ex2f((m - mm) * kLog2e);
                const float e_lb = ex2f((xl - mm) * kLog2e);
                const float s_all = e_no + e_lb;
                const float rr = __fdividef(e_no, s_all);
                if (!BWD) {
                    if (tid == 0) {
                        float l = 0.f;
                        if (lbi != -1) l = (mm + __logf(s_all)) - xl + kc.half_lam * (sqx - kc.a * sd);
                        if (losses) losses[r] = from_f32<T>(l);
                        if (REDUCE && lbi != -1) {
                            acc_loss += double(l);
                            acc_cnt += 1.0;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.empty[s]);
                } else {
                    if (REDUCE && tid == 0 && lbi != -1) {      // fused step
                        sh_acc[0] += double((mm + __logf(s_all)) - xl + kc.half_lam * (sqx - kc.a * sd));
                        sh_acc[1] += 1.0;
                    }
                    const float sc = lbi != -1 ? psc : 0.f;
                    const float2 qa = splat2((rr + kc.half_lam * (1.f - sqx)) * sc);
                    const float2 qb = splat2(kc.half_lam * sc);
                    const float2 cc = splat2(-kc.half_lam * kc.a * sc);
                    const float2 qs = splat2(lbi != -1 ? inv_s : 0.f);
                    for (int v = tid; v < nvec; v += kRowsCompute) {
                        V xv = *reinterpret_cast<const V *>(row + v * VN);
#pragma unroll
                        for (int q = 0; q < NP; ++q) {
                            const float2 d = add2(pair_of(xv, q), negm);
                            const float2 qq = mul2(ex2_2(mul2(d, splat2(kLog2e))), qs);
                            set_pair(xv, q, fma2(qq, fma2(qb, d, qa), cc));
                        }
                        *reinterpret_cast<V *>(row + v * VN) = xv;
                    }
                    if (own) row[lbi] = from_f32<T>(-rr * psc);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.ready[s]);
                }
            }
        }
    }
    if (BWD && REDUCE && threadIdx.x == 0) {
        acc_loss = sh_acc[0];
        acc_cnt = sh_acc[1];
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// -------------------------------------------------------------------- dispatch

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------- rows regime, forward: one warp per row
//
// Forward for M == 1 and long rows.  Every warp streams its own rows through its own small
// ring of shared-memory stages (lane 0 issues the bulk copies and re-arms a stage as soon as
// the warp has read it), each lane keeps running statistics of the vectors it reads (online
// softmax: one rescale per chunk), and the 32 lanes combine them with shuffles at the end of
// a row.  Warps never wait for each other: no block barrier, no whole-row residency (so no
// limit on the row length), and each element is read from shared memory once.
constexpr int kWarpRowWarps = 8;                         // warps per block
constexpr int kWarpRowVecs = 8;                          // 16-byte vectors per lane and chunk
constexpr int kWarpRowChunk = 32 * 16 * kWarpRowVecs;    // 4 KB
constexpr int kWarpRowStages = 2;

template <typename T, int KIND, bool REDUCE>
__global__ void __launch_bounds__(kWarpRowWarps * 32)
rows_warp_fwd_kernel(const SoftmaxParams prm) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char(*ring)[kWarpRowStages][kWarpRowChunk] = reinterpret_cast<unsigned char(*)[kWarpRowStages][kWarpRowChunk]>(
        smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u));
    __shared__ __align__(8) uint64_t full[kWarpRowWarps][kWarpRowStages];
    __shared__ double sh_red[64];
    using V = Vec16<T>;
    constexpr int VN = V::N, NP = VN / 2, NS = kWarpRowStages;
    const int C = static_cast<int>(prm.C);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;
    const uint32_t row_bytes = uint32_t(C) * sizeof(T);                 // a multiple of 16
    const int nchunks = int((row_bytes + kWarpRowChunk - 1) / kWarpRowChunk);
    const int64_t gw = int64_t(blockIdx.x) * kWarpRowWarps + warp, nw = int64_t(gridDim.x) * kWarpRowWarps;
    const int64_t my_rows = gw < prm.N ? (prm.N - gw + nw - 1) / nw : 0;
    const int64_t my_chunks = my_rows * nchunks;
    T *losses = static_cast<T *>(prm.losses);
    const LossConsts kc = prm.k;
    double acc_loss = 0.0, acc_cnt = 0.0;

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(&full[warp][s], 1);
        fence_mbar_init();
    }
    __syncwarp();
    // chunk q of this warp's stream: row gw + (q / nchunks) * nw, chunk q % nchunks
    auto issue = [&](int64_t q) {
        const int s = int(q % NS);
        const int64_t r = gw + (q / nchunks) * nw;
        const uint32_t off = uint32_t(q % nchunks) * kWarpRowChunk;
        const uint32_t nb = row_bytes - off < uint32_t(kWarpRowChunk) ? row_bytes - off : uint32_t(kWarpRowChunk);
        const unsigned char *src = static_cast<const unsigned char *>(prm.logits) + r * prm.C * sizeof(T) + off;
        mbar_expect_tx(&full[warp][s], nb);
        bulk_load_1d(ring[warp][s], src, nb, &full[warp][s]);
    };
    if (lane == 0)
        for (int64_t q = 0; q < NS && q < my_chunks; ++q) issue(q);

    int64_t q = 0;
    bool alive = true;
    for (int64_t ri = 0; ri < my_rows && alive; ++ri) {
        const int64_t r = gw + ri * nw;
        const int64_t lb = __ldg(prm.labels + r);
        const bool valid = lb != prm.ignore;
        const int lbi = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
        float m = kNegInf, sum = 0.f, sde = 0.f, sx = 0.f, xl = kNegInf;
        for (int c = 0; c < nchunks; ++c, ++q) {
            const int s = int(q % NS);
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&full[warp][s], uint32_t(q / NS) & 1u, status);
            if (!__shfl_sync(0xffffffffu, ok, 0)) {
                alive = false;
                break;
            }
            const int ebase = c * (kWarpRowChunk / int(sizeof(T)));     // first element of the chunk
            // my vectors of this chunk into registers; their maximum first
            V xv[kWarpRowVecs];
            float vmax = kNegInf;
            const int jt = lbi - ebase;                                  // target's offset in the chunk, if inside
#pragma unroll
            for (int v = 0; v < kWarpRowVecs; ++v) {
                const int e0 = ebase + (v * 32 + lane) * VN;
                if (e0 < C) {
                    xv[v] = *reinterpret_cast<const V *>(ring[warp][s] + (v * 32 + lane) * 16);
#pragma unroll
                    for (int p = 0; p < NP; ++p) {
                        const float2 x = pair_of(xv[v], p);
                        vmax = fmaxf(vmax, fmaxf(x.x, x.y));
                    }
                }
            }
            __syncwarp();                       // every lane has its data: the stage can be refilled
            if (lane == 0 && q + NS < my_chunks) issue(q + NS);
            // the target element (at most one lane, one vector): remember it; large margin takes
            // it out of the statistics, so that lane redoes its maximum without it
            const bool in_chunk = lbi >= 0 && jt >= 0 && jt < kWarpRowChunk / int(sizeof(T));
            const int tv = in_chunk ? (jt / VN) / 32 : -1, tl = in_chunk ? (jt / VN) % 32 : -1, tq = in_chunk ? jt % VN : -1;
            const bool mine = in_chunk && tl == lane;
            if (mine) {
#pragma unroll
                for (int v = 0; v < kWarpRowVecs; ++v)
#pragma unroll
                    for (int e = 0; e < VN; ++e)
                        if (v == tv && e == tq) xl = to_f32(xv[v].v[e]);
                if (KIND == kLMargin) {
                    vmax = kNegInf;
#pragma unroll
                    for (int v = 0; v < kWarpRowVecs; ++v) {
                        const int e0 = ebase + (v * 32 + lane) * VN;
                        if (e0 < C) {
#pragma unroll
                            for (int e = 0; e < VN; ++e)
                                if (!(v == tv && e == tq)) vmax = fmaxf(vmax, to_f32(xv[v].v[e]));
                        }
                    }
                }
            }
            const float mn = fmaxf(m, vmax);
            const float dm = m - mn;
            const float rs = ex2f(dm * kLog2e);
            if (KIND == kLMargin) sde = rs * fmaf(dm, sum, sde);
            sum *= rs;
            m = mn;
            const float2 nml = splat2(-mn * kLog2e), negm = splat2(-mn);
            float2 sum2 = make_float2(sum, 0.f), sde2 = make_float2(sde, 0.f), sx2 = make_float2(sx, 0.f);
#pragma unroll
            for (int v = 0; v < kWarpRowVecs; ++v) {
                const int e0 = ebase + (v * 32 + lane) * VN;
                if (e0 < C) {
#pragma unroll
                    for (int p = 0; p < NP; ++p) {
                        float2 x = pair_of(xv[v], p);
                        float2 e = ex2_2(fma2(x, splat2(kLog2e), nml));
                        if (KIND == kLMargin && mine && v == tv && p == tq / 2) {
                            // drop the target from the pair
                            if (tq & 1) { e.y = 0.f; x.y = mn; } else { e.x = 0.f; x.x = mn; }
                            sx2 = add2(sx2, make_float2((tq & 1) ? x.x : 0.f, (tq & 1) ? 0.f : x.y));
                        } else {
                            sx2 = add2(sx2, x);
                        }
                        sum2 = add2(sum2, e);
                        if (KIND == kLMargin) sde2 = fma2(add2(x, negm), e, sde2);
                    }
                }
            }
            sum = sum2.x + sum2.y;
            sde = sde2.x + sde2.y;
            sx = sx2.x + sx2.y;
        }
        if (!alive) break;
        // ---- the warp's statistics: common maximum, then the rescaled sums
        float M = m, xlw = xl;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            xlw = fmaxf(xlw, __shfl_xor_sync(0xffffffffu, xlw, o));
        }
        const float dmt = m - M;
        const float f = ex2f(dmt * kLog2e);
        float ssum = sum * f, ssde = (KIND == kLMargin) ? f * fmaf(dmt, sum, sde) : 0.f, ssx = sx;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
            ssx += __shfl_xor_sync(0xffffffffu, ssx, o);
            if (KIND == kLMargin) ssde += __shfl_xor_sync(0xffffffffu, ssde, o);
        }
        if (lane == 0) {
            const float xlv = lbi >= 0 ? xlw : 0.f;
            float l = 0.f;
            if (lbi != -1) {
                if (KIND == kLSR) {
                    l = kc.sumy * (M + __logf(ssum)) - kc.lb_neg * ssx - (kc.lb_pos - kc.lb_neg) * xlv;
                } else {
                    const float nother = lbi >= 0 ? float(C - 1) : float(C);
                    const float sd = ssx - nother * M;
                    const float sqx = ssde * __fdividef(1.f, ssum);
                    const float mm = fmaxf(M, xlv);
                    const float e_no = ssum * ex2f((M - mm) * kLog2e);
                    const float e_lb = lbi >= 0 ? ex2f((xlv - mm) * kLog2e) : 0.f;
                    l = (mm + __logf(e_no + e_lb)) - xlv + kc.half_lam * (sqx - kc.a * sd);
                }
            }
            if (losses) losses[r] = from_f32<T>(l);
            if (REDUCE && lbi != -1) {
                acc_loss += double(l);
                acc_cnt += 1.0;
            }
        }
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// ------------------------------------------------------------- short-rows regime
// M == 1 with up to 2048 channels: [N, C] classification inputs and channels-last images, where
// every pixel is a row of C contiguous logits (C x element size need not be a multiple of 16).  A
// stage holds R = 256 / TPR consecutive rows -- ONE contiguous run of R * C elements, moved by one bulk copy in and, in
// backward, one bulk copy out (R is a multiple of 8 and an element has 2 or 4 bytes, so every run starts and ends on 16 bytes) --
// together with the R labels.  TPR adjacent lanes (1 to 32: at most 32 channels per lane up to
// 1024 channels, 64 beyond) share a row and combine their statistics with shuffles: no block barrier, no shared-memory
// exchange.  The last rows of the input (fewer than R) have no 16-byte guarantee: the
// compute threads move them with plain loads and stores.
constexpr int kShortCompute = 256;
constexpr int kShortBlock = kShortCompute + 64;
constexpr int kShortRowsMaxC = 2048;          // a warp per row, 64 channels per lane

// Statistics of a row combined over its TPR adjacent lanes.  `mask` names exactly those lanes: the
// lanes of a row take the same branches (a row is valid or ignored as a whole), other rows of
// the warp may be elsewhere.
template <int KIND> struct LaneMerge;
template <> struct LaneMerge<kLSR> {
    static __device__ __forceinline__ void s1(Stat1<kLSR> &a, int tpr, unsigned mask) {
        for (int o = tpr >> 1; o > 0; o >>= 1) a.m = fmaxf(a.m, __shfl_xor_sync(mask, a.m, o));
    }
    static __device__ __forceinline__ void s2(Stat2<kLSR> &b, int tpr, unsigned mask) {
        for (int o = tpr >> 1; o > 0; o >>= 1) {
            b.s += __shfl_xor_sync(mask, b.s, o);
            b.sx += __shfl_xor_sync(mask, b.sx, o);
            b.xl += __shfl_xor_sync(mask, b.xl, o);
        }
    }
};
template <> struct LaneMerge<kLMargin> {
    static __device__ __forceinline__ void s1(Stat1<kLMargin> &a, int tpr, unsigned mask) {
        for (int o = tpr >> 1; o > 0; o >>= 1) {
            a.m_no = fmaxf(a.m_no, __shfl_xor_sync(mask, a.m_no, o));
            a.xl = fmaxf(a.xl, __shfl_xor_sync(mask, a.xl, o));
        }
    }
    static __device__ __forceinline__ void s2(Stat2<kLMargin> &b, int tpr, unsigned mask) {
        for (int o = tpr >> 1; o > 0; o >>= 1) {
            b.s_no += __shfl_xor_sync(mask, b.s_no, o);
            b.sde += __shfl_xor_sync(mask, b.sde, o);
            b.sd += __shfl_xor_sync(mask, b.sd, o);
        }
    }
};

template <typename T, int KIND, bool BWD, bool REDUCE>
__global__ void __launch_bounds__(kShortBlock)
rows_multi_kernel(const SoftmaxParams prm) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    __shared__ double sh_red[64];

    const int C = static_cast<int>(prm.C), NS = prm.stages, TPR = prm.KS;
    const int R = kShortCompute / TPR;                       // rows per stage
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const size_t label_off = (size_t(R) * C * sizeof(T) + 127) & ~size_t(127);
    const size_t stage_bytes = label_off + size_t(R) * sizeof(int64_t);
    const int tid = threadIdx.x;
    unsigned *status = prm.workspace ? reinterpret_cast<unsigned *>(prm.workspace) + 1 : nullptr;
    const int64_t n_stages = (prm.N + R - 1) / R;
    const uint32_t full_bytes = uint32_t(R) * C * sizeof(T);

    pipe_init<kShortCompute, BWD>(bars, NS);
    const int64_t first = blockIdx.x, stride = gridDim.x;
    double acc_loss = 0.0, acc_cnt = 0.0;

    if (tid == kShortCompute) {
        int k = 0;
        for (int64_t st = first; st < n_stages; st += stride, ++k) {
            const int s = k % NS;
            if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, status)) break;
            const int64_t row0 = st * R;
            if (prm.N - row0 >= R) {
                unsigned char *stage = base + s * stage_bytes;
                const unsigned char *src = static_cast<const unsigned char *>(prm.logits) + row0 * C * sizeof(T);
                mbar_expect_tx(&bars.full[s], full_bytes + uint32_t(R) * sizeof(int64_t));
                for (uint32_t off = 0; off < full_bytes; off += 32768u) {
                    const uint32_t nb = full_bytes - off < 32768u ? full_bytes - off : 32768u;
                    bulk_load_1d(stage + off, src + off, nb, &bars.full[s]);
                }
                bulk_load_1d(stage + label_off, prm.labels + row0, uint32_t(R) * sizeof(int64_t), &bars.full[s]);
            } else {
                mbar_expect_tx(&bars.full[s], 0);            // ragged end: the compute threads fetch it themselves
            }
        }
    } else if (BWD && tid == kShortCompute + 32) {
        int k = 0;
        for (int64_t st = first; st < n_stages; st += stride, ++k) {
            const int s = k % NS;
            if (!mbar_wait_bounded(&bars.ready[s], (k / NS) & 1, status)) break;
            const int64_t row0 = st * R;
            if (prm.N - row0 >= R) {
                const unsigned char *stage = base + s * stage_bytes;
                unsigned char *dst = static_cast<unsigned char *>(prm.grads) + row0 * C * sizeof(T);
                for (uint32_t off = 0; off < full_bytes; off += 32768u) {
                    const uint32_t nb = full_bytes - off < 32768u ? full_bytes - off : 32768u;
                    bulk_store_1d(dst + off, stage + off, nb);
                }
                bulk_commit();
                bulk_wait_read_all();
            }
            mbar_arrive(&bars.empty[s]);
        }
        bulk_wait_all();
    } else if (tid < kShortCompute) {
        const int lane = tid & 31;
        const int rowl = tid / TPR, t = tid % TPR;           // my row inside a stage, my lane inside the row
        // A lane visits the units (channels, or channel pairs) u = c * TPR + t of its row, chunk c
        // after chunk c.  Few lanes per row and an even C: the rows of a warp lie an even number of
        // words apart and would share banks, so the walk starts at a chunk that depends on the row
        // and wraps around (same trip count in every lane: no divergence).  Otherwise (odd C, or
        // 8+ lanes per row = few rows per warp) a plain strided loop.
        const bool rotate = TPR <= 4 && (C & 1) == 0;
        const int chunks_c = (C + TPR - 1) / TPR, chunks_p = ((C >> 1) + TPR - 1) / TPR;
        const int rot_c = rotate ? rowl % chunks_c : 0, rot_p = (rotate && chunks_p > 0) ? rowl % chunks_p : 0;
        auto walk_units = [&](int n, int chunks, int rot, auto &&body) {
            if (!rotate && TPR == 1) {
#pragma unroll 4
                for (int u = 0; u < n; ++u) body(u);            // (unit stride: immediate offsets after unrolling)
            } else if (!rotate) {
#pragma unroll 4
                for (int u = t; u < n; u += TPR) body(u);
            } else {
                int c = rot;
#pragma unroll 4
                for (int i = 0; i < chunks; ++i) {
                    const int u = c * TPR + t;
                    if (u < n) body(u);
                    c = (c + 1 == chunks) ? 0 : c + 1;
                }
            }
        };
        auto walk = [&](auto &&body) { walk_units(C, chunks_c, rot_c, body); };
        const unsigned row_mask = (TPR == 32 ? 0xffffffffu : ((1u << TPR) - 1u)) << (lane & ~(TPR - 1));
        const T *gout = static_cast<const T *>(prm.grad_out);
        T *losses = static_cast<T *>(prm.losses);
        const LossConsts kc = prm.k;
        float gscale = 1.f;
        if (BWD && REDUCE) pdl_wait();                       // (see tile_pair_kernel)
        if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
        int k = 0;
        for (int64_t st = first; st < n_stages; st += stride, ++k) {
            const int s = k % NS;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, status);
            // (the ragged last stage needs all compute threads at a named barrier, which has no
            // time limit: every stage's decision to go on is taken by all of them together)
            if (!compute_all(ok, kShortCompute)) break;
            const int64_t row0 = st * R;
            const int nrows = prm.N - row0 >= R ? R : int(prm.N - row0);
            const bool ragged = nrows < R;
            T *tile = reinterpret_cast<T *>(base + s * stage_bytes);
            int64_t *tile_labels = reinterpret_cast<int64_t *>(base + s * stage_bytes + label_off);
            if (ragged) {
                const T *src = static_cast<const T *>(prm.logits) + row0 * C;
                for (int e = tid; e < nrows * C; e += kShortCompute) tile[e] = src[e];
                for (int e = tid; e < nrows; e += kShortCompute) tile_labels[e] = prm.labels[row0 + e];
                compute_sync(kShortCompute);
            }
            const bool live = rowl < nrows;
            const int64_t row = row0 + rowl;
            const int64_t lb = live ? tile_labels[rowl] : prm.ignore;
            const bool valid = live && lb != prm.ignore;
            const int lbi = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
            T *rp = tile + size_t(rowl) * C;
            if (KIND == kLSR && valid && (C & 1) == 0) {
                // Label smooth, even C: the lane's channels as adjacent PAIRS (one 8-byte -- half
                // types 4-byte -- access and packed fp32x2 arithmetic per pair), e^{x-m} kept in the
                // tile between the sum and the gradient (one exponential per element), the target
                // term added by the lane that owns the label's pair (tile_pair_kernel's scheme).
                const int npair = C >> 1;
                const float xl = lbi >= 0 ? to_f32(rp[lbi]) : 0.f;
                __syncwarp(row_mask);                          // all of the row's lanes hold x_lb before e^{x-m} overwrites it
                float2 m2 = splat2(kNegInf);
                walk_units(npair, chunks_p, rot_p, [&](int q) { m2 = max2(m2, ld_pair(rp + 2 * q)); });
                float m = fmaxf(m2.x, m2.y);
                for (int o = TPR >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(row_mask, m, o));
                pk_t psum = psplat(0.f), psx = psplat(0.f);
                {
                    const pk_t nml = psplat(-m * kLog2e), l2e = psplat(kLog2e);
                    walk_units(npair, chunks_p, rot_p, [&](int q) {
                        const pk_t x = ld_pk(rp + 2 * q);
                        const pk_t e = pex2(pfma(x, l2e, nml));
                        psum = padd(psum, e);
                        psx = padd(psx, x);
                        if (BWD) st_pk(rp + 2 * q, e);
                    });
                }
                float2 s2v = upk2(psum), sxv = upk2(psx);
                float sum = s2v.x + s2v.y, sx = sxv.x + sxv.y;
                for (int o = TPR >> 1; o > 0; o >>= 1) {
                    sum += __shfl_xor_sync(row_mask, sum, o);
                    sx += __shfl_xor_sync(row_mask, sx, o);
                }
                const float loss = kc.sumy * (m + __logf(sum)) - kc.lb_neg * sx - (kc.lb_pos - kc.lb_neg) * xl;
                if (t == 0) {
                    if (!BWD && losses) losses[row] = from_f32<T>(loss);
                    if (REDUCE) {
                        acc_loss += double(loss);
                        acc_cnt += 1.0;
                    }
                }
                if (BWD) {
                    float psc = gscale;
                    if (prm.grad_mode == 2) psc *= to_f32(gout[row]);
                    // g = (sumy e / s - lb_neg) scale, then the target's lb_neg -> lb_pos
                    const pk_t pa = psplat(kc.sumy * __fdividef(psc, sum)), pb = psplat(-kc.lb_neg * psc);
                    walk_units(npair, chunks_p, rot_p, [&](int q) { st_pk(rp + 2 * q, pfma(ld_pk(rp + 2 * q), pa, pb)); });
                    if (lbi >= 0 && (lbi >> 1) % TPR == t)
                        rp[lbi] = from_f32<T>(to_f32(rp[lbi]) - (kc.lb_pos - kc.lb_neg) * psc);
                }
            } else if (KIND == kLMargin && valid && lbi >= 0 && (C & 1) == 0) {
                // Large margin, even C: channel pairs and packed arithmetic as above, the target
                // handled as in tile_pair_kernel: its logit is parked at -FLT_MAX for the maximum
                // sweep and at min(x_lb, m') for the sum sweep, its terms are then taken back out of
                // the sums (s' >= 1 >= e^{min(x_lb - m', 0)}: nothing cancels), and its gradient
                // overwrites what the sweep left there.
                const int npair = C >> 1;
                const float xl = to_f32(rp[lbi]);
                __syncwarp(row_mask);                          // all of the row's lanes hold x_lb before it is parked
                const bool owner = (lbi >> 1) % TPR == t;      // my walk visits the label's pair
                if (owner) rp[lbi] = from_f32<T>(sizeof(T) == 2 ? -65504.f : kNegInf);
                float2 m2 = splat2(kNegInf);
                walk_units(npair, chunks_p, rot_p, [&](int q) { m2 = max2(m2, ld_pair(rp + 2 * q)); });
                float m = fmaxf(m2.x, m2.y);
                for (int o = TPR >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(row_mask, m, o));
                const float cl = fminf(xl, m);
                if (owner) rp[lbi] = from_f32<T>(cl);
                const pk_t pnegm = psplat(-m), l2e = psplat(kLog2e);
                pk_t psum = psplat(0.f), psde = psplat(0.f), psx = psplat(0.f);
                walk_units(npair, chunks_p, rot_p, [&](int q) {
                    const pk_t x = ld_pk(rp + 2 * q);
                    const pk_t d = padd(x, pnegm);
                    const pk_t e = pex2(pmul(d, l2e));
                    psum = padd(psum, e);
                    psde = pfma(d, e, psde);
                    psx = padd(psx, x);
                });
                const float2 v1 = upk2(psum), v2 = upk2(psde), v3 = upk2(psx);
                float sum = v1.x + v1.y, sde = v2.x + v2.y, sx = v3.x + v3.y;
                for (int o = TPR >> 1; o > 0; o >>= 1) {
                    sum += __shfl_xor_sync(row_mask, sum, o);
                    sde += __shfl_xor_sync(row_mask, sde, o);
                    sx += __shfl_xor_sync(row_mask, sx, o);
                }
                // (half tiles hold the parked value rounded to T: use what the sweep read)
                const float clr = to_f32(from_f32<T>(cl));
                const float dc = clr - m;
                const float ec = ex2f(dc * kLog2e);
                const float s_no = sum - ec;
                const float sde_no = sde - dc * ec;
                const float sd = (sx - clr) - float(C - 1) * m;
                const float inv_s = __fdividef(1.f, s_no);
                const float sqx = sde_no * inv_s;
                const float mm = fmaxf(m, xl);
                const float e_no = s_no * ex2f((m - mm) * kLog2e);
                const float e_lb = ex2f((xl - mm) * kLog2e);
                const float s_all = e_no + e_lb;
                const float rr = __fdividef(e_no, s_all);
                const float loss = (mm + __logf(s_all)) - xl + kc.half_lam * (sqx - kc.a * sd);
                if (t == 0) {
                    if (!BWD && losses) losses[row] = from_f32<T>(loss);
                    if (REDUCE) {
                        acc_loss += double(loss);
                        acc_cnt += 1.0;
                    }
                }
                if (BWD) {
                    float psc = gscale;
                    if (prm.grad_mode == 2) psc *= to_f32(gout[row]);
                    // g_j = scale (r q + lam/2 (q (d + 1 - sqx) - a)) = q (A + B d) + Cc,  q = e^d / s'
                    const pk_t pqa = psplat((rr + kc.half_lam * (1.f - sqx)) * psc), pqb = psplat(kc.half_lam * psc);
                    const pk_t pcc = psplat(-kc.half_lam * kc.a * psc), pqs = psplat(inv_s);
                    walk_units(npair, chunks_p, rot_p, [&](int q) {
                        const pk_t d = padd(ld_pk(rp + 2 * q), pnegm);
                        const pk_t qq = pmul(pex2(pmul(d, l2e)), pqs);
                        st_pk(rp + 2 * q, pfma(qq, pfma(pqb, d, pqa), pcc));
                    });
                    if (owner) rp[lbi] = from_f32<T>(-rr * psc);
                }
            } else if (valid) {
                Stat1<KIND> s1;
                s1.init();
                walk([&](int j) { s1.add(to_f32(rp[j]), j == lbi); });
                LaneMerge<KIND>::s1(s1, TPR, row_mask);
                Stat2<KIND> s2;
                s2.init();
                walk([&](int j) { s2.add(to_f32(rp[j]), j == lbi, s1); });
                LaneMerge<KIND>::s2(s2, TPR, row_mask);
                PixelFinal<KIND> fin;
                fin.finish(s1, s2, kc);
                if (t == 0) {
                    if (!BWD && losses) losses[row] = from_f32<T>(fin.loss);
                    if (REDUCE) {
                        acc_loss += double(fin.loss);
                        acc_cnt += 1.0;
                    }
                }
                if (BWD) {
                    float psc = gscale;
                    if (prm.grad_mode == 2) psc *= to_f32(gout[row]);
                    walk([&](int j) { rp[j] = from_f32<T>(fin.grad(to_f32(rp[j]), j == lbi, kc) * psc); });
                }
            } else if (live) {
                if (!BWD && losses && t == 0) losses[row] = from_f32<T>(0.f);
                if (BWD)
                    for (int p = t; p < C; p += TPR) rp[p] = from_f32<T>(0.f);
            }
            if (!BWD) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.empty[s]);
            } else {
                if (ragged) {
                    compute_sync(kShortCompute);
                    T *dst = static_cast<T *>(prm.grads) + row0 * C;
                    for (int e = tid; e < nrows * C; e += kShortCompute) dst[e] = tile[e];
                } else {
                    fence_proxy_async_smem();
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.ready[s]);
            }
        }
    }
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// The layouts rows_multi_kernel takes.
inline bool short_rows_eligible(const void *logits, const void *io, const void *labels, int64_t N, int64_t C, int64_t M) {
    return M == 1 && N >= 1 && C >= 1 && C <= kShortRowsMaxC && aligned16(logits) && aligned16(io) && aligned16(labels);
}

// ------------------------------------------------------------- any-alignment spatial regime
// M > 1 where the rows of a channel do not start on 16 bytes (M not a multiple of 4 floats: 769 x
// 769 or 713 x 713 crops) or the pointers are not aligned: no tensor map, no bulk copy.  The 256
// threads of a block are KS channel slices x (256 / KS) adjacent pixels; a thread keeps its
// slice's channels (every KS-th, at most CPT) of ONE pixel in registers -- 4-byte accesses, a warp
// reads 128 contiguous bytes per channel wherever they start, all of a thread's loads in flight
// together -- and the slices combine their statistics through shared memory (two block barriers
// per group of pixels; none with a single slice).  The logits are read once.  float32 only.
constexpr int kAnyThreads = 256;
template <int KIND, bool BWD, bool REDUCE, int KS, int CPT>
__global__ void __launch_bounds__(kAnyThreads, KS == 1 ? 3 : 2)
spatial_any_kernel(const SoftmaxParams prm) {
    constexpr int PX = kAnyThreads / KS;
    __shared__ double sh_red[64];
    __shared__ float ex[2][5][KS][PX];           // [round parity][statistic word][slice][pixel]
    const float *x = static_cast<const float *>(prm.logits);
    float *grads = static_cast<float *>(prm.grads);
    float *losses = static_cast<float *>(prm.losses);
    const float *gout = static_cast<const float *>(prm.grad_out);
    const int C = static_cast<int>(prm.C);
    const int Mi = static_cast<int>(prm.M);      // C * M < 2^31 (host check): 32-bit channel offsets
    const int px = threadIdx.x % PX, ks = threadIdx.x / PX;
    const int64_t groups_per_row = (prm.M + PX - 1) / PX;
    const int64_t groups = prm.N * groups_per_row;
    const LossConsts kc = prm.k;
    float gscale = 1.f;
    bool first = true;
    double acc_loss = 0.0, acc_cnt = 0.0;
    int par = 0;
    for (int64_t gi = blockIdx.x; gi < groups; gi += gridDim.x, par ^= 1) {
        const int64_t n = gi / groups_per_row;
        const int64_t m = (gi % groups_per_row) * PX + px;
        const bool live = m < prm.M;
        const int64_t base = n * prm.C * prm.M + (live ? m : 0);
        float xv[CPT];
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int j = ks + i * KS;
            xv[i] = (live && j < C) ? __ldcs(x + base + j * Mi) : 0.f;
        }
        const int64_t lb = live ? prm.labels[n * prm.M + m] : prm.ignore;
        if (first) {
            if (BWD && REDUCE) pdl_wait();        // the divisor comes from the label count in front
            if (BWD) gscale = uniform_grad_scale(prm.grad_out, prm.grad_mode, prm.denom);
            first = false;
        }
        const bool valid = live && lb != prm.ignore;
        const int lbi = valid ? ((lb >= 0 && lb < C) ? int(lb) : -2) : -1;
        Stat1<KIND> s1;
        s1.init();
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int j = ks + i * KS;
            if (j < C) s1.add(xv[i], j == lbi);
        }
        if (KS > 1) {
            s1.store(&ex[par][0][ks][px], KS * PX);
            __syncthreads();
#pragma unroll
            for (int q = 1; q < KS; ++q) {
                Stat1<KIND> o;
                o.load(&ex[par][0][(ks + q) % KS][px], KS * PX);
                s1.merge(o);
            }
        }
        Stat2<KIND> s2;
        s2.init();
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
            const int j = ks + i * KS;
            if (j < C) {
                if constexpr (KIND == kLSR) {
                    // e^{x-m} takes x's place: the gradient needs nothing else (one exponential per element)
                    const float e = exp_fast(xv[i] - s1_max(s1));
                    s2_add_with_exp(s2, xv[i], e, j == lbi);
                    xv[i] = e;
                } else {
                    s2.add(xv[i], j == lbi, s1);
                }
            }
        }
        if (KS > 1) {
            s2.store(&ex[par][2][ks][px], KS * PX);
            __syncthreads();
            s2.init();
#pragma unroll
            for (int q = 0; q < KS; ++q) {       // (fixed order: every slice gets the same bits)
                Stat2<KIND> o;
                o.load(&ex[par][2][q][px], KS * PX);
                s2.merge(o);
            }
        }
        if (!live) continue;
        PixelFinal<KIND> fin;
        fin.finish(s1, s2, kc);
        if (ks == 0) {
            if (!BWD && losses) losses[n * prm.M + m] = valid ? fin.loss : 0.f;
            if (REDUCE && valid) {
                acc_loss += double(fin.loss);
                acc_cnt += 1.0;
            }
        }
        if (BWD) {
            float psc = gscale;
            if (prm.grad_mode == 2) psc *= gout[n * prm.M + m];
            float *gb = grads + base;
#pragma unroll
            for (int i = 0; i < CPT; ++i) {
                const int j = ks + i * KS;
                if (j < C) __stcs(gb + j * Mi, valid ? grad_phase3<KIND>(fin, xv[i], j == lbi, kc) * psc : 0.f);
            }
        }
    }
    if (first && BWD && REDUCE) pdl_wait();
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

inline bool spatial_any_eligible(size_t es, int64_t C, int64_t M) {
    return es == 4 && M > 1 && C <= 320 && C * M < (int64_t(1) << 31);
}

template <int KIND, bool BWD, bool REDUCE>
int launch_spatial_any(const SoftmaxParams &prm, cudaStream_t stream) {
    // slices x channels per thread; the unrolled loops run over all CPT slots, so CPT follows C
    const int ks = prm.C <= 40 ? 1 : (prm.C <= 160 ? 4 : 8);
    const int px = kAnyThreads / ks;
    const int64_t rounds = prm.N * ((prm.M + px - 1) / px);
    int64_t grid = int64_t(sm_count()) * 2 * (ks == 1 ? 4 : 1);   // a single slice has no barrier: short-lived blocks are fine
    if (grid > rounds) grid = rounds;
    if (grid > kMaxPartials) grid = kMaxPartials;
    const dim3 gd{unsigned(grid)}, bd(kAnyThreads);
    const bool dep = BWD && REDUCE && prm.after_count;
    if (prm.C <= 8) launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 1, 8>, gd, bd, 0, stream, dep, prm);
    else if (prm.C <= 20) launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 1, 20>, gd, bd, 0, stream, dep, prm);
    else if (prm.C <= 40) launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 1, 40>, gd, bd, 0, stream, dep, prm);
    else if (prm.C <= 80) launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 4, 20>, gd, bd, 0, stream, dep, prm);
    else if (prm.C <= 160) launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 4, 40>, gd, bd, 0, stream, dep, prm);
    else launch_kernel(spatial_any_kernel<KIND, BWD, REDUCE, 8, 40>, gd, bd, 0, stream, dep, prm);
    return launch_status("softmax any-alignment kernel launch");
}

// Integer tuning override from the environment (tile size, ring depth, blocks per SM);
// unset or unparsable -> the default.

template <typename K> int set_smem(K kernel, size_t bytes) {
    if (bytes > 40 * 1024) {   // static shared memory shares the default 48 KiB
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess)
            return launch_status("cudaFuncSetAttribute(max dynamic shared memory)");
    }
    return B200_OK;
}

// True when the chunked kernels (tile_chunk_fwd_kernel / tile_chunk_bwd_kernel) take the call:
// tile regime, TMA-capable layout, at least one 512-pixel tile, and more classes than the
// 512-pixel-wide resident tile of tile_pair_kernel holds.  `io`: the gradient (backward) or
// the logits again (forward).
inline bool chunk_eligible(size_t es, const void *logits, const void *io, const void *labels, int64_t N, int64_t C,
                           int64_t M) {
    if (M <= 1 || size_t(C) * 32 * es + 8192 > kSmemLimit) return false;
    const bool tma_ok = (M * es) % 16 == 0 && aligned16(logits) && aligned16(io) && M < (int64_t(1) << 31) &&
                        N < (int64_t(1) << 31) && aligned16(labels);
    if (!tma_ok || M < kChunkTile) return false;
    const int64_t nbox = (C + 255) / 256, rows = nbox * ((C + nbox - 1) / nbox);
    return 2 * size_t(rows) * 256 * es > size_t(40) * 1024;
}

template <typename T, int KIND, bool BWD, bool REDUCE>
int launch_regime(SoftmaxParams prm, int dtype, cudaStream_t stream) {
    const size_t es = sizeof(T);
    const int sms = sm_count();
    const void *io = BWD ? prm.grads : prm.logits;

    const bool aligned_io = aligned16(prm.logits) && aligned16(io);
    if (prm.M > 1 && size_t(prm.C) * 32 * es + 8192 <= kSmemLimit) {
        // ---- tile regime
        const bool tma_ok = (prm.M * es) % 16 == 0 && aligned_io && prm.M < (int64_t(1) << 31) &&
                            prm.N < (int64_t(1) << 31) && aligned16(prm.labels);
        // Tile size.  Backward: ~40 KB tiles, two stages (the store of one tile overlaps the math
        // of the next).  Forward with many channels: ~80 KB tiles in a single stage -- twice the
        // elements per thread under the same per-tile costs (label handling, slice exchange,
        // per-pixel epilogue) measured 0.67 of peak against 0.55 for config 3; overlap comes from
        // the second block on the SM.
        size_t target = tma_ok ? size_t(40) * 1024 : kTileTargetBytes;
        int default_stages = 2;
        if (tma_ok && !BWD && size_t(prm.C) * 256 * es > target) {
            target = size_t(80) * 1024;
            default_stages = 1;
        }
        int TP = 256;
        while (TP > 32 && size_t(prm.C) * TP * es > target) TP >>= 1;
        while (TP > 32 && TP / 2 >= prm.M) TP >>= 1;   // tiny images: do not waste lanes
        prm.TP = TP;
        prm.KS = kThreads / TP;
        prm.nbox = int((prm.C + 255) / 256);
        prm.CB = int((prm.C + prm.nbox - 1) / prm.nbox);
        prm.rows = prm.nbox * prm.CB;
        // few channels: two boxes side by side, so that one thread pair-column spans all channels
        prm.nbx = (tma_ok && TP == 256 && 2 * size_t(prm.rows) * TP * es <= size_t(40) * 1024 && prm.M > TP) ? 2 : 1;
        if constexpr (!BWD) {
            // many channels, forward: 512-pixel tiles streamed in channel chunks (no slice exchange)
            if (chunk_eligible(es, prm.logits, prm.logits, prm.labels, prm.N, prm.C, prm.M)) {
                const ChunkLayout lay = chunk_layout<T>();
                // measured on config 3 (C = 150): 2 stages x 3 blocks per SM 206 us, 3 stages x 2 blocks 222 us
                int stages = (2);
                if (stages > kMaxStages) stages = kMaxStages;
                prm.stages = stages;
                const size_t smem = 128 + size_t(stages) * lay.stage_bytes;
                int per_sm = int((224 * 1024) / (smem + 1024));
                const int cap_sm = (3);
                if (per_sm > cap_sm) per_sm = cap_sm;
                if (per_sm < 1) per_sm = 1;
                const int64_t tiles = prm.N * ((prm.M + kChunkTile - 1) / kChunkTile);
                int64_t grid = int64_t(sms) * per_sm;
                if (grid > tiles) grid = tiles;
                if (grid > kMaxPartials) grid = kMaxPartials;
                CUtensorMap map_in{};
                const uint64_t dims[3] = {uint64_t(prm.M), uint64_t(prm.C), uint64_t(prm.N)};
                const uint64_t strides[3] = {es, uint64_t(prm.M) * es, uint64_t(prm.C) * prm.M * es};
                const uint32_t box[3] = {uint32_t(kChunkTP), uint32_t(kChunkCh), 1u};
                if (!encode_tensor_map(&map_in, dtype, prm.logits, 3, dims, strides, box)) return B200_ERR_LAUNCH;
                auto kern = tile_chunk_fwd_kernel<T, KIND, REDUCE>;
                int rc2;
                if ((rc2 = set_smem(kern, smem)) != B200_OK) return rc2;
                kern<<<dim3(unsigned(grid)), kTileBlock, smem, stream>>>(prm, map_in);
                return launch_status("softmax chunked forward kernel launch");
            }
        }
        if constexpr (BWD && KIND != kPC) {
            // many channels, backward from the statistics the chunked forward saved
            if (prm.stats && aligned16(prm.stats) &&
                chunk_eligible(es, prm.logits, prm.grads, prm.labels, prm.N, prm.C, prm.M)) {
                const ChunkBwdLayout lay = chunk_bwd_layout<T>();
                // a stage is busy from its load to the end of its store: backward wants a deeper ring
                // than forward (config 3: 3 stages in one block per SM 396 us, 2 stages x 2 blocks 430 us)
                int stages = (3);
                if (stages > kMaxStages) stages = kMaxStages;
                prm.stages = stages;
                const size_t smem = 128 + size_t(stages) * lay.stage_bytes;
                int per_sm = int((224 * 1024) / (smem + 1024));
                const int cap_sm = (3);
                if (per_sm > cap_sm) per_sm = cap_sm;
                if (per_sm < 1) per_sm = 1;
                const int64_t tiles = prm.N * ((prm.M + kChunkTile - 1) / kChunkTile);
                int64_t grid = int64_t(sms) * per_sm;
                if (grid > tiles) grid = tiles;
                CUtensorMap map_in{}, map_out{};
                const uint64_t dims[3] = {uint64_t(prm.M), uint64_t(prm.C), uint64_t(prm.N)};
                const uint64_t strides[3] = {es, uint64_t(prm.M) * es, uint64_t(prm.C) * prm.M * es};
                const uint32_t box[3] = {uint32_t(kChunkTP), uint32_t(kChunkCh), 1u};
                if (!encode_tensor_map(&map_in, dtype, prm.logits, 3, dims, strides, box)) return B200_ERR_LAUNCH;
                if (!encode_tensor_map(&map_out, dtype, prm.grads, 3, dims, strides, box)) return B200_ERR_LAUNCH;
                auto kern = tile_chunk_bwd_kernel<T, KIND>;
                int rc2;
                if ((rc2 = set_smem(kern, smem)) != B200_OK) return rc2;
                kern<<<dim3(unsigned(grid)), kTileBlock, smem, stream>>>(prm, map_in, map_out);
                return launch_status("softmax chunked backward kernel launch");
            }
        }
        const int TPT = TP * prm.nbx;
        prm.tiles_per_image = (prm.M + TPT - 1) / TPT;
        prm.total_tiles = prm.N * prm.tiles_per_image;
        const size_t tile_bytes = (size_t(prm.rows) * TPT * es + 127) & ~size_t(127);
        const size_t red_bytes = size_t(6) * kThreads * sizeof(float);
        int rc;
        if (tma_ok) {
            // statistics exchange area: 5 words x (slices * TP = 2 * 256) floats
            const size_t xchg_bytes = size_t(5) * kTileCompute * 2 * sizeof(float);
            // a stage holds the logits tile, the tile's labels and its coordinates
            const size_t stage_bytes = tile_bytes + size_t(TPT) * sizeof(int64_t) + 128;
            int stages = (default_stages);
            while (stages > 1 && 128 + stages * stage_bytes + xchg_bytes > kSmemLimit) --stages;
            if (stages > kMaxStages) stages = kMaxStages;
            prm.stages = stages;
            const size_t smem = 128 + stages * stage_bytes + xchg_bytes;
            int per_sm = int((224 * 1024) / (smem + 1024));
            const int cap_sm = (3);
            if (per_sm > cap_sm) per_sm = cap_sm;
            if (per_sm < 1) per_sm = 1;
            int64_t grid = int64_t(sms) * per_sm;
            if (grid > prm.total_tiles) grid = prm.total_tiles;
            if (grid > kMaxPartials) grid = kMaxPartials;
            CUtensorMap map_in{}, map_out{};
            const uint64_t dims[3] = {uint64_t(prm.M), uint64_t(prm.C), uint64_t(prm.N)};
            const uint64_t strides[3] = {es, uint64_t(prm.M) * es, uint64_t(prm.C) * prm.M * es};
            const uint32_t box[3] = {uint32_t(TP), uint32_t(prm.CB), 1u};
            if (!encode_tensor_map(&map_in, dtype, prm.logits, 3, dims, strides, box)) return B200_ERR_LAUNCH;
            if (BWD && !encode_tensor_map(&map_out, dtype, prm.grads, 3, dims, strides, box)) return B200_ERR_LAUNCH;
            auto kern = tile_pair_kernel<T, KIND, BWD, REDUCE>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            launch_kernel(kern, dim3(unsigned(grid)), dim3(kTileBlock), smem, stream, BWD && REDUCE && prm.after_count,
                          prm, map_in, map_out);
        } else if constexpr (KIND != kPC) {
            if constexpr (sizeof(T) == 4) {
                if (spatial_any_eligible(es, prm.C, prm.M)) return launch_spatial_any<KIND, BWD, REDUCE>(prm, stream);
            }
            const size_t smem = 128 + tile_bytes + red_bytes;
            int per_sm = int((220 * 1024) / (smem + 1024));
            if (per_sm > 8) per_sm = 8;
            if (per_sm < 1) per_sm = 1;
            int64_t grid = int64_t(sms) * per_sm;
            if (grid > prm.total_tiles) grid = prm.total_tiles;
            if (grid > kMaxPartials) grid = kMaxPartials;
            CUtensorMap unused{};
            auto kern = tile_kernel<T, KIND, BWD, REDUCE, false>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            kern<<<dim3(unsigned(grid)), kThreads, smem, stream>>>(prm, unused, unused);
        } else {
            (void)red_bytes;
            set_error("pc softmax step: this layout has no fused step");
            return B200_ERR_UNSUPPORTED;
        }
        return launch_status("softmax tile kernel launch");
    }
    if constexpr (KIND == kPC) {
        set_error("pc softmax step: this layout has no fused step");
        return B200_ERR_UNSUPPORTED;
    } else {
    if (short_rows_eligible(prm.logits, io, prm.labels, prm.N, prm.C, prm.M)) {
        // ---- short-rows regime
        // at most 32 channels per lane, 3 stages in backward (measured on the fused steps of configs 1
        // and 3 in channels-last: 0.148 / 0.797 ms; 2 or 4 stages 0.162 / 0.93-0.95 ms; 16 channels per
        // lane doubles config 1's time; 40 per lane and 2 stages: 0.163 / 0.760 ms)
        int tpr = 1;
        while (tpr < 32 && (prm.C + tpr - 1) / tpr > 32) tpr <<= 1;
        prm.KS = tpr;
        const int R = kShortCompute / tpr;
        const size_t label_off = (size_t(R) * prm.C * es + 127) & ~size_t(127);
        const size_t stage_bytes = label_off + size_t(R) * sizeof(int64_t);
        prm.stages = (BWD && stage_bytes <= size_t(36) * 1024) ? 3 : 2;
        const size_t smem = 128 + size_t(prm.stages) * stage_bytes;
        int per_sm = int((224 * 1024) / (smem + 2048));
        if (per_sm > 4) per_sm = 4;
        if (per_sm < 1) per_sm = 1;
        const int64_t n_stages = (prm.N + R - 1) / R;
        int64_t grid = int64_t(sms) * per_sm;
        if (grid > n_stages) grid = n_stages;
        if (grid > kMaxPartials) grid = kMaxPartials;
        auto kern = rows_multi_kernel<T, KIND, BWD, REDUCE>;
        int rc;
        if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
        launch_kernel(kern, dim3(unsigned(grid)), dim3(kShortBlock), smem, stream, BWD && REDUCE && prm.after_count, prm);
        return launch_status("softmax short-rows kernel launch");
    }
    if constexpr (!BWD) {
        // ---- rows regime, forward, long rows: one warp per row, streamed (any row length)
        if (prm.M == 1 && (size_t(prm.C) * es) % 16 == 0 && size_t(prm.C) * es >= 2 * size_t(kWarpRowChunk) &&
            aligned_io) {
            const size_t smem = 128 + size_t(kWarpRowWarps) * kWarpRowStages * kWarpRowChunk;
            // measured on config 5: 2 stages x 3 blocks per SM 223 us, 3 stages x 2 blocks 237 us,
            // 2 KB chunks x 5 blocks 246 us (whole-row kernel below: 251 us)
            const int per_sm = (3);
            int64_t grid = int64_t(sms) * per_sm;
            const int64_t need = (prm.N + kWarpRowWarps - 1) / kWarpRowWarps;
            if (grid > need) grid = need;
            if (grid > kMaxPartials) grid = kMaxPartials;
            auto kern = rows_warp_fwd_kernel<T, KIND, REDUCE>;
            int rc2;
            if ((rc2 = set_smem(kern, smem)) != B200_OK) return rc2;
            kern<<<dim3(unsigned(grid)), kWarpRowWarps * 32, smem, stream>>>(prm);
            return launch_status("softmax warp-per-row forward kernel launch");
        }
    }
    if (prm.M == 1 && prm.C >= 256 && size_t(prm.C) * es + 1024 <= kSmemLimit) {
        // ---- rows regime
        const size_t row_al = (size_t(prm.C) * es + 127) & ~size_t(127);
        const bool bulk = (size_t(prm.C) * es) % 16 == 0 && aligned_io;
        int rc;
        if (bulk) {
            // One row per block in flight and several blocks per SM beat a deep ring in one block:
            // the phases of a row (max sweep, block reduction, sum sweep, ...) cannot overlap inside
            // a block, they can across blocks (config 5: forward 0.60 of peak with 2 blocks x 1 stage
            // against 0.52 with 1 block x 3 stages; backward 0.85 with 3 blocks).
            int stages = (row_al > 32 * 1024 ? 1 : 2);
            while (stages > 1 && 128 + stages * row_al > kSmemLimit) --stages;
            if (stages > kMaxStages) stages = kMaxStages;
            prm.stages = stages;
            const size_t smem = 128 + stages * row_al;
            int per_sm = int((224 * 1024) / (smem + 2048));
            const int rows_cap = (BWD ? 3 : 2);
            if (per_sm > rows_cap) per_sm = rows_cap;
            if (per_sm < 1) per_sm = 1;
            int64_t grid = int64_t(sms) * per_sm;
            if (grid > prm.N) grid = prm.N;
            if (grid > kMaxPartials) grid = kMaxPartials;
            auto kern = rows_pipe_kernel<T, KIND, BWD, REDUCE>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            launch_kernel(kern, dim3(unsigned(grid)), dim3(kRowsBlock), smem, stream, BWD && REDUCE && prm.after_count, prm);
        } else {
            const size_t smem = 128 + row_al;
            int per_sm = int((220 * 1024) / (smem + 2048));
            if (per_sm > 8) per_sm = 8;
            if (per_sm < 1) per_sm = 1;
            int64_t grid = int64_t(sms) * per_sm;
            if (grid > prm.N) grid = prm.N;
            if (grid > kMaxPartials) grid = kMaxPartials;
            auto kern = rows_kernel<T, KIND, BWD, REDUCE, false>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            kern<<<dim3(unsigned(grid)), kThreads, smem, stream>>>(prm);
        }
        return launch_status("softmax rows kernel launch");
    }
    // ---- sweep regime
    const int64_t P = prm.N * prm.M;
    int64_t grid = (P + kThreads - 1) / kThreads;
    const int64_t cap = int64_t(sms) * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    sweep_kernel<T, KIND, BWD, REDUCE><<<dim3(unsigned(grid)), kThreads, 0, stream>>>(prm);
    return launch_status("softmax sweep kernel launch");
    }
}

template <int KIND, bool BWD>
int dispatch(const SoftmaxParams &prm, int dtype, bool reduce, cudaStream_t stream) {
    if (dtype == B200_F32)
        return reduce ? launch_regime<float, KIND, BWD, true>(prm, dtype, stream)
                      : launch_regime<float, KIND, BWD, false>(prm, dtype, stream);
    if (dtype == B200_F16)
        return reduce ? launch_regime<__half, KIND, BWD, true>(prm, dtype, stream)
                      : launch_regime<__half, KIND, BWD, false>(prm, dtype, stream);
    if (dtype == B200_BF16)
        return reduce ? launch_regime<__nv_bfloat16, KIND, BWD, true>(prm, dtype, stream)
                      : launch_regime<__nv_bfloat16, KIND, BWD, false>(prm, dtype, stream);
    set_error("unknown dtype code %d", dtype);
    return B200_ERR_ARG;
}

int check_shape(const char *who, int64_t N, int64_t C, int64_t M) {
    if (N < 0 || C < 1 || M < 0) {
        set_error("%s: bad shape N=%lld C=%lld M=%lld", who, (long long)N, (long long)C, (long long)M);
        return B200_ERR_ARG;
    }
    if (C >= (int64_t(1) << 31)) {
        set_error("%s: C=%lld does not fit 31 bits", who, (long long)C);
        return B200_ERR_UNSUPPORTED;
    }
    return B200_OK;
}

__global__ void empty_record_kernel(void *workspace, ReduceRecord *out) {
    __shared__ double sh[64];
    grid_reduce_finish(0.0, 0.0, workspace, out, sh);
}

template <int KIND>
int forward(const char *who, const void *logits, const int64_t *labels, void *losses, void *out,
            void *workspace, size_t workspace_bytes, int64_t N, int64_t C, int64_t M, int dtype,
            int64_t ignore_index, float hp, void *stream, void *stats = nullptr) {
    int rc = check_shape(who, N, C, M);
    if (rc != B200_OK) return rc;
    const int64_t P = N * M;
    if (P == 0 && !out) return B200_OK;   // empty input, nothing to write
    if (!losses && !out) {
        set_error("%s: at least one of losses / out must be given", who);
        return B200_ERR_ARG;
    }
    if (out && (!workspace || workspace_bytes < kReduceWorkspaceBytes)) {
        set_error("%s: workspace of %zu bytes required", who, kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    if (P > 0 && (!logits || !labels)) {
        set_error("%s: null input pointer", who);
        return B200_ERR_ARG;
    }
    if (P == 0) {
        // no pixels: the record of an empty sum (count 0, mean 0/0), still added over attached ranks
        empty_record_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(workspace, static_cast<ReduceRecord *>(out));
        return launch_status("empty reduction launch");
    }
    if (dtype == B200_F64)
        return stats ? (set_error("%s: no per-pixel statistics in float64", who), B200_ERR_UNSUPPORTED)
                     : f64_softmax_forward(KIND, logits, labels, losses, out, workspace, N, C, M, ignore_index, hp, stream);
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.losses = losses;
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.stats = static_cast<float4 *>(stats);
    prm.N = N;
    prm.C = C;
    prm.M = M;
    prm.ignore = ignore_index;
    prm.k = make_consts(KIND, C, hp);
    return dispatch<KIND, false>(prm, dtype, out != nullptr, static_cast<cudaStream_t>(stream));
}

template <int KIND>
int backward(const char *who, const void *logits, const int64_t *labels, const void *grad_out,
             int grad_mode, const void *denom, void *grad_logits, int64_t N, int64_t C, int64_t M,
             int dtype, int64_t ignore_index, float hp, void *stream, const void *stats = nullptr) {
    int rc = check_shape(who, N, C, M);
    if (rc != B200_OK) return rc;
    if (grad_mode < 0 || grad_mode > 2 || (grad_mode != 0 && !grad_out)) {
        set_error("%s: bad grad_mode / grad_out", who);
        return B200_ERR_ARG;
    }
    if (N * M == 0) return B200_OK;
    if (!logits || !labels || !grad_logits) {
        set_error("%s: null pointer", who);
        return B200_ERR_ARG;
    }
    if (dtype == B200_F64)
        return stats ? (set_error("%s: no per-pixel statistics in float64", who), B200_ERR_UNSUPPORTED)
                     : f64_softmax_backward(KIND, logits, labels, grad_out, grad_mode, denom, grad_logits, N, C, M,
                                            ignore_index, hp, stream);
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.grad_out = grad_out;
    prm.grad_mode = grad_mode;
    prm.denom = static_cast<const double *>(denom);
    prm.stats = static_cast<float4 *>(const_cast<void *>(stats));
    prm.N = N;
    prm.C = C;
    prm.M = M;
    prm.ignore = ignore_index;
    prm.k = make_consts(KIND, C, hp);
    return dispatch<KIND, true>(prm, dtype, false, static_cast<cudaStream_t>(stream));
}

// The fused training step runs in the TMA tile kernel and in the whole-row kernel: both keep all
// channels of a pixel (a row) resident in shared memory, so one read of the logits serves the
// loss and the gradient.
// M > 1: the layouts the TMA tile pipeline takes (16-byte aligned rows and pointers).
inline bool tile_pipeline_eligible(size_t es, const void *logits, const void *grads, const void *labels, int64_t N,
                                   int64_t C, int64_t M) {
    return N >= 1 && M > 1 && size_t(C) * 32 * es + 8192 <= kSmemLimit && (M * es) % 16 == 0 && aligned16(logits) &&
           aligned16(grads) && aligned16(labels) && M < (int64_t(1) << 31) && N < (int64_t(1) << 31);
}

inline bool fused_step_eligible(size_t es, const void *logits, const void *grads, const void *labels, int64_t N,
                                int64_t C, int64_t M) {
    if (N < 1 || M < 1) return false;
    if (M == 1) {
        if (C <= kShortRowsMaxC && aligned16(logits) && aligned16(grads) && aligned16(labels)) return true;   // short rows
        return size_t(C) * es + 1024 <= kSmemLimit && (size_t(C) * es) % 16 == 0 && aligned16(logits) && aligned16(grads);
    }
    if (size_t(C) * 32 * es + 8192 > kSmemLimit) return false;
    if (es == 4 && C <= 320 && C * M < (int64_t(1) << 31)) return true;      // any alignment: the tile pipeline or spatial_any_kernel
    return tile_pipeline_eligible(es, logits, grads, labels, N, C, M);
}

// Label-smooth training step for few channels (C <= CMAX, float32, M even, 8-byte aligned
// pointers): a thread owns 2 adjacent pixels and keeps all their channels in registers, so the
// logits are read once with 8-byte accesses and the gradient is written once -- no shared
// memory, no barrier before the final reduction.  The label channel's gradient is a second
// 4-byte store over the first one instead of a compare per channel.
constexpr int kResidentThreads = 256;
// EXACT: C == CMAX, the channel loops carry no predicate.
template <int CMAX, bool EXACT>
__global__ void __launch_bounds__(kResidentThreads, 2)
lsr_resident_step_kernel(const SoftmaxParams prm) {
    __shared__ double sh_red[64];
    const float *x = static_cast<const float *>(prm.logits);
    float *grads = static_cast<float *>(prm.grads);
    const int C = EXACT ? CMAX : prm.k.C;
    const int M = int(prm.M);                      // C * M < 2^31 (host check): 32-bit channel offsets
    const int64_t groups_per_row = prm.M / 2;
    const int64_t groups = prm.N * groups_per_row;
    const int64_t stride = int64_t(gridDim.x) * kResidentThreads;
    pdl_wait();                                    // the divisor comes from the label count in front
    const float gs = uniform_grad_scale(nullptr, 0, prm.denom);
    const float sumy_gs = prm.k.sumy * gs, neg_gs = prm.k.lb_neg * gs;
    const float dpn = prm.k.lb_pos - prm.k.lb_neg;
    constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
    float acc = 0.f, cnt = 0.f;
    for (int64_t gi = int64_t(blockIdx.x) * kResidentThreads + threadIdx.x; gi < groups; gi += stride) {
        const int64_t n = gi / groups_per_row, m0 = (gi % groups_per_row) * 2;
        const int64_t base = n * prm.C * prm.M + m0;
        const float *xb = x + base;
        float2 xv[CMAX];
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (EXACT || j < C) xv[j] = __ldcs(reinterpret_cast<const float2 *>(xb + j * M));
        const longlong2 lb2 = __ldcs(reinterpret_cast<const longlong2 *>(prm.labels + n * prm.M + m0));
        const bool v0 = lb2.x != prm.ignore, v1 = lb2.y != prm.ignore;
        // (labels outside [0, C) that are not the ignore value are undefined in the reference;
        // here no channel takes the target term)
        const int l0 = v0 ? int(lb2.x) : -1, l1 = v1 ? int(lb2.y) : -1;
        float2 mx = make_float2(kNegInf, kNegInf), sx = make_float2(0.f, 0.f);
        float xl0 = 0.f, xl1 = 0.f;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (EXACT || j < C) {
                mx = max2(mx, xv[j]);
                sx = add2(sx, xv[j]);
                if (j == l0) xl0 = xv[j].x;
                if (j == l1) xl1 = xv[j].y;
            }
        const float2 nm2 = make_float2(-mx.x * kLog2e, -mx.y * kLog2e);
        float2 s = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (EXACT || j < C) {
                xv[j] = ex2_2(fma2(xv[j], splat2(kLog2e), nm2));      // e^{x - m} takes x's place
                s = add2(s, xv[j]);
            }
        if (v0) {
            acc += prm.k.sumy * fmaf(__log2f(s.x), kLn2, mx.x) - prm.k.lb_neg * sx.x - dpn * xl0;
            cnt += 1.f;
        }
        if (v1) {
            acc += prm.k.sumy * fmaf(__log2f(s.y), kLn2, mx.y) - prm.k.lb_neg * sx.y - dpn * xl1;
            cnt += 1.f;
        }
        // g_j = (sumy e_j / s - y_j) gs with y_j = lb_neg, lb_pos at the label; zero at ignored pixels
        const float2 a = make_float2(v0 ? __fdividef(sumy_gs, s.x) : 0.f, v1 ? __fdividef(sumy_gs, s.y) : 0.f);
        const float2 b = make_float2(v0 ? -neg_gs : 0.f, v1 ? -neg_gs : 0.f);
        const float dl = -dpn * gs;
        float *gb = grads + base;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (EXACT || j < C) {
                float2 g = fma2(xv[j], a, b);
                if (j == l0) g.x += dl;
                if (j == l1) g.y += dl;
                __stcs(reinterpret_cast<float2 *>(gb + j * M), g);
            }
    }
    grid_reduce_finish(double(acc), double(cnt), prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

// Label-smooth training step over classification rows (M == 1, float32, C a multiple of 4 between
// 64 and 2048, 16-byte aligned pointers): a warp owns a row and keeps it in registers -- NV 16-byte
// vectors per lane, all of a lane's loads in flight together -- so the logits are read once and the
// gradient is written once, with no shared memory and no barrier before the final reduction.  The
// target's logit is fetched again (one 4-byte load per row) and its gradient is a 4-byte store by
// the lane that wrote the vector around it.
template <int NV>
__global__ void __launch_bounds__(kResidentThreads, NV <= 8 ? 3 : 2)
lsr_rows_resident_step_kernel(const SoftmaxParams prm) {
    __shared__ double sh_red[64];
    const float4 *x = static_cast<const float4 *>(prm.logits);
    float4 *grads = static_cast<float4 *>(prm.grads);
    const int lane = threadIdx.x & 31;
    const int C = prm.k.C, nvec = C >> 2;
    const int64_t warps = int64_t(gridDim.x) * (kResidentThreads / 32);
    pdl_wait();                                    // the divisor comes from the label count in front
    const float gs = uniform_grad_scale(nullptr, 0, prm.denom);
    const float dpn = prm.k.lb_pos - prm.k.lb_neg;
    float acc = 0.f, cnt = 0.f;
    for (int64_t r = int64_t(blockIdx.x) * (kResidentThreads / 32) + (threadIdx.x >> 5); r < prm.N; r += warps) {
        const float4 *xr = x + r * nvec;
        float4 xv[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) xv[i] = __ldcs(xr + v);
        }
        const int64_t lb = __ldg(prm.labels + r);
        const bool valid = lb != prm.ignore;
        // (a label outside [0, C) that is not the ignore value is undefined in the reference: no target term here)
        const int lbi = (valid && lb >= 0 && lb < C) ? int(lb) : -1;
        const float xl = lbi >= 0 ? __ldg(static_cast<const float *>(prm.logits) + r * C + lbi) : 0.f;
        float4 *grow = grads + r * nvec;
        if (!valid) {                              // (uniform over the warp)
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = lane + 32 * i;
                if (v < nvec) __stcs(grow + v, make_float4(0.f, 0.f, 0.f, 0.f));
            }
            continue;
        }
        float m = kNegInf, sx = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32 * i < nvec) {
                m = fmaxf(fmaxf(m, fmaxf(xv[i].x, xv[i].y)), fmaxf(xv[i].z, xv[i].w));
                sx += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float nm2 = -m * kLog2e;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32 * i < nvec) {
                xv[i].x = ex2f(fmaf(xv[i].x, kLog2e, nm2));         // e^{x-m} takes x's place
                xv[i].y = ex2f(fmaf(xv[i].y, kLog2e, nm2));
                xv[i].z = ex2f(fmaf(xv[i].z, kLog2e, nm2));
                xv[i].w = ex2f(fmaf(xv[i].w, kLog2e, nm2));
                s += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, o);
            sx += __shfl_xor_sync(0xffffffffu, sx, o);
        }
        if (lane == 0) {
            acc += prm.k.sumy * (m + __log2f(s) * kLn2) - prm.k.lb_neg * sx - dpn * xl;
            cnt += 1.f;
        }
        const float a = prm.k.sumy * __fdividef(gs, s), b = -prm.k.lb_neg * gs;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec)
                __stcs(grow + v, make_float4(fmaf(xv[i].x, a, b), fmaf(xv[i].y, a, b), fmaf(xv[i].z, a, b), fmaf(xv[i].w, a, b)));
        }
        // target: (sumy e_l / s - lb_pos) gs, by the lane whose vector store covers it (program order)
        if (lbi >= 0 && ((lbi >> 2) & 31) == lane)
            reinterpret_cast<float *>(grow)[lbi] = fmaf(ex2f(fmaf(xl, kLog2e, nm2)), a, -prm.k.lb_pos * gs);
    }
    grid_reduce_finish(double(acc), double(cnt), prm.workspace, prm.out, sh_red, kTagSum, prm.defer != 0);
}

inline bool rows_resident_step_eligible(int kind, int dtype, const void *logits, const void *grads, const void *labels,
                                        int64_t N, int64_t C, int64_t M) {
    return kind == kLSR && dtype == B200_F32 && M == 1 && N >= 1 && C % 4 == 0 && C >= 64 && C <= 2048 &&
           aligned16(logits) && aligned16(grads) && labels != nullptr;
}

int launch_rows_resident_step(const SoftmaxParams &prm, cudaStream_t stream) {
    int64_t grid = (prm.N + kResidentThreads / 32 - 1) / (kResidentThreads / 32);
    const int64_t cap = int64_t(sm_count()) * (prm.C <= 1024 ? 3 : 2);   // all blocks resident: one reduction barrier per block
    if (grid > cap) grid = cap;
    const dim3 gd{unsigned(grid)}, bd(kResidentThreads);
    const bool dep = prm.after_count != 0;
    if (prm.C <= 256) launch_kernel(lsr_rows_resident_step_kernel<2>, gd, bd, 0, stream, dep, prm);
    else if (prm.C <= 1024) launch_kernel(lsr_rows_resident_step_kernel<8>, gd, bd, 0, stream, dep, prm);
    else launch_kernel(lsr_rows_resident_step_kernel<16>, gd, bd, 0, stream, dep, prm);
    return launch_status("label-smooth resident rows step launch");
}

inline bool aligned8(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; }

// The layouts lsr_resident_step_kernel takes, and the sizes it wins at: up to ~40 M elements its
// short ramp (no tensor maps, no barrier set-up, no pipeline fill) beats the tile pipeline (label
// count + step: 29.6 against 35.4 us at 10 M elements, 42.3 against 49.5 us at 20 M, level at
// 80 M); larger inputs keep the pipeline.  Layouts
// the pipeline cannot take (M even but not a multiple of 4, 8-byte alignment) come here at any size.
inline bool resident_step_eligible(int kind, int dtype, const void *logits, const void *grads, const void *labels,
                                   int64_t N, int64_t C, int64_t M, bool pipeline_ok) {
    if (!(kind == kLSR && dtype == B200_F32 && N >= 1 && M >= 2 && M % 2 == 0 && C <= 32 &&
          C * M < (int64_t(1) << 31) && aligned8(logits) && aligned8(grads) && aligned16(labels)))
        return false;
    return !pipeline_ok || N * C * M <= (int64_t(40) << 20);
}

int launch_resident_step(const SoftmaxParams &prm, cudaStream_t stream) {
    const int64_t groups = prm.N * (prm.M / 2);
    int64_t grid = (groups + kResidentThreads - 1) / kResidentThreads;
    const int64_t cap = int64_t(sm_count()) * 2;        // all blocks resident: one reduction barrier per block
    if (grid > cap) grid = cap;
    const unsigned g = unsigned(grid);
    cudaStream_t st = stream;
    const bool dep = prm.after_count != 0;
    const dim3 gd(g), bd(kResidentThreads);
    if (prm.C == 19) launch_kernel(lsr_resident_step_kernel<19, true>, gd, bd, 0, st, dep, prm);
    else if (prm.C == 21) launch_kernel(lsr_resident_step_kernel<21, true>, gd, bd, 0, st, dep, prm);
    else if (prm.C <= 8) launch_kernel(lsr_resident_step_kernel<8, false>, gd, bd, 0, st, dep, prm);
    else if (prm.C <= 20) launch_kernel(lsr_resident_step_kernel<20, false>, gd, bd, 0, st, dep, prm);
    else launch_kernel(lsr_resident_step_kernel<32, false>, gd, bd, 0, st, dep, prm);
    return launch_status("label-smooth resident step launch");
}

template <int KIND>
int fused_step(const char *who, const void *logits, const int64_t *labels, void *grad_logits, void *out,
               void *workspace, size_t workspace_bytes, const void *denom, int64_t N, int64_t C, int64_t M,
               int dtype, int64_t ignore_index, float hp, int defer, void *stream) {
    int rc = check_shape(who, N, C, M);
    if (rc != B200_OK) return rc;
    if (!out || !workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("%s: out and a workspace of %zu bytes are required", who, kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    if (!logits || !labels || !grad_logits) {
        set_error("%s: null pointer", who);
        return B200_ERR_ARG;
    }
    const size_t es = dtype_size(dtype);
    const bool any_ok = fused_step_eligible(es, logits, grad_logits, labels, N, C, M);
    const bool pipeline_ok = M == 1 ? any_ok : tile_pipeline_eligible(es, logits, grad_logits, labels, N, C, M);
    const bool resident = resident_step_eligible(KIND, dtype, logits, grad_logits, labels, N, C, M, pipeline_ok);
    if (!resident && !any_ok) {
        set_error("%s: this layout has no fused step (ask b200_softmax_fused_step_path first)", who);
        return B200_ERR_UNSUPPORTED;
    }
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.denom = static_cast<const double *>(denom);
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.N = N;
    prm.C = C;
    prm.M = M;
    prm.ignore = ignore_index;
    prm.k = make_consts(KIND, C, hp);
    prm.defer = defer & B200_STEP_DEFER;
    prm.after_count = (denom != nullptr && (defer & B200_STEP_AFTER_COUNT)) ? 1 : 0;
    if (resident) return launch_resident_step(prm, static_cast<cudaStream_t>(stream));
    if (rows_resident_step_eligible(KIND, dtype, logits, grad_logits, labels, N, C, M))
        return launch_rows_resident_step(prm, static_cast<cudaStream_t>(stream));
    return dispatch<KIND, true>(prm, dtype, true, static_cast<cudaStream_t>(stream));
}

// Proportion-corrected softmax cross entropy as a training step on the resident-tile pipeline
// (tile_pair_kernel<T, kPC, true, true>): loss sum record and final gradient from one read of the
// logits.  Layouts: those of the tile pipeline (M > 1, 16-byte aligned rows), up to kPcMaxC classes.
inline bool pc_step_eligible(int dtype, const void *logits, const void *grads, const void *labels, int64_t N,
                             int64_t C, int64_t M) {
    return dtype_known(dtype) && dtype != B200_F64 && M > 1 && C >= 1 && C <= kPcMaxC &&
           tile_pipeline_eligible(dtype_size(dtype), logits, grads, labels, N, C, M);
}

// Number of labels != ignore, 16-byte loads, four in flight per thread.
__global__ void __launch_bounds__(256) count_valid_kernel(const int64_t *labels, int64_t P, int64_t ignore,
                                                          void *workspace, ReduceRecord *out) {
    __shared__ double sh[64];
    pdl_launch_dependents();      // a fused step behind this kernel may start filling its pipeline
    const bool al = (reinterpret_cast<uintptr_t>(labels) & 15u) == 0;
    const int64_t nvec = al ? P / 2 : 0;
    const longlong2 *v = reinterpret_cast<const longlong2 *>(labels);
    const int64_t stride = int64_t(gridDim.x) * 256;
    int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
    int cnt = 0;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        longlong2 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = __ldcs(v + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u) cnt += int(a[u].x != ignore) + int(a[u].y != ignore);
    }
    for (; i < nvec; i += stride) {
        const longlong2 a = __ldcs(v + i);
        cnt += int(a.x != ignore) + int(a.y != ignore);
    }
    for (int64_t j = nvec * 2 + int64_t(blockIdx.x) * 256 + threadIdx.x; j < P; j += stride)
        cnt += int(labels[j] != ignore);
    grid_reduce_finish(0.0, double(cnt), workspace, out, sh, kTagCount);
}

}  // namespace
}  // namespace b200

using namespace b200;

// out->count = number of labels != ignore_index among `P` (summed over the ranks attached to the
// workspace, if any); out->sum = 0.  The divisor of a 'mean' that the fused step needs on the
// device BEFORE it writes gradients.
extern "C" int b200_count_valid(const int64_t *labels, int64_t P, int64_t ignore_index, void *out,
                                void *workspace, size_t workspace_bytes, void *stream) {
    if (P < 0 || !out || (P > 0 && !labels)) {
        set_error("b200_count_valid: bad arguments");
        return B200_ERR_ARG;
    }
    if (!workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("b200_count_valid: workspace of %zu bytes required", kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    int64_t grid = (P / 2 + 256 * 4 - 1) / (256 * 4);
    const int64_t cap = int64_t(sm_count()) * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    count_valid_kernel<<<unsigned(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        labels, P, ignore_index, workspace, static_cast<ReduceRecord *>(out));
    return launch_status("label count kernel launch");
}

// 1 when (logits, labels, grad_logits, N, C, M, dtype) has a fused training step, else 0.
extern "C" int b200_softmax_fused_step_path(const void *logits, const int64_t *labels, const void *grad_logits,
                                            int64_t N, int64_t C, int64_t M, int dtype) {
    if (!dtype_known(dtype)) return 0;
    if (C < 1 || C >= (int64_t(1) << 31)) return 0;
    return fused_step_eligible(dtype_size(dtype), logits, grad_logits, labels, N, C, M) ? 1 : 0;
}

extern "C" int b200_pc_softmax_step_path(const void *logits, const int64_t *labels, const void *grad_logits,
                                         int64_t N, int64_t C, int64_t M, int dtype) {
    return pc_step_eligible(dtype, logits, grad_logits, labels, N, C, M) ? 1 : 0;
}

// PC-softmax cross entropy (see pc_softmax.cu for the formulas): out = reduction record of the loss
// over the valid pixels, grad_logits = d(loss sum)/d(logits) / *denom (denom optional), one pass.
extern "C" int b200_pc_softmax_step(const void *logits, const int64_t *labels, const float *weight, void *grad_logits,
                                    void *out, void *workspace, size_t workspace_bytes, const void *denom,
                                    int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index, int flags,
                                    void *stream) {
    const char *who = "b200_pc_softmax_step";
    int rc = check_shape(who, N, C, M);
    if (rc != B200_OK) return rc;
    if (!out || !workspace || workspace_bytes < kReduceWorkspaceBytes) {
        set_error("%s: out and a workspace of %zu bytes are required", who, kReduceWorkspaceBytes);
        return B200_ERR_WORKSPACE;
    }
    if (!logits || !labels || !grad_logits || !weight) {
        set_error("%s: null pointer", who);
        return B200_ERR_ARG;
    }
    if (!pc_step_eligible(dtype, logits, grad_logits, labels, N, C, M)) {
        set_error("%s: this layout has no fused step (ask b200_pc_softmax_step_path first)", who);
        return B200_ERR_UNSUPPORTED;
    }
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.denom = static_cast<const double *>(denom);
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
    prm.N = N;
    prm.C = C;
    prm.M = M;
    prm.ignore = ignore_index;
    prm.k = make_consts(kLSR, C, 0.f);          // cross entropy: smoothing 0
    prm.chan_w = weight;
    prm.defer = 0;
    prm.after_count = (denom != nullptr && (flags & B200_STEP_AFTER_COUNT)) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == B200_F32) return launch_regime<float, kPC, true, true>(prm, dtype, st);
    if (dtype == B200_F16) return launch_regime<__half, kPC, true, true>(prm, dtype, st);
    return launch_regime<__nv_bfloat16, kPC, true, true>(prm, dtype, st);
}

// Loss sum (record in `out`) and FINAL gradient (divided by *denom when given: a device double,
// e.g. out->count of b200_count_valid) of the label-smooth cross entropy in one pass over the logits.
extern "C" int b200_lsr_forward_backward_reduced(const void *logits, const int64_t *labels, void *grad_logits,
                                                 void *out, void *workspace, size_t workspace_bytes,
                                                 const void *denom, int64_t N, int64_t C, int64_t M, int dtype,
                                                 int64_t ignore_index, float smooth, int defer, void *stream) {
    return fused_step<kLSR>("b200_lsr_forward_backward_reduced", logits, labels, grad_logits, out, workspace,
                            workspace_bytes, denom, N, C, M, dtype, ignore_index, smooth, defer, stream);
}

// The same for the large-margin softmax loss.
extern "C" int b200_lmargin_forward_backward_reduced(const void *logits, const int64_t *labels, void *grad_logits,
                                                     void *out, void *workspace, size_t workspace_bytes,
                                                     const void *denom, int64_t N, int64_t C, int64_t M, int dtype,
                                                     int64_t ignore_index, float lam, int defer, void *stream) {
    return fused_step<kLMargin>("b200_lmargin_forward_backward_reduced", logits, labels, grad_logits, out, workspace,
                           workspace_bytes, denom, N, C, M, dtype, ignore_index, lam, defer, stream);
}

extern "C" int b200_lsr_forward(const void *logits, const int64_t *labels, void *losses, void *out,
                                void *workspace, size_t workspace_bytes, int64_t N, int64_t C,
                                int64_t M, int dtype, int64_t ignore_index, float smooth,
                                void *stream) {
    return forward<kLSR>("b200_lsr_forward", logits, labels, losses, out, workspace, workspace_bytes,
                         N, C, M, dtype, ignore_index, smooth, stream);
}
extern "C" int b200_lsr_backward(const void *logits, const int64_t *labels, const void *grad_out,
                                 int grad_mode, const void *denom, void *grad_logits, int64_t N,
                                 int64_t C, int64_t M, int dtype, int64_t ignore_index,
                                 float smooth, void *stream) {
    return backward<kLSR>("b200_lsr_backward", logits, labels, grad_out, grad_mode, denom,
                          grad_logits, N, C, M, dtype, ignore_index, smooth, stream);
}
extern "C" int b200_lmargin_forward(const void *logits, const int64_t *labels, void *losses,
                                    void *out, void *workspace, size_t workspace_bytes, int64_t N,
                                    int64_t C, int64_t M, int dtype, int64_t ignore_index,
                                    float lam, void *stream) {
    return forward<kLMargin>("b200_lmargin_forward", logits, labels, losses, out, workspace,
                             workspace_bytes, N, C, M, dtype, ignore_index, lam, stream);
}
extern "C" int b200_lmargin_backward(const void *logits, const int64_t *labels,
                                     const void *grad_out, int grad_mode, const void *denom,
                                     void *grad_logits, int64_t N, int64_t C, int64_t M, int dtype,
                                     int64_t ignore_index, float lam, void *stream) {
    return backward<kLMargin>("b200_lmargin_backward", logits, labels, grad_out, grad_mode, denom,
                              grad_logits, N, C, M, dtype, ignore_index, lam, stream);
}

// ---- the same four entry points with per-pixel statistics handed from forward to backward
extern "C" int b200_softmax_stats_path(const void *logits, const int64_t *labels, const void *grad_logits,
                                       int64_t N, int64_t C, int64_t M, int dtype) {
    const size_t es = dtype_size(dtype);
    return chunk_eligible(es, logits, grad_logits ? grad_logits : logits, labels, N, C, M) ? 1 : 0;
}
extern "C" int b200_lsr_forward_ex(const void *logits, const int64_t *labels, void *losses, void *out,
                                   void *workspace, size_t workspace_bytes, void *stats, int64_t N, int64_t C,
                                   int64_t M, int dtype, int64_t ignore_index, float smooth, void *stream) {
    return forward<kLSR>("b200_lsr_forward_ex", logits, labels, losses, out, workspace, workspace_bytes, N, C, M,
                         dtype, ignore_index, smooth, stream, stats);
}
extern "C" int b200_lsr_backward_ex(const void *logits, const int64_t *labels, const void *stats,
                                    const void *grad_out, int grad_mode, const void *denom, void *grad_logits,
                                    int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index,
                                    float smooth, void *stream) {
    return backward<kLSR>("b200_lsr_backward_ex", logits, labels, grad_out, grad_mode, denom, grad_logits, N, C, M,
                          dtype, ignore_index, smooth, stream, stats);
}
extern "C" int b200_lmargin_forward_ex(const void *logits, const int64_t *labels, void *losses, void *out,
                                       void *workspace, size_t workspace_bytes, void *stats, int64_t N,
                                       int64_t C, int64_t M, int dtype, int64_t ignore_index, float lam,
                                       void *stream) {
    return forward<kLMargin>("b200_lmargin_forward_ex", logits, labels, losses, out, workspace, workspace_bytes, N,
                             C, M, dtype, ignore_index, lam, stream, stats);
}
extern "C" int b200_lmargin_backward_ex(const void *logits, const int64_t *labels, const void *stats,
                                        const void *grad_out, int grad_mode, const void *denom, void *grad_logits,
                                        int64_t N, int64_t C, int64_t M, int dtype, int64_t ignore_index,
                                        float lam, void *stream) {
    return backward<kLMargin>("b200_lmargin_backward_ex", logits, labels, grad_out, grad_mode, denom, grad_logits, N,
                              C, M, dtype, ignore_index, lam, stream, stats);
}
