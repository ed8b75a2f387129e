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

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr size_t kTileTargetBytes = 48 * 1024;
constexpr size_t kSmemLimit = 200 * 1024;

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
    int64_t N, C, M;
    int64_t ignore;
    LossConsts k;
    // tile geometry
    int TP, KS, CB, nbox, rows;
    int64_t tiles_per_image, total_tiles;
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
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red);
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
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red);
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
    if (REDUCE) grid_reduce_finish(acc_loss, acc_cnt, prm.workspace, prm.out, sh_red);
}

// -------------------------------------------------------------------- dispatch

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename K> int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess)
            return launch_status("cudaFuncSetAttribute(max dynamic shared memory)");
    }
    return B200_OK;
}

template <typename T, int KIND, bool BWD, bool REDUCE>
int launch_regime(SoftmaxParams prm, int dtype, cudaStream_t stream) {
    const size_t es = sizeof(T);
    const int sms = sm_count();
    const void *io = BWD ? prm.grads : prm.logits;

    if (prm.M > 1 && size_t(prm.C) * 32 * es + 8192 <= kSmemLimit) {
        // ---- tile regime
        int TP = 256;
        while (TP > 32 && size_t(prm.C) * TP * es > kTileTargetBytes) TP >>= 1;
        while (TP > 32 && TP / 2 >= prm.M) TP >>= 1;   // tiny images: do not waste lanes
        prm.TP = TP;
        prm.KS = kThreads / TP;
        prm.nbox = int((prm.C + 255) / 256);
        prm.CB = int((prm.C + prm.nbox - 1) / prm.nbox);
        prm.rows = prm.nbox * prm.CB;
        prm.tiles_per_image = (prm.M + TP - 1) / TP;
        prm.total_tiles = prm.N * prm.tiles_per_image;
        const size_t tile_bytes = (size_t(prm.rows) * TP * es + 127) & ~size_t(127);
        const size_t smem = 128 + tile_bytes + size_t(6) * kThreads * sizeof(float);
        int per_sm = int((220 * 1024) / (smem + 1024));
        if (per_sm > 8) per_sm = 8;
        if (per_sm < 1) per_sm = 1;
        int64_t grid = int64_t(sms) * per_sm;
        if (grid > prm.total_tiles) grid = prm.total_tiles;
        if (grid > kMaxPartials) grid = kMaxPartials;

        const bool tma_ok = (prm.M * es) % 16 == 0 && aligned16(prm.logits) && aligned16(io) &&
                            prm.M < (int64_t(1) << 31) && prm.N < (int64_t(1) << 31);
        CUtensorMap map_in{}, map_out{};
        bool use_tma = tma_ok;
        if (use_tma) {
            const uint64_t dims[3] = {uint64_t(prm.M), uint64_t(prm.C), uint64_t(prm.N)};
            const uint64_t strides[3] = {es, uint64_t(prm.M) * es, uint64_t(prm.C) * prm.M * es};
            const uint32_t box[3] = {uint32_t(TP), uint32_t(prm.CB), 1u};
            use_tma = encode_tensor_map(&map_in, dtype, prm.logits, 3, dims, strides, box);
            if (use_tma && BWD) use_tma = encode_tensor_map(&map_out, dtype, prm.grads, 3, dims, strides, box);
            if (!use_tma) return B200_ERR_LAUNCH;   // message already set by the encoder
        }
        int rc;
        if (use_tma) {
            auto kern = tile_kernel<T, KIND, BWD, REDUCE, true>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            kern<<<dim3(unsigned(grid)), kThreads, smem, stream>>>(prm, map_in, map_out);
        } else {
            auto kern = tile_kernel<T, KIND, BWD, REDUCE, false>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            kern<<<dim3(unsigned(grid)), kThreads, smem, stream>>>(prm, map_in, map_out);
        }
        return launch_status("softmax tile kernel launch");
    }
    if (prm.M == 1 && prm.C >= 256 && size_t(prm.C) * es + 1024 <= kSmemLimit) {
        // ---- rows regime
        const size_t smem = 128 + ((size_t(prm.C) * es + 127) & ~size_t(127));
        int per_sm = int((220 * 1024) / (smem + 2048));
        if (per_sm > 8) per_sm = 8;
        if (per_sm < 1) per_sm = 1;
        int64_t grid = int64_t(sms) * per_sm;
        if (grid > prm.N) grid = prm.N;
        if (grid > kMaxPartials) grid = kMaxPartials;
        const bool bulk = (size_t(prm.C) * es) % 16 == 0 && aligned16(prm.logits) && aligned16(io);
        int rc;
        if (bulk) {
            auto kern = rows_kernel<T, KIND, BWD, REDUCE, true>;
            if ((rc = set_smem(kern, smem)) != B200_OK) return rc;
            kern<<<dim3(unsigned(grid)), kThreads, smem, stream>>>(prm);
        } else {
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

template <int KIND, bool BWD>
int dispatch(const SoftmaxParams &prm, int dtype, bool reduce, cudaStream_t stream) {
    if (dtype == B200_F32)
        return reduce ? launch_regime<float, KIND, BWD, true>(prm, dtype, stream)
                      : launch_regime<float, KIND, BWD, false>(prm, dtype, stream);
    if (dtype == B200_F16)
        return reduce ? launch_regime<__half, KIND, BWD, true>(prm, dtype, stream)
                      : launch_regime<__half, KIND, BWD, false>(prm, dtype, stream);
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

template <int KIND>
int forward(const char *who, const void *logits, const int64_t *labels, void *losses, void *out,
            void *workspace, size_t workspace_bytes, int64_t N, int64_t C, int64_t M, int dtype,
            int64_t ignore_index, float hp, void *stream) {
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
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.losses = losses;
    prm.workspace = workspace;
    prm.out = static_cast<ReduceRecord *>(out);
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
             int dtype, int64_t ignore_index, float hp, void *stream) {
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
    SoftmaxParams prm{};
    prm.logits = logits;
    prm.labels = labels;
    prm.grads = grad_logits;
    prm.grad_out = grad_out;
    prm.grad_mode = grad_mode;
    prm.denom = static_cast<const double *>(denom);
    prm.N = N;
    prm.C = C;
    prm.M = M;
    prm.ignore = ignore_index;
    prm.k = make_consts(KIND, C, hp);
    return dispatch<KIND, true>(prm, dtype, false, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace b200

using namespace b200;

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
