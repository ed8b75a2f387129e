// Lovasz-softmax for sm_100a.
//
// What is computed (reference csrc/lovasz_softmax.cu:72-152,183-211,243-278,380-417):
// for every segment = (group, class), over the group's L pixels,
//   err_i  = |1[label_i == c] - softmax(x_i)_c|            (ignored pixels sort last, count 0)
//   sort err descending; fg_i = 1[label == c] in sorted order; n_pos = sum fg
//   J_i    = 1 - (n_pos - cumsum(fg)_i) / (n_pos - cumsum(fg)_i + i + 1);  dJ_i = J_i - J_{i-1}
//   loss   = sum_i err_i * dJ_i;     d loss / d p_{i,c} = dJ(rank of i) * (label_i == c ? -1 : +1)
// followed by the softmax Jacobian in backward.  A group is the whole batch (per_image = 0,
// the reference's behaviour) or one image (per_image = 1).
//
// How (all integer work exact, nothing compares floats):
//   keys     one tile kernel (TMA in, TMA out): softmax, then a 32-bit key per (pixel, class)
//            key = ((0x3F800000 - bits(err)) << 1) | fg  -> ascending key order = descending err,
//            ignored pixels get 0xFFFFFFFF.  err is in [0, 1] so 30 key bits carry it exactly.
//            The kernel also tracks, per segment, the largest foreground key and a sample of
//            the smallest keys (see track_fg).
//   prune    everything after the last foreground element of a segment in sorted order has
//            dJ = 0 exactly, so only elements with key <= that foreground key are sorted:
//            count per tile -> scan -> stable compaction of (key, pixel index), dJ = 0 written
//            for the rest.  A segment that would keep more than 3/4 is sorted from the full
//            array instead (`direct`).  What is kept depends on the data: ~7% for random
//            logits over 19 classes, everything when some foreground pixel has error 0.
//   sort     segmented LSD radix sort of the kept (key, pixel index) pairs, kBits per pass: all 30
//            key bits in three stable passes, or -- segments with many foreground elements,
//            see "Key bits" below -- the top 20 bits in two.  Each pass: per-tile digit histogram -> per-segment scan ->
//            stable scatter.  The scatter ranks with kBits ballots per round + per-warp
//            counters, reorders the tile in shared memory and writes each digit's run
//            contiguously.  The kept counts exist on the device only: the kernels run over a
//            device-built list of tiles in use.  No kernel waits on another.
//   jaccard  the last pass ranks in place: integer prefix count of fg (from a foreground
//            histogram), dJ from the integer counts
//                fg step: dJ = 1/U,   bg step: dJ = I/(U*(U+1)),   U = 0 (no fg, first) -> 1
//            with I = remaining fg, U = union before the step; accumulates err*dJ and scatters
//            dJ to pixel order (the `jacc` output).
//   backward one tile kernel: softmax recomputed, g = p*(gp - sum p*gp), zero at ignored pixels.
//
// Key bits.  Swapping two neighbours of the sorted order moves the loss by (their error
// difference) x (their dJ difference) and their dJ by the step between adjacent ranks, which is
// at most 1/U^2 with U >= n_pos (the segment's foreground count).  A segment with n_pos >=
// kFastMinFg that sorts at least kFastMinKept elements is therefore sorted on the top 20 of its 30
// error bits only ("fast": two passes instead of three): elements whose errors agree to 2^-13
// relative may come out in either order, which moves a pixel's dJ by at most 1/4096^2 = 6e-8
// (measured on 1 Mpixel segments with 55 000 foreground pixels: 1.7e-9 absolute, 8e-5 of the
// largest dJ of the class, loss 4e-13 relative) -- far inside the 1e-5 gradient tolerance.  The
// reference's own order among such near-ties is no better defined: its errors carry the
// rounding of its own softmax (1e-7 relative) and thrust's sort is not stable.  Fast segments
// are also ranked with one shared-memory atomic per element (see rank_round); every other
// segment takes three stable passes over all 30 bits, exact array order among equal keys.
#include "common.cuh"
#include "pipeline.cuh"

#include <cstdlib>
#include <utility>
#include <type_traits>

namespace b200 {
namespace {

constexpr int kBits = 10;
constexpr int kBins = 1 << kBits;
constexpr int kPasses = 3;                 // key bits 1..30; "fast" segments skip the first pass (see Key bits)
constexpr uint32_t kFastMinFg = 4096;      // foreground elements a segment needs to sort on 20 bits
constexpr uint32_t kFastMinKept = 32u * kBins;   // ... and elements it sorts
constexpr int kSortThreads = 256;
constexpr int kSortItems = 32;
constexpr int kSortTile = kSortThreads * kSortItems;   // 8192 pairs per tile
constexpr int kSortWarps = kSortThreads / 32;
static_assert(kBins % kSortThreads == 0, "each thread scans kBins / kSortThreads bins");
constexpr uint32_t kKeyIgnored = 0xFFFFFFFFu;
constexpr uint32_t kOneBits = 0x3F800000u;

constexpr int kTileThreads = 256;

__device__ __forceinline__ uint32_t lanemask_lt() {
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// ---------------------------------------------------------------- geometry

struct LovaszGeom {
    int64_t N, C, M;
    int per_image;
    int64_t G, L, S;          // groups, pixels per group, segments
    int64_t T;                // sort tiles per segment
    // tile kernels
    int TP, KS, CB, nbox, rows;
    int64_t tiles_per_image, total_tiles;
};

struct Workspace {
    uint32_t *keysA, *keysB, *valsA, *valsB;
    uint32_t *hist;       // [S][T][kBins]
    uint32_t *fghist;     // [S][T][kBins]  (last pass)
    uint32_t *n_pos;      // [S]
    double *partial;      // [S][T]
    unsigned *status;     // 1 word
    uint32_t *maxfg;      // [S]  largest foreground key seen (0: none)
    uint32_t *minkey;     // [S]  smallest key among the sampled tiles (0xFFFFFFFF: none)
    uint32_t *kept;       // [S][T] kept elements per tile -> exclusive offsets
    uint32_t *fgkept;     // [S][T] foreground elements per tile
    uint32_t *Lp;         // [S]  elements of the segment that go through the sort
    uint32_t *direct;     // [S]  segment flags: kSegFlagDirect (sorted from the full key array, not compacted), kSegFlagFast
    uint2 *tilemap;       // [S*T] (segment, tile) of every sort tile in use, segment-major
    uint32_t *n_tiles;    // 1 word: sort tiles in use
    size_t bytes;
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

Workspace carve(void *base, const LovaszGeom &g) {
    Workspace w{};
    char *p = static_cast<char *>(base);
    size_t off = 0;
    const size_t e = size_t(g.S) * g.L;
    auto take = [&](size_t bytes) {
        char *r = p ? p + off : nullptr;
        off += align256(bytes);
        return r;
    };
    w.status = reinterpret_cast<unsigned *>(take(256));
    w.maxfg = reinterpret_cast<uint32_t *>(take(size_t(g.S) * 4));
    w.minkey = reinterpret_cast<uint32_t *>(take(size_t(g.S) * 4));
    w.kept = reinterpret_cast<uint32_t *>(take(size_t(g.S) * g.T * 4));
    w.fgkept = reinterpret_cast<uint32_t *>(take(size_t(g.S) * g.T * 4));
    w.Lp = reinterpret_cast<uint32_t *>(take(size_t(g.S) * 4));
    w.direct = reinterpret_cast<uint32_t *>(take(size_t(g.S) * 4));
    w.tilemap = reinterpret_cast<uint2 *>(take(size_t(g.S) * g.T * 8));
    w.n_tiles = reinterpret_cast<uint32_t *>(take(256));
    w.keysA = reinterpret_cast<uint32_t *>(take(e * 4));
    w.keysB = reinterpret_cast<uint32_t *>(take(e * 4));
    w.valsA = reinterpret_cast<uint32_t *>(take(e * 4));
    w.valsB = reinterpret_cast<uint32_t *>(take(e * 4));
    w.hist = reinterpret_cast<uint32_t *>(take(size_t(g.S) * g.T * kBins * 4));
    w.fghist = reinterpret_cast<uint32_t *>(take(size_t(g.S) * g.T * kBins * 4));
    w.n_pos = reinterpret_cast<uint32_t *>(take(size_t(g.S) * 4));
    w.partial = reinterpret_cast<double *>(take(size_t(g.S) * g.T * 8));
    w.bytes = off;
    return w;
}

bool make_geom(LovaszGeom &g, int64_t N, int64_t C, int64_t M, int per_image) {
    g.N = N; g.C = C; g.M = M; g.per_image = per_image;
    g.G = per_image ? N : 1;
    g.L = per_image ? M : N * M;
    g.S = g.G * C;
    g.T = (g.L + kSortTile - 1) / kSortTile;
    int TP = 256;
    while (TP > 32 && size_t(C) * TP * 4 > 40 * 1024) TP >>= 1;
    while (TP > 32 && TP / 2 >= M) TP >>= 1;
    g.TP = TP;
    g.KS = kTileThreads / TP;
    g.nbox = int((C + 255) / 256);
    g.CB = int((C + g.nbox - 1) / g.nbox);
    g.rows = g.nbox * g.CB;
    g.tiles_per_image = (M + TP - 1) / TP;
    g.total_tiles = N * g.tiles_per_image;
    return true;
}

// --------------------------------------------------- tile kernels (keys, backward)

struct TileArgs {
    const float *logits;
    const int64_t *labels;
    uint32_t *keys;          // keys kernel: segment-major output
    const float *jacc;       // backward: segment-major input
    const float *seg_grad;   // backward: [S]
    float *grads;            // backward: [N, C, M]
    uint32_t *maxfg;         // keys kernel: per-segment trackers of the pruning bound
    uint32_t *minkey;
    unsigned *status;
    int64_t ignore;
    LovaszGeom g;
};

// Offset of (image n, class c, pixel m) in a segment-major array.
__device__ __forceinline__ int64_t seg_offset(const LovaszGeom &g, int64_t n, int64_t c, int64_t m) {
    return g.per_image ? (n * g.C + c) * g.M + m : c * (g.N * g.M) + n * g.M + m;
}

// Pruning bound of a segment.  Once the last foreground element of a class has gone by in the
// sorted order, the intersection count is zero and every later element has dJ = 0 exactly: it
// adds nothing to the loss and its gradient weight is zero.  So only elements whose error is
// at least the SMALLEST foreground error (the largest foreground key) need sorting; a class
// without foreground pixels needs only its largest error, for which any lower bound of it (the
// smallest key among a sample of the tiles) serves.  The keys kernels track both per segment.
//
// One pixel's foreground key: when the whole warp holds the same class (the usual case inside
// an object) one redux + one atomic, else one atomic per lane.
__device__ __forceinline__ void track_fg(uint32_t *maxfg, int cls, uint32_t key, int lane) {
    const int c0 = __shfl_sync(0xffffffffu, cls, 0);
    if (__all_sync(0xffffffffu, cls == c0)) {
        if (c0 >= 0) {
            const uint32_t v = __reduce_max_sync(0xffffffffu, key);
            if (lane == 0) atomicMax(maxfg + c0, v);
        }
    } else if (cls >= 0) {
        atomicMax(maxfg + cls, key);
    }
}
constexpr int kSampleEvery = 16;    // tiles of an image whose keys feed the smallest-key sample

// BWD = false: logits tile -> key tile (in place, 4 bytes each) -> keys.
// BWD = true : logits tile + jacc tile -> gradient tile (in place) -> grads.
template <bool BWD, bool TMA>
__global__ void __launch_bounds__(kTileThreads)
lovasz_tile_kernel(const TileArgs a, const __grid_constant__ CUtensorMap map_logits,
                   const __grid_constant__ CUtensorMap map_seg,
                   const __grid_constant__ CUtensorMap map_grads) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    const LovaszGeom &g = a.g;
    const int TP = g.TP, KS = g.KS, C = int(g.C);
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const size_t tile_bytes_al = (size_t(g.rows) * TP * 4 + 127) & ~size_t(127);
    float *tile = reinterpret_cast<float *>(base);
    float *jt = reinterpret_cast<float *>(base + tile_bytes_al);                 // BWD only
    float *red = reinterpret_cast<float *>(base + (BWD ? 2 : 1) * tile_bytes_al);  // [2][256]

    const int tid = threadIdx.x, p = tid % TP, ks = tid / TP, slab = KS * TP;
    if (TMA && tid == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    uint32_t phase = 0;
    const uint32_t tx_bytes = uint32_t(g.nbox) * g.CB * TP * 4 * (BWD ? 2 : 1);

    for (int64_t t = blockIdx.x; t < g.total_tiles; t += gridDim.x) {
        const int64_t n = t / g.tiles_per_image;
        const int64_t p0 = (t % g.tiles_per_image) * TP;
        const int64_t img_base = n * g.C * g.M;
        if (TMA) {
            if (tid == 0) {
                mbar_expect_tx(&bar, tx_bytes);
                for (int b = 0; b < g.nbox; ++b) {
                    tma_load_3d(tile + size_t(b) * g.CB * TP, &map_logits, int(p0), b * g.CB, int(n), &bar);
                    if (BWD) tma_load_3d(jt + size_t(b) * g.CB * TP, &map_seg, int(p0), b * g.CB, int(n), &bar);
                }
            }
        } else {
            for (int idx = tid; idx < C * TP; idx += kTileThreads) {
                const int j = idx / TP, pp = idx % TP;
                const int64_t px = p0 + pp;
                tile[idx] = px < g.M ? a.logits[img_base + int64_t(j) * g.M + px] : 0.f;
                if (BWD) jt[idx] = px < g.M ? a.jacc[seg_offset(g, n, j, px)] : 0.f;
            }
        }
        const int64_t pix = p0 + p;
        const bool inb = pix < g.M;
        const int64_t lb = inb ? a.labels[n * g.M + pix] : a.ignore;
        const bool valid = inb && lb != a.ignore;
        if (TMA) {
            const bool ok = mbar_wait_bounded(&bar, phase, a.status);
            if (!__syncthreads_and(ok)) break;
            phase ^= 1;
        } else {
            __syncthreads();
        }
        float *col = tile + p;
        // softmax statistics
        float m = -3.402823466e38f;
        for (int j = ks; j < C; j += KS) m = fmaxf(m, col[j * TP]);
        if (KS > 1) {
            red[tid] = m;
            __syncthreads();
            for (int q = 0; q < KS; ++q) m = fmaxf(m, red[q * TP + p]);
        }
        float s = 0.f;
        for (int j = ks; j < C; j += KS) s += exp_fast(col[j * TP] - m);
        if (KS > 1) {
            red[slab + tid] = s;
            __syncthreads();
            s = 0.f;
            for (int q = 0; q < KS; ++q) s += red[slab + q * TP + p];
        }
        const float inv_s = 1.f / s;

        if (!BWD) {
            uint32_t *kcol = reinterpret_cast<uint32_t *>(col);
            const int64_t seg0 = g.per_image ? n * g.C : 0;
            const bool sample = (t % g.tiles_per_image) % kSampleEvery == 0;
            uint32_t kfg = 0;
            for (int j = ks; j < C; j += KS) {
                uint32_t key = kKeyIgnored;
                if (valid) {
                    const float pr = exp_fast(col[j * TP] - m) * inv_s;
                    const bool fg = (j == lb);
                    const float err = fg ? 1.f - pr : pr;
                    uint32_t eb = __float_as_uint(fmaxf(err, 0.f));
                    eb = eb > kOneBits ? kOneBits : eb;
                    key = ((kOneBits - eb) << 1) | (fg ? 1u : 0u);
                    if (fg) kfg = key;
                }
                kcol[j * TP] = key;
                if (sample) {       // a warp shares its channel slice: same j in every lane
                    const uint32_t v = __reduce_min_sync(0xffffffffu, key);
                    if ((tid & 31) == 0 && v != kKeyIgnored) atomicMin(a.minkey + seg0 + j, v);
                }
            }
            track_fg(a.maxfg + seg0, kfg ? int(lb) : -1, kfg, tid & 31);
        } else {
            const float *jcol = jt + p;
            const int64_t gseg = g.per_image ? n * g.C : 0;
            float dot = 0.f;
            for (int j = ks; j < C; j += KS) {
                const float pr = exp_fast(col[j * TP] - m) * inv_s;
                const float gp = (j == lb ? -jcol[j * TP] : jcol[j * TP]) * a.seg_grad[gseg + j];
                dot += pr * gp;
            }
            if (KS > 1) {
                __syncthreads();          // red[0..slab) is free again (everyone has read the maxima)
                red[tid] = dot;
                __syncthreads();
                dot = 0.f;
                for (int q = 0; q < KS; ++q) dot += red[q * TP + p];
            }
            for (int j = ks; j < C; j += KS) {
                float gl = 0.f;
                if (valid) {
                    const float pr = exp_fast(col[j * TP] - m) * inv_s;
                    const float gp = (j == lb ? -jcol[j * TP] : jcol[j * TP]) * a.seg_grad[gseg + j];
                    gl = pr * (gp - dot);
                }
                col[j * TP] = gl;
            }
        }
        // write the tile back
        if (TMA) {
            fence_proxy_async_smem();
            __syncthreads();
            if (tid == 0) {
                for (int b = 0; b < g.nbox; ++b)
                    tma_store_3d(BWD ? &map_grads : &map_seg, int(p0), b * g.CB, int(n),
                                 tile + size_t(b) * g.CB * TP);
                bulk_commit();
                bulk_wait_read_all();
            }
        } else {
            __syncthreads();
            for (int idx = tid; idx < C * TP; idx += kTileThreads) {
                const int j = idx / TP, pp = idx % TP;
                const int64_t px = p0 + pp;
                if (px < g.M) {
                    if (BWD) a.grads[img_base + int64_t(j) * g.M + px] = tile[idx];
                    else a.keys[seg_offset(g, n, j, px)] = reinterpret_cast<uint32_t *>(tile)[idx];
                }
            }
            __syncthreads();
        }
    }
    if (TMA && tid == 0) bulk_wait_all();
}

// ------------------------------------------------- keys / backward for unaligned layouts
//
// Images whose pixel count is not a multiple of 4 (769 x 769 crops), or unaligned pointers: no
// tensor map.  Up to CMAX classes: a thread owns ONE pixel and keeps all its channels in
// registers (4-byte accesses, 128 contiguous bytes per warp and channel, every load of a thread
// in flight together); a block walks groups of 256 adjacent pixels of one image, so a warp never
// spans two images.  Same arithmetic as lovasz_tile_kernel.
constexpr int kAnyThreads = 256;
template <bool BWD, int CMAX>
__global__ void __launch_bounds__(kAnyThreads, BWD ? 2 : 3)
lovasz_any_kernel(const TileArgs a) {
    const LovaszGeom &g = a.g;
    const int C = int(g.C);
    const int lane = threadIdx.x & 31;
    const int64_t groups_per_image = (g.M + kAnyThreads - 1) / kAnyThreads;
    const int64_t groups = g.N * groups_per_image;
    for (int64_t gi = blockIdx.x; gi < groups; gi += gridDim.x) {
        const int64_t n = gi / groups_per_image, grp = gi % groups_per_image;
        const int64_t pix = grp * kAnyThreads + threadIdx.x;
        const bool inb = pix < g.M;
        const int64_t img_base = n * g.C * g.M + (inb ? pix : 0);
        float xv[CMAX], jv[BWD ? CMAX : 1];
#pragma unroll
        for (int j = 0; j < CMAX; ++j) {
            if (j < C) {
                xv[j] = inb ? __ldcs(a.logits + img_base + int64_t(j) * g.M) : 0.f;
                if (BWD) jv[j] = inb ? __ldcs(a.jacc + seg_offset(g, n, j, pix)) : 0.f;
            }
        }
        const int64_t lb = inb ? a.labels[n * g.M + pix] : a.ignore;
        const bool valid = inb && lb != a.ignore;
        float m = -3.402823466e38f;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) m = fmaxf(m, xv[j]);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < CMAX; ++j)
            if (j < C) {
                xv[j] = exp_fast(xv[j] - m);              // e^{x-m} takes x's place
                s += xv[j];
            }
        const float inv_s = 1.f / s;
        if (!BWD) {
            const int64_t seg0 = g.per_image ? n * g.C : 0;
            const bool sample = grp % (2 * kSampleEvery) == 0;    // (256-pixel groups: half a 512-pixel tile)
            uint32_t kfg = 0;
#pragma unroll
            for (int j = 0; j < CMAX; ++j) {
                if (j < C) {
                    uint32_t key = kKeyIgnored;
                    if (valid) {
                        const float pr = xv[j] * inv_s;
                        const bool fg = (j == lb);
                        const float err = fg ? 1.f - pr : pr;
                        uint32_t eb = __float_as_uint(fmaxf(err, 0.f));
                        eb = eb > kOneBits ? kOneBits : eb;
                        key = ((kOneBits - eb) << 1) | (fg ? 1u : 0u);
                        if (fg) kfg = key;
                    }
                    if (inb) a.keys[seg_offset(g, n, j, pix)] = key;
                    if (sample) {        // every lane of the warp is at the same j
                        const uint32_t v = __reduce_min_sync(0xffffffffu, key);
                        if (lane == 0 && v != kKeyIgnored) atomicMin(a.minkey + seg0 + j, v);
                    }
                }
            }
            track_fg(a.maxfg + seg0, kfg ? int(lb) : -1, kfg, lane);
        } else {
            const int64_t gseg = g.per_image ? n * g.C : 0;
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < CMAX; ++j)
                if (j < C) {
                    jv[j] = (j == lb ? -jv[j] : jv[j]) * __ldg(a.seg_grad + gseg + j);    // gp
                    dot += xv[j] * inv_s * jv[j];
                }
            if (inb) {
#pragma unroll
                for (int j = 0; j < CMAX; ++j)
                    if (j < C) __stcs(a.grads + img_base + int64_t(j) * g.M, valid ? xv[j] * inv_s * (jv[j] - dot) : 0.f);
            }
        }
    }
}

// -------------------------------------------- pipelined pair-per-thread tile kernels
//
// The production form of the keys and backward kernels for few classes (a tile of all C
// channels x 512 pixels fits one shared-memory stage).  Block = 256 compute threads + a loader
// warp + a storer warp on the mbarrier ring of pipeline.cuh; a stage holds the logits tile
// (two TMA boxes of 256 pixels side by side), in backward the dJ tile behind it, and the 512
// labels of the tile.  A compute thread owns two adjacent pixels over ALL channels, so the
// per-pixel statistics never leave its registers, and every sweep moves 8-byte pairs through
// packed fp32x2 arithmetic.  The label channel is not compared per element: the thread edits
// that one element of its column instead (keys: rewrites the key after the sweep; backward:
// flips the sign of dJ before it).

constexpr int kPairTP = 256;               // pixels per TMA box
constexpr int kPairTile = 2 * kPairTP;     // pixels per tile
constexpr int kPairMaxC = 40;              // classes whose 256-pixel box stays within 40 KB

struct PairLayout {
    int box_elems;          // floats of one box (C * 256)
    uint32_t tile_bytes;    // one C x 512 fp32 tile
    uint32_t label_off;     // byte offset of the labels inside a stage
    uint32_t coord_off;     // (image, first pixel) of the tile, written by the loader
    uint32_t stage_bytes;
};

__host__ __device__ inline PairLayout pair_layout(int C, bool bwd) {
    PairLayout l;
    l.box_elems = C * kPairTP;
    l.tile_bytes = uint32_t(C) * kPairTile * 4u;
    l.label_off = (bwd ? 2u : 1u) * l.tile_bytes;          // multiples of 2 KB: 128-byte aligned
    l.coord_off = l.label_off + kPairTile * 8u;
    l.stage_bytes = l.coord_off + 128u;                     // stages stay 128-byte aligned
    return l;
}

template <bool BWD>
__global__ void __launch_bounds__(kTileBlock)
lovasz_pair_kernel(const TileArgs a, const int NS, const __grid_constant__ CUtensorMap map_logits,
                   const __grid_constant__ CUtensorMap map_seg,
                   const __grid_constant__ CUtensorMap map_grads) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ PipeBarriers bars;
    const LovaszGeom &g = a.g;
    const int C = int(g.C);
    const PairLayout lay = pair_layout(C, BWD);
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int tid = threadIdx.x;
    const int64_t tiles_per_image = (g.M + kPairTile - 1) / kPairTile;
    const int64_t total_tiles = g.N * tiles_per_image;
    const int64_t first = blockIdx.x, stride = gridDim.x;

    // keys: block-level trackers of the pruning bound, flushed to the segment's words when the
    // block moves to another image (per-image segments) and at the end
    __shared__ uint32_t blk_maxfg[kPairMaxC], blk_min[kPairMaxC];
    if (!BWD && tid < kPairMaxC) {
        blk_maxfg[tid] = 0u;
        blk_min[tid] = kKeyIgnored;
    }
    // keys: the storer frees the stage, as in backward
    pipe_init<kTileCompute, true>(bars, NS);

    if (tid == kTileCompute) {
        int k = 0;
        for (int64_t t = first; t < total_tiles; t += stride, ++k) {
            const int s = k % NS;
            if (k >= NS && !mbar_wait_bounded(&bars.empty[s], ((k / NS) - 1) & 1, a.status)) break;
            const int64_t n = t / tiles_per_image;
            const int64_t p0 = (t % tiles_per_image) * kPairTile;
            unsigned char *stage = base + size_t(s) * lay.stage_bytes;
            float *lt = reinterpret_cast<float *>(stage);
            float *jt = reinterpret_cast<float *>(stage + lay.tile_bytes);
            int64_t npix = g.M - p0;
            if (npix > kPairTile) npix = kPairTile;
            const int nbx = int((npix + kPairTP - 1) / kPairTP);
            const uint32_t label_bytes = uint32_t(npix) * 8u;        // M % 4 == 0: a multiple of 16
            *reinterpret_cast<int2 *>(stage + lay.coord_off) = make_int2(int(n), int(p0));
            mbar_expect_tx(&bars.full[s], uint32_t(nbx) * (BWD ? 2u : 1u) * (lay.tile_bytes / 2) + label_bytes);
            for (int bx = 0; bx < nbx; ++bx) {
                tma_load_3d(lt + size_t(bx) * lay.box_elems, &map_logits, int(p0) + bx * kPairTP, 0, int(n),
                            &bars.full[s]);
                if (BWD)
                    tma_load_3d(jt + size_t(bx) * lay.box_elems, &map_seg, int(p0) + bx * kPairTP, 0, int(n),
                                &bars.full[s]);
            }
            bulk_load_1d(stage + lay.label_off, a.labels + n * g.M + p0, label_bytes, &bars.full[s]);
        }
    } else if (tid == kTileCompute + 32) {
        int k = 0;
        for (int64_t t = first; t < total_tiles; t += stride, ++k) {
            const int s = k % NS;
            if (!mbar_wait_bounded(&bars.ready[s], (k / NS) & 1, a.status)) break;
            const int64_t n = t / tiles_per_image;
            const int64_t p0 = (t % tiles_per_image) * kPairTile;
            const float *lt = reinterpret_cast<const float *>(base + size_t(s) * lay.stage_bytes);
            int64_t npix = g.M - p0;
            if (npix > kPairTile) npix = kPairTile;
            const int nbx = int((npix + kPairTP - 1) / kPairTP);
            for (int bx = 0; bx < nbx; ++bx)
                tma_store_3d(BWD ? &map_grads : &map_seg, int(p0) + bx * kPairTP, 0, int(n),
                             lt + size_t(bx) * lay.box_elems);
            bulk_commit();
            bulk_wait_read_all();
            mbar_arrive(&bars.empty[s]);
        }
        bulk_wait_all();
    } else if (tid < kTileCompute) {
        const int lane = tid & 31;
        const int pix = tid * 2;                                          // my pair inside the tile
        const int bxo = (pix / kPairTP) * lay.box_elems + (pix % kPairTP);   // its offset in channel 0
        auto flush_trackers = [&](int64_t img) {
            compute_sync(kTileCompute);
            if (tid < C) {
                const int64_t seg = (g.per_image ? img * C : 0) + tid;
                if (blk_maxfg[tid]) atomicMax(a.maxfg + seg, blk_maxfg[tid]);
                if (blk_min[tid] != kKeyIgnored) atomicMin(a.minkey + seg, blk_min[tid]);
                blk_maxfg[tid] = 0u;
                blk_min[tid] = kKeyIgnored;
            }
            compute_sync(kTileCompute);
        };
        int64_t cur_n = -1;
        int k = 0;
        for (int64_t t = first; t < total_tiles; t += stride, ++k) {
            const int s = k % NS;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(&bars.full[s], (k / NS) & 1, a.status);
            // keys: the tracker flushes below meet at a block barrier, so the warps give up together;
            // backward: a warp owns whole pixel columns and decides for itself
            if (BWD) {
                if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            } else if (!compute_all(ok, kTileCompute)) {
                break;
            }
            unsigned char *stage = base + size_t(s) * lay.stage_bytes;
            const int2 coord = *reinterpret_cast<const int2 *>(stage + lay.coord_off);
            const int64_t n = coord.x;
            const int64_t px0 = int64_t(coord.y) + pix;
            if (!BWD && g.per_image && n != cur_n && cur_n >= 0) flush_trackers(cur_n);
            cur_n = n;

            const int64_t *tile_labels = reinterpret_cast<const int64_t *>(stage + lay.label_off);
            bool valid[2];
            int lbi[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bool inb = px0 + i < g.M;
                const int64_t lb = inb ? tile_labels[pix + i] : a.ignore;
                valid[i] = inb && lb != a.ignore;
                lbi[i] = (valid[i] && lb >= 0 && lb < C) ? int(lb) : -1;   // -1: no foreground channel
            }
            float *mine = reinterpret_cast<float *>(stage) + bxo;

            // ---- sweep 1: maximum
            float2 m = splat2(-3.402823466e38f);
            {
                const float *q = mine;
#pragma unroll 4
                for (int j = 0; j < C; ++j, q += kPairTP) m = max2(m, ld_pair(q));
            }
            // ---- sweep 2: e = 2^((x - m) log2 e) left in the tile, and its sum
            float2 sum;
            {
                const pk_t nml = pk2(mul2(m, splat2(-kLog2e))), l2e = psplat(kLog2e);
                pk_t psum = psplat(0.f);
                float *q = mine;
#pragma unroll 4
                for (int j = 0; j < C; ++j, q += kPairTP) {
                    const pk_t e = pex2(pfma(ld_pk(q), l2e, nml));
                    psum = padd(psum, e);
                    st_pk(q, e);
                }
                sum = upk2(psum);
            }
            const float2 inv = make_float2(__fdividef(1.f, sum.x), __fdividef(1.f, sum.y));

            if constexpr (!BWD) {
                // ---- sweep 3: key = ((bits(1.0) - bits(err)) << 1) | fg with err = p off the label
                // channel; an ignored pixel gets multiplier 0 and addend 0xFFFFFFFF instead.
                float e_lb[2] = {0.f, 0.f};
                if (lbi[0] >= 0) e_lb[0] = mine[lbi[0] * kPairTP];
                if (lbi[1] >= 0) e_lb[1] = mine[lbi[1] * kPairTP + 1];
                const uint32_t mul0 = valid[0] ? 0xFFFFFFFEu : 0u, add0 = valid[0] ? 2u * kOneBits : kKeyIgnored;
                const uint32_t mul1 = valid[1] ? 0xFFFFFFFEu : 0u, add1 = valid[1] ? 2u * kOneBits : kKeyIgnored;
                const pk_t pinv = pk2(inv);
                auto key_sweep = [&](auto sampled) {
                    float *q = mine;
#pragma unroll 4
                    for (int j = 0; j < C; ++j, q += kPairTP) {
                        const float2 p = upk2(pmul(ld_pk(q), pinv));
                        const uint32_t b0 = min(__float_as_uint(p.x), kOneBits);
                        const uint32_t b1 = min(__float_as_uint(p.y), kOneBits);
                        uint2 key;
                        key.x = b0 * mul0 + add0;
                        key.y = b1 * mul1 + add1;
                        *reinterpret_cast<uint2 *>(q) = key;
                        if (decltype(sampled)::value) {
                            // (the label channel still holds its background-style key here; the
                            // sample only matters for classes that have no label pixel at all)
                            const uint32_t v = __reduce_min_sync(0xffffffffu, min(key.x, key.y));
                            if (lane == 0) atomicMin(&blk_min[j], v);
                        }
                    }
                };
                if ((coord.y / kPairTile) % kSampleEvery == 0) key_sweep(std::true_type{});
                else key_sweep(std::false_type{});
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t kf = 0u;
                    if (lbi[i] >= 0) {
                        const float err = fmaxf(1.f - e_lb[i] * (i ? inv.y : inv.x), 0.f);
                        const uint32_t eb = min(__float_as_uint(err), kOneBits);
                        kf = ((kOneBits - eb) << 1) | 1u;
                        reinterpret_cast<uint32_t *>(mine)[lbi[i] * kPairTP + i] = kf;
                    }
                    track_fg(blk_maxfg, lbi[i], kf, lane);
                }
            } else {
                float *jmine = reinterpret_cast<float *>(stage + lay.tile_bytes) + bxo;
                const float *go = a.seg_grad + (g.per_image ? n * g.C : 0);
                // the label channel's dJ enters with the opposite sign
                if (lbi[0] >= 0) jmine[lbi[0] * kPairTP] = -jmine[lbi[0] * kPairTP];
                if (lbi[1] >= 0) jmine[lbi[1] * kPairTP + 1] = -jmine[lbi[1] * kPairTP + 1];
                // ---- sweep 3: gp = dJ * dL/dloss_c (left in the dJ tile), dot = sum e * gp
                float2 dot;
                {
                    pk_t pdot = psplat(0.f);
                    const float *q = mine;
                    float *jq = jmine;
#pragma unroll 4
                    for (int j = 0; j < C; ++j, q += kPairTP, jq += kPairTP) {
                        const pk_t gp = pmul(ld_pk(jq), psplat(__ldg(go + j)));
                        pdot = pfma(ld_pk(q), gp, pdot);
                        st_pk(jq, gp);
                    }
                    dot = upk2(pdot);
                }
                // ---- sweep 4: g = p * (gp - sum p gp) = e * (gp * inv - dot * inv^2); 0 if ignored
                const float2 iv = make_float2(valid[0] ? inv.x : 0.f, valid[1] ? inv.y : 0.f);
                const pk_t piv = pk2(iv);
                const pk_t pc = pk2(make_float2(-dot.x * iv.x * iv.x, -dot.y * iv.y * iv.y));
                {
                    float *q = mine;
                    const float *jq = jmine;
#pragma unroll 4
                    for (int j = 0; j < C; ++j, q += kPairTP, jq += kPairTP)
                        st_pk(q, pmul(ld_pk(q), pfma(ld_pk(jq), piv, pc)));
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.ready[s]);
        }
        if (!BWD && cur_n >= 0) flush_trackers(cur_n);
    }
}

// ------------------------------------------------------------------ sort kernels
//
// Element order inside a tile is "warp-striped": warp w owns the contiguous chunk
// [w*32*kSortItems, (w+1)*32*kSortItems) and in round r its lane l holds element
// chunk + r*32 + l, so every global access of a round is one coalesced 128-byte line and
// (warp, round, lane) order equals array order -- which is what makes the ranking stable.

__device__ __forceinline__ uint32_t digit_of(uint32_t key, int shift) {
    return (key >> shift) & (kBins - 1);
}
__device__ __forceinline__ bool key_is_fg(uint32_t key) { return (key & 1u) && key != kKeyIgnored; }

// One entry of the list of sort tiles in use: everything a block needs to start on the tile,
// in one 8-byte load.   x = segment | direct << 30 | fast << 31,
//                       y = tile | (elements - 1) << 18 | swapped << 31
// The launches pass the two buffer pairs in the roles they have for a compacted segment that
// takes all three passes (B -> A -> B, ranked from B).  A segment that was not compacted
// (`direct`) starts in A, and a `fast` segment skips the first pass: either shifts the segment's
// data to the other pair in every pass it takes, both together cancel: swapped = direct ^ fast.
struct TileRef {
    int64_t seg, tile;
    int n;
    bool direct;       // the segment was not compacted: its first pass makes up the values (positions)
    bool fast;         // two passes on the top 20 key bits, atomic ranking
    bool swapped;      // the segment uses the two buffer pairs in swapped roles
};
constexpr uint32_t kSegFlagDirect = 1u, kSegFlagFast = 2u;
__device__ __forceinline__ uint2 encode_tile(uint32_t seg, uint32_t tile, uint32_t n, uint32_t flags) {
    const bool direct = flags & kSegFlagDirect, fast = flags & kSegFlagFast;
    return make_uint2(seg | (direct ? 0x40000000u : 0u) | (fast ? 0x80000000u : 0u),
                      tile | ((n - 1u) << 18) | (direct != fast ? 0x80000000u : 0u));
}
__device__ __forceinline__ TileRef decode_tile(uint2 e) {
    TileRef t;
    t.seg = e.x & 0x3FFFFFFFu;
    t.direct = (e.x >> 30) & 1u;
    t.fast = (e.x >> 31) != 0u;
    t.tile = e.y & 0x3FFFFu;
    t.n = int((e.y >> 18) & 0x1FFFu) + 1;
    t.swapped = (e.y >> 31) != 0u;
    return t;
}
// The block's next tile: thread 0 draws a ticket while the tile's key loads are in flight, and
// later pulls the list entry into L2, so the next iteration starts without a chain of misses.
__device__ __forceinline__ void draw_next_tile(uint32_t *next, unsigned *ticket) {
    if (threadIdx.x == 0) *next = gridDim.x + atomicAdd(ticket, 1u);
}
__device__ __forceinline__ void prefetch_next_tile(const uint32_t *next, const uint2 *tilemap, uint32_t total) {
    if (threadIdx.x == 0) {
        const uint32_t w = *next;
        if (w < total) asm volatile("prefetch.global.L2 [%0];" ::"l"(tilemap + w));
    }
}

// Elements with (key >> 1) >= the segment's limit are past the pruning bound (see track_fg):
// the first sort pass drops them.
__device__ __forceinline__ uint32_t prune_limit(const uint32_t *maxfg, const uint32_t *minkey, int64_t seg,
                                                int prune) {
    if (!prune) return 0x80000000u;                       // keep everything, ignored pixels included
    const uint32_t mf = __ldg(maxfg + seg);
    if (mf) return (mf >> 1) + 1u;                        // up to the last foreground element (ties too)
    const uint32_t mk = __ldg(minkey + seg);
    return mk != kKeyIgnored ? (mk >> 1) + 1u : 0x80000000u;
}

// Per-tile digit histogram (plain shared-memory atomics: cost follows the multiplicity of a
// digit inside a warp, which is low for the uniform low digits and bounded by 32 otherwise).
// LAST: also a histogram of the foreground elements.   hist[seg][tile][bin]
// Segments flagged in `direct` (sorted from the full array) use the two buffers in swapped roles:
// their input of this pass is keys_alt.
template <bool LAST>
__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const uint32_t *__restrict__ keys, uint32_t *__restrict__ hist,
                 uint32_t *__restrict__ fghist, const uint2 *__restrict__ tilemap,
                 const uint32_t *__restrict__ n_tiles, const uint32_t *__restrict__ keys_alt, int64_t L, int64_t T,
                 int shift, int first_pass) {
    __shared__ uint32_t sh[kBins];
    __shared__ uint32_t shfg[LAST ? kBins : 1];
    const uint32_t total = __ldg(n_tiles);
  for (uint32_t w = blockIdx.x; w < total; w += gridDim.x) {
    const TileRef tr = decode_tile(__ldg(tilemap + w));
    if (first_pass && tr.fast) continue;               // fast segments have no first pass
    const int64_t seg = tr.seg, tile = tr.tile;
    const int64_t t0 = tile * kSortTile;
    const int n = tr.n;
    const uint32_t *src = (tr.swapped ? keys_alt : keys) + seg * L + t0;
    for (int b = threadIdx.x; b < kBins; b += kSortThreads) {
        sh[b] = 0;
        if (LAST) shfg[b] = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wbase = warp * (32 * kSortItems);
    uint32_t key[kSortItems];
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        key[r] = idx < n ? __ldg(src + idx) : 0u;
    }
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        if (idx < n) {
            const uint32_t d = digit_of(key[r], shift);
            atomicAdd(&sh[d], 1u);
            if (LAST && key_is_fg(key[r])) atomicAdd(&shfg[d], 1u);
        }
    }
    __syncthreads();
    const int64_t o = (seg * T + tile) * kBins;
    for (int b = threadIdx.x; b < kBins; b += kSortThreads) {
        hist[o + b] = sh[b];
        if (LAST) fghist[o + b] = shfg[b];
    }
    __syncthreads();
  }
}

// Exclusive scan of kBins per-thread values across a block of kBins threads.
__device__ __forceinline__ uint32_t block_excl_scan_1024(uint32_t v, uint32_t *warp_tot, uint32_t *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const uint32_t w = warp_tot[lane];
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += u;
        }
        warp_tot[lane] = wi - w;
        if (lane == 31 && total) *total = wi;
    }
    __syncthreads();
    return warp_tot[warp] + incl - v;
}

// Per-segment scan: counts hist[seg][tile][bin] -> exclusive offsets inside the segment in
// (bin, tile) order.  One block of kBins threads per segment.  LAST: the foreground
// histogram gets the same treatment and its grand total is the segment's n_pos.
template <bool LAST>
__global__ void __launch_bounds__(kBins)
sort_scan_kernel(uint32_t *__restrict__ hist, uint32_t *__restrict__ fghist,
                 uint32_t *__restrict__ n_pos, const uint32_t *__restrict__ Lp,
                 const uint32_t *__restrict__ seg_flags, int64_t T, int first_pass) {
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t grand;
    const int64_t seg = blockIdx.x;
    if (first_pass && (__ldg(seg_flags + seg) & kSegFlagFast)) return;
    const int b = threadIdx.x;
    const int64_t Tk = (int64_t(__ldg(Lp + seg)) + kSortTile - 1) / kSortTile;   // tiles in use
#pragma unroll
    for (int which = 0; which < (LAST ? 2 : 1); ++which) {
        uint32_t *h = (which ? fghist : hist) + seg * T * kBins;
        // (a thread walks its digit's column tile by tile: eight independent loads in flight)
        uint32_t total = 0;
        int64_t t = 0;
        for (; t + 8 <= Tk; t += 8) {
            uint32_t c[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) c[u] = h[(t + u) * kBins + b];
#pragma unroll
            for (int u = 0; u < 8; ++u) total += c[u];
        }
        for (; t < Tk; ++t) total += h[t * kBins + b];
        uint32_t run = block_excl_scan_1024(total, warp_tot, &grand);
        for (t = 0; t + 8 <= Tk; t += 8) {
            uint32_t c[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) c[u] = h[(t + u) * kBins + b];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                h[(t + u) * kBins + b] = run;
                run += c[u];
            }
        }
        for (; t < Tk; ++t) {
            const uint32_t c = h[t * kBins + b];
            h[t * kBins + b] = run;
            run += c;
        }
        if (which && b == 0) n_pos[seg] = grand;
        __syncthreads();
    }
}

// ------------------------------------------------------------------ pruning
//
// Elements past the pruning bound (see track_fg) are dropped before the sort: a count per
// sort tile, a scan per segment, and a stable compaction that also writes the dropped
// elements' dJ (zero).  The sort then runs on the kept elements only (Lp per segment).

// kept[seg][tile] = number of elements of the tile with (key >> 1) < limit;
// fgkept[seg][tile] = number of foreground elements of the tile.
__global__ void __launch_bounds__(kSortThreads)
prune_count_kernel(const uint32_t *__restrict__ keys, const uint32_t *__restrict__ maxfg,
                   const uint32_t *__restrict__ minkey, uint32_t *__restrict__ kept, uint32_t *__restrict__ fgkept,
                   int64_t L, int64_t T, int prune) {
    __shared__ uint32_t wsum[kSortWarps], wfg[kSortWarps];
    const int64_t seg = blockIdx.x / T, tile = blockIdx.x % T;
    const uint32_t limit = prune_limit(maxfg, minkey, seg, prune);
    const int64_t t0 = tile * kSortTile;
    const int n = int(L - t0 < kSortTile ? L - t0 : kSortTile);
    const uint32_t *src = keys + seg * L + t0;
    uint32_t c = 0, f = 0;
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = r * kSortThreads + threadIdx.x;
        if (idx < n) {
            const uint32_t k = __ldg(src + idx);
            c += (k >> 1) < limit ? 1u : 0u;
            f += key_is_fg(k) ? 1u : 0u;
        }
    }
    c = __reduce_add_sync(0xffffffffu, c);
    f = __reduce_add_sync(0xffffffffu, f);
    if ((threadIdx.x & 31) == 0) {
        wsum[threadIdx.x >> 5] = c;
        wfg[threadIdx.x >> 5] = f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t tot = 0, fg = 0;
        for (int w = 0; w < kSortWarps; ++w) {
            tot += wsum[w];
            fg += wfg[w];
        }
        kept[seg * T + tile] = tot;
        fgkept[seg * T + tile] = fg;
    }
}

// kept[seg][*] -> exclusive offsets, Lp[seg] = total.  One block of kBins threads per segment.
// A segment that keeps more than 3/4 of its elements is not worth compacting: it is flagged
// `direct`, Lp = L, and its first sort pass reads it from the full array (the ignored pixels'
// keys sort last and the Jaccard kernel passes over them).  A segment with enough foreground
// and enough sorted elements is flagged `fast` (see "Key bits").
__global__ void __launch_bounds__(kBins)
prune_scan_kernel(uint32_t *__restrict__ kept, const uint32_t *__restrict__ fgkept, uint32_t *__restrict__ Lp,
                  uint32_t *__restrict__ seg_flags, int64_t L, int64_t T, int allow_fast) {
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t grand;
    __shared__ uint32_t fgw[32];
    const int64_t seg = blockIdx.x;
    uint32_t carry = 0, fg = 0;
    for (int64_t base = 0; base < T; base += kBins) {
        const int64_t t = base + threadIdx.x;
        const uint32_t v = t < T ? kept[seg * T + t] : 0u;
        fg += t < T ? fgkept[seg * T + t] : 0u;
        const uint32_t ex = block_excl_scan_1024(v, warp_tot, &grand);
        if (t < T) kept[seg * T + t] = carry + ex;
        carry += grand;
    }
    fg = __reduce_add_sync(0xffffffffu, fg);
    if ((threadIdx.x & 31) == 0) fgw[threadIdx.x >> 5] = fg;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t n_fg = 0;
        for (int w = 0; w < kBins / 32; ++w) n_fg += fgw[w];
        const bool d = int64_t(carry) * 4 > L * 3;
        const uint32_t sorted = d ? uint32_t(L) : carry;
        const bool fast = allow_fast && n_fg >= kFastMinFg && sorted >= kFastMinKept;
        Lp[seg] = sorted;
        seg_flags[seg] = (d ? kSegFlagDirect : 0u) | (fast ? kSegFlagFast : 0u);
    }
}

// Kept (key, position) pairs of a tile, in order, to offsets[seg][tile]...; dJ = 0 everywhere
// (the Jaccard kernel overwrites the kept ones).
__global__ void __launch_bounds__(kSortThreads)
prune_compact_kernel(const uint32_t *__restrict__ keys, const uint32_t *__restrict__ maxfg,
                     const uint32_t *__restrict__ minkey, const uint32_t *__restrict__ offsets,
                     const uint32_t *__restrict__ direct, uint32_t *__restrict__ keys_out,
                     uint32_t *__restrict__ vals_out, float *__restrict__ jacc, int64_t L, int64_t T, int prune) {
    __shared__ uint32_t wtot[kSortWarps];
    const int64_t seg = blockIdx.x / T, tile = blockIdx.x % T;
    if (__ldg(direct + seg) & kSegFlagDirect) return;
    const uint32_t limit = prune_limit(maxfg, minkey, seg, prune);
    const int64_t t0 = tile * kSortTile;
    const int n = int(L - t0 < kSortTile ? L - t0 : kSortTile);
    const int64_t sbase = seg * L;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wbase = warp * (32 * kSortItems);
    const uint32_t lt = lanemask_lt();
    uint32_t key[kSortItems];
    uint32_t keepbits = 0;                       // bit r: my element of round r stays
    uint32_t wc = 0;
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        key[r] = idx < n ? __ldg(keys + sbase + t0 + idx) : kKeyIgnored;
        if (idx < n) jacc[sbase + t0 + idx] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        if (idx < n && (key[r] >> 1) < limit) keepbits |= 1u << r;
    }
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) wc += __popc(__ballot_sync(0xffffffffu, (keepbits >> r) & 1u));
    if (lane == 0) wtot[warp] = wc;
    __syncthreads();
    uint32_t base = __ldg(offsets + seg * T + tile);
    for (int w = 0; w < warp; ++w) base += wtot[w];
    if (wc == 0) return;
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const bool keep = (keepbits >> r) & 1u;
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) {
            const uint32_t pos = base + __popc(m & lt);
            keys_out[sbase + pos] = key[r];
            vals_out[sbase + pos] = uint32_t(t0 + wbase + r * 32 + lane);
        }
        base += __popc(m);
    }
}

// The sort tiles in use, listed segment by segment (entries: encode_tile).  The kept
// counts exist on the device only, so the sort kernels run a fixed grid whose blocks stride
// over this list.  One block per segment; it finds its first slot by adding up the tiles of
// the segments before it.
__global__ void __launch_bounds__(256)
tile_map_kernel(const uint32_t *__restrict__ Lp, const uint32_t *__restrict__ direct,
                uint2 *__restrict__ tilemap, uint32_t *__restrict__ n_tiles, int64_t S) {
    __shared__ uint32_t wsum[8];
    const int64_t seg = blockIdx.x;
    uint32_t before = 0;
    for (int64_t q = threadIdx.x; q < seg; q += 256) before += (__ldg(Lp + q) + kSortTile - 1) / kSortTile;
    before = __reduce_add_sync(0xffffffffu, before);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = before;
    __syncthreads();
    uint32_t first = 0;
    for (int w = 0; w < 8; ++w) first += wsum[w];
    const uint32_t Lk = __ldg(Lp + seg);
    const uint32_t mine = (Lk + kSortTile - 1) / kSortTile;
    const uint32_t flags = __ldg(direct + seg);
    for (uint32_t t = threadIdx.x; t < mine; t += 256) {
        const uint32_t left = Lk - t * kSortTile;
        tilemap[first + t] = encode_tile(uint32_t(seg), t, left < kSortTile ? left : uint32_t(kSortTile), flags);
    }
    if (seg == S - 1 && threadIdx.x == 0) *n_tiles = first + mine;
}

// Shared-memory layout of the two ranking kernels.
//   match  u32 [warps][kBins]   per-warp lane masks of the current round (zero between rounds)
//   wcnt   u16 [warps][kBins]   per-warp digit counters -> exclusive prefix over warps
//   (scatter) bufk u32 [tile], bufv u32 [tile] (aliases match), binstart/goff u32 [kBins]
//   (jaccard) wfg u16 [warps][kBins], off/fgoff u32 [kBins]
constexpr size_t kMatchBytes = size_t(kSortWarps) * kBins * 4;
constexpr size_t kCntBytes = size_t(kSortWarps) * kBins * 2;
constexpr size_t kTileWordsBytes = size_t(kSortTile) * 4;
static_assert(kMatchBytes <= kTileWordsBytes, "the value buffer reuses the match masks");
// The scatter kernel runs 512 threads x 16 elements on the same 8192-element tile: half the
// registers per thread, twice the warps per SM to hide the ranking's shared-memory latency.
constexpr int kScatThreads = 512;
constexpr int kScatItems = kSortTile / kScatThreads;
constexpr int kScatWarps = kScatThreads / 32;
constexpr size_t kScatCntBytes = size_t(kScatWarps) * kBins * 2;
constexpr size_t kScatterSmem = kTileWordsBytes /*bufv*/ + kTileWordsBytes /*bufk*/ + kScatCntBytes + 2 * kBins * 4;
constexpr size_t kJaccardSmem = kMatchBytes + 2 * kCntBytes + 2 * kBins * 4 + kTileWordsBytes;

// One ranking round of a warp, two ways.
//
// rank_round_exact: which lanes hold my digit (lane masks from kBits ballots, all independent of
// each other), my rank among them in lane order, and the warp counter update by the lowest such
// lane: ranks follow array order exactly.  ~45 issue slots per round.
//
// rank_round_fast ("fast" segments only): one shared-memory atomic on the warp's own packed
// counter (two 16-bit counters per word; a warp sees at most 1024 elements per tile, so a half
// never carries into its neighbour).  Rounds follow each other in program order and every warp
// owns its counters, so ranks respect (warp, round) order = array order; WITHIN a round, lanes
// that hold the same digit are ranked in the order the hardware serialises the atomic.  That
// order only separates elements that are 32 or fewer positions apart in the input.  In a fast
// segment's first pass their final order is decided by the second digit unless both digits agree
// (a tie of the 20-bit sort key); in its last pass the input is already sorted by the first
// digit and holds at least 32 elements per value of it, so neighbours with the same last digit
// differ by at most one step of the first.  Either way the two errors agree to 2^-13 relative:
// the resolution a fast segment is sorted to (see "Key bits").  ~6 issue slots per round.
__device__ __forceinline__ uint32_t rank_round_exact(uint32_t d, uint16_t *wcnt, int lane, uint32_t lt) {
    uint32_t peers = 0xffffffffu;
#pragma unroll
    for (int b = 0; b < kBits; ++b) {
        const bool bit = (d >> b) & 1u;
        const uint32_t bal = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? bal : ~bal;
    }
    const int leader = __ffs(peers) - 1;
    uint32_t old = 0;
    if (lane == leader) {
        old = wcnt[d];
        wcnt[d] = uint16_t(old + __popc(peers));
    }
    __syncwarp();
    old = __shfl_sync(0xffffffffu, old, leader);
    return old + __popc(peers & lt);
}
__device__ __forceinline__ uint32_t rank_round_fast(uint32_t d, uint16_t *wcnt) {
    uint32_t *w32 = reinterpret_cast<uint32_t *>(wcnt);
    const uint32_t sh = (d & 1u) << 4;
    const uint32_t old = atomicAdd(&w32[d >> 1], 1u << sh);
    return (old >> sh) & 0xffffu;
}

// Stable scatter of one tile (passes that are not the last).  kin / vin point at the tile,
// kout / vout at the segment, off at the tile's row of scanned offsets.  vin == nullptr: the
// values are the positions pos0 + index (a segment that was not compacted, first pass).
//
// The n elements are dealt to the warps in contiguous chunks of R rounds of 32
// (R = ceil(n / 512), at most kScatItems), so (warp, round, lane) order equals array order
// and a partly filled tile skips the rounds it does not need.
template <bool FULL, bool FAST>   // FULL: a tile of exactly kSortTile elements -- straight-line code, no round tests
__device__ __forceinline__ void scatter_tile(const uint32_t *__restrict__ kin, const uint32_t *__restrict__ vin,
                                             uint32_t *__restrict__ kout, uint32_t *__restrict__ vout,
                                             const uint32_t *__restrict__ off, int n, int shift, uint32_t pos0,
                                             uint32_t *next, unsigned *ticket, const uint2 *tilemap,
                                             const uint32_t *n_tiles) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t *bufv = reinterpret_cast<uint32_t *>(smem_raw);
    uint32_t *bufk = reinterpret_cast<uint32_t *>(smem_raw + kTileWordsBytes);
    uint16_t *wcnt_all = reinterpret_cast<uint16_t *>(smem_raw + 2 * kTileWordsBytes);
    uint32_t *binstart = reinterpret_cast<uint32_t *>(smem_raw + 2 * kTileWordsBytes + kScatCntBytes);
    uint32_t *goff = binstart + kBins;
    __shared__ uint32_t warp_tot[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t lt = lanemask_lt();

    for (int i = tid; i < int(kScatCntBytes / 4); i += kScatThreads) reinterpret_cast<uint32_t *>(wcnt_all)[i] = 0;
    uint32_t key[kScatItems];
    const int cnt = n;
    const int R = FULL ? kScatItems : (cnt + kScatThreads - 1) / kScatThreads;      // rounds in use
    const int wbase = warp * (32 * R);
#pragma unroll
    for (int r = 0; r < kScatItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        key[r] = 0xFFFFFFFFu;
        if (r < R && idx < cnt) key[r] = __ldg(kin + idx);
    }
    draw_next_tile(next, ticket);
    __syncthreads();
    uint32_t rank2[kScatItems / 2];     // two 16-bit ranks per register
    uint16_t *wcnt = wcnt_all + warp * kBins;
#pragma unroll
    for (int r = 0; r < kScatItems; r += 2) {
        if (r < R) {
            uint32_t r0 = 0, r1 = 0;
            if (FAST) {
                // (padding lanes of a partly filled round take no rank: the hardware might serialise
                // them ahead of real elements of the same digit)
                if (FULL || wbase + r * 32 + lane < cnt) r0 = rank_round_fast(digit_of(key[r], shift), wcnt);
                if (r + 1 < R && (FULL || wbase + (r + 1) * 32 + lane < cnt))
                    r1 = rank_round_fast(digit_of(key[r + 1], shift), wcnt);
            } else {
                // (padding lanes hold all-ones keys in the highest positions: ranked last)
                r0 = rank_round_exact(digit_of(key[r], shift), wcnt, lane, lt);
                if (r + 1 < R) r1 = rank_round_exact(digit_of(key[r + 1], shift), wcnt, lane, lt);
            }
            rank2[r / 2] = r0 | (r1 << 16);
        }
    }
    __syncthreads();
    prefetch_next_tile(next, tilemap, __ldg(n_tiles));
    // per digit: exclusive prefix over warps (in place), then over digits
    constexpr int BPT = kBins / kScatThreads;
    uint32_t cntb[BPT];
    uint32_t mine = 0;
#pragma unroll
    for (int q = 0; q < BPT; ++q) {
        const int b = BPT * tid + q;
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < kScatWarps; ++w) {
            const uint32_t c = wcnt_all[w * kBins + b];
            wcnt_all[w * kBins + b] = uint16_t(run);
            run += c;
        }
        cntb[q] = run;
        mine += run;
    }
    {
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const uint32_t w = lane < kScatWarps ? warp_tot[lane] : 0;
            uint32_t wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += v;
            }
            warp_tot[lane] = wi - w;
        }
        __syncthreads();
        uint32_t excl = warp_tot[warp] + incl - mine;
#pragma unroll
        for (int q = 0; q < BPT; ++q) {
            const int b = BPT * tid + q;
            binstart[b] = excl;
            goff[b] = __ldg(off + b) - excl;
            excl += cntb[q];
        }
    }
    __syncthreads();
    // local sorted position (kept in place of the rank); keys into the reorder buffer
#pragma unroll
    for (int r = 0; r < kScatItems; ++r) {
        if (r < R && (FULL || wbase + r * 32 + lane < cnt)) {      // padding lanes hold no element
            const uint32_t d = digit_of(key[r], shift);
            const uint32_t rk = (r & 1) ? (rank2[r / 2] >> 16) : (rank2[r / 2] & 0xffffu);
            const uint32_t lp = binstart[d] + wcnt[d] + rk;
            bufk[lp] = key[r];
            rank2[r / 2] = (r & 1) ? ((rank2[r / 2] & 0xffffu) | (lp << 16)) : ((rank2[r / 2] & 0xffff0000u) | lp);
        }
    }
    // values: all loads are issued before the first is used
    {
        uint32_t v[kScatItems];
#pragma unroll
        for (int r = 0; r < kScatItems; ++r) {
            const int idx = wbase + r * 32 + lane;
            v[r] = pos0 + uint32_t(idx);
            if (vin && r < R && idx < cnt) v[r] = __ldg(vin + idx);
        }
#pragma unroll
        for (int r = 0; r < kScatItems; ++r) {
            if (r < R && (FULL || wbase + r * 32 + lane < cnt)) {
                const uint32_t lp = (r & 1) ? (rank2[r / 2] >> 16) : (rank2[r / 2] & 0xffffu);
                bufv[lp] = v[r];
            }
        }
    }
    __syncthreads();
    // each digit's run goes out contiguously
#pragma unroll 4
    for (int i = tid; i < cnt; i += kScatThreads) {
        const uint32_t k = bufk[i];
        const uint32_t gp = goff[digit_of(k, shift)] + uint32_t(i);
        kout[gp] = k;
        vout[gp] = bufv[i];
    }
}

// The blocks take tiles from the list of sort tiles in use: the first by block index, the
// following ones from a shared counter, so an uneven tile costs nobody a wait.  (The list
// cursor lives in shared memory: the tile body needs all 64 registers of a thread.)
// Segments flagged in `direct` were not compacted: they use the two buffer pairs in swapped
// roles (segments occupy disjoint ranges of every buffer), and in the first pass their values
// are their positions.
__global__ void __launch_bounds__(kScatThreads, 2)
sort_scatter_kernel(const uint32_t *keys_in, const uint32_t *vals_in, uint32_t *keys_out, uint32_t *vals_out,
                    const uint32_t *__restrict__ offsets, const uint2 *__restrict__ tilemap,
                    const uint32_t *__restrict__ n_tiles, unsigned *__restrict__ ticket, int64_t L, int64_t T,
                    int shift, int first_pass) {
    __shared__ uint32_t cursor, cursor_next;
    if (threadIdx.x == 0) cursor = blockIdx.x;
    __syncthreads();
    while (true) {
        const uint32_t w = *const_cast<volatile uint32_t *>(&cursor);
        if (w >= __ldg(n_tiles)) break;
        const TileRef tr = decode_tile(__ldg(tilemap + w));
        if (first_pass && tr.fast) {                   // fast segments have no first pass
            __syncthreads();
            if (threadIdx.x == 0) cursor = gridDim.x + atomicAdd(ticket, 1u);
            __syncthreads();
            continue;
        }
        const int64_t seg = tr.seg, tile = tr.tile;
        const int64_t sbase = seg * L, t0 = tile * kSortTile;
        const int n = tr.n;
        const bool sw = tr.swapped;
        const uint32_t *ki = sw ? keys_out : keys_in;
        const uint32_t *vi = sw ? vals_out : vals_in;
        uint32_t *ko = sw ? const_cast<uint32_t *>(keys_in) : keys_out;
        uint32_t *vo = sw ? const_cast<uint32_t *>(vals_in) : vals_out;
        // the first pass a segment takes: a segment that was not compacted has no values yet
        const bool seg_first = first_pass || tr.fast;
        const uint32_t *vin = (tr.direct && seg_first) ? nullptr : vi + sbase + t0;
        const uint32_t *off = offsets + (seg * T + tile) * kBins;
        if (tr.fast) {
            if (n == kSortTile)
                scatter_tile<true, true>(ki + sbase + t0, vin, ko + sbase, vo + sbase, off, n, shift, uint32_t(t0),
                                         &cursor_next, ticket, tilemap, n_tiles);
            else
                scatter_tile<false, true>(ki + sbase + t0, vin, ko + sbase, vo + sbase, off, n, shift, uint32_t(t0),
                                          &cursor_next, ticket, tilemap, n_tiles);
        } else {
            scatter_tile<false, false>(ki + sbase + t0, vin, ko + sbase, vo + sbase, off, n, shift, uint32_t(t0),
                                       &cursor_next, ticket, tilemap, n_tiles);
        }
        __syncthreads();
        if (threadIdx.x == 0) cursor = cursor_next;
        __syncthreads();
    }
}

// Last pass, fused with the Jaccard step.  Nothing is moved: the final rank of an element is
//   i  = offsets[digit][tile] + (rank among the tile's elements with this digit)
//   cs = fgoffsets[digit][tile] + (rank among the tile's FOREGROUND elements with this digit)
// (elements with a smaller top digit come first, equal digits keep the order of the previous
// passes), which is all dJ needs.  Writes dJ to the pixel's slot and a loss partial per tile.
__global__ void __launch_bounds__(kSortThreads, 2)
rank_jaccard_kernel(const uint32_t *__restrict__ keys_main, const uint32_t *__restrict__ vals_main,
                    const uint32_t *__restrict__ keys_alt, const uint32_t *__restrict__ vals_alt,
                    const uint32_t *__restrict__ offsets, const uint32_t *__restrict__ fgoffsets,
                    const uint32_t *__restrict__ n_pos_seg, float *__restrict__ jacc,
                    double *__restrict__ partial, const uint2 *__restrict__ tilemap, const uint32_t *__restrict__ n_tiles,
                    unsigned *__restrict__ ticket, int64_t L, int64_t T, int shift) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t *match = reinterpret_cast<uint32_t *>(smem_raw);                     // [kSortTile] pixel indices of the tile
    uint32_t *wpk_all = reinterpret_cast<uint32_t *>(smem_raw + kMatchBytes);     // [warps][kBins]
    uint32_t *off = reinterpret_cast<uint32_t *>(smem_raw + kMatchBytes + 2 * kCntBytes);
    uint32_t *fgoff = off + kBins;
    uint32_t *keybuf = fgoff + kBins;                  // [kSortTile] keys of the tile
    __shared__ double sh_d[32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wbase = warp * (32 * kSortItems);
    __shared__ uint32_t cursor, cursor_next;  // position in the tile list (kept out of the registers)
    if (tid == 0) cursor = blockIdx.x;
    __syncthreads();
  while (true) {
    const uint32_t w = *const_cast<volatile uint32_t *>(&cursor);
    if (w >= __ldg(n_tiles)) break;
    const TileRef tr = decode_tile(__ldg(tilemap + w));
    const int64_t seg = tr.seg, tile = tr.tile;
    const int64_t sbase = seg * L;
    const int64_t t0 = tile * kSortTile;
    const int n = tr.n;

    const bool swapped = tr.swapped;
    const uint32_t *keys = (swapped ? keys_alt : keys_main) + sbase + t0;
    const uint32_t *vals = (swapped ? vals_alt : vals_main) + sbase + t0;
    for (int i = tid; i < int(2 * kCntBytes / 4); i += kSortThreads) wpk_all[i] = 0;
    {
        const int64_t o = (seg * T + tile) * kBins;
        for (int b = tid; b < kBins; b += kSortThreads) {
            off[b] = __ldg(offsets + o + b);
            fgoff[b] = __ldg(fgoffsets + o + b);
        }
    }
    // keys and pixel indices wait in shared memory (same slot, same thread: no barrier needed
    // for them): all their global loads are in flight together and the registers stay free for
    // the ranks.  (Reading the pixel indices from global memory where they are used instead would
    // fit a third block on the SM, but measured 9 % slower: 3.81 against 3.49 ms unpruned.)
#pragma unroll
    for (int r0 = 0; r0 < kSortItems; r0 += 16) {
        uint32_t kk[16], v[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int idx = wbase + (r0 + r) * 32 + lane;
            kk[r] = idx < n ? __ldg(keys + idx) : 0xFFFFFFFFu;
            v[r] = idx < n ? __ldg(vals + idx) : 0u;
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            keybuf[wbase + (r0 + r) * 32 + lane] = kk[r];
            match[wbase + (r0 + r) * 32 + lane] = v[r];
        }
    }
    draw_next_tile(&cursor_next, ticket);
    __syncthreads();
    uint32_t rkfg[kSortItems];          // rank | fg rank << 16
    // per (warp, digit) one packed counter: elements seen | foreground elements seen << 16.  ONE
    // atomic returns both, so an element's rank and the number of foreground elements before it
    // come from the same serialisation of the warp's lanes (see rank_round).
    uint32_t *wpk = wpk_all + warp * kBins;
    // fast segments: one atomic per element (see rank_round_fast); all others: exact array order
    // from kBits ballots per round, the leader lane updates the counter (rank_round_exact)
    const bool exact_order = !tr.fast;
    if (!exact_order) {
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            const uint32_t kr = keybuf[wbase + r * 32 + lane];
            const uint32_t d = digit_of(kr, shift);
            rkfg[r] = 0;
            if (wbase + r * 32 + lane < n) rkfg[r] = atomicAdd(&wpk[d], key_is_fg(kr) ? 0x10001u : 1u);
        }
    } else {
        const uint32_t lt = lanemask_lt();
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            const uint32_t kr = keybuf[wbase + r * 32 + lane];
            const uint32_t d = digit_of(kr, shift);     // (padding lanes: last digit, highest positions)
            const uint32_t fgball = __ballot_sync(0xffffffffu, key_is_fg(kr));
            uint32_t peers = 0xffffffffu;
#pragma unroll
            for (int b = 0; b < kBits; ++b) {
                const bool bit = (d >> b) & 1u;
                const uint32_t bal = __ballot_sync(0xffffffffu, bit);
                peers &= bit ? bal : ~bal;
            }
            const int leader = __ffs(peers) - 1;
            uint32_t old = 0;
            if (lane == leader) {
                old = wpk[d];
                wpk[d] = old + __popc(peers) + (__popc(peers & fgball) << 16);
            }
            __syncwarp();
            old = __shfl_sync(0xffffffffu, old, leader);
            rkfg[r] = old + __popc(peers & lt) + (__popc(peers & fgball & lt) << 16);
        }
    }
    __syncthreads();
    constexpr int BPT = kBins / kSortThreads;
#pragma unroll
    for (int q = 0; q < BPT; ++q) {
        const int b = BPT * tid + q;
        uint32_t run = 0;                // both halves at once: a tile holds at most 8192 < 65536 elements
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = wpk_all[w * kBins + b];
            wpk_all[w * kBins + b] = run;
            run += c;
        }
    }
    prefetch_next_tile(&cursor_next, tilemap, __ldg(n_tiles));
    __syncthreads();
    const uint32_t n_pos = __ldg(n_pos_seg + seg);
    float acc = 0.f;
    float *dst = jacc + sbase;
#pragma unroll
    for (int r = 0; r < kSortItems; ++r) {
        const int idx = wbase + r * 32 + lane;
        if (idx < n) {
            const uint32_t k = keybuf[idx];
            const uint32_t d = digit_of(k, shift);
            const bool ign = k == kKeyIgnored;
            const bool fg = key_is_fg(k);
            const uint32_t before = wpk[d] + rkfg[r];            // packed: this tile's earlier elements of digit d
            const uint32_t i_glob = off[d] + (before & 0xffffu);
            const uint32_t cs_before = fgoff[d] + (before >> 16);
            const uint32_t union_before = n_pos + (i_glob - cs_before);
            const float I = float(n_pos - cs_before);
            const float U = float(union_before);
            float dj;
            if (fg) dj = __fdividef(1.f, U);
            else dj = union_before == 0u ? 1.f : __fdividef(I, U * (U + 1.f));
            const float err = ign ? 0.f : __uint_as_float(kOneBits - (k >> 1));
            acc += err * dj;
            dst[match[idx]] = dj;
        }
    }
    double a = double(acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) sh_d[warp] = a;
    __syncthreads();
    if (tid == 0) {
        double s = 0.0;
        for (int q = 0; q < kSortWarps; ++q) s += sh_d[q];
        partial[seg * T + tile] = s;
        cursor = cursor_next;
    }
    __syncthreads();
  }
}

// loss[seg] = sum of the segment's tile partials, fixed order.
__global__ void __launch_bounds__(32)
loss_kernel(const double *__restrict__ partial, float *__restrict__ loss, const uint32_t *__restrict__ Lp,
            int64_t T) {
    const int64_t seg = blockIdx.x;
    const int64_t Tk = (int64_t(__ldg(Lp + seg)) + kSortTile - 1) / kSortTile;
    double s = 0.0;
    for (int64_t t = threadIdx.x; t < Tk; t += 32) s += partial[seg * T + t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) loss[seg] = float(s);
}

// ------------------------------------------------------------------- host side

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_args(const char *who, int64_t N, int64_t C, int64_t M, int dtype) {
    if (N < 0 || C < 1 || M < 0) {
        set_error("%s: bad shape N=%lld C=%lld M=%lld", who, (long long)N, (long long)C, (long long)M);
        return B200_ERR_ARG;
    }
    if (dtype != B200_F32) {
        set_error("%s: float32 logits only (cast half inputs first, as autocast does)", who);
        return B200_ERR_UNSUPPORTED;
    }
    if (C > 1024) {
        set_error("%s: C=%lld exceeds the supported 1024 classes", who, (long long)C);
        return B200_ERR_UNSUPPORTED;
    }
    if (N * M >= (int64_t(1) << 31) || N * C * M >= (int64_t(1) << 40)) {
        set_error("%s: tensor too large (N*M must stay below 2^31)", who);
        return B200_ERR_UNSUPPORTED;
    }
    return B200_OK;
}

// Tensor maps of the two layouts a tile kernel touches.
bool make_maps(const LovaszGeom &g, const void *logits_like, const void *seg_like, CUtensorMap *map_img,
               CUtensorMap *map_seg, int seg_dtype) {
    const uint64_t dims[3] = {uint64_t(g.M), uint64_t(g.C), uint64_t(g.N)};
    const uint32_t box[3] = {uint32_t(g.TP), uint32_t(g.CB), 1u};
    const uint64_t st_img[3] = {4, uint64_t(g.M) * 4, uint64_t(g.C) * g.M * 4};
    const uint64_t st_glob[3] = {4, uint64_t(g.N) * g.M * 4, uint64_t(g.M) * 4};
    if (logits_like && !encode_tensor_map(map_img, B200_F32, logits_like, 3, dims, st_img, box)) return false;
    if (seg_like &&
        !encode_tensor_map(map_seg, seg_dtype, seg_like, 3, dims, g.per_image ? st_img : st_glob, box))
        return false;
    return true;
}

inline int env_int(const char *name, int dflt) {
    const char *v = std::getenv(name);
    return (v && *v) ? std::atoi(v) : dflt;
}

template <bool BWD>
int launch_tile(const TileArgs &a, cudaStream_t stream) {
    const LovaszGeom &g = a.g;
    const size_t tile_al = (size_t(g.rows) * g.TP * 4 + 127) & ~size_t(127);
    const size_t smem = 128 + (BWD ? 2 : 1) * tile_al + 2 * kTileThreads * sizeof(float);
    int per_sm = int((220 * 1024) / (smem + 1024));
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) {
        set_error("lovasz: C=%lld needs %zu bytes of shared memory per tile", (long long)g.C, smem);
        return B200_ERR_UNSUPPORTED;
    }
    int64_t grid = int64_t(sm_count()) * per_sm;
    if (grid > g.total_tiles) grid = g.total_tiles;
    const void *seg_ptr = BWD ? static_cast<const void *>(a.jacc) : static_cast<const void *>(a.keys);
    const bool tma_ok = (g.M * 4) % 16 == 0 && aligned16(a.logits) && aligned16(seg_ptr) &&
                        (!BWD || aligned16(a.grads));
    CUtensorMap m_logits{}, m_seg{}, m_grads{};
    if (tma_ok) {
        if (!make_maps(g, a.logits, seg_ptr, &m_logits, &m_seg, BWD ? B200_F32 : 99)) return B200_ERR_LAUNCH;
        if (BWD && !make_maps(g, a.grads, nullptr, &m_grads, nullptr, 0)) return B200_ERR_LAUNCH;
    }
    // few classes, aligned: the pipelined pair-per-thread kernel
    const PairLayout lay = pair_layout(int(g.C), BWD);
    if (tma_ok && g.TP == kPairTP && g.nbox == 1 && g.M >= kPairTile && g.M % 4 == 0 && aligned16(a.labels) &&
        lay.stage_bytes <= 110u * 1024 && true) {
        // measured at C = 19: keys 1 stage x 4 blocks per SM; backward (two tiles per stage)
        // 2 stages in one block per SM beat 1 stage x 2 blocks (334 vs 371 us on 8 x 1 Mpixel)
        int stages = (BWD ? 2 : 1);
        if (stages < 1) stages = 1;
        if (stages > kMaxStages) stages = kMaxStages;
        while (stages > 1 && size_t(stages) * lay.stage_bytes > 200u * 1024) --stages;
        const size_t psmem = 128 + size_t(stages) * lay.stage_bytes;
        int ctas = int((224u * 1024) / (psmem + 1280));
        const int cap = (BWD ? 3 : 4);
        if (ctas > cap) ctas = cap;
        if (ctas < 1) ctas = 1;
        const int64_t ptiles = g.N * ((g.M + kPairTile - 1) / kPairTile);
        int64_t pgrid = int64_t(sm_count()) * ctas;
        if (pgrid > ptiles) pgrid = ptiles;
        auto kern = lovasz_pair_kernel<BWD>;
        if (psmem > 40 * 1024 &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(psmem)) != cudaSuccess)
            return launch_status("cudaFuncSetAttribute(lovasz pair)");
        kern<<<dim3(unsigned(pgrid)), kTileBlock, psmem, stream>>>(a, stages, m_logits, m_seg, m_grads);
        return launch_status(BWD ? "lovasz backward kernel launch" : "lovasz keys kernel launch");
    }
    auto launch = [&](auto kern) -> int {
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
            return launch_status("cudaFuncSetAttribute(lovasz tile)");
        kern<<<dim3(unsigned(grid)), kTileThreads, smem, stream>>>(a, m_logits, m_seg, m_grads);
        return launch_status(BWD ? "lovasz backward kernel launch" : "lovasz keys kernel launch");
    };
    if (!tma_ok && g.C <= 40) {
        // unaligned, few classes: a pixel's channels in one thread's registers
        const int64_t groups = g.N * ((g.M + kAnyThreads - 1) / kAnyThreads);
        int64_t agrid = int64_t(sm_count()) * (BWD ? 2 : 3) * 4;
        if (agrid > groups) agrid = groups;
        if (g.C <= 20) lovasz_any_kernel<BWD, 20><<<dim3(unsigned(agrid)), kAnyThreads, 0, stream>>>(a);
        else lovasz_any_kernel<BWD, 40><<<dim3(unsigned(agrid)), kAnyThreads, 0, stream>>>(a);
        return launch_status(BWD ? "lovasz backward kernel launch" : "lovasz keys kernel launch");
    }
    return tma_ok ? launch(lovasz_tile_kernel<BWD, true>) : launch(lovasz_tile_kernel<BWD, false>);
}



}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200_lovasz_workspace_bytes(int64_t N, int64_t C, int64_t M, int per_image) {
    if (N <= 0 || C <= 0 || M <= 0) return 256;
    if (N * M >= (int64_t(1) << 31) || C > 1024) return 0;      // a size b200_lovasz_forward refuses
    LovaszGeom g{};
    make_geom(g, N, C, M, per_image);
    return carve(nullptr, g).bytes;
}

extern "C" int b200_lovasz_forward(const void *logits, const int64_t *labels, float *loss,
                                   float *jacc, void *workspace, size_t workspace_bytes, int64_t N,
                                   int64_t C, int64_t M, int dtype, int64_t ignore_index,
                                   int per_image, void *stream) {
    int rc = check_args("b200_lovasz_forward", N, C, M, dtype);
    if (rc != B200_OK) return rc;
    if (N * M == 0) return B200_OK;
    if (!logits || !labels || !loss || !jacc || !workspace) {
        set_error("b200_lovasz_forward: null pointer");
        return B200_ERR_ARG;
    }
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) {
        set_error("b200_lovasz_forward: workspace must be 256-byte aligned");
        return B200_ERR_ARG;
    }
    LovaszGeom g{};
    make_geom(g, N, C, M, per_image);
    Workspace w = carve(workspace, g);
    if (workspace_bytes < w.bytes) {
        set_error("b200_lovasz_forward: workspace of %zu bytes required, got %zu", w.bytes, workspace_bytes);
        return B200_ERR_WORKSPACE;
    }
    if (g.S * g.T >= (int64_t(1) << 31)) {
        set_error("b200_lovasz_forward: too many sort tiles");
        return B200_ERR_UNSUPPORTED;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // status word and the foreground trackers start at 0, the smallest-key samples at all ones
    if (cudaMemsetAsync(w.status, 0, reinterpret_cast<char *>(w.minkey) - reinterpret_cast<char *>(w.status), s) !=
            cudaSuccess ||
        cudaMemsetAsync(w.minkey, 0xFF, size_t(g.S) * 4, s) != cudaSuccess)
        return launch_status("lovasz workspace memset");

    TileArgs ta{};
    ta.logits = static_cast<const float *>(logits);
    ta.labels = labels;
    ta.keys = w.keysA;
    ta.maxfg = w.maxfg;
    ta.minkey = w.minkey;
    ta.status = w.status;
    ta.ignore = ignore_index;
    ta.g = g;
    if ((rc = launch_tile<false>(ta, s)) != B200_OK) return rc;

    if (cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(kScatterSmem)) != cudaSuccess ||
        cudaFuncSetAttribute(rank_jaccard_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(kJaccardSmem)) != cudaSuccess)
        return launch_status("cudaFuncSetAttribute(lovasz sort kernels)");
    // drop the elements past the pruning bound
    const unsigned nblk_all = unsigned(g.S * g.T);
    const int prune = env_int("B200_LOVASZ_NO_PRUNE", 0) ? 0 : 1;
    const int allow_fast = env_int("B200_LOVASZ_EXACT", 0) ? 0 : 1;     // 0: every segment sorts on all 30 bits
    prune_count_kernel<<<nblk_all, kSortThreads, 0, s>>>(w.keysA, w.maxfg, w.minkey, w.kept, w.fgkept, g.L, g.T,
                                                         prune);
    if ((rc = launch_status("lovasz prune count launch")) != B200_OK) return rc;
    prune_scan_kernel<<<unsigned(g.S), kBins, 0, s>>>(w.kept, w.fgkept, w.Lp, w.direct, g.L, g.T, allow_fast);
    if ((rc = launch_status("lovasz prune scan launch")) != B200_OK) return rc;
    prune_compact_kernel<<<nblk_all, kSortThreads, 0, s>>>(w.keysA, w.maxfg, w.minkey, w.kept, w.direct, w.keysB,
                                                           w.valsB, jacc, g.L, g.T, prune);
    if ((rc = launch_status("lovasz prune compact launch")) != B200_OK) return rc;

    // The number of sorted elements is known on the device only: fixed grids (a multiple of the
    // SM count, by each kernel's blocks per SM) take tiles from the list of sort tiles in use.
    tile_map_kernel<<<unsigned(g.S), 256, 0, s>>>(w.Lp, w.direct, w.tilemap, w.n_tiles, g.S);
    if ((rc = launch_status("lovasz tile map launch")) != B200_OK) return rc;
    auto grid_of = [&](int per_sm) {
        // (measured on 8 x 19 x 1 Mpixel: a resident grid that loops costs 5.6 ms unpruned and 1.10 ms
        // pruned, one block per possible tile 5.0 and 1.13 ms: many more blocks than fit, capped)
        const int64_t want = int64_t(sm_count()) * per_sm * 32;
        return unsigned(want < g.S * g.T ? want : g.S * g.T);
    };
    const unsigned nblk_hist = grid_of(8), nblk = grid_of(2);
    unsigned *tickets = w.status + 16;           // zeroed with the status word; one per kernel

    // Buffer roles as a compacted segment that takes all three passes sees them: B -> A -> B,
    // ranked from B (other segments: see TileRef).  Fast segments sit out the first pass.
    uint32_t *kin = w.keysB, *vin = w.valsB, *kout = w.keysA, *vout = w.valsA;
    for (int pass = 0; pass < kPasses - 1; ++pass) {
        const int shift = 1 + pass * kBits;
        const int first_pass = pass == 0 ? 1 : 0;
        sort_hist_kernel<false><<<nblk_hist, kSortThreads, 0, s>>>(kin, w.hist, nullptr, w.tilemap, w.n_tiles, kout,
                                                                  g.L, g.T, shift, first_pass);
        if ((rc = launch_status("lovasz sort histogram launch")) != B200_OK) return rc;
        sort_scan_kernel<false><<<unsigned(g.S), kBins, 0, s>>>(w.hist, nullptr, nullptr, w.Lp, w.direct, g.T,
                                                                first_pass);
        if ((rc = launch_status("lovasz sort scan launch")) != B200_OK) return rc;
        sort_scatter_kernel<<<nblk, kScatThreads, kScatterSmem, s>>>(kin, vin, kout, vout, w.hist, w.tilemap,
                                                                     w.n_tiles, tickets + pass, g.L, g.T, shift,
                                                                     first_pass);
        if ((rc = launch_status("lovasz sort scatter launch")) != B200_OK) return rc;
        std::swap(kin, kout);
        std::swap(vin, vout);
    }
    {
        const int shift = 1 + (kPasses - 1) * kBits;
        sort_hist_kernel<true><<<nblk_hist, kSortThreads, 0, s>>>(kin, w.hist, w.fghist, w.tilemap, w.n_tiles, kout,
                                                                 g.L, g.T, shift, 0);
        if ((rc = launch_status("lovasz last histogram launch")) != B200_OK) return rc;
        sort_scan_kernel<true><<<unsigned(g.S), kBins, 0, s>>>(w.hist, w.fghist, w.n_pos, w.Lp, w.direct, g.T, 0);
        if ((rc = launch_status("lovasz last scan launch")) != B200_OK) return rc;
        rank_jaccard_kernel<<<nblk, kSortThreads, kJaccardSmem, s>>>(kin, vin, kout, vout, w.hist, w.fghist,
                                                                      w.n_pos, jacc,
                                                                      w.partial, w.tilemap, w.n_tiles,
                                                                      tickets + 3, g.L, g.T, shift);
        if ((rc = launch_status("lovasz rank+jaccard launch")) != B200_OK) return rc;
    }
    loss_kernel<<<unsigned(g.S), 32, 0, s>>>(w.partial, loss, w.Lp, g.T);
    return launch_status("lovasz loss launch");
}

extern "C" int b200_lovasz_backward(const float *grad, const void *logits, const int64_t *labels,
                                    const float *jacc, void *grad_logits, int64_t N, int64_t C,
                                    int64_t M, int dtype, int64_t ignore_index, int per_image,
                                    void *stream) {
    int rc = check_args("b200_lovasz_backward", N, C, M, dtype);
    if (rc != B200_OK) return rc;
    if (N * M == 0) return B200_OK;
    if (!grad || !logits || !labels || !jacc || !grad_logits) {
        set_error("b200_lovasz_backward: null pointer");
        return B200_ERR_ARG;
    }
    LovaszGeom g{};
    make_geom(g, N, C, M, per_image);
    TileArgs ta{};
    ta.logits = static_cast<const float *>(logits);
    ta.labels = labels;
    ta.jacc = jacc;
    ta.seg_grad = grad;
    ta.grads = static_cast<float *>(grad_logits);
    ta.status = nullptr;
    ta.ignore = ignore_index;
    ta.g = g;
    return launch_tile<true>(ta, static_cast<cudaStream_t>(stream));
}
