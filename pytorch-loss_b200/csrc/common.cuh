// Shared device/host helpers of libb200loss: error reporting, dtype access,
// warp/block reductions, the deterministic grid reduction that ends every
// reducing forward kernel, and thin wrappers over the sm_100a bulk-async (TMA)
// and mbarrier PTX used to stage tiles in shared memory.
#pragma once
#include <utility>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/b200loss.h"

namespace b200 {

// ----------------------------------------------------------------- host side

void set_error(const char *fmt, ...);
int launch_status(const char *what);   // cudaGetLastError -> B200_OK / B200_ERR_LAUNCH; counts the launch
int sm_count();                         // SMs of the current device (cached per device)

// float64 paths (fp64.cu), called by the per-pixel entry points when dtype == B200_F64
int f64_softmax_forward(int kind, const void *logits, const int64_t *labels, void *losses, void *out, void *workspace,
                        int64_t N, int64_t C, int64_t M, int64_t ignore_index, float hp, void *stream);
int f64_softmax_backward(int kind, const void *logits, const int64_t *labels, const void *grad_out, int grad_mode,
                         const void *denom, void *grad_logits, int64_t N, int64_t C, int64_t M,
                         int64_t ignore_index, float hp, void *stream);
int f64_focal(const void *logits, const void *labels, void *losses, void *grads, const void *grad_out, int grad_mode,
              const void *denom, void *out, void *workspace, int64_t E, float gamma, float alpha, void *stream);

// Workspace layout shared by all reducing kernels.
//   [0]   uint32  ticket   (must be zero between kernels; kernels reset it)
//   [4]   uint32  status   (non-zero: a bounded wait gave up)
//   [8]   ExchangeCtx*     (optional, see below; null: the record holds this GPU's sums)
//   [64]  double2 partials[kMaxPartials]
constexpr int kMaxPartials = 65536;
constexpr size_t kPartialsOffset = 64;
constexpr size_t kReduceWorkspaceBytes = kPartialsOffset + size_t(kMaxPartials) * 16;

// Cross-GPU sum of [sum, count] inside the reducing kernels (one process per GPU, batch
// sharded over the ranks).  Every rank owns an array of message slots that its peers can write
// (peer-mapped device memory).  A message is five 8-byte words, each {32 data bits, 32-bit
// flag}: the two doubles in four words and a tag word.  The flag is derived from the call's
// sequence number, so a word validates itself: the sender needs no fence between data and
// flag and the receiver polls ITS OWN memory until all five words carry the flag.  Plain peer
// stores and local polls only: no peer loads, no multicast, no atomics across GPUs.
//   post    lane p of one warp stores this rank's message into slot [seq & 3][rank] of rank p
//   collect lane p polls slot [seq & 3][p] of this rank's own array -- bounded -- and lane 0
//           adds the pairs in rank order, so every rank gets the same bits
// The sequence number is a device-side counter (graph replays keep working).  Four slot sets
// (two would do): a rank cannot post message k+2 before every peer has collected message k,
// because it collects k+1 first and that needs the peers' posts, which follow their own
// collection of k.
// The tag names what the message carries (a count, a loss sum).  Ranks whose call sequences
// differ (one took a path with one exchange, another a path with two) meet a foreign tag or
// never see the flag: both give NaN sums, status bit 0x200 / 0x100, and never a silently
// wrong number.
struct ExchangeSlot {       // 64 bytes
    unsigned long long w[8];    // w[0..3]: sum lo/hi, count lo/hi; w[4]: tag; each | flag << 32
};
constexpr int kExchangeSets = 4;
constexpr unsigned kTagSum = 0x53554d21u;      // 'SUM!'
constexpr unsigned kTagCount = 0x434e5421u;    // 'CNT!'
constexpr int kMaxExchangeRanks = 16;
struct ExchangeCtx {        // lives in device memory; filled by the host once (layout is ABI)
    int world;
    int rank;
    unsigned poll_limit;    // polls of one slot before a wait gives up (status bit 0x100)
    unsigned reserved;
    unsigned long long *seq;                    // [0] this rank's call counter; [1] sequence number of a
                                                // loss sum that is posted but not yet collected (0: none)
    ExchangeSlot *slots[kMaxExchangeRanks];     // slots[p]: rank p's array [kExchangeSets][world]
};
constexpr size_t kExchangeCtxOffset = 8;

struct ReduceRecord {       // the 32-byte "out" record of the C ABI
    double sum;
    double count;
    float mean;
    float sum32;
    float pad[2];
};

// --------------------------------------------------------------- dtype access

template <typename T> struct Vec16;   // 16-byte vector of T; alignas makes a copy ONE 128-bit access
template <> struct alignas(16) Vec16<float> {
    static constexpr int N = 4;
    float v[4];
};
template <> struct alignas(16) Vec16<__half> {
    static constexpr int N = 8;
    __half v[8];
};

template <> struct alignas(16) Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __nv_bfloat16 v[8];
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
// bytes of one element of a dtype code (B200_F32 / B200_F16 / B200_BF16)
inline size_t dtype_size(int dtype) { return dtype == B200_F32 ? 4 : 2; }
inline bool dtype_known(int dtype) { return dtype == B200_F32 || dtype == B200_F16 || dtype == B200_BF16; }

// Streaming 16-byte global access (read-once data: keep it out of L1).
template <typename V> __device__ __forceinline__ V ld_stream16(const void *p) {
    static_assert(sizeof(V) == 16, "16-byte vector expected");
    int4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return *reinterpret_cast<V *>(&r);
}
template <typename V> __device__ __forceinline__ void st_stream16(void *p, const V &v) {
    static_assert(sizeof(V) == 16, "16-byte vector expected");
    const int4 r = *reinterpret_cast<const int4 *>(&v);
    asm volatile("st.global.cs.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z),
                 "r"(r.w)
                 : "memory");
}

// ------------------------------------------------------------ math (fp32 core)

// e^x for x <= 0 in softmax sums: ex2.approx on x*log2(e).  Relative error of a
// term is below 2^-21 for the arguments that contribute to a sum (|x| < 16).
__device__ __forceinline__ float exp_fast(float x) { return __expf(x); }

// --------------------------------------------------------------- reductions

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum of (loss, count) pairs in double; result valid in thread 0.
// `sh` must hold 64 doubles.  All threads of the block must call it.
__device__ __forceinline__ void block_sum2(double &a, double &b, double *sh) {
    a = warp_sum(a);
    b = warp_sum(b);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) {
        sh[warp] = a;
        sh[32 + warp] = b;
    }
    __syncthreads();
    if (warp == 0) {
        a = lane < nwarp ? sh[lane] : 0.0;
        b = lane < nwarp ? sh[32 + lane] : 0.0;
        a = warp_sum(a);
        b = warp_sum(b);
    }
}

// ---- programmatic dependent launch (a kernel that starts under the tail of the one in front)
// The dependent may only touch what the kernel in front produces after pdl_wait(): it returns
// when that grid has completed and its writes are visible (at once in a plain launch).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The kernel in front: its dependents may be scheduled from now on (once every block has said so
// or exited); a no-op when nothing depends on it this way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// kernel<<<grid, block, smem, stream>>>(args...), optionally as a programmatic dependent of the
// operation in front of it on the stream.
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool dependent, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- cross-GPU messages (see ExchangeSlot).  All three functions are called by ONE full warp.

__device__ __forceinline__ unsigned exchange_flag(unsigned long long seq) {
    return unsigned(seq % 0xffffffffull) + 1u;          // never 0: fresh slots are zero
}
__device__ __forceinline__ unsigned long long ll_word(unsigned data, unsigned flag) {
    return (static_cast<unsigned long long>(flag) << 32) | data;
}
// Takes the next sequence number (lane 0 increments the device counter) and stores this rank's
// message {a, b, tag} into every rank's array.  Returns the sequence number in all lanes.
__device__ __forceinline__ unsigned long long exchange_post(ExchangeCtx *ex, unsigned tag, double a, double b) {
    const int lane = threadIdx.x & 31;
    unsigned long long seq = 0;
    if (lane == 0) seq = ++ex->seq[0];
    seq = __shfl_sync(0xffffffffu, seq, 0);
    const int world = ex->world;
    if (lane < world) {
        volatile unsigned long long *dst =
            ex->slots[lane][(seq & (kExchangeSets - 1)) * world + ex->rank].w;
        const unsigned flag = exchange_flag(seq);
        const unsigned long long ua = __double_as_longlong(a), ub = __double_as_longlong(b);
        dst[0] = ll_word(unsigned(ua), flag);
        dst[1] = ll_word(unsigned(ua >> 32), flag);
        dst[2] = ll_word(unsigned(ub), flag);
        dst[3] = ll_word(unsigned(ub >> 32), flag);
        dst[4] = ll_word(tag, flag);
    }
    return seq;
}
// Waits (bounded) for message `seq` of every rank in this rank's own array and adds the pairs in
// rank order.  Returns 0 in all lanes on success (sums valid in lane 0), else the status bits:
// 0x100 a rank's message did not arrive within poll_limit polls, 0x200 it carried another tag.
__device__ __forceinline__ unsigned exchange_collect(ExchangeCtx *ex, unsigned long long seq, unsigned tag,
                                                     double &a, double &b) {
    const int lane = threadIdx.x & 31;
    const int world = ex->world;
    const unsigned flag = exchange_flag(seq);
    unsigned bad = 0;
    double ma = 0.0, mb = 0.0;
    if (lane < world) {
        const volatile unsigned long long *src =
            ex->slots[ex->rank][(seq & (kExchangeSets - 1)) * world + lane].w;
        unsigned long long w[5];
        unsigned polls = 0;
        for (;;) {
            bool all = true;
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                w[k] = src[k];
                all = all && unsigned(w[k] >> 32) == flag;
            }
            if (all) break;
            if (++polls > ex->poll_limit) {
                bad = 0x100u;
                break;
            }
            __nanosleep(32);
        }
        if (!bad && unsigned(w[4]) != tag) bad = 0x200u;
        ma = __longlong_as_double((w[1] << 32) | (w[0] & 0xffffffffull));
        mb = __longlong_as_double((w[3] << 32) | (w[2] & 0xffffffffull));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    a = 0.0;
    b = 0.0;
    for (int p = 0; p < world; ++p) {       // rank order: the same bits on every rank
        a += __shfl_sync(0xffffffffu, ma, p);
        b += __shfl_sync(0xffffffffu, mb, p);
    }
    return bad;
}

__device__ __forceinline__ ExchangeCtx *exchange_of(void *workspace) {
    return workspace ? *reinterpret_cast<ExchangeCtx **>(reinterpret_cast<char *>(workspace) + kExchangeCtxOffset)
                     : nullptr;
}

// Collects a loss sum that grid_reduce_finish<defer> posted earlier and completes its record.
// One full warp calls it.  Nothing pending: returns at once (so it may be called twice).
// Returns true in lane 0 when it has just written the record.
__device__ __forceinline__ bool exchange_finish_pending(void *workspace, ReduceRecord *out) {
    ExchangeCtx *ex = exchange_of(workspace);
    if (!ex) return false;
    const unsigned long long seq = ex->seq[1];
    if (seq == 0ull) return false;
    double a, b;
    const unsigned bad = exchange_collect(ex, seq, kTagSum, a, b);
    if ((threadIdx.x & 31) != 0) return false;
    if (bad) {
        atomicOr(reinterpret_cast<unsigned *>(workspace) + 1, bad);
        a = b = __longlong_as_double(0x7ff8000000000000ll);
    }
    out->sum = a;
    out->count = b;
    out->mean = static_cast<float>(a / b);
    out->sum32 = static_cast<float>(a);
    ex->seq[1] = 0ull;
    return true;
}

// Final step of a reducing forward kernel.  Every block calls it once with its
// partial (sum, count).  The block that takes the last ticket adds all partials
// in a fixed order, writes the record and re-arms the ticket: deterministic,
// no spinning, no second launch.  blockDim.x must be a multiple of 32, <= 1024.
// With an exchange attached to the workspace the pair is first added over the ranks (message
// tag `tag`).  `defer` (and an exchange): this rank's pair is only POSTED; the record keeps
// NaN in its float fields until a later kernel of the stream collects the ranks' pairs
// (exchange_finish_pending) -- the wait for the slowest rank and for the link then overlaps
// whatever runs in between instead of holding this kernel.
// Returns true in exactly one thread of the grid: the one that has just written the record.
__device__ __forceinline__ bool grid_reduce_finish(double sum, double cnt, void *workspace,
                                                   ReduceRecord *out, double *sh,
                                                   unsigned tag = kTagSum, bool defer = false) {
    block_sum2(sum, cnt, sh);
    unsigned *ticket = reinterpret_cast<unsigned *>(workspace);
    double2 *partials =
        reinterpret_cast<double2 *>(reinterpret_cast<char *>(workspace) + kPartialsOffset);
    __shared__ unsigned s_last;
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = make_double2(sum, cnt);
        __threadfence();
        const unsigned t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return false;
    __threadfence();
    double a = 0.0, b = 0.0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) {
        const double2 p = __ldcg(&partials[i]);
        a += p.x;
        b += p.y;
    }
    block_sum2(a, b, sh);
    if (threadIdx.x >= 32) return false;
    ExchangeCtx *ex = exchange_of(workspace);
    bool pending = false;
    if (ex) {
        a = __shfl_sync(0xffffffffu, a, 0);
        b = __shfl_sync(0xffffffffu, b, 0);
        const unsigned long long seq = exchange_post(ex, tag, a, b);
        if (defer) {
            if (threadIdx.x == 0) ex->seq[1] = seq;
            pending = true;
        } else {
            const unsigned bad = exchange_collect(ex, seq, tag, a, b);
            if (bad) {
                if (threadIdx.x == 0) atomicOr(reinterpret_cast<unsigned *>(workspace) + 1, bad);
                a = b = __longlong_as_double(0x7ff8000000000000ll);
            }
        }
    }
    if (threadIdx.x == 0) {
        const float nan32 = __int_as_float(0x7fc00000);
        out->sum = a;                   // (pending: this rank's sums for now)
        out->count = b;
        out->mean = pending ? nan32 : static_cast<float>(a / b);
        out->sum32 = pending ? nan32 : static_cast<float>(a);
        out->pad[0] = 0.f;
        out->pad[1] = 0.f;
        *ticket = 0u;
        return !pending;
    }
    return false;
}

// ------------------------------------------------- mbarrier + bulk-async (TMA)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
constexpr uint32_t kMbarSuspendNs = 2000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    // the suspend-time hint lets the thread sleep inside the instruction for up to that many
    // nanoseconds instead of returning to spin, which would take issue slots from working warps
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kMbarSuspendNs)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kMbarSpinLimit polls (each poll blocks for at most the
// suspend-time hint: about a second in total), records it in the status word and reports false.
constexpr uint32_t kMbarSpinLimit = 1u << 19;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  unsigned *status_word) {
    for (uint32_t i = 0; i < kMbarSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (status_word) atomicOr(status_word, 1u);
    // second, shorter bounded wait so copies still in flight land before the CTA exits
    for (uint32_t i = 0; i < (kMbarSpinLimit >> 4); ++i) {
        if (mbar_try_wait(bar, parity)) break;
    }
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Named barrier 1 over the first `n` threads of a block (the compute warps of a
// warp-specialised kernel; the copy warps never join it).  n must be a multiple of 32.
__device__ __forceinline__ void compute_sync(int n) {
    asm volatile("bar.sync 1, %0;" ::"r"(n) : "memory");
}
// Same barrier with an AND reduction of a per-thread predicate (uniform result).
__device__ __forceinline__ bool compute_all(bool ok, int n) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(uint32_t(ok)), "r"(n)
        : "memory");
    return r != 0;
}

// 2-D / 3-D tiled loads global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
// Tiled stores shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
                 "r"(x), "r"(y), "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int x, int y, int z,
                                             const void *src) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map),
        "r"(x), "r"(y), "r"(z), "r"(smem_u32(src))
        : "memory");
}
// Untiled bulk copies (16-byte aligned addresses, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes,
                                             uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void *dst, const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                 "r"(smem_u32(src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Host: encode a tiled tensor map over a row-major array.  `dims`/`strides_bytes`
// are innermost-first; strides_bytes[0] is implied (element size).  Returns false
// (with the error string set) if the driver entry point is missing or refuses.
bool encode_tensor_map(CUtensorMap *map, int dtype, const void *base, int rank,
                       const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box);

}  // namespace b200
