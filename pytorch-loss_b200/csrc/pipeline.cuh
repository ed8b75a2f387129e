// Shared pieces of the warp-specialised copy pipelines (softmax_losses.cu, lovasz.cu): the
// mbarrier ring, and packed fp32x2 arithmetic on pixel / element pairs.
#pragma once

#include "common.cuh"

namespace b200 {

// ------------------------------------------------- warp-specialised copy pipelines
//
// The aligned (TMA) forms of the tile and rows regimes.  A block is kCompute compute threads
// plus two copy warps.  One thread of the first copy warp keeps up to `stages` loads in flight
// into a ring of shared-memory stages; the compute warps consume a stage and, in backward,
// leave the gradients in it; one thread of the second copy warp stores finished stages and
// hands them back to the loader.  Three mbarriers per stage carry the hand-offs:
//     full[s]   loader -> compute   (transaction bytes of the stage's copies)
//     ready[s]  compute -> storer   (one arrival per compute warp; backward only)
//     empty[s]  storer -> loader (backward) or compute -> loader (forward, one per warp)
// so the copy of tile k+1.. overlaps the math of tile k and the store of tile k-1 inside one
// block, whatever the other blocks on the SM are doing.  Every wait is bounded; a wait that runs
// out sets the status word and the block leaves its loop.

constexpr int kMaxStages = 4;

struct PipeBarriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t ready[kMaxStages];
};

template <int NCOMPUTE, bool BWD>
__device__ __forceinline__ void pipe_init(PipeBarriers &bars, int stages) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&bars.full[s], 1);
            mbar_init(&bars.empty[s], BWD ? 1 : NCOMPUTE / 32);
            mbar_init(&bars.ready[s], NCOMPUTE / 32);
        }
        fence_mbar_init();
    }
    __syncthreads();
}

constexpr int kTileCompute = 256;
constexpr int kTileBlock = kTileCompute + 64;

// ---------------------------------------------------------- pair-per-thread tile kernel
//
// The production form of the tile regime.  The softmax kernels are bound by instruction
// issue, not by bytes (B200 offers ~22 issue slots per fp32 element read at HBM speed), so the
// inner loops are written for instruction count:
//   * a thread owns TWO adjacent pixels of one channel slice: one 8-byte shared-memory access
//     per channel, and all arithmetic on the pair goes through Blackwell's packed fp32x2
//     instructions (add/mul/fma.f32x2: one issue slot for two elements);
//   * no per-element label compare: element (channel, pixel) is always visited by the same
//     thread, so the thread that owns the label channel of a pixel edits that one element in
//     place instead (LSR: adds the target term after the sweep; large margin: parks the target
//     logit at -FLT_MAX for the max sweep and at min(x_lb, m') for the sum sweep, then takes its
//     terms back out of the sums -- s' >= 1 >= e^{min(x_lb - m', 0)}, so nothing cancels);
//   * exponentials are ex2.approx on a fused x*log2(e) - m*log2(e).
// Copy pipeline and hand-offs as described above (loader, storer, full/ready/empty).

__device__ __forceinline__ unsigned long long pk2(float2 v) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(v.x), "f"(v.y));
    return r;
}
__device__ __forceinline__ float2 upk2(unsigned long long r) {
    float2 v;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(v.x), "=f"(v.y) : "l"(r));
    return v;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(pk2(a)), "l"(pk2(b)));
    return upk2(r);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(pk2(a)), "l"(pk2(b)));
    return upk2(r);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(pk2(a)), "l"(pk2(b)), "l"(pk2(c)));
    return upk2(r);
}
__device__ __forceinline__ float ex2f(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float2 ex2_2(float2 t) { return make_float2(ex2f(t.x), ex2f(t.y)); }
__device__ __forceinline__ float2 max2(float2 a, float2 b) { return make_float2(fmaxf(a.x, b.x), fmaxf(a.y, b.y)); }
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

// Two adjacent pixels of one channel in a shared-memory tile.
__device__ __forceinline__ float2 ld_pair(const float *p) { return *reinterpret_cast<const float2 *>(p); }
__device__ __forceinline__ float2 ld_pair(const __half *p) {
    return __half22float2(*reinterpret_cast<const __half2 *>(p));
}
__device__ __forceinline__ void st_pair(float *p, float2 v) { *reinterpret_cast<float2 *>(p) = v; }
__device__ __forceinline__ void st_pair(__half *p, float2 v) {
    *reinterpret_cast<__half2 *>(p) = __float22half2_rn(v);
}
__device__ __forceinline__ float2 ld_pair(const __nv_bfloat16 *p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
}
__device__ __forceinline__ void st_pair(__nv_bfloat16 *p, float2 v) {
    *reinterpret_cast<__nv_bfloat162 *>(p) = __float22bfloat162_rn(v);
}

// The same operations on values that STAY packed in one 64-bit register pair across a loop
// (loads and stores move the pair as one 8-byte word; only the two ex2 need the halves).
typedef unsigned long long pk_t;
__device__ __forceinline__ pk_t padd(pk_t a, pk_t b) {
    pk_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ pk_t pmul(pk_t a, pk_t b) {
    pk_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ pk_t pfma(pk_t a, pk_t b, pk_t c) {
    pk_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ pk_t pex2(pk_t t) {
    pk_t r;
    asm("{\n\t.reg .f32 a, b;\n\t"
        "mov.b64 {a, b}, %1;\n\t"
        "ex2.approx.ftz.f32 a, a;\n\t"
        "ex2.approx.ftz.f32 b, b;\n\t"
        "mov.b64 %0, {a, b};\n\t}"
        : "=l"(r)
        : "l"(t));
    return r;
}
__device__ __forceinline__ pk_t psplat(float v) { return pk2(make_float2(v, v)); }
__device__ __forceinline__ pk_t ld_pk(const float *p) { return *reinterpret_cast<const pk_t *>(p); }
__device__ __forceinline__ pk_t ld_pk(const __half *p) { return pk2(ld_pair(p)); }
__device__ __forceinline__ pk_t ld_pk(const __nv_bfloat16 *p) { return pk2(ld_pair(p)); }
__device__ __forceinline__ void st_pk(float *p, pk_t v) { *reinterpret_cast<pk_t *>(p) = v; }
__device__ __forceinline__ void st_pk(__half *p, pk_t v) { st_pair(p, upk2(v)); }
__device__ __forceinline__ void st_pk(__nv_bfloat16 *p, pk_t v) { st_pair(p, upk2(v)); }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace b200
