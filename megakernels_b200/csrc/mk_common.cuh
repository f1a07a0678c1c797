// Shared definitions of the decode megakernel: geometry, kernel parameters and
// the PTX wrappers (mbarrier, bulk-copy TMA, release/acquire global counters).
//
// Design (replaces include/megakernel.cuh, include/controller/*, include/util.cuh
// and include/config.cuh of the reference):
//   * one persistent CTA per SM, each walking its own instruction queue;
//   * 16 consumer warps + 1 loader warp + 1 storer warp, every role decodes the
//     instruction words itself, so there is no controller warp and no page
//     allocator: the weight ring is one continuous sequence of 32 KiB stages
//     that runs across instruction boundaries, which lets the loader stream the
//     next instruction's weights while the consumers still wait on a barrier;
//   * counters in HBM (`barriers[layer][opcode-1][slot]`) order instructions of
//     different SMs: producers `red.release.gpu`, waiters `ld.acquire.gpu`;
//   * every wait is bounded and reports into a status record instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mkb200.h"

// The kernel source is compiled three times.
//   MKB_BATCH == 1 (default): one sequence per launch, the latency-optimised build.
//   MKB_BATCH == 8: up to 8 independent sequences per launch; the activation vectors of all
//     sequences are the 8 columns of the mma.sync B operand, so the weights are still streamed
//     once; it trades two ring stages for room to park 8 activation vectors.
//   MKB_BATCH == 64: 9..64 sequences per launch; the projections become small-M GEMMs on the
//     5th-generation tensor cores: blocks of 128 weight rows are the M side of tcgen05.mma, the
//     sequences its N side, the accumulator lives in tensor memory, and the activations are
//     streamed per 128-column slice next to the weights instead of being parked.
#ifndef MKB_BATCH
#define MKB_BATCH 1
#endif
#if MKB_BATCH == 1
#define MKB_NAMESPACE mkb
#elif MKB_BATCH <= 8
#define MKB_NAMESPACE mkb_batched
#else
#define MKB_NAMESPACE mkb_gemm
#endif

namespace MKB_NAMESPACE {

// ---- geometry ------------------------------------------------------------ //
constexpr int kBatch = MKB_BATCH;
constexpr bool kGemm = kBatch > 8;
constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;  // 512
constexpr int kLoaderWarp = kConsumerWarps;            // warp 16
constexpr int kStorerWarp = kConsumerWarps + 1;        // warp 17
// Loader warps (one issuing thread each): warp 16 and, if more than one, the warps after the storer.
#ifndef MKB_LOADERS
#define MKB_LOADERS 1
#endif
constexpr int kLoaders = MKB_LOADERS;
constexpr int kBlockThreads = (kConsumerWarps + 1 + kLoaders) * 32;  // 576 with one loader

constexpr int kStageBytes = 32768;  // one ring stage
constexpr int kNumStages = kBatch == 1 ? 6 : 4;  // 192 (128) KiB of weights / KV in flight per SM
constexpr int kOutSlots = kGemm ? 1 : kBatch == 1 ? 4 : 2;  // ring of per-block partial sums, consumer -> storer
constexpr int kOutSlotFloats = kGemm ? 16 : 16 * 16 * kBatch;  // [row][sequence][partial] (unused by the GEMM build)
constexpr int kBlockRows = kGemm ? 128 : 16;     // output rows per block
constexpr int kStageCols = kGemm ? 128 : 1024;   // input columns per ring stage: a stage is kBlockRows x kStageCols bf16
static_assert(kBlockRows * kStageCols * 2 == kStageBytes, "");
// Parked activation vectors: one per sequence, kActStride bytes apart.  The stride is 64 mod
// 128 so that the 8 lanes of a quarter warp (two sequences x four chunks) hit 8 different
// 16-byte bank groups when they load their B-operand fragments.
constexpr int kActBytes = kBatch == 1 ? 16384 : 8192;  // longest vector: H (or R) bf16 elements
constexpr int kActStride = kBatch == 1 ? 0 : kActBytes + 64;
// GEMM build: a second ring carries the activation slices, [sequence][kStageCols] bf16 per stage
constexpr int kXStages = kGemm ? 4 : 0;
constexpr int kXStageBytes = kBatch * kStageCols * 2;
constexpr int kTmemCols = 2 * (kBatch < 32 ? 32 : kBatch);  // two accumulators of kBatch fp32 columns

// attention: cross-warp merge scratch, 8 slots x 4 heads x (D + m + l)
constexpr int kAttnHeadsPerPass = 4;
constexpr int kAttnSlotFloats = kAttnHeadsPerPass * (128 + 4);
constexpr int kAttnScratchFloats = 8 * kAttnSlotFloats;
constexpr int kActAreaBytes = (kBatch == 1 || kGemm) ? kAttnScratchFloats * 4 : kBatch * kActStride;
static_assert(kActAreaBytes >= kAttnScratchFloats * 4 && (kGemm || kActAreaBytes >= kActBytes), "");

// shared-memory map (byte offsets from the 1024-aligned base)
constexpr int kSmemRing = 0;
constexpr int kSmemXRing = kSmemRing + kNumStages * kStageBytes;  // GEMM build only (1024-byte aligned tiles)
constexpr int kSmemOut = kSmemXRing + kXStages * kXStageBytes;
constexpr int kSmemAttn = kSmemOut + kOutSlots * kOutSlotFloats * 4;  // activations / attention scratch
constexpr int kSmemRed = kSmemAttn + kActAreaBytes;            // 32 floats
constexpr int kSmemRope = kSmemRed + 32 * 4;                   // cos[D], sin[D] at every sequence's position
constexpr int kSmemBars = kSmemRope + (kGemm ? 0 : kBatch * 2 * 128 * 4);  // mbarriers, 8 B each
// ring full/empty, out-slot full/empty, then (GEMM build) X-ring full/empty and accumulator full/empty x 2
constexpr int kNumMbars = 2 * kNumStages + 2 * kOutSlots + 2 * kXStages + (kGemm ? 4 : 0);
constexpr int kSmemCtl = kSmemBars + kNumMbars * 8;            // control words, then the positions
constexpr int kCtlWords = 8 + (kBatch < 8 ? 8 : kBatch);
// A few launch constants that out-of-line code on the critical path reads from shared memory
// (HotConsts, 16-byte aligned) instead of chasing pointers through local and parameter memory.
constexpr int kSmemHot = (kSmemCtl + kCtlWords * 4 + 15) & ~15;
constexpr int kSmemTotal = kSmemHot + 64;
static_assert(kSmemTotal + 1024 <= 227 * 1024, "shared memory budget of one CTA");
constexpr int kSmemAlloc = kSmemTotal + 1024;  // slack to align the base

enum Role { kRoleLoader = 0, kRoleConsumer = 1, kRoleStorer = 2 };

// status record layout (int32 words), mirrors MkbStatus; word 15 is the abort flag
constexpr int kStatusAbortWord = 15;

// ---- kernel parameters ---------------------------------------------------- //
struct KParams {
    // vm
    int* barriers;
    const int* instructions;
    int* timings;
    int* status;
    int queue_len, barrier_ops, barrier_width;
    // weights
    const __nv_bfloat16 *qkv_w, *attn_ln_w, *o_w, *mlp_ln_w, *up_w, *gate_w, *down_w, *lm_norm_w,
        *lm_head_w;
    __nv_bfloat16 *k_cache, *v_cache;
    const float *rope_cos, *rope_sin;
    __nv_bfloat16 *hidden, *q_rope, *attn_out, *silu_out, *logits;
    float *attn_lse, *attn_o;
    // Residual stream of the token = hidden (the embedding, never written) + residual_acc:
    // o-proj / down-proj add their outputs as 64-bit fixed point (Q31.32) with integer atomics,
    // so the sum does not depend on the order in which the SMs arrive (bit-reproducible).
    long long* residual_acc;  // [H], zeroed by the caller before every launch
    long long residual_mult;  // integer factor on every contribution (1; the TP degree under the NCCL exchange)
    // dims
    int L, H, I, D, Hq, Hkv, V, T, B, max_partials, R;
    int qkv_rows;  // (Hq + 2 Hkv) * D
    int o_in;      // Hq * D
    // per token
    int pos_id;
    const int* pos_id_ptr;   // when set, the position(s) are read from device memory instead
    // batched build: sequences decoded by this launch, their positions when pos_id_ptr is not
    // set, and the RMS-normalised activations [batch][H] that RMS_NORM instructions publish
    int batch;
    int pos_ids[8];
    __nv_bfloat16* normed;
    // GEMM build: activations as 3-D [64, batch, K/64] views with the 128-byte swizzle; a box is
    // one X-ring stage {64, kBatch rows (rows beyond `batch` read as zero), kStageCols/64}
    CUtensorMap x_normed_map, x_attn_map, x_silu_map;
    int gemm_n;  // N of the MMAs: batch rounded up to a multiple of 16
    float attn_scale_log2e;  // attn_scale * log2(e)
    float rms_eps;
    int skip_attn_reduction;
    // fused argmax over the logits: result word, and library-owned scratch
    // [0] = CTAs finished, then {value bits, index} per CTA
    int* argmax_out;
    int* argmax_scratch;
    // in-kernel tensor-parallel all-reduce (MkbTensorParallel); tp_size <= 1: off
    int tp_size, tp_rank, tp_chunks;
    const int* tp_epoch_ptr;
    uint2* tp_hidden_ll[MKB_MAX_TP];  // [H/2] x {bf16x2, tag} of every rank
    float* tp_recv[MKB_MAX_TP];       // [size][H/2] x {f32, tag, f32, tag} of every rank
    float* tp_partial;
    // barrier thresholds, derived on the host from the shapes
    int thr_qkv_waits_down;     // (H/16) * (I/R)
    int thr_attn_waits_qkv;     // D/16
    int thr_oproj_waits_attn;   // Hq
    int thr_upgate_waits_oproj; // (H/16) * (o_in/R)
    int thr_down_waits_upgate;  // R/16
    int thr_down_waits_rms;     // up/gate instructions of a layer (0: the schedule does not say)
    unsigned long long timeout_ns;
    int poll_sleep_ns;     // back-off between polls of a barrier counter
    int l2_window_stages;  // how many ring stages the loader may prefetch into L2 ahead of the ring
    int l2_stall_window_stages;  // the same while this SM's consumers wait on a barrier counter
    // TMA descriptors of the KV cache, 4-D [D, Hkv, T, L*B], box {D, 1, TS, 1}
    CUtensorMap k_map, v_map;
    // weight matrices as 4-D [64, rows, K/64, L] with the 128-byte swizzle; one box is a ring
    // stage: 16 rows x up to 1024 columns, stored [64-column chunk][row][128 B]
    CUtensorMap qkv_map, o_map, up_map, gate_map, down_map, lm_map;
};

// ---- PTX wrappers ---------------------------------------------------------- //
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// contiguous global -> shared bulk copy (TMA engine), completes on an mbarrier
__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
// 4-D tiled tensor copy global -> shared
__device__ __forceinline__ void tma_tile4_g2s(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                              int c2, int c3, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
        : "memory");
}
// 5-D tiled tensor copy global -> shared (K/V tiles)
__device__ __forceinline__ void tma_tile5_g2s(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                              int c3, int c4, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void prefetch_l1(const void* p) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// ordered variants (volatile, memory clobber) for data another GPU wrote or will read
__device__ __forceinline__ uint2 ldv_cg_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ldv_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16-byte accesses whose two 8-byte halves {value, tag} each arrive whole: the receiver
// needs no separate flag (and the sender no fence) to know that a value is valid
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c2, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c2), "r"(d)
                 : "memory");
}
// AND of a predicate over the 512 consumer threads (one barrier)
__device__ __forceinline__ bool consumer_all(bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.and.pred q, 1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)pred), "n"(kConsumerThreads)
        : "memory");
    return out != 0;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_cg_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void red_add_u64(void* p, unsigned long long v) {
    asm volatile("red.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// fixed-point format of the residual accumulators: value * 2^32 in a signed 64-bit integer
constexpr float kResidualScale = 4294967296.f;
constexpr float kResidualInvScale = 1.f / 4294967296.f;
// A Q31.32 accumulator (low word, high word) as fp32: integer part and fraction are converted
// separately (two 32-bit conversions and an FMA instead of a 64-bit conversion, which costs a
// dozen instructions on the critical path of every RMSNorm).  The result is within one fp32 ulp of
// the exactly rounded value and, like it, a function of the accumulator's bits alone.
__device__ __forceinline__ float q32_to_float(uint32_t lo, uint32_t hi) {
    return fmaf(__uint2float_rn(lo), kResidualInvScale, __int2float_rn((int)hi));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace MKB_NAMESPACE
