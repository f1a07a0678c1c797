// The persistent decode megakernel: one CTA per SM interprets its instruction
// queue.  Replaces the reference's `mk` kernel template and its seven op
// structs (include/megakernel.cuh:166-171; demos/low-latency-llama/*.cu) with
// shape-generic, hand-written sm_100a code:
//
//   loader warp   - walks the queue ahead of everybody else and streams every
//                   weight block and KV tile (one tiled cp.async.bulk.tensor per
//                   stage) into a ring of 32 KiB stages; it never looks at a
//                   barrier, because weights and old KV positions depend on nothing.
//   16 consumer   - wait for the instruction's global barrier, park the (RMS-
//   warps           normalised) activation vector in shared memory, then multiply
//                   ring stages against it with mma.sync (weights are the A operand,
//                   the activation vector column 0 of B); each warp owns a column
//                   slice of the stage.
//   storer warp   - sums the per-warp partials of a 16-row block, applies the
//                   op's epilogue (RoPE + KV append, SiLU*up, residual add,
//                   logits) and signals the next op's barrier counter.
#include "mk_common.cuh"

namespace MKB_NAMESPACE {

// --------------------------------------------------------------------------- //
// control / error reporting
// --------------------------------------------------------------------------- //
struct Ctx {
    const KParams* p;
    uint32_t base;            // shared-window address of the aligned smem base
    volatile int* cta_abort;  // generic pointer to the CTA-wide abort word
    int pos;                  // position of the token being decoded (sequence 0)
    int instr;                // instruction index being executed (for reports)
    int opcode;
    int role;

    // position of sequence b's token (batched build: kept behind the control words)
    __device__ __forceinline__ int pos_of(int b) const {
        if constexpr (kBatch == 1) return pos;
        else return cta_abort[8 + b];  // control words 0..7, then one position per sequence
    }

    __device__ __forceinline__ uint32_t full_bar(int slot) const { return base + kSmemBars + slot * 8; }
    __device__ __forceinline__ uint32_t empty_bar(int slot) const {
        return base + kSmemBars + (kNumStages + slot) * 8;
    }
    __device__ __forceinline__ uint32_t out_full_bar(int slot) const {
        return base + kSmemBars + (2 * kNumStages + slot) * 8;
    }
    __device__ __forceinline__ uint32_t out_empty_bar(int slot) const {
        return base + kSmemBars + (2 * kNumStages + kOutSlots + slot) * 8;
    }
    __device__ __forceinline__ uint32_t stage_addr(int slot) const {
        return base + kSmemRing + slot * kStageBytes;
    }
    // GEMM build: activation ring and the two tensor-memory accumulators
    __device__ __forceinline__ uint32_t xfull_bar(int slot) const {
        return base + kSmemBars + (2 * kNumStages + 2 * kOutSlots + slot) * 8;
    }
    __device__ __forceinline__ uint32_t xempty_bar(int slot) const {
        return base + kSmemBars + (2 * kNumStages + 2 * kOutSlots + kXStages + slot) * 8;
    }
    __device__ __forceinline__ uint32_t acc_full_bar(int buf) const {
        return base + kSmemBars + (2 * kNumStages + 2 * kOutSlots + 2 * kXStages + buf) * 8;
    }
    __device__ __forceinline__ uint32_t acc_empty_bar(int buf) const {
        return base + kSmemBars + (2 * kNumStages + 2 * kOutSlots + 2 * kXStages + 2 + buf) * 8;
    }
    __device__ __forceinline__ uint32_t xstage_addr(int slot) const {
        return base + kSmemXRing + slot * kXStageBytes;
    }
    __device__ __forceinline__ uint32_t tmem_base() const { return (uint32_t)cta_abort[6]; }
};

// one thread per role stamps event times (ns) into the instruction's timing row
__device__ __forceinline__ void rec(const Ctx& c, int slot) {
    int* t = c.p->timings;
    if (t != nullptr && c.instr >= 0)
        t[((size_t)blockIdx.x * c.p->queue_len + c.instr) * MKB_TIMING_SLOTS + slot] =
            (int)(uint32_t)globaltimer_ns();
}

__device__ __noinline__ void report_error(const Ctx& c, int code, int d0, int d1, int d2, int d3) {
    int* st = c.p->status;
    if (atomicCAS(&st[0], 0, code) == 0) {
        st[1] = blockIdx.x;
        st[2] = c.instr;
        st[3] = c.opcode;
        st[4] = c.role;
        st[5] = d0;
        st[6] = d1;
        st[7] = d2;
        st[8] = d3;
        __threadfence();
    }
    atomicExch(&st[kStatusAbortWord], 1);
    *c.cta_abort = 1;
}

__device__ __forceinline__ bool global_abort(const Ctx& c) {
    return *reinterpret_cast<volatile int*>(&c.p->status[kStatusAbortWord]) != 0;
}

// Bounded mbarrier wait.  Returns false when the CTA is aborting or the budget ran out.
__device__ __noinline__ bool mbar_wait_slow(const Ctx& c, uint32_t bar, uint32_t parity,
                                            bool honour_abort) {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 127u) == 0) {
            if (honour_abort && *c.cta_abort) return false;
            unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > 2 * c.p->timeout_ns) {
                // twice the counter budget: when a global counter is stuck, the report
                // should come from the wait on that counter, not from its bystanders
                report_error(c, MKB_ERR_DEVICE_TIMEOUT, -1, (int)bar, (int)parity, 0);
                return false;
            }
            if (honour_abort && (spins & 2047u) == 0 && global_abort(c)) {
                *c.cta_abort = 1;
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(const Ctx& c, uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(c, bar, parity, true);
}

// Warp-collective bounded wait: lane 0 runs the bounded loop, then EVERY lane
// observes the completed phase itself.  The second step is not optional: data
// written by TMA (or by other warps before their arrive) is only guaranteed
// visible to a thread that performed the acquiring try_wait itself; lanes that
// merely learn of the completion through a shuffle were seen reading stale
// shared memory.  Returns false (uniformly) if the wait was abandoned.
__device__ __forceinline__ bool warp_mbar_wait(const Ctx& c, uint32_t bar, uint32_t parity,
                                               bool skip, int lane) {
    int ok = 1;
    if (!skip && lane == 0) ok = mbar_wait(c, bar, parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (skip || !ok) return false;
    for (int k = 0; k < 4096 && !mbar_try_wait(bar, parity); ++k) {
    }
    return true;
}

// Bounded wait for `*addr >= threshold` with acquire semantics.
// (`sleep_ns` travels in a register: the loop must not reach through `c`, which lives in local
// memory, on every poll - that is an L1 miss of 600 cycles between two polls.)
__device__ __noinline__ bool wait_counter(const Ctx& c, const int* addr, int threshold, int layer,
                                          int row, int slot, unsigned sleep_ns) {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (true) {
        int v = ld_acquire_gpu(addr);
        if (v >= threshold) return true;
        if ((++spins & 63u) == 0) {
            if (*c.cta_abort) return false;
            if (global_abort(c)) {
                *c.cta_abort = 1;
                return false;
            }
            unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > c.p->timeout_ns) {
                report_error(c, MKB_ERR_DEVICE_TIMEOUT, layer, row, slot, v);
                return false;
            }
        }
        __nanosleep(sleep_ns);
    }
}

// Warp-collective bounded wait on up to 32 counters at once: lane i polls addr (nullptr =
// nothing to wait for).  Sequential waits would cost one L2 round trip per counter.
__device__ __noinline__ bool warp_wait_counters(const Ctx& c, const int* addr, int threshold,
                                                int layer, int row, int slot, unsigned sleep_ns) {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (true) {
        const int v = addr ? ld_acquire_gpu(addr) : threshold;
        if (__all_sync(0xffffffffu, v >= threshold)) return true;
        if ((++spins & 63u) == 0) {
            int stop = 0;
            if ((threadIdx.x & 31) == 0) {
                if (*c.cta_abort) stop = 1;
                else if (global_abort(c)) {
                    *c.cta_abort = 1;
                    stop = 1;
                } else {
                    const unsigned long long now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > c.p->timeout_ns) stop = 2;
                }
            }
            stop = __shfl_sync(0xffffffffu, stop, 0);
            if (stop == 2) {  // the first lane still waiting names the stuck counter
                const unsigned late = __ballot_sync(0xffffffffu, v < threshold);
                if ((int)(threadIdx.x & 31) == __ffs(late) - 1)
                    report_error(c, MKB_ERR_DEVICE_TIMEOUT, layer, row, slot, v);
            }
            if (stop) return false;
        }
        __nanosleep(sleep_ns);
    }
}

__device__ __forceinline__ int* bar_addr(const KParams& p, int layer, int row, int slot) {
    return p.barriers + ((size_t)layer * p.barrier_ops + row) * p.barrier_width + slot;
}

// ---- tensor-parallel exchange: tagged values ------------------------------- //
// Values that cross GPUs travel as 8-byte {value, tag} words (two per 16-byte store).  The
// tag names the all-reduce (launch, layer, which) the value belongs to, so a reader that
// sees the expected tag knows the value beside it is current: no fence on the sender, no
// flag or counter on the receiver, and nothing is ever reset.
__device__ __forceinline__ uint32_t tp_tag(const Ctx& c, int layer, int which) {
    // the launch counter is read where it is needed (only tensor-parallel paths get here) so
    // that it does not occupy a register in everybody else's code
    const uint32_t epoch = (uint32_t)__ldg(c.p->tp_epoch_ptr);
    return (epoch * (uint32_t)c.p->L * 2u + (uint32_t)(layer * 2 + which)) % 0x7fffffffu + 1u;
}
// Bookkeeping of a bounded poll loop; tick() returns false when the thread must give up.
struct TpPoll {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    __device__ __forceinline__ bool tick(const Ctx& c, int layer, int what, int index, int observed) {
        if ((++spins & 63u) != 0) return true;
        if (*c.cta_abort) return false;
        if (global_abort(c)) {
            *c.cta_abort = 1;
            return false;
        }
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > c.p->timeout_ns) {
            report_error(c, MKB_ERR_DEVICE_TIMEOUT, layer, what, index, observed);
            return false;
        }
        return true;
    }
};

// --------------------------------------------------------------------------- //
// matvec geometry
// --------------------------------------------------------------------------- //
// A 16-row x KC block of a weight matrix is streamed as KC/1024 ring stages of
// 16 rows x 1024 columns (one stage of 16 x KC when KC < 1024; the GEMM build streams
// 128-row blocks as KC/128 stages of 128 x 128).  A stage is one
// tiled TMA copy with the 128-byte swizzle, laid out [64-column chunk][row][128 B];
// consumer warp w multiplies column chunk w with four m16n8k16 tensor-core MMAs.
__host__ __device__ inline int stages_per_block(int kc) { return kc > kStageCols ? kc / kStageCols : 1; }
__host__ __device__ inline int stage_cols(int kc) { return kc > kStageCols ? kStageCols : kc; }

// Sum N per-lane values across the warp so that lane `l` ends with the total
// of element `l / (32 / N)`; costs N shuffles instead of 5 * N.
template <int N>
__device__ __forceinline__ float warp_transpose_reduce(float (&v)[N], int lane) {
    static_assert(N == 1 || N == 2 || N == 4 || N == 8 || N == 16 || N == 32, "");
    int o = 16;
#pragma unroll
    for (int n = N / 2; n >= 1; n >>= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < n; ++i) {
            float send = upper ? v[i] : v[i + n];
            float keep = upper ? v[i + n] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
        o >>= 1;
    }
    float r = v[0];
#pragma unroll
    for (; o >= 1; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// --------------------------------------------------------------------------- //
// loader
// --------------------------------------------------------------------------- //
// split-KV geometry shared by loader and consumers
struct AttnRange {
    int t0;         // first position of this partial
    int t_old_end;  // end of the positions that were in the cache before this token
    int has_cur;    // the token being decoded falls into this partial
    int n_stages;
};
__device__ __forceinline__ AttnRange attn_range(const KParams& p, int pos, int num_partials,
                                                int partial_idx) {
    const int seq_len = pos + 1;
    const int total_blocks = (seq_len + 15) / 16;
    const int per = (total_blocks + num_partials - 1) / num_partials;
    const int b0 = partial_idx * per;
    const int b1 = min(b0 + per, total_blocks);
    AttnRange r;
    r.t0 = b0 * 16;
    const int t1 = min(b1 * 16, seq_len);
    r.has_cur = (pos >= r.t0 && pos < t1) ? 1 : 0;
    r.t_old_end = r.has_cur ? pos : t1;
    const int n_old = max(0, r.t_old_end - r.t0);
    const int ts = (kStageBytes / 4) / p.D;  // positions per stage: K and V halves of 16 KiB
    r.n_stages = (n_old + ts - 1) / ts;
    return r;
}

__device__ __forceinline__ void prefetch_l2_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// One ring stage worth of work for the loader: a tiled TMA copy.
struct StageDesc {
    const CUtensorMap* map;  // weights: 4-D view [64, rows, K/64, L]; nullptr for a K/V tile
    int c1, c2, c3;          // weights: row, 64-column chunk, layer
    uint32_t bytes;
    int kvh, t, lb;          // K/V tile coordinates
};

// Walks the instruction queue and yields its ring stages in consumption order.
// The loader keeps two of these: one for the stages it copies into the ring and
// one that runs ahead of it and only pulls the same bytes into L2.
struct StreamCursor {
    int i = -1;  // instruction index
    int op = 0;
    int b = 0, eb = 0;  // block (or KV stage) counter within the instruction
    int st = 0;         // stage inside the current block
    int sb = 0;         // first block index of a range instruction
    const int* w = nullptr;
    const CUtensorMap* map = nullptr;
    const CUtensorMap* map2 = nullptr;  // gate matrix of the up/gate op
    int chunk0 = 0, layer = 0;          // first 64-column chunk of the slice, layer
    int spb = 1;                        // stages per block
    uint32_t bytes = 0;
    int kvh = 0, t0 = 0, lb = 0, ts = 0;
    const Ctx* ctx = nullptr;  // positions of the tokens being decoded

    __device__ __forceinline__ void set_matrix(const CUtensorMap* m, int kc, int chunk0_, int layer_) {
        map = m;
        spb = stages_per_block(kc);
        bytes = (uint32_t)kBlockRows * stage_cols(kc) * 2u;
        chunk0 = chunk0_;
        layer = layer_;
    }

    // decode instruction `i`; leaves b == eb when it streams nothing
    __device__ void decode(const KParams& p, const int* queue) {
        w = queue + i * MKB_INTS_PER_INSTRUCTION;
        op = __ldg(w);
        b = eb = 0;
        st = 0;
        switch (op) {
            case MKB_OP_RMS_QKV_ROPE_APPEND:
                sb = __ldg(w + 2);
                eb = __ldg(w + 3) - sb;
                set_matrix(&p.qkv_map, p.H, 0, __ldg(w + 1));
                break;
            case MKB_OP_O_PROJ_RESIDUAL:
                sb = __ldg(w + 2);
                eb = __ldg(w + 3) - sb;
                set_matrix(&p.o_map, p.R, __ldg(w + 4) * (p.R / 64), __ldg(w + 1));
                break;
            case MKB_OP_RMS_UPGATE_SILU:
                eb = 2 * __ldg(w + 2);
                set_matrix(&p.up_map, p.H, 0, __ldg(w + 1));
                map2 = &p.gate_map;
                break;
            case MKB_OP_DOWN_PROJ_RESIDUAL:
                sb = __ldg(w + 2);
                eb = __ldg(w + 3) - sb;
                set_matrix(&p.down_map, p.R, __ldg(w + 4) * (p.R / 64), __ldg(w + 1));
                break;
            case MKB_OP_RMS_LM_HEAD:
                sb = __ldg(w + 1);
                eb = __ldg(w + 2) - sb;
                set_matrix(&p.lm_map, p.H, 0, 0);
                break;
            case MKB_OP_PARTIAL_ATTENTION: {
                const int seq = kBatch == 1 ? 0 : __ldg(w + 5);
                const AttnRange r = attn_range(p, ctx->pos_of(seq), __ldg(w + 3), __ldg(w + 4));
                kvh = __ldg(w + 2);
                lb = __ldg(w + 1) * p.B + seq;
                t0 = r.t0;
                ts = (kStageBytes / 4) / p.D;
                eb = r.n_stages;
            } break;
            default:
                break;
        }
    }

    // next stage of the stream; false when the queue is exhausted
    __device__ bool next(const KParams& p, const int* queue, StageDesc& d) {
        while (b >= eb) {
            if (++i >= p.queue_len) return false;
            decode(p, queue);
        }
        if (op == MKB_OP_PARTIAL_ATTENTION) {
            d.map = nullptr;
            d.kvh = kvh;
            d.t = t0 + b * ts;
            d.lb = lb;
            d.bytes = kStageBytes;
            ++b;
            return true;
        }
        int blk;
        const CUtensorMap* m = map;
        if (op == MKB_OP_RMS_UPGATE_SILU) {
            blk = __ldg(w + 3 + (b >> 1));
            if (b & 1) m = map2;
        } else {
            blk = sb + b;
        }
        d.map = m;
        d.c1 = blk * kBlockRows;
        d.c2 = chunk0 + st * (kStageCols / 64);
        d.c3 = layer;
        d.bytes = bytes;
        if (++st >= spb) {
            st = 0;
            ++b;
        }
        return true;
    }
};

__device__ __forceinline__ void prefetch_l2_tile4(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(map),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// The loader: one thread in each of `kLoaders` warps, each a complete copy of the loop below.
// Every loader walks the whole stage sequence and copies the stages dealt to it round-robin
// (stage % kLoaders == which); the L2 look-ahead is dealt the same way.  (The issue of a tiled
// 32 KiB copy occupies its thread for about 0.5 us: one thread feeds the ring at no more than
// 61 GB/s; two lanes of one warp would reconverge after every stage and issue one after the
// other, hence separate warps.)
__device__ __forceinline__ int loader_index(int warp) { return warp == kLoaderWarp ? 0 : warp - kStorerWarp; }

__device__ void loader_main(Ctx c, const int which) {
    const KParams& p = *c.p;
    const uint64_t policy = l2_policy_evict_first();
    const int* queue = p.instructions + (size_t)blockIdx.x * p.queue_len * MKB_INTS_PER_INSTRUCTION;
    c.role = kRoleLoader;

    // Norm weights are tiny but sit on the critical path right after every barrier; a miss
    // to HBM under full streaming load costs microseconds.  Pin them in L2 up front: CTA b
    // takes rows b, b + gridDim.x, ... of the 2 L + 1 norm vectors.
    if (which == 0) {
        uint64_t keep;
        asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep));
        for (int row = blockIdx.x; row < 2 * p.L + 1; row += gridDim.x) {
            const __nv_bfloat16* src = row < p.L ? p.attn_ln_w + (size_t)row * p.H
                                       : row < 2 * p.L ? p.mlp_ln_w + (size_t)(row - p.L) * p.H
                                                       : p.lm_norm_w;
            asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(src),
                         "r"((uint32_t)p.H * 2u), "l"(keep)
                         : "memory");
        }
    }
    StreamCursor issue, ahead;  // `ahead` is never behind `issue`
    issue.ctx = ahead.ctx = &c;
    StageDesc d, da;
    uint32_t stage = 0;       // stages of the sequence walked so far (all loaders' stages)
    uint32_t ahead_stage = 0; // stages the look-ahead cursor has passed
    uint32_t own_issued = 0;  // one past the last stage this loader copied into the ring
    bool ahead_more = true;
    bool stop = false;
    int last_instr = -1;
    bool have = issue.next(p, queue, d);
    while (have && !stop) {
        if (issue.i != last_instr) {
            if (which == 0 && last_instr >= 0) rec(c, MKB_T_LOADER_DONE);
            last_instr = issue.i;
            c.instr = issue.i;
            c.opcode = issue.op;
            if (which == 0) {
                rec(c, MKB_T_LOADER_START);
                if (issue.i + 2 < p.queue_len) prefetch_l1(queue + (issue.i + 2) * MKB_INTS_PER_INSTRUCTION);
            }
            if (*c.cta_abort) break;
        }
        if ((int)(stage % kLoaders) == which) {
            const int slot = stage % kNumStages;
            const uint32_t parity = ((stage / kNumStages) & 1u) ^ 1u;
            while (!mbar_try_wait(c.empty_bar(slot), parity)) {
                // ring full: use the time to pull upcoming weights into L2, where the
                // stalls of this SM's consumers cannot stop HBM from streaming
                // while the consumers sit in a barrier wait the ring cannot drain, so the
                // look-ahead may run deeper than in steady state
                const int window = c.cta_abort[4] ? p.l2_stall_window_stages : p.l2_window_stages;
                if (ahead_more && (int)(ahead_stage - stage) < window) {
                    ahead_more = ahead.next(p, queue, da);
                    // skip what the ring already holds or is about to receive, and the other loaders'
                    // share.  Weights only: K/V tiles in the look-ahead measured no gain (batched and
                    // 64k-context runs alike)
                    if (ahead_more && ahead_stage >= stage + kNumStages &&
                        (int)(ahead_stage % kLoaders) == which && da.map)
                        prefetch_l2_tile4(da.map, 0, da.c1, da.c2, da.c3);
                    ++ahead_stage;
                    continue;
                }
                if (!mbar_wait_slow(c, c.empty_bar(slot), parity, true)) stop = true;
                break;
            }
            if (stop) break;
            const uint32_t bar = c.full_bar(slot);
            const uint32_t dst = c.stage_addr(slot);
            mbar_expect_tx(bar, d.bytes);
            if (d.map == nullptr) {
                tma_tile5_g2s(dst, &p.k_map, 0, d.t, 0, d.kvh, d.lb, bar, policy);
                tma_tile5_g2s(dst + kStageBytes / 2, &p.v_map, 0, d.t, 0, d.kvh, d.lb, bar, policy);
            } else {
                tma_tile4_g2s(dst, d.map, 0, d.c1, d.c2, d.c3, bar, policy);
            }
            own_issued = stage + 1;
        }
        ++stage;
        have = issue.next(p, queue, d);
    }
    if (which == 0 && last_instr >= 0) rec(c, MKB_T_LOADER_DONE);
    // hand the extent of this loader's copies to the exit path (spare words of the HotConsts block)
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(c.base + kSmemHot + 56 + 4 * which), "r"(own_issued) : "memory");
}

// --------------------------------------------------------------------------- //
// consumers: matvec
// --------------------------------------------------------------------------- //
struct ConsumerState {
    uint32_t xstage = 0;  // GEMM build: activation-ring stages consumed so far
    uint32_t acc = 0;     // GEMM build: accumulator blocks issued so far (buffer = acc & 1)
    uint32_t slot = 0;    // ring slot of the next stage (mirrors the loader's sequence)
    uint32_t phase = 0;   // parity of that slot's current use
    uint32_t oslot = 0;   // output-ring slot of the next block (mirrors the storer's)
    uint32_t ophase = 0;
    uint32_t nverdict = 0;  // verdicts broadcast so far (selects one of two smem words)
    bool dead = false;   // a wait of this thread failed: finish the instruction without waiting
};

// The 512 consumer threads must leave the instruction loop together (they share
// a named barrier), so the decision to stop is taken by thread 0 only, written
// to one of two alternating shared words and read by everyone after a barrier.
__device__ __forceinline__ volatile int* verdict_word(const Ctx& c, ConsumerState& cs) {
    return c.cta_abort + 2 + (cs.nverdict++ & 1u);
}

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    f[0] = bf16_lo(w.x); f[1] = bf16_hi(w.x);
    f[2] = bf16_lo(w.y); f[3] = bf16_hi(w.y);
    f[4] = bf16_lo(w.z); f[5] = bf16_hi(w.z);
    f[6] = bf16_lo(w.w); f[7] = bf16_hi(w.w);
}

// D(16x8, fp32) += A(16x16, bf16, row-major) * B(16x8, bf16, column-major)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Wait for the ring stage at cs.slot.  Every lane performs the acquiring
// try_wait itself (see warp_mbar_wait for why); the bounded slow path is rare.
__device__ __forceinline__ uint32_t consumer_wait_stage(const Ctx& c, ConsumerState& cs) {
    const uint32_t bar = c.full_bar(cs.slot);
    if (!cs.dead && !mbar_try_wait(bar, cs.phase)) {
        if (!mbar_wait_slow(c, bar, cs.phase, true)) cs.dead = true;
    }
    return c.stage_addr(cs.slot);
}
__device__ __forceinline__ void consumer_release_stage(const Ctx& c, ConsumerState& cs, int lane) {
    if constexpr (kGemm) {
        // one arrival frees a stage in this build (the MMA issuer's commit, for the GEMM
        // instructions); the attention warps therefore meet before thread 0 arrives
        consumer_sync();
        if (threadIdx.x == 0) mbar_arrive(c.empty_bar(cs.slot));
    } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(c.empty_bar(cs.slot));
    }
    if (++cs.slot == kNumStages) {
        cs.slot = 0;
        cs.phase ^= 1u;
    }
}

// Multiply `nblocks` consecutive ring blocks (16 rows x kc) against the bf16
// activation vector parked in shared memory and hand each block's per-warp
// partial sums to the storer.
//
// Tensor-core formulation of the matvec: weights are the A operand (16 rows x 16
// k), the activation vector is column 0 of the B operand (the other 7 columns are
// zero; a batch of up to 8 tokens would fill them).  The k order inside an MMA is
// free as long as A and B agree, so thread (g = lane / 4, t = lane % 4) feeds the
// MMAs straight from 16-byte chunks: chunk t (and t + 4) of weight rows pi(g),
// pi(g) + 8 and the same chunk of the activations.  pi interleaves rows so that
// the two rows of one shared-memory phase fall into different swizzle classes,
// which makes the loads bank-conflict free.  After the last stage of a block the
// lanes with t == 0 hold the 16 row sums of this warp's 64 columns per stage.
__device__ __forceinline__ void consume_blocks(const Ctx& c, ConsumerState& cs, int nblocks, int kc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = ((g & 1) << 2) | (g >> 1);  // pi(g): 0,4,1,5,2,6,3,7
    const int spb = stages_per_block(kc);
    const bool has_cols = warp * 64 < stage_cols(kc);
    // byte offsets of this thread's two chunks inside a stage, rows row0 and row0 + 8
    const uint32_t line = (uint32_t)(warp * 16 + row0) * 128u;
    const uint32_t off_a = line + (uint32_t)((t ^ row0) << 4);
    const uint32_t off_b = line + (uint32_t)(((t + 4) ^ row0) << 4);
    // batched build: column g of the B operand is sequence g's activation vector
    const uint32_t act0 = c.base + kSmemAttn + (uint32_t)(warp * 64 + t * 8) * 2u + (uint32_t)(g * kActStride);

    for (int b = 0; b < nblocks; ++b) {
        // two accumulators: the four MMAs of a stage form two chains of two instead of one of four
        // (the latency of a dependent mma.sync, not its issue rate, bounds a warp's time per stage)
        float d[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f};
        for (int st = 0; st < spb; ++st) {
            const uint32_t sbase = consumer_wait_stage(c, cs);
            if (st == 0 && b == 0 && tid == 0) rec(c, MKB_T_CONSUMER_FIRST_STAGE);
            if (has_cols) {
                const uint4 w0 = lds_v4(sbase + off_a);
                const uint4 w1 = lds_v4(sbase + off_a + 8 * 128);
                const uint4 w2 = lds_v4(sbase + off_b);
                const uint4 w3 = lds_v4(sbase + off_b + 8 * 128);
                uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
                if (kBatch > 1 || g == 0) {
                    x0 = lds_v4(act0 + (uint32_t)st * (kStageCols * 2));
                    x1 = lds_v4(act0 + (uint32_t)st * (kStageCols * 2) + 64);
                }
                mma_16816(d, w0.x, w1.x, w0.y, w1.y, x0.x, x0.y);
                mma_16816(d2, w0.z, w1.z, w0.w, w1.w, x0.z, x0.w);
                mma_16816(d, w2.x, w3.x, w2.y, w3.y, x1.x, x1.y);
                mma_16816(d2, w2.z, w3.z, w2.w, w3.w, x1.z, x1.w);
            }
            consumer_release_stage(c, cs, lane);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) d[e] += d2[e];
        const uint32_t obar = c.out_empty_bar(cs.oslot);
        if (!cs.dead && !mbar_try_wait(obar, cs.ophase ^ 1u)) {
            if (!mbar_wait_slow(c, obar, cs.ophase ^ 1u, true)) cs.dead = true;
        }
        if constexpr (kBatch == 1) {
            if (t == 0) {  // column 0 of D: rows row0 (d[0]) and row0 + 8 (d[2])
                float* out = reinterpret_cast<float*>(__cvta_shared_to_generic(
                    c.base + kSmemOut + (cs.oslot * kOutSlotFloats + row0 * 16 + warp) * 4));
                out[0] = d[0];
                out[8 * 16] = d[2];
            }
        } else {
            // columns 2t, 2t + 1 of D are sequences 2t, 2t + 1: slot layout [row][sequence][16 partials].
            // Every (row, sequence) group starts on a 64-byte boundary, so without a rotation all 32
            // lanes of a store would hit one bank; the storer only sums a group's 16 floats, so the
            // position inside the group is free: rotate it per lane (2-way instead of 32-way conflicts).
            const int w_rot = (warp + ((g & 3) << 2) + t) & 15;
            float* out = reinterpret_cast<float*>(__cvta_shared_to_generic(
                c.base + kSmemOut + (cs.oslot * kOutSlotFloats + (row0 * kBatch + 2 * t) * 16 + w_rot) * 4));
            out[0] = d[0];
            out[16] = d[1];
            out[8 * kBatch * 16] = d[2];
            out[8 * kBatch * 16 + 16] = d[3];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(c.out_full_bar(cs.oslot));
        if (++cs.oslot == kOutSlots) {
            cs.oslot = 0;
            cs.ophase ^= 1u;
        }
    }
}

// Activation chunks (8 bf16 = 16 bytes) are parked in shared memory at
// act[chunk]; warp w only ever reads chunks {st * 128 + w * 8 + j}, so each warp
// loads, normalises and writes exactly its own chunks and a __syncwarp suffices.
// Lane l of warp w owns chunk (st, j) = (l / 8 + 4 * k, l % 8) for k = 0, 1.
// (The partition is in 1024-element groups whatever the ring-stage geometry of the build is.)
__device__ __forceinline__ int own_chunk(int warp, int lane, int k, int kc) {
    constexpr int kGroup = 1024;
    const int st = (lane >> 3) + 4 * k;
    const int col_chunk = warp * 8 + (lane & 7);  // within the group
    if (st >= (kc > kGroup ? kc / kGroup : 1) || col_chunk * 8 >= (kc > kGroup ? kGroup : kc)) return -1;
    return st * (kGroup / 8) + col_chunk;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c2, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c2), "r"(d) : "memory");
}

// Park a bf16 activation vector of `kc` elements in shared memory (batched build: the vectors
// of all sequences, `seq_stride` elements apart in global memory; unused columns are zeroed so
// that no stale NaN pattern ever enters an MMA).
__device__ __forceinline__ void stage_activation(const Ctx& c, const __nv_bfloat16* vec, int kc,
                                                 size_t seq_stride = 0) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if constexpr (kBatch == 1) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int ch = own_chunk(warp, lane, k, kc);
            if (ch >= 0) {
                const uint4 v = ld_cg_v4(vec + (size_t)ch * 8);
                st_shared_v4(c.base + kSmemAttn + ch * 16, v.x, v.y, v.z, v.w);
            }
        }
    } else if constexpr (!kGemm) {
        const int ch = own_chunk(warp, lane, 0, kc);  // kc <= 4096: one chunk per thread
        if (ch >= 0) {
            uint4 v[kBatch];
#pragma unroll
            for (int s = 0; s < kBatch; ++s) {
                v[s] = make_uint4(0, 0, 0, 0);
                if (s < c.p->batch) v[s] = ld_cg_v4(vec + s * seq_stride + (size_t)ch * 8);
            }
#pragma unroll
            for (int s = 0; s < kBatch; ++s)
                st_shared_v4(c.base + kSmemAttn + s * kActStride + ch * 16, v[s].x, v[s].y, v[s].z, v[s].w);
        }
    }
    __syncwarp();
}

// RMSNorm of the residual stream into shared memory (bf16).  Mirrors the reference's
// arithmetic: fp32 statistics, bf16 round of x * rstd, then times the bf16 weight, rounded to bf16
// (python_vm.py:50-56).  The code is rms_activation_body further down.

// Consumer thread 0 waits for a counter; the verdict reaches all 512 consumer
// threads through shared memory so that they leave the instruction together.
__device__ __forceinline__ bool consumers_wait_counter(const Ctx& c, ConsumerState& cs, int layer,
                                                       int row, int slot, int threshold,
                                                       bool needed) {
    volatile int* verdict = verdict_word(c, cs);
    if (threadIdx.x == 0) {
        bool ok = !*c.cta_abort;
        if (ok && needed) {
            c.cta_abort[4] = 1;  // tells the loader that the ring is not being drained
            ok = wait_counter(c, bar_addr(*c.p, layer, row, slot), threshold, layer, row, slot, (unsigned)c.p->poll_sleep_ns);
            c.cta_abort[4] = 0;
        }
        rec(c, MKB_T_CONSUMER_WAIT_DONE);
        *verdict = ok ? 1 : 0;
    }
    consumer_sync();
    return *verdict != 0;
}

// What rms_activation_body needs, in shared memory (written once by thread 0 at kernel start;
// `trow` = the timing row of the consumers' current instruction, or null, by consumer thread 0).
struct HotConsts {
    const __nv_bfloat16* hidden;
    const long long* acc;
    __nv_bfloat16* normed;
    int* trow;
    const uint4* ll;  // tensor parallelism: this rank's tagged residual stream
    int H;
    float inv_H;
    float eps;
    int pad;
};
static_assert(sizeof(HotConsts) == 56 && kLoaders <= 2, "two loader words follow at byte 56");

// The residual stream of an RMSNorm comes from one of three places:
//   kRmsAcc    `hidden` (the token embedding) + the Q31.32 accumulators the row-split projections
//              add into (single-GPU and batched builds); `read_done` (may be null) is a counter
//              bumped once every thread's loads have returned, for producers that must not add to
//              the accumulators before this instruction has read them;
//   kRmsHidden `hidden` alone (tensor parallelism: the embedding, before the first all-reduce);
//   kRmsTagged this rank's tagged buffer (tensor parallelism): every thread polls its own chunks
//              until they carry `tag`; returns false if the wait was abandoned.
// Batched build: `seq` selects the sequence, and the result goes to the global `normed` buffer
// (one RMS_NORM instruction per sequence) instead of shared memory.
//
// Nothing on the hot path comes through the stack: a function that receives the context by
// reference reads it back from local memory, and with 220 KB of the SM's 256 KB given to shared
// memory those loads miss L1 three times out of four - measured as 600 - 700 cycles each, eight
// or so in a row, 3 - 3.8 us per activation on the critical path of every layer where the loads
// of the vector itself take 0.3.  Constants come from shared memory (HotConsts); `c` is only
// touched when a tagged poll runs out of time.
enum RmsSource { kRmsAcc = 0, kRmsHidden = 1, kRmsTagged = 2 };
template <int CHUNKS, int SRC>
__device__ __forceinline__ bool rms_activation_body(const Ctx& c, const __nv_bfloat16* norm_w, int* read_done,
                                                    int seq, const uint4 w0, uint32_t tag, int layer, int which) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint4 h0 = lds_v4(base + kSmemHot), h1 = lds_v4(base + kSmemHot + 16), h2 = lds_v4(base + kSmemHot + 32);
    const __nv_bfloat16* hidden = reinterpret_cast<const __nv_bfloat16*>(((unsigned long long)h0.y << 32) | h0.x);
    const long long* accp = reinterpret_cast<const long long*>(((unsigned long long)h0.w << 32) | h0.z);
    [[maybe_unused]] __nv_bfloat16* normed = reinterpret_cast<__nv_bfloat16*>(((unsigned long long)h1.y << 32) | h1.x);
    int* trow = reinterpret_cast<int*>(((unsigned long long)h1.w << 32) | h1.z);
    const uint4* ll = reinterpret_cast<const uint4*>(((unsigned long long)h2.y << 32) | h2.x);
    const int H = (int)h2.z;
    const float inv_H = __uint_as_float(h2.w), eps = __uint_as_float(lds_u32(base + kSmemHot + 48));
    const size_t seq_off = kBatch == 1 ? 0 : (size_t)seq * H;

    // one chunk of 8 elements per thread up to H = 4096, a second one (loaded after the first has
    // been converted: fewer live registers, one more round trip) beyond
    int chs[CHUNKS];
    uint4 wv[CHUNKS];
    float x[CHUNKS][8];
    float ss = 0.f;
    bool ok = true;
    if constexpr (SRC == kRmsTagged) {
        // tells the loader that the ring is not being drained (control word 4)
        if (tid == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + kSmemCtl + 16), "r"(1) : "memory");
    }
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        chs[k] = own_chunk(warp, lane, k, H);
        if (chs[k] < 0) continue;
        if constexpr (CHUNKS == 1) wv[k] = w0;
        else wv[k] = ld_nc_v4(norm_w + (size_t)chs[k] * 8);
        if constexpr (SRC == kRmsTagged) {
            // 8 bf16 = four {bf16x2, tag} words = two 16-byte loads
            TpPoll poll;
            uint4 a, b;
            while (true) {
                a = ld_volatile_v4(ll + (size_t)chs[k] * 2);
                b = ld_volatile_v4(ll + (size_t)chs[k] * 2 + 1);
                if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) break;
                if (!poll.tick(c, layer, 100 + which, chs[k], (int)a.y)) {
                    ok = false;
                    break;
                }
            }
            unpack8(make_uint4(a.x, a.z, b.x, b.z), x[k]);
        } else {
            const uint4 hv = ld_cg_v4(hidden + seq_off + (size_t)chs[k] * 8);
            if constexpr (SRC == kRmsAcc) {
                const long long* acc = accp + seq_off + (size_t)chs[k] * 8;
                uint4 a[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = ld_cg_v4(acc + 2 * i);
                unpack8(hv, x[k]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    x[k][2 * i] += q32_to_float(a[i].x, a[i].y);
                    x[k][2 * i + 1] += q32_to_float(a[i].z, a[i].w);
                }
            } else {
                unpack8(hv, x[k]);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(x[k][e], x[k][e], ss);
    }
    if constexpr (SRC == kRmsTagged) {
        if (tid == 0) {
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + kSmemCtl + 16), "r"(0) : "memory");
            if (trow != nullptr) trow[MKB_T_CONSUMER_WAIT_DONE] = (int)(uint32_t)globaltimer_ns();
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) asm volatile("st.shared.f32 [%0], %1;" ::"r"(base + kSmemRed + warp * 4), "f"(ss) : "memory");
    if (tid == 0 && trow != nullptr) trow[MKB_T_RMS_LOADED] = (int)(uint32_t)globaltimer_ns();
    if constexpr (SRC == kRmsTagged) {
        if (!consumer_all(ok)) return false;
    } else {
        consumer_sync();
        // every thread's loads of the residual stream have returned (their values went into
        // the sums above), so later writers may now be let in.  A relaxed add is enough: a
        // load that has delivered its value cannot observe a store issued afterwards, and a
        // releasing add would stall this thread (and with it warp 0 and the whole ring) on a fence.
        if (tid == 0 && read_done != nullptr) atomicAdd(read_done, 1);
    }
    if (tid == 0 && trow != nullptr) trow[MKB_T_RMS_SUMMED] = (int)(uint32_t)globaltimer_ns();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < kConsumerWarps; k += 4) {
        const uint4 r = lds_v4(base + kSmemRed + k * 4);
        tot += __uint_as_float(r.x) + __uint_as_float(r.y) + __uint_as_float(r.z) + __uint_as_float(r.w);
    }
    const float rstd = rsqrtf(tot * inv_H + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        if (chs[k] >= 0) {
            float wgt[8];
            unpack8(wv[k], wgt);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                o[e] = pack_bf16x2(wgt[2 * e] * bf16_round(x[k][2 * e] * rstd),
                                   wgt[2 * e + 1] * bf16_round(x[k][2 * e + 1] * rstd));
            if constexpr (kBatch == 1)
                st_shared_v4(base + kSmemAttn + chs[k] * 16, o[0], o[1], o[2], o[3]);
            else
                *reinterpret_cast<uint4*>(normed + seq_off + (size_t)chs[k] * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    __syncwarp();
    return true;
}

// Up to 4096 elements a thread holds one chunk and the code is light enough to be inlined (an
// out-of-line copy pays for its callee-saved registers with 2 x 48 KB of local-memory traffic per
// call, over a microsecond); wider models (two chunks per thread) take an out-of-line copy, whose
// inlining would make the compiler spill state of the whole consumer loop.
template <int SRC>
__device__ __noinline__ bool rms_activation_wide(const Ctx& c, const __nv_bfloat16* norm_w, int* read_done, int seq,
                                                 uint32_t tag, int layer, int which) {
    return rms_activation_body<2, SRC>(c, norm_w, read_done, seq, make_uint4(0, 0, 0, 0), tag, layer, which);
}
template <int SRC>
__device__ __forceinline__ bool rms_activation_from(const Ctx& c, int H, const __nv_bfloat16* norm_w, const uint4 w0,
                                                    int* read_done = nullptr, int seq = 0, uint32_t tag = 0,
                                                    int layer = 0, int which = 0) {
    if (H <= 4096) return rms_activation_body<1, SRC>(c, norm_w, read_done, seq, w0, tag, layer, which);
    return rms_activation_wide<SRC>(c, norm_w, read_done, seq, tag, layer, which);
}
// The norm weights do not depend on the barrier: the one-chunk path fetches them before waiting
// (the 48 KB an activation reads go through the SM's load pipe at 64 bytes per cycle; 8 KB less
// after the barrier is 0.1 us less on the critical path).
__device__ __forceinline__ uint4 rms_weights_early(int H, const __nv_bfloat16* norm_w) {
    const int ch = own_chunk(threadIdx.x >> 5, threadIdx.x & 31, 0, H);
    return (H <= 4096 && ch >= 0) ? ld_nc_v4(norm_w + (size_t)ch * 8) : make_uint4(0, 0, 0, 0);
}

// kTP selects the tensor-parallel build of the kernel.  It is a compile-time switch and the two
// builds are separate kernels: merely having the exchange code in the same kernel cost the
// single-GPU path 4 % (measured; the compiler's register allocation for the whole kernel moves).
template <bool kTP>
__device__ __forceinline__ bool consumer_rms_matvec(const Ctx& c, ConsumerState& cs,
                                                    const __nv_bfloat16* norm_w, int nblocks,
                                                    int wait_layer, int wait_row, int threshold,
                                                    bool needed, int* read_done = nullptr,
                                                    int norm_layer = 0, int norm_slot = 0) {
    if constexpr (kBatch > 1) {
        // batched build: RMS_NORM instructions (one per sequence) have published the normalised
        // activations of all sequences; wait for them and park the vectors
        if (!consumers_wait_counter(c, cs, norm_layer, MKB_BARRIER_ROW_RMS_NORM, norm_slot, c.p->batch, true))
            return false;
        stage_activation(c, c.p->normed, c.p->H, (size_t)c.p->H);
        if (threadIdx.x == 0) rec(c, MKB_T_CONSUMER_ACT_READY);
        consume_blocks(c, cs, nblocks, c.p->H);
        return true;
    }
    const int H = c.p->H;
    const uint4 w0 = rms_weights_early(H, norm_w);
    bool tagged = false;
    if constexpr (kTP) {
        if (c.p->tp_size > 1) {
            if (needed) {
                // the residual stream arrives as tagged values from the chunk owners
                const int which = wait_row == MKB_OP_O_PROJ_RESIDUAL - 1 ? 0 : 1;
                if (!rms_activation_from<kRmsTagged>(c, H, norm_w, w0, nullptr, 0, tp_tag(c, wait_layer, which),
                                                     wait_layer, which))
                    return false;
            } else {
                // the tensor-parallel exchange keeps the running residual stream in its tagged
                // buffer; the only plain read there is the token embedding before the first all-reduce
                rms_activation_from<kRmsHidden>(c, H, norm_w, w0);
            }
            tagged = true;
        }
    }
    if (!tagged) {
        if (!consumers_wait_counter(c, cs, wait_layer, wait_row, 0, threshold, needed)) return false;
        rms_activation_from<kRmsAcc>(c, H, norm_w, w0, read_done);
    }
    if (threadIdx.x == 0) rec(c, MKB_T_CONSUMER_ACT_READY);
    consume_blocks(c, cs, nblocks, c.p->H);
    return true;
}

// Warp 0 polls up to 32 counters in parallel (lane i: addr / threshold, nullptr = none); the
// verdict reaches all 512 consumer threads through shared memory.
__device__ __forceinline__ bool consumers_wait_lanes(const Ctx& c, ConsumerState& cs, const int* addr,
                                                     int threshold, int layer, int row, int slot) {
    volatile int* verdict = verdict_word(c, cs);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        bool ok = __shfl_sync(0xffffffffu, *c.cta_abort, 0) == 0;  // uniform over the warp
        if (lane == 0) c.cta_abort[4] = 1;  // tells the loader that the ring is not being drained
        ok = ok && warp_wait_counters(c, addr, threshold, layer, row, slot, (unsigned)c.p->poll_sleep_ns);
        if (lane == 0) {
            c.cta_abort[4] = 0;
            rec(c, MKB_T_CONSUMER_WAIT_DONE);
            *verdict = ok ? 1 : 0;
        }
    }
    consumer_sync();
    return *verdict != 0;
}

// `also` (may be null) is a second counter that must reach `also_threshold` before the vector
// may be read or the outputs added: both are polled in the same round trips.
__device__ __forceinline__ bool consumer_plain_matvec(const Ctx& c, ConsumerState& cs,
                                                      const __nv_bfloat16* vec, int nblocks,
                                                      int wait_layer, int wait_row, int wait_slot,
                                                      int threshold, const int* also = nullptr,
                                                      int also_threshold = 0, size_t seq_stride = 0) {
    if (also != nullptr) {
        const int lane = threadIdx.x & 31;
        const int* addr = lane == 0 ? bar_addr(*c.p, wait_layer, wait_row, wait_slot) : lane == 1 ? also : nullptr;
        if (!consumers_wait_lanes(c, cs, addr, lane == 1 ? also_threshold : threshold, wait_layer,
                                  lane == 1 ? MKB_BARRIER_ROW_RMS_READ : wait_row, lane == 1 ? 0 : wait_slot))
            return false;
    } else if (!consumers_wait_counter(c, cs, wait_layer, wait_row, wait_slot, threshold, true)) {
        return false;
    }
    stage_activation(c, vec, c.p->R, seq_stride);
    if (threadIdx.x == 0) rec(c, MKB_T_CONSUMER_ACT_READY);
    consume_blocks(c, cs, nblocks, c.p->R);
    return true;
}

// --------------------------------------------------------------------------- //
// consumers: attention
// --------------------------------------------------------------------------- //
// Online-softmax state of one warp for GQA heads, DPL = D / 32 dims per lane.
template <int GQA, int DPL>
struct AttnAcc {
    float m[GQA];       // running max (log2 domain)
    float l[GQA];       // running denominator
    float o[GQA][DPL];  // running numerator, this lane's dims
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
            m[h] = -INFINITY;
            l[h] = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[h][i] = 0.f;
        }
    }
};

template <int DPL>
__device__ __forceinline__ void load_row_smem(uint32_t addr, float (&f)[DPL]) {
    if constexpr (DPL == 4) {
        const uint2 w = lds_v2(addr);
        f[0] = bf16_lo(w.x); f[1] = bf16_hi(w.x); f[2] = bf16_lo(w.y); f[3] = bf16_hi(w.y);
    } else {
        const uint32_t w = lds_u32(addr);
        f[0] = bf16_lo(w); f[1] = bf16_hi(w);
    }
}
template <int DPL>
__device__ __forceinline__ void load_row_gmem(const __nv_bfloat16* ptr, float (&f)[DPL]) {
    if constexpr (DPL == 4) {
        const uint2 w = ld_cg_v2(ptr);
        f[0] = bf16_lo(w.x); f[1] = bf16_hi(w.x); f[2] = bf16_lo(w.y); f[3] = bf16_hi(w.y);
    } else {
        const uint32_t w = ld_cg_u32(ptr);
        f[0] = bf16_lo(w); f[1] = bf16_hi(w);
    }
}

// Fold NP positions (scores already reduced: every lane holds s[j][h]) into acc.
template <int GQA, int DPL, int NP>
__device__ __forceinline__ void attn_fold(AttnAcc<GQA, DPL>& a, const float (&s)[NP][GQA],
                                          const float (&v)[NP][DPL]) {
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
        float mx = a.m[h];
#pragma unroll
        for (int j = 0; j < NP; ++j) mx = fmaxf(mx, s[j][h]);
        const float ms = (mx == -INFINITY) ? 0.f : mx;
        const float alpha = exp2f(a.m[h] - ms);
        a.m[h] = mx;
        float lsum = a.l[h] * alpha;
#pragma unroll
        for (int i = 0; i < DPL; ++i) a.o[h][i] *= alpha;
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const float pj = exp2f(s[j][h] - ms);
            lsum += pj;
#pragma unroll
            for (int i = 0; i < DPL; ++i) a.o[h][i] = fmaf(pj, v[j][i], a.o[h][i]);
        }
        a.l[h] = lsum;
    }
}

// skip_attn_reduction == 2: no AttentionReduction instructions.  Every partial-attention
// instruction, once its (O, LSE) rows are stored, bumps the counters of its heads; the bump of the
// first head returns the previous count, and the instruction that finds np - 1 there is the last of
// its KV head to arrive: it merges the np partial rows of the GQA heads (all visible to it: each
// writer's bump was a release, this one is an acquire) with the arithmetic of the terminal
// reduction, writes attn_out and signals the o-proj's counter.  Compared with a separate
// instruction this takes the poll for the partials, an instruction boundary and the reduction
// instruction's own start-up off the critical path of every layer.
template <int D, int GQA>
__device__ __forceinline__ void attn_arrive_and_merge(const Ctx& c, ConsumerState& cs, int layer, int kvh,
                                                      int np, int part_slot0, const float* attn_o,
                                                      const float* attn_lse, __nv_bfloat16* attn_out) {
    const KParams& p = *c.p;
    const int tid = threadIdx.x, lane = tid & 31;
    volatile int* verdict = verdict_word(c, cs);
    if (tid < 32) {
        int last = 0;
        if (lane < GQA && !cs.dead) {
            int* addr = bar_addr(p, layer, MKB_OP_PARTIAL_ATTENTION - 1, part_slot0 + kvh * GQA + lane);
            if (lane == 0) {
                int old;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(addr) : "memory");
                last = old == np - 1;
            } else {
                red_release_gpu_add(addr, 1);
            }
        }
        if (lane == 0) *verdict = last;
    }
    consumer_sync();
    if (*verdict == 0) return;
    for (int idx = tid; idx < GQA * D; idx += kConsumerThreads) {  // whole warps: a warp stays inside one head
        const int head = kvh * GQA + idx / D, dim = idx % D;
        float lse = -INFINITY;
        if (lane < np) lse = ld_cg_f32(attn_lse + (size_t)head * p.max_partials + lane);
        constexpr int NB = 12;
        const float* base = attn_o + (size_t)head * p.max_partials * D + dim;
        float acc = 0.f, wgt = 0.f, denom = 0.f;
        for (int j0 = 0; j0 < np; j0 += NB) {
            float part[NB];
#pragma unroll
            for (int jj = 0; jj < NB; ++jj) part[jj] = ld_cg_f32(base + (size_t)(j0 + jj < np ? j0 + jj : 0) * D);
            if (j0 == 0) {
                float mx = lse;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float ms = (mx == -INFINITY) ? 0.f : mx;
                wgt = exp2f(lse - ms);
                denom = wgt;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
            }
#pragma unroll
            for (int jj = 0; jj < NB; ++jj) {
                const int j = j0 + jj;
                const float wj = (j < np) ? __shfl_sync(0xffffffffu, wgt, j & 31) : 0.f;
                acc = fmaf(wj, part[jj], acc);
            }
        }
        const float val = acc * (denom > 0.f ? 1.f / denom : 0.f);
        const float hi = __shfl_down_sync(0xffffffffu, val, 1);
        if ((dim & 1) == 0) *reinterpret_cast<uint32_t*>(attn_out + (size_t)head * D + dim) = pack_bf16x2(val, hi);
    }
    consumer_sync();  // every thread's stores precede the signal
    if (tid == 0) red_release_gpu_add(bar_addr(p, layer, MKB_OP_ATTENTION_REDUCTION - 1, 0), GQA);
}

template <int D, int GQA>
__device__ bool consumer_attention(const Ctx& c, ConsumerState& cs, const int* w) {
    constexpr int DPL = D / 32;
    constexpr int TS = (kStageBytes / 4) / D;      // positions per stage
    const KParams& p = *c.p;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int layer = __ldg(w + 1), kvh = __ldg(w + 2), np = __ldg(w + 3), pi = __ldg(w + 4);
    // batched build: the sequence this instruction serves, its position and its activation rows
    const int seq = kBatch == 1 ? 0 : __ldg(w + 5);
    const int pos_tok = c.pos_of(seq);
    const AttnRange r = attn_range(p, pos_tok, np, pi);
    const __nv_bfloat16* q_rope = p.q_rope + (size_t)seq * p.o_in;
    __nv_bfloat16* attn_out = p.attn_out + (size_t)seq * p.o_in;
    float* attn_o = p.attn_o + (size_t)seq * p.Hq * p.max_partials * D;
    float* attn_lse = p.attn_lse + (size_t)seq * p.Hq * p.max_partials;
    const int part_slot0 = seq * p.Hq;  // this sequence's slots in the partial-attention barrier row

    // barrier: the GQA query heads, then this KV head's K and V blocks
    {
        volatile int* verdict = verdict_word(c, cs);
        if (warp == 0) {
            // lanes 0..GQA-1: the query heads; then this KV head's K and V slots
            const int row = MKB_OP_RMS_QKV_ROPE_APPEND - 1;
            int slot = -1;
            if (lane < GQA) slot = kvh * GQA + lane;
            else if (lane == GQA) slot = p.Hq + kvh;
            else if (lane == GQA + 1) slot = p.Hq + p.Hkv + kvh;
            bool ok = __shfl_sync(0xffffffffu, *c.cta_abort, 0) == 0;  // uniform over the warp
            ok = ok && warp_wait_counters(c, slot >= 0 ? bar_addr(p, layer, row, slot) : nullptr,
                                          p.thr_attn_waits_qkv, layer, row, slot, (unsigned)p.poll_sleep_ns);
            if (lane == 0) {
                rec(c, MKB_T_CONSUMER_WAIT_DONE);
                *verdict = ok ? 1 : 0;
            }
        }
        consumer_sync();
        if (*verdict == 0) return false;
    }

    // ---- tensor-core flash decoding ------------------------------------------------
    // A stage holds TS positions of K and V.  It is cut into units of 16 positions
    // and the head dimension into slices of 32: warp (unit, slice) computes the
    // scores of its unit over the full head dimension (S^T = Q K^T, M = heads padded
    // to 16, N = 8 positions per MMA) and accumulates O for its 32 dimensions
    // (O = P V with V fed through ldmatrix.trans).  Warps of the same unit repeat the
    // cheap score computation so that no exchange is needed before the end.
    constexpr int U = TS / 16;            // units per stage
    constexpr int SL = D / 32;            // 32-dim slices; U * SL == 16 warps
    static_assert(U * SL == kConsumerWarps, "warp grid must cover a stage");
    constexpr int KP = D / 32;            // 16-byte chunk pairs of a K row per thread (2 k-steps each)
    const int unit = warp / SL, slice = warp % SL;
    const int g = lane >> 2, t = lane & 3;
    const bool head_ok = g < GQA;

    // Q as A operand: row g = head g, chunk (t + 4 j) of the head dimension
    uint4 qa[KP];
#pragma unroll
    for (int j = 0; j < KP; ++j) {
        qa[j] = make_uint4(0, 0, 0, 0);
        if (head_ok) qa[j] = ld_cg_v4(q_rope + (size_t)(kvh * GQA + g) * D + (t + 4 * j) * 8);
    }
    if (tid == 0) rec(c, MKB_T_CONSUMER_ACT_READY);
    // the token being decoded: its K/V were appended by another SM in this launch,
    // so warp 0 reads them straight from global memory (issued now, used last)
    float k_cur[DPL], v_cur[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) k_cur[i] = v_cur[i] = 0.f;
    // its score is taken right away (these loads return together with the Q fragments, which
    // the first stage needs anyway), so that only GQA scores and the V row stay in registers
    float s_cur[GQA];
#pragma unroll
    for (int h = 0; h < GQA; ++h) s_cur[h] = -INFINITY;
    if (warp == 0 && r.has_cur) {
        const size_t off = (((size_t)layer * p.B + seq) * p.T + pos_tok) * p.Hkv * D + (size_t)kvh * D + lane * DPL;
        load_row_gmem<DPL>(p.k_cache + off, k_cur);
        load_row_gmem<DPL>(p.v_cache + off, v_cur);
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
            float q_cur[DPL];
            load_row_gmem<DPL>(q_rope + (size_t)(kvh * GQA + h) * D + lane * DPL, q_cur);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) d = fmaf(q_cur[i], k_cur[i], d);
            s_cur[h] = d;
        }
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
            float d = s_cur[h];
#pragma unroll
            for (int o2 = 16; o2 >= 1; o2 >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o2);
            s_cur[h] = d * p.attn_scale_log2e;
        }
    }

    float m_run = -INFINITY, l_run = 0.f;  // head g, replicated over t
    float o[4][4];                          // 4 n-tiles of 8 dims; [i][0..1] belong to head g
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int s = 0; s < r.n_stages; ++s) {
        const uint32_t kbase = consumer_wait_stage(c, cs);
        const uint32_t vbase = kbase + kStageBytes / 2;
        const int pos0 = r.t0 + s * TS + unit * 16;  // first position of this warp's unit
        if (pos0 < r.t_old_end) {
            // scores: two n-tiles of 8 positions
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
                // position (unit * 16 + nt * 8 + g) is line g of its 1024-byte swizzle block; the
                // 16-byte chunk at byte (t * 16 + j * 64) of the row lives in sub-tile j / 2
                const uint32_t krow = kbase + (uint32_t)(unit * 16 + nt * 8 + g) * 128u;
#pragma unroll
                for (int j = 0; j < KP; ++j) {
                    const uint4 kk = lds_v4(krow + (uint32_t)(j >> 1) * (TS * 128) + (uint32_t)(((t + 4 * (j & 1)) ^ g) << 4));
                    mma_16816(sc[nt], qa[j].x, 0u, qa[j].y, 0u, kk.x, kk.y);
                    mma_16816(sc[nt], qa[j].z, 0u, qa[j].w, 0u, kk.z, kk.w);
                }
            }
            // scale into the log2 domain, mask, running max of head g
            float smax = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int pos = pos0 + nt * 8 + 2 * t + e;
                    const float v = (pos < r.t_old_end) ? sc[nt][e] * p.attn_scale_log2e : -INFINITY;
                    sc[nt][e] = v;
                    smax = fmaxf(smax, v);
                }
            smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, 1));
            smax = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, 2));
            const float m_new = fmaxf(m_run, smax);
            const float ms = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = exp2f(m_run - ms);
            m_run = m_new;
            float psum = 0.f;
            uint32_t pa[2];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float p0 = exp2f(sc[nt][0] - ms), p1 = exp2f(sc[nt][1] - ms);
                psum += p0 + p1;
                pa[nt] = pack_bf16x2(p0, p1);
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run = l_run * alpha + psum;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                o[i][0] *= alpha;
                o[i][1] *= alpha;
            }
            // O += P V: V rows (positions) x 8-dim column tiles through ldmatrix.trans
            const int mat = lane >> 3, rr = lane & 7;
            // row (position) rr of a swizzle block; byte column slice * 64 + (mat >> 1) * 16 + h2 * 32
            // of the 2 D-byte row: sub-tile slice / 2, chunk (slice & 1) * 4 + (mat >> 1) + 2 * h2
            const uint32_t vrow = vbase + (uint32_t)(slice >> 1) * (TS * 128) +
                                  (uint32_t)(unit * 16 + (mat & 1) * 8 + rr) * 128u;
            const uint32_t vchunk = (uint32_t)((slice & 1) * 4 + (mat >> 1));
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {  // two pairs of n-tiles
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                             : "r"(vrow + (((vchunk + 2 * h2) ^ (uint32_t)rr) << 4)));
                mma_16816(o[2 * h2], pa[0], 0u, pa[1], 0u, b0, b1);
                mma_16816(o[2 * h2 + 1], pa[0], 0u, pa[1], 0u, b2, b3);
            }
        }
        // the last KV stage stays ours: its 32 KiB become the merge scratch below
        if (s + 1 < r.n_stages) consumer_release_stage(c, cs, lane);
    }
    if (tid == 0) rec(c, MKB_T_ATTN_STAGES_DONE);

    if (r.n_stages == 0) {
        // no cached positions in this slice: at most the current token, whose softmax weight is 1
        if (warp == 0 && !cs.dead) {
#pragma unroll
            for (int h = 0; h < GQA; ++h) {
                const int head = kvh * GQA + h;
                const float wgt = r.has_cur ? 1.f : 0.f;
                if (p.skip_attn_reduction == 1) {
                    __nv_bfloat16* dst = attn_out + (size_t)head * D + lane * DPL;
                    if constexpr (DPL == 4) {
                        uint2 v;
                        v.x = pack_bf16x2(v_cur[0] * wgt, v_cur[1] * wgt);
                        v.y = pack_bf16x2(v_cur[2] * wgt, v_cur[3] * wgt);
                        *reinterpret_cast<uint2*>(dst) = v;
                    } else {
                        *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(v_cur[0] * wgt, v_cur[1] * wgt);
                    }
                } else {
                    float* dst = attn_o + ((size_t)head * p.max_partials + pi) * D + lane * DPL;
#pragma unroll
                    for (int i = 0; i < DPL; ++i) dst[i] = v_cur[i] * wgt;
                    if (lane == 0)
                        attn_lse[(size_t)head * p.max_partials + pi] = r.has_cur ? s_cur[h] : -INFINITY;
                }
            }
            __syncwarp();
            if (p.skip_attn_reduction == 1) {
                if (lane == 0)
                    red_release_gpu_add(bar_addr(p, layer, MKB_OP_ATTENTION_REDUCTION - 1, 0), GQA);
            } else if (p.skip_attn_reduction == 0) {
                if (lane < GQA)
                    red_release_gpu_add(bar_addr(p, layer, MKB_OP_PARTIAL_ATTENTION - 1, part_slot0 + kvh * GQA + lane), 1);
            }
        }
        if (p.skip_attn_reduction == 2) {
            consumer_sync();  // warp 0's rows are stored
            attn_arrive_and_merge<D, GQA>(c, cs, layer, kvh, np, part_slot0, attn_o, attn_lse, attn_out);
        }
        return true;
    }

    // One-round merge of the U units (+ the current token as entry U): O goes into the
    // KV stage we still own, [entry][head][D]; (m, l) into the small scratch.
    float* so = reinterpret_cast<float*>(__cvta_shared_to_generic(c.stage_addr(cs.slot)));
    float* sml = reinterpret_cast<float*>(__cvta_shared_to_generic(c.base + kSmemAttn));
    consumer_sync();  // every warp is done reading K/V from the stage
    if (head_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float* dst = so + (size_t)(unit * GQA + g) * D + slice * 32 + i * 8 + 2 * t;
            dst[0] = o[i][0];
            dst[1] = o[i][1];
        }
        if (slice == 0 && t == 0) {
            sml[(unit * GQA + g) * 2 + 0] = m_run;
            sml[(unit * GQA + g) * 2 + 1] = l_run;
        }
    }
    if (warp == 0) {
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) so[(size_t)(U * GQA + h) * D + lane * DPL + i] = v_cur[i];
            if (lane == 0) {
                sml[(U * GQA + h) * 2 + 0] = s_cur[h];
                sml[(U * GQA + h) * 2 + 1] = r.has_cur ? 1.f : 0.f;
            }
        }
    }
    consumer_sync();
    for (int idx = tid; idx < GQA * D; idx += kConsumerThreads) {  // whole warps: D is a multiple of 32
        const int hh = idx / D, d = idx % D;
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e <= U; ++e) mx = fmaxf(mx, sml[(e * GQA + hh) * 2]);
        const float ms = (mx == -INFINITY) ? 0.f : mx;
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int e = 0; e <= U; ++e) {
            const float a2 = exp2f(sml[(e * GQA + hh) * 2] - ms);
            den = fmaf(a2, sml[(e * GQA + hh) * 2 + 1], den);
            num = fmaf(a2, so[(size_t)(e * GQA + hh) * D + d], num);
        }
        const float val = den > 0.f ? num / den : 0.f;
        const int head = kvh * GQA + hh;
        if (p.skip_attn_reduction == 1) {
            const float hi = __shfl_down_sync(0xffffffffu, val, 1);
            if ((d & 1) == 0 && !cs.dead)
                *reinterpret_cast<uint32_t*>(attn_out + (size_t)head * D + d) = pack_bf16x2(val, hi);
        } else if (!cs.dead) {
            attn_o[((size_t)head * p.max_partials + pi) * D + d] = val;
            if (d == 0)
                attn_lse[(size_t)head * p.max_partials + pi] = den > 0.f ? mx + log2f(den) : -INFINITY;
        }
    }
    consumer_sync();  // scratch reads and global stores of all threads are done
    consumer_release_stage(c, cs, lane);
    if (p.skip_attn_reduction == 2) {
        attn_arrive_and_merge<D, GQA>(c, cs, layer, kvh, np, part_slot0, attn_o, attn_lse, attn_out);
        return true;
    }
    if (warp == 0 && !cs.dead) {
        if (p.skip_attn_reduction) {
            if (lane == 0)
                red_release_gpu_add(bar_addr(p, layer, MKB_OP_ATTENTION_REDUCTION - 1, 0), GQA);
        } else {
            if (lane < GQA)
                red_release_gpu_add(bar_addr(p, layer, MKB_OP_PARTIAL_ATTENTION - 1, part_slot0 + kvh * GQA + lane), 1);
        }
    }
    return true;
}

// AttentionReduction: merge `n` partial (O, LSE) pairs for 4 consecutive heads.
// One output element per thread (thread = head * D + dim), so a batch of 12 partial rows costs 12
// registers and all its loads are in flight together: one L2 round trip for up to 12 partials.
template <int D>
__device__ bool consumer_attn_reduction(const Ctx& c, ConsumerState& cs, const int* w) {
    const KParams& p = *c.p;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int layer = __ldg(w + 1), h0 = __ldg(w + 2), num_partials = __ldg(w + 3);
    const int is_terminal = __ldg(w + 4), n = __ldg(w + 5);
    const int out_idx = __ldg(w + 6 + n);
    // batched build: the sequence's own intermediates, output rows and barrier slots
    const int seq = kBatch == 1 ? 0 : __ldg(w + 7 + n);
    float* attn_o = p.attn_o + (size_t)seq * p.Hq * p.max_partials * D;
    float* attn_lse = p.attn_lse + (size_t)seq * p.Hq * p.max_partials;
    __nv_bfloat16* attn_out = p.attn_out + (size_t)seq * p.o_in;
    const int part_slot0 = seq * p.Hq;
    volatile int* verdict = verdict_word(c, cs);
    if (warp == 0) {
        const int row = MKB_OP_PARTIAL_ATTENTION - 1;
        bool ok = __shfl_sync(0xffffffffu, *c.cta_abort, 0) == 0;  // uniform over the warp
        ok = ok && warp_wait_counters(c, lane < 4 ? bar_addr(p, layer, row, part_slot0 + h0 + lane) : nullptr,
                                      num_partials, layer, row, h0 + lane, (unsigned)p.poll_sleep_ns);
        if (lane == 0) {
            rec(c, MKB_T_CONSUMER_WAIT_DONE);
            *verdict = ok ? 1 : 0;
        }
    }
    consumer_sync();
    if (*verdict == 0) return false;

    const bool active = tid < 4 * D;  // whole warps: D is a multiple of 32
    if (active) {
        const int head = h0 + tid / D, dim = tid % D;
        int idx = 0;
        float lse = -INFINITY;
        if (lane < n) {
            idx = __ldg(w + 6 + lane);
            lse = ld_cg_f32(attn_lse + (size_t)head * p.max_partials + idx);
        }
        constexpr int NB = 12;
        const float* base = attn_o + (size_t)head * p.max_partials * D + dim;
        float acc = 0.f, mx = 0.f, wgt = 0.f, denom = 0.f;
        for (int j0 = 0; j0 < n; j0 += NB) {
            float part[NB];
#pragma unroll
            for (int jj = 0; jj < NB; ++jj) {
                const int j = j0 + jj;
                const int ij = __shfl_sync(0xffffffffu, idx, j & 31);
                part[jj] = ld_cg_f32(base + (size_t)(j < n ? ij : 0) * D);
            }
            if (j0 == 0) {
                mx = lse;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float ms = (mx == -INFINITY) ? 0.f : mx;
                wgt = exp2f(lse - ms);
                denom = wgt;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
            }
#pragma unroll
            for (int jj = 0; jj < NB; ++jj) {
                const int j = j0 + jj;
                const float wj = (j < n) ? __shfl_sync(0xffffffffu, wgt, j & 31) : 0.f;
                acc = fmaf(wj, part[jj], acc);
            }
        }
        const float val = acc * (denom > 0.f ? 1.f / denom : 0.f);
        if (is_terminal) {
            const float hi = __shfl_down_sync(0xffffffffu, val, 1);
            if ((dim & 1) == 0)
                *reinterpret_cast<uint32_t*>(attn_out + (size_t)head * D + dim) = pack_bf16x2(val, hi);
        } else {
            attn_o[((size_t)head * p.max_partials + out_idx) * D + dim] = val;
            if (dim == 0)
                attn_lse[(size_t)head * p.max_partials + out_idx] =
                    denom > 0.f ? mx + log2f(denom) : -INFINITY;
        }
    }
    consumer_sync();  // every thread's stores precede the signal below
    if (warp == 0) {
        if (is_terminal) {
            if (lane == 0) red_release_gpu_add(bar_addr(p, layer, MKB_OP_ATTENTION_REDUCTION - 1, 0), 4);
        } else if (lane < 4) {
            red_release_gpu_add(bar_addr(p, layer, MKB_OP_PARTIAL_ATTENTION - 1, part_slot0 + h0 + lane), 1);
        }
    }
    return true;
}

// --------------------------------------------------------------------------- //
// consumers: tensor-parallel all-reduce of one chunk of the residual stream
// --------------------------------------------------------------------------- //
// Reduce-scatter and all-gather over peer memory with tagged stores only (protocol in
// MkbTensorParallel).  No thread ever waits without a budget: a rank that never arrives turns
// into MKB_ERR_DEVICE_TIMEOUT on the others.
constexpr int kTpBatch = 4;  // column slices loaded per round trip
__device__ __forceinline__ bool consumer_tp_all_reduce(const Ctx& c, ConsumerState& cs, const int* w) {
    const KParams& p = *c.p;
    const int tid = threadIdx.x;
    const int layer = __ldg(w + 1), which = __ldg(w + 2), chunk = __ldg(w + 3), nchunks = __ldg(w + 4);
    const int E = p.H / nchunks, e0 = chunk * E;
    const int owner = chunk % p.tp_size;
    const int slices = (which == 0 ? p.o_in : p.I) / p.R;
    const int row = (which == 0 ? MKB_OP_O_PROJ_RESIDUAL : MKB_OP_DOWN_PROJ_RESIDUAL) - 1;
    const int thr = which == 0 ? p.thr_upgate_waits_oproj : p.thr_qkv_waits_down;
    const uint32_t tag = tp_tag(c, layer, which);

    // 1. this rank's projection is complete: sum its column slices, send the sums to the owner
    if (!consumers_wait_counter(c, cs, layer, row, 0, thr, true)) return false;
    {
        uint4* dst = reinterpret_cast<uint4*>(p.tp_recv[owner]) + ((size_t)p.tp_rank * p.H + e0) / 2;
        for (int e = tid * 2; e < E; e += kConsumerThreads * 2) {
            float sx = 0.f, sy = 0.f;
            for (int s0 = 0; s0 < slices; s0 += kTpBatch) {  // all loads of a batch in flight at once
                uint2 v[kTpBatch];
#pragma unroll
                for (int k = 0; k < kTpBatch; ++k) {
                    v[k] = make_uint2(0u, 0u);
                    if (s0 + k < slices) v[k] = ldv_cg_v2(p.tp_partial + (size_t)(s0 + k) * p.H + e0 + e);
                }
#pragma unroll
                for (int k = 0; k < kTpBatch; ++k) {
                    sx += __uint_as_float(v[k].x);
                    sy += __uint_as_float(v[k].y);
                }
            }
            st_volatile_v4(dst + e / 2, __float_as_uint(sx), tag, __float_as_uint(sy), tag);
        }
    }
    if (tid == 0) rec(c, MKB_T_TP_SENT);
    if (owner != p.tp_rank) return true;

    // 2. owner: every thread polls the pairs it reduces until all ranks' tags are current, adds
    // them in rank order to the residual stream in fp32, rounds once and sends the new values
    // (tagged again) to every rank.  The old residual value is the previous all-reduce's result
    // in this rank's own tagged buffer, or the token embedding for the first one of a launch.
    const bool first = layer == 0 && which == 0;
    const uint32_t prev_tag = first ? 0u : (which == 1 ? tp_tag(c, layer, 0) : tp_tag(c, layer - 1, 1));
    const uint4* src = reinterpret_cast<const uint4*>(p.tp_recv[p.tp_rank]) + e0 / 2;
    const uint2* old = p.tp_hidden_ll[p.tp_rank] + e0 / 2;
    bool ok = true;
    TpPoll poll;
    for (int e = tid * 2; e < E && ok; e += kConsumerThreads * 2) {
        // old residual value: plain embedding for the first all-reduce of a launch, else the
        // previous all-reduce's tagged result
        uint2 h = make_uint2(0u, prev_tag);
        if (first) {
            h.x = ldv_cg_u32(p.hidden + e0 + e);
        } else {
            while (true) {
                h = ld_volatile_v2(old + e / 2);
                if (h.y == prev_tag) break;
                if (!poll.tick(c, layer, 300 + which, chunk, (int)h.y)) {
                    ok = false;
                    break;
                }
            }
        }
        // ranks in groups of four (keeps the registers of this rarely-run path few), in rank
        // order: the same sum whoever owns the chunk
        float sx = 0.f, sy = 0.f;
        for (int r0 = 0; r0 < p.tp_size && ok; r0 += 4) {
            uint4 v[4];
            while (true) {
                int late = -1;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[k] = make_uint4(0u, tag, 0u, tag);
                    if (r0 + k < p.tp_size) {
                        v[k] = ld_volatile_v4(src + ((size_t)(r0 + k) * p.H + e) / 2);
                        if (v[k].y != tag || v[k].w != tag) late = r0 + k;
                    }
                }
                if (late < 0) break;
                if (!poll.tick(c, layer, 200 + which, chunk, late)) {
                    ok = false;
                    break;
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                sx += __uint_as_float(v[k].x);
                sy += __uint_as_float(v[k].z);
            }
        }
        if (!ok) break;
        const uint32_t out = pack_bf16x2(bf16_lo(h.x) + sx, bf16_hi(h.x) + sy);
        for (int r = 0; r < p.tp_size; ++r) st_volatile_v2(p.tp_hidden_ll[r] + (e0 + e) / 2, out, tag);
    }
    if (tid == 0) rec(c, MKB_T_TP_ARRIVED);
    return consumer_all(ok);
}

// --------------------------------------------------------------------------- //
// consumer dispatch
// --------------------------------------------------------------------------- //
template <bool kTP>
__device__ bool consumer_rms_op(const Ctx& c, ConsumerState& cs, int op, const int* w) {
    const KParams& p = *c.p;
    switch (op) {
        case MKB_OP_RMS_QKV_ROPE_APPEND: {
            const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3);
            return consumer_rms_matvec<kTP>(c, cs, p.attn_ln_w + (size_t)layer * p.H, eb - sb, layer - 1,
                                       MKB_OP_DOWN_PROJ_RESIDUAL - 1, p.thr_qkv_waits_down, layer > 0,
                                       nullptr, layer, 0);
        }
        case MKB_OP_RMS_UPGATE_SILU: {
            const int layer = __ldg(w + 1), n = __ldg(w + 2);
            // down-proj adds to the residual accumulators this instruction reads: it waits
            // for one arrival per up/gate instruction on row MKB_BARRIER_ROW_RMS_READ
            return consumer_rms_matvec<kTP>(c, cs, p.mlp_ln_w + (size_t)layer * p.H, 2 * n, layer,
                                       MKB_OP_O_PROJ_RESIDUAL - 1, p.thr_upgate_waits_oproj, true,
                                       bar_addr(p, layer, MKB_BARRIER_ROW_RMS_READ, 0), layer, 1);
        }
        default: {  // MKB_OP_RMS_LM_HEAD
            const int sb = __ldg(w + 1), eb = __ldg(w + 2);
            return consumer_rms_matvec<kTP>(c, cs, p.lm_norm_w, eb - sb, p.L - 1,
                                       MKB_OP_DOWN_PROJ_RESIDUAL - 1, p.thr_qkv_waits_down, true,
                                       nullptr, p.L - 1, 2);
        }
    }
}

// RMS_NORM (batched build): normalise one sequence's residual stream once, for all SMs.
// words: [9, layer, which (0 attention norm, 1 MLP norm, 2 final norm), sequence]
__device__ bool consumer_rms_norm(const Ctx& c, ConsumerState& cs, const int* w) {
    const KParams& p = *c.p;
    const int layer = __ldg(w + 1), which = __ldg(w + 2), seq = __ldg(w + 3);
    const __nv_bfloat16* norm_w = which == 0 ? p.attn_ln_w + (size_t)layer * p.H
                                  : which == 1 ? p.mlp_ln_w + (size_t)layer * p.H
                                               : p.lm_norm_w;
    const bool needed = !(which == 0 && layer == 0);
    const int wait_layer = which == 0 ? layer - 1 : layer;
    const int wait_row = (which == 1 ? MKB_OP_O_PROJ_RESIDUAL : MKB_OP_DOWN_PROJ_RESIDUAL) - 1;
    const int thr = which == 1 ? p.thr_upgate_waits_oproj : p.thr_qkv_waits_down;
    const uint4 w0 = rms_weights_early(p.H, norm_w);
    if (!consumers_wait_counter(c, cs, wait_layer, wait_row, 0, thr, needed)) return false;
    rms_activation_from<kRmsAcc>(c, p.H, norm_w, w0, nullptr, seq);
    consumer_sync();  // every thread's part of the vector is written
    if (threadIdx.x == 0) red_release_gpu_add(bar_addr(p, layer, MKB_BARRIER_ROW_RMS_NORM, which), 1);
    return true;
}

__device__ bool consumer_residual_op(const Ctx& c, ConsumerState& cs, int op, const int* w) {
    const KParams& p = *c.p;
    const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3), rb = __ldg(w + 4);
    if (op == MKB_OP_O_PROJ_RESIDUAL)  // every sequence's attention must be complete
        return consumer_plain_matvec(c, cs, p.attn_out + (size_t)rb * p.R, eb - sb, layer,
                                     MKB_OP_ATTENTION_REDUCTION - 1, 0, p.thr_oproj_waits_attn * p.batch,
                                     nullptr, 0, (size_t)p.o_in);
    // with tensor parallelism inside the kernel the outputs go to a partial-sum buffer nobody
    // else is reading, so only the single-GPU residual needs the read-before-add ordering
    const bool order = p.thr_down_waits_rms > 0 && p.tp_size <= 1;
    return consumer_plain_matvec(c, cs, p.silu_out + (size_t)rb * p.R, eb - sb, layer,
                                 MKB_OP_RMS_UPGATE_SILU - 1, rb, p.thr_down_waits_upgate,
                                 order ? bar_addr(p, layer, MKB_BARRIER_ROW_RMS_READ, 0) : nullptr,
                                 p.thr_down_waits_rms, (size_t)p.I);
}


#if MKB_BATCH > 8
// --------------------------------------------------------------------------- //
// GEMM build: the projections on the 5th-generation tensor cores
// --------------------------------------------------------------------------- //
// out[sequence][row] = sum_k W[row][k] * X[sequence][k] for a block of 128 weight rows:
// A = the weight tile of a ring stage (128 rows x 128 columns, K-major, 128-byte swizzle, as the
// tiled TMA copy leaves it), B = the activation slice of the same columns ([sequences] x 128,
// K-major, same swizzle), D = 128 lanes x N fp32 columns in tensor memory (N = batch rounded up
// to 16).  One thread issues the MMAs; twelve warps read finished accumulators back and apply the
// epilogue; a second loader thread streams the activation slices once their producer is done.
struct GemmOp {
    int op, layer, nblocks, kc;   // blocks of this instruction (up/gate: 2 per listed block), input columns
    int first_block;              // range instructions
    const int* list;              // up/gate block list
    const CUtensorMap* xmap;      // activations
    int xchunk0;                  // first 64-column chunk of the input slice
    int wait_layer, wait_row, wait_slot, wait_thr;  // what the activations wait for
};
__device__ __forceinline__ bool gemm_decode(const KParams& p, const int* w, GemmOp& g) {
    g.op = __ldg(w);
    g.list = nullptr;
    g.xchunk0 = 0;
    switch (g.op) {
        case MKB_OP_RMS_QKV_ROPE_APPEND:
            g.layer = __ldg(w + 1); g.first_block = __ldg(w + 2); g.nblocks = __ldg(w + 3) - g.first_block;
            g.kc = p.H; g.xmap = &p.x_normed_map;
            g.wait_layer = g.layer; g.wait_row = MKB_BARRIER_ROW_RMS_NORM; g.wait_slot = 0; g.wait_thr = p.batch;
            return true;
        case MKB_OP_RMS_UPGATE_SILU:
            g.layer = __ldg(w + 1); g.nblocks = 2 * __ldg(w + 2); g.list = w + 3; g.first_block = 0;
            g.kc = p.H; g.xmap = &p.x_normed_map;
            g.wait_layer = g.layer; g.wait_row = MKB_BARRIER_ROW_RMS_NORM; g.wait_slot = 1; g.wait_thr = p.batch;
            return true;
        case MKB_OP_RMS_LM_HEAD:
            g.layer = p.L - 1; g.first_block = __ldg(w + 1); g.nblocks = __ldg(w + 2) - g.first_block;
            g.kc = p.H; g.xmap = &p.x_normed_map;
            g.wait_layer = p.L - 1; g.wait_row = MKB_BARRIER_ROW_RMS_NORM; g.wait_slot = 2; g.wait_thr = p.batch;
            return true;
        case MKB_OP_O_PROJ_RESIDUAL:
            g.layer = __ldg(w + 1); g.first_block = __ldg(w + 2); g.nblocks = __ldg(w + 3) - g.first_block;
            g.kc = p.R; g.xmap = &p.x_attn_map; g.xchunk0 = __ldg(w + 4) * (p.R / 64);
            g.wait_layer = g.layer; g.wait_row = MKB_OP_ATTENTION_REDUCTION - 1; g.wait_slot = 0;
            g.wait_thr = p.thr_oproj_waits_attn * p.batch;
            return true;
        case MKB_OP_DOWN_PROJ_RESIDUAL:
            g.layer = __ldg(w + 1); g.first_block = __ldg(w + 2); g.nblocks = __ldg(w + 3) - g.first_block;
            g.kc = p.R; g.xmap = &p.x_silu_map; g.xchunk0 = __ldg(w + 4) * (p.R / 64);
            g.wait_layer = g.layer; g.wait_row = MKB_OP_RMS_UPGATE_SILU - 1; g.wait_slot = __ldg(w + 4);
            g.wait_thr = p.thr_down_waits_upgate;
            return true;
        default:
            return false;
    }
}

__device__ __forceinline__ void tma_tile3_g2s(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                              uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

// Second loader thread: waits for the producer of every GEMM instruction's activations (the wait
// the consumers of the other builds perform), then streams the [N x 128] slices stage by stage.
__device__ void xloader_main(Ctx c) {
    const KParams& p = *c.p;
    const int* queue = p.instructions + (size_t)blockIdx.x * p.queue_len * MKB_INTS_PER_INSTRUCTION;
    c.role = kRoleLoader;
    const uint32_t xbytes = (uint32_t)p.gemm_n * kStageCols * 2u;
    uint32_t xstage = 0;
    bool alive = true;
    for (int i = 0; i < p.queue_len && alive; ++i) {
        GemmOp g;
        if (!gemm_decode(p, queue + i * MKB_INTS_PER_INSTRUCTION, g)) continue;
        c.instr = i;
        c.opcode = g.op;
        if (*c.cta_abort) break;
        c.cta_abort[4] = 1;  // the weight loader may look further ahead while this instruction waits
        const bool ok = wait_counter(c, bar_addr(p, g.wait_layer, g.wait_row, g.wait_slot), g.wait_thr,
                                     g.wait_layer, g.wait_row, g.wait_slot, (unsigned)p.poll_sleep_ns);
        c.cta_abort[4] = 0;
        if (!ok) break;
        rec(c, MKB_T_CONSUMER_WAIT_DONE);
        // the activations were written with ordinary stores by other SMs and are read here by
        // the TMA engine: order the two proxies after the acquiring poll
        asm volatile("fence.proxy.async.global;" ::: "memory");
        const int spb = stages_per_block(g.kc);
        for (int b = 0; b < g.nblocks && alive; ++b)
            for (int st = 0; st < spb; ++st) {
                const int slot = xstage % kXStages;
                const uint32_t parity = ((xstage / kXStages) & 1u) ^ 1u;
                if (!mbar_try_wait(c.xempty_bar(slot), parity) && !mbar_wait_slow(c, c.xempty_bar(slot), parity, true)) {
                    alive = false;
                    break;
                }
                mbar_expect_tx(c.xfull_bar(slot), xbytes);
                tma_tile3_g2s(c.xstage_addr(slot), g.xmap, 0, 0, g.xchunk0 + st * (kStageCols / 64), c.xfull_bar(slot));
                ++xstage;
            }
    }
    reinterpret_cast<volatile int*>(c.cta_abort)[5] = (int)xstage;  // for the exit path
}

// K-major operand tile with the 128-byte swizzle: rows 128 bytes apart, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 2, 384;" ::: "memory"); }  // warps 4..15
__device__ __forceinline__ bool gemm_wait(const Ctx& c, ConsumerState& cs, uint32_t bar, uint32_t parity) {
    if (!cs.dead && !mbar_try_wait(bar, parity)) {
        if (!mbar_wait_slow(c, bar, parity, true)) cs.dead = true;
    }
    return !cs.dead;
}

// One GEMM instruction.  Consumer warp 0 (one lane) issues the MMAs, warps 4..15 are the
// epilogue (tensor-memory lane quarter = warp % 4, thread = weight row; the three groups of four
// warps split the sequences), the others only keep their ring bookkeeping in step.
__device__ bool gemm_instruction(const Ctx& c, ConsumerState& cs, const int* w) {
    const KParams& p = *c.p;
    GemmOp g;
    gemm_decode(p, w, g);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int spb = stages_per_block(g.kc);
    const uint32_t n = (uint32_t)p.gemm_n;
    const uint32_t tmem = c.tmem_base();

    if (warp == 0 && lane == 0) {
        // fp32 accumulate, bf16 x bf16, both operands K-major, N = n, M = 128
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kBlockRows >> 4) << 24);
        uint32_t slot = cs.slot, phase = cs.phase, xstage = cs.xstage, acc = cs.acc;
        for (int b = 0; b < g.nblocks; ++b) {
            const uint32_t buf = acc & 1u, use = acc >> 1;
            gemm_wait(c, cs, c.acc_empty_bar(buf), (use & 1u) ^ 1u);  // the epilogue has drained this accumulator
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int st = 0; st < spb; ++st) {
                const uint32_t xslot = xstage % kXStages;
                gemm_wait(c, cs, c.full_bar(slot), phase);
                gemm_wait(c, cs, c.xfull_bar(xslot), (xstage / kXStages) & 1u);
                if (b == 0 && st == 0) rec(c, MKB_T_CONSUMER_FIRST_STAGE);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t wb = c.stage_addr(slot), xb = c.xstage_addr(xslot);
                if (!cs.dead) {
#pragma unroll
                    for (int ch = 0; ch < kStageCols / 64; ++ch)  // one swizzle atom (64 columns) at a time
#pragma unroll
                        for (int k = 0; k < 4; ++k)                // four K = 16 steps inside the 128-byte rows
                            umma_f16(tmem + buf * kBatch, umma_smem_desc(wb + ch * (kBlockRows * 128) + k * 32),
                                     umma_smem_desc(xb + ch * (n * 128) + k * 32), idesc, (uint32_t)((st | ch | k) != 0));
                }
                umma_commit(c.empty_bar(slot));    // both stages are free once these MMAs have read them
                umma_commit(c.xempty_bar(xslot));
                if (++slot == kNumStages) { slot = 0; phase ^= 1u; }
                ++xstage;
            }
            umma_commit(c.acc_full_bar(buf));
            ++acc;
        }
        rec(c, MKB_T_ATTN_STAGES_DONE);  // (GEMM instructions: every MMA of the instruction is issued)
    } else if (warp >= 4) {
        // Twelve epilogue warps: warp w reads the lane quarter w % 4 of tensor memory (its rows), and
        // the three groups of four warps share the sequences (accumulator columns) of every block.
        const int q = warp & 3, r = q * 32 + lane;  // this thread's row inside the block
        const uint32_t cols_per_group = ((n / 8 + 2) / 3) * 8;
        const uint32_t c_lo = min(n, (uint32_t)((warp - 4) >> 2) * cols_per_group), c_hi = min(n, c_lo + cols_per_group);
        uint32_t acc = cs.acc;
        const bool pair = g.op == MKB_OP_RMS_UPGATE_SILU;
        for (int b = 0; b < g.nblocks; b += pair ? 2 : 1) {
            const int blk = g.list ? __ldg(g.list + (b >> 1)) : g.first_block + b;
            const uint32_t buf = acc & 1u, use = acc >> 1;
            gemm_wait(c, cs, c.acc_full_bar(buf), use & 1u);
            const uint32_t buf2 = (acc + 1) & 1u, use2 = (acc + 1) >> 1;
            if (pair) gemm_wait(c, cs, c.acc_full_bar(buf2), use2 & 1u);
            cs.dead = __any_sync(0xffffffffu, cs.dead);  // the lanes shuffle below: leave together
            if (b == 0 && tid == 4 * 32) rec(c, MKB_T_RMS_LOADED);  // (GEMM instructions: first accumulator complete)
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
            const int grow = blk * kBlockRows + r;  // row of the projection's output
            for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 8) {
                float v[8], v2[8];
                tmem_ld8(lane_addr + buf * kBatch + c0, v);
                if (pair) tmem_ld8(lane_addr + buf2 * kBatch + c0, v2);
                if (cs.dead) continue;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int s = (int)c0 + j;  // sequence
                    const bool live = s < p.batch;
                    switch (g.op) {
                        case MKB_OP_RMS_QKV_ROPE_APPEND: {
                            float x = bf16_round(v[j]);
                            const int k_start = p.Hq * p.D, v_start = (p.Hq + p.Hkv) * p.D;
                            const int start = blk * kBlockRows;
                            const int ps = live ? c.pos_of(s) : 0;
                            if (start < v_start) {  // head_dim == 128 == block: the block is one head
                                const float cs_ = __ldg(p.rope_cos + (size_t)ps * p.D + r);
                                const float sn = __ldg(p.rope_sin + (size_t)ps * p.D + r);
                                const float other = __shfl_xor_sync(0xffffffffu, x, 1);
                                x = x * cs_ + ((r & 1) ? other : -other) * sn;
                            }
                            if (live) {
                                __nv_bfloat16* dst;
                                if (start < k_start) {
                                    dst = p.q_rope + (size_t)s * p.o_in + start;
                                } else {
                                    const size_t tok = (((size_t)g.layer * p.B + s) * p.T + ps) * p.Hkv * p.D;
                                    dst = (start < v_start) ? p.k_cache + tok + (start - k_start)
                                                            : p.v_cache + tok + (start - v_start);
                                }
                                dst[r] = __float2bfloat16_rn(x);
                            }
                        } break;
                        case MKB_OP_O_PROJ_RESIDUAL:
                        case MKB_OP_DOWN_PROJ_RESIDUAL:
                            if (live)
                                red_add_u64(p.residual_acc + (size_t)s * p.H + grow,
                                            (unsigned long long)(__float2ll_rn(v[j] * kResidualScale) * p.residual_mult));
                            break;
                        case MKB_OP_RMS_UPGATE_SILU: {
                            const float up = bf16_round(v[j]), gate = bf16_round(v2[j]);
                            const float x = bf16_round(gate / (1.f + __expf(-gate))) * up;
                            if (live) p.silu_out[(size_t)s * p.I + grow] = __float2bfloat16_rn(x);
                        } break;
                        default:  // MKB_OP_RMS_LM_HEAD
                            if (live) p.logits[(size_t)s * p.V + grow] = __float2bfloat16_rn(v[j]);
                            break;
                    }
                }
            }
            // hand the accumulator(s) back, then publish what this block wrote
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(c.acc_empty_bar(buf));
                if (pair) mbar_arrive(c.acc_empty_bar(buf2));
            }
            acc += pair ? 2 : 1;
            if (g.op == MKB_OP_RMS_QKV_ROPE_APPEND || pair) {
                epilogue_sync();  // all epilogue warps' global writes of this block precede the signal
                if (tid == 4 * 32 && !cs.dead) {
                    const int slot = pair ? blk * kBlockRows / p.R : blk * kBlockRows / p.D;
                    red_release_gpu_add(bar_addr(p, g.layer, g.op - 1, slot), 1);
                }
            }
        }
        if (tid == 4 * 32) rec(c, MKB_T_RMS_SUMMED);  // (GEMM instructions: last epilogue done)
        if (g.op == MKB_OP_O_PROJ_RESIDUAL || g.op == MKB_OP_DOWN_PROJ_RESIDUAL) {
            epilogue_sync();
            if (tid == 4 * 32 && !cs.dead) red_release_gpu_add(bar_addr(p, g.layer, g.op - 1, 0), g.nblocks);
        }
    }
    // everybody's view of the rings moves past this instruction
    const uint32_t stages = (uint32_t)(g.nblocks * spb);
    const uint32_t total = cs.slot + stages;
    cs.phase ^= (total / kNumStages) & 1u;
    cs.slot = total % kNumStages;
    cs.xstage += stages;
    cs.acc += (uint32_t)g.nblocks;
    volatile int* verdict = verdict_word(c, cs);
    if (cs.dead) *c.cta_abort = 1;
    consumer_sync();
    if (tid == 0) *verdict = *c.cta_abort ? 0 : 1;
    consumer_sync();
    return *verdict != 0;
}
#endif  // MKB_BATCH > 8

template <bool kTP>
__device__ void consumer_main(Ctx c) {
    const KParams& p = *c.p;
    ConsumerState cs;
    const int* queue = p.instructions + (size_t)blockIdx.x * p.queue_len * MKB_INTS_PER_INSTRUCTION;
    c.role = kRoleConsumer;
    for (int i = 0; i < p.queue_len; ++i) {
        const int* w = queue + i * MKB_INTS_PER_INSTRUCTION;
        const int op = __ldg(w);
        c.instr = i;
        c.opcode = op;
        bool ok = true;
        if (threadIdx.x == 0 && op != MKB_OP_NOOP) {
            rec(c, MKB_T_CONSUMER_START);
            if (p.timings != nullptr) {  // where rms_activation_body stamps its phases
                int* trow = p.timings + ((size_t)blockIdx.x * p.queue_len + i) * MKB_TIMING_SLOTS;
                asm volatile("st.shared.u64 [%0], %1;" ::"r"(c.base + kSmemHot + 24), "l"(trow) : "memory");
            }
        }
        switch (op) {
            case MKB_OP_NOOP:
                break;
#if MKB_BATCH > 8
            case MKB_OP_RMS_QKV_ROPE_APPEND:
            case MKB_OP_RMS_UPGATE_SILU:
            case MKB_OP_RMS_LM_HEAD:
            case MKB_OP_O_PROJ_RESIDUAL:
            case MKB_OP_DOWN_PROJ_RESIDUAL:
                ok = gemm_instruction(c, cs, w);
                break;
#else
            case MKB_OP_RMS_QKV_ROPE_APPEND:
            case MKB_OP_RMS_UPGATE_SILU:
            case MKB_OP_RMS_LM_HEAD:
                ok = consumer_rms_op<kTP>(c, cs, op, w);
                break;
            case MKB_OP_O_PROJ_RESIDUAL:
            case MKB_OP_DOWN_PROJ_RESIDUAL:
                ok = consumer_residual_op(c, cs, op, w);
                break;
#endif
            case MKB_OP_PARTIAL_ATTENTION: {
                const int gqa = p.Hq / p.Hkv;
                if (p.D == 64) ok = consumer_attention<64, 4>(c, cs, w);
                else if (gqa == 4) ok = consumer_attention<128, 4>(c, cs, w);
                else ok = consumer_attention<128, 8>(c, cs, w);
            } break;
            case MKB_OP_ATTENTION_REDUCTION:
                if (p.D == 64) ok = consumer_attn_reduction<64>(c, cs, w);
                else ok = consumer_attn_reduction<128>(c, cs, w);
                break;
            case MKB_OP_RMS_NORM:
                if constexpr (kBatch > 1) {
                    ok = consumer_rms_norm(c, cs, w);
                    break;
                } else {
                    if (threadIdx.x == 0) report_error(c, MKB_ERR_BAD_OPCODE, op, 0, 0, 0);
                    ok = false;
                    break;
                }
            case MKB_OP_TP_ALL_REDUCE:
                if (kTP && p.tp_size > 1) {
                    ok = consumer_tp_all_reduce(c, cs, w);
                    break;
                }
                [[fallthrough]];
            default:
                if (threadIdx.x == 0) report_error(c, MKB_ERR_BAD_OPCODE, op, 0, 0, 0);
                ok = false;
                break;
        }
        if (threadIdx.x == 0 && op != MKB_OP_NOOP) rec(c, MKB_T_CONSUMER_DONE);
        if (!ok) break;  // `ok` is uniform over the 512 consumer threads
    }
}

// --------------------------------------------------------------------------- //
// storer
// --------------------------------------------------------------------------- //
struct StorerState {
    uint32_t oslot = 0, ophase = 0;
    bool dead = false;
    // barrier arrivals not yet signalled: entry k lives in lane k
    int* my_addr = nullptr;
    int my_count = 0;
    int n_entries = 0;
    // running argmax of the logits this lane has stored (bf16-rounded value, vocabulary index)
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;
};

// (value, index) ordering of torch.argmax: larger value wins, then the smaller index
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// End of the storer's queue: publish this CTA's best logit; the CTA that arrives last merges
// all of them, writes the token id and re-arms the arrival counter for the next launch.
__device__ __noinline__ void storer_finish_argmax(const Ctx& c, StorerState& ss, int lane) {
    const KParams& p = *c.p;
    float v = ss.best_val;
    int i = ss.best_idx;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
        argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
    int* slots = p.argmax_scratch + 2;
    int old = 0;
    if (lane == 0) {
        slots[2 * blockIdx.x] = __float_as_int(v);
        slots[2 * blockIdx.x + 1] = i;
        __threadfence();
        old = atomicAdd(p.argmax_scratch, 1);
    }
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != (int)gridDim.x - 1) return;
    __threadfence();
    v = -INFINITY;
    i = 0x7fffffff;
    for (int k = lane; k < (int)gridDim.x; k += 32)
        argmax_merge(v, i, __int_as_float((int)ld_cg_u32(slots + 2 * k)), (int)ld_cg_u32(slots + 2 * k + 1));
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1)
        argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
    if (lane == 0) {
        *p.argmax_out = i;
        *p.argmax_scratch = 0;
    }
}

// sum the per-warp partials of the next finished block; lane r < 16 gets row r
__device__ __forceinline__ float storer_take_block(const Ctx& c, StorerState& ss, int lane,
                                                   int partials) {
    const int oslot = ss.oslot;
    const uint32_t obar = c.out_full_bar(oslot);
    if (!ss.dead && !mbar_try_wait(obar, ss.ophase)) {
        if (!mbar_wait_slow(c, obar, ss.ophase, true)) ss.dead = true;
    }
    // lane = row + 16 * half: each half sums every other partial
    const int row = lane & 15, half = lane >> 4;
    const uint32_t src = c.base + kSmemOut + (oslot * kOutSlotFloats + row * 16) * 4;
    float v = 0.f;
    for (int k = half; k < partials; k += 2) v += __uint_as_float(lds_u32(src + k * 4));
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    __syncwarp();
    if (lane == 0) mbar_arrive(c.out_empty_bar(oslot));
    if (++ss.oslot == kOutSlots) {
        ss.oslot = 0;
        ss.ophase ^= 1u;
    }
    return v;
}

// Publish every pending arrival with ONE warp-wide `red.release.gpu`: the
// release orders all global writes this warp made before the __syncwarp, so a
// whole instruction's signals cost a single fence.
__device__ __forceinline__ void storer_flush(StorerState& ss, int lane) {
    __syncwarp();
    if (lane < ss.n_entries && ss.my_count > 0) red_release_gpu_add(ss.my_addr, ss.my_count);
    ss.my_count = 0;
    ss.my_addr = nullptr;
    ss.n_entries = 0;
}
__device__ __forceinline__ void storer_signal(StorerState& ss, int lane, int* addr, int count) {
    const unsigned hit = __ballot_sync(0xffffffffu, lane < ss.n_entries && ss.my_addr == addr);
    if (hit) {
        if (lane == __ffs(hit) - 1) ss.my_count += count;
        return;
    }
    if (ss.n_entries == 32) storer_flush(ss, lane);
    if (lane == ss.n_entries) {
        ss.my_addr = addr;
        ss.my_count = count;
    }
    ss.n_entries++;
}

#if MKB_BATCH > 8
// ---- GEMM build: the epilogue warps write the outputs themselves; this warp's first lane is
// the activation loader (a warp of its own, so that it never time-slices with the weight loader)
template <bool kTP>
__device__ void storer_main(Ctx c) {
    if ((threadIdx.x & 31) == 0) xloader_main(c);
}
#elif MKB_BATCH > 1
// ---- batched build: every block carries 16 rows x up to 8 sequences -------------------- //
// Lane = row + 16 * half; the lane owns sequences 4 * half .. 4 * half + 3 of its row.
constexpr int kSeqPerLane = kBatch / 2;
__device__ __forceinline__ void storer_take_block_batched(const Ctx& c, StorerState& ss, int lane,
                                                          float (&v)[kSeqPerLane]) {
    const int oslot = ss.oslot;
    const uint32_t obar = c.out_full_bar(oslot);
    if (!ss.dead && !mbar_try_wait(obar, ss.ophase)) {
        if (!mbar_wait_slow(c, obar, ss.ophase, true)) ss.dead = true;
    }
    const int row = lane & 15, half = lane >> 4;
#pragma unroll
    for (int j = 0; j < kSeqPerLane; ++j) {
        const uint32_t src = c.base + kSmemOut + (oslot * kOutSlotFloats + (row * kBatch + half * kSeqPerLane + j) * 16) * 4;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // the 16 per-warp partials of this (row, sequence)
            const uint4 q = lds_v4(src + k * 16);
            acc += (__uint_as_float(q.x) + __uint_as_float(q.y)) + (__uint_as_float(q.z) + __uint_as_float(q.w));
        }
        v[j] = acc;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(c.out_empty_bar(oslot));
    if (++ss.oslot == kOutSlots) {
        ss.oslot = 0;
        ss.ophase ^= 1u;
    }
}

struct BatchedArgmax {
    float val[kSeqPerLane];
    int idx[kSeqPerLane];
};

// Per-sequence version of storer_finish_argmax: scratch = [arrivals, pad, {value, index} x CTA x sequence]
__device__ __noinline__ void storer_finish_argmax_batched(const Ctx& c, BatchedArgmax& best, int lane) {
    const KParams& p = *c.p;
    const int half = lane >> 4;
    int* slots = p.argmax_scratch + 2;
#pragma unroll
    for (int j = 0; j < kSeqPerLane; ++j) {
        float v = best.val[j];
        int i = best.idx[j];
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1)  // within the 16 lanes that own this sequence
            argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
        if ((lane & 15) == 0) {
            const int s = half * kSeqPerLane + j;
            slots[2 * (s * gridDim.x + blockIdx.x)] = __float_as_int(v);
            slots[2 * (s * gridDim.x + blockIdx.x) + 1] = i;
        }
    }
    __syncwarp();
    int old = 0;
    if (lane == 0) {
        __threadfence();
        old = atomicAdd(p.argmax_scratch, 1);
    }
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != (int)gridDim.x - 1) return;
    __threadfence();
    for (int s = 0; s < p.batch; ++s) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int k = lane; k < (int)gridDim.x; k += 32)
            argmax_merge(v, i, __int_as_float((int)ld_cg_u32(slots + 2 * (s * gridDim.x + k))),
                         (int)ld_cg_u32(slots + 2 * (s * gridDim.x + k) + 1));
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1)
            argmax_merge(v, i, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, i, o));
        if (lane == 0) p.argmax_out[s] = i;
    }
    if (lane == 0) *p.argmax_scratch = 0;
}

template <bool kTP>
__device__ void storer_main(Ctx c) {
    const KParams& p = *c.p;
    StorerState ss;
    BatchedArgmax best;
    const int lane = threadIdx.x & 31;
    const int row = lane & 15, half = lane >> 4;
    const int* queue = p.instructions + (size_t)blockIdx.x * p.queue_len * MKB_INTS_PER_INSTRUCTION;
    c.role = kRoleStorer;
#pragma unroll
    for (int j = 0; j < kSeqPerLane; ++j) {
        best.val[j] = -INFINITY;
        best.idx[j] = 0x7fffffff;
    }
    // RoPE rows at every sequence's position: [sequence][cos 128 | sin 128]
    float* rope = reinterpret_cast<float*>(__cvta_shared_to_generic(c.base + kSmemRope));
    for (int s = 0; s < p.batch; ++s)
        for (int d = lane; d < p.D; d += 32) {
            rope[s * 256 + d] = __ldg(p.rope_cos + (size_t)c.pos_of(s) * p.D + d);
            rope[s * 256 + 128 + d] = __ldg(p.rope_sin + (size_t)c.pos_of(s) * p.D + d);
        }
    __syncwarp();
    const int k_start = p.Hq * p.D, v_start = (p.Hq + p.Hkv) * p.D;
    const bool even = (row & 1) == 0;

    for (int i = 0; i < p.queue_len; ++i) {
        const int* w = queue + i * MKB_INTS_PER_INSTRUCTION;
        const int op = __ldg(w);
        c.instr = i;
        c.opcode = op;
        const int stop = (*c.cta_abort != 0) || ss.dead;
        if (__any_sync(0xffffffffu, stop)) break;
        if (lane == 0 && op != MKB_OP_NOOP) rec(c, MKB_T_STORER_START);
        float v[kSeqPerLane];
        switch (op) {
            case MKB_OP_RMS_QKV_ROPE_APPEND: {
                const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3);
                for (int b = sb; b < eb; ++b) {
                    storer_take_block_batched(c, ss, lane, v);
                    const int start = b * kBlockRows;
                    const int seg = start % p.D;
#pragma unroll
                    for (int j = 0; j < kSeqPerLane; ++j) {
                        const int s = half * kSeqPerLane + j;
                        float x = bf16_round(v[j]);
                        if (start < v_start) {
                            const float cs_ = rope[s * 256 + seg + row];
                            const float sn = rope[s * 256 + 128 + seg + row];
                            const float other = __shfl_xor_sync(0xffffffffu, x, 1);
                            x = x * cs_ + ((row & 1) ? other : -other) * sn;
                        }
                        const float hi = __shfl_down_sync(0xffffffffu, x, 1);
                        __nv_bfloat16* dst;
                        if (start < k_start) {
                            dst = p.q_rope + (size_t)s * p.o_in + start;
                        } else {
                            const size_t tok = (((size_t)layer * p.B + s) * p.T + c.pos_of(s)) * p.Hkv * p.D;
                            dst = (start < v_start) ? p.k_cache + tok + (start - k_start)
                                                    : p.v_cache + tok + (start - v_start);
                        }
                        if (even && s < p.batch) *reinterpret_cast<uint32_t*>(dst + row) = pack_bf16x2(x, hi);
                    }
                    storer_signal(ss, lane, bar_addr(p, layer, op - 1, start / p.D), 1);
                }
                storer_flush(ss, lane);
            } break;
            case MKB_OP_O_PROJ_RESIDUAL:
            case MKB_OP_DOWN_PROJ_RESIDUAL: {
                const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3);
                for (int b = sb; b < eb; ++b) {
                    storer_take_block_batched(c, ss, lane, v);
#pragma unroll
                    for (int j = 0; j < kSeqPerLane; ++j) {
                        const int s = half * kSeqPerLane + j;
                        if (s < p.batch)
                            red_add_u64(p.residual_acc + (size_t)s * p.H + b * kBlockRows + row,
                                        (unsigned long long)(__float2ll_rn(v[j] * kResidualScale) * p.residual_mult));
                    }
                }
                storer_signal(ss, lane, bar_addr(p, layer, op - 1, 0), eb - sb);
                storer_flush(ss, lane);
            } break;
            case MKB_OP_RMS_UPGATE_SILU: {
                const int layer = __ldg(w + 1), n = __ldg(w + 2);
                for (int jb = 0; jb < n; ++jb) {
                    const int b = __ldg(w + 3 + jb);
                    float g[kSeqPerLane];
                    storer_take_block_batched(c, ss, lane, v);
                    storer_take_block_batched(c, ss, lane, g);
#pragma unroll
                    for (int j = 0; j < kSeqPerLane; ++j) {
                        const int s = half * kSeqPerLane + j;
                        const float up = bf16_round(v[j]), gate = bf16_round(g[j]);
                        const float x = bf16_round(gate / (1.f + __expf(-gate))) * up;
                        const float hi = __shfl_down_sync(0xffffffffu, x, 1);
                        if (even && s < p.batch)
                            *reinterpret_cast<uint32_t*>(p.silu_out + (size_t)s * p.I + b * kBlockRows + row) = pack_bf16x2(x, hi);
                    }
                    storer_signal(ss, lane, bar_addr(p, layer, op - 1, b * kBlockRows / p.R), 1);
                }
                storer_flush(ss, lane);
            } break;
            case MKB_OP_RMS_LM_HEAD: {
                const int sb = __ldg(w + 1), eb = __ldg(w + 2);
                for (int b = sb; b < eb; ++b) {
                    storer_take_block_batched(c, ss, lane, v);
#pragma unroll
                    for (int j = 0; j < kSeqPerLane; ++j) {
                        const int s = half * kSeqPerLane + j;
                        const float hi = __shfl_down_sync(0xffffffffu, v[j], 1);
                        if (even && s < p.batch)
                            *reinterpret_cast<uint32_t*>(p.logits + (size_t)s * p.V + b * kBlockRows + row) = pack_bf16x2(v[j], hi);
                        argmax_merge(best.val[j], best.idx[j], bf16_round(v[j]), b * kBlockRows + row);
                    }
                }
            } break;
            default:
                break;
        }
        if (lane == 0 && op != MKB_OP_NOOP) rec(c, MKB_T_STORER_DONE);
    }
    if (p.argmax_out != nullptr) storer_finish_argmax_batched(c, best, lane);
}
#else
template <bool kTP>
__device__ void storer_main(Ctx c) {
    const KParams& p = *c.p;
    StorerState ss;
    const int lane = threadIdx.x & 31;
    const int row = lane & 15;
    const int* queue = p.instructions + (size_t)blockIdx.x * p.queue_len * MKB_INTS_PER_INSTRUCTION;
    c.role = kRoleStorer;
    const int kh_partials = kConsumerWarps, kr_partials = kConsumerWarps;  // one partial per warp
    // this token's RoPE row is only read by this warp: fetch it once, off the critical path
    for (int d = lane; d < p.D; d += 32) {
        float* rope = reinterpret_cast<float*>(__cvta_shared_to_generic(c.base + kSmemRope));
        rope[d] = __ldg(p.rope_cos + (size_t)c.pos * p.D + d);
        rope[128 + d] = __ldg(p.rope_sin + (size_t)c.pos * p.D + d);
    }
    __syncwarp();
    const int k_start = p.Hq * p.D, v_start = (p.Hq + p.Hkv) * p.D;

    for (int i = 0; i < p.queue_len; ++i) {
        const int* w = queue + i * MKB_INTS_PER_INSTRUCTION;
        const int op = __ldg(w);
        c.instr = i;
        c.opcode = op;
        const int stop = (*c.cta_abort != 0) || ss.dead;
        if (__any_sync(0xffffffffu, stop)) break;
        if (lane == 0 && op != MKB_OP_NOOP) rec(c, MKB_T_STORER_START);
        switch (op) {
            case MKB_OP_RMS_QKV_ROPE_APPEND: {
                const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3);
                for (int b = sb; b < eb; ++b) {
                    float v = bf16_round(storer_take_block(c, ss, lane, kh_partials));
                    const int start = b * kBlockRows;
                    if (start < v_start) {
                        const int seg = start % p.D;
                        const float cs_ = __uint_as_float(lds_u32(c.base + kSmemRope + (seg + row) * 4));
                        const float sn = __uint_as_float(lds_u32(c.base + kSmemRope + (128 + seg + row) * 4));
                        const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                        const float rot = (row & 1) ? other : -other;
                        v = v * cs_ + rot * sn;
                    }
                    const float hi = __shfl_down_sync(0xffffffffu, v, 1);
                    __nv_bfloat16* dst;
                    if (start < k_start) {
                        dst = p.q_rope + start;
                    } else {
                        const size_t tok = (((size_t)layer * p.B) * p.T + c.pos) * p.Hkv * p.D;
                        dst = (start < v_start) ? p.k_cache + tok + (start - k_start)
                                                : p.v_cache + tok + (start - v_start);
                    }
                    if (lane < 16 && (lane & 1) == 0)
                        *reinterpret_cast<uint32_t*>(dst + row) = pack_bf16x2(v, hi);
                    storer_signal(ss, lane, bar_addr(p, layer, op - 1, start / p.D), 1);
                }
                storer_flush(ss, lane);
            } break;
            case MKB_OP_O_PROJ_RESIDUAL:
            case MKB_OP_DOWN_PROJ_RESIDUAL: {
                const int layer = __ldg(w + 1), sb = __ldg(w + 2), eb = __ldg(w + 3);
                if (kTP && p.tp_size > 1) {
                    // in-kernel tensor parallelism: the fp32 block sums of this column slice
                    // go to the rank's partial buffer; MKB_OP_TP_ALL_REDUCE adds them up
                    float* part = p.tp_partial + (size_t)__ldg(w + 4) * p.H;
                    for (int b = sb; b < eb; ++b) {
                        const float v = storer_take_block(c, ss, lane, kr_partials);
                        if (lane < 16) part[b * kBlockRows + row] = v;
                    }
                } else {
                    for (int b = sb; b < eb; ++b) {
                        // Integer addition is associative: whatever order the column slices of
                        // the SMs arrive in, the accumulator ends up with the same bits.
                        // residual_mult is the tensor-parallel degree when the host averages the
                        // ranks' accumulators between launches (sum of the partials after the
                        // exact division), else 1.
                        const float v = storer_take_block(c, ss, lane, kr_partials);
                        if (lane < 16)
                            red_add_u64(p.residual_acc + b * kBlockRows + row,
                                        (unsigned long long)(__float2ll_rn(v * kResidualScale) * p.residual_mult));
                    }
                }
                storer_signal(ss, lane, bar_addr(p, layer, op - 1, 0), eb - sb);
                storer_flush(ss, lane);
            } break;
            case MKB_OP_RMS_UPGATE_SILU: {
                const int layer = __ldg(w + 1), n = __ldg(w + 2);
                for (int j = 0; j < n; ++j) {
                    const int b = __ldg(w + 3 + j);
                    const float up = bf16_round(storer_take_block(c, ss, lane, kh_partials));
                    const float gate = bf16_round(storer_take_block(c, ss, lane, kh_partials));
                    const float act = bf16_round(gate / (1.f + __expf(-gate)));
                    const float v = act * up;
                    const float hi = __shfl_down_sync(0xffffffffu, v, 1);
                    if (lane < 16 && (lane & 1) == 0)
                        *reinterpret_cast<uint32_t*>(p.silu_out + b * kBlockRows + row) = pack_bf16x2(v, hi);
                    storer_signal(ss, lane, bar_addr(p, layer, op - 1, b * kBlockRows / p.R), 1);
                }
                storer_flush(ss, lane);
            } break;
            case MKB_OP_RMS_LM_HEAD: {
                const int sb = __ldg(w + 1), eb = __ldg(w + 2);
                for (int b = sb; b < eb; ++b) {
                    const float v = storer_take_block(c, ss, lane, kh_partials);
                    const float hi = __shfl_down_sync(0xffffffffu, v, 1);
                    if (lane < 16 && (lane & 1) == 0)
                        *reinterpret_cast<uint32_t*>(p.logits + b * kBlockRows + row) = pack_bf16x2(v, hi);
                    if (lane < 16) argmax_merge(ss.best_val, ss.best_idx, bf16_round(v), b * kBlockRows + row);
                }
            } break;
            default:
                break;
        }
        if (lane == 0 && op != MKB_OP_NOOP) rec(c, MKB_T_STORER_DONE);
    }
    if (p.argmax_out != nullptr) storer_finish_argmax(c, ss, lane);
}
#endif  // MKB_BATCH

// --------------------------------------------------------------------------- //
// kernel
// --------------------------------------------------------------------------- //
template <bool kTP>
__device__ __forceinline__ void megakernel_body(const KParams& p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - raw);

    Ctx c;
    c.p = &p;
    c.base = base;
    c.cta_abort = reinterpret_cast<volatile int*>(gbase + kSmemCtl);
    c.instr = -1;
    c.opcode = -1;
    c.role = -1;
    if constexpr (kBatch == 1) c.pos = p.pos_id_ptr ? __ldg(p.pos_id_ptr) : p.pos_id;
    else c.pos = p.pos_id_ptr ? __ldg(p.pos_id_ptr) : p.pos_ids[0];

    if (threadIdx.x == 0) {
        for (int s = 0; s < kNumStages; ++s) {
            mbar_init(c.full_bar(s), 1);
            mbar_init(c.empty_bar(s), kGemm ? 1 : kConsumerWarps);
        }
        if constexpr (kGemm) {
            for (int s = 0; s < kXStages; ++s) {
                mbar_init(c.xfull_bar(s), 1);
                mbar_init(c.xempty_bar(s), 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(c.acc_full_bar(b), 1);
                mbar_init(c.acc_empty_bar(b), 12);  // one arrival per epilogue warp (warps 4..15)
            }
        }
        for (int s = 0; s < kOutSlots; ++s) {
            mbar_init(c.out_full_bar(s), kConsumerWarps);
            mbar_init(c.out_empty_bar(s), 1);
        }
        for (int k = 0; k < 8; ++k) c.cta_abort[k] = 0;
        HotConsts* hot = reinterpret_cast<HotConsts*>(gbase + kSmemHot);
        hot->hidden = p.hidden;
        hot->acc = p.residual_acc;
        hot->normed = p.normed;
        hot->trow = nullptr;
        hot->H = p.H;
        hot->inv_H = 1.f / (float)p.H;
        hot->eps = p.rms_eps;
        hot->ll = reinterpret_cast<const uint4*>(p.tp_size > 1 ? p.tp_hidden_ll[p.tp_rank] : nullptr);
        for (int k = 0; k < 2; ++k) reinterpret_cast<int*>(gbase + kSmemHot + 56)[k] = 0;  // loaders' issued counts
        if constexpr (kBatch > 1)
            for (int s = 0; s < kBatch; ++s)
                c.cta_abort[8 + s] = s >= p.batch ? 0 : p.pos_id_ptr ? __ldg(p.pos_id_ptr + s) : p.pos_ids[s & 7];
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if constexpr (kBatch == 1) {
        if (c.pos < 0 || c.pos >= p.T) {  // uniform over the grid: every thread read the same word
            if (threadIdx.x == 0) report_error(c, MKB_ERR_INVALID_ARGUMENT, c.pos, p.T, 0, 0);
            return;
        }
    } else {
        for (int s = 0; s < p.batch; ++s) {
            const int ps = c.pos_of(s);
            if (ps < 0 || ps >= p.T) {  // uniform over the grid as well
                if (threadIdx.x == 0) report_error(c, MKB_ERR_INVALID_ARGUMENT, ps, p.T, s, 0);
                return;
            }
        }
    }

    const int warp = threadIdx.x >> 5;
#if MKB_BATCH > 8
    // tensor memory for the two accumulators: allocated and freed by warp 0, address through shared memory
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c.base + kSmemCtl + 6 * 4),
                     "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#endif
    if (warp < kConsumerWarps) {
        consumer_main<kTP>(c);
    } else if (warp == kStorerWarp) {
        storer_main<kTP>(c);
    } else {
        if ((threadIdx.x & 31) == 0) loader_main(c, loader_index(warp));
    }
#if MKB_BATCH > 8
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
#endif
    __syncthreads();
#if MKB_BATCH > 8
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(c.tmem_base()), "r"((uint32_t)kTmemCols)
                     : "memory");
    // activation slices still in flight (only after an abort: every issued slice is otherwise consumed)
    if (warp == kStorerWarp && (threadIdx.x & 31) == 0) {
        const uint32_t issued = (uint32_t)c.cta_abort[5];
        const uint32_t first = issued > (uint32_t)kXStages ? issued - kXStages : 0u;
        c.role = kRoleLoader;
        for (uint32_t s = first; s < issued; ++s) {
            const uint32_t bar = c.xfull_bar(s % kXStages);
            const uint32_t parity = (s / kXStages) & 1u;
            if (!mbar_try_wait(bar, parity)) mbar_wait_slow(c, bar, parity, false);
        }
    }
#endif

    // No bulk copy may still be in flight when the CTA's shared memory goes away:
    // every loader waits (bounded) for the stages it issued most recently.
    if (warp >= kLoaderWarp && warp != kStorerWarp && (threadIdx.x & 31) == 0) {
        const uint32_t which = (uint32_t)loader_index(warp);
        uint32_t issued;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(issued) : "r"(c.base + kSmemHot + 56 + 4 * which) : "memory");
        const uint32_t first = issued > (uint32_t)kNumStages ? issued - kNumStages : 0u;
        c.role = kRoleLoader;
        for (uint32_t s = first; s < issued; ++s) {
            if (s % kLoaders != which) continue;
            const uint32_t bar = c.full_bar(s % kNumStages);
            const uint32_t parity = (s / kNumStages) & 1u;
            if (!mbar_try_wait(bar, parity)) mbar_wait_slow(c, bar, parity, false);
        }
    }
}

#if MKB_BATCH == 1
// Two kernels from one body: the single-GPU one, and the one that can exchange partial sums
// with peer GPUs (MkbTensorParallel), launched when tp.size > 1.
__global__ void __launch_bounds__(kBlockThreads, 1) megakernel(const __grid_constant__ KParams p) {
    megakernel_body<false>(p);
}
__global__ void __launch_bounds__(kBlockThreads, 1) megakernel_tp(const __grid_constant__ KParams p) {
    megakernel_body<true>(p);
}
#elif MKB_BATCH <= 8
// The batched build: up to kBatch sequences per launch (MkbGlobals.batch = 2..8).
__global__ void __launch_bounds__(kBlockThreads, 1) megakernel_batched(const __grid_constant__ KParams p) {
    megakernel_body<false>(p);
}
#else
// The GEMM build: 9..kBatch sequences per launch, projections on tcgen05 tensor cores.
__global__ void __launch_bounds__(kBlockThreads, 1) megakernel_gemm(const __grid_constant__ KParams p) {
    megakernel_body<false>(p);
}
#endif

}  // namespace MKB_NAMESPACE
