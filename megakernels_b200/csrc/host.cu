// C ABI of libmkb200.so (declared in include/mkb200.h): host-side validation,
// TMA descriptor cache, launch and status read-back.  Replaces the pybind11
// glue of the reference (demos/low-latency-llama/llama.cu:26-53), which builds
// its descriptors on every call inside ThunderKittens' bind_kernel.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "mk_common.cuh"

namespace mkb {
__global__ void megakernel(const __grid_constant__ KParams p);
__global__ void megakernel_tp(const __grid_constant__ KParams p);
}
namespace mkb_batched {  // megakernel_batched.cu
int max_batch();
cudaError_t launch(const void* params, size_t params_bytes, int grid, cudaStream_t stream);
}
namespace mkb_gemm {  // megakernel_gemm.cu
int max_batch();
int block_rows();
int stage_cols();
cudaError_t launch(const void* params, size_t params_bytes, int grid, cudaStream_t stream);
}

using namespace mkb;

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

#define MKB_CUDA(call)                                                                   \
    do {                                                                                 \
        cudaError_t e_ = (call);                                                         \
        if (e_ != cudaSuccess)                                                           \
            return fail(MKB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));   \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct KvMapKey {  // also used for weight maps: (ptr, K, R, rows, L, box) and activation maps
    const void* ptr;
    int D, Hkv, T, LB;
    int box = 0;
    bool operator==(const KvMapKey& o) const {
        return ptr == o.ptr && D == o.D && Hkv == o.Hkv && T == o.T && LB == o.LB && box == o.box;
    }
};
struct KvMapEntry {
    KvMapKey key;
    CUtensorMap map;
};

struct DeviceState {
    bool attr_set = false;
    int sm_count = 0;
    int* status = nullptr;  // library-owned status record
    std::vector<KvMapEntry> maps;
};

// L2 look-ahead of the loader beyond the ring, in 32 KiB stages per SM.  MKB_L2_WINDOW_KB is the
// depth while the consumers drain the ring (0 disables), MKB_L2_STALL_WINDOW_KB the depth while
// they sit in a barrier wait, when HBM would otherwise idle.  Measured on the 8B shape: a deep
// steady window re-reads from DRAM (L2 evictions), a deep stall window does not.
int l2_window_from_env(const char* name, int default_kb) {
    const char* e = getenv(name);
    int kb = e ? atoi(e) : default_kb;
    if (kb < 0) kb = 0;
    if (kb > 4096) kb = 4096;
    return kb == 0 ? 0 : kNumStages + kb * 1024 / kStageBytes;
}
const int g_l2_window_stages = l2_window_from_env("MKB_L2_WINDOW_KB", 64);
const int g_l2_stall_window_stages = l2_window_from_env("MKB_L2_STALL_WINDOW_KB", 1024);

std::mutex g_mutex;
DeviceState g_devices[64];
EncodeTiledFn g_encode = nullptr;

int get_encode_fn() {
    if (g_encode) return MKB_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MKB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
        return fail(MKB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return MKB_OK;
}

// 4-D view [D, Hkv, T, L*B] of a KV cache; one box is TS positions of one head.
int kv_tensor_map(DeviceState* ds, const void* ptr, int D, int Hkv, int T, int LB, CUtensorMap* out) {
    KvMapKey key{ptr, D, Hkv, T, LB};
    if (ds)
        for (auto& e : ds->maps)
            if (e.key == key) {
                *out = e.map;
                return MKB_OK;
            }
    int rc = get_encode_fn();
    if (rc) return rc;
    // 5-D view [64, T, D/64, Hkv, L*B] with the 128-byte swizzle: a box is `ts` positions of one
    // head and lands as D/64 sub-tiles of [ts][128 bytes], so that the 8 positions a warp reads
    // side by side (16 bytes each, same column) fall into 8 different bank groups.  With whole
    // 256-byte rows in shared memory they all hit the same banks (8-way conflicts, the attention
    // stages then cost 1.7 us each).
    const int ts = (kStageBytes / 4) / D;
    cuuint64_t dims[5] = {64, (cuuint64_t)T, (cuuint64_t)D / 64, (cuuint64_t)Hkv, (cuuint64_t)LB};
    cuuint64_t strides[4] = {(cuuint64_t)Hkv * D * 2, 128, (cuuint64_t)D * 2, (cuuint64_t)T * Hkv * D * 2};
    cuuint32_t box[5] = {64, (cuuint32_t)ts, (cuuint32_t)D / 64, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUtensorMap m;
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MKB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    if (ds) {
        if (ds->maps.size() >= 64) ds->maps.erase(ds->maps.begin());
        ds->maps.push_back({key, m});
    }
    *out = m;
    return MKB_OK;
}

// 4-D view [64, rows, K/64, L] of a stacked weight [L, rows, K] with the 128-byte swizzle;
// one box is one ring stage of a `kc`-column slice: {64, box_rows, min(kc, stage_cols)/64, 1}
// (16 rows x 1024 columns; 128 x 128 for the GEMM build).
int weight_tensor_map(DeviceState* ds, const void* ptr, int K, int kc, int rows, int L, CUtensorMap* out,
                      int box_rows = 16, int stage_cols = 1024) {
    KvMapKey key{ptr, -K, kc, rows, L, box_rows};
    if (ds)
        for (auto& e : ds->maps)
            if (e.key == key) {
                *out = e.map;
                return MKB_OK;
            }
    int rc = get_encode_fn();
    if (rc) return rc;
    const int cols = kc > stage_cols ? stage_cols : kc;
    cuuint64_t dims[4] = {64, (cuuint64_t)rows, (cuuint64_t)K / 64, (cuuint64_t)L};
    cuuint64_t strides[3] = {(cuuint64_t)K * 2, 128, (cuuint64_t)rows * K * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)cols / 64, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap m;
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MKB_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed with CUresult %d", (int)r);
    if (ds) {
        if (ds->maps.size() >= 64) ds->maps.erase(ds->maps.begin());
        ds->maps.push_back({key, m});
    }
    *out = m;
    return MKB_OK;
}

// GEMM build: activations [batch, K] bf16 as a 3-D view [64, batch, K/64] with the 128-byte
// swizzle; a box is {64, n rows, stage_cols / 64}: rows beyond `batch` read as zero.
int activation_tensor_map(DeviceState* ds, const void* ptr, int K, int batch, int n, int stage_cols, CUtensorMap* out) {
    KvMapKey key{ptr, -K, batch, n, -1, stage_cols};
    if (ds)
        for (auto& e : ds->maps)
            if (e.key == key) {
                *out = e.map;
                return MKB_OK;
            }
    int rc = get_encode_fn();
    if (rc) return rc;
    cuuint64_t dims[3] = {64, (cuuint64_t)batch, (cuuint64_t)K / 64};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)n, (cuuint32_t)stage_cols / 64};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MKB_ERR_CUDA, "cuTensorMapEncodeTiled (activations) failed with CUresult %d", (int)r);
    if (ds) {
        if (ds->maps.size() >= 64) ds->maps.erase(ds->maps.begin());
        ds->maps.push_back({key, m});
    }
    *out = m;
    return MKB_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate(const MkbGlobals* g) {
    if (!g) return fail(MKB_ERR_INVALID_ARGUMENT, "globals pointer is NULL");
    if (g->abi_version != MKB_ABI_VERSION)
        return fail(MKB_ERR_INVALID_ARGUMENT, "ABI version %u, library has %d", g->abi_version,
                    MKB_ABI_VERSION);
    if (g->struct_bytes != sizeof(MkbGlobals))
        return fail(MKB_ERR_INVALID_ARGUMENT, "struct_bytes %u != %zu", g->struct_bytes,
                    sizeof(MkbGlobals));
    const struct {
        const void* p;
        const char* name;
    } ptrs[] = {
        {g->barriers, "barriers"},
        {g->instructions, "instructions"},
        {g->qkv_weights, "qkv_weights"},
        {g->attn_ln_weights, "attn_ln_weights"},
        {g->o_proj_weights, "o_proj_weights"},
        {g->mlp_ln_weights, "mlp_ln_weights"},
        {g->up_proj_weights, "up_proj_weights"},
        {g->gate_proj_weights, "gate_proj_weights"},
        {g->down_proj_weights, "down_proj_weights"},
        {g->lm_head_norm_weights, "lm_head_norm_weights"},
        {g->lm_head_weights, "lm_head_weights"},
        {g->k_cache, "k_cache"},
        {g->v_cache, "v_cache"},
        {g->rope_cos, "rope_cos"},
        {g->rope_sin, "rope_sin"},
        {g->hidden_states, "hidden_states"},
        {g->post_ln_rope_q, "post_ln_rope_q"},
        {g->attn_out, "attn_out"},
        {g->attn_lse_intermediates, "attn_lse_intermediates"},
        {g->attn_out_intermediates, "attn_out_intermediates"},
        {g->silu_out, "silu_out"},
        {g->logits, "logits"},
    };
    for (const auto& e : ptrs) {
        if (!e.p) return fail(MKB_ERR_INVALID_ARGUMENT, "%s is NULL", e.name);
        if (!aligned16(e.p))
            return fail(MKB_ERR_INVALID_ARGUMENT, "%s must be 16-byte aligned", e.name);
    }
    const int H = g->hidden_size, I = g->intermediate_size, D = g->head_dim, R = g->matvec_reduction_size;
    const int Hq = g->num_attention_heads, Hkv = g->num_kv_heads;
    if (g->num_layers < 1 || g->queue_len < 1 || g->num_sms < 1)
        return fail(MKB_ERR_INVALID_ARGUMENT, "num_layers, queue_len and num_sms must be positive");
    if (H != 2048 && H != 4096 && H != 8192)
        return fail(MKB_ERR_UNSUPPORTED, "hidden_size %d: supported are 2048, 4096, 8192", H);
    if (D != 64 && D != 128) return fail(MKB_ERR_UNSUPPORTED, "head_dim %d: supported are 64, 128", D);
    if (Hkv < 1 || Hq % Hkv != 0) return fail(MKB_ERR_INVALID_ARGUMENT, "Hq %d not a multiple of Hkv %d", Hq, Hkv);
    const int gqa = Hq / Hkv;
    if (!(gqa == 4 || (gqa == 8 && D == 128)))
        return fail(MKB_ERR_UNSUPPORTED, "GQA ratio %d with head_dim %d is not supported", gqa, D);
    if (Hq % 4 != 0) return fail(MKB_ERR_UNSUPPORTED, "Hq %d must be a multiple of 4", Hq);
    if (R != 256 && R != 512 && R != 1024 && R != 2048)
        return fail(MKB_ERR_UNSUPPORTED, "matvec_reduction_size %d: supported are 256, 512, 1024, 2048", R);
    if ((Hq * D) % R != 0 || I % R != 0)
        return fail(MKB_ERR_INVALID_ARGUMENT, "o-proj inputs %d and intermediate %d must be multiples of %d", Hq * D, I, R);
    if (I % 16 != 0 || g->vocab_size % 16 != 0)
        return fail(MKB_ERR_INVALID_ARGUMENT, "intermediate and vocab sizes must be multiples of 16");
    if (g->barrier_width < Hq + 2 * Hkv || g->barrier_width < I / R || g->barrier_ops < 7)
        return fail(MKB_ERR_INVALID_ARGUMENT, "barriers tensor too small: ops %d width %d", g->barrier_ops, g->barrier_width);
    if (g->kv_batch < 1 || g->kv_max_len < 1)
        return fail(MKB_ERR_INVALID_ARGUMENT, "KV cache needs batch >= 1 and length >= 1");
    if (g->batch <= 1 && !g->pos_id_device && (g->pos_id < 0 || g->pos_id >= g->kv_max_len))
        return fail(MKB_ERR_INVALID_ARGUMENT, "pos_id %d outside the KV cache length %d", g->pos_id, g->kv_max_len);
    if (g->max_partials < 1) return fail(MKB_ERR_INVALID_ARGUMENT, "max_partials must be >= 1");
    if (g->skip_attn_reduction < 0 || g->skip_attn_reduction > 2)
        return fail(MKB_ERR_INVALID_ARGUMENT, "skip_attn_reduction must be 0, 1 or 2");
    const MkbTensorParallel& tp = g->tp;
    if (tp.size > 1) {
        if (tp.size > MKB_MAX_TP || tp.rank < 0 || tp.rank >= tp.size)
            return fail(MKB_ERR_INVALID_ARGUMENT, "tp: size %d (max %d), rank %d", tp.size, MKB_MAX_TP, tp.rank);
        if (tp.num_chunks < tp.size || tp.num_chunks > MKB_TP_MAX_CHUNKS || tp.num_chunks % tp.size != 0 ||
            H % (2 * tp.num_chunks) != 0)
            return fail(MKB_ERR_INVALID_ARGUMENT,
                        "tp: num_chunks %d must be a multiple of size %d, at most %d, and divide H/2",
                        tp.num_chunks, tp.size, MKB_TP_MAX_CHUNKS);
        for (int r = 0; r < tp.size; ++r) {
            if (!tp.hidden_ll_peers[r] || !tp.recv_peers[r])
                return fail(MKB_ERR_INVALID_ARGUMENT, "tp: peer pointers of rank %d are NULL", r);
            if (!aligned16(tp.hidden_ll_peers[r]) || !aligned16(tp.recv_peers[r]))
                return fail(MKB_ERR_INVALID_ARGUMENT, "tp: peer pointers of rank %d must be 16-byte aligned", r);
        }
        if (!tp.partial || !aligned16(tp.partial)) return fail(MKB_ERR_INVALID_ARGUMENT, "tp: partial buffer is NULL or unaligned");
        if (!tp.epoch_device) return fail(MKB_ERR_INVALID_ARGUMENT, "tp: epoch_device is NULL");
    } else {
        if (!g->residual_acc || !aligned16(g->residual_acc))
            return fail(MKB_ERR_INVALID_ARGUMENT, "residual_acc (int64 [H], zeroed per launch) is NULL or not 16-byte aligned");
        if (g->residual_scale != 0.f && (g->residual_scale < 1.f || g->residual_scale != (float)(int)g->residual_scale))
            return fail(MKB_ERR_INVALID_ARGUMENT, "residual_scale %g must be a positive integer", g->residual_scale);
    }
    if (g->batch > 1) {
        if (g->batch > MKB_MAX_BATCH || g->batch > mkb_gemm::max_batch())
            return fail(MKB_ERR_UNSUPPORTED, "batch %d: at most %d sequences per launch", g->batch, MKB_MAX_BATCH);
        if (H > 4096) return fail(MKB_ERR_UNSUPPORTED, "batched decode supports hidden_size <= 4096, got %d", H);
        if (g->batch > mkb_batched::max_batch()) {  // the tcgen05 build: 128-row blocks, one head per block
            if (D != 128 || H % 128 != 0 || I % 128 != 0 || g->vocab_size % 128 != 0 || R % 128 != 0)
                return fail(MKB_ERR_UNSUPPORTED, "batch > %d needs head_dim 128 and sizes that are multiples of 128",
                            mkb_batched::max_batch());
            if (!g->pos_id_device)
                return fail(MKB_ERR_INVALID_ARGUMENT, "batch > %d needs pos_id_device (one position per sequence)",
                            mkb_batched::max_batch());
        }
        if (tp.size > 1) return fail(MKB_ERR_UNSUPPORTED, "batched decode has no tensor-parallel variant");
        if (!g->normed_states || !aligned16(g->normed_states))
            return fail(MKB_ERR_INVALID_ARGUMENT, "batch > 1 needs normed_states (bf16 [batch, H], 16-byte aligned)");
        if (g->kv_batch < g->batch)
            return fail(MKB_ERR_INVALID_ARGUMENT, "KV cache holds %d sequences, batch is %d", g->kv_batch, g->batch);
        if (g->barrier_width < g->batch * Hq || g->barrier_ops <= MKB_BARRIER_ROW_RMS_NORM)
            return fail(MKB_ERR_INVALID_ARGUMENT, "batch %d needs barrier_width >= %d and barrier_ops > %d",
                        g->batch, g->batch * Hq, MKB_BARRIER_ROW_RMS_NORM);
        if (!g->pos_id_device)
            for (int s = 0; s < g->batch; ++s)
                if (g->pos_ids[s] < 0 || g->pos_ids[s] >= g->kv_max_len)
                    return fail(MKB_ERR_INVALID_ARGUMENT, "pos_ids[%d] = %d outside the KV cache length %d", s,
                                g->pos_ids[s], g->kv_max_len);
    } else if (g->batch < 0) {
        return fail(MKB_ERR_INVALID_ARGUMENT, "batch %d", g->batch);
    }
    if (g->upgate_instructions_per_layer < 0 || g->barrier_ops <= MKB_BARRIER_ROW_RMS_READ)
        return fail(MKB_ERR_INVALID_ARGUMENT, "upgate_instructions_per_layer %d / barrier_ops %d (row %d is needed)",
                    g->upgate_instructions_per_layer, g->barrier_ops, MKB_BARRIER_ROW_RMS_READ);
    return MKB_OK;
}

int device_state(DeviceState** out) {
    int dev = 0;
    MKB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MKB_ERR_UNSUPPORTED, "device index %d", dev);
    DeviceState& ds = g_devices[dev];
    if (!ds.attr_set) {
        cudaDeviceProp prop;
        MKB_CUDA(cudaGetDeviceProperties(&prop, dev));
        if (prop.major < 10)
            return fail(MKB_ERR_UNSUPPORTED, "device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);
        ds.sm_count = prop.multiProcessorCount;
        MKB_CUDA(cudaFuncSetAttribute(megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc));
        MKB_CUDA(cudaFuncSetAttribute(megakernel_tp, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc));
        // status record, then the fused-argmax scratch: arrival counter + {value, index} per CTA
        const size_t words = MKB_STATUS_WORDS + 2 + 2 * (size_t)ds.sm_count * MKB_MAX_BATCH;
        MKB_CUDA(cudaMalloc(&ds.status, words * sizeof(int)));
        MKB_CUDA(cudaMemset(ds.status, 0, words * sizeof(int)));
        ds.attr_set = true;
    }
    *out = &ds;
    return MKB_OK;
}

// Validate `g` and build the kernel parameters.  `ds` carries the descriptor cache; with
// ds == nullptr the TMA descriptors are encoded afresh and no host memory is allocated.
int prepare_launch(const MkbGlobals* g, DeviceState* ds, int* status, int sm_count, KParams& p) {
    int rc = validate(g);
    if (rc) return rc;
    if (g->num_sms > sm_count)
        return fail(MKB_ERR_INVALID_ARGUMENT,
                    "%d instruction queues but the device has %d SMs: all CTAs must be co-resident",
                    g->num_sms, sm_count);

    memset(&p, 0, sizeof(p));
    p.barriers = g->barriers;
    p.instructions = g->instructions;
    p.timings = (g->flags & MKB_FLAG_RECORD_TIMINGS) ? g->timings : nullptr;
    if ((g->flags & MKB_FLAG_RECORD_TIMINGS) && !g->timings)
        return fail(MKB_ERR_INVALID_ARGUMENT, "MKB_FLAG_RECORD_TIMINGS needs a timings tensor");
    p.status = status;
    p.queue_len = g->queue_len;
    p.barrier_ops = g->barrier_ops;
    p.barrier_width = g->barrier_width;
    p.qkv_w = (const __nv_bfloat16*)g->qkv_weights;
    p.attn_ln_w = (const __nv_bfloat16*)g->attn_ln_weights;
    p.o_w = (const __nv_bfloat16*)g->o_proj_weights;
    p.mlp_ln_w = (const __nv_bfloat16*)g->mlp_ln_weights;
    p.up_w = (const __nv_bfloat16*)g->up_proj_weights;
    p.gate_w = (const __nv_bfloat16*)g->gate_proj_weights;
    p.down_w = (const __nv_bfloat16*)g->down_proj_weights;
    p.lm_norm_w = (const __nv_bfloat16*)g->lm_head_norm_weights;
    p.lm_head_w = (const __nv_bfloat16*)g->lm_head_weights;
    p.k_cache = (__nv_bfloat16*)g->k_cache;
    p.v_cache = (__nv_bfloat16*)g->v_cache;
    p.rope_cos = g->rope_cos;
    p.rope_sin = g->rope_sin;
    p.hidden = (__nv_bfloat16*)g->hidden_states;
    p.q_rope = (__nv_bfloat16*)g->post_ln_rope_q;
    p.attn_out = (__nv_bfloat16*)g->attn_out;
    p.silu_out = (__nv_bfloat16*)g->silu_out;
    p.logits = (__nv_bfloat16*)g->logits;
    p.attn_lse = g->attn_lse_intermediates;
    p.attn_o = g->attn_out_intermediates;
    p.L = g->num_layers;
    p.H = g->hidden_size;
    p.I = g->intermediate_size;
    p.D = g->head_dim;
    p.Hq = g->num_attention_heads;
    p.Hkv = g->num_kv_heads;
    p.V = g->vocab_size;
    p.T = g->kv_max_len;
    p.B = g->kv_batch;
    p.max_partials = g->max_partials;
    p.R = g->matvec_reduction_size;
    p.qkv_rows = (p.Hq + 2 * p.Hkv) * p.D;
    p.o_in = p.Hq * p.D;
    p.pos_id = g->pos_id;
    p.pos_id_ptr = g->pos_id_device;
    p.residual_acc = (long long*)g->residual_acc;
    p.residual_mult = g->residual_scale > 0.f ? (long long)g->residual_scale : 1;
    p.batch = g->batch > 1 ? g->batch : 1;
    for (int s = 0; s < 8; ++s) p.pos_ids[s] = g->pos_ids[s];
    p.normed = (__nv_bfloat16*)g->normed_states;
    // batched launches order the down-proj behind the RMS_NORM instructions through the up/gate
    p.thr_down_waits_rms = g->batch > 1 ? 0 : g->upgate_instructions_per_layer;
    if (g->argmax_out && ds) {  // the scratch sits behind the library's own status record
        p.argmax_out = g->argmax_out;
        p.argmax_scratch = ds->status + MKB_STATUS_WORDS;
    }
    if (g->tp.size > 1) {
        p.tp_size = g->tp.size;
        p.tp_rank = g->tp.rank;
        p.tp_chunks = g->tp.num_chunks;
        p.tp_epoch_ptr = g->tp.epoch_device;
        p.tp_partial = g->tp.partial;
        for (int r = 0; r < g->tp.size; ++r) {
            p.tp_hidden_ll[r] = (uint2*)g->tp.hidden_ll_peers[r];
            p.tp_recv[r] = (float*)g->tp.recv_peers[r];
        }
    }
    p.attn_scale_log2e = g->attn_scale * 1.4426950408889634f;
    p.rms_eps = g->rms_norm_eps;
    p.skip_attn_reduction = g->skip_attn_reduction;
    // rows per block of the schedule: 16, or 128 for the tcgen05 build (batch > 8)
    const bool gemm = p.batch > mkb_batched::max_batch();
    const int br = gemm ? mkb_gemm::block_rows() : 16;
    p.thr_qkv_waits_down = (p.H / br) * (p.I / p.R);
    p.thr_attn_waits_qkv = p.D / br;
    p.thr_oproj_waits_attn = p.Hq;
    p.thr_upgate_waits_oproj = (p.H / br) * (p.o_in / p.R);
    p.thr_down_waits_upgate = p.R / br;
    p.gemm_n = (p.batch + 15) / 16 * 16;
    if (gemm) p.argmax_out = nullptr;  // no fused argmax in this build: the host reduces the logits
    const unsigned ms = g->wait_timeout_ms ? g->wait_timeout_ms : 2000u;
    p.timeout_ns = (unsigned long long)ms * 1000000ull;
    p.l2_window_stages = g_l2_window_stages;
    p.l2_stall_window_stages = g_l2_stall_window_stages > g_l2_window_stages ? g_l2_stall_window_stages
                                                                             : g_l2_window_stages;
    p.poll_sleep_ns = 20;

    rc = kv_tensor_map(ds, g->k_cache, p.D, p.Hkv, p.T, p.L * p.B, &p.k_map);
    if (rc) return rc;
    rc = kv_tensor_map(ds, g->v_cache, p.D, p.Hkv, p.T, p.L * p.B, &p.v_map);
    if (rc) return rc;

    const struct {
        const void* ptr;
        int K, kc, rows, L;
        CUtensorMap* out;
    } wmaps[] = {
        {g->qkv_weights, p.H, p.H, p.qkv_rows, p.L, &p.qkv_map},
        {g->o_proj_weights, p.o_in, p.R, p.H, p.L, &p.o_map},
        {g->up_proj_weights, p.H, p.H, p.I, p.L, &p.up_map},
        {g->gate_proj_weights, p.H, p.H, p.I, p.L, &p.gate_map},
        {g->down_proj_weights, p.I, p.R, p.H, p.L, &p.down_map},
        {g->lm_head_weights, p.H, p.H, p.V, 1, &p.lm_map},
    };
    for (const auto& wm : wmaps) {
        rc = gemm ? weight_tensor_map(ds, wm.ptr, wm.K, wm.kc, wm.rows, wm.L, wm.out, br, mkb_gemm::stage_cols())
                  : weight_tensor_map(ds, wm.ptr, wm.K, wm.kc, wm.rows, wm.L, wm.out);
        if (rc) return rc;
    }
    if (gemm) {
        const int sc = mkb_gemm::stage_cols();
        rc = activation_tensor_map(ds, g->normed_states, p.H, p.batch, p.gemm_n, sc, &p.x_normed_map);
        if (rc) return rc;
        rc = activation_tensor_map(ds, g->attn_out, p.o_in, p.batch, p.gemm_n, sc, &p.x_attn_map);
        if (rc) return rc;
        rc = activation_tensor_map(ds, g->silu_out, p.I, p.batch, p.gemm_n, sc, &p.x_silu_map);
        if (rc) return rc;
    }

    return MKB_OK;
}

// Synchronise the stream, copy the status record at `st` (device memory) into `out` through a
// stack buffer, re-arm it when it holds an error.  Allocates nothing.
int read_status(int* st, void* cuda_stream, MkbStatus* out) {
    MKB_CUDA(cudaStreamSynchronize((cudaStream_t)cuda_stream));
    int words[MKB_STATUS_WORDS];
    MKB_CUDA(cudaMemcpy(words, st, sizeof(words), cudaMemcpyDeviceToHost));
    memcpy(out, words, sizeof(MkbStatus));
    if (words[0] == MKB_OK && words[kStatusAbortWord] == 0) return MKB_OK;
    MKB_CUDA(cudaMemset(st, 0, sizeof(words)));  // re-arm for the next launch
    static const char* roles[] = {"loader", "consumer", "storer"};
    const char* role = (out->role >= 0 && out->role < 3) ? roles[out->role] : "?";
    return fail(out->code ? out->code : MKB_ERR_DEVICE_TIMEOUT,
                "device error %d on queue %d, instruction %d (opcode %d, %s): detail %d %d %d %d",
                out->code, out->sm, out->instruction_index, out->opcode, role, out->detail[0],
                out->detail[1], out->detail[2], out->detail[3]);
}

}  // namespace

namespace mkb {
// Shared with the other translation units of the library (not part of the C ABI).
int prepare_launch_uncached(const MkbGlobals* g, int* status, int sm_count, KParams& p) {
    return prepare_launch(g, nullptr, status, sm_count, p);
}
int set_error(int code, const char* msg) { return fail(code, "%s", msg); }
int read_status_record(int* st, void* cuda_stream, MkbStatus* out) { return read_status(st, cuda_stream, out); }
std::mutex& library_mutex() { return g_mutex; }
}  // namespace mkb

extern "C" {

int mkb_launch(const MkbGlobals* g, void* cuda_stream) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    KParams p;
    rc = prepare_launch(g, ds, (g && g->status) ? g->status : ds->status, ds->sm_count, p);
    if (rc) return rc;
    if (p.batch > mkb_batched::max_batch()) {
        MKB_CUDA(mkb_gemm::launch(&p, sizeof(p), g->num_sms, (cudaStream_t)cuda_stream));
        return MKB_OK;
    }
    if (p.batch > 1) {
        MKB_CUDA(mkb_batched::launch(&p, sizeof(p), g->num_sms, (cudaStream_t)cuda_stream));
        return MKB_OK;
    }
    if (p.tp_size > 1)
        megakernel_tp<<<g->num_sms, kBlockThreads, kSmemAlloc, (cudaStream_t)cuda_stream>>>(p);
    else
        megakernel<<<g->num_sms, kBlockThreads, kSmemAlloc, (cudaStream_t)cuda_stream>>>(p);
    MKB_CUDA(cudaGetLastError());
    return MKB_OK;
}



int mkb_sync_status(const MkbGlobals* g, void* cuda_stream, MkbStatus* out) {
    if (!out) return fail(MKB_ERR_INVALID_ARGUMENT, "status output pointer is NULL");
    std::lock_guard<std::mutex> lock(g_mutex);
    int dev = 0;
    MKB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MKB_ERR_UNSUPPORTED, "device index %d", dev);
    // A record in caller memory is read without touching the library's per-device state, so
    // that this call allocates nothing (it is the read-back path of mkb_launch_no_alloc).
    int* st = (g && g->status) ? g->status : nullptr;
    if (!st) {
        DeviceState* ds = nullptr;
        int rc = device_state(&ds);
        if (rc) return rc;
        st = ds->status;
    }
    int rc = read_status(st, cuda_stream, out);
    // an aborted launch may have left the fused-argmax arrival counter short of a full round
    if (rc != MKB_OK && g_devices[dev].attr_set)
        cudaMemset(g_devices[dev].status + MKB_STATUS_WORDS, 0, sizeof(int));
    return rc;
}

// Host-side check of an instruction tensor (a HOST copy, [num_sms, queue_len, 32]):
// every index an instruction carries must stay inside the tensors of `g`.
int mkb_validate_instructions(const MkbGlobals* g, const int32_t* host_instructions) {
    int rc = validate(g);
    if (rc) return rc;
    if (!host_instructions) return fail(MKB_ERR_INVALID_ARGUMENT, "host_instructions is NULL");
    const int L = g->num_layers, H = g->hidden_size, I = g->intermediate_size, D = g->head_dim;
    const int Hq = g->num_attention_heads, Hkv = g->num_kv_heads, R = g->matvec_reduction_size;
    const int br = g->batch > mkb_batched::max_batch() ? mkb_gemm::block_rows() : 16;  // rows per block
    const int qkv_blocks = (Hq + 2 * Hkv) * D / br;
    for (int sm = 0; sm < g->num_sms; ++sm) {
        for (int i = 0; i < g->queue_len; ++i) {
            const int32_t* w = host_instructions + ((size_t)sm * g->queue_len + i) * MKB_INTS_PER_INSTRUCTION;
            auto bad = [&](const char* what) {
                return fail(MKB_ERR_INVALID_ARGUMENT, "queue %d instruction %d (opcode %d): %s", sm, i, w[0], what);
            };
            auto range_ok = [](int s, int e, int n) { return 0 <= s && s <= e && e <= n; };
            switch (w[0]) {
                case MKB_OP_NOOP:
                    break;
                case MKB_OP_RMS_QKV_ROPE_APPEND:
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (!range_ok(w[2], w[3], qkv_blocks)) return bad("block range outside the QKV rows");
                    break;
                case MKB_OP_PARTIAL_ATTENTION:
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (w[2] < 0 || w[2] >= Hkv) return bad("KV head out of range");
                    if (w[3] < 1 || w[4] < 0 || w[4] >= w[3]) return bad("partial index outside num_partials");
                    if (g->skip_attn_reduction != 1 && w[4] >= g->max_partials) return bad("partial index beyond max_partials");
                    if (g->skip_attn_reduction == 1 && w[3] != 1) return bad("skip_attn_reduction = 1 needs num_partials == 1");
                    if (g->skip_attn_reduction == 2 && w[3] > 24) return bad("at most 24 partials can be merged by the last one");
                    if (w[5] < 0 || w[5] >= (g->batch > 1 ? g->batch : 1)) return bad("sequence outside the batch");
                    break;
                case MKB_OP_ATTENTION_REDUCTION: {
                    if (g->skip_attn_reduction == 2) return bad("AttentionReduction instruction although the last partial merges (skip_attn_reduction = 2)");
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (w[2] < 0 || w[2] + 4 > Hq) return bad("head range outside the Q heads");
                    const int n = w[5];
                    if (n < 1 || n > 24) return bad("reduction list length must be 1..24");
                    if (w[7 + n] < 0 || w[7 + n] >= (g->batch > 1 ? g->batch : 1)) return bad("sequence outside the batch");
                    for (int j = 0; j < n; ++j)
                        if (w[6 + j] < 0 || w[6 + j] >= g->max_partials) return bad("reduction index beyond max_partials");
                    if (!w[4] && (w[6 + n] < 0 || w[6 + n] >= g->max_partials)) return bad("output partial index beyond max_partials");
                } break;
                case MKB_OP_O_PROJ_RESIDUAL:
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (!range_ok(w[2], w[3], H / br)) return bad("block range outside the hidden rows");
                    if (w[4] < 0 || w[4] >= Hq * D / R) return bad("reduction block out of range");
                    break;
                case MKB_OP_RMS_UPGATE_SILU:
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (w[2] < 0 || w[2] > MKB_INTS_PER_INSTRUCTION - 3) return bad("block list too long");
                    for (int j = 0; j < w[2]; ++j)
                        if (w[3 + j] < 0 || w[3 + j] >= I / br) return bad("block outside the intermediate rows");
                    break;
                case MKB_OP_DOWN_PROJ_RESIDUAL:
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (!range_ok(w[2], w[3], H / br)) return bad("block range outside the hidden rows");
                    if (w[4] < 0 || w[4] >= I / R) return bad("reduction block out of range");
                    break;
                case MKB_OP_RMS_LM_HEAD:
                    if (!range_ok(w[1], w[2], g->vocab_size / br)) return bad("block range outside the vocabulary");
                    break;
                case MKB_OP_RMS_NORM:
                    if (g->batch <= 1) return bad("RMS_NORM instruction in a single-sequence launch");
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (w[2] < 0 || w[2] > 2) return bad("which must be 0, 1 or 2");
                    if (w[3] < 0 || w[3] >= g->batch) return bad("sequence outside the batch");
                    break;
                case MKB_OP_TP_ALL_REDUCE:
                    if (g->tp.size <= 1) return bad("all-reduce instruction without tensor parallelism");
                    if (w[1] < 0 || w[1] >= L) return bad("layer out of range");
                    if (w[2] < 0 || w[2] > 1) return bad("which must be 0 (o-proj) or 1 (down-proj)");
                    if (w[4] != g->tp.num_chunks || w[3] < 0 || w[3] >= w[4]) return bad("chunk outside tp.num_chunks");
                    break;
                default:
                    return bad("unknown opcode");
            }
        }
    }
    return MKB_OK;
}

const char* mkb_last_error(void) { return g_error; }

int mkb_sm_count(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

int mkb_smem_bytes(void) { return kSmemAlloc; }
int mkb_block_threads(void) { return kBlockThreads; }
int mkb_abi_version(void) { return MKB_ABI_VERSION; }

}  // extern "C"
