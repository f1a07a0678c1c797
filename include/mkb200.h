/*
 * mkb200.h - C ABI of the B200 decode megakernel library (libmkb200.so).
 *
 * The library replaces the compiled extension module the reference loads as
 * `mk_llama` (megakernels/mk.py:5-9) and calls once per decoded token with 23
 * tensors and 4 scalars (megakernels/demos/latency/mk.py:15-49; binding order
 * demos/low-latency-llama/llama.cu:29-52).  Here the same argument set is one
 * plain struct of device pointers and sizes; nothing in the signatures is a
 * torch or C++ type, so any host language with a C FFI can bind it.
 *
 * All pointers are device pointers owned by the caller and must stay valid
 * until the stream has executed the launch.  The library keeps no pointer
 * after mkb_launch returns, except cached TMA descriptors keyed by the KV
 * cache addresses and shape.
 */
#ifndef MKB200_H
#define MKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MKB_ABI_VERSION 4

/* instruction encoding (megakernels/scheduler.py:13-14) */
#define MKB_INTS_PER_INSTRUCTION 32
#define MKB_TIMING_SLOTS 128
#define MKB_STATUS_WORDS 16

/* opcodes (megakernels/demos/latency/instructions.py:32-196;
 * demos/low-latency-llama/llama.cuh:7-13) */
enum {
    MKB_OP_NOOP = 0,
    MKB_OP_RMS_QKV_ROPE_APPEND = 1,
    MKB_OP_PARTIAL_ATTENTION = 2,
    MKB_OP_ATTENTION_REDUCTION = 3,
    MKB_OP_O_PROJ_RESIDUAL = 4,
    MKB_OP_RMS_UPGATE_SILU = 5,
    MKB_OP_DOWN_PROJ_RESIDUAL = 6,
    MKB_OP_RMS_LM_HEAD = 7,
    /* No counterpart in the reference (its kernel is single-GPU): one chunk of the
     * tensor-parallel all-reduce of the residual stream, see MkbTensorParallel.
     * words: [8, layer, which (0 after o-proj, 1 after down-proj), chunk, num_chunks] */
    MKB_OP_TP_ALL_REDUCE = 8,
    /* No counterpart in the reference's latency instruction set (its kernel decodes one
     * sequence and fuses the norm into the consuming matvec).  Batched launches only
     * (MkbGlobals.batch > 1): RMSNorm of ONE sequence's residual stream into `normed_states`,
     * so that the 148 SMs do not each normalise all sequences.
     * words: [9, layer, which (0 attention norm, 1 MLP norm, 2 final norm), sequence];
     * counts into barriers[layer][MKB_BARRIER_ROW_RMS_NORM][which]; the RMS + matvec
     * opcodes 1, 5 and 7 then wait for `batch` arrivals there instead of normalising. */
    MKB_OP_RMS_NORM = 9,
};

/* Barrier rows: opcode k counts into row k - 1 (rows 0..6), as in the reference.  Row 8 has
 * no counterpart there: every RMS + up/gate instruction bumps barriers[layer][8][0] once its
 * read of the residual stream is complete, and the down-proj of that layer, which adds to the
 * residual stream, waits for MkbGlobals.upgate_instructions_per_layer arrivals (the reference
 * orders down-proj after the up/gate blocks of its input slice only, matvec_adds.cu:181-186,
 * which leaves a slow SM reading a residual that already holds part of the layer's output). */
#define MKB_BARRIER_ROW_RMS_READ 8
#define MKB_BARRIER_ROW_RMS_NORM 9 /* batched launches: see MKB_OP_RMS_NORM */

#define MKB_MAX_BATCH 64

/* MkbGlobals.flags */
#define MKB_FLAG_RECORD_TIMINGS 1u /* write per-instruction event times (ns) into `timings` */

/* timing slots inside one instruction's 128-int row (low 32 bits of %globaltimer, ns);
 * the reference records clock64 deltas at ids of its own (include/util.cuh:214-246) */
enum {
    MKB_T_CONSUMER_START = 0,      /* consumers reach the instruction */
    MKB_T_CONSUMER_WAIT_DONE = 1,  /* its global barrier is satisfied */
    MKB_T_CONSUMER_ACT_READY = 2,  /* activation vector (and RMSNorm) in registers */
    MKB_T_CONSUMER_FIRST_STAGE = 3,/* first ring stage of the instruction has arrived */
    MKB_T_CONSUMER_DONE = 4,       /* last block handed to the storer */
    MKB_T_ATTN_STAGES_DONE = 5,    /* partial attention: all KV stages folded, merge starts */
    MKB_T_RMS_LOADED = 6,          /* RMS ops: hidden state loaded, partial sums of squares written */
    MKB_T_RMS_SUMMED = 7,          /* RMS ops: block-wide sum of squares available */
    MKB_T_TP_SENT = 5,             /* all-reduce: this rank's sums stored at the owner, arrival signalled */
    MKB_T_TP_ARRIVED = 6,          /* all-reduce, owner only: all ranks' sums have arrived */
    MKB_T_LOADER_START = 8,        /* loader reaches the instruction */
    MKB_T_LOADER_DONE = 9,         /* last stage of the instruction issued */
    MKB_T_STORER_START = 16,       /* storer reaches the instruction */
    MKB_T_STORER_DONE = 17,        /* last barrier signal of the instruction sent */
};

/* return / status codes */
enum {
    MKB_OK = 0,
    MKB_ERR_INVALID_ARGUMENT = 1, /* a shape/pointer check failed; nothing was launched */
    MKB_ERR_CUDA = 2,             /* a CUDA runtime/driver call failed */
    MKB_ERR_DEVICE_TIMEOUT = 3,   /* a device-side wait gave up; see MkbStatus */
    MKB_ERR_BAD_OPCODE = 4,       /* the device met an opcode it does not know */
    MKB_ERR_UNSUPPORTED = 5,      /* valid request this build cannot run */
};

/*
 * Tensor parallelism inside the kernel (no counterpart in the reference, which shards
 * only its torch model, megakernels/llama.py:665-691).  With `size` > 1 every rank runs
 * the same launch on its shard and the o-proj / down-proj partial sums are exchanged by
 * MKB_OP_TP_ALL_REDUCE instructions over peer memory instead of a library collective:
 *
 *   1. o-proj / down-proj store their fp32 block sums into `partial[slice][H]` (local)
 *      instead of adding them to hidden_states;
 *   2. the instruction for chunk c (elements [c*H/n, (c+1)*H/n), n = num_chunks) waits
 *      for the local projection, sums the slices and stores the result into row `rank` of
 *      the receive buffer of the chunk's owner (rank c % size).  Every pair of sums travels
 *      as one 16-byte store {x, tag, y, tag}: each 8-byte half arrives whole, and the tag,
 *      unique per all-reduce, marks the value next to it as this round's, so the sender
 *      needs no fence and the receiver no separate flag;
 *   3. on the owner the threads of the same instruction poll the pairs they reduce until all
 *      ranks' tags are current, add the rows in rank order to the residual stream in fp32,
 *      round to bf16 once and store {bf16x2, tag} words into the tagged residual buffer of
 *      EVERY rank;
 *   4. the following RMSNorm instruction reads the residual stream from that buffer, every
 *      thread polling the words it needs until they carry the tag.
 *
 * All ranks therefore hold bit-identical residual streams, and no step needs a fence, a
 * counter or a reset: a tag is derived from (*epoch_device, layer, which), so every all-reduce
 * of every launch has its own.  `*epoch_device` must be the number of launches completed so
 * far on this rank group (same value on all ranks; the caller increments it after every
 * launch).  Recovery rule: a launch that ends in an error may already have stored sums
 * tagged with the current value, so before the next launch EVERY rank must set
 * `*epoch_device` to a value larger than any rank has used (the maximum over ranks plus
 * one, agreed through a host-side collective); a rank that merely increments its own
 * counter either reuses the aborted launch's tags or drifts apart from its peers.
 * hidden_states keeps its meaning as the kernel's INPUT (the token embedding); the
 * running residual stream of a tensor-parallel launch lives in the tagged buffer.
 * Every peer pointer must be valid on THIS device (cudaIpcOpenMemHandle or an equivalent
 * mapping with peer access enabled); entry `rank` is the local buffer.  All buffers must be
 * zero before the first launch.
 */
#define MKB_MAX_TP 8
#define MKB_TP_MAX_CHUNKS 32
typedef struct MkbTensorParallel {
    int32_t size;        /* ranks; 0 or 1 disables everything below */
    int32_t rank;
    int32_t num_chunks;  /* chunks per all-reduce: a multiple of size, <= MKB_TP_MAX_CHUNKS */
    int32_t reserved;
    void *hidden_ll_peers[MKB_MAX_TP]; /* [H/2] x {bf16x2, tag} (8 bytes): residual stream of every rank */
    void *recv_peers[MKB_MAX_TP];      /* [size][H/2] x {f32, tag, f32, tag} (16 bytes): receive
                                          buffer of every rank */
    float *partial;                    /* local fp32 [max(Hq*D, I) / R][H] */
    const int32_t *epoch_device;       /* launches completed so far */
} MkbTensorParallel;

/*
 * The kernel's argument set.  Replaces `globals_t` of the reference
 * (demos/low-latency-llama/llama.cuh:48-158) and the Python-side `Globals`
 * (megakernels/instructions.py:10-69, demos/latency/instructions.py:9-29).
 * Model dimensions are run-time values (the reference compiles them in,
 * llama.cuh:15-26); under tensor parallelism they are the per-rank values.
 * This build instantiates its pipelines for hidden_size 2048, 4096 or 8192,
 * head_dim 64 or 128, a GQA ratio of 4 (or 8 with head_dim 128) and
 * matvec_reduction_size 256, 512, 1024 or 2048; anything else is refused with
 * MKB_ERR_UNSUPPORTED before a launch.
 */
typedef struct MkbGlobals {
    uint32_t abi_version; /* MKB_ABI_VERSION */
    uint32_t struct_bytes; /* sizeof(MkbGlobals) as the caller sees it */

    /* ---- virtual-machine state ---- */
    int32_t *barriers;           /* [num_layers, barrier_ops, barrier_width] int32, zeroed per token */
    const int32_t *instructions; /* [num_sms, queue_len, 32] int32 */
    int32_t *timings;            /* [num_sms, queue_len, 128] int32 or NULL */
    int32_t num_sms;             /* number of instruction queues == grid size */
    int32_t queue_len;
    int32_t barrier_ops;         /* 10 in the reference (latency/scheduler.py:59) */
    int32_t barrier_width;       /* Hq + 2*Hkv */

    /* ---- weights, bf16, row-major [.., out, in], stacked over layers ---- */
    const void *qkv_weights;          /* [L, (Hq+2Hkv)*D, H] */
    const void *attn_ln_weights;      /* [L, H] */
    const void *o_proj_weights;       /* [L, H, Hq*D] */
    const void *mlp_ln_weights;       /* [L, H] */
    const void *up_proj_weights;      /* [L, I, H] */
    const void *gate_proj_weights;    /* [L, I, H] */
    const void *down_proj_weights;    /* [L, H, I] */
    const void *lm_head_norm_weights; /* [H] */
    const void *lm_head_weights;      /* [V, H] */

    /* ---- KV cache, bf16 [L*B, T, Hkv, D] (latency/mk.py:12-13) ---- */
    void *k_cache;
    void *v_cache;

    /* ---- RoPE tables, fp32 [>= pos_id+1, D] (>= kv_max_len rows when pos_id_device is
     * used: the kernel checks a device-side position against kv_max_len only),
     * interleaved pair layout ---- */
    const float *rope_cos;
    const float *rope_sin;

    /* ---- activations ---- */
    void *hidden_states;            /* bf16 [H]  input: the token embedding.  The reference's kernel
                                       adds every o-proj / down-proj output into this vector with
                                       bf16 atomics (matvec_adds.cu:78), whose rounding depends on the
                                       arrival order; here it is never written, the outputs are summed
                                       in `residual_acc` */
    void *post_ln_rope_q;           /* bf16 [Hq*D] */
    void *attn_out;                 /* bf16 [Hq*D] */
    float *attn_lse_intermediates;  /* fp32 [Hq, max_partials] */
    float *attn_out_intermediates;  /* fp32 [Hq, max_partials, D] */
    void *silu_out;                 /* bf16 [I] */
    void *logits;                   /* bf16 [V] */

    /* ---- model dimensions ---- */
    int32_t num_layers;
    int32_t hidden_size;         /* H */
    int32_t intermediate_size;   /* I */
    int32_t head_dim;            /* D: 64 or 128 */
    int32_t num_attention_heads; /* Hq */
    int32_t num_kv_heads;        /* Hkv */
    int32_t vocab_size;          /* V */
    int32_t kv_max_len;          /* T */
    int32_t kv_batch;            /* B (sequence 0 is decoded) */
    int32_t max_partials;        /* second dimension of the attention intermediates */
    int32_t matvec_reduction_size; /* input-column slice of o-proj / down-proj instructions */

    /* ---- per-token scalars ---- */
    int32_t pos_id;
    float attn_scale;
    float rms_norm_eps;
    int32_t skip_attn_reduction; /* 1: one partition per KV head, PartialAttention writes attn_out (the
                                    reference's only mode); 0: split-KV partials merged by
                                    AttentionReduction instructions; 2: split-KV without reduction
                                    instructions - the PartialAttention of a KV head that arrives last
                                    merges the partial rows itself and signals the o-proj */

    /* ---- extensions without a counterpart in the reference call ---- */
    const int32_t *pos_id_device; /* if not NULL the position is read from this device word at
                                     kernel start (lets one CUDA graph replay every token) */
    float residual_scale;         /* integer factor (as a float) on every o-proj / down-proj output
                                     added to `residual_acc`; 0 means 1.  Tensor-parallel ranks that
                                     exchange through the host set it to the TP degree, sum their
                                     accumulators over ranks and divide by the degree (exact) */
    int64_t *residual_acc;        /* int64 [H], zeroed by the caller before every launch like the
                                     barriers: sum of the token's o-proj / down-proj outputs in
                                     Q31.32 fixed point (value * 2^32), accumulated with integer
                                     atomics, so the result is independent of the order in which
                                     SMs arrive and bit-identical from run to run.  The residual
                                     stream after the launch is hidden_states + residual_acc / 2^32.
                                     Not used (may be NULL) when tp.size > 1; with NULL,
                                     mkb_launch_no_alloc keeps it in its static array */
    int32_t upgate_instructions_per_layer; /* RMS + up/gate instructions per layer in `instructions`
                                     (see MKB_BARRIER_ROW_RMS_READ); 0: down-proj does not wait for
                                     them */

    /* Batched decode (no counterpart in the reference's latency kernel): `batch` independent
     * sequences, 2..MKB_MAX_BATCH, advance by one token in ONE launch that streams the weights
     * once (the sequences' activation vectors are the columns of the MMA's B operand).  Then
     *   - every activation tensor has a leading batch dimension: hidden_states [batch, H],
     *     residual_acc [batch, H], post_ln_rope_q / attn_out [batch, Hq*D], silu_out [batch, I],
     *     logits [batch, V], attn_lse_intermediates [batch, Hq, max_partials],
     *     attn_out_intermediates [batch, Hq, max_partials, D], argmax_out [batch];
     *   - sequence s lives in slot s of the KV cache (kv_batch >= batch) at its own position
     *     pos_ids[s] (or pos_id_device[s]); lengths may differ;
     *   - PartialAttention carries the sequence as a sixth word, AttentionReduction after its
     *     output index, and barriers[layer][1] has one slot per (sequence, Q head):
     *     barrier_width >= batch * Hq;
     *   - the schedule holds one MKB_OP_RMS_NORM per sequence and norm; `normed_states`
     *     (bf16 [batch, H]) receives their output;
     *   - hidden_size <= 4096, tp.size <= 1, not available through mkb_launch_no_alloc.
     * batch 9..MKB_MAX_BATCH runs a third build in which the projections are small-M GEMMs on
     * the tcgen05 tensor cores (blocks of 128 weight rows x the sequences, accumulators in
     * tensor memory, activations streamed per 128-column slice): the schedule's blocks are then
     * 128 rows (every block size of the Python Globals is 128), head_dim must be 128,
     * pos_id_device is required (pos_ids holds 8 entries), and argmax_out is not written.
     * batch 0 or 1: the single-sequence kernel and the layout of the reference. */
    int32_t batch;
    int32_t pos_ids[8];
    void *normed_states;

    MkbTensorParallel tp;         /* in-kernel tensor-parallel all-reduce; tp.size <= 1: off */
    int32_t *argmax_out;          /* if not NULL: device int32 that receives argmax(logits) (smallest
                                     index among equal bf16 maxima, as torch.argmax), computed by the
                                     LM-head epilogue so that the host needs no reduction kernel
                                     (the reference calls torch.argmax, megakernels/generators.py:143).
                                     Valid only for schedules that hold the LM head; ignored by
                                     mkb_launch_no_alloc */

    /* ---- options ---- */
    uint32_t flags;           /* MKB_FLAG_* */
    uint32_t wait_timeout_ms; /* device-side wait budget; 0 selects the default (2000 ms) */
    int32_t *status;          /* MKB_STATUS_WORDS int32 written on device errors, or NULL to use
                                 the library's own per-device buffer */
} MkbGlobals;

/* Device-side error record, MKB_STATUS_WORDS int32. */
typedef struct MkbStatus {
    int32_t code;       /* MKB_OK or the first error raised on the device */
    int32_t sm;         /* queue index of the CTA that raised it */
    int32_t instruction_index;
    int32_t opcode;
    int32_t role;       /* 0 loader, 1 consumer, 2 storer */
    int32_t detail[4];  /* barrier coordinates and the observed / expected values */
    int32_t reserved[7];
} MkbStatus;

/*
 * Validate `g` on the host and enqueue one decode step (one token) on
 * `cuda_stream` (a cudaStream_t; NULL = legacy default stream).  Asynchronous:
 * returns after the launch is enqueued, as the reference call does
 * (megakernels/demos/latency/mk.py:48).  Replaces `mk_llama(...)`.
 */
int mkb_launch(const MkbGlobals *g, void *cuda_stream);

/*
 * Synchronise `cuda_stream` and copy the device status record to `out`.
 * Returns out->code (MKB_OK when the last launches ran clean).  The reference
 * has no counterpart: its device waits are unbounded and a bad opcode traps
 * (include/util.cuh:38).
 */
int mkb_sync_status(const MkbGlobals *g, void *cuda_stream, MkbStatus *out);

/*
 * Check a HOST copy of the instruction tensor ([num_sms, queue_len, 32] int32)
 * against the shapes in `g`: every layer, block range, head and partial index
 * must stay inside its tensor.  Call once per schedule, before the first launch.
 * The reference has no counterpart (a bad schedule hangs or traps its kernel).
 */
int mkb_validate_instructions(const MkbGlobals *g, const int32_t *host_instructions);

/*
 * Same decode step as mkb_launch for callers that cannot allocate: no counterpart in
 * the reference.  Some hosts of this kernel run where cudaMalloc is not an option
 * (all device memory already handed to their own pool, a memory plan fixed before
 * the run, a latency-critical loop), yet mkb_launch allocates a status record on
 * its first call per device and a host-side descriptor cache, and its caller must
 * allocate the split-KV attention scratch.  This variant calls no cudaMalloc,
 * cudaFree or other allocating routine, on the device or on the host: the status
 * record and the attention scratch live in one static device array of
 * MKB_NO_ALLOC_SCRATCH_BYTES that every GPU loading the library holds until exit.
 *
 *  - `g->attn_lse_intermediates` and `g->attn_out_intermediates` are ignored (may be
 *    NULL), and so may `g->residual_acc` (with NULL the accumulators live in the array
 *    too and are cleared by every call); `g->hidden_size`, `g->num_attention_heads`,
 *    `g->max_partials` and `g->head_dim` size the scratch:
 *    256 + roundup256(H * 8) + roundup256(Hq * max_partials * 4) + Hq * max_partials * D * 4
 *    bytes must fit MKB_NO_ALLOC_SCRATCH_BYTES (e.g. H 8192, Hq 64, 24 partials, D 128),
 *    otherwise MKB_ERR_UNSUPPORTED is returned and nothing is launched;
 *  - `g->status` may point at MKB_STATUS_WORDS int32 of caller memory; with NULL the
 *    record is kept inside the static array and cleared on every call.  Either way
 *    mkb_sync_status_no_alloc(g, ...) reads it back without allocating (so does
 *    mkb_sync_status when `g->status` is caller memory; with NULL that function reads
 *    the allocating entry point's own record, which it creates on first use);
 *  - the first call on each device looks up the array's device address and sets a
 *    kernel attribute; make that first call outside any stream capture;
 *  - every call shares the one array and it keeps the previous call's contents: two
 *    calls whose kernels overlap on the GPU (different streams, no ordering) race;
 *  - `g->tp.size` > 1 returns MKB_ERR_UNSUPPORTED (the tensor-parallel exchange needs
 *    peer-mapped buffers, which somebody has to allocate), and `g->argmax_out` is ignored.
 */
#define MKB_NO_ALLOC_SCRATCH_BYTES (1u << 20)
int mkb_launch_no_alloc(const MkbGlobals *g, void *cuda_stream);

/*
 * mkb_sync_status for callers of mkb_launch_no_alloc (no counterpart in the reference):
 * synchronises `cuda_stream` and copies out the record the last no-alloc launch on the
 * current device used - `g->status` if the caller supplied one, otherwise the record in
 * the static array.  Calls no allocator; goes through a buffer on the host stack.
 */
int mkb_sync_status_no_alloc(const MkbGlobals *g, void *cuda_stream, MkbStatus *out);

/*
 * Peer-visible device memory for MkbTensorParallel (no counterpart in the reference).
 * mkb_peer_alloc: cudaMalloc + zero-fill of `bytes` on the current device and an opaque
 * 64-byte handle another process can open; mkb_peer_open maps such a handle into the
 * calling process for the current device (peer access is enabled on demand);
 * mkb_peer_close / mkb_peer_free undo them.  The handle travels by whatever channel the
 * host has (a torch.distributed all-gather in this repository).
 */
#define MKB_PEER_HANDLE_BYTES 64
int mkb_peer_alloc(size_t bytes, void **device_ptr, unsigned char handle[MKB_PEER_HANDLE_BYTES]);
int mkb_peer_open(const unsigned char handle[MKB_PEER_HANDLE_BYTES], void **device_ptr);
int mkb_peer_close(void *device_ptr);
int mkb_peer_free(void *device_ptr);

/* Message of the last host-side error raised on the calling thread. */
const char *mkb_last_error(void);

/* Number of SMs of the current CUDA device (megakernels/utils.py:107-109). */
int mkb_sm_count(void);

/* Dynamic shared memory in bytes the kernel asks for, and its block size. */
int mkb_smem_bytes(void);
int mkb_block_threads(void);

/* ABI version the library was built with. */
int mkb_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MKB200_H */
