// mkb_launch_no_alloc: the decode step for callers that must not allocate.
//
// Who needs this: code that runs where cudaMalloc is off limits - inside a
// stream-ordered region whose memory was planned up front, in a process that
// handed all device memory to its own pool, or in a real-time loop where an
// allocation (and the device synchronisation it can imply) is not acceptable.
// mkb_launch allocates twice: a 64-byte status record per device on its first
// call, and host memory for its descriptor cache.  The caller of the reference
// interface additionally has to allocate the split-KV attention scratch
// (`attn_lse_intermediates`, `attn_out_intermediates`).  This entry point needs
// none of that: the scratch and the status record live in one file-scope
// `__device__` array that every GPU loading this library holds until exit.
#include <cstring>
#include <mutex>

#include "mk_common.cuh"

namespace mkb {
__global__ void megakernel(const __grid_constant__ KParams p);
int prepare_launch_uncached(const MkbGlobals* g, int* status, int sm_count, KParams& p);
int set_error(int code, const char* msg);
int read_status_record(int* st, void* cuda_stream, MkbStatus* out);
std::mutex& library_mutex();
}  // namespace mkb

using namespace mkb;

namespace {

// [0, 256): status record (MKB_STATUS_WORDS int32, padded)
// then ACC  [H] int64 residual accumulators (cleared on every call; only when the caller passes none)
// then LSE  [Hq][max_partials] fp32, rounded up to 256 bytes
// then O    [Hq][max_partials][D] fp32
constexpr size_t kStatusBytes = 256;
static __device__ __align__(256) unsigned char g_static_scratch[MKB_NO_ALLOC_SCRATCH_BYTES];

struct PerDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // DEVICE address of g_static_scratch on this device
    int sm_count = 0;
};
PerDevice g_per_device[64];

size_t round256(size_t n) { return (n + 255) & ~size_t(255); }

// In host code `g_static_scratch` is only a stand-in for the symbol, not a device
// address; the address each device uses must be asked for, once, with that device
// current.  Nothing here allocates: the array is part of the loaded module.  The caller
// holds the library mutex (two host threads may make the first call on a device together).
int setup_device(int dev, PerDevice** out) {
    PerDevice& pd = g_per_device[dev];
    if (!pd.ready) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return set_error(MKB_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed");
        e = cudaFuncSetAttribute(megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
        if (e != cudaSuccess) return set_error(MKB_ERR_CUDA, "cudaFuncSetAttribute failed");
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return set_error(MKB_ERR_CUDA, "cudaDeviceGetAttribute failed");
        pd.scratch = static_cast<unsigned char*>(ptr);
        pd.sm_count = n;
        pd.ready = true;
    }
    *out = &pd;
    return MKB_OK;
}

}  // namespace

extern "C" int mkb_launch_no_alloc(const MkbGlobals* g, void* cuda_stream) {
    if (!g) return set_error(MKB_ERR_INVALID_ARGUMENT, "globals pointer is NULL");
    // the two leading words say how much of *g may be read at all: check them before anything else
    if (g->abi_version != MKB_ABI_VERSION || g->struct_bytes != sizeof(MkbGlobals))
        return set_error(MKB_ERR_INVALID_ARGUMENT,
                         "abi_version / struct_bytes do not match this library's MkbGlobals");
    std::lock_guard<std::mutex> lock(library_mutex());
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return set_error(MKB_ERR_CUDA, "cudaGetDevice failed");
    PerDevice* pd = nullptr;
    int rc = setup_device(dev, &pd);
    if (rc) return rc;

    if (g->tp.size > 1)
        return set_error(MKB_ERR_UNSUPPORTED, "mkb_launch_no_alloc has no tensor-parallel variant");
    if (g->batch > 1)
        return set_error(MKB_ERR_UNSUPPORTED, "mkb_launch_no_alloc decodes one sequence per launch");
    if (g->num_attention_heads < 1 || g->max_partials < 1 || g->head_dim < 1)
        return set_error(MKB_ERR_INVALID_ARGUMENT,
                         "num_attention_heads, max_partials and head_dim must be positive");
    if (g->hidden_size < 1)
        return set_error(MKB_ERR_INVALID_ARGUMENT, "hidden_size must be positive");
    const size_t acc_bytes = g->residual_acc ? 0 : round256((size_t)g->hidden_size * 8);
    const size_t lse_bytes = round256((size_t)g->num_attention_heads * g->max_partials * 4);
    const size_t o_bytes = (size_t)g->num_attention_heads * g->max_partials * g->head_dim * 4;
    if (kStatusBytes + acc_bytes + lse_bytes + o_bytes > (size_t)MKB_NO_ALLOC_SCRATCH_BYTES)
        return set_error(MKB_ERR_UNSUPPORTED,
                         "mkb_launch_no_alloc: attention scratch for Hq x max_partials x head_dim "
                         "exceeds the built-in MKB_NO_ALLOC_SCRATCH_BYTES; lower max_partials or "
                         "use mkb_launch with caller-allocated intermediates");

    MkbGlobals local;
    memcpy(&local, g, sizeof(local));
    if (!g->residual_acc) local.residual_acc = reinterpret_cast<int64_t*>(pd->scratch + kStatusBytes);
    local.attn_lse_intermediates = reinterpret_cast<float*>(pd->scratch + kStatusBytes + acc_bytes);
    local.attn_out_intermediates = reinterpret_cast<float*>(pd->scratch + kStatusBytes + acc_bytes + lse_bytes);
    int* status = g->status ? g->status : reinterpret_cast<int*>(pd->scratch);

    KParams p;
    rc = prepare_launch_uncached(&local, status, pd->sm_count, p);
    if (rc) return rc;
    // The array keeps whatever the previous call left.  The built-in status record and the
    // residual accumulators must start at zero; the attention scratch is always written
    // before it is read.
    if (!g->status) {
        cudaError_t e = cudaMemsetAsync(pd->scratch, 0, kStatusBytes, (cudaStream_t)cuda_stream);
        if (e != cudaSuccess) return set_error(MKB_ERR_CUDA, "cudaMemsetAsync(status) failed");
    }
    if (acc_bytes) {
        cudaError_t e = cudaMemsetAsync(pd->scratch + kStatusBytes, 0, acc_bytes, (cudaStream_t)cuda_stream);
        if (e != cudaSuccess) return set_error(MKB_ERR_CUDA, "cudaMemsetAsync(residual accumulators) failed");
    }
    megakernel<<<local.num_sms, kBlockThreads, kSmemAlloc, (cudaStream_t)cuda_stream>>>(p);
    if (cudaGetLastError() != cudaSuccess) return set_error(MKB_ERR_CUDA, "kernel launch failed");
    return MKB_OK;
}

// Read-back for mkb_launch_no_alloc, equally free of allocations: the record the last call on
// this device wrote - `g->status` when the caller passed one, else the one inside the static
// array (which only exists once mkb_launch_no_alloc has run on this device).
extern "C" int mkb_sync_status_no_alloc(const MkbGlobals* g, void* cuda_stream, MkbStatus* out) {
    if (!out) return set_error(MKB_ERR_INVALID_ARGUMENT, "status output pointer is NULL");
    std::lock_guard<std::mutex> lock(library_mutex());
    int* st = (g && g->status) ? g->status : nullptr;
    if (!st) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
            return set_error(MKB_ERR_CUDA, "cudaGetDevice failed");
        if (!g_per_device[dev].ready)
            return set_error(MKB_ERR_INVALID_ARGUMENT,
                             "mkb_launch_no_alloc has not run on this device: no built-in status record");
        st = reinterpret_cast<int*>(g_per_device[dev].scratch);
    }
    return read_status_record(st, cuda_stream, out);
}
