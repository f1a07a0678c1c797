// The batched build of the decode megakernel: the same source compiled for up to 8
// independent sequences per launch (MKB_BATCH in mk_common.cuh says what changes), and the
// host-side launcher the C ABI calls for MkbGlobals.batch > 1.  No counterpart in the
// reference, whose latency kernel decodes one sequence and whose batched instruction set
// needs batches that are multiples of 128 (megakernels/demos/throughput/instructions.py:30-31).
#define MKB_BATCH 8
#include "megakernel.cu"

#include <cstring>

namespace mkb_batched {

int max_batch() { return kBatch; }
int smem_bytes() { return kSmemAlloc; }

// `params` are the bytes of the single-sequence build's KParams: both builds declare the
// same struct, only the constants around it differ.
cudaError_t launch(const void* params, size_t params_bytes, int grid, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (params_bytes != sizeof(KParams) || dev < 0 || dev >= 64) return cudaErrorInvalidValue;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(megakernel_batched, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    KParams p;
    memcpy(&p, params, sizeof(p));
    megakernel_batched<<<grid, kBlockThreads, kSmemAlloc, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace mkb_batched
