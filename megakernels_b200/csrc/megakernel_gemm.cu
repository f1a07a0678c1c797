// The GEMM build of the decode megakernel: the same source compiled for 9..64 independent
// sequences per launch, with the projections as small-M GEMMs on the tcgen05 tensor cores
// (MKB_BATCH in mk_common.cuh says what changes), and the host-side launcher the C ABI calls
// for MkbGlobals.batch > 8.  No counterpart in the reference: its batched instruction set needs
// batches that are multiples of 128 (megakernels/demos/throughput/instructions.py:30-31).
#define MKB_BATCH 64
#include "megakernel.cu"

#include <cstring>

namespace mkb_gemm {

int max_batch() { return kBatch; }
int block_rows() { return kBlockRows; }
int stage_cols() { return kStageCols; }

cudaError_t launch(const void* params, size_t params_bytes, int grid, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (params_bytes != sizeof(KParams) || dev < 0 || dev >= 64) return cudaErrorInvalidValue;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(megakernel_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    KParams p;
    memcpy(&p, params, sizeof(p));
    megakernel_gemm<<<grid, kBlockThreads, kSmemAlloc, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace mkb_gemm
