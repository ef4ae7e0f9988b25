// gemm_api.h - host entry points of the tcgen05 GEMM family.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "hccl/hccl_types.h"

namespace hc {

// Tiled, 128-byte swizzled tensor map over a row-major bf16 matrix (cols contiguous, pitch ldElems).
HcclResult MakeTensorMap2dBf16(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ldElems, uint32_t boxRows, uint32_t boxCols);
// C[M,N] = A[M,K] * B[N,K]^T, bf16 in / bf16 out, fp32 accumulation in tensor memory.
HcclResult GemmBf16(const void *A, const void *B, void *C, int M, int N, int K, int lda, int ldb, int ldc, void *stream);
int GemmSmCount();
// Tile width (256, 224, 192, 160 or 128, a divisor of N) of the CTA-pair kernels with the least work in whole waves.
int PickPairTileWidth(int rowBlocks256, int N, int pairs);
int PairGroupRows(int K);        // rasterisation group of the CTA-pair kernels (row blocks of 256 rows)
int ForcedPairTileWidth();       // HCOMM_GEMM_BN / HcommGemmSetTuning, 0 = automatic
uint32_t *GemmErrorFlag();

}  // namespace hc
