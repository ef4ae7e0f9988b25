/* hcomm_fused.h - compute operators of the library: the tcgen05 bf16 GEMM, the tensor-parallel GEMMs fused with
 * their collective, and the phase clocks of the fused kernels.  (The MoE dispatch / combine exchange is declared in
 * hcomm_moe.h.)
 *
 * Matrices are bf16, row-major with the last dimension contiguous; B / W are given as [N, K] ("TN" product
 * C = A * B^T); accumulation is fp32.  `stream` is a cudaStream_t.  All functions return an HcclResult value.
 * The reference library has no compute operators; its nearest relative is the matmul + collective handshake server
 * (framework/device/aicpu_kfc/).
 */
#ifndef HCOMM_FUSED_H
#define HCOMM_FUSED_H

#include <stdint.h>

#include "hccl/hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* How a GEMM + collective operator runs. */
#define HCOMM_FUSED_MODE_AUTO 0  /* the library's choice; HCOMM_FUSED_MODE=fused|split overrides it */
#define HCOMM_FUSED_MODE_FUSED 1 /* one kernel: tiles travel while other tiles are computed */
#define HCOMM_FUSED_MODE_SPLIT 2 /* two launches of the library's own kernels (collective kernel + GEMM) */

/* C[M,N] = A[M,K] * B[N,K]^T on the current device.  N, K and ldc multiples of 8, C 16-byte aligned. */
int HcommGemmBf16(const void *A, const void *B, void *C, int M, int N, int K, int lda, int ldb, int ldc, void *stream);
/* Tuning overrides of the CTA-pair GEMM kernels (0 = automatic): rasterisation group in 256-row blocks, tile width (128..256, multiple of 32). */
void HcommGemmSetTuning(int groupRows, int tileWidth);
/* With HCOMM_GEMM_AUTOTUNE=1, large shapes (2 * M * N * K >= 2e11) seen for the first time are timed once with the candidate
 * tile widths and groups on the caller's stream (not while it is being captured) and the fastest is kept for the process.
 * Returns what was chosen for a shape, 0 / 0 if nothing was measured. */
void HcommGemmGetTuned(int M, int N, int K, int *tileWidth, int *groupRows);
/* Reads and clears the "a bounded wait expired inside a GEMM kernel" flag of the current device (0 = none). */
int HcommGemmTakeError(void);

/* Row-parallel linear: every rank holds a K slice, A [M, K_local] and B [N, K_local]; rank r receives rows
 * [r * M / size, (r + 1) * M / size) of the sum over ranks of A * B^T in out [M / size, N].
 * M a multiple of 128 * size, N of 128, K of 8. */
int HcommFusedGemmReduceScatterBf16(HcclComm comm, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut,
                                    void *stream);
int HcommFusedGemmReduceScatterBf16Mode(HcclComm comm, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut,
                                        void *stream, int mode);
/* Column-parallel linear: x is this rank's contiguous shard [Mshard, K] of the activations, W [N_local, K];
 * out [Mshard * size, N_local] = all_gather(x) * W^T.  Mshard a multiple of 128, N of 128, K of 8. */
int HcommFusedAllGatherGemmBf16(HcclComm comm, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut,
                                void *stream);
int HcommFusedAllGatherGemmBf16Mode(HcclComm comm, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut,
                                    void *stream, int mode);

/* Phase clocks of the CTA-pair fused kernels.  When on, every fused call records eight 64-bit words per CTA
 * (nanoseconds of the GPU's global timer): 0 start, 1 end, 2 time the TMA producer waited for rows from other
 * ranks, 3 time the epilogue waited for an accumulator, 4 time it waited for the peers' partial tiles, 5 duration of
 * the CTA's share of the all-gather push, 6 time stamp of the end of that push, 7 time inside fences and signals.
 * Read them after synchronising the stream of the call. */
int HcommFusedSetPhaseClocks(HcclComm comm, int on);
int HcommFusedGetPhaseClocks(HcclComm comm, uint64_t *words, int maxCtas, int *ctas);

#ifdef __cplusplus
}
#endif
#endif
