/* hccl_sym_win.h - address of a symmetric window on another rank (reference: include/hccl/hccl_sym_win.h). */
#ifndef HCCL_SYM_WIN_H
#define HCCL_SYM_WIN_H
#include "hccl_types.h"
#ifdef __cplusplus
extern "C" {
#endif
/* *ptr is valid in the caller's address space: loads and stores through it travel over NVLink. */
HcclResult HcclSymWinGetPeerPointer(HcclCommSymWindow winHandle, size_t offset, uint32_t peerRank, void **ptr);
/* B200 extension: the NVLS multicast alias of the window (NULL when multicast is unavailable). */
HcclResult HcclSymWinGetMulticastPointer(HcclCommSymWindow winHandle, size_t offset, void **ptr);
#ifdef __cplusplus
}
#endif
#endif
