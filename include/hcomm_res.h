/*
 * hcomm_res.h - base resources: endpoints, registered memory, execution threads, device memory.
 * (reference: include/hcomm_res.h)
 *
 * Endpoint  = one GPU's NVLink port group (or the host, for the simulator).
 * Memory    = a range registered with an endpoint; exporting it yields a byte descriptor a peer
 *             imports to obtain a pointer it can load from / store to directly.
 * Thread    = an ordered execution context (a CUDA stream on CPU_TS, one CTA slot on the SM
 *             engine) with N local notify slots.
 */
#ifndef HCOMM_RES_H
#define HCOMM_RES_H

#include "hcomm_channel.h"
#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

HcommResult HcommEndpointCreate(const EndpointDesc *endpoint, EndpointHandle *handle);
HcommResult HcommEndpointDestroy(EndpointHandle handle);
HcommResult HcommEndpointGetDescNum(int32_t deviceLogicId, uint32_t *descNum);
HcommResult HcommEndpointGetDescs(int32_t deviceLogicId, uint32_t *descNum, EndpointDesc *descs);
HcommResult HcommEndpointGetListenPort(EndpointHandle handle, uint32_t *port);
HcommResult HcommEndpointCheckFeature(HcommEndpointFeatureType feature, const EndpointDesc *desc, bool *value);

HcommResult HcommMemReg(EndpointHandle handle, const char *memTag, const CommMem *mem, HcommMemHandle *memHandle);
HcommResult HcommMemUnreg(EndpointHandle handle, HcommMemHandle memHandle);
/* *memDesc points at library-owned bytes that stay valid until HcommMemUnreg. */
HcommResult HcommMemExport(EndpointHandle handle, HcommMemHandle memHandle, void **memDesc, uint32_t *memDescLen);
HcommResult HcommMemImport(EndpointHandle handle, const void *memDesc, uint32_t descLen, CommMem *outMem);
HcommResult HcommMemUnimport(EndpointHandle handle, const void *memDesc, uint32_t descLen);

HcommResult HcommThreadAlloc(CommEngine engine, uint32_t threadNum, const uint32_t *notifyNumPerThread,
                             ThreadHandle *threads);
HcommResult HcommThreadFree(const ThreadHandle *threads, uint32_t threadNum);
HcommResult HcommThreadResGetInfo(ThreadHandle thread, ThreadResType resType, uint32_t infoLen, void **info);

/* Device memory that can be exported to peers (VMM-backed on CUDA, memfd-backed on the simulator). */
HcommResult HcommMemAlloc(void **ptr, size_t size);
HcommResult HcommMemFree(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* HCOMM_RES_H */
