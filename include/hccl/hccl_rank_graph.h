/*
 * hccl_rank_graph.h - topology queries (reference: include/hccl/hccl_rank_graph.h:38-380).
 *
 * On a B200 NVSwitch box the graph has one net layer (0) with one instance that contains every
 * rank, topology COMM_TOPO_1DMESH, and one NVLINK link per ordered rank pair whose hop count is 2
 * (GPU -> NVSwitch -> GPU).  Jobs described by a multi-level rank table keep their extra layers.
 * Arrays returned through ** are owned by the communicator and stay valid until it is destroyed.
 */
#ifndef HCCL_RANK_GRAPH_H
#define HCCL_RANK_GRAPH_H

#include "hccl_res.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ENDPOINT_ATTR_INVALID = -1,
    ENDPOINT_ATTR_BW_COEFF = 0, /* active NVLink links of the port group */
    ENDPOINT_ATTR_DIE_ID = 1,
    ENDPOINT_ATTR_LOCATION = 2
} EndpointAttr;
typedef uint32_t EndpointAttrBwCoeff;
typedef uint32_t EndpointAttrDieId;
typedef uint32_t EndpointAttrLocation;

typedef enum {
    COMM_TOPO_RESERVED = -1,
    COMM_TOPO_CLOS = 0,
    COMM_TOPO_1DMESH = 1,
    COMM_TOPO_910_93 = 2,
    COMM_TOPO_310P = 3,
    COMM_TOPO_A2AXSERVER = 4,
    COMM_TOPO_CUSTOM = 5
} CommTopo;

typedef enum {
    HCCL_HETEROG_MODE_INVALID = -1,
    HCCL_HETEROG_MODE_HOMOGENEOUS = 0,
    HCCL_HETEROG_MODE_MIX_A2_A3
} HcclHeterogMode;

#define COMM_LINK_MAGIC_WORD 0x0f0e0f0fu
#define COMM_LINK_VERSION 1u

typedef struct {
    CommAbiHeader header;
    EndpointDesc srcEndpointDesc;
    EndpointDesc dstEndpointDesc;
    union {
        uint8_t raws[128];
        struct {
            CommProtocol linkProtocol;
            uint8_t hop;
        };
    } linkAttr;
} CommLink;

static inline HcclResult CommLinkInit(CommLink *link, uint32_t linkNum)
{
    if (link == NULL) {
        return HCCL_E_PTR;
    }
    for (uint32_t i = 0; i < linkNum; ++i, ++link) {
        memset(link, 0xFF, sizeof(*link));
        link->header.version = COMM_LINK_VERSION;
        link->header.magicWord = COMM_LINK_MAGIC_WORD;
        link->header.size = (uint32_t)sizeof(*link);
        link->header.reserved = 0;
        (void)EndpointDescInit(&link->srcEndpointDesc, 1);
        (void)EndpointDescInit(&link->dstEndpointDesc, 1);
        link->linkAttr.linkProtocol = COMM_PROTOCOL_RESERVED;
        link->linkAttr.hop = 1;
    }
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetLayers(HcclComm comm, uint32_t **netLayers, uint32_t *netLayerNum);
HcclResult HcclRankGraphGetRanksByLayer(HcclComm comm, uint32_t netLayer, uint32_t **ranks, uint32_t *rankNum);
HcclResult HcclRankGraphGetRankSizeByLayer(HcclComm comm, uint32_t netLayer, uint32_t *rankNum);
HcclResult HcclRankGraphGetTopoTypeByLayer(HcclComm comm, uint32_t netLayer, CommTopo *topoType);
HcclResult HcclRankGraphGetInstSizeListByLayer(HcclComm comm, uint32_t netLayer, uint32_t **instSizeList,
                                               uint32_t *listSize);
HcclResult HcclRankGraphGetLinks(HcclComm comm, uint32_t netLayer, uint32_t srcRank, uint32_t dstRank,
                                 CommLink **links, uint32_t *linkNum);
HcclResult HcclRankGraphGetTopoInstsByLayer(HcclComm comm, uint32_t netLayer, uint32_t **topoInsts,
                                            uint32_t *topoInstNum);
HcclResult HcclRankGraphGetTopoType(HcclComm comm, uint32_t netLayer, uint32_t topoInstId, CommTopo *topoType);
HcclResult HcclRankGraphGetRanksByTopoInst(HcclComm comm, uint32_t netLayer, uint32_t topoInstId, uint32_t **ranks,
                                           uint32_t *rankNum);
HcclResult HcclGetHeterogMode(HcclComm comm, HcclHeterogMode *mode);
HcclResult HcclRankGraphGetEndpointNum(HcclComm comm, uint32_t layer, uint32_t topoInstId, uint32_t *num);
HcclResult HcclRankGraphGetEndpointDesc(HcclComm comm, uint32_t layer, uint32_t topoInstId, uint32_t *descNum,
                                        EndpointDesc *endpointDesc);
HcclResult HcclRankGraphGetEndpointInfo(HcclComm comm, uint32_t rankId, const EndpointDesc *endpointDesc,
                                        EndpointAttr endpointAttr, uint32_t infoLen, void *info);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_RANK_GRAPH_H */
