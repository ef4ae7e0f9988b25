// rank_graph_api.cc - C queries over the communicator's RankGraph (include/hccl/hccl_rank_graph.h;
// reference adapters: api_c_adpt/coll_comm_rank_graph_a_adpt.cc:63-386).
#include <cstring>

#include "../comm/comm.h"
#include "../core/log.h"
#include "hccl/hccl_rank_graph.h"

using namespace hc;

namespace {
// Arrays handed to C callers live as long as the communicator.
uint32_t *Keep(Comm *c, const std::vector<uint32_t> &v)
{
    c->graph.scratchU32.push_back(v);
    if (c->graph.scratchU32.size() > 4096) c->graph.scratchU32.erase(c->graph.scratchU32.begin(), c->graph.scratchU32.begin() + 2048);
    return c->graph.scratchU32.back().data();
}
bool HasLayer(Comm *c, uint32_t layer)
{
    for (uint32_t l : c->graph.Layers())
        if (l == layer) return true;
    return false;
}
}  // namespace

extern "C" {

HcclResult HcclRankGraphGetLayers(HcclComm comm, uint32_t **netLayers, uint32_t *netLayerNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(netLayers); CHK_PTR_NULL(netLayerNum);
    *netLayers = Keep(c, c->graph.Layers());
    *netLayerNum = (uint32_t)c->graph.Layers().size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetRanksByLayer(HcclComm comm, uint32_t netLayer, uint32_t **ranks, uint32_t *rankNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ranks); CHK_PTR_NULL(rankNum);
    const NetInstance *ni = c->graph.InstanceOf(netLayer, c->rank);
    if (!ni) { RPT_ERR("EI0003", "net layer %u does not exist for rank %u", netLayer, c->rank); return HCCL_E_PARA; }
    *ranks = Keep(c, ni->ranks);
    *rankNum = (uint32_t)ni->ranks.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetRankSizeByLayer(HcclComm comm, uint32_t netLayer, uint32_t *rankNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(rankNum);
    const NetInstance *ni = c->graph.InstanceOf(netLayer, c->rank);
    if (!ni) return HCCL_E_PARA;
    *rankNum = (uint32_t)ni->ranks.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetTopoTypeByLayer(HcclComm comm, uint32_t netLayer, CommTopo *topoType)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(topoType);
    const NetInstance *ni = c->graph.InstanceOf(netLayer, c->rank);
    if (!ni) return HCCL_E_PARA;
    *topoType = ni->topo;
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetInstSizeListByLayer(HcclComm comm, uint32_t netLayer, uint32_t **instSizeList, uint32_t *listSize)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(instSizeList); CHK_PTR_NULL(listSize);
    if (!HasLayer(c, netLayer)) return HCCL_E_PARA;
    std::vector<uint32_t> sizes;
    for (auto &ni : c->graph.Instances(netLayer)) sizes.push_back((uint32_t)ni.ranks.size());
    *instSizeList = Keep(c, sizes);
    *listSize = (uint32_t)sizes.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetLinks(HcclComm comm, uint32_t netLayer, uint32_t srcRank, uint32_t dstRank, CommLink **links, uint32_t *linkNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(links); CHK_PTR_NULL(linkNum);
    std::vector<GraphLink> gl;
    CHK_RET(c->graph.Links(netLayer, srcRank, dstRank, &gl));
    std::vector<CommLink> out(gl.size());
    for (size_t i = 0; i < gl.size(); ++i) {
        CommLinkInit(&out[i], 1);
        c->graph.EndpointDescOf(netLayer, gl[i].src, &out[i].srcEndpointDesc);
        c->graph.EndpointDescOf(netLayer, gl[i].dst, &out[i].dstEndpointDesc);
        memset(out[i].linkAttr.raws, 0, sizeof(out[i].linkAttr.raws));
        out[i].linkAttr.linkProtocol = gl[i].protocol;
        out[i].linkAttr.hop = gl[i].hop;
    }
    c->graph.scratchLinks.push_back(out);
    if (c->graph.scratchLinks.size() > 1024) c->graph.scratchLinks.erase(c->graph.scratchLinks.begin(), c->graph.scratchLinks.begin() + 512);
    *links = c->graph.scratchLinks.back().data();
    *linkNum = (uint32_t)out.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetTopoInstsByLayer(HcclComm comm, uint32_t netLayer, uint32_t **topoInsts, uint32_t *topoInstNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(topoInsts); CHK_PTR_NULL(topoInstNum);
    if (!HasLayer(c, netLayer)) return HCCL_E_PARA;
    std::vector<uint32_t> ids;
    for (auto &ni : c->graph.Instances(netLayer)) ids.push_back(ni.topoInstId);
    *topoInsts = Keep(c, ids);
    *topoInstNum = (uint32_t)ids.size();
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetTopoType(HcclComm comm, uint32_t netLayer, uint32_t topoInstId, CommTopo *topoType)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(topoType);
    for (auto &ni : c->graph.Instances(netLayer))
        if (ni.topoInstId == topoInstId) { *topoType = ni.topo; return HCCL_SUCCESS; }
    return HCCL_E_PARA;
}

HcclResult HcclRankGraphGetRanksByTopoInst(HcclComm comm, uint32_t netLayer, uint32_t topoInstId, uint32_t **ranks, uint32_t *rankNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ranks); CHK_PTR_NULL(rankNum);
    for (auto &ni : c->graph.Instances(netLayer))
        if (ni.topoInstId == topoInstId) { *ranks = Keep(c, ni.ranks); *rankNum = (uint32_t)ni.ranks.size(); return HCCL_SUCCESS; }
    return HCCL_E_PARA;
}

HcclResult HcclGetHeterogMode(HcclComm comm, HcclHeterogMode *mode)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(mode);
    *mode = HCCL_HETEROG_MODE_HOMOGENEOUS;
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetEndpointNum(HcclComm comm, uint32_t layer, uint32_t topoInstId, uint32_t *num)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(num);
    for (auto &ni : c->graph.Instances(layer))
        if (ni.topoInstId == topoInstId) { *num = std::binary_search(ni.ranks.begin(), ni.ranks.end(), c->rank) ? 1u : 0u; return HCCL_SUCCESS; }
    return HCCL_E_PARA;
}

// The local rank's endpoints inside the given topology instance (one NVLink port group per GPU).
HcclResult HcclRankGraphGetEndpointDesc(HcclComm comm, uint32_t layer, uint32_t topoInstId, uint32_t *descNum, EndpointDesc *endpointDesc)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(descNum); CHK_PTR_NULL(endpointDesc);
    uint32_t have = 0;
    CHK_RET(HcclRankGraphGetEndpointNum(comm, layer, topoInstId, &have));
    if (*descNum < have) return HCCL_E_PARA;
    if (have) CHK_RET(c->graph.EndpointDescOf(layer, c->rank, endpointDesc));
    *descNum = have;
    return HCCL_SUCCESS;
}

HcclResult HcclRankGraphGetEndpointInfo(HcclComm comm, uint32_t rankId, const EndpointDesc *endpointDesc, EndpointAttr endpointAttr, uint32_t infoLen, void *info)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(endpointDesc); CHK_PTR_NULL(info);
    if (rankId >= c->nRanks || infoLen < sizeof(uint32_t)) return HCCL_E_PARA;
    uint32_t v;
    switch (endpointAttr) {
        case ENDPOINT_ATTR_BW_COEFF: v = c->table.ranks[rankId].nvlinkCount ? c->table.ranks[rankId].nvlinkCount : 18; break;
        case ENDPOINT_ATTR_DIE_ID: v = 0; break;
        case ENDPOINT_ATTR_LOCATION: v = (uint32_t)ENDPOINT_LOC_TYPE_DEVICE; break;
        default: return HCCL_E_PARA;
    }
    memcpy(info, &v, sizeof(v));
    return HCCL_SUCCESS;
}

}  // extern "C"
