#include "algo_plugin.h"
#include <dlfcn.h>
#include <cstddef>
#include <cstring>
#include <mutex>
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "../topo/topo.h"
#include "config.h"
#include "log.h"

namespace hccl {
namespace {
std::mutex g_mu;
bool g_tried = false;
void* g_handle = nullptr;
const HcclAlgoPluginTable* g_table = nullptr;

const HcclAlgoPluginTable* Table()
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_tried) return g_table;
    g_tried = true;
    const std::string& path = GetEnvConfig().algoPlugin;
    if (path.empty()) return nullptr;
    g_handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!g_handle) { HCCL_WARNING("algorithm plugin '%s' cannot be loaded (%s): built-in algorithms only", path.c_str(), dlerror()); return nullptr; }
    using GetFn = const HcclAlgoPluginTable* (*)();
    GetFn get = (GetFn)dlsym(g_handle, "GetHcclAlgoPlugin");
    const HcclAlgoPluginTable* t = get ? get() : nullptr;
    if (!t || t->magic != HCCL_ALGO_PLUGIN_TABLE_MAGIC || t->apiVersion != HCCL_PLUGIN_API_VERSION || t->structSize < offsetof(HcclAlgoPluginTable, QueryAlgs) ||
        !t->SelectAlg || !t->ExecuteAlg) {
        HCCL_WARNING("algorithm plugin '%s': missing GetHcclAlgoPlugin, wrong version or incomplete table: ignored", path.c_str());
        dlclose(g_handle);
        g_handle = nullptr;
        return nullptr;
    }
    g_table = t;
    HCCL_INFO("algorithm plugin '%s' loaded", path.c_str());
    return g_table;
}
}  // namespace

void AlgoPluginReload()
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_handle) dlclose(g_handle);
    g_handle = nullptr;
    g_table = nullptr;
    g_tried = false;
}

bool AlgoPluginTryExecute(CommImpl* comm, const OpParam& p, HcclResult* result, std::string* algName)
{
    const HcclAlgoPluginTable* t = Table();
    if (!t || (t->IsReady && !t->IsReady())) return false;
    HcclAlgoPluginParam q;
    memset(&q, 0, sizeof(q));
    q.version = 1;
    q.magic = HCCL_ALGO_PLUGIN_PARAM_MAGIC;
    q.structSize = sizeof(q);
    q.opType = (int)p.op;
    snprintf(q.opName, sizeof(q.opName), "%s", CmdName(p.op));
    q.count = p.count;
    q.root = p.root;
    static const char* shapes[] = {"MESH_1D", "CLOS", "MESH_1D_CLOS", "RING", "SINGLE"};
    snprintf(q.topoName, sizeof(q.topoName), "%s", comm->topo ? shapes[(int)comm->topo->level0] : "MESH_1D");
    q.rankNum = (uint32_t)comm->nRanks;
    q.rank = (uint32_t)comm->rank;
    q.serverNum = comm->topo ? comm->topo->nServers : 1;
    q.sendBuf = const_cast<void*>(p.send);
    q.recvBuf = p.recv;
    q.stream = (hcclStream_t)p.stream;
    q.comm = (HcclComm)comm;
    q.dataType = p.dtype;
    q.reduceOp = p.redOp;
    q.remoteRank = p.root;
    q.deviceNumPerModule = comm->topo && !comm->topo->serverSizes.empty() ? comm->topo->serverSizes[0] : (uint32_t)comm->nRanks;
    q.isAsymmetricTopo = comm->topo ? !comm->topo->symmetric : false;
    char name[HCCL_ALGO_PLUGIN_ALG_NAME_LEN] = {0};
    if (t->SelectAlg(&q, name) != HCCL_SUCCESS || name[0] == 0) return false;
    *algName = name;
    *result = t->ExecuteAlg(name, &q);
    if (*result != HCCL_SUCCESS) HCCL_ERROR("algorithm plugin: %s failed in %s: %s", name, q.opName, ResultString(*result));
    return true;
}

HcclResult AlgoPluginQueryAlgs(const char* opName, char* buf, uint32_t bufLen, uint32_t* count)
{
    if (!buf || !count || bufLen == 0) return HCCL_E_PTR;
    *count = 0;
    buf[0] = 0;
    const HcclAlgoPluginTable* t = Table();
    if (!t) return HCCL_E_NOT_FOUND;
    if (t->structSize < sizeof(HcclAlgoPluginTable) || !t->QueryAlgs) return HCCL_E_NOT_SUPPORT;
    const int n = t->QueryAlgs(opName ? opName : "", buf, bufLen);
    if (n < 0) return HCCL_E_MEMORY;
    *count = (uint32_t)n;
    return HCCL_SUCCESS;
}

}  // namespace hccl
