// Algorithm plugin ABI: a shared object named by HCCL_ALGO_PLUGIN_PATH may take
// over the execution of an operator.
//
// Behaviour follows HCCL's plugin broker (src/algo_plugin/hccl_algo_plugin_mgr.cc,
// parameter block src/algo_plugin/inc/hccl_algo_plugin_common.h:76-107; hook
// sites op_common.cc:116-172, :1275-1281): the library asks SelectAlg for every
// call; when the plugin claims the call (returns HCCL_SUCCESS and a name)
// ExecuteAlg fully replaces the built-in execution; any other answer falls
// through to the built-in selector.  The plugin exports `GetHcclAlgoPlugin`.
#ifndef HCCL_B200_ALGO_PLUGIN_H_
#define HCCL_B200_ALGO_PLUGIN_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_PLUGIN_API_VERSION 1u
#define HCCL_ALGO_PLUGIN_PARAM_MAGIC 0x48415050u
#define HCCL_ALGO_PLUGIN_TABLE_MAGIC 0x48415054u
#define HCCL_ALGO_PLUGIN_ALG_NAME_LEN 128u

typedef struct {
    uint32_t version;
    uint32_t magic;
    uint32_t structSize;
    int opType;                 /* HcclCMDType */
    char opName[32];            /* "AllReduce", ... : plugins should key on the name */
    uint64_t count;
    uint32_t root;
    char topoName[32];          /* "MESH_1D", "CLOS", ... */
    uint32_t rankNum;
    uint32_t rank;
    uint32_t serverNum;
    void* sendBuf;
    void* recvBuf;
    hcclStream_t stream;
    HcclComm comm;
    HcclDataType dataType;
    HcclReduceOp reduceOp;
    uint32_t remoteRank;
    uint32_t deviceNumPerModule;
    bool isAsymmetricTopo;
    uint32_t reserved[7];
} HcclAlgoPluginParam;

typedef struct {
    uint32_t apiVersion;        /* HCCL_PLUGIN_API_VERSION */
    uint32_t magic;             /* HCCL_ALGO_PLUGIN_TABLE_MAGIC */
    uint32_t structSize;
    bool (*IsReady)(void);
    /* HCCL_SUCCESS + algName: the plugin will run this call.  Anything else: the built-in path runs. */
    HcclResult (*SelectAlg)(const HcclAlgoPluginParam* param, char algName[HCCL_ALGO_PLUGIN_ALG_NAME_LEN]);
    HcclResult (*ExecuteAlg)(const char* algName, const HcclAlgoPluginParam* param);
    /* Optional (a table whose structSize ends before it has none): the names of the algorithms the plugin offers for
       an operator ("AllReduce", ...; NULL or "" = all), written to buf as a sequence of '\0'-terminated names closed
       by an empty one.  Returns the number of names, or a negative value when bufLen is too small.  (HCCL's broker
       table has the same query, hccl_algo_plugin_broker_api.h:52-54.) */
    int (*QueryAlgs)(const char* opName, char* buf, size_t bufLen);
} HcclAlgoPluginTable;

const HcclAlgoPluginTable* GetHcclAlgoPlugin(void);   /* exported by the plugin */

/* Fills the common fields of a parameter block (what the library does before it calls SelectAlg; for plugin tests). */
static inline void HcclAlgoPluginParamInit(HcclAlgoPluginParam* param)
{
    if (param == NULL) return;
    memset(param, 0, sizeof(*param));
    param->version = HCCL_PLUGIN_API_VERSION;
    param->magic = HCCL_ALGO_PLUGIN_PARAM_MAGIC;
    param->structSize = (uint32_t)sizeof(HcclAlgoPluginParam);
}

/* Library side: the algorithm names of the loaded plugin (HCCL_ALGO_PLUGIN_PATH) for an operator, in the format of
   QueryAlgs.  HCCL_E_NOT_FOUND without a plugin, HCCL_E_NOT_SUPPORT when the plugin has no query, HCCL_E_MEMORY when
   buf is too small; *count receives the number of names. */
HcclResult HcclAlgoPluginQueryAlgs(const char* opName, char* buf, uint32_t bufLen, uint32_t* count);

#ifdef __cplusplus
}
#endif
#endif  /* HCCL_B200_ALGO_PLUGIN_H_ */
