// Tuner plugin ABI: a shared object named by HCCL_ALG_TUNER_PLUGIN may rewrite
// the per-call algorithm cost table.
//
// Binary layout and semantics follow the reference ABI
// (src/ops/op_common/selector/pub_inc/hccl_tuner_plugin.h:34-168): every struct
// starts with a 16-byte header {version, magicWord, size, reserved}; the plugin
// exports `HcclTunerPluginOpsGet`; `Create` runs once per communicator and may
// return a malloc'ed context blob that the host copies and frees;
// `UpdateAlgoCostTable` runs once per op and edits `cost`: <0 disables the
// algorithm, 0 marks it preferred, >0 overrides the model's cost.  Entries are
// walked with the stride entries[0].header.size so that newer hosts can append
// fields.
#ifndef HCCL_B200_TUNER_PLUGIN_H_
#define HCCL_B200_TUNER_PLUGIN_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    uint32_t version;
    uint32_t magicWord;
    uint32_t size;
    uint32_t reserved;
} HcclAbiHeader;

#define HCCL_TUNER_TOPO_INFO_MAGIC_WORD 0x0f0f0f31u
#define HCCL_TUNER_TOPO_INFO_VERSION 1u
#define HCCL_TUNER_COMM_INFO_MAGIC_WORD 0x0f0f0f32u
#define HCCL_TUNER_COMM_INFO_VERSION 1u
#define HCCL_TUNER_COLL_OP_INFO_MAGIC_WORD 0x0f0f0f33u
#define HCCL_TUNER_COLL_OP_INFO_VERSION 1u
#define HCCL_TUNER_ALGO_COST_ENTRY_MAGIC_WORD 0x0f0f0f34u
#define HCCL_TUNER_ALGO_COST_ENTRY_VERSION 1u
#define HCCL_TUNER_PLUGIN_OPS_MAGIC_WORD 0x0f0f0f35u
#define HCCL_TUNER_PLUGIN_OPS_VERSION 1u

static inline HcclResult HcclAbiHeaderInit(HcclAbiHeader* h, uint32_t magic, uint32_t version, uint32_t size)
{
    if (h == NULL) return HCCL_E_PTR;
    h->version = version;
    h->magicWord = magic;
    h->size = size;
    h->reserved = 0u;
    return HCCL_SUCCESS;
}

typedef struct {
    HcclAbiHeader header;
    uint32_t nRanks;
    uint32_t nNpusPerServer;   /* GPUs per NVLink domain */
    uint32_t nServers;
    uint32_t nPods;
    uint32_t nSuperPods;
} HcclTunerTopoInfo;

typedef struct {
    HcclAbiHeader header;
    const char* commName;      /* owned by the host */
    uint64_t bufferSize;
} HcclTunerCommInfo;

typedef struct {
    HcclAbiHeader header;
    uint64_t nBytes;
    HcclCMDType collType;
    HcclDataType dataType;
    HcclReduceOp reduceOp;
} HcclTunerCollOpInfo;

typedef struct {
    HcclAbiHeader header;
    const char* algName;       /* e.g. "P2pAllReduceSoleMeshTwoShot" */
    const char* engineName;    /* "p2p" | "nvls" | "host" */
    const char* executorName;  /* "sole" ... */
    const char* templateName;  /* "meshtwoshot" ... */
    float cost;                /* editable */
} HcclTunerAlgoCostEntry;

typedef struct {
    HcclAbiHeader header;
    HcclResult (*Create)(HcclComm comm, const HcclTunerCommInfo* commInfo, const HcclTunerTopoInfo* topoInfo,
                         void** tunerCtx, uint32_t* tunerCtxSize);
    HcclResult (*UpdateAlgoCostTable)(void* tunerCtx, const HcclTunerCollOpInfo* collOpInfo,
                                      HcclTunerAlgoCostEntry* algoCostEntries, uint32_t algoCount, bool* matched);
} HcclTunerPluginOps;

#define HCCL_TUNER_DEFINE_INIT(Type, fn, MAGIC, VERSION)                 \
    static inline HcclResult fn(Type* p)                                 \
    {                                                                    \
        if (p == NULL) return HCCL_E_PTR;                                \
        (void)memset(p, 0, sizeof(Type));                                \
        return HcclAbiHeaderInit(&p->header, MAGIC, VERSION, (uint32_t)sizeof(Type)); \
    }
HCCL_TUNER_DEFINE_INIT(HcclTunerTopoInfo, HcclTunerTopoInfoInit, HCCL_TUNER_TOPO_INFO_MAGIC_WORD, HCCL_TUNER_TOPO_INFO_VERSION)
HCCL_TUNER_DEFINE_INIT(HcclTunerCommInfo, HcclTunerCommInfoInit, HCCL_TUNER_COMM_INFO_MAGIC_WORD, HCCL_TUNER_COMM_INFO_VERSION)
HCCL_TUNER_DEFINE_INIT(HcclTunerCollOpInfo, HcclTunerCollOpInfoInit, HCCL_TUNER_COLL_OP_INFO_MAGIC_WORD, HCCL_TUNER_COLL_OP_INFO_VERSION)
HCCL_TUNER_DEFINE_INIT(HcclTunerAlgoCostEntry, HcclTunerAlgoCostEntryInit, HCCL_TUNER_ALGO_COST_ENTRY_MAGIC_WORD, HCCL_TUNER_ALGO_COST_ENTRY_VERSION)
HCCL_TUNER_DEFINE_INIT(HcclTunerPluginOps, HcclTunerPluginOpsInit, HCCL_TUNER_PLUGIN_OPS_MAGIC_WORD, HCCL_TUNER_PLUGIN_OPS_VERSION)

/* Exported by the plugin shared object. */
const HcclTunerPluginOps* HcclTunerPluginOpsGet(void);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_B200_TUNER_PLUGIN_H_ */
