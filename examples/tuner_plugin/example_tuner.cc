// Example tuner plugin: prefers the two-shot AllReduce above a size threshold taken from TUNER_TWOSHOT_MIN_BYTES and
// disables the LL algorithm below TUNER_LL_MAX_BYTES (the workflow of HCCL's examples/07_tuner_plugin: measure,
// derive thresholds, feed them back through the plugin).
//   g++ -shared -fPIC -std=c++17 -Icsrc/include examples/tuner_plugin/example_tuner.cc -o libexample_tuner.so
//   HCCL_ALG_TUNER_PLUGIN=$PWD/libexample_tuner.so python ...
#include <stdlib.h>
#include <string.h>
#include "hccl/hccl_tuner_plugin.h"

struct TunerCtx { uint64_t twoShotMin; uint64_t llMax; };

static HcclResult Create(HcclComm, const HcclTunerCommInfo*, const HcclTunerTopoInfo*, void** ctx, uint32_t* size)
{
    TunerCtx* c = (TunerCtx*)malloc(sizeof(TunerCtx));   // the host copies the blob and frees it with free()
    const char* a = getenv("TUNER_TWOSHOT_MIN_BYTES");
    const char* b = getenv("TUNER_LL_MAX_BYTES");
    c->twoShotMin = a ? strtoull(a, NULL, 10) : (1ull << 20);
    c->llMax = b ? strtoull(b, NULL, 10) : (64ull << 10);
    *ctx = c;
    *size = sizeof(TunerCtx);
    return HCCL_SUCCESS;
}

static HcclResult Update(void* ctx, const HcclTunerCollOpInfo* op, HcclTunerAlgoCostEntry* entries, uint32_t n, bool* matched)
{
    const TunerCtx* c = (const TunerCtx*)ctx;
    if (!c || op->collType != HCCL_CMD_ALLREDUCE) return HCCL_SUCCESS;
    const uint32_t stride = entries[0].header.size;
    for (uint32_t i = 0; i < n; ++i) {
        HcclTunerAlgoCostEntry* e = (HcclTunerAlgoCostEntry*)((char*)entries + (size_t)i * stride);
        if (strcmp(e->templateName, "meshtwoshot") == 0 && op->nBytes >= c->twoShotMin) { e->cost = 0.0f; *matched = true; }
        if (strcmp(e->templateName, "meshll") == 0 && op->nBytes > c->llMax) { e->cost = -1.0f; *matched = true; }
    }
    return HCCL_SUCCESS;
}

static HcclTunerPluginOps g_ops;
extern "C" const HcclTunerPluginOps* HcclTunerPluginOpsGet(void)
{
    HcclTunerPluginOpsInit(&g_ops);
    g_ops.Create = Create;
    g_ops.UpdateAlgoCostTable = Update;
    return &g_ops;
}
