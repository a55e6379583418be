// Tuner plugin driven by a measured configuration file - the last step of the tuning workflow of HCCL's
// examples/07_tuner_plugin (perf_test.py -> optimize_config.py -> JSON -> plugin):
//
//   1. python examples/tuner_plugin/perf_test.py --host-sim 8 --out perf.jsonl      (or under torchrun on GPUs)
//        times every algorithm the selector could run, per operator and message size
//   2. python examples/tuner_plugin/optimize_config.py perf.jsonl -o tuned.json
//        keeps the fastest algorithm per (operator, size range)
//   3. g++ -shared -fPIC -std=c++17 -Icsrc/include examples/tuner_plugin/config_tuner.cc -o libconfig_tuner.so
//      HCCL_ALG_TUNER_PLUGIN=$PWD/libconfig_tuner.so HCCL_ALG_CONFIG_FILE=$PWD/tuned.json <program>
//        every call whose (operator, bytes) falls in a rule gets that rule's algorithm at cost 0 (= preferred)
//
// File format: {"rules": [{"op": <HcclCMDType>, "min_bytes": a, "max_bytes": b, "alg": "<algorithm name>"}, ...]}
// with min_bytes <= bytes < max_bytes.  HCCL_ALG_FORCE="<algorithm name>" (used by perf_test.py) prefers one
// algorithm for every call instead.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>
#include "hccl/hccl_tuner_plugin.h"

namespace {

struct Rule { int op; unsigned long long lo, hi; char alg[96]; };
struct Ctx { uint32_t nRules; char force[96]; Rule rules[1]; };     // variable length, copied as one blob by the host

bool Field(const std::string& obj, const char* key, std::string* out)
{
    const std::string k = std::string("\"") + key + "\"";
    size_t p = obj.find(k);
    if (p == std::string::npos) return false;
    p = obj.find(':', p + k.size());
    if (p == std::string::npos) return false;
    ++p;
    while (p < obj.size() && (obj[p] == ' ' || obj[p] == '\t' || obj[p] == '\n')) ++p;
    if (p < obj.size() && obj[p] == '"') {
        const size_t e = obj.find('"', p + 1);
        if (e == std::string::npos) return false;
        *out = obj.substr(p + 1, e - p - 1);
    } else {
        size_t e = p;
        while (e < obj.size() && obj[e] != ',' && obj[e] != '}' && obj[e] != ' ' && obj[e] != '\n') ++e;
        *out = obj.substr(p, e - p);
    }
    return true;
}

std::vector<Rule> LoadRules(const char* path)
{
    std::vector<Rule> rules;
    FILE* f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "config_tuner: cannot open %s\n", path); return rules; }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    size_t p = text.find("\"rules\"");
    if (p == std::string::npos) return rules;
    p = text.find('[', p);
    const size_t end = text.find(']', p == std::string::npos ? 0 : p);
    while (p != std::string::npos && p < end) {
        const size_t b = text.find('{', p);
        if (b == std::string::npos || b > end) break;
        const size_t e = text.find('}', b);
        if (e == std::string::npos) break;
        const std::string obj = text.substr(b, e - b + 1);
        std::string op, lo, hi, alg;
        if (Field(obj, "op", &op) && Field(obj, "min_bytes", &lo) && Field(obj, "max_bytes", &hi) && Field(obj, "alg", &alg) && alg.size() < sizeof(Rule::alg)) {
            Rule r;
            r.op = atoi(op.c_str());
            r.lo = strtoull(lo.c_str(), nullptr, 10);
            r.hi = strtoull(hi.c_str(), nullptr, 10);
            snprintf(r.alg, sizeof(r.alg), "%s", alg.c_str());
            rules.push_back(r);
        }
        p = e + 1;
    }
    return rules;
}

HcclResult Create(HcclComm, const HcclTunerCommInfo*, const HcclTunerTopoInfo*, void** ctx, uint32_t* size)
{
    std::vector<Rule> rules;
    const char* path = getenv("HCCL_ALG_CONFIG_FILE");
    if (path && *path) rules = LoadRules(path);
    const size_t bytes = sizeof(Ctx) + (rules.empty() ? 0 : (rules.size() - 1) * sizeof(Rule));
    Ctx* c = (Ctx*)calloc(1, bytes);                     // the host copies the blob and frees it with free()
    if (!c) return HCCL_E_MEMORY;
    c->nRules = (uint32_t)rules.size();
    const char* force = getenv("HCCL_ALG_FORCE");
    snprintf(c->force, sizeof(c->force), "%s", force ? force : "");
    for (size_t i = 0; i < rules.size(); ++i) c->rules[i] = rules[i];
    *ctx = c;
    *size = (uint32_t)bytes;
    return HCCL_SUCCESS;
}

HcclResult Update(void* ctx, const HcclTunerCollOpInfo* op, HcclTunerAlgoCostEntry* entries, uint32_t n, bool* matched)
{
    const Ctx* c = (const Ctx*)ctx;
    if (!c || n == 0) return HCCL_SUCCESS;
    const char* want = c->force[0] ? c->force : nullptr;
    for (uint32_t i = 0; !want && i < c->nRules; ++i)
        if (c->rules[i].op == (int)op->collType && op->nBytes >= c->rules[i].lo && op->nBytes < c->rules[i].hi) want = c->rules[i].alg;
    if (!want) return HCCL_SUCCESS;
    const uint32_t stride = entries[0].header.size;
    for (uint32_t i = 0; i < n; ++i) {
        HcclTunerAlgoCostEntry* e = (HcclTunerAlgoCostEntry*)((char*)entries + (size_t)i * stride);
        if (e->algName && strcmp(e->algName, want) == 0) { e->cost = 0.0f; *matched = true; }
    }
    return HCCL_SUCCESS;
}

HcclTunerPluginOps g_ops;

}  // namespace

extern "C" const HcclTunerPluginOps* HcclTunerPluginOpsGet(void)
{
    HcclTunerPluginOpsInit(&g_ops);
    g_ops.Create = Create;
    g_ops.UpdateAlgoCostTable = Update;
    return &g_ops;
}
