#include "ranktable.h"
#include <fstream>
#include <sstream>
#include "../core/config.h"
#include "../core/json.h"
#include "../core/log.h"
#include "../core/plan_cache.h"

namespace hccl {

uint64_t RankTable::Fingerprint() const
{
    uint64_t h = Fnv1a(rootIp.data(), rootIp.size());
    h = Fnv1a(&rootPort, sizeof(rootPort), h);
    for (auto& r : ranks) {
        h = Fnv1a(&r.rankId, sizeof(r.rankId), h);
        h = Fnv1a(&r.deviceId, sizeof(r.deviceId), h);
        h = Fnv1a(r.serverId.data(), r.serverId.size(), h);
    }
    return h;
}

HcclResult ParseRankTable(const std::string& json, RankTable* out)
{
    JsonValue root;
    std::string err;
    if (!JsonParser(json).Parse(&root, &err) || root.kind != JsonValue::OBJ) { HCCL_ERROR("rank table is not valid JSON: %s", err.c_str()); return HCCL_E_PARA; }
    if (const JsonValue* st = root.Get("status"))
        if (st->kind == JsonValue::STR && st->str != "completed") { HCCL_ERROR("rank table status is '%s', expected 'completed'", st->str.c_str()); return HCCL_E_PARA; }
    const JsonValue* servers = root.Get("server_list");
    if (!servers || servers->kind != JsonValue::ARR || servers->arr.empty()) { HCCL_ERROR("rank table has no server_list"); return HCCL_E_PARA; }
    unsigned long long declared = 0;
    if (const JsonValue* sc = root.Get("server_count"))
        if (sc->AsU64(&declared) && declared != servers->arr.size()) { HCCL_ERROR("rank table: server_count %llu but %zu servers listed", declared, servers->arr.size()); return HCCL_E_PARA; }
    std::vector<RankTableEntry> entries;
    std::string firstHostIp;
    for (const JsonValue& s : servers->arr) {
        const JsonValue* devs = s.Get("device");
        if (!devs || devs->kind != JsonValue::ARR || devs->arr.empty()) { HCCL_ERROR("rank table: a server has no device list"); return HCCL_E_PARA; }
        std::string sid = s.Get("server_id") && s.Get("server_id")->kind == JsonValue::STR ? s.Get("server_id")->str : std::to_string(out->serverSizes.size());
        if (firstHostIp.empty() && s.Get("host_ip") && s.Get("host_ip")->kind == JsonValue::STR) firstHostIp = s.Get("host_ip")->str;
        out->serverSizes.push_back((uint32_t)devs->arr.size());
        for (const JsonValue& d : devs->arr) {
            RankTableEntry e;
            unsigned long long v;
            if (!d.Get("rank_id") || !d.Get("rank_id")->AsU64(&v)) { HCCL_ERROR("rank table: device without rank_id"); return HCCL_E_PARA; }
            e.rankId = (uint32_t)v;
            if (!d.Get("device_id") || !d.Get("device_id")->AsU64(&v)) { HCCL_ERROR("rank table: device without device_id"); return HCCL_E_PARA; }
            e.deviceId = (int)v;
            if (d.Get("device_ip") && d.Get("device_ip")->kind == JsonValue::STR) e.deviceIp = d.Get("device_ip")->str;
            if (d.Get("device_port") && d.Get("device_port")->AsU64(&v)) e.devicePort = (uint32_t)v;
            e.serverId = sid;
            entries.push_back(e);
        }
    }
    out->ranks.assign(entries.size(), RankTableEntry());
    std::vector<bool> seen(entries.size(), false);
    for (auto& e : entries) {
        if (e.rankId >= entries.size() || seen[e.rankId]) { HCCL_ERROR("rank table: rank ids must be unique and cover 0..%zu (bad id %u)", entries.size() - 1, e.rankId); return HCCL_E_PARA; }
        seen[e.rankId] = true;
        out->ranks[e.rankId] = e;
    }
    unsigned long long port = 0;
    if (root.Get("root_ip") && root.Get("root_ip")->kind == JsonValue::STR) out->rootIp = root.Get("root_ip")->str;
    else out->rootIp = firstHostIp.empty() ? "127.0.0.1" : firstHostIp;
    if (root.Get("root_port") && root.Get("root_port")->AsU64(&port)) out->rootPort = (uint32_t)port;
    else if (out->ranks[0].devicePort) out->rootPort = out->ranks[0].devicePort;
    else out->rootPort = GetEnvConfig().ifBasePort ? GetEnvConfig().ifBasePort : 60000;
    return HCCL_SUCCESS;
}

HcclResult LoadRankTable(const char* clusterInfo, RankTable* out)
{
    std::string text(clusterInfo);
    size_t first = text.find_first_not_of(" \t\r\n");
    if (first == std::string::npos) return HCCL_E_PARA;
    if (text[first] != '{') {
        std::ifstream f(clusterInfo);
        if (!f) { HCCL_ERROR("cannot open rank table file '%s'", clusterInfo); return HCCL_E_OPEN_FILE_FAILURE; }
        std::stringstream ss;
        ss << f.rdbuf();
        text = ss.str();
    }
    return ParseRankTable(text, out);
}

}  // namespace hccl
