// Rank-table (cluster information) loader for HcclCommInitClusterInfo.
//
// Accepts the JSON layout documented for HCCL rank tables
// (docs/en/user_guide/cluster_info_config/rank_table_config_a2.md: "status",
// "version", "server_count", "server_list"[{"server_id", "device"[{"device_id",
// "device_ip", "device_port", "rank_id"}]}]).  The rendezvous endpoint is
// "root_ip"/"root_port" when present, else the host_ip of rank 0's server (or
// 127.0.0.1) and rank 0's device_port (or HCCL_IF_BASE_PORT, or 60000).
// `clusterInfo` may be a file path or the JSON text itself.
#pragma once
#include <cstdint>
#include <string>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

struct RankTableEntry {
    uint32_t rankId = 0;
    int deviceId = -1;
    std::string serverId;
    std::string deviceIp;
    uint32_t devicePort = 0;
};
struct RankTable {
    std::vector<RankTableEntry> ranks;   // indexed by rank id
    std::vector<uint32_t> serverSizes;
    std::string rootIp;
    uint32_t rootPort = 0;
    uint64_t Fingerprint() const;
};
HcclResult LoadRankTable(const char* clusterInfo, RankTable* out);
HcclResult ParseRankTable(const std::string& json, RankTable* out);

}  // namespace hccl
